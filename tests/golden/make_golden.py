#!/usr/bin/env python3
"""Generate the committed golden vectors from the UNMODIFIED reference.

Run in the build container only (it imports the read-only JetFire checkout):

    python tests/golden/make_golden.py /path/to/JetFire

Writes ``tests/golden/pack_golden.npz``: seeded bf16 / fp16 inputs and the bytes and
bf16 scales that ``jetfire_vllm/kernels/intN_pack.py:quantize_and_pack`` returns for
them, for INT2/3/4 at group sizes 64 and 128, plus the round trip through ``unpack``.
Inputs include N(0,1) rows with log-normal outlier channels, all-zero groups,
exact rounding ties (x / scale == n + 0.5) and saturating values.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch


def build_inputs(seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    rows = []
    x = torch.randn(96, 128, generator=g)
    c = torch.exp(0.75 * torch.randn(128, generator=g))
    rows.append(x * c)                                  # outlier channels
    rows.append(torch.randn(32, 128, generator=g) * 1e-3)
    rows.append(torch.randn(32, 128, generator=g) * 300.0)
    z = torch.randn(8, 128, generator=g)
    z[:, :64] = 0                                      # one all-zero group
    rows.append(z)
    rows.append(torch.zeros(4, 128))
    # exact ties: amax chosen so the bf16 scale is a power of two; values at n + 0.5
    for qmax in (1, 3, 7):
        t = torch.zeros(8, 128)
        t[:, 0] = float(qmax)                          # amax -> scale == 1
        t[:, 64] = float(qmax)
        steps = torch.arange(-qmax, qmax).float() + 0.5
        for r in range(8):
            t[r, 1:1 + len(steps)] = steps * (1 if r % 2 == 0 else -1)
            t[r, 65:65 + len(steps)] = steps
        rows.append(t)
    return torch.cat(rows, 0)


def main() -> int:
    # the reference checkout: argument, else $JETFIRE_REFERENCE_ROOT, else `reference` beside the repo
    default = os.environ.get("JETFIRE_REFERENCE_ROOT") or str(Path(__file__).resolve().parents[3] / "reference")
    ref_root = Path(sys.argv[1] if len(sys.argv) > 1 else default)
    sys.path.insert(0, str(ref_root))
    from jetfire_vllm.kernels.intN_pack import quantize_and_pack, unpack

    out = {}
    x32 = build_inputs(20251)
    for dt_name, dt in (("bf16", torch.bfloat16), ("fp16", torch.float16)):
        x = x32.to(dt)
        out[f"x_{dt_name}"] = x.view(torch.int16).numpy().view(np.uint16)
        for bits in (2, 3, 4):
            for gs in (64, 128):
                data, scales = quantize_and_pack(x, group_size=gs, nbits=bits)
                back = unpack(data, scales, group_size=gs, nbits=bits)
                key = f"{dt_name}_b{bits}_g{gs}"
                out[key + "_data"] = data.numpy()
                out[key + "_scales"] = scales.view(torch.int16).numpy().view(np.uint16)
                out[key + "_unpack"] = back.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    dst = Path(__file__).resolve().parent / "pack_golden.npz"
    np.savez_compressed(dst, **out)
    print("wrote", dst, dst.stat().st_size, "bytes")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
