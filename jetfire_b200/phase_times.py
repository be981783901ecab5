"""Phase stamps of the decode kernels (a tuning aid, not part of the product path).

Needs a library built with the stamps compiled in::

    JF_NVCC_EXTRA=-DJF_PHASE_TIMING python -m jetfire_b200.build --force
    python -m jetfire_b200.phase_times --mode k4v4 --batch 4 --ctx 32768

Prints, for the first CTA of the K4V4 scan and of the fused select+finish kernel, the SM
clock cycles spent between consecutive ``JF_PHASE`` marks (``csrc/jf_common.cuh``).  Rebuild
without the flag afterwards: the stamps cost a few instructions per mark.
"""
from __future__ import annotations

import argparse
import ctypes as C

import torch

from . import _lib, ops

SELECT_MARKS = [(0, "small loads"), (11, "query model, zeroing"), (1, "wait for the score chunk"),
                (2, "group-maxima histogram"), (3, "histogram scan"), (4, "collect candidates"),
                (5, "slots"), (6, "row gathers"), (7, "canonical scores"), (8, "ranking"), (9, "(to output)"),
                (10, "outputs, wait for V rows"), (20, "split merge"), (21, "weights"), (22, "V rows"),
                (23, "accumulate"), (24, "final reduce"), (25, None)]
SCAN_MARKS = [(0, "barrier setup, wait for the previous kernel"), (1, "first loads, first copies, query fragments"),
              (2, "wait for the first page"), (3, "page loop"), (4, "other warps"), (5, "CTA merge, partial store"),
              (6, None)]


def _stamps(name: str):
    fn = getattr(_lib.lib, name, None)
    if fn is None:
        raise SystemExit(f"{name} is not in the library: rebuild with JF_NVCC_EXTRA=-DJF_PHASE_TIMING")
    buf = (C.c_ulonglong * 64)()
    fn(buf)
    return list(buf)


def _report(title, t, marks):
    parts = [f"{label} {t[b] - t[a]}" for (a, label), (b, _) in zip(marks[:-1], marks[1:])]
    print(f"{title}: " + " | ".join(parts) + f" | total {t[marks[-1][0]] - t[marks[0][0]]} cycles")


def _collect_detail(t):
    """Inside 'collect candidates' (stamps 30..33 of the select kernel's first collection)."""
    if t[30] and t[33]:
        print(f"  collect: threshold pass {t[30] - t[4]} | offsets {t[31] - t[30]} | scatter {t[32] - t[31]} | "
              f"barrier {t[33] - t[32]} | to the next phase {t[5] - t[33]}")


def _cta_timeline():
    """Per-CTA wall-clock stamps of the last K4V4 scan launch (globaltimer, ns): when the CTAs
    started, entered and left their page loops and finished; and the loop time by the CTA's
    launch rank on its SM (the warp scheduler favours the older CTAs)."""
    import numpy as np
    fn = getattr(_lib.lib, "jf_debug_scan_cta_times", None)
    if fn is None:
        raise SystemExit("rebuild with JF_NVCC_EXTRA=-DJF_PHASE_TIMING")
    buf = (C.c_ulonglong * (1024 * 8))()
    fn(buf)
    t = np.array(list(buf), dtype=np.int64).reshape(1024, 8)
    t = t[t[:, 0] > 0]   # the CTAs that ran (this tool launches one shape only)
    t0 = t[:, 0].min()
    span = lambda a: f"{int(a.min() - t0)} / {int(np.median(a) - t0)} / {int(a.max() - t0)}"
    print(f"  ns from the first CTA's start (min / median / max over {len(t)} CTAs): start {span(t[:, 0])}, "
          f"past the wait for the previous kernel {span(t[:, 1])}, loop start {span(t[:, 2])}, "
          f"loop end {span(t[:, 3])}, end {span(t[:, 4])}")
    loop = t[:, 3] - t[:, 2]
    print(f"  loop ns min / median / max: {int(loop.min())} / {int(np.median(loop))} / {int(loop.max())}")
    sm = t[:, 5]
    by_rank = {}
    for s_ in np.unique(sm):
        idx = np.sort(np.where(sm == s_)[0])
        for r, i in enumerate(idx):
            by_rank.setdefault((len(idx), r), []).append(loop[i])
    print("  median loop ns by (CTAs on the SM, launch rank): " +
          ", ".join(f"({k[0]},{k[1]}): {int(np.median(v))}" for k, v in sorted(by_rank.items())))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="k4v4", choices=("k4v4", "k3v2"))
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--ctx", type=int, default=32768)
    ap.add_argument("--top-k", type=int, default=256)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--cta-timeline", action="store_true", help="per-CTA wall-clock summary of the K4V4 scan")
    a = ap.parse_args()
    kb, vb, gs = {"k4v4": (4, 4, 128), "k3v2": (3, 2, 64)}[a.mode]
    H_q, H_kv, dev = 32, 8, torch.device("cuda", 0)
    t = a.batch * a.ctx
    g = torch.Generator(device=dev).manual_seed(1)
    ch = torch.exp(0.75 * torch.randn(1, H_kv, 128, generator=g, device=dev))
    k = (torch.randn(t, H_kv, 128, generator=g, device=dev) * ch).to(torch.bfloat16)
    v = torch.randn(t, H_kv, 128, generator=g, device=dev).to(torch.bfloat16)
    kd = torch.empty(H_kv, t, 16 * kb, dtype=torch.uint8, device=dev)
    vd = torch.empty(H_kv, t, 16 * vb, dtype=torch.uint8, device=dev)
    ks = torch.empty(H_kv, t, 128 // gs, dtype=torch.bfloat16, device=dev)
    vs = torch.empty_like(ks)
    ops.fused_quant_write_kv(k, v, torch.arange(t, dtype=torch.int64, device=dev), kd, ks, vd, vs, gs, kb, vb)
    bt = torch.arange(t // 16, dtype=torch.int64, device=dev).reshape(a.batch, a.ctx // 16)
    lens = torch.full((a.batch,), a.ctx, dtype=torch.int32, device=dev)
    q = torch.randn(a.batch, H_q, 128, generator=g, device=dev).to(torch.bfloat16)
    call = ops.DecodeCall(a.mode, q, kd, ks, vd, vs, bt, lens, a.ctx, H_q, H_kv, 16, a.top_k, 128 ** -0.5)
    for _ in range(a.reps):
        call.fused()
        call.fused()      # back to back, as in a decode step: the second launch is the one reported
        torch.cuda.synchronize()
        if a.mode == "k4v4":
            _report("scan_k4v4", _stamps("jf_debug_scan_times"), SCAN_MARKS)
            if a.cta_timeline:
                _cta_timeline()
        sel = _stamps("jf_debug_phase_times")
        _report(f"select+finish {a.mode}", sel, SELECT_MARKS)
        _collect_detail(sel)


if __name__ == "__main__":
    main()
