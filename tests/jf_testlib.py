"""Shared helpers for the parity tests: seeded synthetic inputs in the reference's
layouts, and conversions between torch tensors and the oracle's numpy conventions."""
from __future__ import annotations

import numpy as np
import torch

from oracle import jf_oracle as O

MODES = {"k3v2": (3, 2, 64), "k4v4": (4, 4, 128)}


def to_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def f32_values(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().float().numpy()


def from_bits(bits: np.ndarray, dtype) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(dtype)


class Case:
    """One layer's worth of seeded inputs (N(0,1) Q/K/V, K scaled per channel by
    log-normal(0, 0.75)), a shuffled paged layout, ragged lengths."""

    def __init__(self, mode, B, H_q, H_kv, ctx, lens=None, seed=0, dtype=torch.bfloat16, spare_blocks=1):
        self.mode, self.B, self.H_q, self.H_kv, self.ctx = mode, B, H_q, H_kv, ctx
        self.kb, self.vb, self.gs = MODES[mode]
        self.dtype = dtype
        g = torch.Generator().manual_seed(seed)
        blocks_per_seq = (ctx + 15) // 16
        self.n_blocks = B * blocks_per_seq + spare_blocks
        self.num_slots = self.n_blocks * 16
        ch = torch.exp(0.75 * torch.randn(H_kv, 1, 128, generator=g))
        self.k_full = (torch.randn(H_kv, self.num_slots, 128, generator=g) * ch).to(dtype)
        self.v_full = torch.randn(H_kv, self.num_slots, 128, generator=g).to(dtype)
        self.q = torch.randn(B, H_q, 128, generator=g).to(dtype)
        perm = torch.randperm(self.n_blocks, generator=g)[: B * blocks_per_seq]
        self.block_table = perm.reshape(B, blocks_per_seq).to(torch.int64)
        if lens is None:
            lens = [max(ctx - 13 * b, 0) for b in range(B)]
        self.seq_lens = torch.tensor(lens, dtype=torch.int32)
        self.attn_scale = 128 ** -0.5

    # -- oracle-side packed cache (numpy) --
    def oracle_cache(self):
        kd, ks = O.quantize_and_pack(f32_values(self.k_full), self.gs, self.kb)
        vd, vs = O.quantize_and_pack(f32_values(self.v_full), self.gs, self.vb)
        return kd, ks, vd, vs

    def oracle_step(self, top_k, stage_b="fp32", with_correction=True):
        kd, ks, vd, vs = self.oracle_cache()
        kw = {}
        if with_correction:
            kw = dict(k_shadow=f32_values(self.k_full), v_shadow=f32_values(self.v_full))
        return O.decode_step(self.mode, f32_values(self.q), kd, ks, vd, vs, self.block_table.numpy(),
                             self.seq_lens.numpy(), top_k, self.attn_scale, stage_b=stage_b,
                             max_s=self.ctx, **kw)

    # -- device-side packed cache through the product's append path --
    def device_cache(self, device="cuda"):
        from jetfire_b200 import ops
        kdim, vdim, ng = 16 * self.kb, 16 * self.vb, 128 // self.gs
        k_data = torch.full((self.H_kv, self.num_slots, kdim), 0xA5, dtype=torch.uint8, device=device)
        v_data = torch.full((self.H_kv, self.num_slots, vdim), 0xA5, dtype=torch.uint8, device=device)
        k_scales = torch.zeros(self.H_kv, self.num_slots, ng, dtype=torch.bfloat16, device=device)
        v_scales = torch.zeros_like(k_scales)
        key_tok = self.k_full.transpose(0, 1).contiguous().to(device)   # (T, H_kv, 128)
        val_tok = self.v_full.transpose(0, 1).contiguous().to(device)
        slots = torch.arange(self.num_slots, dtype=torch.int64, device=device)
        ops.fused_quant_write_kv(key_tok, val_tok, slots, k_data, k_scales, v_data, v_scales,
                                 self.gs, self.kb, self.vb)
        return k_data, k_scales, v_data, v_scales


def causal_prefill_attention(*, q, k, v, out, cu_seqlens, max_seqlen, impl, layer, attn_metadata) -> None:
    """Plain causal attention in fp32 over the sequences ``cu_seqlens`` delimits (rows of ``q
    (T, H_q, D)``, ``k`` / ``v (T, H_kv, D)``): what a variable-length flash attention computes
    for prefill rows without cached context.  Stands in for it in the tests of mixed steps."""
    H_q, H_kv = q.shape[1], k.shape[1]
    bounds = [int(x) for x in cu_seqlens]
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        qs = q[lo:hi].float().transpose(0, 1)                                   # (H_q, L, D)
        ks = k[lo:hi].float().transpose(0, 1).repeat_interleave(H_q // H_kv, 0)
        vs = v[lo:hi].float().transpose(0, 1).repeat_interleave(H_q // H_kv, 0)
        s = (qs @ ks.transpose(1, 2)) * float(impl.scale)
        L = hi - lo
        s = s.masked_fill(torch.ones(L, L, dtype=torch.bool, device=q.device).triu(1), float("-inf"))
        out[lo:hi].copy_((torch.softmax(s, -1) @ vs).transpose(0, 1).to(out.dtype))
