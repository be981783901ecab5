"""numpy restatement of the JetFire decode hot path (the parity oracle).

TEST INFRASTRUCTURE ONLY -- see ``oracle/__init__.py``.  Every function cites
the reference file:line (paths inside the JetFire project) whose arithmetic it
restates.  Pinning: ``tests/test_oracle_golden.py`` checks this file against
the reference's own wire-format fixtures (tests/test_int_pack.py:10-35), its
top-k width table and head map (tests/test_runtime_edge_cases.py:13-35), and
against byte-for-byte outputs of the reference's ``quantize_and_pack`` run in
the build container (``tests/golden/make_golden.py`` is the generating script).

Conventions
-----------
* bf16 tensors are carried as ``uint16`` bit patterns; helper converters are
  RNE (round to nearest even), the rounding torch and CUDA use.
* "f32 values" means a float32 array whose entries are exactly representable
  in the source dtype (bf16 or fp16), i.e. ``x.float()`` of the reference.
* Layouts are the reference's: ``k_data (H_kv, num_slots, Dp) u8``,
  ``k_scales (H_kv, num_slots, NG) bf16``, ``block_table (B, max_blocks) i64``,
  ``seq_lens (B,) i32``, ``q (B, H_q, 128)``;
  ``slot(b, p) = block_table[b, p // 16] * 16 + p % 16``.
"""
from __future__ import annotations

import numpy as np

HEAD_DIM = 128
BLOCK = 16

# ---------------------------------------------------------------------------
# bf16 helpers
# ---------------------------------------------------------------------------


def f32_to_bf16_bits(x) -> np.ndarray:
    """float32 -> bf16 bit pattern, round-to-nearest-even (torch ``.to(bfloat16)``)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    out = rounded.astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        out = np.where(nan, np.uint16(0x7FC0), out)
    return out


def bf16_bits_to_f32(b) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << 16).view(np.float32)


def round_to_bf16(x) -> np.ndarray:
    """float32 -> nearest bf16 value, returned as float32."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


# ---------------------------------------------------------------------------
# PACK  (kernels/intN_pack.py:47-107, 172-222)
# ---------------------------------------------------------------------------


def packed_dim(head_dim: int, nbits: int) -> int:
    """kernels/intN_pack.py:35-44."""
    return {2: head_dim // 4, 3: head_dim * 3 // 8, 4: head_dim // 2}[nbits]


def qmax_of(nbits: int) -> int:
    return (1 << (nbits - 1)) - 1


def offset_of(nbits: int) -> int:
    return 1 << (nbits - 1)


def quantize_codes(x, group_size: int, nbits: int):
    """Per-group symmetric quantisation (kernels/intN_pack.py:81-98).

    amax -> fp32 ``amax / qmax`` clamped to 1e-8 -> bf16 (RNE) -> back to fp32;
    ``q = clamp(round_half_even(x / scale), -qmax, qmax)`` with an IEEE divide.
    Returns (signed codes int8 (..., D), scale bf16 bits (..., D // group_size)).
    """
    x = np.asarray(x, dtype=np.float32)
    d = x.shape[-1]
    ng = d // group_size
    qmax = qmax_of(nbits)
    xg = x.reshape(*x.shape[:-1], ng, group_size)
    amax = np.abs(xg).max(axis=-1)
    scales = np.maximum(amax / np.float32(qmax), np.float32(1e-8)).astype(np.float32)
    sbits = f32_to_bf16_bits(scales)
    sf = bf16_bits_to_f32(sbits)[..., None]
    with np.errstate(over="ignore", invalid="ignore"):
        q = np.rint(xg / sf)  # np.rint is round-half-even, like torch.round
    q = np.clip(q, -qmax, qmax).reshape(x.shape).astype(np.int8)
    return q, sbits


def pack_codes(q, nbits: int) -> np.ndarray:
    """Signed codes -> wire bytes (kernels/intN_pack.py:172-222)."""
    u = q.astype(np.int32) + offset_of(nbits)
    if nbits == 4:
        return ((u[..., 0::2] << 4) | u[..., 1::2]).astype(np.uint8)
    if nbits == 2:
        return ((u[..., 0::4] << 6) | (u[..., 1::4] << 4) | (u[..., 2::4] << 2) | u[..., 3::4]).astype(np.uint8)
    if nbits == 3:
        g = u.reshape(*u.shape[:-1], -1, 8)
        w = np.zeros(g.shape[:-1], dtype=np.int32)
        for i in range(8):
            w |= g[..., i] << (21 - 3 * i)
        planes = [((w >> 16) & 255), ((w >> 8) & 255), (w & 255)]
        return np.concatenate(planes, axis=-1).astype(np.uint8)
    raise ValueError(nbits)


def quantize_and_pack(x, group_size: int, nbits: int):
    """kernels/intN_pack.py:60-107 -> (data u8 (..., Dp), scales bf16 bits (..., NG))."""
    q, sbits = quantize_codes(x, group_size, nbits)
    return pack_codes(q, nbits), sbits


def decode_codes(data, nbits: int) -> np.ndarray:
    """Wire bytes -> unsigned codes int32 (scripts/validate_runtime.py:22-32)."""
    d = np.asarray(data).astype(np.int32)
    if nbits == 3:
        n = d.shape[-1] // 3
        w = (d[..., :n] << 16) | (d[..., n:2 * n] << 8) | d[..., 2 * n:]
        return np.stack([(w >> (21 - 3 * i)) & 7 for i in range(8)], -1).reshape(*d.shape[:-1], n * 8)
    lanes = 8 // nbits
    mask = (1 << nbits) - 1
    return np.stack([(d >> (8 - nbits * (i + 1))) & mask for i in range(lanes)], -1).reshape(
        *d.shape[:-1], d.shape[-1] * lanes)


def dequant(data, scale_bits, nbits: int, group_size: int, *, bf16: bool) -> np.ndarray:
    """scripts/validate_runtime.py:35-43.  ``bf16=True`` is the Stage-A rounding
    ``bf16(float(code - off) * float(scale))`` of csrc/int3_qk_scores.cu:90-100."""
    codes = (decode_codes(data, nbits) - offset_of(nbits)).astype(np.float32)
    shape = codes.shape
    s = bf16_bits_to_f32(scale_bits)
    out = (codes.reshape(*shape[:-1], -1, group_size) * s[..., None]).reshape(shape)
    return round_to_bf16(out) if bf16 else out


def unpack(data, scale_bits, nbits: int, group_size: int) -> np.ndarray:
    """kernels/intN_pack.py:227-… : dequantised values rounded to bf16 (as f32)."""
    return dequant(data, scale_bits, nbits, group_size, bf16=True)


def scatter_pack(x_tok, slots, out_data, out_scales, group_size: int, nbits: int) -> None:
    """Quantise-on-append (kernels/fused_quant_write.py:136-194, 634-781): row t of
    ``x_tok (T, H_kv, 128)`` goes to ``out[h, slots[t]]``; negative slots are skipped
    (:150-152).  Arithmetic is the torch reference's (IEEE divide), which the Triton
    writers only approximate (scripts/validate_runtime.py:88-92)."""
    data, sbits = quantize_and_pack(x_tok, group_size, nbits)  # (T, H, Dp), (T, H, NG)
    for t, s in enumerate(np.asarray(slots).tolist()):
        if s < 0:
            continue
        out_data[:, s, :] = data[t]
        out_scales[:, s, :] = sbits[t]


# ---------------------------------------------------------------------------
# Addressing
# ---------------------------------------------------------------------------


def slots_of(block_table, b: int, n: int, block: int = BLOCK) -> np.ndarray:
    """slot(b, p) for p in [0, n) (csrc/int3_qk_scores.cu:399-417)."""
    p = np.arange(n, dtype=np.int64)
    if n == 0:
        return p
    return np.asarray(block_table)[b, p // block].astype(np.int64) * block + p % block


def head_map(batch: int, h_q: int, group: int, k: int) -> np.ndarray:
    """adapter/decode_path.py:400-408: (B, H_q, K) int64, value h_q // group."""
    hm = (np.arange(h_q, dtype=np.int64) // group)[None, :, None]
    return np.ascontiguousarray(np.broadcast_to(hm, (batch, h_q, k)))


def select_top_k(config_top_k: int, seq_len: int, supported) -> int | None:
    """adapter/decode_path.py:1156-1182: largest supported width <= length, else the
    smallest supported one; None for empty sequences / nothing configured."""
    requested, length = int(config_top_k), int(seq_len)
    configured = [k for k in supported if 0 < k <= requested]
    if not configured or length <= 0:
        return None
    cands = [k for k in configured if k <= length]
    return max(cands) if cands else min(configured)


# ---------------------------------------------------------------------------
# STAGE A -- canonical scores
# ---------------------------------------------------------------------------


def canonical_scores_bf16path(q_row, k_hat, attn_scale) -> np.ndarray:
    """K3 (and K4/G64) scores in the canonical order.

    Reference arithmetic (csrc/int3_qk_scores.cu:90-100, 284-311):
    ``k_hat = bf16(float(code - off) * float(scale))``, products of two 16-bit
    floats are exact in fp32 and are accumulated in fp32, then multiplied by
    ``attn_scale``.  The tensor-core accumulation order is unspecified, so the
    canonical order is fixed here (any fixed order stays inside the reference's own
    2e-5 score gate, scripts/validate_runtime.py:147-148):

      * 32 partial sums: partial ``l`` takes channels ``l, l+32, l+64, l+96`` in that
        order, ``part = fmaf(q[d], k_hat[d], part)`` from 0 -- each product is exact, so
        a float32 multiply followed by a float32 add reproduces ``fmaf`` bit for bit;
      * a butterfly over distances 16, 8, 4, 2, 1: ``part[l] += part[l ^ o]``.

    q_row (128,) f32 values, k_hat (n, 128) f32 values (bf16-representable).
    """
    q_row = np.asarray(q_row, dtype=np.float32)
    k_hat = np.asarray(k_hat, dtype=np.float32)
    part = np.zeros((k_hat.shape[0], 32), dtype=np.float32)
    for r in range(4):
        part = part + q_row[None, 32 * r:32 * r + 32] * k_hat[:, 32 * r:32 * r + 32]
    lanes = np.arange(32)
    for o in (16, 8, 4, 2, 1):
        part = part + part[:, lanes ^ o]
    return part[:, 0] * np.float32(attn_scale)


def quantize_query_int8(q):
    """INT8 query model of the K4/G128 Stage A (csrc/int8tc_qk_scores.cu:272-290;
    scripts/validate_runtime.py:46-58).  Per 32-channel block: ``qs = max(amax/127,
    1e-12)`` (IEEE divide), ``qi = clamp(rn(q * (1/qs)), -128, 127)``.
    Returns (qi int32 (..., 128), qs f32 (..., 4))."""
    q = np.asarray(q, dtype=np.float32)
    g = q.reshape(*q.shape[:-1], -1, 32)
    amax = np.abs(g).max(-1)
    qs = np.maximum(amax / np.float32(127.0), np.float32(1e-12)).astype(np.float32)
    inv = (np.float32(1.0) / qs).astype(np.float32)
    qi = np.clip(np.rint((g * inv[..., None]).astype(np.float32)), -128, 127).astype(np.int32)
    return qi.reshape(q.shape), qs


def canonical_scores_int8path(qi_row, qs_row, k_codes_signed, k_scale_f32, attn_scale) -> np.ndarray:
    """K4/G128 scores (csrc/int8tc_qk_scores.cu:445-487): exact int32 dot per
    32-channel block, then ``s = fma(float(acc_c), qs_c, s)`` for c = 0..3, then
    ``* k_scale``, then ``* attn_scale`` -- all fp32.  The fma is replayed in float64
    (a 24-bit by 24-bit product plus a 24-bit addend is exact there before the single
    rounding to fp32 ... the addend can be far smaller, so round via exact rational
    arithmetic when needed)."""
    kc = np.asarray(k_codes_signed, dtype=np.int64).reshape(-1, 4, 32)
    qi = np.asarray(qi_row, dtype=np.int64).reshape(4, 32)
    acc = np.einsum("ncd,cd->nc", kc, qi)  # exact
    s = np.zeros(kc.shape[0], dtype=np.float32)
    for c in range(4):
        s = _fma_f32(acc[:, c].astype(np.float32), np.float32(qs_row[c]), s)
    s = s * np.asarray(k_scale_f32, dtype=np.float32)
    return s * np.float32(attn_scale)


def _fma_f32(a, b, c) -> np.ndarray:
    """fp32 fused multiply-add with a single rounding (CUDA ``fmaf``).  ``a*b`` of two
    fp32 values is exact in float64; the float64 add may round, so the sum is put in
    round-to-odd form (the two-sum error term says which neighbour brackets the exact
    value) before the final RNE cast -- 53 >= 24 + 2 bits makes that cast correct."""
    a = np.asarray(a, dtype=np.float32)
    b = np.asarray(b, dtype=np.float32)
    c = np.asarray(c, dtype=np.float32)
    prod = a.astype(np.float64) * b.astype(np.float64)  # exact
    c64 = np.broadcast_to(c.astype(np.float64), prod.shape)
    s64 = prod + c64
    bb = s64 - prod
    err = (prod - (s64 - bb)) + (c64 - bb)  # exact: true sum = s64 + err
    inexact = err != 0
    if np.any(inexact):
        even = (s64.view(np.int64) & 1) == 0
        toward = np.nextafter(s64, np.where(err > 0, np.inf, -np.inf))
        s64 = np.where(inexact & even, toward, s64)
    return s64.astype(np.float32)


# ---------------------------------------------------------------------------
# TOP-K
# ---------------------------------------------------------------------------


def topk_select(scores_valid, k: int) -> np.ndarray:
    """Indices of the k largest entries of ``scores_valid`` (positions [0, n)),
    ordered by (score descending, index ascending); ties go to the lower index;
    fewer than k valid positions -> the tail is -1.

    The reference's radix select (csrc/int3_qk_scores.cu:426-554) returns the same
    *set* when no two scores tie, in an atomics-dependent order; its own gate
    compares value multisets only (scripts/validate_runtime.py:150-151).  The
    deterministic order and tie rule are this build's."""
    s = np.asarray(scores_valid, dtype=np.float32) + np.float32(0.0)  # -0.0 -> +0.0
    n = s.shape[0]
    out = np.full(k, -1, dtype=np.int64)
    if n == 0:
        return out
    order = np.lexsort((np.arange(n), -s.astype(np.float64)))
    m = min(k, n)
    out[:m] = order[:m]
    return out


# ---------------------------------------------------------------------------
# STAGE B, correction, blend
# ---------------------------------------------------------------------------


def softmax_stats(scores_valid):
    """m, 1/Z of csrc/int2_softmax_v.cu:120-143 (m = 0 when not finite; 1/Z = 0 when Z <= 0)."""
    s = np.asarray(scores_valid, dtype=np.float32)
    if s.size == 0:
        return np.float32(0.0), np.float32(0.0)
    m = s.max()
    if not np.isfinite(m):
        m = np.float32(0.0)
    z = np.exp((s - m).astype(np.float64)).sum()
    inv_z = np.float32(1.0 / z) if z > 0 else np.float32(0.0)
    return np.float32(m), inv_z


def stage_b_fp32(scores_valid, v_codes_signed, v_scale_f32, group_size: int, topk_idx):
    """fp32 Stage B (csrc/int2_softmax_v.cu:681-705, 738-788):
    ``p = exp(s - m) / Z``; ``o_hat[d] = sum_p (p * vs[p, g(d)]) * code[p, d]``;
    over the selected set T: ``o_old_unnorm`` likewise and ``W = sum p``.
    Sums are carried in float64 here (the reference's order is atomics-dependent)."""
    s = np.asarray(scores_valid, dtype=np.float32)
    n = s.shape[0]
    o_hat = np.zeros(HEAD_DIM, np.float64)
    o_old = np.zeros(HEAD_DIM, np.float64)
    w_sum = 0.0
    if n:
        m, inv_z = softmax_stats(s)
        p = np.exp((s - m).astype(np.float64)) * float(inv_z)
        vs = np.repeat(np.asarray(v_scale_f32, np.float64), group_size, axis=-1)  # (n, 128)
        v = vs * np.asarray(v_codes_signed, np.float64)
        o_hat = p @ v
        sel = np.asarray(topk_idx)
        sel = sel[(sel >= 0) & (sel < n)]
        if sel.size:
            o_old = p[sel] @ v[sel]
            w_sum = p[sel].sum()
    return o_hat.astype(np.float32), o_old.astype(np.float32), np.float32(w_sum)


def stage_b_int8p(scores_valid, v_codes_signed, v_scale_f32, max_s: int, topk_idx):
    """INT8-P Stage B of the K4V4 batch>1 release plan
    (csrc/int8tc_softmax_v_fused.cu:1049-1053, 1203-1311; model in
    scripts/validate_runtime_edges.py:146-164): positions are cut into 8 splits of
    ``ceil(max_S / 8)``; inside a split, 32-token tiles start at the split's first
    16-token block; per tile ``pv = p * vs``, ``ts = max|pv| / 127``,
    ``pq = clamp(rn(pv / ts), -127, 127)``, ``o_hat += (sum pq * code) * ts``.
    The selected-set terms stay fp32."""
    s = np.asarray(scores_valid, dtype=np.float32)
    n = s.shape[0]
    o_hat = np.zeros(HEAD_DIM, np.float64)
    _, o_old, w_sum = stage_b_fp32(s, v_codes_signed, v_scale_f32, HEAD_DIM, topk_idx)
    if n:
        m, inv_z = softmax_stats(s)
        p = (np.exp((s - m).astype(np.float64)) * float(inv_z)).astype(np.float32)
        vs = np.asarray(v_scale_f32, np.float32).reshape(n)
        pv = p * vs
        codes = np.asarray(v_codes_signed, np.float64)
        chunk = (max_s + 7) // 8
        for sp in range(8):
            lo, hi = sp * chunk, min((sp + 1) * chunk, n)
            if lo >= hi:
                continue
            t0 = (lo // BLOCK) * BLOCK
            while t0 < hi:
                a, b = max(t0, lo), min(t0 + 32, hi)
                if a < b:
                    seg = pv[a:b]
                    ts = np.float32(np.abs(seg).max()) / np.float32(127.0)
                    if ts > 0:
                        pq = np.clip(np.rint(seg * (np.float32(1.0) / ts)), -127, 127)
                        o_hat += (pq.astype(np.float64) @ codes[a:b]) * float(ts)
                t0 += 32
    return o_hat.astype(np.float32), o_old, w_sum


def cpu_correction_row(q_row, k_rows, v_rows, valid, scale):
    """Host correction for one (b, h_q) (csrc/cpu_topk_attn.cpp:602-690):
    invalid slot -> score -inf; ``s = (sum_d q[d] * K[d]) * scale`` in fp32;
    softmax with ``exp``; ``o_new = bf16(sum_k p_k * V_k)``; all-invalid or a
    non-positive / non-finite normaliser -> zeros.  Returns bf16 bits (128,)."""
    q_row = np.asarray(q_row, np.float32)
    k_rows = np.asarray(k_rows, np.float32)
    v_rows = np.asarray(v_rows, np.float32)
    valid = np.asarray(valid, bool)
    if not valid.any():
        return np.zeros(HEAD_DIM, np.uint16)
    dot = np.zeros(k_rows.shape[0], np.float32)
    for d in range(HEAD_DIM):
        dot = dot + q_row[d] * k_rows[:, d]
    s = np.where(valid, dot * np.float32(scale), -np.inf).astype(np.float32)
    mx = s[valid].max()
    e = np.where(valid, np.exp((s - mx).astype(np.float32)), 0).astype(np.float32)
    denom = np.float32(0.0)
    for x in e:
        denom = np.float32(denom + x)
    if not (denom > 0) or not np.isfinite(denom):
        return np.zeros(HEAD_DIM, np.uint16)
    p = e * (np.float32(1.0) / denom)
    out = np.zeros(HEAD_DIM, np.float32)
    for k in range(k_rows.shape[0]):
        if valid[k]:
            out = out + p[k] * v_rows[k]
    return f32_to_bf16_bits(out)


def cpu_correction(q, k_shadow, v_shadow, hmap, ts_buf, scale):
    """csrc/cpu_topk_attn.cpp:854-956 over (B, H_q); mirrors are f32 values
    ``(H_kv, num_slots, 128)``; returns bf16 bits (B, H_q, 128)."""
    b_n, h_n, _ = q.shape
    num_slots = k_shadow.shape[1]
    out = np.zeros((b_n, h_n, HEAD_DIM), np.uint16)
    for b in range(b_n):
        for h in range(h_n):
            slots = np.asarray(ts_buf[b, h], np.int64)
            valid = (slots >= 0) & (slots < num_slots)
            safe = np.where(valid, slots, 0)
            hk = np.asarray(hmap[b, h], np.int64)
            out[b, h] = cpu_correction_row(q[b, h], k_shadow[hk, safe], v_shadow[hk, safe], valid, scale)
    return out


def blend(o_hat, o_old_unnorm, w, o_new_bits):
    """csrc/blend.cu:202-226: ``bf16(o_hat + W * float(o_new) - o_old_unnorm)``, fp32."""
    o_new = bf16_bits_to_f32(o_new_bits)
    v = (np.asarray(o_hat, np.float32) + np.asarray(w, np.float32)[..., None] * o_new).astype(np.float32)
    v = (v - np.asarray(o_old_unnorm, np.float32)).astype(np.float32)
    return v


# ---------------------------------------------------------------------------
# Whole decode step for one layer
# ---------------------------------------------------------------------------

MODES = {
    # name: (k_bits, v_bits, group_size, stage-A arithmetic)
    "k3v2": (3, 2, 64, "bf16"),
    "k4v4": (4, 4, 128, "int8"),
}


def decode_step(mode: str, q, k_data, k_scales, v_data, v_scales, block_table, seq_lens,
                top_k: int, attn_scale: float, *, k_shadow=None, v_shadow=None,
                stage_b: str = "fp32", max_s: int | None = None):
    """One layer of the reference pipeline (adapter/decode_path.py:1712-3237 in the
    order Stage A -> top-k -> Stage B -> host correction -> blend) on CPU.

    q: (B, H_q, 128) f32 values.  Returns a dict with scores (list per b of
    (H_q, len) f32), topk_idx / topk_slots (B, H_q, k) i64, o_hat, o_old_unnorm
    (B, H_q, 128) f32, W, m, inv_z (B, H_q) f32 and, when mirrors are given,
    o_new (bf16 bits) and out (f32 before the final bf16/fp16 store)."""
    kb, vb, gs, arith = MODES[mode]
    q = np.asarray(q, np.float32)
    b_n, h_q, _ = q.shape
    h_kv = k_data.shape[0]
    grp = h_q // h_kv
    if max_s is None:
        max_s = int(np.max(seq_lens)) if len(seq_lens) else 0
    res = dict(scores=[], topk_idx=np.full((b_n, h_q, top_k), -1, np.int64),
               topk_slots=np.full((b_n, h_q, top_k), -1, np.int64),
               o_hat=np.zeros((b_n, h_q, HEAD_DIM), np.float32),
               o_old_unnorm=np.zeros((b_n, h_q, HEAD_DIM), np.float32),
               W=np.zeros((b_n, h_q), np.float32), m=np.zeros((b_n, h_q), np.float32),
               inv_z=np.zeros((b_n, h_q), np.float32))
    for b in range(b_n):
        n = int(min(int(seq_lens[b]), max_s))
        sl = slots_of(block_table, b, n)
        sc_b = np.zeros((h_q, n), np.float32)
        if n == 0:  # padded / inactive row: nothing selected, zero outputs
            res["scores"].append(sc_b)
            continue
        for hk in range(h_kv):
            kd, ks = k_data[hk, sl], k_scales[hk, sl]
            vd, vs = v_data[hk, sl], v_scales[hk, sl]
            v_codes = decode_codes(vd, vb) - offset_of(vb)
            v_sc = bf16_bits_to_f32(vs)
            if arith == "bf16":
                k_hat = dequant(kd, ks, kb, gs, bf16=True)
            else:
                k_codes = decode_codes(kd, kb) - offset_of(kb)
                k_sc = bf16_bits_to_f32(ks).reshape(n)
            for r in range(grp):
                h = hk * grp + r
                if arith == "bf16":
                    s = canonical_scores_bf16path(q[b, h], k_hat, attn_scale)
                else:
                    qi, qs = quantize_query_int8(q[b, h])
                    s = canonical_scores_int8path(qi, qs, k_codes, k_sc, attn_scale)
                sc_b[h] = s
                idx = topk_select(s, top_k)
                res["topk_idx"][b, h] = idx
                res["topk_slots"][b, h] = np.where(idx >= 0, sl[np.maximum(idx, 0)] if n else -1, -1)
                if stage_b == "int8p":
                    oh, oo, w = stage_b_int8p(s, v_codes, v_sc, max_s, idx)
                else:
                    oh, oo, w = stage_b_fp32(s, v_codes, v_sc, gs, idx)
                res["o_hat"][b, h], res["o_old_unnorm"][b, h], res["W"][b, h] = oh, oo, w
                res["m"][b, h], res["inv_z"][b, h] = softmax_stats(s)
        res["scores"].append(sc_b)
    if k_shadow is not None:
        hm = head_map(b_n, h_q, grp, top_k)
        res["o_new"] = cpu_correction(q, k_shadow, v_shadow, hm, res["topk_slots"], attn_scale)
        res["out"] = blend(res["o_hat"], res["o_old_unnorm"], res["W"], res["o_new"])
    return res
