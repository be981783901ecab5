"""Fused decode scan / top-k / finish / merge on the GPU against the CPU oracle.

Gates (stated once): packed bytes and top-k index lists bit-exact; K4V4 scores bit-exact; K3V2
scores within the bound the select kernel itself relies on AND within the reference's own gate
for this tensor (atol = rtol = 2e-5, scripts/validate_runtime.py:147-148 of JetFire); attention
outputs within 2e-3 max-abs + 1e-3 relative, checked on the fp32 value before the 16-bit store
(the store itself must then be a correct rounding of that value).
"""
import numpy as np
import pytest
import torch

from oracle import jf_oracle as O
from jf_testlib import Case, to_bits, f32_values

pytestmark = pytest.mark.gpu

ATOL, RTOL = 2e-3, 1e-3


def _close(got, want, what, atol=ATOL, rtol=RTOL):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    err = np.abs(got - want)
    lim = atol + rtol * np.abs(want)
    assert (err <= lim).all(), f"{what}: max err {err.max():.3e} (limit {lim[np.unravel_index(err.argmax(), err.shape)]:.3e})"


def run_gpu(case: Case, top_k: int, want_scores=True, stage_b="fp32"):
    from jetfire_b200 import ops
    kd, ks, vd, vs = case.device_cache()
    res = ops.fused_attn_topk(case.mode, case.q.cuda(), kd, ks, vd, vs, case.block_table.cuda(),
                              case.seq_lens.cuda(), case.ctx, case.H_q, case.H_kv, 16, top_k,
                              case.attn_scale, want_scores=want_scores, stage_b=stage_b)
    torch.cuda.synchronize()
    return res, (kd, ks, vd, vs)


def k3_score_bound(case: Case, k_scale_bits: np.ndarray, b: int, n: int) -> np.ndarray:
    """Per query head, the bound on |tensor-core score - canonical score| that the select kernel
    derives for a K3V2 row (csrc/topk_select.cu, "delta"): both sums add the same exact products
    in fp32 in different orders, each within (roundings) * 2^-24 * sum|q_d * k_hat_d|, and
    sum|q_d * k_hat_d| <= sum_g 3 * (largest scale of group g in the row) * sum_{d in g} |q_d|."""
    slots = O.slots_of(case.block_table.numpy(), b, n)
    grp = case.H_q // case.H_kv
    out = np.zeros(case.H_q, np.float32)
    q = np.abs(f32_values(case.q)[b]).astype(np.float32) + np.float32(2.0 ** -9)
    for h in range(case.H_q):
        sc = O.bf16_bits_to_f32(k_scale_bits[h // grp, slots])          # (n, 2)
        mag = np.float32(abs(case.attn_scale)) * np.float32(3.0) * (
            sc[:, 0].max() * q[h, :64].sum(dtype=np.float32) + sc[:, 1].max() * q[h, 64:].sum(dtype=np.float32))
        out[h] = mag * np.float32(36.0 / 16777216.0) + np.float32(1e-7)
    return out


def check_case(case: Case, top_k: int, stage_b="fp32"):
    from jetfire_b200 import ops
    res, (kd, ks, vd, vs) = run_gpu(case, top_k, stage_b=stage_b)
    okd, oks, ovd, ovs = case.oracle_cache()
    # the cache the GPU wrote is the oracle's, byte for byte
    assert np.array_equal(kd.cpu().numpy(), okd) and np.array_equal(to_bits(ks), oks)
    assert np.array_equal(vd.cpu().numpy(), ovd) and np.array_equal(to_bits(vs), ovs)
    ref = case.oracle_step(top_k, stage_b=stage_b)
    # top-k: identical lists (order: score desc, position asc), -1 padded
    assert np.array_equal(res.topk_idx.cpu().numpy(), ref["topk_idx"]), "top-k positions differ"
    assert np.array_equal(res.topk_slots.cpu().numpy(), ref["topk_slots"]), "top-k slots differ"
    # approximate scores stay near the canonical ones; -inf past the sequence end
    sc = res.scores.cpu().numpy()
    for b in range(case.B):
        n = min(int(case.seq_lens[b]), case.ctx)
        assert np.isneginf(sc[b, :, n:]).all()
        if n and case.mode == "k4v4":
            # integer MMA + a fixed fp32 rescale order: bit-equal to the oracle
            assert np.array_equal(sc[b, :, :n], ref["scores"][b]), "K4 scores are not bit-exact"
        elif n:
            err = np.abs(sc[b, :, :n] - ref["scores"][b])
            bound = k3_score_bound(case, oks, b, n)
            assert (err <= bound[:, None]).all(), f"K3 scores leave the select kernel's bound: {err.max():.3e} vs {bound.min():.3e}"
            assert np.allclose(sc[b, :, :n], ref["scores"][b], atol=2e-5, rtol=2e-5), \
                f"K3 scores miss the reference's own gate: max err {err.max():.3e}"
    _close(res.o_hat.cpu().numpy(), ref["o_hat"], "o_hat")
    _close(res.o_old_unnorm.cpu().numpy(), ref["o_old_unnorm"], "o_old_unnorm")
    _close(res.W.cpu().numpy(), ref["W"], "W", atol=1e-4, rtol=1e-3)
    # correction merge with the oracle's o_new, then with the product's host correction
    o_new = torch.from_numpy(ref["o_new"].view(np.int16).copy()).view(torch.bfloat16)
    if case.dtype == torch.float16:
        o_new = o_new.float().half()
    out = torch.empty(case.B, case.H_q, 128, dtype=case.dtype, device="cuda")
    ops.blend_unnorm_into(res.o_hat, res.o_old_unnorm, res.W, o_new.cuda(), out)
    want = O.blend(ref["o_hat"], ref["o_old_unnorm"], ref["W"], O.f32_to_bf16_bits(f32_values(o_new)))
    # the gate applies to the fp32 value before the 16-bit store (the oracle's `out` is that value) ...
    pre = (res.o_hat.cpu().numpy() + res.W.cpu().numpy()[..., None] * f32_values(o_new)).astype(np.float32)
    pre = (pre - res.o_old_unnorm.cpu().numpy()).astype(np.float32)
    _close(pre, want, "out before the store")
    # ... and the stored value is a correct rounding of it: within half a unit of the 16-bit type
    # (8 significant bits for bf16: at most 2^-8 relative; 11 for fp16: 2^-11) plus an fp32 unit for the
    # kernel's own operation order
    half_ulp = 2.0 ** -8 if case.dtype == torch.bfloat16 else 2.0 ** -11
    got = out.float().cpu().numpy().astype(np.float64)
    assert (np.abs(got - pre) <= half_ulp * np.abs(pre) + 1e-6).all(), "the merge's store is not a rounding of the fp32 value"
    return res, ref


@pytest.mark.parametrize("B,H_q,H_kv,ctx,top_k,seed", [
    (2, 8, 2, 512, 256, 1),      # the reference's validate_runtime geometry
    (1, 32, 8, 4096, 256, 2),    # Llama-3.1-8B geometry, histogram path
    (2, 16, 2, 2048, 128, 3),    # GQA group 8
    (3, 4, 4, 1024, 64, 4),      # group 1
    (2, 4, 2, 1536, 512, 5),     # group 2, wide k
])
def test_k3v2_matches_oracle(B, H_q, H_kv, ctx, top_k, seed):
    check_case(Case("k3v2", B, H_q, H_kv, ctx, seed=seed), top_k)


@pytest.mark.parametrize("B,H_q,H_kv,ctx,top_k,seed", [
    (2, 8, 2, 512, 256, 31),
    (1, 32, 8, 4096, 256, 32),
    (4, 16, 2, 2048, 128, 33),
    (2, 4, 4, 1024, 64, 34),
])
def test_k4v4_matches_oracle(B, H_q, H_kv, ctx, top_k, seed):
    """Full-precision weights: the reference's K4V4 plan for a configured batch of 1
    (int4_softmax_v_with_pre_corr_wvs2_scores, release_policy.py:453-454)."""
    check_case(Case("k4v4", B, H_q, H_kv, ctx, seed=seed), top_k)


@pytest.mark.parametrize("B,H_q,H_kv,ctx,lens,top_k,seed", [
    (2, 8, 2, 512, None, 256, 31),                 # the reference's validate_runtime geometry, batch 2
    (4, 16, 2, 2048, None, 128, 33),               # aligned tiles (max_S a multiple of 256), ragged ends
    (4, 32, 8, 4096, None, 256, 37),               # the benchmarked geometry at a short context
    (3, 8, 2, 1000, [1000, 999, 17], 64, 38),      # 1000 / 8 = 125: split boundaries cut 16-token blocks
    (2, 8, 2, 336, [336, 40], 32, 39),             # 42-position splits, odd block counts per split
    (3, 8, 4, 48, [48, 1, 0], 32, 40),             # splits shorter than a block
])
def test_k4v4_int8p_matches_the_reference_batched_arithmetic(B, H_q, H_kv, ctx, lens, top_k, seed):
    """The reference's K4V4 plan whenever the configured batch exceeds 1
    (int8tc_softmax_v_with_pre_corr_reg_stats, release_policy.py:443-451): softmax weights times
    the V scale rounded to 127 levels per 32-token tile, tiles laid out over 8 splits of
    ceil(max_S / 8).  o_hat must be within the output gate of THAT arithmetic (its own distance
    to full-precision weights is larger than the gate, so the mode is observable)."""
    case = Case("k4v4", B, H_q, H_kv, ctx, lens=lens, seed=seed)
    res, ref8 = check_case(case, top_k, stage_b="int8p")
    ref32 = case.oracle_step(top_k, with_correction=False)
    d8 = np.abs(res.o_hat.cpu().numpy() - ref8["o_hat"]).max()
    d32 = np.abs(res.o_hat.cpu().numpy() - ref32["o_hat"]).max()
    print(f"k4v4 int8p o_hat max-abs: vs INT8-P oracle {d8:.2e}, vs fp32 oracle {d32:.2e}")
    # check_case has held o_hat to the gate against the INT8-P oracle; against full-precision
    # weights the same result sits further away than it does from its own arithmetic
    assert d8 < d32 or d32 < 1e-4


@pytest.mark.parametrize("mode,stage_b", [("k3v2", "fp32"), ("k4v4", "fp32"), ("k4v4", "int8p")])
def test_gqa_group_of_sixteen(mode, stage_b):
    """The reference's largest GQA ratio (adapter/release_policy.py:31-34, csrc/int3_qk_scores.cu:621-629):
    16 query heads per KV head, handled as two halves of eight that read the same cache rows."""
    check_case(Case(mode, 2, 32, 2, 1536, lens=[1536, 1000], seed=47), 128, stage_b=stage_b)
    check_case(Case(mode, 1, 16, 1, 300, seed=48), 32, stage_b=stage_b)


def test_k4v4_short_and_ragged():
    case = Case("k4v4", 4, 8, 2, 512, lens=[0, 1, 17, 512], seed=35)
    check_case(case, 32)
    check_case(Case("k4v4", 3, 32, 4, 512, lens=[17, 257, 512], seed=36, dtype=torch.float16), 256)


@pytest.mark.parametrize("mode", ["k4v4", "k3v2"])
def test_neighbouring_blocks_and_mixed_tables(mode):
    """Block tables whose consecutive pages sit in neighbouring cache blocks (the K4V4 scan then
    fetches two pages per copy), tables that mix neighbouring and scattered blocks, odd page
    counts and a partial last page."""
    case = Case(mode, 3, 8, 2, 1000, lens=[1000, 777, 33], seed=44, spare_blocks=3)
    per = case.block_table.shape[1]
    ident = torch.arange(case.B * per, dtype=torch.int64).reshape(case.B, per)
    case.block_table = ident.clone()
    check_case(case, 64)
    mixed = ident.clone()
    mixed[0, 5], mixed[0, 6] = ident[0, 6].item(), ident[0, 5].item()   # a descending pair
    mixed[1, 10:20] = ident[1, 10:20].flip(0)                           # a reversed run
    mixed[2, 1] = ident[2, 2].item() + 1                                # a gap of one block (the last one is spare)
    mixed[2, 2] = case.n_blocks - 1
    case.block_table = mixed
    check_case(case, 64)


def test_k3v2_fp16_inputs():
    check_case(Case("k3v2", 2, 8, 2, 1024, seed=11, dtype=torch.float16), 128)


@pytest.mark.parametrize("ctx,lens,top_k,H_q,H_kv", [
    (16, [1], 32, 8, 2),
    (32, [0, 1, 9, 17], 32, 8, 2),
    (512, [17, 257, 512], 256, 32, 4),
    (512, [17, 257, 512], 256, 32, 8),
    (4096, [4096, 4083, 600, 0], 256, 8, 2),
])
def test_k3v2_short_and_ragged(ctx, lens, top_k, H_q, H_kv):
    """Lengths shorter than top_k including 0 and 1 (scripts/validate_runtime_edges.py:229-232):
    every real position once, -1 elsewhere."""
    case = Case("k3v2", len(lens), H_q, H_kv, ctx, lens=lens, seed=21 + ctx)
    res, ref = check_case(case, top_k)
    idx = res.topk_idx.cpu().numpy()
    for b, n in enumerate(lens):
        for h in range(H_q):
            real = idx[b, h][idx[b, h] >= 0]
            assert real.size == min(top_k, n) and np.unique(real).size == real.size
            assert (real < max(n, 1)).all()


def test_k3v2_massive_ties_take_lowest_positions():
    """All-zero keys: every score ties at 0, so the k lowest positions win (slow exact path)."""
    case = Case("k3v2", 1, 8, 2, 2048, seed=5)
    case.k_full.zero_()
    res, ref = check_case(case, 64)
    assert np.array_equal(res.topk_idx.cpu().numpy()[0, 0], np.arange(64))


def test_phases_one_by_one_equal_fused():
    from jetfire_b200 import ops
    case = Case("k3v2", 2, 8, 2, 1024, seed=8)
    kd, ks, vd, vs = case.device_cache()
    args = (case.mode, case.q.cuda(), kd, ks, vd, vs, case.block_table.cuda(), case.seq_lens.cuda(),
            case.ctx, case.H_q, case.H_kv, 16, 128, case.attn_scale)
    fused = ops.fused_attn_topk(*args)
    call = ops.DecodeCall(*args)
    call.scan(); call.select(); call.finish(); call.status()
    step = call.result()
    for a, b in zip(fused[:7], step[:7]):
        assert torch.equal(a, b)


def test_phases_one_by_one_equal_fused_k4v4_long_row():
    """Long enough for the histogram tiers (ctx > 2 * top_k); K4V4; both kernels must agree bit for bit."""
    from jetfire_b200 import ops
    case = Case("k4v4", 2, 8, 2, 4096, seed=18)
    kd, ks, vd, vs = case.device_cache()
    args = (case.mode, case.q.cuda(), kd, ks, vd, vs, case.block_table.cuda(), case.seq_lens.cuda(),
            case.ctx, case.H_q, case.H_kv, 16, 256, case.attn_scale)
    fused = ops.fused_attn_topk(*args)
    call = ops.DecodeCall(*args)
    call.scan(); call.select(); call.finish(); call.status()
    step = call.result()
    for a, b in zip(fused[:7], step[:7]):
        assert torch.equal(a, b)


@pytest.mark.parametrize("mode,ctx,top_k", [("k3v2", 1024, 128), ("k4v4", 4096, 256), ("k3v2", 32768, 256)])
def test_slots_as_32_bit_integers_equal_the_64_bit_list(mode, ctx, top_k):
    """The optional int32 copy of the selected slots (-1 padding included) equals the int64 list, from
    the fused call and from the stand-alone select, in both select kernels; the phase-by-phase
    results of a long K3V2 row (page-maxima select) equal the fused call's bit for bit."""
    from jetfire_b200 import ops
    case = Case(mode, 2, 8, 2, ctx, lens=[ctx, max(top_k // 2, ctx // 3 - 5)], seed=19)
    kd, ks, vd, vs = case.device_cache()
    args = (case.mode, case.q.cuda(), kd, ks, vd, vs, case.block_table.cuda(), case.seq_lens.cuda(),
            case.ctx, case.H_q, case.H_kv, 16, top_k, case.attn_scale)
    call = ops.DecodeCall(*args, slots_i32=True)
    call.fused(); call.status()
    fused = [t.clone() for t in call.result()[:7]]
    s32 = call.out["topk_slots_i32"].clone()
    assert s32.dtype == torch.int32 and torch.equal(s32.to(torch.int64), fused[1])
    call.out["topk_slots_i32"].fill_(-7)
    call.scan(); call.select(); call.finish(); call.status()
    assert torch.equal(call.out["topk_slots_i32"], s32)
    for a, b in zip(fused, call.result()[:7]):
        assert torch.equal(a, b)


def test_status_record_is_read_once_and_needs_no_initialisation():
    """The workspace's status record counts only when tagged; reading an error clears it.
    The record is written from the host here: no kernel is made to time out."""
    import struct
    from jetfire_b200 import ops
    case = Case("k3v2", 1, 8, 2, 256, seed=3)
    kd, ks, vd, vs = case.device_cache()
    nbytes = ops.decode_workspace_bytes("k3v2", 1, case.H_q, case.H_kv, case.ctx, 32) + 256
    ws = torch.full((nbytes,), 0xA5, dtype=torch.uint8, device="cuda")     # garbage, never zeroed
    call = ops.DecodeCall(case.mode, case.q.cuda(), kd, ks, vd, vs, case.block_table.cuda(), case.seq_lens.cuda(),
                          case.ctx, case.H_q, case.H_kv, 16, 32, case.attn_scale, workspace=ws)
    call.fused()
    call.status()                                                           # untagged garbage reads as ok
    off = (ws.data_ptr() + 255) // 256 * 256 - ws.data_ptr()
    rec = struct.pack("<Qii", 0x4A46535441545553, 2, 0)                     # tag, JF_ERR_TIMEOUT
    ws[off:off + 16] = torch.tensor(list(rec), dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError):
        call.status()
    call.status()                                                           # cleared by the read


def test_stream_ordered_host_correction_matches_blocking_call():
    """stream_submit / stream_wait (host callbacks in the CUDA stream) around the slot copy and
    the merge give the blocking path's result, for several layers queued without host syncs."""
    from jetfire_b200 import ops
    case = Case("k3v2", 2, 8, 2, 1024, seed=71)
    kd, ks, vd, vs = case.device_cache()
    top_k, n_layers = 64, 4
    g = torch.Generator().manual_seed(5)
    qs = [torch.randn(case.B, case.H_q, 128, generator=g).to(case.dtype).pin_memory() for _ in range(n_layers)]
    main, side = torch.cuda.current_stream(), torch.cuda.Stream()
    layers = []
    for q_host in qs:
        q = q_host.cuda()
        call = ops.DecodeCall(case.mode, q, kd, ks, vd, vs, case.block_table.cuda(), case.seq_lens.cuda(),
                              case.ctx, case.H_q, case.H_kv, 16, top_k, case.attn_scale)
        slots_host = torch.empty(case.B, case.H_q, top_k, dtype=torch.int64).pin_memory()
        o_new_host = torch.zeros(case.B, case.H_q, 128, dtype=case.dtype).pin_memory()
        host = ops.HostCorrectionCall(q_host, case.k_full, case.v_full, None, slots_host, o_new_host, case.attn_scale)
        layers.append((call, slots_host, o_new_host, host, torch.empty_like(q), torch.empty_like(q), torch.cuda.Event()))
    ops.set_cpu_attn_threads(4)
    for call, slots_host, o_new_host, host, o_new, out, ev in layers:      # everything queued, no host sync
        call.fused()
        slots_host.copy_(call.out["topk_slots"], non_blocking=True)
        host.stream_submit(main)
        ev.record(main)
        side.wait_event(ev)
        host.stream_wait(side)
        with torch.cuda.stream(side):
            o_new.copy_(o_new_host, non_blocking=True)
            ops.blend_unnorm_into(call.out["o_hat"], call.out["o_old_unnorm"], call.out["W"], o_new, out)
    torch.cuda.synchronize()
    for call, slots_host, o_new_host, host, o_new, out, ev in layers:
        host.stream_status()
        want_new = torch.empty_like(o_new_host)
        ops.cpu_topk_attn(host._keep[0], case.k_full, case.v_full, None, slots_host, want_new, case.attn_scale)
        assert torch.equal(o_new_host, want_new)
        want = torch.empty_like(out)
        ops.blend_unnorm_into(call.out["o_hat"], call.out["o_old_unnorm"], call.out["W"], want_new.cuda(), want)
        assert torch.equal(out, want)
        host.close()


def test_reference_named_ops_int2_fused_and_wait_and_blend():
    """``int2_fused_attn_topk`` (reference name and argument order) and ``wait_and_blend_unnorm_into``
    over a mapped o_new / completion flag give the plain calls' results."""
    from jetfire_b200 import ops
    case = Case("k4v4", 2, 8, 2, 1024, seed=81)
    kd, ks, vd, vs = case.device_cache()
    qd, bt, sl = case.q.cuda(), case.block_table.cuda(), case.seq_lens.cuda()
    o_hat, slots, o_old, W = ops.int2_fused_attn_topk(qd, kd, ks, None, vd, vs, bt, sl, case.ctx, case.H_q, case.H_kv,
                                                      16, 64, case.attn_scale)
    ref = ops.fused_attn_topk("k4v4", qd, kd, ks, vd, vs, bt, sl, case.ctx, case.H_q, case.H_kv, 16, 64, case.attn_scale)
    assert torch.equal(o_hat, ref.o_hat) and torch.equal(slots, ref.topk_slots)
    assert torch.equal(o_old, ref.o_old_unnorm) and torch.equal(W, ref.W)
    with pytest.raises(RuntimeError):
        ops.int2_fused_attn_topk(qd, kd, ks, torch.zeros(1), vd, vs, bt, sl, case.ctx, case.H_q, case.H_kv, 16, 64,
                                 case.attn_scale)
    o_new_host, o_new_dev = ops.alloc_mapped_pinned_pair((case.B, case.H_q, 128), case.dtype)
    flag = torch.zeros(1, dtype=torch.int64)
    ops.set_cpu_attn_threads(3)
    ops.cpu_topk_attn_submit(case.q, case.k_full, case.v_full, None, slots.cpu(), o_new_host, case.attn_scale, flag)
    out = torch.empty(case.B, case.H_q, 128, dtype=case.dtype, device="cuda")
    ops.wait_and_blend_unnorm_into(flag, o_hat, o_old, W, o_new_dev, out)
    torch.cuda.synchronize()
    want = torch.empty_like(out)
    ops.blend_unnorm_into(o_hat, o_old, W, o_new_host.cuda(), want)
    assert torch.equal(out, want)
    never = torch.zeros(1, dtype=torch.int64)
    with pytest.raises(RuntimeError):
        ops.wait_and_blend_unnorm_into(never, o_hat, o_old, W, o_new_dev, out, timeout_s=0.05)


@pytest.mark.parametrize("mode,stage_b", [("k3v2", "fp32"), ("k4v4", "fp32"), ("k4v4", "int8p")])
def test_reference_call_order_through_the_reference_named_ops(mode, stage_b):
    """The reference's decode step, op by op and under its own op names (adapter/decode_path.py:
    2081-2131 Stage A, :2237-2257 the copies to pinned memory, :2499-2528 the stream-ordered submit,
    :2785-2935 Stage B, :3069-3070 the join, :3137-3163 the blend), gives the bits of the one-call
    fused step followed by the blocking host correction."""
    from jetfire_b200 import ops
    case = Case(mode, 3, 8, 2, 1500, lens=[1500, 1487, 40], seed=91)
    kd, ks, vd, vs = case.device_cache()
    qd, bt, sl = case.q.cuda(), case.block_table.cuda(), case.seq_lens.cuda()
    top_k, scale = 64, case.attn_scale
    geom = (case.ctx, case.H_q, case.H_kv, 16)
    # -- the one-call form --
    fused = ops.fused_attn_topk(mode, qd, kd, ks, vd, vs, bt, sl, *geom, top_k, scale, want_scores=True, stage_b=stage_b)
    want_new = torch.empty(case.B, case.H_q, 128, dtype=case.dtype)
    ops.set_cpu_attn_threads(3)
    ops.cpu_topk_attn(case.q, case.k_full, case.v_full, None, fused.topk_slots.cpu(), want_new, scale)
    want_out = torch.empty(case.B, case.H_q, 128, dtype=case.dtype, device="cuda")
    ops.blend_unnorm_into(fused.o_hat, fused.o_old_unnorm, fused.W, want_new.cuda(), want_out)
    # -- the reference's sequence --
    stream = torch.cuda.current_stream().cuda_stream
    q_buf = torch.empty(case.B, case.H_q, 128, dtype=case.dtype).pin_memory()
    ts_buf = torch.empty(case.B, case.H_q, top_k, dtype=torch.int64).pin_memory()
    o_new_host, o_new_dev = ops.alloc_mapped_pinned_pair((case.B, case.H_q, 128), case.dtype)
    flag_host, flag_dev = ops.alloc_mapped_pinned_pair((1,), torch.int64)
    flag_host.fill_(7)
    head_map = torch.from_numpy(O.head_map(case.B, case.H_q, case.H_q // case.H_kv, top_k))
    handle = ops.create_cpu_topk_submit_ctx(q_buf, case.k_full, case.v_full, head_map, ts_buf, o_new_host, scale, flag_host)
    if mode == "k3v2":
        scores, topk_idx, topk_slots = ops.int3_qk_scores_topk(qd, kd, ks, bt, sl, *geom, scale, top_k)
    else:
        scores, topk_idx, topk_slots, m, inv_z = ops.int8tc_qk_scores_topk_stats(qd, kd, ks, bt, sl, *geom, scale, top_k)
    q_buf.copy_(qd, non_blocking=True)
    ts_buf.copy_(topk_slots, non_blocking=True)
    ops.stream_write_value64(stream, flag_dev, 0)
    ops.stream_submit_cpu_topk_attn(stream, handle)
    if mode == "k3v2":
        o_hat, o_old, W = ops.int2_softmax_v_with_pre_corr_wvs2(scores, vd, vs, bt, sl, topk_idx, *geom, top_k)
    elif stage_b == "int8p":
        o_hat, o_old, W = ops.int8tc_softmax_v_with_pre_corr_reg_stats(scores, m, inv_z, vd, vs, bt, sl, topk_idx, *geom, top_k)
    else:
        o_hat, o_old, W = ops.int4_softmax_v_with_pre_corr_wvs2_scores(scores, vd, vs, bt, sl, topk_idx, *geom, top_k)
    ops.stream_wait_cpu_topk_attn(stream, handle)
    out = torch.empty(case.B, case.H_q, 128, dtype=case.dtype, device="cuda")
    ops.blend_unnorm_into(o_hat, o_old, W, o_new_dev, out)
    torch.cuda.synchronize()
    assert int(flag_host[0]) == 1, "the submit context did not publish completion"
    assert torch.equal(scores, fused.scores) and torch.equal(topk_idx, fused.topk_idx) and torch.equal(topk_slots, fused.topk_slots)
    assert torch.equal(o_hat, fused.o_hat) and torch.equal(o_old, fused.o_old_unnorm) and torch.equal(W, fused.W)
    assert torch.equal(o_new_host, want_new) and torch.equal(out, want_out)
    if mode == "k4v4":
        # the statistics outputs: exact row maximum and 1 / sum exp(s - max), empty rows -> (0, 0)
        sc = scores.cpu().numpy()
        for b in range(case.B):
            n = int(case.seq_lens[b])
            mx = sc[b, :, :n].max(axis=1)
            np.testing.assert_array_equal(m[b].cpu().numpy(), mx)
            z = np.exp((sc[b, :, :n] - mx[:, None]).astype(np.float64)).sum(axis=1)
            np.testing.assert_allclose(inv_z[b].cpu().numpy(), 1.0 / z, rtol=1e-5)
    # caller-owned outputs (the reference's _inplace variant); `weights` is accepted and ignored
    if mode == "k3v2":
        o2, old2, w2 = torch.full_like(o_hat, 9.0), torch.full_like(o_old, 9.0), torch.full_like(W, 9.0)
        ops.int2_softmax_v_with_pre_corr_wvs2_inplace(scores, vd, vs, bt, sl, topk_idx, torch.empty(1, device="cuda"),
                                                      o2, old2, w2, *geom, top_k)
        assert torch.equal(o2, o_hat) and torch.equal(old2, o_old) and torch.equal(w2, W)


def test_reference_named_shadow_append_scatters_staged_rows_in_stream_order():
    """create_shadow_append_submit_ctx / stream_submit_shadow_append with the reference's contract
    (csrc/cpu_topk_attn.cpp:1611-1665): the caller's stream-ordered copies fill pinned staging, the
    queued host callback scatters the staged rows into the mirror, padding slots are skipped."""
    from jetfire_b200 import ops
    g = torch.Generator().manual_seed(12)
    T, H_kv, num_slots = 5, 2, 64
    key = torch.randn(T, H_kv, 128, generator=g).to(torch.bfloat16).cuda()
    val = torch.randn(T, H_kv, 128, generator=g).to(torch.bfloat16).cuda()
    slots = torch.tensor([3, -1, 63, 64, 10], dtype=torch.int64, device="cuda")
    k_app, v_app = torch.empty(T, H_kv, 128, dtype=torch.bfloat16).pin_memory(), torch.empty(T, H_kv, 128, dtype=torch.bfloat16).pin_memory()
    s_app = torch.empty(T, dtype=torch.int64).pin_memory()
    k_sh, v_sh = torch.zeros(H_kv, num_slots, 128, dtype=torch.bfloat16), torch.zeros(H_kv, num_slots, 128, dtype=torch.bfloat16)
    h = ops.create_shadow_append_submit_ctx(k_app, v_app, s_app, k_sh, v_sh)
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        k_app.copy_(key, non_blocking=True); v_app.copy_(val, non_blocking=True); s_app.copy_(slots, non_blocking=True)
        ops.stream_submit_shadow_append(stream, h)
    torch.cuda.synchronize()
    assert ops.get_shadow_append_count(h) == 2
    for t, s_ in ((0, 3), (2, 63), (4, 10)):
        assert torch.equal(k_sh[:, s_], key[t].cpu()) and torch.equal(v_sh[:, s_], val[t].cpu())
    rest = [s_ for s_ in range(num_slots) if s_ not in (3, 63, 10)]
    assert not k_sh[:, rest].any() and not v_sh[:, rest].any()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("slot_dtype", [torch.int64, torch.int32])
def test_correction_rows_on_the_gpu_over_the_host_mirror(dtype, slot_dtype):
    """A range of the correction's rows computed by the GPU straight from the host mirror (mapped
    pinned memory) agrees with the host correction to the rounding of the 16-bit result; entries
    that are negative or beyond the cache are skipped, a row without a valid entry gives zeros,
    rows outside the range are not touched; host rows + GPU rows together are the full result."""
    from jetfire_b200 import ops
    g = torch.Generator().manual_seed(13)
    B, H_q, H_kv, K, slots = 3, 16, 2, 37, 4096          # K neither a multiple of 4 nor of the unrolling
    k_host, k_dev = ops.alloc_mapped_pinned_pair((H_kv, slots, 128), dtype)
    v_host, v_dev = ops.alloc_mapped_pinned_pair((H_kv, slots, 128), dtype)
    k_host.copy_(torch.randn(H_kv, slots, 128, generator=g).to(dtype))
    v_host.copy_(torch.randn(H_kv, slots, 128, generator=g).to(dtype))
    q = torch.randn(B, H_q, 128, generator=g).to(dtype)
    ts = torch.randint(0, slots, (B, H_q, K), generator=g, dtype=slot_dtype)
    ts[0, 3, ::5] = -1                                     # padding of a short sequence
    ts[1, 0, 7] = slots + 5                                # beyond the cache
    ts[2, 9, :] = -1                                       # nothing valid at all
    want = torch.empty_like(q)
    ops.set_cpu_attn_threads(3)
    ops.cpu_topk_attn(q, k_host, v_host, None, ts, want, 0.11)
    rows = B * H_q
    got = torch.full((B, H_q, 128), 7.0, dtype=dtype, device="cuda")
    ops.gpu_topk_attn_rows(q.cuda(), k_dev, v_dev, ts.cuda(), got, 0.11, (5, rows - 2))
    torch.cuda.synchronize()
    gotc, wantc = got.cpu().view(rows, 128).float(), want.view(rows, 128).float()
    assert bool((gotc[:5] == 7).all()) and bool((gotc[rows - 2:] == 7).all())
    err = (gotc[5:rows - 2] - wantc[5:rows - 2]).abs()
    lim = 1e-3 + 2.0 ** -7 * wantc[5:rows - 2].abs()
    assert bool((err <= lim).all()), f"max err {float(err.max()):.3e}"
    assert not gotc[2 * H_q + 9].any()                     # the row without a valid entry
    # the split the end-to-end loop uses: the host takes the first rows, the GPU the rest
    cut = 29
    both_host = torch.full_like(q, 7.0).pin_memory()
    both = torch.full((B, H_q, 128), 7.0, dtype=dtype, device="cuda")
    call = ops.HostCorrectionCall(q, k_host, v_host, None, ts, both_host, 0.11, rows=(0, cut))
    ticket = call.submit()
    ops.gpu_topk_attn_rows(q.cuda(), k_dev, v_dev, ts.cuda(), both, 0.11, (cut, rows))
    call.wait_ticket(ticket)
    both.view(rows, 128)[:cut].copy_(both_host.view(rows, 128)[:cut])
    torch.cuda.synchronize()
    bc = both.cpu().view(rows, 128).float()
    assert torch.equal(bc[:cut], wantc[:cut])
    assert bool(((bc[cut:] - wantc[cut:]).abs() <= 1e-3 + 2.0 ** -7 * wantc[cut:].abs()).all())
    ops.gpu_topk_attn_rows(q.cuda(), k_dev, v_dev, ts.cuda(), both, 0.11, (4, 4))      # an empty range is a no-op
    with pytest.raises(RuntimeError):
        ops.gpu_topk_attn_rows(q.cuda(), k_dev, v_dev, ts.cuda(), both, 0.11, (0, rows + 1))
