"""This library against the reference's OWN GPU kernels, compiled from their unmodified sources
for sm_100 by ``oracle/build_oracle.py`` (the two ``int8tc_*`` files with only the architecture
flag of their loader changed), on the same bf16 inputs.

Gates are the reference's own (scripts/validate_runtime.py:143-195 of JetFire) where this
library follows the same arithmetic -- scores atol = rtol = 2e-5; top-k compared as value
multisets, with the boundary gap reported for any index that differs; blend within one 16-bit
unit -- and this project's output gate (2e-3 max-abs + 1e-3 relative) for Stage B, whose
weights meet V as 16-bit floats here and as fp32 there.  The same files pin the numpy / C
restatement that every other parity test uses.

Skipped when the reference extensions were not built (no reference checkout at build time).
"""
import numpy as np
import pytest
import torch

from oracle import native
from jf_testlib import Case

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2e-3, 1e-3


def _need(name):
    mod = native.ref_gpu_module(name)
    if mod is None:
        pytest.skip(f"reference extension {name} not built on this machine")
    return mod


def _inputs(mode, B, H_q, H_kv, ctx, lens, seed):
    case = Case(mode, B, H_q, H_kv, ctx, lens=lens, seed=seed)
    kd, ks, vd, vs = case.device_cache()
    return case, (case.q.cuda(), kd, ks, vd, vs, case.block_table.cuda(), case.seq_lens.cuda())


def _close(got, want, what, atol=ATOL, rtol=RTOL):
    got, want = got.double().cpu().numpy(), want.double().cpu().numpy()
    err = np.abs(got - want)
    assert (err <= atol + rtol * np.abs(want)).all(), f"{what}: max err {err.max():.3e}"
    return err.max()


def _compare_topk(ref_scores, ref_idx, my_idx, lens, what):
    """Both lists must select the same multiset of reference scores; where the index sets differ
    (two scores closer than the tensor-core summation noise), report the gap at the boundary."""
    rs = ref_scores.cpu().numpy()
    ri, mi = ref_idx.cpu().numpy(), my_idx.cpu().numpy()
    differing, worst_gap = 0, 0.0
    for b in range(rs.shape[0]):
        n = int(lens[b])
        for h in range(rs.shape[1]):
            a, c = ri[b, h][ri[b, h] >= 0], mi[b, h][mi[b, h] >= 0]
            assert a.size == c.size == min(ri.shape[2], n), f"{what}: list lengths differ at ({b},{h})"
            if a.size == 0:
                continue
            va, vc = np.sort(rs[b, h, a]), np.sort(rs[b, h, c])
            assert np.allclose(va, vc, atol=2e-5, rtol=2e-5), f"{what}: selected score multisets differ at ({b},{h})"
            only = np.setxor1d(a, c)
            if only.size:
                differing += 1
                kth = va[0]
                worst_gap = max(worst_gap, float(np.abs(rs[b, h, only] - kth).max()))
    print(f"{what}: rows whose index sets differ from the reference's: {differing}, largest gap to the k-th score {worst_gap:.2e}")
    assert worst_gap < 1e-4


@pytest.mark.parametrize("B,H_q,H_kv,ctx,lens,top_k,seed", [
    (2, 8, 2, 512, None, 256, 1),           # the reference's validation geometry
    (2, 32, 8, 4096, None, 256, 2),         # Llama-3.1-8B geometry
    (3, 16, 2, 2048, [2048, 700, 17], 64, 3),
])
def test_k3v2_against_the_reference_kernels(B, H_q, H_kv, ctx, lens, top_k, seed):
    from jetfire_b200 import ops
    qk, sv = _need("int3_qk_scores"), _need("int2_softmax_v")
    case, (q, kd, ks, vd, vs, bt, sl) = _inputs("k3v2", B, H_q, H_kv, ctx, lens, seed)
    geom = (ctx, H_q, H_kv, 16)
    r_scores, r_idx, r_slots = qk.int3_qk_scores_topk(q, kd, ks, bt, sl, *geom, case.attn_scale, top_k)
    mine = ops.fused_attn_topk("k3v2", q, kd, ks, vd, vs, bt, sl, *geom, top_k, case.attn_scale, want_scores=True)
    torch.cuda.synchronize()
    for b in range(B):
        n = int(case.seq_lens[b])
        assert torch.allclose(mine.scores[b, :, :n], r_scores[b, :, :n], atol=2e-5, rtol=2e-5), "scores"
        assert torch.isneginf(r_scores[b, :, n:]).all() and torch.isneginf(mine.scores[b, :, n:]).all()
    _compare_topk(r_scores, r_idx, mine.topk_idx, case.seq_lens, "K3 top-k")
    # Stage B of the reference on the reference's scores and THIS library's selection
    r_hat, r_old, r_w = sv.int2_softmax_v_with_pre_corr_wvs2(r_scores, vd, vs, bt, sl, mine.topk_idx, *geom, top_k)
    torch.cuda.synchronize()
    e1 = _close(mine.o_hat, r_hat, "o_hat")
    e2 = _close(mine.o_old_unnorm, r_old, "o_old_unnorm")
    e3 = _close(mine.W, r_w, "W", atol=1e-4)
    print(f"K3V2 vs reference kernels: o_hat {e1:.2e}, o_old_unnorm {e2:.2e}, W {e3:.2e}")


@pytest.mark.parametrize("B,H_q,H_kv,ctx,lens,top_k,seed", [
    (2, 8, 2, 512, None, 256, 31),
    (4, 32, 8, 4096, None, 256, 32),
    (3, 16, 2, 2048, [2048, 700, 17], 64, 33),
])
def test_k4v4_against_the_reference_kernels(B, H_q, H_kv, ctx, lens, top_k, seed):
    from jetfire_b200 import ops
    qk, sv8, sv4 = _need("int8tc_qk_scores"), _need("int8tc_softmax_v_fused"), _need("int4_softmax_v")
    case, (q, kd, ks, vd, vs, bt, sl) = _inputs("k4v4", B, H_q, H_kv, ctx, lens, seed)
    geom = (ctx, H_q, H_kv, 16)
    r_scores, r_idx, r_slots, r_m, r_iz = qk.int8tc_qk_scores_topk_stats(q, kd, ks, bt, sl, *geom, case.attn_scale, top_k)
    mine = ops.fused_attn_topk("k4v4", q, kd, ks, vd, vs, bt, sl, *geom, top_k, case.attn_scale, want_scores=True)
    mine8 = ops.fused_attn_topk("k4v4", q, kd, ks, vd, vs, bt, sl, *geom, top_k, case.attn_scale, stage_b="int8p")
    torch.cuda.synchronize()
    same = 0.0
    for b in range(B):
        n = int(case.seq_lens[b])
        assert torch.allclose(mine.scores[b, :, :n], r_scores[b, :, :n], atol=2e-5, rtol=2e-5), "scores"
        same += float((mine.scores[b, :, :n] == r_scores[b, :, :n]).float().mean()) / B
    print(f"K4 scores bit-equal to the reference kernel's: {100 * same:.2f} %")
    _compare_topk(r_scores, r_idx, mine.topk_idx, case.seq_lens, "K4 top-k")
    # configured batch 1: fp32 weights; above 1: weights rounded per 32-token tile
    r_hat, r_old, r_w = sv4.int4_softmax_v_with_pre_corr_wvs2_scores(r_scores, vd, vs, bt, sl, mine.topk_idx, *geom, top_k)
    q_hat, q_old, q_w = sv8.int8tc_softmax_v_with_pre_corr_reg_stats(r_scores, r_m, r_iz, vd, vs, bt, sl, mine.topk_idx,
                                                                     *geom, top_k)
    torch.cuda.synchronize()
    e1 = _close(mine.o_hat, r_hat, "o_hat (fp32 weights)")
    _close(mine.o_old_unnorm, r_old, "o_old_unnorm")
    _close(mine.W, r_w, "W", atol=1e-4)
    e2 = _close(mine8.o_hat, q_hat, "o_hat (weights rounded per tile)")
    _close(mine8.o_old_unnorm, q_old, "o_old_unnorm (tile variant)")
    _close(mine8.W, q_w, "W (tile variant)", atol=1e-4)
    gap = float((q_hat - r_hat).abs().max())
    print(f"K4V4 vs reference kernels: o_hat fp32 {e1:.2e}, per-tile {e2:.2e}; the reference's two variants differ by {gap:.2e}")


def test_blend_against_the_reference_kernel():
    from jetfire_b200 import ops
    ref = _need("blend")
    g = torch.Generator(device="cuda").manual_seed(5)
    o_hat = torch.randn(4, 32, 128, generator=g, device="cuda")
    o_old = 0.3 * torch.randn(4, 32, 128, generator=g, device="cuda")
    W = torch.rand(4, 32, generator=g, device="cuda")
    o_new = torch.randn(4, 32, 128, generator=g, device="cuda").to(torch.bfloat16)
    a, b = torch.empty_like(o_new), torch.empty_like(o_new)
    ref.blend_unnorm_into(o_hat, o_old, W, o_new, a)
    ops.blend_unnorm_into(o_hat, o_old, W, o_new, b)
    torch.cuda.synchronize()
    # the same three fp32 operations; a different contraction can move a result by one 16-bit unit at most
    diff = (a.float() - b.float()).abs()
    assert (diff <= 2.0 ** -7 * a.float().abs() + 1e-6).all()
    assert float((a == b).float().mean()) > 0.999
