"""The oracle's native pieces agree with the numpy restatement, and the host correction
(product C++ vs the reference's own cpu_topk_attn.cpp compiled unmodified vs numpy)."""
import numpy as np
import pytest
import torch

from oracle import jf_oracle as O
from oracle import native
from jf_testlib import Case, f32_values


@pytest.mark.parametrize("mode,seed", [("k3v2", 3), ("k4v4", 4)])
def test_c_restatement_equals_numpy(mode, seed):
    case = Case(mode, 3, 8, 2, 700, lens=[700, 0, 333], seed=seed)
    ref = case.oracle_step(64, with_correction=False)
    kd, ks, vd, vs = case.oracle_cache()
    c = native.c_decode(mode, f32_values(case.q), kd, ks, vd, vs, case.block_table.numpy(),
                        case.seq_lens.numpy(), case.ctx, 64, case.attn_scale, n_threads=2, want_scores=True)
    assert np.array_equal(c["topk_idx"], ref["topk_idx"])
    assert np.array_equal(c["topk_slots"], ref["topk_slots"])
    for b in range(case.B):
        n = int(case.seq_lens[b])
        assert np.array_equal(c["scores"][b][:, :n], ref["scores"][b])
    np.testing.assert_allclose(c["o_hat"], ref["o_hat"], atol=2e-6)
    np.testing.assert_allclose(c["o_old_unnorm"], ref["o_old_unnorm"], atol=2e-6)
    np.testing.assert_allclose(c["W"], ref["W"], atol=2e-6)


@pytest.mark.parametrize("ctx,lens,seed", [(1024, [1024, 513, 17], 14), (1000, [1000, 999, 0], 15), (336, [336, 40], 16)])
def test_c_int8p_stage_b_equals_numpy(ctx, lens, seed):
    """The C restatement of the K4V4 batch > 1 Stage B (weights rounded per 32-token tile, tiles laid
    out over the reference's 8 splits) against the numpy one, with max_S that cuts 16-token blocks
    between splits (1000 / 8 = 125) as well as aligned ones."""
    case = Case("k4v4", len(lens), 8, 2, ctx, lens=lens, seed=seed)
    ref = case.oracle_step(32, stage_b="int8p", with_correction=False)
    kd, ks, vd, vs = case.oracle_cache()
    c = native.c_decode("k4v4", f32_values(case.q), kd, ks, vd, vs, case.block_table.numpy(),
                        case.seq_lens.numpy(), case.ctx, 32, case.attn_scale, n_threads=2, stage_b="int8p")
    assert np.array_equal(c["topk_idx"], ref["topk_idx"])
    # the two differ only in the float type of exp (and so, rarely, in one rounding step of one weight)
    np.testing.assert_allclose(c["o_hat"], ref["o_hat"], atol=2e-5)
    np.testing.assert_allclose(c["o_old_unnorm"], ref["o_old_unnorm"], atol=2e-6)
    np.testing.assert_allclose(c["W"], ref["W"], atol=2e-6)
    fp32 = case.oracle_step(32, with_correction=False)
    assert np.abs(ref["o_hat"] - fp32["o_hat"]).max() > 1e-4, "the rounding must be visible against fp32 weights"


def _correction_inputs(dtype=torch.bfloat16, K=64):
    case = Case("k3v2", 2, 8, 2, 512, seed=9, dtype=dtype)
    g = torch.Generator().manual_seed(1)
    slots = torch.randint(0, case.num_slots, (2, 8, K), generator=g, dtype=torch.int64)
    slots[0, 0, 5:] = -1                 # mostly padded row
    slots[1, 3, :] = -1                  # all invalid -> zeros
    slots[1, 4, 7] = case.num_slots + 3  # out of range -> skipped
    return case, slots


def test_product_correction_matches_numpy_oracle():
    from jetfire_b200 import ops
    for dtype, K in ((torch.bfloat16, 64), (torch.float16, 64), (torch.bfloat16, 70), (torch.float16, 33)):
        case, slots = _correction_inputs(dtype, K)
        hm = torch.from_numpy(O.head_map(2, 8, 4, slots.shape[2]))
        out = torch.full((2, 8, 128), 7.0, dtype=dtype)
        flag = torch.zeros(1, dtype=torch.int64)
        ops.set_cpu_attn_threads(3)
        ops.cpu_topk_attn(case.q, case.k_full, case.v_full, hm, slots, out, case.attn_scale, flag)
        assert int(flag[0]) == 1, "completion flag was not set"
        want = O.bf16_bits_to_f32(O.cpu_correction(f32_values(case.q), f32_values(case.k_full),
                                                   f32_values(case.v_full), hm.numpy(), slots.numpy(),
                                                   case.attn_scale))
        # the reference's own gate for this op: atol 2e-3, rtol 6e-3 (scripts/validate_runtime.py:178-191)
        np.testing.assert_allclose(out.float().numpy(), want, atol=2e-3, rtol=6e-3)
        assert bool((out[1, 3] == 0).all())


def test_reference_correction_pins_oracle_and_product():
    mod = native.ref_cpu_topk_attn_module()
    if mod is None:
        pytest.skip("reference extension not built on this machine")
    from jetfire_b200 import ops
    case, slots = _correction_inputs()
    hm = torch.from_numpy(O.head_map(2, 8, 4, slots.shape[2]))
    ref_out = torch.empty(2, 8, 128, dtype=torch.bfloat16)
    mod.set_cpu_attn_threads(2)
    mod.cpu_topk_attn(case.q, case.k_full, case.v_full, hm, slots, ref_out, case.attn_scale, None)
    want = O.bf16_bits_to_f32(O.cpu_correction(f32_values(case.q), f32_values(case.k_full),
                                               f32_values(case.v_full), hm.numpy(), slots.numpy(), case.attn_scale))
    np.testing.assert_allclose(ref_out.float().numpy(), want, atol=2e-3, rtol=6e-3)
    mine = torch.empty_like(ref_out)
    ops.cpu_topk_attn(case.q, case.k_full, case.v_full, hm, slots, mine, case.attn_scale)
    np.testing.assert_allclose(mine.float().numpy(), ref_out.float().numpy(), atol=2e-3, rtol=6e-3)


def test_pool_submit_wait_and_single_flight():
    from jetfire_b200 import ops, _lib
    case, slots = _correction_inputs()
    out = torch.empty(2, 8, 128, dtype=torch.bfloat16)
    ops.set_cpu_attn_threads(2)
    ops.cpu_topk_attn_submit(case.q, case.k_full, case.v_full, None, slots, out, case.attn_scale)
    ops.cpu_topk_attn_wait(30000)
    again = torch.empty_like(out)
    ops.cpu_topk_attn(case.q, case.k_full, case.v_full, None, slots, again, case.attn_scale)
    assert torch.equal(out, again)
    assert _lib.lib.jf_pool_wait_timeout(0) == 0
    with pytest.raises(RuntimeError):
        ops.cpu_topk_attn(case.q.float(), case.k_full, case.v_full, None, slots, out, case.attn_scale)


def test_slot_lists_of_32_bit_integers_give_the_same_rows():
    """The host correction takes the selected slots as int64 (the reference's type) or as int32
    (half the device-to-host bytes): same bits out, through the blocking call, the pool and the
    prebuilt call; -1 padding and out-of-range slots are skipped in both widths."""
    from jetfire_b200 import ops
    case, slots = _correction_inputs()
    slots = slots.clone()
    slots[0, 0, -3:] = -1
    slots[1, 2, 0] = case.num_slots + 5
    slots32 = slots.to(torch.int32)
    ops.set_cpu_attn_threads(3)
    want = torch.empty(2, 8, 128, dtype=torch.bfloat16)
    ops.cpu_topk_attn(case.q, case.k_full, case.v_full, None, slots, want, case.attn_scale)
    got = torch.zeros_like(want)
    ops.cpu_topk_attn(case.q, case.k_full, case.v_full, None, slots32, got, case.attn_scale)
    assert torch.equal(got, want)
    got.zero_()
    ops.cpu_topk_attn_submit(case.q, case.k_full, case.v_full, None, slots32, got, case.attn_scale)
    ops.cpu_topk_attn_wait(30000)
    assert torch.equal(got, want)
    got.zero_()
    call = ops.HostCorrectionCall(case.q, case.k_full, case.v_full, None, slots32, got, case.attn_scale)
    ops.HostCorrectionCall.wait_ticket(call.submit())
    assert torch.equal(got, want)
    with pytest.raises(RuntimeError):
        ops.cpu_topk_attn(case.q, case.k_full, case.v_full, None, slots.to(torch.int16), got, case.attn_scale)


def test_prebuilt_host_call_equals_plain_call():
    from jetfire_b200 import ops
    case, slots = _correction_inputs()
    ops.set_cpu_attn_threads(3)
    want = torch.empty(2, 8, 128, dtype=torch.bfloat16)
    ops.cpu_topk_attn(case.q, case.k_full, case.v_full, None, slots, want, case.attn_scale)
    out = torch.zeros_like(want)
    call = ops.HostCorrectionCall(case.q, case.k_full, case.v_full, None, slots, out, case.attn_scale)
    call.submit(); call.wait()
    assert torch.equal(out, want)
    out.zero_()
    call.run()
    assert torch.equal(out, want)


def test_queued_jobs_complete_in_any_interleaving():
    """Several jobs queued ahead (workers flow from one job into the next); every ticket can be
    waited on, results equal the blocking call's, a fifth job is refused while four are queued
    or running, and changing the worker count between batches works."""
    from jetfire_b200 import ops, _lib
    case, _ = _correction_inputs()
    g = torch.Generator().manual_seed(11)
    for threads in (3, 5, 2):
        ops.set_cpu_attn_threads(threads)
        jobs = []
        for i in range(12):
            slots = torch.randint(0, case.num_slots, (2, 8, 64), generator=g, dtype=torch.int64)
            q = torch.randn(2, 8, 128, generator=g).to(torch.bfloat16)
            want = torch.empty(2, 8, 128, dtype=torch.bfloat16)
            ops.cpu_topk_attn(q, case.k_full, case.v_full, None, slots, want, case.attn_scale)
            out = torch.zeros_like(want)
            jobs.append((ops.HostCorrectionCall(q, case.k_full, case.v_full, None, slots, out, case.attn_scale), out, want))
        tickets = []
        for call, out, want in jobs:
            while True:
                try:
                    tickets.append(call.submit())
                    break
                except RuntimeError:           # queue full: wait for the oldest outstanding job
                    ops.HostCorrectionCall.wait_ticket(tickets[len(tickets) - 4])
        for t, (call, out, want) in zip(tickets, jobs):
            ops.HostCorrectionCall.wait_ticket(t)
            assert torch.equal(out, want)
        assert _lib.lib.jf_pool_wait_timeout(0) == 0


def test_host_correction_over_a_range_of_rows():
    """The host correction restricted to a range of the (sequence, query head) rows -- the rest being
    left to the GPU -- computes exactly those rows, bit for bit as in the full job, and touches no
    other part of ``o_new``; the ranges of a partition add up to the full result."""
    import torch
    from jetfire_b200 import _lib, ops
    g = torch.Generator().manual_seed(11)
    B, H_q, H_kv, K, slots = 3, 8, 2, 24, 96
    q = torch.randn(B, H_q, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(H_kv, slots, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(H_kv, slots, 128, generator=g).to(torch.bfloat16)
    ops.set_cpu_attn_threads(3)
    for dtype in (torch.int64, torch.int32):
        ts = torch.randint(-2, slots + 2, (B, H_q, K), generator=g, dtype=dtype)      # some invalid entries
        full = torch.empty_like(q)
        ops.cpu_topk_attn(q, k, v, None, ts, full, 0.09)
        part = torch.full_like(q, 7.0)
        ops.HostCorrectionCall(q, k, v, None, ts, part, 0.09, rows=(5, 17)).run()
        got, want = part.view(-1, 128), full.view(-1, 128)
        assert torch.equal(got[5:17], want[5:17])
        assert bool((got[:5] == 7).all()) and bool((got[17:] == 7).all())
        pieces = torch.full_like(q, 7.0)
        tickets = [ops.HostCorrectionCall(q, k, v, None, ts, pieces, 0.09, rows=r).submit() for r in ((0, 1), (1, 20), (20, 24))]
        for t in tickets:
            ops.HostCorrectionCall.wait_ticket(t)
        assert torch.equal(pieces, full)
    for bad in ((4, 4), (-1, 3), (3, 25), (9, 2)):
        with pytest.raises(RuntimeError):
            ops.HostCorrectionCall(q, k, v, None, ts, part, 0.09, rows=bad)
    t = _lib.C.c_int64(0)
    args = (q.data_ptr(), k.data_ptr(), v.data_ptr(), None, ts.data_ptr(), 1, part.data_ptr(), 0, B, H_q, H_kv, slots, K, 0.09, None)
    assert _lib.lib.jf_pool_submit_rows(*args, 4, 4, _lib.C.byref(t)) == _lib.JF_ERR_ARG
    assert _lib.lib.jf_pool_submit_rows(*args, 0, B * H_q + 1, _lib.C.byref(t)) == _lib.JF_ERR_ARG
    assert _lib.lib.jf_pool_submit_rows(*args, 0, 4, None) == _lib.JF_ERR_ARG
