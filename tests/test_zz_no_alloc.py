"""The workspace-free entry point, ``jf_decode_fused_static``, against ``jf_decode_fused``.

Some callers of this library cannot obtain device memory for scratch: they run inside a
host program that owns every allocation, or on a path where an allocator call (and the
synchronisation it can imply) is off limits, or with a memory budget that was fixed ahead
of time.  For them the library carries a fixed scratch array of its own.  This test calls
the entry point through the C ABI exactly as such a caller would -- inputs and outputs
only, no workspace -- twice in a row with different problems, and requires the same bits
as the ordinary entry point produces (both run the same deterministic kernels; the second
call also shows that what the first one left in the shared array does not matter).

Collected last on purpose: if it fails, a run that stops at the first failure has already
run everything else.  It does not depend on any other test having run.
"""
import ctypes as C

import pytest
import torch

from jf_testlib import Case

pytestmark = pytest.mark.gpu

STATIC_BYTES = 64 << 20  # JF_STATIC_SCRATCH_BYTES in include/jetfire_b200.h


def _run_both(case, top_k):
    from jetfire_b200 import _lib, ops
    kd, ks, vd, vs = case.device_cache()
    args = (case.mode, case.q.cuda(), kd, ks, vd, vs, case.block_table.cuda(), case.seq_lens.cuda(),
            case.ctx, case.H_q, case.H_kv, 16, top_k, case.attn_scale)
    ref = ops.DecodeCall(*args)
    ref.fused()
    # same argument block, fresh outputs, and no workspace at all
    mine = ops.DecodeCall(*args)
    mine.args.workspace = None
    mine.args.workspace_bytes = 0
    st = _lib.lib.jf_decode_fused_static(C.byref(mine.args), torch.cuda.current_stream().cuda_stream)
    assert st == 0, _lib.status_string(st)
    torch.cuda.synchronize()
    for name in ("topk_idx", "topk_slots", "o_hat", "o_old_unnorm", "W", "softmax_m", "softmax_inv_z"):
        assert torch.equal(mine.out[name], ref.out[name]), f"{name} differs from jf_decode_fused"
    assert (mine.out["topk_idx"][0, 0] >= 0).any()


def test_static_scratch_matches_workspace_entry_point_twice():
    _run_both(Case("k3v2", 2, 8, 2, 2048, seed=71), 128)
    # a second, differently shaped call right after: stale scratch contents must not leak in
    _run_both(Case("k3v2", 3, 16, 2, 1000, lens=[1000, 17, 0], seed=72), 64)
    _run_both(Case("k3v2", 2, 8, 2, 2048, seed=71), 128)


def test_rejects_requests_beyond_the_built_in_buffer():
    from jetfire_b200 import _lib
    a = _lib.DecodeArgs()
    a.mode, a.q_dtype = _lib.JF_MODE_K3V2, _lib.JF_DTYPE_BF16
    a.B, a.H_q, a.H_kv, a.max_S, a.block_size, a.top_k = 16, 32, 8, 131072, 16, 256
    need = _lib.lib.jf_decode_workspace_bytes(a.mode, a.B, a.H_q, a.H_kv, a.max_S, a.top_k)
    assert need > STATIC_BYTES
    st = _lib.lib.jf_decode_fused_static(C.byref(a), None)
    assert st == _lib.JF_ERR_STATIC_LIMIT
    assert "static" in _lib.status_string(st)
    a.mode = _lib.JF_MODE_K4V4
    assert _lib.lib.jf_decode_fused_static(C.byref(a), None) == _lib.JF_ERR_UNSUPPORTED
    assert _lib.lib.jf_decode_fused_static(None, None) == _lib.JF_ERR_ARG


def _packed_problem(B, H_q, H_kv, max_S, lens, num_slots, top_k, seed):
    """Argument block over a small random packed cache (bytes and scales drawn directly: only the
    two entry points are compared here, the arithmetic is pinned elsewhere) with a block table wide
    enough for ``max_S`` -- the scratch a call needs grows with max_S, not with the tokens present."""
    from jetfire_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(seed)
    dev = dict(device="cuda")
    kd = torch.randint(0, 256, (H_kv, num_slots, 48), dtype=torch.uint8, generator=g, **dev)
    vd = torch.randint(0, 256, (H_kv, num_slots, 32), dtype=torch.uint8, generator=g, **dev)
    ks = (torch.rand(H_kv, num_slots, 2, generator=g, **dev) + 0.5).to(torch.bfloat16)
    vs = (torch.rand(H_kv, num_slots, 2, generator=g, **dev) + 0.5).to(torch.bfloat16)
    q = torch.randn(B, H_q, 128, generator=g, **dev).to(torch.bfloat16)
    bt = torch.zeros(B, (max_S + 15) // 16, dtype=torch.int64, **dev)
    per = num_slots // 16 // B
    for b in range(B):
        bt[b, :per] = torch.arange(b * per, (b + 1) * per, dtype=torch.int64, **dev)
    sl = torch.tensor(lens, dtype=torch.int32, **dev)
    return ("k3v2", q, kd, ks, vd, vs, bt, sl, max_S, H_q, H_kv, 16, top_k, 128 ** -0.5)


def _largest_max_s_that_fits(B, H_q, H_kv, top_k):
    from jetfire_b200 import _lib
    need = lambda s: _lib.lib.jf_decode_workspace_bytes(_lib.JF_MODE_K3V2, B, H_q, H_kv, s, top_k)
    max_s = 262144
    while need(max_s) > STATIC_BYTES:
        max_s -= 16
    assert need(max_s) <= STATIC_BYTES < need(max_s + 16)
    return max_s


def test_limit_is_exact_and_the_call_allocates_nothing():
    """The largest request that fits the built-in array is served (same bits as the workspace
    entry point), the next larger one is refused, and a call changes nothing about the device's
    free memory -- which is the reason this entry point exists."""
    from jetfire_b200 import _lib, ops
    B, H_q, H_kv, top_k = 2, 32, 8, 64
    max_s = _largest_max_s_that_fits(B, H_q, H_kv, top_k)
    args = _packed_problem(B, H_q, H_kv, max_s, [4000, 1000], 8192, top_k, seed=5)
    ref = ops.DecodeCall(*args)
    ref.fused()
    mine = ops.DecodeCall(*args)
    mine.args.workspace, mine.args.workspace_bytes = None, 0
    stream = torch.cuda.current_stream().cuda_stream
    assert _lib.lib.jf_decode_fused_static(C.byref(mine.args), stream) == 0
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    assert _lib.lib.jf_decode_fused_static(C.byref(mine.args), stream) == 0      # nothing but this call in between
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "the static entry point changed the device's free memory"
    for name in ("topk_idx", "topk_slots", "o_hat", "o_old_unnorm", "W"):
        assert torch.equal(mine.out[name], ref.out[name]), name
    # a timed-out wait inside its kernels would be recorded in the built-in array: none here
    assert _lib.lib.jf_decode_status(C.byref(mine.args), stream) == 0
    too_big = _lib.DecodeArgs()
    C.memmove(C.byref(too_big), C.byref(mine.args), C.sizeof(_lib.DecodeArgs))
    too_big.max_S = max_s + 16
    too_big.max_blocks = (max_s + 16 + 15) // 16
    assert _lib.lib.jf_decode_fused_static(C.byref(too_big), stream) == _lib.JF_ERR_STATIC_LIMIT
