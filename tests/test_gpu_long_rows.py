"""Rows longer than one shared-memory chunk of the select kernel (32768 positions), odd row
strides, the select kernel that works from the scan's page maxima (rows longer than one staged
chunk; one block of 1024 threads per row, or two of 512 per multiprocessor once there are more
rows than multiprocessors), and the bench geometry at full size, checked against the C restatement of the
oracle (itself pinned to the numpy oracle in test_oracle_native.py).  The packed cache is the
one the GPU append path wrote (its bytes are pinned elsewhere), so no numpy pass over the
whole cache is needed."""
import numpy as np
import pytest
import torch

from oracle import native
from jf_testlib import Case, to_bits, f32_values

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2e-3, 1e-3


def _run(case, top_k, stage_b="fp32"):
    from jetfire_b200 import ops
    kd, ks, vd, vs = case.device_cache()
    res = ops.fused_attn_topk(case.mode, case.q.cuda(), kd, ks, vd, vs, case.block_table.cuda(),
                              case.seq_lens.cuda(), case.ctx, case.H_q, case.H_kv, 16, top_k, case.attn_scale,
                              want_scores=True, stage_b=stage_b)
    torch.cuda.synchronize()
    ref = native.c_decode(case.mode, f32_values(case.q), kd.cpu().numpy(), to_bits(ks), vd.cpu().numpy(), to_bits(vs),
                          case.block_table.numpy(), case.seq_lens.numpy(), case.ctx, top_k, case.attn_scale,
                          want_scores=True, stage_b=stage_b)
    assert np.array_equal(res.topk_idx.cpu().numpy(), ref["topk_idx"]), "top-k positions differ"
    assert np.array_equal(res.topk_slots.cpu().numpy(), ref["topk_slots"]), "top-k slots differ"
    sc = res.scores.cpu().numpy()
    for b in range(case.B):
        n = min(int(case.seq_lens[b]), case.ctx)
        if case.mode == "k4v4":
            assert np.array_equal(sc[b, :, :n], ref["scores"][b, :, :n]), "K4 scores are not bit-exact"
        else:
            # the reference's own gate for this tensor (scripts/validate_runtime.py:147-148 of JetFire)
            assert np.allclose(sc[b, :, :n], ref["scores"][b, :, :n], atol=2e-5, rtol=2e-5), \
                f"K3 scores: max err {np.abs(sc[b, :, :n] - ref['scores'][b, :, :n]).max():.3e}"
    for name in ("o_hat", "o_old_unnorm"):
        got, want = getattr(res, name).cpu().numpy(), ref[name]
        assert np.all(np.abs(got - want) <= ATOL + RTOL * np.abs(want)), name
    np.testing.assert_allclose(res.W.cpu().numpy(), ref["W"], atol=1e-4, rtol=1e-3)
    return res, ref


@pytest.mark.parametrize("mode,B,H_q,H_kv,ctx,lens,top_k,seed", [
    ("k4v4", 1, 8, 2, 40000, [39987], 256, 51),              # two chunks, ragged end
    ("k3v2", 2, 4, 2, 70000, [70000, 33001], 256, 52),       # three chunks and two chunks
    ("k3v2", 1, 4, 2, 40002, [40002], 128, 53),              # row stride not a multiple of 4: plain-copy path
    ("k4v4", 2, 8, 2, 33000, [33000, 32768], 512, 54),       # wide k: two staging rounds
])
def test_rows_longer_than_one_chunk(mode, B, H_q, H_kv, ctx, lens, top_k, seed):
    _run(Case(mode, B, H_q, H_kv, ctx, lens=lens, seed=seed), top_k)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H_q,H_kv,lens", [
    (4, 8, 2, [32768, 3000, 300, 8209]),          # 32 rows: the wide block
    (5, 32, 8, [32768, 32767, 2049, 511, 17]),    # 160 rows, more than multiprocessors: two narrow blocks on each
])
def test_page_maxima_select_with_ragged_lengths(dtype, B, H_q, H_kv, lens):
    """K3V2 rows long enough for the threshold to come from the scan's page-pair maxima, next to
    sequences of the same batch that are too short for it: fewer pairs than top-k (the exact radix
    tier over memory), fewer positions than the sort buffer (every position a candidate), a
    partial last page."""
    _run(Case("k3v2", B, H_q, H_kv, 32768, lens=lens, seed=62 + B, dtype=dtype), 256)


@pytest.mark.parametrize("mode,ctx,lens,top_k,stage_b", [
    ("k4v4", 4096, [4096, 4090, 300, 4096, 17], 256, "int8p"),       # one chunk of a 512-thread block
    ("k4v4", 40000, [40000, 39999, 16385, 20000, 5], 256, "fp32"),   # three chunks, streamed twice (no side table)
    ("k3v2", 8192, [8192, 8000, 600, 8192, 100], 256, "fp32"),       # too short for the page-maxima kernel
    ("k3v2", 20004, [20004, 16384, 16383, 9, 20000], 128, "fp32"),   # row stride not a multiple of 16: staged rows
])
def test_staged_row_select_with_two_blocks_per_multiprocessor(mode, ctx, lens, top_k, stage_b):
    """160 rows, more than multiprocessors: the kernel that stages the row in shared memory also
    comes as a 512-thread block (16384 positions per chunk), two to a multiprocessor."""
    _run(Case(mode, 5, 32, 8, ctx, lens=lens, seed=71), top_k, stage_b=stage_b)


@pytest.mark.parametrize("mode,ctx,lens", [
    ("k3v2", 131072, [131072, 70001]),    # 4096 page pairs = top-k: the histogram tier gives way to the radix tier
    ("k4v4", 262144, [262144, 9000]),     # 16384 pages = 4 * top-k: threshold from the page maxima; a row shorter than 2 * top-k
])
def test_top_k_4096(mode, ctx, lens):
    """The widest top-k: its sort buffer has no room beside a staged row, so every such call takes the
    kernel that works from the scan's page maxima (bitonic ranking, finish in sixteen rounds)."""
    _run(Case(mode, 2, 4, 1, ctx, lens=lens, seed=88), 4096)
    from jetfire_b200 import ops
    case = Case("k3v2", 1, 2, 1, 20002, lens=[20002], seed=89)   # row stride not a multiple of 16: not served
    kd, ks, vd, vs = case.device_cache()
    with pytest.raises(RuntimeError):
        ops.fused_attn_topk(case.mode, case.q.cuda(), kd, ks, vd, vs, case.block_table.cuda(), case.seq_lens.cuda(),
                            case.ctx, case.H_q, case.H_kv, 16, 4096, case.attn_scale)


def test_select_with_other_arguments_than_the_scan_is_reported():
    """The scan leaves page maxima only for calls whose select kernel works from them; a select
    called with arguments under which it would (here: a smaller top-k) after a scan that left none
    reports an error through the status record instead of selecting from stale maxima."""
    from jetfire_b200 import ops
    case = Case("k3v2", 1, 8, 2, 65536, lens=[65536], seed=77)
    kd, ks, vd, vs = case.device_cache()
    ws = torch.empty(ops.decode_workspace_bytes("k3v2", 1, 8, 2, 65536, 1024) + 256, dtype=torch.uint8, device="cuda")
    args = (case.mode, case.q.cuda(), kd, ks, vd, vs, case.block_table.cuda(), case.seq_lens.cuda(),
            case.ctx, case.H_q, case.H_kv, 16)
    wide = ops.DecodeCall(*args, 1024, case.attn_scale, workspace=ws)   # 2048 page pairs < 4 * 1024: rows are staged
    narrow = ops.DecodeCall(*args, 512, case.attn_scale, workspace=ws)  # 2048 page pairs >= 4 * 512: page maxima
    wide.scan(); narrow.select()
    with pytest.raises(RuntimeError):
        narrow.status()
    narrow.scan(); narrow.select(); narrow.status()                      # matching arguments: fine
    assert int(narrow.out["topk_idx"].min()) >= 0


def _random_cases(n, seed=2024):
    """Seeded random geometries: every select kernel (staged row / page maxima, 1024 / 512 threads),
    every GQA ratio, ragged lengths down to one token, top-k from 32 to 512, both dtypes."""
    rng = np.random.default_rng(seed)
    out = []
    for i in range(n):
        mode = "k3v2" if i % 2 == 0 else "k4v4"
        H_kv = int(rng.choice([1, 2, 4, 8]))
        G = int(rng.choice([1, 2, 4, 8, 16]))
        many_rows = i % 3 == 0
        B = int(rng.integers(1, 4)) if not many_rows else max(2, -(-149 // (H_kv * G)))
        top_k = int(rng.choice([32, 64, 128, 256, 512]))
        # a row stride that is a multiple of 16 and long enough for the page-maxima kernel in a third of the cases
        ctx = int(rng.choice([128 * top_k, 16 * int(rng.integers(40, 1500)), int(rng.integers(600, 24000))]))
        ctx = min(ctx, 36000 if B * H_kv * G <= 64 else 12000)
        lens = [int(rng.integers(1, ctx + 1)) for _ in range(B)]
        lens[int(rng.integers(0, B))] = ctx
        stage_b = "int8p" if (mode == "k4v4" and B > 1 and i % 4 == 1) else "fp32"
        dtype = torch.float16 if i % 5 == 0 else torch.bfloat16
        out.append(pytest.param(mode, B, H_kv * G, H_kv, ctx, lens, top_k, stage_b, dtype, 900 + i,
                                id=f"{i}-{mode}-B{B}-H{H_kv * G}x{H_kv}-ctx{ctx}-k{top_k}-{stage_b}"))
    return out


@pytest.mark.parametrize("mode,B,H_q,H_kv,ctx,lens,top_k,stage_b,dtype,seed", _random_cases(24))
def test_random_geometries(mode, B, H_q, H_kv, ctx, lens, top_k, stage_b, dtype, seed):
    _run(Case(mode, B, H_q, H_kv, ctx, lens=lens, seed=seed, dtype=dtype), top_k, stage_b=stage_b)


def _random_wide_cases(n, seed=515):
    """Seeded geometries with top-k 1024 / 2048 / 4096: rows around and below twice the top-k
    (every position a candidate), rows of a multiple of 16 positions that may or may not be long
    enough for the page maxima, ragged lengths, both modes and dtypes."""
    rng = np.random.default_rng(seed)
    out = []
    for i in range(n):
        mode = "k3v2" if i % 2 == 0 else "k4v4"
        top_k = int(rng.choice([1024, 2048, 4096]))
        H_kv = int(rng.choice([1, 2]))
        G = int(rng.choice([1, 4, 8, 16]))
        B = int(rng.integers(1, 3))
        if i % 3 == 0:
            ctx = 16 * int(rng.integers(top_k // 16 + 1, 4500))
        elif i % 3 == 1:
            ctx = int(rng.integers(100, 3 * top_k))
            if top_k > 2048:            # above 2048 the row stride has to be a multiple of 16
                ctx = (ctx + 15) // 16 * 16
        else:
            ctx = 16 * int(rng.integers(2000, 4400))
        lens = [int(rng.integers(1, ctx + 1)) for _ in range(B)]
        lens[int(rng.integers(0, B))] = ctx
        stage_b = "int8p" if (mode == "k4v4" and B > 1 and i % 4 == 1) else "fp32"
        dtype = torch.float16 if i % 5 == 0 else torch.bfloat16
        out.append(pytest.param(mode, B, H_kv * G, H_kv, ctx, lens, top_k, stage_b, dtype, 4000 + i,
                                id=f"{i}-{mode}-B{B}-H{H_kv * G}x{H_kv}-ctx{ctx}-k{top_k}-{stage_b}"))
    return out


@pytest.mark.parametrize("mode,B,H_q,H_kv,ctx,lens,top_k,stage_b,dtype,seed", _random_wide_cases(18))
def test_random_geometries_with_wide_top_k(mode, B, H_q, H_kv, ctx, lens, top_k, stage_b, dtype, seed):
    _run(Case(mode, B, H_q, H_kv, ctx, lens=lens, seed=seed, dtype=dtype), top_k, stage_b=stage_b)


@pytest.mark.parametrize("mode,top_k,ctx", [("k4v4", 1024, 8192), ("k3v2", 2048, 8192), ("k3v2", 1024, 2000)])
def test_wide_top_k(mode, top_k, ctx):
    """top-k above 512: the sort buffer no longer fits the counting / bucket ranking (bitonic
    path), the finish stage gathers its own rows; ctx 2000 < 2 * top_k takes the
    every-position-is-a-candidate path."""
    _run(Case(mode, 2, 8, 2, ctx, lens=[ctx, ctx - 37], seed=57 + top_k), top_k)


def test_bench_geometry_full_size_k4v4():
    """One layer of the headline bench workload at full size: K4V4, B 4, 32 query / 8 KV heads, ctx 32768, top-k 256."""
    res, _ = _run(Case("k4v4", 4, 32, 8, 32768, lens=[32768] * 4, seed=55), 256)
    idx = res.topk_idx.cpu().numpy()
    assert (idx >= 0).all() and (idx < 32768).all()
    assert all(np.unique(idx[b, h]).size == 256 for b in range(4) for h in range(32))


def test_config1_geometry_full_size_k3v2():
    """The single-sequence configuration at full size: K3V2, B 1, 32 query / 8 KV heads, ctx 32768, top-k 256."""
    _run(Case("k3v2", 1, 32, 8, 32768, lens=[32768], seed=56), 256)


def test_bench_geometry_full_size_k4v4_int8p():
    """The same layer with the reference's batch > 1 Stage B (weights rounded per 32-token tile):
    B 4 is a configured batch above 1, so this is the arithmetic the reference runs there."""
    _run(Case("k4v4", 4, 32, 8, 32768, lens=[32768, 32755, 20000, 32768], seed=58), 256, stage_b="int8p")


def test_llama70b_geometry_full_size_k3v2():
    """Llama-3.3-70B attention geometry at full size: 64 query / 8 KV heads (group 8), B 4, ctx 65536,
    top-k 512, K3V2 -- rows of two select chunks, the wide sort buffer, every MMA column in use."""
    res, _ = _run(Case("k3v2", 4, 64, 8, 65536, lens=[65536, 65536, 65523, 40000], seed=59), 512)
    idx = res.topk_idx.cpu().numpy()
    assert (idx >= 0).all() and all(np.unique(idx[b, h]).size == 512 for b in range(4) for h in (0, 31, 63))


def test_qwen3_moe_geometry_full_size_k3v2():
    """Qwen3-30B-A3B attention geometry at full size: 32 query / 4 KV heads (group 8), B 8, ctx 32768, top-k 256."""
    _run(Case("k3v2", 8, 32, 4, 32768, lens=[32768] * 6 + [32755, 9], seed=60), 256)


@pytest.mark.parametrize("mode,stage_b", [("k3v2", "fp32"), ("k4v4", "fp32"), ("k4v4", "int8p")])
def test_context_131072(mode, stage_b):
    """The longest context of the sweep, one sequence and one shorter one: four select chunks per row."""
    _run(Case(mode, 2, 8, 2, 131072, lens=[131072, 100003], seed=61), 256, stage_b=stage_b)


def _select_us(case, top_k, reps=5):
    """Device time of the select kernel alone (CUDA events on the launching stream, best of `reps`)."""
    from jetfire_b200 import ops
    kd, ks, vd, vs = case.device_cache()
    call = ops.DecodeCall(case.mode, case.q.cuda(), kd, ks, vd, vs, case.block_table.cuda(), case.seq_lens.cuda(),
                          case.ctx, case.H_q, case.H_kv, 16, top_k, case.attn_scale)
    call.scan(); call.select(); torch.cuda.synchronize()
    best = 1e9
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); call.select(); e1.record(); torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3)
    call.status()
    return best


@pytest.mark.parametrize("mode", ["k3v2", "k4v4"])
@pytest.mark.parametrize("shape", ["outlier", "flat"])
def test_rows_that_do_not_fit_the_fixed_bins_stay_exact_and_fast(mode, shape):
    """Rows on which the first selection tier gives up -- one score far above all others (the k-th
    largest then lies outside the histogram's range) or scores packed far closer than a bin -- take
    the exact radix tier.  The result is still the oracle's, and such a row may cost a few extra
    passes over shared memory, not a scan of the cache per pass: at most 10x an ordinary row."""
    normal = Case(mode, 1, 8, 2, 32768, lens=[32768], seed=70)
    odd = Case(mode, 1, 8, 2, 32768, lens=[32768], seed=70)
    if shape == "outlier":
        # the key at position 12345 of every KV head points along the query of the group's first head
        for hk in range(odd.H_kv):
            slot = int(odd.block_table[0, 12345 // 16]) * 16 + 12345 % 16
            odd.k_full[hk, slot] = (40.0 * odd.q[0, hk * 4].float()).to(odd.dtype)
    else:
        odd.q = (odd.q.float() * 2.0 ** -12).to(odd.dtype)     # every score within a few 1e-3 of zero
    res, ref = _run(odd, 256)
    if shape == "outlier":
        assert int(res.topk_idx[0, 0, 0]) == 12345
    t_norm, t_odd = _select_us(normal, 256), _select_us(odd, 256)
    print(f"{mode} {shape}: select {t_odd:.1f} us against {t_norm:.1f} us for an ordinary row")
    assert t_odd <= 10.0 * t_norm
