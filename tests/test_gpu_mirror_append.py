"""Appending to the host mirror: rows stored by the packing kernel into a mapped mirror, the
stream-ordered staged path for ordinary host memory, and the adapter's cache store + decode
entry on top of them, against the oracle.

Gates: mirror rows and packed bytes bit-exact; attention outputs within 2e-3 max-abs + 1e-3
relative (+ one bf16 ulp for the final store)."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from oracle import jf_oracle as O
from jf_testlib import Case, MODES, f32_values, to_bits

pytestmark = pytest.mark.gpu


def _tokens(T, H, dtype, seed, pad=0):
    """(T, H, 128) key / value tokens; pad > 0 makes the token stride wider than H * 128."""
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(T, H + pad, 128, generator=g).to(dtype).cuda()[:, :H]
    v = torch.randn(T, H + pad, 128, generator=g).to(dtype).cuda()[:, :H]
    return k, v


def _caches(mode, H, num_slots):
    kb, vb, gs = MODES[mode]
    ng = 128 // gs
    kd = torch.full((H, num_slots, 16 * kb), 0xA5, dtype=torch.uint8, device="cuda")
    vd = torch.full((H, num_slots, 16 * vb), 0xA5, dtype=torch.uint8, device="cuda")
    ks = torch.zeros(H, num_slots, ng, dtype=torch.bfloat16, device="cuda")
    vs = torch.zeros_like(ks)
    return kd, ks, vd, vs


def _expected_mirror(tok, slots, num_slots, fill):
    """Rows of live tokens at their slots, `fill` bits elsewhere (later tokens win a slot)."""
    T, H, _ = tok.shape
    want = np.full((H, num_slots, 128), fill, dtype=np.uint16)
    bits = to_bits(tok.contiguous())
    for t, s in enumerate(slots.tolist()):
        if 0 <= s < num_slots:
            want[:, s] = bits[t]
    return want


@pytest.mark.parametrize("mode,dtype,pad", [("k3v2", torch.bfloat16, 0), ("k4v4", torch.float16, 3),
                                             ("k4v4", torch.bfloat16, 1)])
def test_packing_kernel_stores_mirror_rows(mode, dtype, pad):
    from jetfire_b200 import ops
    kb, vb, gs = MODES[mode]
    T, H, num_slots = 37, 3, 64
    k_tok, v_tok = _tokens(T, H, dtype, 5, pad)
    slots = torch.randperm(num_slots, generator=torch.Generator().manual_seed(6))[:T].to(torch.int64)
    slots[4] = -1
    slots[11] = -7
    slots[20] = num_slots + 2        # out of range: skipped on both sides
    kd, ks, vd, vs = _caches(mode, H, num_slots)
    kd2, ks2, vd2, vs2 = _caches(mode, H, num_slots)
    km_host, km_dev = ops.alloc_mapped_pinned_pair((H, num_slots, 128), dtype)
    vm_host, vm_dev = ops.alloc_mapped_pinned_pair((H, num_slots, 128), dtype)
    km_host.view(torch.int16).fill_(0x1234)
    vm_host.view(torch.int16).fill_(0x1234)
    ops.fused_quant_write_kv_mirror(k_tok, v_tok, slots.cuda(), kd, ks, vd, vs, gs, kb, vb, km_dev, vm_dev)
    ops.fused_quant_write_kv(k_tok, v_tok, slots.cuda(), kd2, ks2, vd2, vs2, gs, kb, vb)
    torch.cuda.synchronize()
    for a, b in ((kd, kd2), (ks, ks2), (vd, vd2), (vs, vs2)):
        assert torch.equal(a, b), "the mirror store changed the packed cache"
    assert np.array_equal(to_bits(km_host), _expected_mirror(k_tok, slots, num_slots, 0x1234))
    assert np.array_equal(to_bits(vm_host), _expected_mirror(v_tok, slots, num_slots, 0x1234))
    with pytest.raises(RuntimeError):   # the mirror must have the tokens' dtype
        other = torch.float16 if dtype == torch.bfloat16 else torch.bfloat16
        ops.fused_quant_write_kv_mirror(k_tok, v_tok, slots.cuda(), kd, ks, vd, vs, gs, kb, vb,
                                        km_dev.view(other), vm_dev.view(other))


def test_stream_ordered_append_to_ordinary_host_memory():
    """Several chunks through the pinned staging (max_tokens 5, 23 tokens), padding slots
    skipped, a second append ordered behind the first on the same stream."""
    from jetfire_b200 import ops
    T, H, num_slots = 23, 2, 48
    k_tok, v_tok = _tokens(T, H, torch.bfloat16, 8, pad=2)
    slots = torch.randperm(num_slots, generator=torch.Generator().manual_seed(9))[:T].to(torch.int64)
    slots[0] = -1
    slots[22] = num_slots            # out of range
    k_shadow = torch.zeros(H, num_slots, 128, dtype=torch.bfloat16)
    v_shadow = torch.zeros(H, num_slots, 128, dtype=torch.bfloat16)
    ctx = ops.MirrorAppendCtx(k_shadow, v_shadow, max_tokens=5)
    ctx.append(k_tok, v_tok, slots.cuda())
    k2, v2 = _tokens(3, H, torch.bfloat16, 10)
    slots2 = slots[1:4].clone()      # overwrites three of the rows just written
    ctx.append(k2, v2, slots2.cuda())
    torch.cuda.synchronize()
    want_k = _expected_mirror(k_tok, slots, num_slots, 0)
    want_v = _expected_mirror(v_tok, slots, num_slots, 0)
    for t, s in enumerate(slots2.tolist()):
        want_k[:, s] = to_bits(k2)[t]
        want_v[:, s] = to_bits(v2)[t]
    assert np.array_equal(to_bits(k_shadow), want_k)
    assert np.array_equal(to_bits(v_shadow), want_v)
    st = ctx.stats()
    assert st["chunks"] == 5 + 1 and st["rows_written"] == (21 + 3) * H and st["rows_skipped"] == 2 * H
    with pytest.raises(RuntimeError):
        ctx.append(k_tok.half(), v_tok.half(), slots.cuda())
    ctx.close()
    with pytest.raises(RuntimeError):
        ctx.append(k_tok, v_tok, slots.cuda())


def test_map_host_tensor_makes_an_existing_mirror_device_visible():
    from jetfire_b200 import ops
    host = torch.zeros(2, 16, 128, dtype=torch.bfloat16)
    dev = ops.map_host_tensor(host)
    try:
        dev.copy_(torch.ones_like(dev))
        torch.cuda.synchronize()
        assert bool((host == 1).all())
    finally:
        del dev
        ops.unmap_host_tensor(host)


@pytest.mark.parametrize("mode_name,mode", [("SymInt3K_SymInt2V", "k3v2"), ("SymInt4K_SymInt4V", "k4v4")])
def test_cache_store_append_modes_and_decode_entry(mode_name, mode):
    """Prefill chunk + one decode token per sequence through the store, with each way of
    filling the mirror; the three mirrors are equal bit for bit, the packed cache is the
    oracle's, and the decode entry (scan, selection, host correction over the mirror, merge)
    gives the oracle's output."""
    from jetfire_b200.adapter.cache_store import JetFireCacheStore
    from jetfire_b200.adapter.config import JetFireConfig
    from jetfire_b200.adapter.decode_path import make_decode_metadata, try_jetfire_decode
    case = Case(mode, 2, 8, 2, 400, lens=[400, 263], seed=21)
    cfg = JetFireConfig(mode=mode_name, top_k=64, group_size=MODES[mode][2], cpu_attn_threads=2)
    key_all = case.k_full.transpose(0, 1).contiguous().cuda()     # (num_slots, H_kv, 128): token t -> slot t
    val_all = case.v_full.transpose(0, 1).contiguous().cuda()
    # the last token of every sequence arrives as the decode-step append
    last_slots = []
    for b in range(case.B):
        n = int(case.seq_lens[b])
        last_slots.append(int(case.block_table[b, (n - 1) // 16]) * 16 + (n - 1) % 16)
    last = torch.tensor(last_slots, dtype=torch.int64)
    first = torch.tensor([s for s in range(case.num_slots) if s not in set(last_slots)], dtype=torch.int64)
    first_padded = torch.cat([first, torch.tensor([-1, -1], dtype=torch.int64)])   # padding as vLLM sends it
    stores = {}
    for how in ("mapped", "stream", "sync"):
        st = JetFireCacheStore(num_blocks=case.n_blocks, num_kv_heads=case.H_kv, head_dim=128, cfg=cfg,
                               device="cuda", dtype=case.dtype, mirror_append=how, stream_chunk_tokens=100)
        pad_rows = torch.zeros(2, case.H_kv, 128, dtype=case.dtype, device="cuda")
        st.write_slots(torch.cat([key_all[first.cuda()], pad_rows]), torch.cat([val_all[first.cuda()], pad_rows]),
                       first_padded.cuda())
        st.write_slots(key_all[last.cuda()], val_all[last.cuda()], last.cuda())
        st.flush_pending_writes()
        stores[how] = st
    okd, oks, ovd, ovs = case.oracle_cache()
    for how, st in stores.items():
        assert np.array_equal(to_bits(st.k_shadow), to_bits(case.k_full)), f"{how}: K mirror differs"
        assert np.array_equal(to_bits(st.v_shadow), to_bits(case.v_full)), f"{how}: V mirror differs"
        assert np.array_equal(st.k_data.cpu().numpy(), okd) and np.array_equal(to_bits(st.k_scales), oks)
        assert np.array_equal(st.v_data.cpu().numpy(), ovd) and np.array_equal(to_bits(st.v_scales), ovs)
        assert bool(st.slot_filled.all())
    ref = case.oracle_step(64)
    want = O.bf16_bits_to_f32(O.f32_to_bf16_bits(ref["out"]))
    md = make_decode_metadata(case.seq_lens.cuda(), case.block_table.cuda())
    impl = SimpleNamespace(scale=case.attn_scale, attn_type=SimpleNamespace(name="DECODER"))
    layer = SimpleNamespace(num_heads=case.H_q, num_kv_heads=case.H_kv, head_size=128, layer_name="l0")
    for how, st in stores.items():
        out = torch.zeros(case.B, case.H_q * 128, dtype=case.dtype, device="cuda")
        got = try_jetfire_decode(impl=impl, layer=layer, query=case.q.cuda(), attn_metadata=md,
                                 output=out, store=st, cfg=cfg)
        assert got is out
        torch.cuda.synchronize()
        err = np.abs(f32_values(out).reshape(case.B, case.H_q, 128) - want)
        lim = 2e-3 + (1e-3 + 2 ** -8) * np.abs(want)
        assert (err <= lim).all(), f"{how}: max err {err.max():.3e}"


def test_store_append_is_capturable_and_skips_out_of_range_slots():
    """``write_slots`` with a mapped mirror is launches only: it can be captured in a CUDA graph and
    replayed, and slots that are negative or beyond the cache (which the packing kernel skips)
    neither mark anything filled nor disturb the device."""
    from jetfire_b200.adapter.cache_store import JetFireCacheStore
    from jetfire_b200.adapter.config import JetFireConfig
    cfg = JetFireConfig(mode="SymInt3K_SymInt2V", top_k=32, group_size=64, cpu_attn_threads=2)
    st = JetFireCacheStore(num_blocks=4, num_kv_heads=2, head_dim=128, cfg=cfg, device="cuda",
                           dtype=torch.bfloat16, mirror_append="mapped")
    g = torch.Generator().manual_seed(3)
    key = torch.randn(6, 2, 128, generator=g).to(torch.bfloat16).cuda()
    val = torch.randn(6, 2, 128, generator=g).to(torch.bfloat16).cuda()
    slots = torch.tensor([5, -1, 63, 64, 1 << 40, 0], dtype=torch.int64, device="cuda")   # 64 and 2^40 are out of range
    st.write_slots(key, val, slots)          # eager once (sets kernel attributes), then captured
    st.flush_pending_writes()
    st._filled_buf.zero_()
    st.k_shadow.zero_()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            st.write_slots(key, val, slots)
    graph.replay()
    torch.cuda.synchronize()
    filled = st.slot_filled.cpu().numpy()
    assert sorted(np.flatnonzero(filled).tolist()) == [0, 5, 63]
    for t, s_ in ((0, 5), (2, 63), (5, 0)):
        assert torch.equal(st.k_shadow[:, s_], key[t].cpu())
    untouched = [s_ for s_ in range(64) if s_ not in (0, 5, 63)]
    assert not st.k_shadow[:, untouched].any()


def test_backend_routes_append_and_decode_through_installed_stores(monkeypatch):
    """The attention-backend shim as vLLM drives it: ``install_layer_stores`` with the planned cache
    geometry, ``do_kv_cache_update`` per layer with vLLM's padded slot mapping, ``forward`` for a
    decode batch (served here, result = the oracle's) and for a prefill batch (handed to the native
    implementation untouched)."""
    from jetfire_b200.adapter.config import JetFireConfig
    from jetfire_b200.adapter.decode_path import make_decode_metadata
    from jetfire_b200.adapter.jetfire_backend import JetFireAttentionImplMixin, get_layer_store
    from jetfire_b200.adapter.registry import install_layer_stores
    case = Case("k3v2", 2, 8, 2, 300, lens=[300, 123], seed=27)
    cfg = JetFireConfig(mode="SymInt3K_SymInt2V", top_k=64, group_size=64, cpu_attn_threads=2)

    class Native:
        calls = []

        def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None, output_scale=None,
                    output_block_scale=None):
            Native.calls.append("forward")
            return "native"

        def do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping):
            Native.calls.append("update")

    class Impl(JetFireAttentionImplMixin, Native):
        scale = case.attn_scale
        attn_type = SimpleNamespace(name="DECODER")

    import jetfire_b200.adapter.jetfire_backend as jb
    monkeypatch.setattr(jb, "get_jetfire_config", lambda: cfg)   # the configuration this test runs under
    layer = SimpleNamespace(num_heads=case.H_q, num_kv_heads=case.H_kv, head_size=128, layer_name="model.layers.0.attn")
    odd = SimpleNamespace(num_heads=8, num_kv_heads=2, head_size=64, layer_name="model.layers.1.attn")
    stores = install_layer_stores({layer.layer_name: layer, odd.layer_name: odd}, num_blocks=case.n_blocks, cfg=cfg,
                                  dtype=case.dtype)
    assert list(stores) == [layer.layer_name] and get_layer_store(odd.layer_name) is None
    impl = Impl()
    key = case.k_full.transpose(0, 1).contiguous().cuda().reshape(case.num_slots, case.H_kv * 128)
    val = case.v_full.transpose(0, 1).contiguous().cuda().reshape(case.num_slots, case.H_kv * 128)
    slot_mapping = torch.arange(case.num_slots, dtype=torch.int64, device="cuda")
    impl.do_kv_cache_update(layer, key, val, None, slot_mapping)
    assert Native.calls == ["update"]                        # vLLM's own cache still gets its update
    md = make_decode_metadata(case.seq_lens.cuda(), case.block_table.cuda())
    out = torch.zeros(case.B, case.H_q * 128, dtype=case.dtype, device="cuda")
    got = impl.forward(layer, case.q.cuda(), None, None, None, md, output=out)
    assert got is out and Native.calls == ["update"]
    torch.cuda.synchronize()
    ref = case.oracle_step(64)
    want = O.bf16_bits_to_f32(O.f32_to_bf16_bits(ref["out"]))
    err = np.abs(f32_values(out).reshape(case.B, case.H_q, 128) - want)
    assert (err <= 2e-3 + (1e-3 + 2 ** -8) * np.abs(want)).all(), f"max err {err.max():.3e}"
    prefill = SimpleNamespace(**{**vars(md), "max_query_len": 7})
    assert impl.forward(layer, case.q.cuda(), None, None, None, prefill, output=out) == "native"


@pytest.mark.parametrize("order", ["decode_first_with_counts", "decode_first", "interleaved"])
def test_step_with_decode_and_prefill_sequences(order):
    """A step in which two sequences decode and two are prefilled: the decode rows come from the
    packed cache (bit for bit what a pure decode step of those two sequences gives), the prefill
    rows from a causal attention over the step's own keys and values, each written to its own
    rows of the output -- with the scheduler's counts on the metadata (slices, nothing read back),
    without them, and with the sequences interleaved."""
    from jetfire_b200.adapter.cache_store import JetFireCacheStore
    from jetfire_b200.adapter.config import JetFireConfig
    from jetfire_b200.adapter.decode_path import make_decode_metadata, try_jetfire_decode
    from jetfire_b200.adapter.mixed_batch import MixedBatchStats, annotate_split_counts, try_jetfire_mixed
    from jf_testlib import causal_prefill_attention
    case = Case("k3v2", 2, 8, 2, 300, lens=[300, 123], seed=41)
    cfg = JetFireConfig(mode="SymInt3K_SymInt2V", top_k=64, group_size=64, cpu_attn_threads=2)
    st = JetFireCacheStore(num_blocks=case.n_blocks, num_kv_heads=case.H_kv, head_dim=128, cfg=cfg, device="cuda",
                           dtype=case.dtype, mirror_append="mapped")
    key_all = case.k_full.transpose(0, 1).contiguous().cuda()
    val_all = case.v_full.transpose(0, 1).contiguous().cuda()
    st.write_slots(key_all, val_all, torch.arange(case.num_slots, dtype=torch.int64, device="cuda"))
    st.flush_pending_writes()
    impl = SimpleNamespace(scale=case.attn_scale, attn_type=SimpleNamespace(name="DECODER"))
    layer = SimpleNamespace(num_heads=case.H_q, num_kv_heads=case.H_kv, head_size=128, layer_name="l0")
    # the pure decode step of the two cached sequences
    want_dec = torch.zeros(2, case.H_q * 128, dtype=case.dtype, device="cuda")
    md_dec = make_decode_metadata(case.seq_lens.cuda(), case.block_table.cuda())
    assert try_jetfire_decode(impl=impl, layer=layer, query=case.q.cuda(), attn_metadata=md_dec, output=want_dec,
                              store=st, cfg=cfg) is want_dec
    # the mixed step: sequences 0 and 1 decode, two new prompts of 5 and 19 tokens are prefilled
    g = torch.Generator().manual_seed(5)
    pre_len = [5, 19]
    if order == "interleaved":
        seqs = [("p", 0), ("d", 0), ("p", 1), ("d", 1)]
    else:
        seqs = [("d", 0), ("d", 1), ("p", 0), ("p", 1)]
    qlens = [1 if kind == "d" else pre_len[i] for kind, i in seqs]
    T = sum(qlens)
    q = torch.randn(T, case.H_q, 128, generator=g).to(case.dtype).cuda()
    k = torch.randn(T, case.H_kv, 128, generator=g).to(case.dtype).cuda()
    v = torch.randn(T, case.H_kv, 128, generator=g).to(case.dtype).cuda()
    starts = [0]
    for n in qlens:
        starts.append(starts[-1] + n)
    n_blk = case.block_table.shape[1]
    bt = torch.zeros(4, n_blk, dtype=case.block_table.dtype)
    lens = []
    for s_i, (kind, i) in enumerate(seqs):
        if kind == "d":
            q[starts[s_i]] = case.q[i].cuda()
            bt[s_i] = case.block_table[i]
            lens.append(int(case.seq_lens[i]))
        else:
            lens.append(pre_len[i])
    md = SimpleNamespace(query_start_loc=torch.tensor(starts, dtype=torch.int32, device="cuda"),
                         seq_lens=torch.tensor(lens, dtype=torch.int32, device="cuda"), block_table=bt.cuda(),
                         max_query_len=max(qlens), max_seq_len=max(lens), num_actual_tokens=T, use_cascade=False,
                         causal=True)
    if order == "decode_first_with_counts":
        annotate_split_counts(md, starts, lens)
        assert (md.num_decodes, md.num_prefills, md.num_prefill_tokens) == (2, 2, 24)
    out = torch.full((T, case.H_q * 128), 9.0, dtype=case.dtype, device="cuda")
    stats = MixedBatchStats()
    got = try_jetfire_mixed(impl=impl, layer=layer, query=q.view(T, -1), key=k.view(T, -1), value=v.view(T, -1),
                            attn_metadata=md, output=out, store=st, cfg=cfg,
                            prefill_attention=causal_prefill_attention, stats=stats)
    assert got is out and stats.mixed_batch_count == 1 and not stats.handed_back
    torch.cuda.synchronize()
    dec_i = 0
    for s_i, (kind, i) in enumerate(seqs):
        lo, hi = starts[s_i], starts[s_i + 1]
        if kind == "d":
            assert torch.equal(out[lo], want_dec[i]), f"decode row of sequence {i} differs"
            dec_i += 1
        else:
            want = torch.empty(hi - lo, case.H_q, 128, dtype=case.dtype, device="cuda")
            causal_prefill_attention(q=q[lo:hi], k=k[lo:hi], v=v[lo:hi], out=want,
                                     cu_seqlens=[0, hi - lo], max_seqlen=hi - lo, impl=impl, layer=None,
                                     attn_metadata=None)
            assert torch.equal(out[lo:hi].view(hi - lo, case.H_q, 128), want), f"prefill rows of prompt {i} differ"
    assert dec_i == 2


def test_default_prefill_attention_of_a_mixed_step_on_the_device():
    """The variable-length flash attention the mixed step uses by default, against plain causal
    attention in fp32 (bf16 inputs: agreement to bf16 rounding of values of order 1)."""
    from jetfire_b200.adapter import mixed_batch as mb
    from jf_testlib import causal_prefill_attention
    try:
        mb._resolve_flash_varlen()
    except ImportError as exc:
        pytest.skip(str(exc))
    g = torch.Generator().manual_seed(9)
    lens = [7, 33, 16]
    T, H_q, H_kv = sum(lens), 8, 2
    q = torch.randn(T, H_q, 128, generator=g).to(torch.bfloat16).cuda()
    k = torch.randn(T, H_kv, 128, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(T, H_kv, 128, generator=g).to(torch.bfloat16).cuda()
    cu = torch.tensor([0, 7, 40, 56], dtype=torch.int32, device="cuda")
    impl = SimpleNamespace(scale=128 ** -0.5, sliding_window=None, logits_soft_cap=None, alibi_slopes=None)
    got = torch.zeros(T, H_q, 128, dtype=torch.bfloat16, device="cuda")
    want = torch.zeros(T, H_q, 128, dtype=torch.float32, device="cuda")
    try:
        mb.flash_varlen_prefill(q=q, k=k, v=v, out=got, cu_seqlens=cu, max_seqlen=33, impl=impl, layer=None,
                                attn_metadata=SimpleNamespace(causal=True))
    except (RuntimeError, NotImplementedError, AssertionError) as exc:
        pytest.skip(f"the installed flash attention does not run on this device: {exc}")
    causal_prefill_attention(q=q, k=k, v=v, out=want, cu_seqlens=cu.tolist(), max_seqlen=33, impl=impl, layer=None,
                             attn_metadata=None)
    torch.cuda.synchronize()
    err = (got.float() - want).abs()
    assert float(err.max()) <= 2e-2, f"max err {float(err.max()):.3e}"


@pytest.mark.parametrize("signal", ["flags", "callbacks"])
@pytest.mark.parametrize("mode_name,mode", [("SymInt3K_SymInt2V", "k3v2"), ("SymInt4K_SymInt4V", "k4v4")])
def test_stream_ordered_decode_entry_eager_and_captured(mode_name, mode, signal):
    """The decode entry in its stream-ordered form (nothing waits on the host: copies, kernels and
    the correction's submit / join are queued on the stream over fixed buffers) gives, bit for bit,
    what the default form gives -- run eagerly over three steps of growing sequences, and with the
    append and the decode of a step captured in one CUDA graph that is replayed for the same steps.
    ``signal``: the stream and the host meet through words in mapped memory (a kernel raises the
    trigger a dispatcher thread polls; a kernel polls the completion word) or through host
    functions in the stream."""
    from dataclasses import replace
    from jetfire_b200.adapter.config import JetFireConfig
    from jetfire_b200.adapter import decode_path as dp
    steps, len0 = 3, [300, 123]
    case = Case(mode, 2, 8, 2, 320, lens=[n + steps for n in len0], seed=43)
    cfg = JetFireConfig(mode=mode_name, top_k=64, group_size=MODES[mode][2], cpu_attn_threads=2, stream_ordered=False)
    cfg_so = replace(cfg, stream_ordered=True, stream_signal=signal)
    slot_of = lambda b, pos: int(case.block_table[b, pos // 16]) * 16 + pos % 16
    key_all = case.k_full.transpose(0, 1).contiguous().cuda()
    val_all = case.v_full.transpose(0, 1).contiguous().cuda()
    init = torch.tensor([slot_of(b, p) for b in range(case.B) for p in range(len0[b])], dtype=torch.int64).cuda()
    impl = SimpleNamespace(scale=case.attn_scale, attn_type=SimpleNamespace(name="DECODER"))
    layer = SimpleNamespace(num_heads=case.H_q, num_kv_heads=case.H_kv, head_size=128, layer_name="l0")
    g = torch.Generator().manual_seed(6)
    queries = [torch.randn(case.B, case.H_q, 128, generator=g).to(case.dtype).cuda() for _ in range(steps)]
    bt = case.block_table.cuda()

    # the same bound on the row length in all three runs (the split of a row into partial sums,
    # and with it the last bits of the result, follows the bound, not the lengths)
    bounded = lambda md: SimpleNamespace(**{**vars(md), "max_seq_len": case.ctx})

    def tokens_of(t):
        slots_t = torch.tensor([slot_of(b, len0[b] + t) for b in range(case.B)], dtype=torch.int64).cuda()
        return key_all[slots_t], val_all[slots_t], slots_t

    def fresh_store():
        from jetfire_b200.adapter.cache_store import JetFireCacheStore
        st = JetFireCacheStore(num_blocks=case.n_blocks, num_kv_heads=case.H_kv, head_dim=128, cfg=cfg, device="cuda",
                               dtype=case.dtype, mirror_append="mapped")
        st.write_slots(key_all[init], val_all[init], init)
        st.flush_pending_writes()
        return st

    # the default form, step by step
    want = []
    st = fresh_store()
    for t in range(steps):
        k_t, v_t, s_t = tokens_of(t)
        st.write_slots(k_t, v_t, s_t)
        lens = torch.tensor([n + t + 1 for n in len0], dtype=torch.int32, device="cuda")
        md = bounded(dp.make_decode_metadata(lens, bt))
        out = torch.zeros(case.B, case.H_q * 128, dtype=case.dtype, device="cuda")
        assert dp.try_jetfire_decode(impl=impl, layer=layer, query=queries[t], attn_metadata=md, output=out,
                                     store=st, cfg=cfg) is out
        torch.cuda.synchronize()
        want.append(out.clone())

    # stream-ordered, eager
    st = fresh_store()
    for t in range(steps):
        k_t, v_t, s_t = tokens_of(t)
        st.write_slots(k_t, v_t, s_t)
        lens = torch.tensor([n + t + 1 for n in len0], dtype=torch.int32, device="cuda")
        md = bounded(dp.make_decode_metadata(lens, bt))
        out = torch.full((case.B, case.H_q * 128), 5.0, dtype=case.dtype, device="cuda")
        assert dp.try_jetfire_decode(impl=impl, layer=layer, query=queries[t], attn_metadata=md, output=out,
                                     store=st, cfg=cfg_so) is out
        torch.cuda.synchronize()
        assert torch.equal(out, want[t]), f"eager, step {t}"
    for step in dp.stream_steps(st):
        step.status()

    # stream-ordered, append + decode of a step captured once and replayed
    st = fresh_store()
    new_k = torch.zeros(case.B, case.H_kv, 128, dtype=case.dtype, device="cuda")
    new_v = torch.zeros_like(new_k)
    new_slots = torch.full((case.B,), -1, dtype=torch.int64, device="cuda")
    lens = torch.tensor(len0, dtype=torch.int32, device="cuda")
    query = torch.zeros(case.B, case.H_q, 128, dtype=case.dtype, device="cuda")
    out = torch.zeros(case.B, case.H_q * 128, dtype=case.dtype, device="cuda")
    md = bounded(dp.make_decode_metadata(lens, bt))

    def one_step():
        st.write_slots(new_k, new_v, new_slots)
        assert dp.try_jetfire_decode(impl=impl, layer=layer, query=query, attn_metadata=md, output=out,
                                     store=st, cfg=cfg_so) is out

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):       # eager once (kernel attributes, worker threads); appends nothing
        one_step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        one_step()
    for t in range(steps):
        k_t, v_t, s_t = tokens_of(t)
        new_k.copy_(k_t); new_v.copy_(v_t); new_slots.copy_(s_t)
        lens.copy_(torch.tensor([n + t + 1 for n in len0], dtype=torch.int32))
        query.copy_(queries[t])
        graph.replay()
        torch.cuda.synchronize()
        for step in dp.stream_steps(st):
            step.status()
        assert torch.equal(out, want[t]), f"replayed, step {t}"
    del graph


def test_stream_ordered_step_with_rows_of_the_correction_on_the_gpu():
    """With a share of the correction's rows given to the GPU (read from the mapped mirror over the
    host link while the workers do the others) the decode entry still gives the oracle's output."""
    from jetfire_b200.adapter.cache_store import JetFireCacheStore
    from jetfire_b200.adapter.config import JetFireConfig
    from jetfire_b200.adapter import decode_path as dp
    case = Case("k3v2", 2, 8, 2, 400, lens=[400, 263], seed=49)
    cfg = JetFireConfig(mode="SymInt3K_SymInt2V", top_k=64, group_size=64, cpu_attn_threads=2, gpu_correction_share=0.3)
    st = JetFireCacheStore(num_blocks=case.n_blocks, num_kv_heads=case.H_kv, head_dim=128, cfg=cfg, device="cuda",
                           dtype=case.dtype, mirror_append="mapped")
    st.write_slots(case.k_full.transpose(0, 1).contiguous().cuda(), case.v_full.transpose(0, 1).contiguous().cuda(),
                   torch.arange(case.num_slots, dtype=torch.int64, device="cuda"))
    impl = SimpleNamespace(scale=case.attn_scale, attn_type=SimpleNamespace(name="DECODER"))
    layer = SimpleNamespace(num_heads=case.H_q, num_kv_heads=case.H_kv, head_size=128, layer_name="l0")
    md = dp.make_decode_metadata(case.seq_lens.cuda(), case.block_table.cuda())
    want = O.bf16_bits_to_f32(O.f32_to_bf16_bits(case.oracle_step(64)["out"]))
    for _ in range(2):                      # the second run reuses the step's buffers
        out = torch.zeros(case.B, case.H_q * 128, dtype=case.dtype, device="cuda")
        assert dp.try_jetfire_decode(impl=impl, layer=layer, query=case.q.cuda(), attn_metadata=md, output=out,
                                     store=st, cfg=cfg) is out
        torch.cuda.synchronize()
        step = dp.stream_steps(st)[0]
        step.status()
        assert (step.rows, step.cut) == (16, 11)            # 5 of the 16 rows on the GPU
        err = np.abs(f32_values(out).reshape(case.B, case.H_q, 128) - want)
        assert (err <= 2e-3 + (1e-3 + 2 ** -8) * np.abs(want)).all(), f"max err {err.max():.3e}"


def test_stream_ordered_step_is_replaced_when_the_sequences_outgrow_it():
    """The stream-ordered step holds buffers for rows up to a multiple of 4096 positions; when a
    sequence grows past that the step is replaced (the old one released once the stream has
    drained) and the results stay the oracle's on both sides of the boundary."""
    from jetfire_b200.adapter.cache_store import JetFireCacheStore
    from jetfire_b200.adapter.config import JetFireConfig
    from jetfire_b200.adapter import decode_path as dp
    case = Case("k3v2", 2, 8, 2, 4112, lens=[4112, 700], seed=47)
    cfg = JetFireConfig(mode="SymInt3K_SymInt2V", top_k=64, group_size=64, cpu_attn_threads=2)
    st = JetFireCacheStore(num_blocks=case.n_blocks, num_kv_heads=case.H_kv, head_dim=128, cfg=cfg, device="cuda",
                           dtype=case.dtype, mirror_append="mapped")
    st.write_slots(case.k_full.transpose(0, 1).contiguous().cuda(), case.v_full.transpose(0, 1).contiguous().cuda(),
                   torch.arange(case.num_slots, dtype=torch.int64, device="cuda"))
    impl = SimpleNamespace(scale=case.attn_scale, attn_type=SimpleNamespace(name="DECODER"))
    layer = SimpleNamespace(num_heads=case.H_q, num_kv_heads=case.H_kv, head_size=128, layer_name="l0")
    seen = []
    for lens in ([4090, 700], [4096, 700], [4100, 640]):
        case.seq_lens = torch.tensor(lens, dtype=torch.int32)
        md = dp.make_decode_metadata(case.seq_lens.cuda(), case.block_table.cuda())
        out = torch.zeros(case.B, case.H_q * 128, dtype=case.dtype, device="cuda")
        assert dp.try_jetfire_decode(impl=impl, layer=layer, query=case.q.cuda(), attn_metadata=md, output=out,
                                     store=st, cfg=cfg) is out
        torch.cuda.synchronize()
        steps = dp.stream_steps(st)
        assert len(steps) == 1
        steps[0].status()
        seen.append(steps[0].max_S)
        want = O.bf16_bits_to_f32(O.f32_to_bf16_bits(case.oracle_step(64)["out"]))
        err = np.abs(f32_values(out).reshape(case.B, case.H_q, 128) - want)
        assert (err <= 2e-3 + (1e-3 + 2 ** -8) * np.abs(want)).all(), f"lens {lens}: max err {err.max():.3e}"
    assert seen == [4096, 4096, 4112]        # the third step needs 4112 positions: all the block table has


def test_wait_for_a_word_nothing_sets_runs_out_and_is_reported():
    """The kernel that holds the stream for the host correction has a time budget: with a word that
    nothing sets it gives up after the budget, writes the timeout into the status record it was
    given and lets the stream go on; a word that is set lets it through at once."""
    import time
    from jetfire_b200 import ops
    words_host, words_dev = ops.alloc_mapped_pinned_pair((16,), torch.int64)
    words_host.zero_()
    record = torch.zeros(ops.STATUS_RECORD_BYTES, dtype=torch.uint8, device="cuda")
    after = torch.zeros(1, device="cuda")
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ops.stream_wait_host_flag(words_dev[8:9], 20, record)
    after.fill_(1.0)                                     # queued behind the wait
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert 0.015 < dt < 2.0, f"waited {dt * 1e3:.1f} ms for a budget of 20 ms"
    assert float(after) == 1.0
    with pytest.raises(RuntimeError):
        ops.decode_status_of_copy(record.cpu())
    record.zero_()
    words_host[8] = 1
    t0 = time.perf_counter()
    ops.stream_wait_host_flag(words_dev[8:9], 2000, record)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 0.5
    ops.decode_status_of_copy(record.cpu())              # nothing recorded
    ops.stream_signal_host(words_dev[8:9], words_dev[0:1])
    torch.cuda.synchronize()
    assert int(words_host[8]) == 0 and int(words_host[0]) == 1


def test_decode_steps_replayed_as_one_cuda_graph_with_host_nodes():
    """A whole decode step of one layer captured once and replayed: append of the new token
    (packed cache + mapped mirror, one kernel), query upload, scan + selection, slot download,
    host correction submitted and joined by host nodes in the graph, o_new upload, merge.  No
    host synchronisation inside a step; every replay's output is the oracle's for the sequence
    lengths of that step."""
    from jetfire_b200 import ops
    mode, top_k, steps = "k3v2", 64, 3
    kb, vb, gs = MODES[mode]
    len0 = [300, 200]
    case = Case(mode, 2, 8, 2, 512, lens=[n + steps for n in len0], seed=33)
    slot_of = lambda b, pos: int(case.block_table[b, pos // 16]) * 16 + pos % 16
    kd, ks, vd, vs = _caches(mode, case.H_kv, case.num_slots)
    km_host, km_dev = ops.alloc_mapped_pinned_pair((case.H_kv, case.num_slots, 128), case.dtype)
    vm_host, vm_dev = ops.alloc_mapped_pinned_pair((case.H_kv, case.num_slots, 128), case.dtype)
    km_host.zero_()
    vm_host.zero_()
    key_all = case.k_full.transpose(0, 1).contiguous().cuda()     # token rows by slot
    val_all = case.v_full.transpose(0, 1).contiguous().cuda()
    init = torch.tensor([slot_of(b, p) for b in range(case.B) for p in range(len0[b])], dtype=torch.int64).cuda()
    ops.fused_quant_write_kv_mirror(key_all[init], val_all[init], init, kd, ks, vd, vs, gs, kb, vb, km_dev, vm_dev)
    # static buffers of the captured step
    new_k = torch.zeros(case.B, case.H_kv, 128, dtype=case.dtype, device="cuda")
    new_v = torch.zeros_like(new_k)
    new_slots = torch.zeros(case.B, dtype=torch.int64, device="cuda")
    seq_lens = torch.tensor(len0, dtype=torch.int32, device="cuda")
    q_host = torch.zeros(case.B, case.H_q, 128, dtype=case.dtype).pin_memory()
    q = torch.zeros(case.B, case.H_q, 128, dtype=case.dtype, device="cuda")
    slots_host = torch.empty(case.B, case.H_q, top_k, dtype=torch.int64).pin_memory()
    o_new_host = torch.zeros(case.B, case.H_q, 128, dtype=case.dtype).pin_memory()
    o_new = torch.empty_like(q)
    out = torch.empty_like(q)
    call = ops.DecodeCall(mode, q, kd, ks, vd, vs, case.block_table.cuda(), seq_lens, case.ctx, case.H_q,
                          case.H_kv, 16, top_k, case.attn_scale)
    host = ops.HostCorrectionCall(q_host, km_host, vm_host, None, slots_host, o_new_host, case.attn_scale)
    ops.set_cpu_attn_threads(3)

    def step(stream):
        ops.fused_quant_write_kv_mirror(new_k, new_v, new_slots, kd, ks, vd, vs, gs, kb, vb, km_dev, vm_dev)
        q.copy_(q_host, non_blocking=True)
        call.fused()
        slots_host.copy_(call.out["topk_slots"], non_blocking=True)
        host.stream_submit(stream)
        host.stream_wait(stream)
        o_new.copy_(o_new_host, non_blocking=True)
        ops.blend_unnorm_into(call.out["o_hat"], call.out["o_old_unnorm"], call.out["W"], o_new, out)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):       # eager once: kernel attributes, worker threads
        new_slots.fill_(-1)             # nothing is appended by the warm-up
        step(side)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step(torch.cuda.current_stream())
    g = torch.Generator().manual_seed(4)
    for t in range(steps):
        lens_now = [n + t + 1 for n in len0]
        slots_t = torch.tensor([slot_of(b, len0[b] + t) for b in range(case.B)], dtype=torch.int64)
        new_k.copy_(key_all[slots_t.cuda()])
        new_v.copy_(val_all[slots_t.cuda()])
        new_slots.copy_(slots_t)
        seq_lens.copy_(torch.tensor(lens_now, dtype=torch.int32))
        case.q = torch.randn(case.B, case.H_q, 128, generator=g).to(case.dtype)
        q_host.copy_(case.q)
        graph.replay()
        torch.cuda.synchronize()
        host.stream_status()
        call.status()
        case.seq_lens = torch.tensor(lens_now, dtype=torch.int32)
        ref = case.oracle_step(top_k)
        assert np.array_equal(slots_host.numpy(), ref["topk_slots"]), f"step {t}: selected slots differ"
        want = O.bf16_bits_to_f32(O.f32_to_bf16_bits(ref["out"]))
        err = np.abs(f32_values(out) - want)
        lim = 2e-3 + (1e-3 + 2 ** -8) * np.abs(want)
        assert (err <= lim).all(), f"step {t}: max err {err.max():.3e}"
    host.close()
