"""Steps that hold decode and prefill sequences together, on CPU: the split of the rows
(jetfire_vllm/adapter/decode_path.py:1402-1663 of the reference), the counts noted on the
metadata when it is built (jetfire_backend.py:66-127) and the routing of each part, with the
decode part replaced by a recorder (the real one needs a GPU and is covered by the GPU tests)."""
import sys
from types import ModuleType, SimpleNamespace

import pytest
import torch

from jetfire_b200.adapter import config as jcfg
from jetfire_b200.adapter import mixed_batch as mb
from jf_testlib import causal_prefill_attention


def test_split_of_an_ordered_step():
    sp = mb.split_mixed_batch([0, 1, 2, 7, 10], [40, 17, 5, 3])
    assert sp.decode_seqs == [0, 1] and sp.decode_rows == [0, 1]
    assert sp.prefill_seqs == [2, 3] and sp.prefill_rows == list(range(2, 10))
    assert sp.prefill_cu == [0, 5, 8] and sp.max_prefill_len == 5
    assert sp.ordered and sp.mixed and not sp.prefill_with_context


def test_split_of_an_interleaved_step_with_padding():
    # prefill, decode, (empty), prefill, decode
    sp = mb.split_mixed_batch([0, 4, 5, 5, 8, 9], [4, 100, 0, 3, 7])
    assert sp.decode_seqs == [1, 4] and sp.decode_rows == [4, 8]
    assert sp.prefill_seqs == [0, 3] and sp.prefill_rows == [0, 1, 2, 3, 5, 6, 7]
    assert sp.prefill_cu == [0, 4, 7] and not sp.ordered and sp.mixed


def test_one_new_token_over_cached_context_is_a_decode_row_and_longer_ones_are_flagged():
    sp = mb.split_mixed_batch([0, 1, 4], [90, 50])      # sequence 1: 3 new tokens, 47 cached
    assert sp.decode_seqs == [0] and sp.prefill_seqs == [1] and sp.prefill_with_context == [1]
    sp = mb.split_mixed_batch([0, 1, 2], [90, 1])       # a one-token prompt decodes over its own token
    assert sp.decode_seqs == [0, 1] and not sp.mixed


def test_split_rejects_inconsistent_input():
    with pytest.raises(ValueError):
        mb.split_mixed_batch([0, 3, 2], [3, 1])
    with pytest.raises(ValueError):
        mb.split_mixed_batch([0, 1, 2, 3], [1, 1])


def test_split_partitions_the_rows_of_any_step():
    """Seeded random steps: every query row belongs to exactly one part, the prefill offsets are the
    running sum of the prefill lengths, and a step counts as ordered exactly when its decode
    sequences come before its prefill sequences (empty sequences aside)."""
    import random
    rnd = random.Random(5)
    for _ in range(300):
        n = rnd.randint(1, 12)
        qlens = [rnd.choice([0, 1, 1, 1, 2, 3, 7, 40]) for _ in range(n)]
        seq_lens = [q + (rnd.choice([0, 0, 5, 100]) if q else 0) for q in qlens]
        qsl = [0]
        for q in qlens:
            qsl.append(qsl[-1] + q)
        sp = mb.split_mixed_batch(qsl, seq_lens)
        assert sorted(sp.decode_rows + sp.prefill_rows) == list(range(qsl[-1]))
        assert sp.decode_seqs == [i for i, q in enumerate(qlens) if q == 1]
        assert sp.prefill_seqs == [i for i, q in enumerate(qlens) if q > 1]
        assert sp.prefill_cu == [0] + [sum(qlens[i] for i in sp.prefill_seqs[:k + 1]) for k in range(len(sp.prefill_seqs))]
        assert sp.max_prefill_len == max([qlens[i] for i in sp.prefill_seqs], default=0)
        assert sp.prefill_with_context == [i for i in sp.prefill_seqs if seq_lens[i] != qlens[i]]
        live = [q for q in qlens if q]
        kinds = ["d" if q == 1 else "p" for q in live]
        decode_first = "".join(kinds) == "d" * kinds.count("d") + "p" * kinds.count("p")
        contiguous_decodes = (not sp.decode_seqs
                              or sp.decode_seqs == list(range(sp.decode_seqs[0], sp.decode_seqs[0] + len(sp.decode_seqs))))
        assert sp.ordered == (decode_first and contiguous_decodes), (qlens, sp)


def test_counts_noted_on_the_metadata():
    md = mb.annotate_split_counts(SimpleNamespace(), torch.tensor([0, 1, 2, 7]), torch.tensor([9, 12, 5]))
    assert (md.num_decodes, md.num_prefills, md.num_decode_tokens, md.num_prefill_tokens) == (2, 1, 2, 5)
    assert md.jetfire_prefill_has_context is False and md.jetfire_max_prefill_context_len == 0
    md = mb.annotate_split_counts(SimpleNamespace(), [0, 1, 6], [9, 25])
    assert md.jetfire_prefill_has_context is True and md.jetfire_max_prefill_context_len == 20
    md = mb.annotate_split_counts(SimpleNamespace(), [0, 5, 6], [5, 9])     # decode after prefill: no counts
    assert not hasattr(md, "num_decodes") and md.jetfire_prefill_has_context is False


H_Q, H_KV, D = 4, 2, 128


class _Recorder:
    """Stands in for the decode entry: notes what it was given, writes row index + 1000."""

    def __init__(self, serve=True):
        self.calls, self.serve = [], serve

    def __call__(self, *, impl, layer, query, attn_metadata, output, store, cfg):
        self.calls.append(SimpleNamespace(query=query.clone(), md=attn_metadata))
        if not self.serve:
            return None
        n = query.shape[0]
        output.copy_((1000 + torch.arange(n, dtype=torch.float32))[:, None].expand(n, output.shape[1]))
        return output


def _step(qlens, seq_lens, flat, seed=0):
    g = torch.Generator().manual_seed(seed)
    T = sum(qlens)
    q = torch.randn(T, H_Q, D, generator=g)
    k = torch.randn(T, H_KV, D, generator=g)
    v = torch.randn(T, H_KV, D, generator=g)
    qsl = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32)
    md = SimpleNamespace(query_start_loc=qsl, seq_lens=torch.tensor(seq_lens, dtype=torch.int32),
                         block_table=torch.arange(len(qlens) * 3, dtype=torch.int64).view(len(qlens), 3),
                         max_query_len=max(qlens), max_seq_len=max(seq_lens), num_actual_tokens=T,
                         use_cascade=False, causal=True)
    out = torch.full((T, H_Q, D), -7.0)
    if flat:
        q, k, v, out = q.view(T, -1), k.view(T, -1), v.view(T, -1), out.view(T, -1)
    return q, k, v, md, out


def _parts():
    impl = SimpleNamespace(attn_type=SimpleNamespace(name="DECODER"), scale=D ** -0.5)
    layer = SimpleNamespace(layer_name="l0", num_heads=H_Q, num_kv_heads=H_KV, head_size=D)
    return impl, layer, SimpleNamespace(head_dim=D), jcfg.JetFireConfig()


def _expected_prefill(q, k, v, lo, hi, scale):
    out = torch.empty(hi - lo, H_Q, D)
    causal_prefill_attention(q=q.view(-1, H_Q, D)[lo:hi], k=k.view(-1, H_KV, D)[lo:hi], v=v.view(-1, H_KV, D)[lo:hi],
                             out=out, cu_seqlens=torch.tensor([0, hi - lo]), max_seqlen=hi - lo,
                             impl=SimpleNamespace(scale=scale), layer=None, attn_metadata=None)
    return out


@pytest.mark.parametrize("flat", [False, True])
@pytest.mark.parametrize("with_counts", [False, True])
def test_ordered_step_is_routed_by_rows(monkeypatch, flat, with_counts):
    rec = _Recorder()
    monkeypatch.setattr(mb, "try_jetfire_decode", rec)
    qlens, lens = [1, 1, 5, 3], [40, 17, 5, 3]
    q, k, v, md, out = _step(qlens, lens, flat)
    if with_counts:
        mb.annotate_split_counts(md, md.query_start_loc, md.seq_lens)
    impl, layer, store, cfg = _parts()
    stats = mb.MixedBatchStats()
    got = mb.try_jetfire_mixed(impl=impl, layer=layer, query=q, key=k, value=v, attn_metadata=md, output=out,
                               store=store, cfg=cfg, prefill_attention=causal_prefill_attention, stats=stats)
    assert got is out
    call = rec.calls[0]
    assert torch.equal(call.query, q.view(-1, H_Q, D)[:2])
    assert call.md.seq_lens.tolist() == [40, 17] and call.md.block_table.tolist() == md.block_table[:2].tolist()
    assert call.md.max_query_len == 1 and call.md.num_actual_tokens == 2
    assert call.md.max_seq_len == 40 and call.md.query_start_loc.tolist() == [0, 1, 2]
    o = out.view(-1, H_Q, D)
    assert bool((o[0] == 1000).all()) and bool((o[1] == 1001).all())
    assert torch.allclose(o[2:7], _expected_prefill(q, k, v, 2, 7, impl.scale), atol=1e-5)
    assert torch.allclose(o[7:10], _expected_prefill(q, k, v, 7, 10, impl.scale), atol=1e-5)
    assert (stats.mixed_batch_count, stats.mixed_batch_decode_seqs, stats.mixed_batch_prefill_seqs,
            stats.mixed_batch_decode_tokens, stats.mixed_batch_prefill_tokens) == (1, 2, 2, 2, 8)


def test_interleaved_step_is_routed_by_rows(monkeypatch):
    rec = _Recorder()
    monkeypatch.setattr(mb, "try_jetfire_decode", rec)
    qlens, lens = [4, 1, 3, 1], [4, 100, 3, 7]
    q, k, v, md, out = _step(qlens, lens, flat=True, seed=3)
    impl, layer, store, cfg = _parts()
    got = mb.try_jetfire_mixed(impl=impl, layer=layer, query=q, key=k, value=v, attn_metadata=md, output=out,
                               store=store, cfg=cfg, prefill_attention=causal_prefill_attention,
                               stats=mb.MixedBatchStats())
    assert got is out
    call = rec.calls[0]
    assert torch.equal(call.query, q.view(-1, H_Q, D)[[4, 8]])
    assert call.md.seq_lens.tolist() == [100, 7] and call.md.max_seq_len == 100
    assert call.md.block_table.tolist() == md.block_table[[1, 3]].tolist()
    o = out.view(-1, H_Q, D)
    assert bool((o[4] == 1000).all()) and bool((o[8] == 1001).all())
    assert torch.allclose(o[0:4], _expected_prefill(q, k, v, 0, 4, impl.scale), atol=1e-5)
    assert torch.allclose(o[5:8], _expected_prefill(q, k, v, 5, 8, impl.scale), atol=1e-5)


def test_steps_that_are_handed_back(monkeypatch):
    rec = _Recorder()
    monkeypatch.setattr(mb, "try_jetfire_decode", rec)
    impl, layer, store, cfg = _parts()

    def run(md, q, k, v, out, **over):
        stats = mb.MixedBatchStats()
        args = dict(impl=impl, layer=layer, query=q, key=k, value=v, attn_metadata=md, output=out, store=store,
                    cfg=cfg, prefill_attention=causal_prefill_attention, stats=stats)
        args.update(over)
        return mb.try_jetfire_mixed(**args), stats.handed_back

    q, k, v, md, out = _step([1, 1, 5], [40, 17, 5], flat=False)
    assert run(md, q, k, v, out, store=None) == (None, {"layer_config_missing": 1})
    assert run(None, q, k, v, out) == (None, {"profiling_run": 1})
    assert run(md, q, k, v, out, cfg=jcfg.JetFireConfig(enabled=False)) == (None, {"pool_disabled": 1})
    assert run(md, q, k, v, out, impl=SimpleNamespace(attn_type=SimpleNamespace(name="ENCODER"), scale=1.0)) \
        == (None, {"attn_type": 1})
    cascade = SimpleNamespace(**{**vars(md), "use_cascade": True})
    assert run(cascade, q, k, v, out) == (None, {"cascade": 1})
    q2, k2, v2, md2, out2 = _step([1, 1], [40, 17], flat=False)
    assert run(md2, q2, k2, v2, out2) == (None, {"pure_decode": 1})
    q3, k3, v3, md3, out3 = _step([6, 2], [6, 2], flat=False)
    assert run(md3, q3, k3, v3, out3) == (None, {"not_mixed": 1})
    q4, k4, v4, md4, out4 = _step([1, 3], [40, 30], flat=False)           # 27 cached tokens under a prefill row
    assert run(md4, q4, k4, v4, out4) == (None, {"prefill_with_context": 1})
    mb.annotate_split_counts(md4, md4.query_start_loc, md4.seq_lens)
    assert run(md4, q4, k4, v4, out4) == (None, {"prefill_with_context": 1})
    spec = SimpleNamespace(**vars(md), num_decodes=1, num_prefills=1, num_decode_tokens=2, num_prefill_tokens=5,
                           jetfire_prefill_has_context=False)
    assert run(spec, q, k, v, out) == (None, {"multi_token_decode": 1})
    assert not rec.calls
    # the decode part refuses: nothing has been written
    monkeypatch.setattr(mb, "try_jetfire_decode", _Recorder(serve=False))
    assert run(md, q, k, v, out) == (None, {"decode_part_unsupported": 1})
    assert bool((out == -7.0).all())


def test_backend_forward_tries_decode_then_mixed_then_native(monkeypatch):
    import jetfire_b200.adapter.jetfire_backend as jb
    seen = []
    monkeypatch.setattr(jb, "try_jetfire_decode", lambda **kw: seen.append("decode") or None)
    monkeypatch.setattr(jb, "try_jetfire_mixed", lambda **kw: seen.append("mixed") or kw["output"])
    monkeypatch.setattr(jb, "get_jetfire_config", lambda: jcfg.JetFireConfig())

    class Native:
        def forward(self, *a, **kw):
            seen.append("native")
            return "native"

    class Impl(jb.JetFireAttentionImplMixin, Native):
        pass

    q, k, v, md, out = _step([1, 4], [9, 4], flat=True)
    layer = SimpleNamespace(layer_name="l0")
    assert Impl().forward(layer, q, k, v, None, md, output=out) is out and seen == ["decode", "mixed"]
    seen.clear()
    monkeypatch.setattr(jb, "try_jetfire_mixed", lambda **kw: seen.append("mixed") or None)
    assert Impl().forward(layer, q, k, v, None, md, output=out) == "native" and seen == ["decode", "mixed", "native"]
    seen.clear()
    assert Impl().forward(layer, q, None, None, None, md, output=out) == "native" and seen == ["decode", "native"]


@pytest.mark.parametrize("module,returns", [("vllm.vllm_flash_attn", False), ("flash_attn", True)])
def test_default_prefill_attention_calls_whichever_flash_attention_is_installed(monkeypatch, module, returns):
    got = {}

    def varlen(**kw):
        got.update(kw)
        if returns:
            return torch.full_like(kw["q"], 2.0)
        kw["out"].fill_(2.0)

    fake = ModuleType(module)
    fake.flash_attn_varlen_func = varlen
    for name in ("vllm.vllm_flash_attn", "flash_attn"):
        monkeypatch.setitem(sys.modules, name, None)        # import of the other one fails
    monkeypatch.setitem(sys.modules, module, fake)
    if "." in module:
        parent = sys.modules.get("vllm") or ModuleType("vllm")
        monkeypatch.setitem(sys.modules, "vllm", parent)
        monkeypatch.setattr(parent, "vllm_flash_attn", fake, raising=False)
    monkeypatch.setattr(mb, "_FLASH_FN", None)
    monkeypatch.setattr(mb, "_FLASH_FROM_VLLM", False)
    q = torch.zeros(5, H_Q, D)
    out = torch.zeros(5, H_Q, D)
    impl = SimpleNamespace(scale=0.25, sliding_window=(-1, -1), logits_soft_cap=0.0, vllm_flash_attn_version=3)
    mb.flash_varlen_prefill(q=q, k=q[:, :H_KV], v=q[:, :H_KV], out=out, cu_seqlens=torch.tensor([0, 5]), max_seqlen=5,
                            impl=impl, layer=None, attn_metadata=SimpleNamespace(causal=True))
    assert bool((out == 2.0).all())
    assert got["softmax_scale"] == 0.25 and got["causal"] is True and got["max_seqlen_q"] == 5
    assert tuple(got["window_size"]) == (-1, -1) and "softcap" not in got
    assert ("fa_version" in got) == (not returns) and ("out" in got) == (not returns)


def test_missing_flash_attention_is_an_import_error(monkeypatch):
    for name in ("vllm.vllm_flash_attn", "flash_attn"):
        monkeypatch.setitem(sys.modules, name, None)
    monkeypatch.setattr(mb, "_FLASH_FN", None)
    with pytest.raises(ImportError, match="prefill_attention"):
        mb._resolve_flash_varlen()
