"""Host-side adapter logic on CPU: top-k width routing and head map (the reference's
tests/test_runtime_edge_cases.py:13-35), configuration, the decode gate."""
from types import SimpleNamespace

import pytest
import torch

from jetfire_b200.adapter import config as jcfg
from jetfire_b200.adapter.decode_path import _decode_unsupported, _select_top_k, make_decode_metadata


@pytest.mark.parametrize("length,expected", [(1, 32), (17, 32), (31, 32), (32, 32), (63, 32), (64, 64),
                                            (255, 128), (256, 256), (4096, 256)])
def test_positive_short_prompts_keep_cpu_correction(length, expected):
    assert _select_top_k(256, length, (32, 64, 128, 256)) == expected


@pytest.mark.parametrize("requested,length,supported", [(0, 128, (32, 64)), (16, 128, (32, 64)),
                                                       (32, 0, (32, 64)), (32, -1, (32, 64)), (256, 128, ())])
def test_empty_or_unsupported_decode_width_is_rejected(requested, length, supported):
    assert _select_top_k(requested, length, supported) is None


def test_tp2_local_gqa_default_head_map_keeps_heads_inside_local_shadow():
    """A TP-2 rank of a 64/8-head model sees 32 query heads over 4 local KV heads (the reference's
    tests/test_runtime_edge_cases.py:29-48).  The host correction called without a head map must
    gather query head h from local KV head h // 8 -- the same rows an explicit map selects."""
    from jetfire_b200 import ops
    from oracle import jf_oracle as O
    g = torch.Generator().manual_seed(7)
    B, H_q, H_kv, K, slots = 2, 32, 4, 16, 64
    q = torch.randn(B, H_q, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(H_kv, slots, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(H_kv, slots, 128, generator=g).to(torch.bfloat16)
    ts = torch.randint(0, slots, (B, H_q, K), generator=g, dtype=torch.int64)
    hm = torch.from_numpy(O.head_map(B, H_q, H_q // H_kv, K))
    for h in range(H_q):
        assert bool((hm[:, h] == h // 8).all())
    a, b = torch.empty_like(q), torch.empty_like(q)
    ops.set_cpu_attn_threads(2)
    ops.cpu_topk_attn(q, k, v, None, ts, a, 128 ** -0.5)
    ops.cpu_topk_attn(q, k, v, hm, ts, b, 128 ** -0.5)
    assert torch.equal(a, b)


def test_config_from_environment(monkeypatch):
    jcfg.reset_jetfire_config()
    monkeypatch.setenv("JETFIRE_MODE", "k4v4")
    monkeypatch.setenv("JETFIRE_TOPK", "512")
    cfg = jcfg.get_jetfire_config()
    assert (cfg.mode, cfg.group_size, cfg.top_k, cfg.kernel_mode) == ("SymInt4K_SymInt4V", 128, 512, "k4v4")
    jcfg.reset_jetfire_config()
    monkeypatch.setenv("JETFIRE_MODE", "SymInt3K_SymInt2V")
    monkeypatch.setenv("JETFIRE_GROUP_SIZE", "128")
    with pytest.raises(ValueError):
        jcfg.get_jetfire_config()
    jcfg.reset_jetfire_config()
    monkeypatch.setenv("JETFIRE_GROUP_SIZE", "64")
    monkeypatch.setenv("JETFIRE_TOPK", "100")
    with pytest.raises(ValueError):
        jcfg.get_jetfire_config()
    jcfg.reset_jetfire_config()


def test_compression_ratios_match_reference_figures():
    assert abs(jcfg.compute_inflate_ratio(jcfg.SYM_INT3K_SYM_INT2V, 64) - 5.82) < 0.01
    assert abs(jcfg.compute_inflate_ratio(jcfg.SYM_INT4K_SYM_INT4V, 128) - 3.88) < 0.01


def test_decode_gate_reasons():
    cfg = jcfg.JetFireConfig()
    impl = SimpleNamespace(attn_type=SimpleNamespace(name="DECODER"), scale=0.088)
    layer = SimpleNamespace(layer_name="l0", num_heads=32, num_kv_heads=8, head_size=128)
    store = SimpleNamespace(head_dim=128)
    q = torch.zeros(2, 32, 128)
    md = make_decode_metadata(torch.tensor([5, 9], dtype=torch.int32), torch.zeros(2, 1, dtype=torch.int64))
    args = dict(impl=impl, layer=layer, query=q, cfg=cfg, store=store)
    assert _decode_unsupported(attn_metadata=md, **args) is None
    assert _decode_unsupported(attn_metadata=None, **args) == "profiling_run"
    md.max_query_len = 7
    assert _decode_unsupported(attn_metadata=md, **args) == "prefill_or_multi_query"
    md.max_query_len = 1
    md.use_cascade = True
    assert _decode_unsupported(attn_metadata=md, **args) == "cascade"
    md.use_cascade = False
    assert _decode_unsupported(attn_metadata=md, **{**args, "store": None}) == "layer_config_missing"
    layer16 = SimpleNamespace(layer_name="l0", num_heads=32, num_kv_heads=2, head_size=128)
    assert _decode_unsupported(attn_metadata=md, **{**args, "layer": layer16}) is None      # ratio 16: two halves of 8
    layer12 = SimpleNamespace(layer_name="l0", num_heads=24, num_kv_heads=2, head_size=128)
    assert _decode_unsupported(attn_metadata=md, **{**args, "layer": layer12}) == "gqa_ratio"
    layer32 = SimpleNamespace(layer_name="l0", num_heads=64, num_kv_heads=2, head_size=128)
    assert _decode_unsupported(attn_metadata=md, **{**args, "layer": layer32}) == "gqa_ratio"
