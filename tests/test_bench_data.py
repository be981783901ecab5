"""The bench's synthetic data and multi-GPU layout, on CPU: the counter-hash generator gives the
same bits through numpy and through torch integer ops (so the GPU's timed rows can be replayed
through the CPU oracle and any rank can build any shard), its values look like N(0,1), and the
gathered per-rank outputs land in the (B, H_q * 128) layout for every shard plan."""
import numpy as np
import pytest
import torch

import bench
from jetfire_b200.adapter.sharding import shard_plan


def _w(**kw):
    w = dict(mode="k3v2", H_q=8, H_kv=2, batch=3, ctx=80, top_k=32, layers=2, name="c1", stage_b="fp32")
    w.update(kw)
    return w


def test_generator_is_identical_in_numpy_and_torch():
    w = _w()
    for layer in (0, 1):
        cs = bench.channel_scale_np(w, layer)
        for tensor in (bench.T_K, bench.T_V):
            rows = bench.kv_rows_torch(torch, w, layer, tensor, 0, 2, 0, 3, "cpu", torch.float32, cs, chunk_tokens=48)
            for b in range(3):
                for h in range(2):
                    want = bench.kv_rows_np(w, layer, tensor, h, b, cs)
                    assert np.array_equal(rows[b * 80:(b + 1) * 80, h].numpy(), want)
    # a shard is the matching slice of the whole
    whole = bench.kv_rows_torch(torch, w, 1, bench.T_K, 0, 2, 0, 3, "cpu", torch.bfloat16, bench.channel_scale_np(w, 1))
    part = bench.kv_rows_torch(torch, w, 1, bench.T_K, 1, 1, 2, 1, "cpu", torch.bfloat16, bench.channel_scale_np(w, 1))
    assert torch.equal(part, whole[2 * 80:3 * 80, 1:2])


def test_generator_values_look_normal_and_layers_differ():
    x = bench._unit_normal_np(np.arange(2_000_000, dtype=np.uint64), 12345)
    assert abs(float(x.mean())) < 5e-3 and abs(float(x.std()) - 1.0) < 5e-3
    kurt = float(((x - x.mean()) ** 4).mean() / x.var() ** 2)
    assert 2.8 < kurt < 3.1
    w = _w()
    assert not np.array_equal(bench.kv_rows_np(w, 0, bench.T_K, 0, 0), bench.kv_rows_np(w, 1, bench.T_K, 0, 0))
    assert not np.array_equal(bench.kv_rows_np(w, 0, bench.T_K, 0, 0), bench.kv_rows_np(w, 0, bench.T_V, 0, 0))
    cs = bench.channel_scale_np(w, 0)
    assert cs.shape == (2, 128) and (cs > 0).all() and 0.5 < float(np.log(cs).std()) < 1.0


@pytest.mark.parametrize("H_q,H_kv,B,world", [(64, 8, 4, 2), (64, 8, 4, 8), (32, 4, 8, 8), (32, 4, 8, 4), (8, 2, 2, 1)])
def test_gathered_shards_land_in_the_tensor_parallel_layout(H_q, H_kv, B, world):
    plan = shard_plan(H_q, H_kv, B, world)
    n_layers = 3
    full = torch.arange(n_layers * B * H_q * 128, dtype=torch.float32).reshape(n_layers, B, H_q, 128)
    b_loc, q_loc = plan[0].b_count, plan[0].q_count
    gathered = torch.empty(world, n_layers, b_loc, q_loc * 128)
    for s in plan:   # what rank s.rank would contribute
        gathered[s.rank] = full[:, s.b_start:s.b_start + b_loc, s.q_start:s.q_start + q_loc].reshape(n_layers, b_loc, -1)
    out = torch.empty(n_layers, B, H_q * 128)
    bench.to_tp_layout(gathered, out, min(world, H_kv))
    assert torch.equal(out, full.reshape(n_layers, B, H_q * 128))
