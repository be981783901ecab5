"""Multi-rank host logic on CPU (gloo, world_size 2 and 4): shard plan and output gather."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from jetfire_b200.adapter.sharding import cpu_threads_per_rank, gather_outputs, shard_plan


def test_plan_llama70b_heads_over_2_4_8():
    for world, kv_per in ((2, 4), (4, 2), (8, 1)):
        plan = shard_plan(64, 8, 4, world)
        assert [s.kv_count for s in plan] == [kv_per] * world
        assert [s.q_start for s in plan] == [r * kv_per * 8 for r in range(world)]
        assert all(s.b_count == 4 and s.b_start == 0 for s in plan)


def test_plan_qwen_batch_split_after_heads_run_out():
    plan = shard_plan(32, 4, 8, 8)            # 4 KV heads -> 4 head shards x 2 batch shards
    assert sorted({(s.kv_start, s.b_start) for s in plan}) == [(h, b) for h in range(4) for b in (0, 4)]
    assert all(s.kv_count == 1 and s.q_count == 8 and s.b_count == 4 for s in plan)
    cover = torch.zeros(8, 32, dtype=torch.int32)
    for s in plan:
        cover[s.b_start:s.b_start + s.b_count, s.q_start:s.q_start + s.q_count] += 1
    assert bool((cover == 1).all())
    with pytest.raises(ValueError):
        shard_plan(32, 4, 3, 8)
    with pytest.raises(ValueError):
        shard_plan(32, 8, 4, 3)
    assert cpu_threads_per_rank(16, 8) == 2 and cpu_threads_per_rank(4, 8) == 1


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, H_q, H_kv, B, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(5)
        full = torch.randn(B, H_q, 128, generator=g).to(torch.bfloat16)      # what one GPU would produce
        plan = shard_plan(H_q, H_kv, B, world)
        s = plan[rank]
        local = full[s.b_start:s.b_start + s.b_count, s.q_start:s.q_start + s.q_count].clone()
        out = gather_outputs(local, plan, B, H_q)
        ok = torch.equal(out, full.reshape(B, H_q * 128))
        flags = [None] * world
        dist.all_gather_object(flags, ok)
        if rank == 0:
            ret.put(all(flags))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,H_q,H_kv,B", [(2, 32, 8, 4), (4, 32, 2, 4)])
def test_gather_into_tp_layout_gloo(world, H_q, H_kv, B):
    ctx = mp.get_context("spawn")
    ret = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, H_q, H_kv, B, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert ret.get() is True
