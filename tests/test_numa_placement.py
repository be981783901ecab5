"""Placement of the host mirrors and the correction workers on a memory node: the machine
layout read from a made-up sysfs tree, the binding call, the confinement of the workers (seen
through the affinity of this process's threads) and the adapter's choice of node.  No GPU."""
import ctypes as C
import os

import pytest
import torch

from jetfire_b200 import _lib, ops
from jetfire_b200.adapter import config as jcfg
from jetfire_b200.adapter.sharding import resolve_numa_node, workers_on_node


@pytest.fixture
def two_nodes(tmp_path, monkeypatch):
    """A host with two memory nodes of which this process may use processors 0 and 1 only."""
    node = tmp_path / "devices" / "system" / "node"
    (node / "node0").mkdir(parents=True)
    (node / "node1").mkdir()
    (node / "online").write_text("0-1\n")
    (node / "node0" / "cpulist").write_text("0-1\n")
    (node / "node1" / "cpulist").write_text("2-3,6,8-9\n")
    monkeypatch.setenv("JF_SYSFS_ROOT", str(tmp_path))
    yield tmp_path
    ops.set_cpu_attn_node(-1)


def test_layout_is_read_from_sysfs(two_nodes):
    assert ops.numa_node_count() == 2
    assert ops.numa_node_cpus(0) == [0, 1] and ops.numa_node_cpus(1) == [2, 3, 6, 8, 9]
    with pytest.raises(RuntimeError):
        ops.numa_node_cpus(2)
    count = C.c_int32(0)
    two = (C.c_int32 * 2)()
    assert _lib.lib.jf_numa_node_cpus(1, two, 2, C.byref(count)) == _lib.JF_OK
    assert count.value == 5 and list(two) == [2, 3]                 # the count is the node's, not the buffer's
    assert _lib.lib.jf_numa_node_cpus(1, None, 2, C.byref(count)) == _lib.JF_ERR_ARG
    assert _lib.lib.jf_numa_node_cpus(1, two, 2, None) == _lib.JF_ERR_ARG


@pytest.mark.parametrize("text", ["", "a-b", "3-1", "1,,2", "0-", "-3"])
def test_malformed_lists_are_refused(two_nodes, text):
    (two_nodes / "devices" / "system" / "node" / "node1" / "cpulist").write_text(text + "\n")
    with pytest.raises(RuntimeError):
        ops.numa_node_cpus(1)
    with pytest.raises(RuntimeError):
        ops.set_cpu_attn_node(1)


def test_a_host_that_says_nothing_has_one_node(tmp_path, monkeypatch):
    monkeypatch.setenv("JF_SYSFS_ROOT", str(tmp_path / "nothing"))
    assert ops.numa_node_count() == 1
    assert ops.numa_node_of_device(0) == -1
    t = torch.empty(1 << 16, dtype=torch.uint8)
    assert ops.bind_memory_to_node(t, 0) is False


def test_binding_memory(two_nodes):
    t = torch.empty(1 << 22, dtype=torch.uint8)
    assert ops.bind_memory_to_node(t, 5) is False                   # not a node of this host
    ops.bind_memory_to_node(t, 1)                                   # listed, but the kernel may know better: either answer
    t.fill_(3)
    assert int(t.sum()) == 3 << 22
    assert _lib.lib.jf_bind_memory_to_node(None, 16, 0) == _lib.JF_ERR_ARG
    assert _lib.lib.jf_bind_memory_to_node(t.data_ptr(), 0, 0) == _lib.JF_ERR_ARG
    assert _lib.lib.jf_bind_memory_to_node(t.data_ptr(), 16, -1) == _lib.JF_ERR_ARG
    small = torch.empty(64, dtype=torch.uint8)                       # no whole page inside: nothing to do
    assert _lib.lib.jf_bind_memory_to_node(small.data_ptr() + 1, 8, 0) == _lib.JF_OK


def test_binding_on_the_real_host():
    """Node 0 of the machine the tests run on: the call either binds or is refused (containers may
    forbid it); the memory stays usable either way."""
    t = torch.empty(1 << 22, dtype=torch.uint8)
    assert ops.bind_memory_to_node(t, 0) in (True, False)
    t.zero_()
    assert not t.any()


def _thread_affinities():
    out = []
    for tid in os.listdir("/proc/self/task"):
        try:
            out.append(frozenset(os.sched_getaffinity(int(tid))))
        except OSError:
            pass
    return out


def _one_job(seed=0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(2, 8, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(2, 64, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(2, 64, 128, generator=g).to(torch.bfloat16)
    ts = torch.randint(0, 64, (2, 8, 16), generator=g, dtype=torch.int64)
    o = torch.empty_like(q)
    ops.cpu_topk_attn(q, k, v, None, ts, o, 128 ** -0.5)
    return o


@pytest.mark.skipif(not {0, 1} <= os.sched_getaffinity(0) or len(os.sched_getaffinity(0)) < 3,
                    reason="needs processors 0 and 1 and one more")
def test_workers_are_confined_to_the_node_and_released_again(two_nodes):
    ops.set_cpu_attn_threads(3)
    ops.set_cpu_attn_node(-1)
    free = _one_job()
    assert frozenset({0, 1}) not in _thread_affinities()
    ops.set_cpu_attn_node(0)
    assert ops.get_cpu_attn_node() == 0
    pinned = _one_job()                                              # the pool restarts with the next job
    assert _thread_affinities().count(frozenset({0, 1})) == 3
    assert torch.equal(free, pinned)
    ops.set_cpu_attn_node(-1)
    again = _one_job()
    assert frozenset({0, 1}) not in _thread_affinities() and torch.equal(free, again)
    with pytest.raises(RuntimeError):
        ops.set_cpu_attn_node(-2)


def test_choice_of_node():
    # (configured, node of the GPU, nodes of the host)
    assert resolve_numa_node(jcfg.NUMA_AUTO, 1, 2) == 1
    assert resolve_numa_node(jcfg.NUMA_AUTO, -1, 2) == -1            # the host does not say where the GPU sits
    assert resolve_numa_node(jcfg.NUMA_AUTO, 0, 1) == -1             # one node: nothing to place
    assert resolve_numa_node(jcfg.NUMA_OFF, 1, 2) == -1
    assert resolve_numa_node(0, 1, 2) == 0
    assert resolve_numa_node(3, 1, 2) == -1                          # a node this host lacks
    assert workers_on_node(32, 56, 4) == 14 and workers_on_node(8, 56, 4) == 8 and workers_on_node(8, 2, 4) == 1


def test_node_from_the_environment(monkeypatch):
    for raw, want in (("auto", jcfg.NUMA_AUTO), ("off", jcfg.NUMA_OFF), ("1", 1), ("", jcfg.NUMA_AUTO)):
        jcfg.reset_jetfire_config()
        monkeypatch.setenv("JETFIRE_NUMA_NODE", raw)
        assert jcfg.get_jetfire_config().numa_node == want
    for raw in ("left", "-3"):
        jcfg.reset_jetfire_config()
        monkeypatch.setenv("JETFIRE_NUMA_NODE", raw)
        with pytest.raises(ValueError):
            jcfg.get_jetfire_config()
    jcfg.reset_jetfire_config()
