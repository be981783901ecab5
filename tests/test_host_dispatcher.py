"""The dispatcher that lets the GPU start a host correction through a word in host memory, on
CPU: the test plays the GPU's part (raises the trigger word, polls the completion word)."""
import time

import pytest
import torch

from jetfire_b200 import _lib, ops


def _buffers(seed, B=2, H_q=8, H_kv=2, K=16, slots=64):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H_q, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(H_kv, slots, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(H_kv, slots, 128, generator=g).to(torch.bfloat16)
    ts = torch.randint(0, slots, (B, H_q, K), generator=g, dtype=torch.int32)
    return q, k, v, ts


def _wait(word, value, seconds=5.0):
    t_end = time.time() + seconds
    while int(word[0]) != value and time.time() < t_end:
        time.sleep(0.0005)
    return int(word[0]) == value


def test_trigger_word_starts_the_job_and_the_completion_word_reports_it():
    ops.set_cpu_attn_threads(3)
    q, k, v, ts = _buffers(1)
    want = torch.empty_like(q)
    ops.cpu_topk_attn(q, k, v, None, ts, want, 0.09)
    words = torch.zeros(16, dtype=torch.int64)
    trigger, done = words[0:1], words[8:9]
    got = torch.zeros_like(q)
    call = ops.HostCorrectionCall(q, k, v, None, ts, got, 0.09, done_flag=done)
    call.watch(trigger)
    for step in range(3):                       # the same words serve step after step, as under graph replay
        q.copy_(_buffers(10 + step)[0])
        ops.cpu_topk_attn(q, k, v, None, ts, want, 0.09)
        got.zero_()
        done.zero_()                            # the GPU's kernel clears the completion word, then raises the trigger
        trigger.fill_(1)
        assert _wait(done, 1), "the job never completed"
        assert int(trigger[0]) == 0             # taken by the dispatcher
        assert torch.equal(got, want)
    call.stream_status()
    call.close()
    trigger.fill_(1)                            # nobody watches any more: nothing happens
    time.sleep(0.05)
    assert int(trigger[0]) == 1 and int(done[0]) == 1


def test_several_contexts_are_watched_at_once():
    ops.set_cpu_attn_threads(2)
    calls = []
    for i in range(5):
        q, k, v, ts = _buffers(20 + i)
        words = torch.zeros(16, dtype=torch.int64)
        got = torch.zeros_like(q)
        call = ops.HostCorrectionCall(q, k, v, None, ts, got, 0.09, done_flag=words[8:9])
        call.watch(words[0:1])
        want = torch.empty_like(q)
        ops.cpu_topk_attn(q, k, v, None, ts, want, 0.09)
        calls.append((call, words, got, want))
    for _, words, _, _ in reversed(calls):
        words[0] = 1
    for call, words, got, want in calls:
        assert _wait(words[8:9], 1) and torch.equal(got, want)
        call.close()


def test_a_watched_context_may_cover_a_range_of_rows():
    ops.set_cpu_attn_threads(2)
    q, k, v, ts = _buffers(31)
    want = torch.empty_like(q)
    ops.cpu_topk_attn(q, k, v, None, ts, want, 0.09)
    words = torch.zeros(16, dtype=torch.int64)
    got = torch.full_like(q, 7.0)
    call = ops.HostCorrectionCall(q, k, v, None, ts, got, 0.09, done_flag=words[8:9], rows=(2, 13))
    call.watch(words[0:1])
    words[0] = 1
    assert _wait(words[8:9], 1)
    g, w = got.view(-1, 128), want.view(-1, 128)
    assert torch.equal(g[2:13], w[2:13]) and bool((g[:2] == 7).all()) and bool((g[13:] == 7).all())
    call.close()
    assert _lib.lib.jf_submit_ctx_set_rows(0, 0, 1) == _lib.JF_ERR_ARG


def test_watch_arguments():
    l = _lib.lib
    assert l.jf_submit_ctx_watch(0, None) == _lib.JF_ERR_ARG
    assert l.jf_submit_ctx_unwatch(0) == _lib.JF_ERR_ARG
    assert l.jf_stream_signal_host(None, None, None) == _lib.JF_ERR_ARG
    assert l.jf_stream_wait_host_flag(None, None, 10, None) == _lib.JF_ERR_ARG
    word = torch.zeros(2, dtype=torch.int64)
    assert l.jf_stream_wait_host_flag(None, word.data_ptr(), 0, None) == _lib.JF_ERR_ARG        # no budget
    assert l.jf_stream_wait_host_flag(None, word.data_ptr() + 4, 10, None) == _lib.JF_ERR_ARG   # misaligned
    q, k, v, ts = _buffers(3)
    call = ops.HostCorrectionCall(q, k, v, None, ts, torch.empty_like(q), 0.09, done_flag=word[1:2])
    with pytest.raises(RuntimeError):
        call.watch(torch.zeros(2, dtype=torch.int64))
    with pytest.raises(RuntimeError):
        call.watch(torch.zeros(1, dtype=torch.int32))
    call.close()
