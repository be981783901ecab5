"""Decode orchestrator (jetfire_vllm/adapter/decode_path.py:1156-1182, 400-408, 1667-1712,
and the op order of ``_decode_batched`` :1712-3237):

    fused scan + top-k + finish (GPU)  ->  D2H of q and the selected slots  ->  host
    correction over the mirror (C++ worker pool)  ->  o_new to the GPU  ->  merge into the
    caller's output.

The reference's Stage A / Stage B pair is one fused call here, so nothing is left to overlap
the host correction with inside a layer; across layers the caller may pipeline.

Two forms of the step.  The host-waiting one (``JETFIRE_STREAM_ORDERED=0``, and whenever the
store's mirror is not the mapped one) waits on the host for the selected slots, runs the
correction and returns with the merge queued.  The stream-ordered one
(``JetFireConfig.stream_ordered``, the default; the reference's graph-mode decode: create_cpu_topk_submit_ctx /
stream_submit_cpu_topk_attn / stream_wait_cpu_topk_attn, csrc/cpu_topk_attn.cpp:2147-2312, call
sites decode_path.py:2253-2492) queues everything on the CUDA stream over buffers that keep their
addresses -- copies, kernels, the correction's submit and join as host functions in the stream --
and never waits on the host, so a whole step can be captured in a CUDA graph and replayed.
``JetFireConfig.stream_signal`` chooses how the stream and the host meet: ``"flags"`` -- a kernel
raises a word in mapped memory that a dispatcher thread polls, and a kernel polls the word the
last worker sets (decode_path.py:2426-2438, :3061-3064 of the reference, with a bounded wait) --
or ``"callbacks"`` -- host functions in the stream.
"""
from __future__ import annotations

from types import SimpleNamespace

import torch

from .. import ops
from .cache_store import JetFireCacheStore
from .config import SUPPORTED_TOP_K, JetFireConfig, get_jetfire_config
from .sharding import cpu_threads_per_rank, workers_on_node

def _select_top_k(config_top_k: int, seq_len: int, supported: tuple[int, ...]) -> int | None:
    """Largest supported width <= the sequence length (short sequences are padded with -1),
    else the smallest configured width; None for empty sequences or nothing configured."""
    requested, length = int(config_top_k), int(seq_len)
    configured = [k for k in supported if 0 < k <= requested]
    if not configured or length <= 0:
        return None
    candidates = [k for k in configured if k <= length]
    return max(candidates) if candidates else min(configured)


def _decode_unsupported(*, impl, layer, query, attn_metadata, cfg: JetFireConfig, store) -> str | None:
    """Gate: a reason string on a miss, None on a hit (decode_path.py:1667-1695)."""
    if not cfg.enabled:
        return "pool_disabled"
    if attn_metadata is None:
        return "profiling_run"
    if getattr(getattr(impl, "attn_type", None), "name", "DECODER") != "DECODER":
        return "attn_type"
    if getattr(attn_metadata, "use_cascade", False):
        return "cascade"
    if int(attn_metadata.max_query_len) != 1:
        return "prefill_or_multi_query"
    n_seqs = int(attn_metadata.seq_lens.numel())
    if int(attn_metadata.num_actual_tokens) != n_seqs:
        return "batch_mismatch"
    if int(query.shape[0]) < n_seqs:
        return "empty_query"
    if store is None:
        return "layer_config_missing"
    if int(query.shape[-1]) != store.head_dim:
        return "head_dim_mismatch"
    ratio = int(layer.num_heads) // max(int(layer.num_kv_heads), 1)
    if int(layer.num_heads) % int(layer.num_kv_heads) != 0 or (ratio > 8 and ratio != 16):
        return "gqa_ratio"
    return None


class _DecodeBuffers:
    """Pinned staging for one (batch, heads, top_k) shape."""

    def __init__(self, B, H_q, K, dtype, slot_dtype=torch.int64):
        self.q_host = torch.empty(B, H_q, 128, dtype=dtype).pin_memory()
        self.ts_host = torch.empty(B, H_q, K, dtype=slot_dtype).pin_memory()
        self.o_new_host = torch.empty(B, H_q, 128, dtype=dtype).pin_memory()


_BUFFERS: dict[tuple, _DecodeBuffers] = {}
_WORKERS_SET: tuple[int, int] | None = None


def _set_worker_count(cfg: JetFireConfig, node: int = -1) -> None:
    """Size and place the correction pool once: the configured count, capped by this rank's share
    of the host cores (the ranks of a node share them; ``sharding.cpu_threads_per_rank``); with a
    memory node given (the store's, where its mirrors are), the workers run on that node's
    processors only and share them with the other ranks placed there."""
    global _WORKERS_SET
    import os
    world = int(os.environ.get("WORLD_SIZE", "1") or 1)
    # One core of the rank's share stays with the thread that drives the GPU (with a worker on every
    # core that thread is preempted and every layer waits for it), one more with the dispatcher
    # thread when the stream starts the corrections through trigger words.
    spare = 2 if (cfg.stream_ordered and cfg.stream_signal == "flags") else 1
    want = max(1, min(int(cfg.cpu_attn_threads), cpu_threads_per_rank(os.cpu_count() or 1, world) - spare))
    if node >= 0:
        try:
            cpus = len(ops.numa_node_cpus(node))
        except RuntimeError:
            node, cpus = -1, 0
        if node >= 0:
            nodes = max(ops.numa_node_count(), 1)
            want = min(want, workers_on_node(int(cfg.cpu_attn_threads), cpus, (world + nodes - 1) // nodes))
    if _WORKERS_SET != (want, node):
        ops.set_cpu_attn_node(node)
        ops.set_cpu_attn_threads(want)
        _WORKERS_SET = (want, node)


class _StreamStep:
    """Buffers and calls of one layer's stream-ordered decode step for one (batch, top-k) shape.
    Everything the kernels and the host correction read or write sits at fixed addresses, so the
    step can be captured once and replayed; the per-step inputs are copied in on the stream."""

    def __init__(self, store: JetFireCacheStore, cfg: JetFireConfig, B: int, H_q: int, top_k: int,
                 max_blocks: int, max_S: int, dtype, device, scale: float):
        self.B, self.H_q, self.top_k, self.max_blocks, self.max_S = B, H_q, top_k, max_blocks, max_S
        self.q = torch.zeros(B, H_q, 128, dtype=dtype, device=device)
        self.block_table = torch.zeros(B, max_blocks, dtype=torch.int64, device=device)
        self.seq_lens = torch.zeros(B, dtype=torch.int32, device=device)
        self.call = ops.DecodeCall(cfg.kernel_mode, self.q, store.k_data, store.k_scales, store.v_data,
                                   store.v_scales, self.block_table, self.seq_lens, max_S, H_q, store.num_kv_heads,
                                   store.block_size, top_k, scale, slots_i32=cfg.slots_i32)
        slot_dtype = torch.int32 if cfg.slots_i32 else torch.int64
        self.slots_dev = self.call.out["topk_slots_i32"] if cfg.slots_i32 else self.call.out["topk_slots"]
        self.q_host = torch.zeros(B, H_q, 128, dtype=dtype).pin_memory()
        self.slots_host = torch.zeros(B, H_q, top_k, dtype=slot_dtype).pin_memory()
        self.out = torch.zeros(B, H_q, 128, dtype=dtype, device=device)
        self.flags = cfg.stream_signal == "flags"
        # rows [cut, B * H_q) of the correction are the GPU's (read from the mapped mirror over the host
        # link while the workers do the others): only with flags, where the kernel that waits for the
        # workers comes after it on the stream
        rows = B * H_q
        self.rows, self.cut = rows, rows
        if self.flags and cfg.gpu_correction_share > 0.0 and store._k_shadow_dev is not None:
            self.cut = max(1, rows - int(round(min(cfg.gpu_correction_share, 0.5) * rows)))
        self.mirrors_dev = (store._k_shadow_dev, store._v_shadow_dev)
        self.scale = scale
        if self.flags:
            # the correction is started and joined through two words in mapped memory (a line apart),
            # and its result is read by the merge kernel where the workers wrote it
            self.words_host, self.words_dev = ops.alloc_mapped_pinned_pair((16,), torch.int64)
            self.words_host.zero_()
            self.o_new_host, self.o_new = ops.alloc_mapped_pinned_pair((B, H_q, 128), dtype)
            self.o_new_host.zero_()
            self.host = ops.HostCorrectionCall(self.q_host, store.k_shadow, store.v_shadow, None, self.slots_host,
                                               self.o_new_host, scale, done_flag=self.words_host[8:9],
                                               rows=(0, self.cut) if self.cut < rows else None)
            self.host.watch(self.words_host[0:1])
        else:
            self.o_new_host = torch.zeros(B, H_q, 128, dtype=dtype).pin_memory()
            self.o_new = torch.zeros(B, H_q, 128, dtype=dtype, device=device)
            self.host = ops.HostCorrectionCall(self.q_host, store.k_shadow, store.v_shadow, None, self.slots_host,
                                               self.o_new_host, scale)
        self.status_host = torch.zeros(ops.STATUS_RECORD_BYTES, dtype=torch.uint8).pin_memory()
        self.status_event: torch.cuda.Event | None = None
        self.captured = False

    def check_previous(self) -> None:
        """Raise if the previous eager run of this step recorded an error.  Looks only at what has
        already arrived on the host: the record's copy once its event has completed, and the
        correction context's own status.  Never waits."""
        ev = self.status_event
        if ev is not None and ev.query():
            self.status_event = None
            ops.decode_status_of_copy(self.status_host)
            self.host.stream_status()

    def run(self, query: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor, out_view: torch.Tensor) -> None:
        capturing = torch.cuda.is_current_stream_capturing()
        if not capturing:
            self.check_previous()
        self.q.copy_(query, non_blocking=True)
        width = min(int(block_table.shape[1]), self.max_blocks)
        self.block_table[:, :width].copy_(block_table[:, :width], non_blocking=True)    # converts the dtype as well
        self.seq_lens.copy_(seq_lens, non_blocking=True)
        self.call.fused()
        self.q_host.copy_(self.q, non_blocking=True)
        self.slots_host.copy_(self.slots_dev, non_blocking=True)
        if self.flags:
            ops.stream_signal_host(self.words_dev[8:9], self.words_dev[0:1])
            if self.cut < self.rows:        # the GPU's rows, while the workers do theirs
                ops.gpu_topk_attn_rows(self.q, self.mirrors_dev[0], self.mirrors_dev[1], self.slots_dev, self.o_new,
                                       self.scale, (self.cut, self.rows))
            ops.stream_wait_host_flag(self.words_dev[8:9], _HOST_WAIT_MS, self.call.status_record())
        else:
            self.host.stream_submit()
            self.host.stream_wait()
            self.o_new.copy_(self.o_new_host, non_blocking=True)
        res = self.call.out
        if out_view.is_contiguous():
            ops.blend_unnorm_into(res["o_hat"], res["o_old_unnorm"], res["W"], self.o_new, out_view)
        else:
            ops.blend_unnorm_into(res["o_hat"], res["o_old_unnorm"], res["W"], self.o_new, self.out)
            out_view.copy_(self.out)
        self.status_host.copy_(self.call.status_record(), non_blocking=True)
        if capturing:
            self.captured = True        # a graph refers to these buffers from now on
        else:
            ev = torch.cuda.Event()
            ev.record()
            self.status_event = ev

    def status(self) -> None:
        """For the owner of a graph, after synchronising a replay: raise if the step recorded an error."""
        ops.decode_status_of_copy(self.status_host)
        self.host.stream_status()

    def close(self) -> None:
        """Release the correction context (the dispatcher stops polling its trigger word).  Only
        once nothing queued on a stream, and no graph, refers to this step any more."""
        self.host.close()


_MAX_S_STEP = 4096      # a step object serves row lengths up to the next multiple of this
_HOST_WAIT_MS = 5000    # budget of the kernel that waits for the host correction


def stream_steps(store: JetFireCacheStore) -> list[_StreamStep]:
    """Every stream-ordered step of a store (for ``status()`` once a graph replay has been
    synchronised).  The steps live on the store: they hold its tensors' addresses."""
    return list(getattr(store, "_stream_steps", {}).values()) + list(getattr(store, "_captured_steps", []))


def decode_batched_stream_ordered(*, store: JetFireCacheStore, query: torch.Tensor, block_table: torch.Tensor,
                                  seq_lens: torch.Tensor, max_seq_len: int, num_heads: int, scale: float,
                                  output: torch.Tensor, cfg: JetFireConfig | None = None) -> torch.Tensor | None:
    """``decode_batched`` without a host wait: everything is queued on the current stream (which
    must be the stream the appends were queued on: the correction reads the mirror when the stream
    reaches its submit).  Capturable.  ``max_seq_len`` is a host integer (under capture: the bound
    the graph is to serve); the mirror must be the mapped one."""
    cfg = cfg or get_jetfire_config()
    B = int(seq_lens.numel())
    top_k = _select_top_k(cfg.top_k, int(max_seq_len), SUPPORTED_TOP_K)
    if top_k is None or not store.shadow_enabled or store.mirror_append != "mapped":
        return None
    width = int(block_table.shape[1])
    need_S = min(width * store.block_size, ((int(max_seq_len) + 15) // 16) * 16)
    steps = store.__dict__.setdefault("_stream_steps", {})
    key = (B, num_heads, top_k, query.dtype, cfg.slots_i32, cfg.stream_signal, float(scale), cfg.gpu_correction_share)
    step = steps.get(key)
    if step is None or step.max_S < need_S or step.max_blocks < min(width, (need_S + 15) // 16):
        max_S = min(width * store.block_size, -(-need_S // _MAX_S_STEP) * _MAX_S_STEP)
        if step is not None:
            # The sequences have outgrown the step's buffers (once per _MAX_S_STEP tokens).  A step a
            # graph refers to stays as it is; any other is released once the stream has drained --
            # its last run may still be waiting for its correction.
            if step.captured or torch.cuda.is_current_stream_capturing():
                store.__dict__.setdefault("_captured_steps", []).append(step)
            else:
                torch.cuda.current_stream().synchronize()
                step.check_previous()
                step.close()
        _set_worker_count(cfg, getattr(store, "numa_node", -1))
        step = steps[key] = _StreamStep(store, cfg, B, num_heads, top_k, max_S // store.block_size, max_S,
                                        query.dtype, query.device, float(scale))
    step.run(query[:B], block_table, seq_lens, output[:B].view(B, num_heads, 128))
    return output


def decode_batched(*, store: JetFireCacheStore, query: torch.Tensor, block_table: torch.Tensor,
                   seq_lens: torch.Tensor, max_seq_len: int, num_heads: int, scale: float,
                   output: torch.Tensor, cfg: JetFireConfig | None = None) -> torch.Tensor | None:
    """One decode step of one layer.  ``query (B, H_q, 128)``, ``output (B, H_q, 128)`` (a view
    of the caller's buffer, written in place).  Returns ``output``, or None when the
    configured top-k cannot be served."""
    cfg = cfg or get_jetfire_config()
    B = int(seq_lens.numel())
    top_k = _select_top_k(cfg.top_k, int(max_seq_len), SUPPORTED_TOP_K)
    if top_k is None:
        return None
    store.flush_pending_writes()
    q = query[:B].contiguous()
    bt = block_table if block_table.dtype == torch.int64 else block_table.to(torch.int64)
    lens = seq_lens if seq_lens.dtype == torch.int32 else seq_lens.to(torch.int32)
    max_S = min(int(bt.shape[1]) * store.block_size, ((int(max_seq_len) + 15) // 16) * 16)
    call = ops.DecodeCall(cfg.kernel_mode, q, store.k_data, store.k_scales, store.v_data, store.v_scales,
                          bt, lens, max_S, num_heads, store.num_kv_heads, store.block_size, top_k, scale,
                          slots_i32=cfg.slots_i32)
    call.fused()
    res = call.result()
    slot_dtype = torch.int32 if cfg.slots_i32 else torch.int64
    key = (B, num_heads, top_k, q.dtype, slot_dtype)
    buf = _BUFFERS.get(key)
    if buf is None:
        buf = _BUFFERS[key] = _DecodeBuffers(B, num_heads, top_k, q.dtype, slot_dtype)
    buf.q_host.copy_(q, non_blocking=True)
    # the slots cross to the host as 32-bit integers (half the bytes) unless configured otherwise
    buf.ts_host.copy_(call.out["topk_slots_i32"] if cfg.slots_i32 else res.topk_slots, non_blocking=True)
    call.status()   # synchronises the stream; raises if a bounded wait inside a kernel ran out
    _set_worker_count(cfg, getattr(store, "numa_node", -1))
    ops.cpu_topk_attn(buf.q_host, store.k_shadow, store.v_shadow, None, buf.ts_host, buf.o_new_host, scale)
    o_new = buf.o_new_host.to(q.device, non_blocking=True)
    out_view = output[:B].view(B, num_heads, 128)
    if out_view.is_contiguous():
        ops.blend_unnorm_into(res.o_hat, res.o_old_unnorm, res.W, o_new, out_view)
    else:
        tmp = torch.empty(B, num_heads, 128, dtype=q.dtype, device=q.device)
        ops.blend_unnorm_into(res.o_hat, res.o_old_unnorm, res.W, o_new, tmp)
        out_view.copy_(tmp)
    return output


def try_jetfire_decode(*, impl, layer, query, attn_metadata, output, store=None, cfg=None,
                       key=None, value=None):
    """Decode entry with the reference's calling convention (decode_path.py:1699-1712):
    returns ``output`` on success, None when a precondition fails (the caller then uses its
    native attention)."""
    cfg = cfg or get_jetfire_config()
    if _decode_unsupported(impl=impl, layer=layer, query=query, attn_metadata=attn_metadata,
                           cfg=cfg, store=store) is not None:
        return None
    n = int(attn_metadata.seq_lens.numel())
    q = query[:n].view(n, int(layer.num_heads), int(layer.head_size))
    # stream-ordered when configured and the store's mirror is the mapped one (the GPU appends to it in
    # stream order); otherwise the host-waiting form, which cannot run under stream capture
    stream_ordered = cfg.stream_ordered and store.shadow_enabled and store.mirror_append == "mapped"
    if not stream_ordered and query.is_cuda and torch.cuda.is_current_stream_capturing():
        return None
    step = decode_batched_stream_ordered if stream_ordered else decode_batched
    return step(store=store, query=q, block_table=attn_metadata.block_table,
                          seq_lens=attn_metadata.seq_lens, max_seq_len=int(attn_metadata.max_seq_len),
                          num_heads=int(layer.num_heads), scale=float(impl.scale), output=output, cfg=cfg)


def make_decode_metadata(seq_lens: torch.Tensor, block_table: torch.Tensor) -> SimpleNamespace:
    """Stand-in for vLLM's decode metadata (the reference builds the same kind of object for
    its sub-batches, decode_path.py:1532-1544)."""
    n = int(seq_lens.numel())
    return SimpleNamespace(seq_lens=seq_lens, max_seq_len=int(seq_lens.max().item()) if n else 0,
                           max_query_len=1, num_actual_tokens=n, block_table=block_table,
                           use_cascade=False, query_start_loc=torch.arange(n + 1, dtype=torch.int32))
