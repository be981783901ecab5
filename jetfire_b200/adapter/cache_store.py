"""Per-layer packed KV cache with its full-precision host mirror
(jetfire_vllm/adapter/cache_store.py:193-359 for the layout, :686-759 for the append).

Layout (unchanged from the reference): ``k_data (H_kv, num_slots, 128*kbits/8) u8``,
``k_scales (H_kv, num_slots, 128/group) bf16``, the same for V, ``slot_filled (num_slots,)
bool``; mirror ``k_shadow / v_shadow (H_kv, num_slots, 128)`` in host DRAM in the model's
16-bit dtype.  ``num_slots = num_blocks * 16``.

Three ways to fill the mirror on an append (``mirror_append``):
  * ``"mapped"`` -- the mirror is mapped pinned host memory and the packing kernel stores the
    rows into it itself: one launch, no host step (the default when a mirror is kept);
  * ``"stream"`` -- ordinary host memory; rows go through pinned staging and a host callback
    in the CUDA stream (the reference's graph-mode path, cache_store.py:616-640);
  * ``"sync"``   -- copy, host synchronisation and ``index_copy_`` as in the reference's eager
    path (cache_store.py:746-756).
With the first two, ``flush_pending_writes`` makes the mirror current for host readers.
"""
from __future__ import annotations

import torch

from .. import ops
from .config import JetFireConfig
from .sharding import resolve_numa_node


class JetFireCacheStore:
    def __init__(self, *, num_blocks: int, num_kv_heads: int, head_dim: int, cfg: JetFireConfig,
                 device, dtype=torch.bfloat16, shadow_enabled: bool = True, block_size: int = 16,
                 mirror_append: str = "mapped", stream_chunk_tokens: int = 4096):
        if head_dim != 128 or block_size != 16:
            raise ValueError("the decode path is built for head_dim 128 and block_size 16")
        if mirror_append not in ("mapped", "stream", "sync"):
            raise ValueError("mirror_append must be 'mapped', 'stream' or 'sync'")
        self.cfg = cfg
        self.block_size = block_size
        self.num_blocks = int(num_blocks)
        self.num_slots = self.num_blocks * block_size
        self.num_kv_heads = int(num_kv_heads)
        self.head_dim = head_dim
        self.group_size = cfg.group_size
        self.k_nbits, self.v_nbits = cfg.scheme.k_nbits, cfg.scheme.v_nbits
        self.device = torch.device(device)
        self.dtype = dtype
        ng = head_dim // self.group_size
        dev = dict(device=self.device)
        self.k_data = torch.zeros(num_kv_heads, self.num_slots, head_dim * self.k_nbits // 8, dtype=torch.uint8, **dev)
        self.v_data = torch.zeros(num_kv_heads, self.num_slots, head_dim * self.v_nbits // 8, dtype=torch.uint8, **dev)
        self.k_scales = torch.zeros(num_kv_heads, self.num_slots, ng, dtype=torch.bfloat16, **dev)
        self.v_scales = torch.zeros(num_kv_heads, self.num_slots, ng, dtype=torch.bfloat16, **dev)
        # one spare entry at the end takes the writes of padding / out-of-range slots, so that the
        # bookkeeping below is a plain scatter with no host step (and can be captured in a graph)
        self._filled_buf = torch.zeros(self.num_slots + 1, dtype=torch.bool, **dev)
        self.slot_filled = self._filled_buf[:self.num_slots]
        self.written_count = 0
        self.shadow_enabled = bool(shadow_enabled)
        self.mirror_append = mirror_append
        self._k_shadow_dev = self._v_shadow_dev = None
        self._append_ctx = None
        self._pending_event = None
        # memory node of the mirrors (and of the workers that gather from them): the GPU's own on a
        # host with several nodes, unless configured otherwise
        self.numa_node = -1
        if self.shadow_enabled and self.device.type == "cuda":
            index = self.device.index if self.device.index is not None else torch.cuda.current_device()
            self.numa_node = resolve_numa_node(cfg.numa_node, ops.numa_node_of_device(index), ops.numa_node_count())
        if self.shadow_enabled:
            shape = (num_kv_heads, self.num_slots, head_dim)
            if mirror_append == "mapped":
                self.k_shadow, self._k_shadow_dev = ops.alloc_mapped_pinned_pair(shape, dtype, node=self.numa_node)
                self.v_shadow, self._v_shadow_dev = ops.alloc_mapped_pinned_pair(shape, dtype, node=self.numa_node)
                self.k_shadow.zero_()
                self.v_shadow.zero_()
            else:
                self.k_shadow = torch.empty(*shape, dtype=dtype)
                self.v_shadow = torch.empty(*shape, dtype=dtype)
                for t in (self.k_shadow, self.v_shadow):   # 2 MB pages under the mirrors, asked for before the first write
                    ops.advise_huge_pages(t)
                    if self.numa_node >= 0:
                        ops.bind_memory_to_node(t, self.numa_node)
                    t.zero_()
                if mirror_append == "stream":
                    self._append_ctx = ops.MirrorAppendCtx(self.k_shadow, self.v_shadow, stream_chunk_tokens)
        else:
            self.k_shadow = self.v_shadow = None

    def write_slots(self, key_tok: torch.Tensor, value_tok: torch.Tensor, slot_idx: torch.Tensor) -> None:
        """Append ``key_tok / value_tok (T, H_kv, 128)`` at ``slot_idx (T,)``: quantise into the
        packed cache on the GPU and copy the rows into the host mirror.  Negative slots are
        padding and are skipped on both sides (jetfire_vllm/kernels/fused_quant_write.py:150-152)."""
        if key_tok.shape != value_tok.shape or key_tok.dim() != 3:
            raise RuntimeError("write_slots: key/value must be (T, H_kv, 128) and match")
        slot_idx = slot_idx.to(torch.int64)
        mapped = self.shadow_enabled and self.mirror_append == "mapped"
        if mapped:
            ops.fused_quant_write_kv_mirror(key_tok, value_tok, slot_idx, self.k_data, self.k_scales, self.v_data,
                                            self.v_scales, self.group_size, self.k_nbits, self.v_nbits,
                                            self._k_shadow_dev, self._v_shadow_dev)
        else:
            ops.fused_quant_write_kv(key_tok, value_tok, slot_idx, self.k_data, self.k_scales, self.v_data,
                                     self.v_scales, self.group_size, self.k_nbits, self.v_nbits)
        live = (slot_idx >= 0) & (slot_idx < self.num_slots)   # what the packing kernel wrote
        self._filled_buf.index_fill_(0, torch.where(live, slot_idx, self.num_slots), True)
        self.written_count += int(key_tok.shape[0])
        if self.shadow_enabled and self.mirror_append == "stream":
            self._append_ctx.append(key_tok, value_tok, slot_idx)
        if self.shadow_enabled and self.mirror_append != "sync":
            # Under stream capture the append is a node of the graph being built: whoever replays
            # the graph orders host reads of the mirror against it, and no event is recorded here
            # (the reference's graph path skips its bookkeeping as well, cache_store.py:611-614).
            if not torch.cuda.is_current_stream_capturing():
                ev = torch.cuda.Event()
                ev.record()
                self._pending_event = ev
            return
        if self.shadow_enabled:
            idx_cpu = slot_idx.to("cpu")                       # host sync, as in the reference's eager path
            keep = (idx_cpu >= 0) & (idx_cpu < self.num_slots)
            idx_cpu = idx_cpu[keep]
            k_cpu = key_tok.to("cpu")[keep].transpose(0, 1).to(self.dtype)
            v_cpu = value_tok.to("cpu")[keep].transpose(0, 1).to(self.dtype)
            self.k_shadow.index_copy_(1, idx_cpu, k_cpu)
            self.v_shadow.index_copy_(1, idx_cpu, v_cpu)

    def flush_pending_writes(self) -> None:
        """Wait until every appended row is in the mirror (cache_store.py:1340-1387).  Needed
        before a host thread reads the mirror; work on the same CUDA stream needs nothing."""
        ev, self._pending_event = self._pending_event, None
        if ev is not None:
            ev.synchronize()
