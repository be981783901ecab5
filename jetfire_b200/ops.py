"""Operator surface of the JetFire decode hot path, on top of the C ABI.

Names, argument order and meaning follow the reference's torch-extension ops and Triton
writers so that its adapter can call these unchanged; torch is used only for device
memory and streams.  Each op validates like the reference's ``TORCH_CHECK``s (raising
``RuntimeError``) and runs on ``torch.cuda.current_stream()``.

Reference interfaces mirrored here (paths inside the JetFire project):
  * ``fused_quant_write_int{2,3,4}_sym`` -- jetfire_vllm/kernels/fused_quant_write.py:242, :337, :746
  * ``fused_quant_write_int4_sym_kv``    -- jetfire_vllm/kernels/fused_quant_write.py:552
  * ``fused_attn_topk``                  -- the single-call form of
    jetfire_vllm/kernels/int2_fused_attn_topk.py:5-10 generalised to K3V2 / K4V4
  * ``blend_unnorm_into``                -- jetfire_vllm/csrc/blend.cu:229-290
  * ``cpu_topk_attn`` and friends        -- jetfire_vllm/csrc/cpu_topk_attn.cpp:854-956, :2509-2663
"""
from __future__ import annotations

import ctypes as C
from typing import NamedTuple

import torch

from . import _lib
from ._lib import DecodeArgs, JetFireError, check, lib

MODE_IDS = {"k3v2": _lib.JF_MODE_K3V2, "k4v4": _lib.JF_MODE_K4V4,
            "SymInt3K_SymInt2V": _lib.JF_MODE_K3V2, "SymInt4K_SymInt4V": _lib.JF_MODE_K4V4}
MODE_BITS = {_lib.JF_MODE_K3V2: (3, 2, 64), _lib.JF_MODE_K4V4: (4, 4, 128)}


def _dtype_id(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _lib.JF_DTYPE_BF16
    if t.dtype == torch.float16:
        return _lib.JF_DTYPE_FP16
    raise RuntimeError(f"expected bfloat16 or float16, got {t.dtype}")


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


# ---------------------------------------------------------------------------------------
# quantise-on-append
# ---------------------------------------------------------------------------------------

def _packed_dim(nbits: int) -> int:
    return 128 * nbits // 8


def _check_side(x_tok, out_data, out_scale, nbits, group_size, name):
    _require(x_tok.is_cuda and out_data.is_cuda and out_scale.is_cuda, f"{name}: tensors must be CUDA")
    _require(x_tok.dim() == 3 and x_tok.shape[2] == 128, f"{name}: x_tok must be (T, H_kv, 128)")
    _require(x_tok.stride(2) == 1, f"{name}: x_tok innermost dim must be contiguous")
    _require(out_data.dtype == torch.uint8 and out_data.is_contiguous(), f"{name}: out_data must be contiguous uint8")
    _require(out_scale.dtype == torch.bfloat16 and out_scale.is_contiguous(), f"{name}: out_scale must be contiguous bf16")
    _require(group_size in (64, 128), f"{name}: group_size must be 64 or 128")
    h = x_tok.shape[1]
    _require(out_data.dim() == 3 and out_data.shape[0] == h and out_data.shape[2] == _packed_dim(nbits),
             f"{name}: out_data must be (H_kv, num_slots, {_packed_dim(nbits)})")
    _require(out_scale.shape[0] == h and out_scale.shape[1] == out_data.shape[1]
             and out_scale.numel() == h * out_data.shape[1] * (128 // group_size),
             f"{name}: out_scale must be (H_kv, num_slots, {128 // group_size})")


def _quant_write(x_tok, slot_idx, out_data, out_scale, group_size, nbits, name):
    _check_side(x_tok, out_data, out_scale, nbits, group_size, name)
    _require(slot_idx.is_cuda and slot_idx.dtype == torch.int64 and slot_idx.dim() == 1
             and slot_idx.shape[0] == x_tok.shape[0], f"{name}: slot_idx must be (T,) int64 CUDA")
    slot_idx = slot_idx.contiguous()
    st = lib.jf_pack_append(x_tok.data_ptr(), _dtype_id(x_tok), x_tok.shape[0], x_tok.shape[1],
                            x_tok.stride(0), x_tok.stride(1), slot_idx.data_ptr(),
                            out_data.data_ptr(), out_scale.data_ptr(), out_data.shape[1],
                            nbits, group_size, _stream())
    check(name, st)


def fused_quant_write_int2_sym(x_tok, slot_idx, out_data, out_scale, group_size=128):
    """In place: INT2 rows of ``x_tok`` into ``out_data[h, slot]`` / ``out_scale[h, slot]``."""
    _quant_write(x_tok, slot_idx, out_data, out_scale, group_size, 2, "fused_quant_write_int2_sym")


def fused_quant_write_int3_sym(x_tok, slot_idx, out_data, out_scale, group_size=128):
    _quant_write(x_tok, slot_idx, out_data, out_scale, group_size, 3, "fused_quant_write_int3_sym")


def fused_quant_write_int4_sym(x_tok, slot_idx, out_data, out_scale, group_size=128):
    _quant_write(x_tok, slot_idx, out_data, out_scale, group_size, 4, "fused_quant_write_int4_sym")


def fused_quant_write_kv(key_tok, value_tok, slot_idx, k_data, k_scales, v_data, v_scales,
                         group_size, k_bits, v_bits):
    """K and V of the same tokens in one launch, any bit pair."""
    name = "fused_quant_write_kv"
    _check_side(key_tok, k_data, k_scales, k_bits, group_size, name)
    _check_side(value_tok, v_data, v_scales, v_bits, group_size, name)
    _require(key_tok.shape == value_tok.shape and key_tok.dtype == value_tok.dtype,
             f"{name}: key/value shape or dtype mismatch")
    _require(k_data.shape[1] == v_data.shape[1], f"{name}: K and V caches differ in num_slots")
    _require(slot_idx.is_cuda and slot_idx.dtype == torch.int64 and slot_idx.dim() == 1
             and slot_idx.shape[0] == key_tok.shape[0], f"{name}: slot_idx must be (T,) int64 CUDA")
    slot_idx = slot_idx.contiguous()
    st = lib.jf_pack_append_kv(key_tok.data_ptr(), value_tok.data_ptr(), _dtype_id(key_tok),
                               key_tok.shape[0], key_tok.shape[1],
                               key_tok.stride(0), key_tok.stride(1), value_tok.stride(0), value_tok.stride(1),
                               slot_idx.data_ptr(), k_data.data_ptr(), k_scales.data_ptr(),
                               v_data.data_ptr(), v_scales.data_ptr(), k_data.shape[1],
                               k_bits, v_bits, group_size, _stream())
    check(name, st)


def fused_quant_write_int4_sym_kv(key_tok, value_tok, slot_idx, k_data, k_scales, v_data, v_scales,
                                  group_size=128):
    fused_quant_write_kv(key_tok, value_tok, slot_idx, k_data, k_scales, v_data, v_scales, group_size, 4, 4)


def _check_mirror(t, key_tok, k_data, name):
    _require(t.is_cuda and t.is_contiguous() and t.dtype == key_tok.dtype and t.dim() == 3
             and t.shape[0] == k_data.shape[0] and t.shape[1] == k_data.shape[1] and t.shape[2] == 128,
             f"{name}: mirror must be a contiguous device-visible (H_kv, num_slots, 128) tensor of the tokens' dtype")


def fused_quant_write_kv_mirror(key_tok, value_tok, slot_idx, k_data, k_scales, v_data, v_scales,
                                group_size, k_bits, v_bits, k_mirror_dev, v_mirror_dev):
    """``fused_quant_write_kv`` that also stores every live row, bit for bit, into the mirrors.
    ``k_mirror_dev / v_mirror_dev`` are the DEVICE views of mapped host mirrors (the second
    tensor of ``alloc_mapped_pinned_pair``, or ``map_host_tensor`` of an existing one): the
    append is one launch with no host step, in place of the reference's copy + sync +
    index_copy_ (jetfire_vllm/adapter/cache_store.py:746-756)."""
    name = "fused_quant_write_kv_mirror"
    _check_side(key_tok, k_data, k_scales, k_bits, group_size, name)
    _check_side(value_tok, v_data, v_scales, v_bits, group_size, name)
    _require(key_tok.shape == value_tok.shape and key_tok.dtype == value_tok.dtype,
             f"{name}: key/value shape or dtype mismatch")
    _require(k_data.shape[1] == v_data.shape[1], f"{name}: K and V caches differ in num_slots")
    _require(slot_idx.is_cuda and slot_idx.dtype == torch.int64 and slot_idx.dim() == 1
             and slot_idx.shape[0] == key_tok.shape[0], f"{name}: slot_idx must be (T,) int64 CUDA")
    _check_mirror(k_mirror_dev, key_tok, k_data, name)
    _check_mirror(v_mirror_dev, key_tok, k_data, name)
    slot_idx = slot_idx.contiguous()
    st = lib.jf_pack_append_kv_mirror(key_tok.data_ptr(), value_tok.data_ptr(), _dtype_id(key_tok),
                                      key_tok.shape[0], key_tok.shape[1],
                                      key_tok.stride(0), key_tok.stride(1), value_tok.stride(0), value_tok.stride(1),
                                      slot_idx.data_ptr(), k_data.data_ptr(), k_scales.data_ptr(),
                                      v_data.data_ptr(), v_scales.data_ptr(), k_data.shape[1],
                                      k_bits, v_bits, group_size, k_mirror_dev.data_ptr(), v_mirror_dev.data_ptr(),
                                      _stream())
    check(name, st)


def map_host_tensor(host: torch.Tensor) -> torch.Tensor:
    """Page-lock an existing contiguous CPU tensor and return a CUDA tensor over the same bytes
    (for ``fused_quant_write_kv_mirror``).  ``unmap_host_tensor(host)`` undoes it."""
    _require(not host.is_cuda and host.is_contiguous(), "map_host_tensor: contiguous CPU tensor expected")
    nbytes = host.numel() * host.element_size()
    d = C.c_void_p()
    check("map_host_tensor", lib.jf_map_host(host.data_ptr(), nbytes, C.byref(d)))
    dev_ptr = d.value

    class _DevView:
        __cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (dev_ptr, False), "version": 2, "strides": None}

    return torch.as_tensor(_DevView(), device="cuda").view(host.dtype)[:host.numel()].reshape(host.shape)


def unmap_host_tensor(host: torch.Tensor) -> None:
    check("unmap_host_tensor", lib.jf_unmap_host(host.data_ptr()))


class MirrorAppendCtx:
    """Stream-ordered append to mirrors in ordinary host memory (the reference's
    create_shadow_append_submit_ctx + stream_submit_shadow_append,
    jetfire_vllm/csrc/cpu_topk_attn.cpp:1611-1665, with its pinned staging of
    adapter/cache_store.py:616-640 owned by the context).  ``append`` returns at once; the
    rows are in the mirror when the stream has passed the work it enqueued."""

    def __init__(self, k_shadow: torch.Tensor, v_shadow: torch.Tensor, max_tokens: int):
        _require(not k_shadow.is_cuda and not v_shadow.is_cuda and k_shadow.is_contiguous()
                 and v_shadow.is_contiguous() and k_shadow.shape == v_shadow.shape and k_shadow.dim() == 3
                 and k_shadow.shape[2] == 128 and k_shadow.dtype == v_shadow.dtype
                 and k_shadow.dtype in (torch.bfloat16, torch.float16),
                 "MirrorAppendCtx: mirrors must be contiguous CPU (H_kv, num_slots, 128) 16-bit tensors")
        self._keep = (k_shadow, v_shadow)
        h = C.c_int64()
        check("MirrorAppendCtx", lib.jf_mirror_append_ctx_create(k_shadow.data_ptr(), v_shadow.data_ptr(),
                                                                 k_shadow.shape[0], k_shadow.shape[1],
                                                                 int(max_tokens), C.byref(h)))
        self.handle = h.value

    def append(self, key_tok, value_tok, slot_idx):
        name = "MirrorAppendCtx.append"
        k_shadow = self._keep[0]
        _require(self.handle != 0, f"{name}: context was closed")
        _require(key_tok.is_cuda and value_tok.is_cuda and key_tok.shape == value_tok.shape and key_tok.dim() == 3
                 and key_tok.shape[1] == k_shadow.shape[0] and key_tok.shape[2] == 128
                 and key_tok.dtype == k_shadow.dtype and value_tok.dtype == k_shadow.dtype
                 and key_tok.stride(2) == 1 and value_tok.stride(2) == 1,
                 f"{name}: key/value must be CUDA (T, H_kv, 128) of the mirror's dtype, innermost contiguous")
        _require(slot_idx.is_cuda and slot_idx.dtype == torch.int64 and slot_idx.dim() == 1
                 and slot_idx.shape[0] == key_tok.shape[0], f"{name}: slot_idx must be (T,) int64 CUDA")
        slot_idx = slot_idx.contiguous()
        check(name, lib.jf_stream_mirror_append(_stream(), self.handle, key_tok.data_ptr(), value_tok.data_ptr(),
                                                key_tok.shape[0], key_tok.stride(0), key_tok.stride(1),
                                                value_tok.stride(0), value_tok.stride(1), slot_idx.data_ptr()))

    def stats(self):
        w, s, c = C.c_int64(), C.c_int64(), C.c_int64()
        check("MirrorAppendCtx.stats", lib.jf_mirror_append_ctx_stats(self.handle, C.byref(w), C.byref(s), C.byref(c)))
        return {"rows_written": w.value, "rows_skipped": s.value, "chunks": c.value}

    def close(self):
        """Synchronise the work that uses the context first."""
        if self.handle:
            lib.jf_mirror_append_ctx_destroy(self.handle)
            self.handle = 0


# ---------------------------------------------------------------------------------------
# fused decode attention
# ---------------------------------------------------------------------------------------

class FusedAttnOut(NamedTuple):
    o_hat: torch.Tensor          # (B, H_q, 128) f32
    topk_slots: torch.Tensor     # (B, H_q, k) i64
    o_old_unnorm: torch.Tensor   # (B, H_q, 128) f32
    W: torch.Tensor              # (B, H_q) f32
    topk_idx: torch.Tensor       # (B, H_q, k) i64
    softmax_m: torch.Tensor      # (B, H_q) f32
    softmax_inv_z: torch.Tensor  # (B, H_q) f32
    scores: torch.Tensor | None  # (B, H_q, max_S) f32 when requested


_WORKSPACES: dict[tuple[int, int], torch.Tensor] = {}
_PARTS = {"all": _lib.JF_SCAN_ALL, "k": _lib.JF_SCAN_K_ONLY, "v": _lib.JF_SCAN_V_ONLY}
_STAGE_B = {"fp32": _lib.JF_STAGE_B_FP32, "int8p": _lib.JF_STAGE_B_INT8P}


def decode_workspace_bytes(mode, B, H_q, H_kv, max_S, top_k) -> int:
    return int(lib.jf_decode_workspace_bytes(MODE_IDS[mode] if isinstance(mode, str) else mode,
                                             B, H_q, H_kv, max_S, top_k))


def get_workspace(nbytes: int, device) -> torch.Tensor:
    """Cached scratch (grows monotonically per device); one per current stream is the
    caller's business when streams overlap."""
    dev = torch.device(device)
    key = (dev.index if dev.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream().cuda_stream)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes + 256, dtype=torch.uint8, device=dev)
        _WORKSPACES[key] = ws
    return ws


class DecodeCall:
    """Argument block for the decode entry points, built once and reusable (pointers are
    captured; tensors are kept alive here).

    ``stage_b``: ``"fp32"`` (full-precision softmax weights) or ``"int8p"`` (K4V4 only: the
    reference's batch > 1 arithmetic, weights rounded to 127 levels per 32-token tile).
    ``parts``: ``"all"``, ``"k"`` (scores and softmax sums only: q and the K cache; V tensors may be
    None) or ``"v"`` (output partials from ``scores``, an input then: the V cache; q and K tensors
    may be None).  ``scores`` / ``topk_idx``: existing tensors to use instead of fresh ones.
    ``slots_i32``: also write the selected slots as 32-bit integers (``out["topk_slots_i32"]``) --
    half the bytes for the copy to the host; the host correction takes either width."""

    def __init__(self, mode, q, k_data, k_scales, v_data, v_scales, block_table, seq_lens,
                 max_S, H_q, H_kv, block_size, top_k, attn_scale, *, workspace=None,
                 want_scores=False, out=None, stage_b="fp32", parts="all", scores=None, topk_idx=None,
                 slots_i32=False):
        name = "fused_attn_topk"
        mode_id = MODE_IDS[mode] if isinstance(mode, str) else int(mode)
        k_bits, v_bits, gs = MODE_BITS[mode_id]
        _require(parts in _PARTS and stage_b in _STAGE_B, f"{name}: bad parts / stage_b")
        need_k, need_v = parts != "v", parts != "k"
        ng = 128 // gs
        dev = block_table.device
        _require(block_table.is_cuda and seq_lens.is_cuda, f"{name}: block_table / seq_lens must be CUDA")
        B = int(seq_lens.shape[0])
        num_slots = None
        if need_k:
            for t, nm in ((q, "q"), (k_data, "k_data"), (k_scales, "k_scales")):
                _require(t is not None and t.is_cuda, f"{name}: {nm} must be CUDA")
            _require(q.dim() == 3 and q.shape[0] == B and q.shape[1] == H_q and q.shape[2] == 128,
                     f"{name}: q must be (B, H_q, 128)")
            q = q.contiguous()
            _require(k_data.dtype == torch.uint8 and k_scales.dtype == torch.bfloat16,
                     f"{name}: packed data must be uint8, scales bf16")
            _require(k_data.is_contiguous() and k_scales.is_contiguous(), f"{name}: cache tensors must be contiguous")
            _require(k_data.dim() == 3 and k_data.shape[0] == H_kv and k_data.shape[2] == _packed_dim(k_bits),
                     f"{name}: k_data must be (H_kv, num_slots, {_packed_dim(k_bits)})")
            num_slots = k_data.shape[1]
            _require(k_scales.numel() == H_kv * num_slots * ng, f"{name}: scales must hold {ng} group(s) per slot")
        if need_v:
            for t, nm in ((v_data, "v_data"), (v_scales, "v_scales")):
                _require(t is not None and t.is_cuda, f"{name}: {nm} must be CUDA")
            _require(v_data.dtype == torch.uint8 and v_scales.dtype == torch.bfloat16,
                     f"{name}: packed data must be uint8, scales bf16")
            _require(v_data.is_contiguous() and v_scales.is_contiguous(), f"{name}: cache tensors must be contiguous")
            _require(v_data.dim() == 3 and v_data.shape[0] == H_kv and v_data.shape[2] == _packed_dim(v_bits),
                     f"{name}: v_data must be (H_kv, num_slots, {_packed_dim(v_bits)})")
            _require(num_slots is None or num_slots == v_data.shape[1], f"{name}: K and V caches differ in num_slots")
            num_slots = v_data.shape[1]
            _require(v_scales.numel() == H_kv * num_slots * ng, f"{name}: scales must hold {ng} group(s) per slot")
        _require(block_table.dtype == torch.int64 and block_table.dim() == 2 and block_table.shape[0] == B,
                 f"{name}: block_table must be (B, max_blocks) int64")
        _require(seq_lens.dtype == torch.int32 and seq_lens.shape == (B,), f"{name}: seq_lens must be (B,) int32")
        block_table = block_table.contiguous()
        seq_lens = seq_lens.contiguous()
        nbytes = decode_workspace_bytes(mode_id, B, H_q, H_kv, max_S, top_k)
        _require(nbytes > 0, f"{name}: bad shape")
        if workspace is None:
            workspace = get_workspace(nbytes, dev)
        ws_ptr = (workspace.data_ptr() + 255) // 256 * 256
        ws_bytes = workspace.numel() - (ws_ptr - workspace.data_ptr())
        f32 = dict(dtype=torch.float32, device=dev)
        if out is None:
            out = dict(
                o_hat=torch.empty(B, H_q, 128, **f32), o_old_unnorm=torch.empty(B, H_q, 128, **f32),
                W=torch.empty(B, H_q, **f32), softmax_m=torch.empty(B, H_q, **f32),
                softmax_inv_z=torch.empty(B, H_q, **f32),
                topk_slots=torch.empty(B, H_q, top_k, dtype=torch.int64, device=dev),
            )
            out["topk_idx"] = topk_idx if topk_idx is not None else \
                torch.empty(B, H_q, top_k, dtype=torch.int64, device=dev)
        if scores is not None:
            _require(scores.is_cuda and scores.dtype == torch.float32 and scores.is_contiguous()
                     and tuple(scores.shape) == (B, H_q, max_S), f"{name}: scores must be contiguous f32 (B, H_q, max_S)")
        elif want_scores:
            scores = torch.empty(B, H_q, max_S, **f32)
        _require(need_k or scores is not None, f"{name}: parts='v' needs the scores")
        _require(out["topk_idx"].is_cuda and out["topk_idx"].dtype == torch.int64 and out["topk_idx"].is_contiguous()
                 and tuple(out["topk_idx"].shape) == (B, H_q, top_k), f"{name}: topk_idx must be contiguous int64 (B, H_q, k)")
        if slots_i32 and "topk_slots_i32" not in out:
            out["topk_slots_i32"] = torch.empty(B, H_q, top_k, dtype=torch.int32, device=dev)
        s32 = out.get("topk_slots_i32")
        if s32 is not None:
            _require(s32.is_cuda and s32.dtype == torch.int32 and s32.is_contiguous()
                     and tuple(s32.shape) == (B, H_q, top_k), f"{name}: topk_slots_i32 must be contiguous int32 (B, H_q, k)")
        self.out = out
        self.scores = scores
        self._keep = (q, k_data, k_scales, v_data, v_scales, block_table, seq_lens, workspace)
        ptr = lambda t: t.data_ptr() if t is not None else None
        a = DecodeArgs()
        a.mode, a.q_dtype = mode_id, (_dtype_id(q) if need_k else _lib.JF_DTYPE_BF16)
        a.B, a.H_q, a.H_kv = B, H_q, H_kv
        a.max_S, a.block_size, a.top_k = int(max_S), int(block_size), int(top_k)
        a.max_blocks = block_table.shape[1]
        a.scan_parts, a.stage_b = _PARTS[parts], _STAGE_B[stage_b]
        a.attn_scale = float(attn_scale)
        a.num_slots = num_slots
        a.q, a.k_data, a.k_scales = (ptr(q), ptr(k_data), ptr(k_scales)) if need_k else (None, None, None)
        a.v_data, a.v_scales = (ptr(v_data), ptr(v_scales)) if need_v else (None, None)
        a.block_table, a.seq_lens = block_table.data_ptr(), seq_lens.data_ptr()
        a.scores = ptr(scores)
        a.topk_idx, a.topk_slots = out["topk_idx"].data_ptr(), out["topk_slots"].data_ptr()
        a.o_hat, a.o_old_unnorm, a.W = out["o_hat"].data_ptr(), out["o_old_unnorm"].data_ptr(), out["W"].data_ptr()
        a.softmax_m, a.softmax_inv_z = out["softmax_m"].data_ptr(), out["softmax_inv_z"].data_ptr()
        a.workspace, a.workspace_bytes = ws_ptr, ws_bytes
        a.topk_slots_i32 = ptr(s32)
        self.args = a
        self._ref = C.byref(a)

    def scan(self):
        check("jf_decode_scan", lib.jf_decode_scan(self._ref, _stream()))

    def select(self):
        check("jf_topk_select", lib.jf_topk_select(self._ref, _stream()))

    def finish(self):
        check("jf_decode_finish", lib.jf_decode_finish(self._ref, _stream()))

    def fused(self):
        check("jf_decode_fused", lib.jf_decode_fused(self._ref, _stream()))

    def select_finish(self):
        """Select and finish in one kernel, after ``scan()`` (together: ``fused()``)."""
        check("jf_select_finish", lib.jf_select_finish(self._ref, _stream()))

    def exact_stats(self):
        """Exact row maximum and 1 / sum exp(s - max) of the stored scores into ``softmax_m`` /
        ``softmax_inv_z`` (what the reference's ``*_topk_stats`` ops return)."""
        a = self.args
        check("jf_softmax_stats", lib.jf_softmax_stats(a.scores, a.seq_lens, a.softmax_m, a.softmax_inv_z,
                                                       a.B, a.H_q, a.max_S, _stream()))

    def status(self):
        """Synchronises the stream and raises if a kernel recorded a bounded-wait timeout."""
        check("jf_decode_status", lib.jf_decode_status(self._ref, _stream()))

    def status_record(self) -> torch.Tensor:
        """The status record's bytes in the workspace (a CUDA uint8 view): copy them to pinned host
        memory in the stream and read the copy with ``decode_status_of_copy`` -- the check without
        a synchronisation."""
        ws = self._keep[-1]
        off = self.args.workspace - ws.data_ptr()
        return ws.view(torch.uint8).reshape(-1)[off:off + STATUS_RECORD_BYTES]

    def result(self) -> FusedAttnOut:
        o = self.out
        return FusedAttnOut(o["o_hat"], o["topk_slots"], o["o_old_unnorm"], o["W"], o["topk_idx"],
                            o["softmax_m"], o["softmax_inv_z"], self.scores)


STATUS_RECORD_BYTES = 16


def decode_status_of_copy(record_copy: torch.Tensor) -> None:
    """Raises if the host copy of a workspace's status record (``DecodeCall.status_record()``)
    holds an error."""
    _require(not record_copy.is_cuda and record_copy.is_contiguous()
             and record_copy.numel() * record_copy.element_size() >= STATUS_RECORD_BYTES,
             "decode_status_of_copy: a contiguous CPU tensor of at least 16 bytes is expected")
    check("jf_decode_status", lib.jf_decode_status_of_copy(record_copy.data_ptr()))


def fused_attn_topk(mode, q, k_data, k_scales, v_data, v_scales, block_table, seq_lens,
                    max_S, H_q, H_kv, block_size, top_k, attn_scale, *, workspace=None,
                    want_scores=False, stage_b="fp32") -> FusedAttnOut:
    """One call: approximate attention over the packed cache, exact top-k, and the
    selected set's approximate contribution.  Returns ``(o_hat, topk_slots, o_old_unnorm,
    W, ...)`` -- the first four as the reference's ``int2_fused_attn_topk``."""
    call = DecodeCall(mode, q, k_data, k_scales, v_data, v_scales, block_table, seq_lens,
                      max_S, H_q, H_kv, block_size, top_k, attn_scale, workspace=workspace,
                      want_scores=want_scores, stage_b=stage_b)
    call.fused()
    return call.result()


def int2_fused_attn_topk(q, k_data, k_scales, k_zp, v_data, v_scales, block_table, seq_lens,
                         max_S, H_q, H_kv, block_size, top_k, attn_scale):
    """The reference's single-call op under its own name and argument order
    (``kernels/int2_fused_attn_topk.py:5-10``, ``csrc/int2_fused_attn_topk.cu:404``):
    ``(o_hat, topk_slots, o_old_unnorm, W)``.  The mode follows the packed row widths
    (K 48 B / V 32 B: K3V2; 64 B / 64 B: K4V4); ``k_zp`` (asymmetric INT2 keys) must be None."""
    _require(k_zp is None, "int2_fused_attn_topk: asymmetric keys (k_zp) are not supported")
    widths = (int(k_data.shape[-1]), int(v_data.shape[-1]))
    _require(widths in ((48, 32), (64, 64)), f"int2_fused_attn_topk: unsupported packed widths {widths}")
    mode = "k3v2" if widths == (48, 32) else "k4v4"
    r = fused_attn_topk(mode, q, k_data, k_scales, v_data, v_scales, block_table, seq_lens,
                        max_S, H_q, H_kv, block_size, top_k, attn_scale)
    return r.o_hat, r.topk_slots, r.o_old_unnorm, r.W


# -- the reference's Stage A / Stage B ops under their own names, argument order and return lists,
#    so that its decode path (jetfire_vllm/adapter/decode_path.py:2081-2131, 2785-2935) can call this
#    library unchanged.  Stage A = the scan's K half + the exact select; Stage B = the scan's V half
#    over the given scores + the finish stage.  Both halves give the bits of the one-pass scan. --

def _stage_a(mode, name, q, k_data, k_scales, block_table, seq_lens, max_S, H_q, H_kv, block_size,
             attn_scale, top_k, stats):
    _require(int(block_size) == 16, f"{name}: block_size must be 16")
    call = DecodeCall(mode, q, k_data, k_scales, None, None, block_table, seq_lens, int(max_S), int(H_q), int(H_kv),
                      int(block_size), int(top_k), float(attn_scale), want_scores=True, parts="k")
    call.scan()
    call.select()
    out = [call.scores, call.out["topk_idx"], call.out["topk_slots"]]
    if stats:
        call.exact_stats()
        out += [call.out["softmax_m"], call.out["softmax_inv_z"]]
    return out


def int3_qk_scores_topk(q, k_data, k_scales, block_table, seq_lens, max_S, H_q, H_kv, block_size, attn_scale, top_k):
    """``[scores f32 (B,H_q,max_S), topk_idx i64 (B,H_q,k), topk_slots i64 (B,H_q,k)]``
    (jetfire_vllm/csrc/int3_qk_scores.cu:562-633).  Unlike the reference, the lists are ordered
    (score descending, position ascending) and ties go to the lower position."""
    return _stage_a("k3v2", "int3_qk_scores_topk", q, k_data, k_scales, block_table, seq_lens, max_S, H_q, H_kv,
                    block_size, attn_scale, top_k, False)


def int8tc_qk_scores_topk_stats(q, k_data, k_scales, block_table, seq_lens, max_S, H_q, H_kv, block_size,
                                attn_scale, top_k):
    """``[scores, topk_idx, topk_slots, softmax_m f32 (B,H_q), softmax_inv_z f32 (B,H_q)]``
    (jetfire_vllm/csrc/int8tc_qk_scores.cu:2426-2482)."""
    return _stage_a("k4v4", "int8tc_qk_scores_topk_stats", q, k_data, k_scales, block_table, seq_lens, max_S, H_q,
                    H_kv, block_size, attn_scale, top_k, True)


def _stage_b(mode, name, stage_b, scores, v_data, v_scales, block_table, seq_lens, topk_idx, max_S, H_q, H_kv,
             block_size, top_k, out=None):
    _require(int(block_size) == 16, f"{name}: block_size must be 16")
    _require(scores.is_cuda and scores.dtype == torch.float32 and scores.dim() == 3, f"{name}: scores must be f32 (B,H_q,max_S)")
    _require(topk_idx.is_cuda and topk_idx.dtype == torch.int64 and topk_idx.dim() == 3
             and topk_idx.shape[2] == int(top_k), f"{name}: topk_idx must be int64 (B,H_q,top_k)")
    B = scores.shape[0]
    if out is not None:
        for t, shape in zip(out, ((B, int(H_q), 128), (B, int(H_q), 128), (B, int(H_q)))):
            _require(t.is_cuda and t.dtype == torch.float32 and t.is_contiguous() and tuple(t.shape) == shape,
                     f"{name}: outputs must be contiguous f32 of shapes (B,H_q,128), (B,H_q,128), (B,H_q)")
        f32 = dict(dtype=torch.float32, device=scores.device)
        out = dict(o_hat=out[0], o_old_unnorm=out[1], W=out[2], softmax_m=torch.empty(B, int(H_q), **f32),
                   softmax_inv_z=torch.empty(B, int(H_q), **f32), topk_idx=topk_idx.contiguous(),
                   topk_slots=torch.empty_like(topk_idx))
    call = DecodeCall(mode, None, None, None, v_data, v_scales, block_table, seq_lens, int(max_S), int(H_q), int(H_kv),
                      int(block_size), int(top_k), 1.0, parts="v", stage_b=stage_b, scores=scores.contiguous(),
                      topk_idx=topk_idx.contiguous(), out=out)
    call.scan()
    call.finish()
    return [call.out["o_hat"], call.out["o_old_unnorm"], call.out["W"]]


def int2_softmax_v_with_pre_corr_wvs2(scores, v_data, v_scales, block_table, seq_lens, topk_idx, max_S, H_q, H_kv,
                                      block_size, top_k):
    """``[o_hat f32 (B,H_q,128), o_old_unnorm f32 (B,H_q,128), W f32 (B,H_q)]``
    (jetfire_vllm/csrc/int2_softmax_v.cu:792-901)."""
    return _stage_b("k3v2", "int2_softmax_v_with_pre_corr_wvs2", "fp32", scores, v_data, v_scales, block_table,
                    seq_lens, topk_idx, max_S, H_q, H_kv, block_size, top_k)


def int2_softmax_v_with_pre_corr_wvs2_inplace(scores, v_data, v_scales, block_table, seq_lens, topk_idx, weights,
                                              o_hat, o_old_unnorm, W_out, max_S, H_q, H_kv, block_size, top_k) -> None:
    """Caller-owned outputs (jetfire_vllm/csrc/int2_softmax_v.cu:903-1025).  ``weights`` (the
    reference's materialised softmax) is not needed and left untouched; the outputs are
    overwritten, so they need not be zeroed."""
    _stage_b("k3v2", "int2_softmax_v_with_pre_corr_wvs2_inplace", "fp32", scores, v_data, v_scales, block_table,
             seq_lens, topk_idx, max_S, H_q, H_kv, block_size, top_k, out=(o_hat, o_old_unnorm, W_out))


def int4_softmax_v_with_pre_corr_wvs2_scores(scores, v_data, v_scales, block_table, seq_lens, topk_idx, max_S, H_q,
                                             H_kv, block_size, top_k):
    """K4V4 Stage B with full-precision weights (jetfire_vllm/csrc/int4_softmax_v.cu:2203-2235)."""
    return _stage_b("k4v4", "int4_softmax_v_with_pre_corr_wvs2_scores", "fp32", scores, v_data, v_scales, block_table,
                    seq_lens, topk_idx, max_S, H_q, H_kv, block_size, top_k)


def int8tc_softmax_v_with_pre_corr_reg_stats(scores, softmax_m, softmax_inv_z, v_data, v_scales, block_table, seq_lens,
                                             topk_idx, max_S, H_q, H_kv, block_size, top_k):
    """K4V4 Stage B of the batch > 1 plan, weights rounded per 32-token tile
    (jetfire_vllm/csrc/int8tc_softmax_v_fused.cu:1591-1604).  ``softmax_m / softmax_inv_z`` are
    accepted for the signature; the normaliser is recomputed from ``scores`` (the same value)."""
    return _stage_b("k4v4", "int8tc_softmax_v_with_pre_corr_reg_stats", "int8p", scores, v_data, v_scales,
                    block_table, seq_lens, topk_idx, max_S, H_q, H_kv, block_size, top_k)


# ---------------------------------------------------------------------------------------
# correction merge
# ---------------------------------------------------------------------------------------

def blend_unnorm_into(o_hat, o_old_unnorm, W, o_new, out) -> None:
    """``out = dtype(o_hat + W * o_new - o_old_unnorm)``; ``out`` contiguous bf16/fp16."""
    name = "blend_unnorm_into"
    _require(o_hat.is_cuda and o_old_unnorm.is_cuda and W.is_cuda and o_new.is_cuda and out.is_cuda,
             f"{name}: all tensors must be CUDA")
    _require(o_hat.dtype == torch.float32 and o_old_unnorm.dtype == torch.float32 and W.dtype == torch.float32,
             f"{name}: o_hat, o_old_unnorm, W must be float32")
    _require(o_new.dtype == out.dtype, f"{name}: o_new and out dtypes differ")
    _require(o_hat.dim() == 3 and o_old_unnorm.dim() == 3 and o_new.dim() == 3 and out.dim() == 3 and W.dim() == 2,
             f"{name}: tensors must be 3D (W 2D)")
    _require(out.is_contiguous(), f"{name}: out must be contiguous")
    _require(o_old_unnorm.shape == o_hat.shape and o_new.shape == o_hat.shape and out.shape == o_hat.shape
             and W.shape == o_hat.shape[:2] and o_hat.shape[2] == 128, f"{name}: shape mismatch")
    o_hat, o_old_unnorm, W, o_new = o_hat.contiguous(), o_old_unnorm.contiguous(), W.contiguous(), o_new.contiguous()
    st = lib.jf_merge_correct(o_hat.data_ptr(), o_old_unnorm.data_ptr(), W.data_ptr(), o_new.data_ptr(),
                              out.data_ptr(), _dtype_id(out), o_hat.shape[0], o_hat.shape[1], _stream())
    check(name, st)


# ---------------------------------------------------------------------------------------
# host correction
# ---------------------------------------------------------------------------------------

def wait_and_blend_unnorm_into(done_flag, o_hat, o_old_unnorm, W, o_new, out, timeout_s: float = 30.0) -> None:
    """Spin on the host correction's completion flag, then launch the merge
    (``csrc/blend.cu:320-376``; ``o_new`` is the device alias of mapped host memory, so no
    copy is needed).  Unlike the reference the wait is bounded: ``RuntimeError`` after
    ``timeout_s``."""
    _require(done_flag.dtype == torch.int64 and done_flag.numel() == 1 and not done_flag.is_cuda,
             "wait_and_blend_unnorm_into: done_flag must be a 1-element int64 CPU tensor")
    # the wait runs in C with the interpreter lock released, so other Python threads keep going
    st = lib.jf_wait_flag(done_flag.data_ptr(), int(float(timeout_s) * 1000.0))
    if st == _lib.JF_ERR_TIMEOUT:
        raise RuntimeError("wait_and_blend_unnorm_into: the host correction did not finish in time")
    check("wait_and_blend_unnorm_into", st)
    blend_unnorm_into(o_hat, o_old_unnorm, W, o_new, out)


def set_cpu_attn_threads(n: int) -> None:
    check("set_cpu_attn_threads", lib.jf_set_cpu_attn_threads(int(n)))


def get_cpu_attn_threads() -> int:
    return int(lib.jf_get_cpu_attn_threads())


def _host_args(q, k_shadow, v_shadow, head_map, ts_buf, o_new, scale, done_flag, name):
    for t, nm in ((q, "q"), (k_shadow, "k_shadow"), (v_shadow, "v_shadow"), (ts_buf, "ts_buf"), (o_new, "o_new")):
        _require(not t.is_cuda, f"{name}: {nm} must be a CPU tensor")
        _require(t.is_contiguous(), f"{name}: {nm} must be contiguous")
    _require(q.dtype == k_shadow.dtype == v_shadow.dtype == o_new.dtype, f"{name}: dtype mismatch")
    _require(q.dim() == 3 and k_shadow.dim() == 3 and v_shadow.dim() == 3 and ts_buf.dim() == 3 and o_new.dim() == 3,
             f"{name}: tensors must be 3D")
    B, H_q, D = q.shape
    H_kv, num_slots = k_shadow.shape[0], k_shadow.shape[1]
    _require(D == 128 and k_shadow.shape[2] == 128, f"{name} currently only supports D=128")
    _require(v_shadow.shape == k_shadow.shape, f"{name}: k/v mirror shape mismatch")
    _require(ts_buf.dtype in (torch.int64, torch.int32) and ts_buf.shape[:2] == (B, H_q),
             f"{name}: ts_buf must be (B,H_q,K) int64 (or int32: the 32-bit slot list of DecodeCall(slots_i32=True))")
    _require(o_new.shape == q.shape, f"{name}: o_new shape mismatch")
    hm_ptr = None
    if head_map is not None:
        _require(head_map.dtype == torch.int64 and head_map.shape == ts_buf.shape and head_map.is_contiguous()
                 and not head_map.is_cuda, f"{name}: head_map must match ts_buf (int64, CPU, contiguous)")
        hm_ptr = head_map.data_ptr()
    flag_ptr = None
    if done_flag is not None:
        _require(done_flag.dtype == torch.int64 and done_flag.numel() == 1 and not done_flag.is_cuda,
                 f"{name}: done_flag must be a 1-element int64 CPU tensor")
        flag_ptr = done_flag.data_ptr()
    return (q.data_ptr(), k_shadow.data_ptr(), v_shadow.data_ptr(), hm_ptr, ts_buf.data_ptr(), o_new.data_ptr(),
            _dtype_id(q), B, H_q, H_kv, num_slots, ts_buf.shape[2], float(scale), flag_ptr)


def _i32(ts_buf) -> bool:
    return ts_buf.dtype == torch.int32


def cpu_topk_attn(q, k_shadow, v_shadow, head_map, ts_buf, o_new, scale, done_flag=None) -> None:
    """Exact attention over the selected mirror rows, blocking.  ``ts_buf`` int64 as in the
    reference, or int32."""
    args = _host_args(q, k_shadow, v_shadow, head_map, ts_buf, o_new, scale, done_flag, "cpu_topk_attn")
    check("cpu_topk_attn", (lib.jf_cpu_topk_attn_i32 if _i32(ts_buf) else lib.jf_cpu_topk_attn)(*args))


def cpu_topk_attn_submit(q, k_shadow, v_shadow, head_map, ts_buf, o_new, scale, done_flag=None) -> None:
    args = _host_args(q, k_shadow, v_shadow, head_map, ts_buf, o_new, scale, done_flag, "cpu_topk_attn_submit")
    if _i32(ts_buf):
        t = C.c_int64(0)
        check("cpu_topk_attn_submit", lib.jf_pool_submit_ticket_i32(*args, C.byref(t)))
    else:
        check("cpu_topk_attn_submit", lib.jf_pool_submit(*args))


def cpu_topk_attn_wait(timeout_ms: int = 30000) -> None:
    check("cpu_topk_attn_wait", lib.jf_pool_wait_timeout(int(timeout_ms)))


class HostCorrectionCall:
    """A host correction over fixed buffers (the per-layer state of the reference's decode
    path, ``adapter/decode_path.py:2448-2492``): the tensors are validated and their addresses
    taken once, ``submit()`` / ``wait()`` / ``run()`` then cost one C call each.  The caller keeps
    the buffers' contents current; the tensors themselves are kept alive here."""

    def __init__(self, q, k_shadow, v_shadow, head_map, ts_buf, o_new, scale, done_flag=None, rows=None):
        self._args = _host_args(q, k_shadow, v_shadow, head_map, ts_buf, o_new, scale, done_flag,
                                "HostCorrectionCall")
        self._keep = (q, k_shadow, v_shadow, head_map, ts_buf, o_new, done_flag)
        i32 = _i32(ts_buf)   # 32-bit slot list: the entry points of the same names with the _i32 suffix
        # rows=(begin, end): only that range of the B * H_q (sequence, query head) rows, the rest being
        # someone else's (gpu_topk_attn_rows)
        self._rows = None
        if rows is not None:
            r0, r1 = int(rows[0]), int(rows[1])
            _require(0 <= r0 < r1 <= q.shape[0] * q.shape[1], "HostCorrectionCall: rows must be a non-empty range of the B * H_q rows")
            a = self._args
            self._rows = (*a[:5], 1 if i32 else 0, *a[5:], r0, r1)
        self._fn_submit = lib.jf_pool_submit_ticket_i32 if i32 else lib.jf_pool_submit_ticket
        self._fn_run = lib.jf_cpu_topk_attn_i32 if i32 else lib.jf_cpu_topk_attn
        self._fn_ctx = lib.jf_submit_ctx_create_i32 if i32 else lib.jf_submit_ctx_create

    def submit(self) -> int:
        """Queue the job (up to four can wait in the pool); returns its ticket for ``wait_ticket``."""
        t = C.c_int64(0)
        if self._rows is not None:
            check("cpu_topk_attn_submit", lib.jf_pool_submit_rows(*self._rows, C.byref(t)))
        else:
            check("cpu_topk_attn_submit", self._fn_submit(*self._args, C.byref(t)))
        return t.value

    @staticmethod
    def wait_ticket(ticket: int, timeout_ms: int = 30000) -> None:
        check("cpu_topk_attn_wait", lib.jf_pool_wait_ticket(int(ticket), int(timeout_ms)))

    @staticmethod
    def wait(timeout_ms: int = 30000) -> None:
        check("cpu_topk_attn_wait", lib.jf_pool_wait_timeout(int(timeout_ms)))

    def run(self) -> None:
        if self._rows is not None:
            self.wait_ticket(self.submit())
        else:
            check("cpu_topk_attn", self._fn_run(*self._args))

    # -- stream-ordered form (the reference's create_cpu_topk_submit_ctx /
    #    stream_submit_cpu_topk_attn / stream_wait_cpu_topk_attn, csrc/cpu_topk_attn.cpp:2147-2312) --
    def _handle(self) -> int:
        if getattr(self, "_ctx", None) is None:
            h = C.c_int64(0)
            check("create_cpu_topk_submit_ctx", self._fn_ctx(*self._args, 0, C.byref(h)))
            self._ctx = h.value
            if self._rows is not None:
                check("submit_ctx_set_rows", lib.jf_submit_ctx_set_rows(self._ctx, self._rows[-2], self._rows[-1]))
        return self._ctx

    def stream_submit(self, stream=None) -> None:
        """Queue the submit on ``stream`` (default: current): the job starts when the stream gets
        there.  ``ts_buf`` and ``q`` must be in host memory by then (stream-ordered copies)."""
        s = stream.cuda_stream if stream is not None else _stream()
        check("stream_submit_cpu_topk_attn", lib.jf_stream_submit_cpu_topk_attn(s, self._handle()))

    def stream_wait(self, stream=None) -> None:
        """Queue a host wait on ``stream``: work queued after it runs once the job is done."""
        s = stream.cuda_stream if stream is not None else _stream()
        check("stream_wait_cpu_topk_attn", lib.jf_stream_wait_cpu_topk_attn(s, self._handle()))

    def watch(self, trigger_host: torch.Tensor) -> None:
        """Let the GPU start this job: from now on a non-zero value stored to ``trigger_host`` (one
        int64 in mapped pinned host memory, see ``stream_signal_host``) queues it; the job's
        ``done_flag`` is set when it is complete."""
        _require(not trigger_host.is_cuda and trigger_host.dtype == torch.int64 and trigger_host.numel() == 1,
                 "watch: trigger_host must be a 1-element int64 CPU tensor")
        check("submit_ctx_watch", lib.jf_submit_ctx_watch(self._handle(), trigger_host.data_ptr()))
        self._keep = self._keep + (trigger_host,)

    def stream_status(self) -> None:
        """Raises if a queued submit or wait ran out of time (call after synchronising)."""
        if getattr(self, "_ctx", None) is not None:
            check("cpu_topk_submit_ctx", lib.jf_submit_ctx_status(self._ctx))

    def close(self) -> None:
        """Free the native context; no stream operation or graph may refer to it any more."""
        if getattr(self, "_ctx", None) is not None:
            lib.jf_submit_ctx_destroy(self._ctx)
            self._ctx = None


# -- the reference's stream-ordered host ops under their own names (bindings at
#    jetfire_vllm/csrc/cpu_topk_attn.cpp:2509-2663).  Handles are plain integers; the contexts and
#    the tensors they point into live until the process ends, as in the reference (:1433-1435). --

_CTX_KEEP: list = []


def create_cpu_topk_submit_ctx(q, k_shadow, v_shadow, head_map, ts_buf, o_new, scale, flag_host) -> int:
    """Context over pre-allocated decode buffers (all CPU; ``flag_host`` a 1-element int64 tensor,
    set to 1 when a submitted job is done).  Returns the handle for ``stream_submit_cpu_topk_attn``."""
    args = _host_args(q, k_shadow, v_shadow, head_map, ts_buf, o_new, scale, flag_host, "create_cpu_topk_submit_ctx")
    h = C.c_int64(0)
    check("create_cpu_topk_submit_ctx",
          (lib.jf_submit_ctx_create_i32 if _i32(ts_buf) else lib.jf_submit_ctx_create)(*args, 0, C.byref(h)))
    _CTX_KEEP.append((q, k_shadow, v_shadow, head_map, ts_buf, o_new, flag_host))
    return h.value


def stream_submit_cpu_topk_attn(stream_id: int, ctx_handle: int) -> None:
    """Queue a host callback on the stream (a raw ``cudaStream_t`` as an integer) that hands the
    context's job to the worker pool when the stream gets there.  Capturable in a CUDA graph."""
    check("stream_submit_cpu_topk_attn", lib.jf_stream_submit_cpu_topk_attn(int(stream_id), int(ctx_handle)))


def stream_wait_cpu_topk_attn(stream_id: int, ctx_handle: int) -> None:
    """Queue a host callback that holds the stream until the context's job is done (bounded:
    30 s, then the timeout is reported by the context's status)."""
    check("stream_wait_cpu_topk_attn", lib.jf_stream_wait_cpu_topk_attn(int(stream_id), int(ctx_handle)))


def stream_write_value64(stream_id: int, flag_device: torch.Tensor, value: int) -> None:
    """Stream-ordered 64-bit store to the device half of an ``alloc_mapped_pinned_pair``."""
    _require(flag_device.is_cuda and flag_device.dtype == torch.int64 and flag_device.numel() == 1,
             "stream_write_value64: flag_device must be a 1-element int64 CUDA tensor")
    check("stream_write_value64", lib.jf_stream_write_value64(int(stream_id), flag_device.data_ptr(), int(value)))


def gpu_topk_attn_rows(q, k_mirror_dev, v_mirror_dev, topk_slots, o_new, scale, rows) -> None:
    """The top-k correction of the (sequence, query head) rows ``rows = (begin, end)`` on the GPU,
    reading the selected K / V rows from the host mirror through its device-visible tensors (the
    device halves of ``alloc_mapped_pinned_pair`` / ``map_host_tensor``): takes those rows off the
    host's workers (``HostCorrectionCall(rows=...)`` for the rest).  ``q (B, H_q, 128)`` and
    ``topk_slots (B, H_q, K)`` int64 or int32 are CUDA tensors, ``o_new (B, H_q, 128)`` a CUDA tensor
    whose rows in the range are written.  Agrees with ``cpu_topk_attn`` to rounding."""
    name = "gpu_topk_attn_rows"
    for t, nm in ((q, "q"), (k_mirror_dev, "k_mirror_dev"), (v_mirror_dev, "v_mirror_dev"), (topk_slots, "topk_slots"),
                  (o_new, "o_new")):
        _require(t.is_cuda and t.is_contiguous(), f"{name}: {nm} must be a contiguous CUDA tensor")
    _require(q.dim() == 3 and q.shape[2] == 128 and o_new.shape == q.shape, f"{name}: q / o_new must be (B, H_q, 128)")
    _require(q.dtype == k_mirror_dev.dtype == v_mirror_dev.dtype == o_new.dtype, f"{name}: dtype mismatch")
    _require(k_mirror_dev.dim() == 3 and k_mirror_dev.shape[2] == 128 and v_mirror_dev.shape == k_mirror_dev.shape,
             f"{name}: mirrors must be (H_kv, num_slots, 128)")
    B, H_q = int(q.shape[0]), int(q.shape[1])
    _require(topk_slots.dtype in (torch.int64, torch.int32) and topk_slots.dim() == 3
             and tuple(topk_slots.shape[:2]) == (B, H_q), f"{name}: topk_slots must be (B, H_q, K) int64 or int32")
    r0, r1 = int(rows[0]), int(rows[1])
    _require(0 <= r0 <= r1 <= B * H_q, f"{name}: rows must be a range of the B * H_q rows")
    check(name, lib.jf_gpu_topk_attn_rows(q.data_ptr(), k_mirror_dev.data_ptr(), v_mirror_dev.data_ptr(),
                                          topk_slots.data_ptr(), 1 if topk_slots.dtype == torch.int32 else 0,
                                          o_new.data_ptr(), _dtype_id(q), B, H_q, int(k_mirror_dev.shape[0]),
                                          int(k_mirror_dev.shape[1]), int(topk_slots.shape[2]), float(scale), r0, r1,
                                          _stream()))


def stream_signal_host(done_dev: torch.Tensor, trigger_dev: torch.Tensor) -> None:
    """Queue a kernel that clears ``done_dev`` and then sets ``trigger_dev`` to 1 (device halves of
    two int64 words from ``alloc_mapped_pinned_pair``): starts the host correction whose context
    watches the trigger word, once the stream's earlier copies have landed.  Capturable."""
    for t in (done_dev, trigger_dev):
        _require(t.is_cuda and t.dtype == torch.int64 and t.numel() == 1, "stream_signal_host: 1-element int64 CUDA views")
    check("stream_signal_host", lib.jf_stream_signal_host(_stream(), done_dev.data_ptr(), trigger_dev.data_ptr()))


def stream_wait_host_flag(flag_dev: torch.Tensor, timeout_ms: int = 2000, status_record: torch.Tensor | None = None) -> None:
    """Queue a kernel that holds the stream until ``flag_dev`` (device half of a mapped int64 word)
    is non-zero, for at most ``timeout_ms``; a wait that runs out is written to ``status_record``
    (``DecodeCall.status_record()``) and the stream continues.  Capturable."""
    _require(flag_dev.is_cuda and flag_dev.dtype == torch.int64 and flag_dev.numel() == 1,
             "stream_wait_host_flag: flag_dev must be a 1-element int64 CUDA view")
    rec = status_record.data_ptr() if status_record is not None else None
    check("stream_wait_host_flag", lib.jf_stream_wait_host_flag(_stream(), flag_dev.data_ptr(), int(timeout_ms), rec))


def submit_cpu_topk_attn_async(q, k_shadow, v_shadow, head_map, ts_buf, o_new, scale, flag) -> None:
    """Returns at once; the last worker stores 1 to ``flag`` when ``o_new`` is complete."""
    cpu_topk_attn_submit(q, k_shadow, v_shadow, head_map, ts_buf, o_new, scale, flag)


def wait_for_flag(flag: torch.Tensor, timeout_s: float = 30.0) -> None:
    """Block (interpreter lock released) until ``flag`` reads non-zero; unlike the reference the
    wait is bounded."""
    _require(flag.dtype == torch.int64 and flag.numel() == 1 and not flag.is_cuda,
             "wait_for_flag: flag must be a 1-element int64 CPU tensor")
    check("wait_for_flag", lib.jf_wait_flag(flag.data_ptr(), int(float(timeout_s) * 1000.0)))


def create_shadow_append_submit_ctx(k_append, v_append, slots, k_shadow, v_shadow) -> int:
    """Context for appending decode tokens to the host mirror in stream order: ``k_append /
    v_append (T, H_kv, 128)`` and ``slots (T,) int64`` are pinned CPU staging tensors that the
    caller's stream-ordered copies fill; ``stream_submit_shadow_append`` scatters them."""
    name = "create_shadow_append_submit_ctx"
    for t, nm in ((k_append, "k_append"), (v_append, "v_append"), (slots, "slots"), (k_shadow, "k_shadow"),
                  (v_shadow, "v_shadow")):
        _require(not t.is_cuda and t.is_contiguous(), f"{name}: {nm} must be a contiguous CPU tensor")
    _require(k_append.dim() == 3 and v_append.shape == k_append.shape and k_append.shape[2] == 128
             and k_append.dtype in (torch.bfloat16, torch.float16) and v_append.dtype == k_append.dtype,
             f"{name}: k_append / v_append must be (T, H_kv, 128) 16-bit and match")
    _require(slots.dim() == 1 and slots.dtype == torch.int64 and slots.shape[0] == k_append.shape[0],
             f"{name}: slots must be (T,) int64")
    _require(k_shadow.dim() == 3 and v_shadow.shape == k_shadow.shape and k_shadow.shape[0] == k_append.shape[1]
             and k_shadow.shape[2] == 128 and k_shadow.dtype == k_append.dtype and v_shadow.dtype == k_append.dtype,
             f"{name}: mirrors must be (H_kv, num_slots, 128) of the staging dtype")
    h = C.c_int64(0)
    check(name, lib.jf_shadow_append_ctx_create(k_append.data_ptr(), v_append.data_ptr(), slots.data_ptr(),
                                                k_append.shape[0], k_append.shape[1], k_shadow.data_ptr(),
                                                v_shadow.data_ptr(), k_shadow.shape[1], C.byref(h)))
    _CTX_KEEP.append((k_append, v_append, slots, k_shadow, v_shadow))
    return h.value


def stream_submit_shadow_append(stream_id: int, ctx_handle: int) -> None:
    check("stream_submit_shadow_append", lib.jf_stream_submit_shadow_append(int(stream_id), int(ctx_handle)))


def get_shadow_append_count(ctx_handle: int) -> int:
    n = C.c_int64(0)
    check("get_shadow_append_count", lib.jf_shadow_append_ctx_calls(int(ctx_handle), C.byref(n)))
    return n.value


def advise_huge_pages(host: torch.Tensor) -> bool:
    """Ask the operating system to back a CPU tensor's memory with 2 MB pages (best right after
    ``torch.empty``, before the first write).  For host mirrors in ordinary memory: the correction's
    random row gathers then miss the TLB far less.  Returns False if the system refuses."""
    _require(not host.is_cuda, "advise_huge_pages: a CPU tensor is expected")
    return lib.jf_advise_huge_pages(host.data_ptr(), host.numel() * host.element_size()) == _lib.JF_OK


def numa_node_count() -> int:
    """Memory nodes of this host (1 when the system does not say)."""
    return int(lib.jf_numa_node_count())


def numa_node_of_device(device: int = 0) -> int:
    """Memory node the GPU is attached to, -1 when unknown."""
    return int(lib.jf_numa_node_of_device(int(device)))


def numa_node_cpus(node: int) -> list[int]:
    """Processors of a memory node, ascending; RuntimeError for a node the system does not list."""
    count = C.c_int32(0)
    check("numa_node_cpus", lib.jf_numa_node_cpus(int(node), None, 0, C.byref(count)))
    buf = (C.c_int32 * max(count.value, 1))()
    check("numa_node_cpus", lib.jf_numa_node_cpus(int(node), buf, count.value, C.byref(count)))
    return [int(buf[i]) for i in range(count.value)]


def bind_memory_to_node(host: torch.Tensor, node: int) -> bool:
    """Bind a CPU tensor's pages to a memory node (right after ``torch.empty``, before the first
    write and before any pinning).  Returns False if the system refuses."""
    _require(not host.is_cuda, "bind_memory_to_node: a CPU tensor is expected")
    return lib.jf_bind_memory_to_node(host.data_ptr(), host.numel() * host.element_size(), int(node)) == _lib.JF_OK


def set_cpu_attn_node(node: int) -> None:
    """Confine the correction workers to one memory node's processors (-1: anywhere); takes effect
    with the next job."""
    check("set_cpu_attn_node", lib.jf_set_cpu_attn_node(int(node)))


def get_cpu_attn_node() -> int:
    return int(lib.jf_get_cpu_attn_node())


def alloc_mapped_pinned_pair(shape, dtype, node: int = -1):
    """``(host_tensor, device_tensor)`` over the same pinned, GPU-mapped bytes; ``node >= 0`` asks
    for the bytes on that memory node."""
    n = 1
    for s in shape:
        n *= int(s)
    itemsize = torch.empty(0, dtype=dtype).element_size()
    nbytes = max(n * itemsize, 1)
    h, d = C.c_void_p(), C.c_void_p()
    check("alloc_mapped_pinned_pair", lib.jf_alloc_mapped_on_node(nbytes, int(node), C.byref(h), C.byref(d)))
    buf = (C.c_uint8 * nbytes).from_address(h.value)
    host = torch.frombuffer(buf, dtype=dtype, count=n).reshape(*shape)
    dev_ptr = d.value

    class _DevView:
        """CUDA array interface over the mapped device alias."""
        __cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (dev_ptr, False), "version": 2, "strides": None}

    device = torch.as_tensor(_DevView(), device="cuda").view(dtype)[:n].reshape(*shape)
    host._jf_mapped = (buf, h.value)  # keep the ctypes view alive with the tensor
    return host, device
