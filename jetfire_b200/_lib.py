"""ctypes binding of ``libjetfire_b200.so`` (the C ABI in ``include/jetfire_b200.h``).

There is no Python or CPU fallback: if the library is missing or fails to load, importing
this module raises, and every op that needs the GPU raises when the call fails.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libjetfire_b200.so"

JF_OK = 0
JF_ERR_ARG, JF_ERR_UNSUPPORTED, JF_ERR_WORKSPACE, JF_ERR_STATIC_LIMIT = -1, -2, -3, -4
JF_ERR_CUDA, JF_ERR_TIMEOUT, JF_ERR_STATE = 1, 2, 3
JF_DTYPE_BF16, JF_DTYPE_FP16 = 0, 1
JF_MODE_K3V2, JF_MODE_K4V4 = 0, 1
JF_SCAN_ALL, JF_SCAN_K_ONLY, JF_SCAN_V_ONLY = 0, 1, 2
JF_STAGE_B_FP32, JF_STAGE_B_INT8P = 0, 1


class JetFireError(RuntimeError):
    """A C-ABI call returned a non-zero status (the reference raises RuntimeError
    from TORCH_CHECK in the same places)."""

    def __init__(self, fn: str, status: int, detail: str):
        super().__init__(f"{fn} failed: status {status} ({detail})")
        self.status = status


class DecodeArgs(C.Structure):
    _fields_ = [
        ("mode", C.c_int32), ("q_dtype", C.c_int32),
        ("B", C.c_int32), ("H_q", C.c_int32), ("H_kv", C.c_int32),
        ("max_S", C.c_int32), ("block_size", C.c_int32), ("top_k", C.c_int32),
        ("max_blocks", C.c_int32), ("scan_parts", C.c_int32),
        ("attn_scale", C.c_float), ("stage_b", C.c_int32),
        ("num_slots", C.c_int64),
        ("q", C.c_void_p), ("k_data", C.c_void_p), ("k_scales", C.c_void_p),
        ("v_data", C.c_void_p), ("v_scales", C.c_void_p),
        ("block_table", C.c_void_p), ("seq_lens", C.c_void_p),
        ("scores", C.c_void_p), ("topk_idx", C.c_void_p), ("topk_slots", C.c_void_p),
        ("o_hat", C.c_void_p), ("o_old_unnorm", C.c_void_p), ("W", C.c_void_p),
        ("softmax_m", C.c_void_p), ("softmax_inv_z", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_uint64),
        ("topk_slots_i32", C.c_void_p),
    ]


_SIGS = {
    "jf_status_string": (C.c_char_p, [C.c_int32]),
    "jf_version": (C.c_int32, []),
    "jf_last_cuda_error": (C.c_int32, []),
    "jf_pack_append": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_int64, C.c_int64,
                                   C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32,
                                   C.c_void_p]),
    "jf_pack_append_kv": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int32,
                                      C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_void_p,
                                      C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                      C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "jf_pack_append_kv_mirror": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int32,
                                             C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_void_p,
                                             C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                             C.c_int64, C.c_int32, C.c_int32, C.c_int32,
                                             C.c_void_p, C.c_void_p, C.c_void_p]),
    "jf_mirror_append_ctx_create": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int64,
                                                C.POINTER(C.c_int64)]),
    "jf_mirror_append_ctx_destroy": (C.c_int32, [C.c_int64]),
    "jf_mirror_append_ctx_stats": (C.c_int32, [C.c_int64, C.POINTER(C.c_int64), C.POINTER(C.c_int64),
                                               C.POINTER(C.c_int64)]),
    "jf_stream_mirror_append": (C.c_int32, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64,
                                            C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "jf_shadow_append_ctx_create": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32,
                                                C.c_void_p, C.c_void_p, C.c_int64, C.POINTER(C.c_int64)]),
    "jf_shadow_append_ctx_destroy": (C.c_int32, [C.c_int64]),
    "jf_shadow_append_ctx_calls": (C.c_int32, [C.c_int64, C.POINTER(C.c_int64)]),
    "jf_stream_submit_shadow_append": (C.c_int32, [C.c_void_p, C.c_int64]),
    "jf_stream_write_value64": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int64]),
    "jf_map_host": (C.c_int32, [C.c_void_p, C.c_uint64, C.POINTER(C.c_void_p)]),
    "jf_unmap_host": (C.c_int32, [C.c_void_p]),
    "jf_decode_workspace_bytes": (C.c_uint64, [C.c_int32] * 6),
    "jf_decode_scan": (C.c_int32, [C.POINTER(DecodeArgs), C.c_void_p]),
    "jf_topk_select": (C.c_int32, [C.POINTER(DecodeArgs), C.c_void_p]),
    "jf_decode_finish": (C.c_int32, [C.POINTER(DecodeArgs), C.c_void_p]),
    "jf_decode_fused": (C.c_int32, [C.POINTER(DecodeArgs), C.c_void_p]),
    "jf_select_finish": (C.c_int32, [C.POINTER(DecodeArgs), C.c_void_p]),
    "jf_decode_status": (C.c_int32, [C.POINTER(DecodeArgs), C.c_void_p]),
    "jf_decode_status_of_copy": (C.c_int32, [C.c_void_p]),
    "jf_softmax_stats": (C.c_int32, [C.c_void_p] * 4 + [C.c_int32] * 3 + [C.c_void_p]),
    "jf_decode_fused_static": (C.c_int32, [C.POINTER(DecodeArgs), C.c_void_p]),
    "jf_merge_correct": (C.c_int32, [C.c_void_p] * 5 + [C.c_int32] * 3 + [C.c_void_p]),
    "jf_cpu_topk_attn": (C.c_int32, [C.c_void_p] * 6 + [C.c_int32] * 4 + [C.c_int64, C.c_int32, C.c_float,
                                                                       C.c_void_p]),
    "jf_cpu_topk_attn_i32": (C.c_int32, [C.c_void_p] * 6 + [C.c_int32] * 4 + [C.c_int64, C.c_int32, C.c_float,
                                                                           C.c_void_p]),
    "jf_advise_huge_pages": (C.c_int32, [C.c_void_p, C.c_uint64]),
    "jf_numa_node_count": (C.c_int32, []),
    "jf_numa_node_of_device": (C.c_int32, [C.c_int32]),
    "jf_numa_node_cpus": (C.c_int32, [C.c_int32, C.POINTER(C.c_int32), C.c_int32, C.POINTER(C.c_int32)]),
    "jf_bind_memory_to_node": (C.c_int32, [C.c_void_p, C.c_uint64, C.c_int32]),
    "jf_alloc_mapped_on_node": (C.c_int32, [C.c_uint64, C.c_int32, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    "jf_set_cpu_attn_node": (C.c_int32, [C.c_int32]),
    "jf_get_cpu_attn_node": (C.c_int32, []),
    "jf_wait_flag": (C.c_int32, [C.c_void_p, C.c_int32]),
    "jf_set_cpu_attn_threads": (C.c_int32, [C.c_int32]),
    "jf_get_cpu_attn_threads": (C.c_int32, []),
    "jf_pool_init": (C.c_int32, [C.c_int32]),
    "jf_pool_submit": (C.c_int32, [C.c_void_p] * 6 + [C.c_int32] * 4 + [C.c_int64, C.c_int32, C.c_float,
                                                                     C.c_void_p]),
    "jf_pool_submit_ticket": (C.c_int32, [C.c_void_p] * 6 + [C.c_int32] * 4 + [C.c_int64, C.c_int32, C.c_float,
                                                                            C.c_void_p, C.POINTER(C.c_int64)]),
    "jf_pool_submit_ticket_i32": (C.c_int32, [C.c_void_p] * 6 + [C.c_int32] * 4 + [C.c_int64, C.c_int32, C.c_float,
                                                                                C.c_void_p, C.POINTER(C.c_int64)]),
    "jf_pool_wait_timeout": (C.c_int32, [C.c_int32]),
    "jf_pool_wait_ticket": (C.c_int32, [C.c_int64, C.c_int32]),
    "jf_submit_ctx_create": (C.c_int32, [C.c_void_p] * 6 + [C.c_int32] * 4 + [C.c_int64, C.c_int32, C.c_float,
                                                                           C.c_void_p, C.c_int32,
                                                                           C.POINTER(C.c_int64)]),
    "jf_submit_ctx_create_i32": (C.c_int32, [C.c_void_p] * 6 + [C.c_int32] * 4 + [C.c_int64, C.c_int32, C.c_float,
                                                                               C.c_void_p, C.c_int32,
                                                                               C.POINTER(C.c_int64)]),
    "jf_submit_ctx_destroy": (C.c_int32, [C.c_int64]),
    "jf_submit_ctx_status": (C.c_int32, [C.c_int64]),
    "jf_stream_submit_cpu_topk_attn": (C.c_int32, [C.c_void_p, C.c_int64]),
    "jf_stream_wait_cpu_topk_attn": (C.c_int32, [C.c_void_p, C.c_int64]),
    "jf_pool_shutdown": (C.c_int32, []),
    "jf_gpu_topk_attn_rows": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32,
                                          C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int32, C.c_float,
                                          C.c_int64, C.c_int64, C.c_void_p]),
    "jf_pool_submit_rows": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p,
                                        C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int32, C.c_float,
                                        C.c_void_p, C.c_int64, C.c_int64, C.POINTER(C.c_int64)]),
    "jf_submit_ctx_watch": (C.c_int32, [C.c_int64, C.c_void_p]),
    "jf_submit_ctx_unwatch": (C.c_int32, [C.c_int64]),
    "jf_submit_ctx_set_rows": (C.c_int32, [C.c_int64, C.c_int64, C.c_int64]),
    "jf_stream_signal_host": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "jf_stream_wait_host_flag": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "jf_alloc_mapped": (C.c_int32, [C.c_uint64, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]),
    "jf_free_mapped": (C.c_int32, [C.c_void_p]),
}

EXPORTED = tuple(_SIGS)


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m jetfire_b200.build` "
            "(there is no fallback path)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in _SIGS.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def status_string(st: int) -> str:
    return lib.jf_status_string(st).decode()


def check(fn: str, st: int) -> None:
    if st != JF_OK:
        detail = status_string(st)
        if st == JF_ERR_CUDA:
            detail += f"; cudaError {lib.jf_last_cuda_error()}"
        raise JetFireError(fn, st, detail)
