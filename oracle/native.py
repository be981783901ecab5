"""Loaders for the oracle's native pieces (test infrastructure only).

``c_decode``: ctypes wrapper of ``oracle/jf_oracle_c.c``.
``ref_cpu_topk_attn_module``: the reference's own ``cpu_topk_attn`` extension built by
``oracle/build_oracle.py`` (None when it was never built, e.g. the reference checkout is
absent and no prebuilt file travelled with the tree).
``ref_gpu_module``: one of the reference's own GPU kernels built for sm_100 by the same script
(None when absent or when it does not load).
"""
from __future__ import annotations

import ctypes as C
import importlib.util
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_C = None
_REF = {}


def _c_lib():
    global _C
    if _C is None:
        from .build_oracle import build_c
        lib = C.CDLL(str(build_c()))
        lib.jf_oracle_decode.restype = C.c_int
        lib.jf_oracle_decode.argtypes = [C.c_int] + [C.c_void_p] * 7 + [C.c_int] * 5 + [C.c_int64, C.c_float,
                                                                                   C.c_int, C.c_int] + [C.c_void_p] * 8
        lib.jf_oracle_decode_stage_b.restype = C.c_int
        lib.jf_oracle_decode_stage_b.argtypes = [C.c_int] + lib.jf_oracle_decode.argtypes
        lib.jf_oracle_num_threads.restype = C.c_int
        _C = lib
    return _C


def c_num_threads() -> int:
    return int(_c_lib().jf_oracle_num_threads())


def c_decode(mode: str, q, k_data, k_scales, v_data, v_scales, block_table, seq_lens, max_s, top_k,
             attn_scale, n_threads: int = 0, want_scores: bool = False, stage_b: str = "fp32"):
    """Run the C restatement.  Arrays as in ``jf_oracle.decode_step`` (scales as bf16 bits);
    ``stage_b="int8p"`` (K4V4 only) selects the reference's batch > 1 Stage-B arithmetic."""
    q = np.ascontiguousarray(q, np.float32)
    k_data, v_data = np.ascontiguousarray(k_data, np.uint8), np.ascontiguousarray(v_data, np.uint8)
    k_scales, v_scales = np.ascontiguousarray(k_scales, np.uint16), np.ascontiguousarray(v_scales, np.uint16)
    block_table = np.ascontiguousarray(block_table, np.int64)
    seq_lens = np.ascontiguousarray(seq_lens, np.int32)
    b_n, h_q, _ = q.shape
    h_kv, num_slots = k_data.shape[0], k_data.shape[1]
    out = dict(topk_idx=np.empty((b_n, h_q, top_k), np.int64), topk_slots=np.empty((b_n, h_q, top_k), np.int64),
               o_hat=np.empty((b_n, h_q, 128), np.float32), o_old_unnorm=np.empty((b_n, h_q, 128), np.float32),
               W=np.empty((b_n, h_q), np.float32), m=np.empty((b_n, h_q), np.float32),
               inv_z=np.empty((b_n, h_q), np.float32))
    scores = np.full((b_n, h_q, max_s), -np.inf, np.float32) if want_scores else None
    p = lambda a: a.ctypes.data_as(C.c_void_p) if a is not None else None
    rc = _c_lib().jf_oracle_decode_stage_b(
        {"k3v2": 0, "k4v4": 1}[mode], {"fp32": 0, "int8p": 1}[stage_b], p(q), p(k_data), p(k_scales), p(v_data), p(v_scales), p(block_table),
        p(seq_lens), b_n, h_q, h_kv, int(max_s), block_table.shape[1], num_slots, float(attn_scale), int(top_k),
        int(n_threads), p(scores), p(out["topk_idx"]), p(out["topk_slots"]), p(out["o_hat"]),
        p(out["o_old_unnorm"]), p(out["W"]), p(out["m"]), p(out["inv_z"]))
    assert rc == 0
    out["scores"] = scores
    return out


def _cpu_flags() -> set[str]:
    try:
        for line in Path("/proc/cpuinfo").read_text().splitlines():
            if line.startswith("flags"):
                return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def ref_isa() -> str | None:
    flags = _cpu_flags()
    if {"avx512f", "avx512bw", "avx512vl", "avx512dq", "avx512_bf16"} <= flags:
        return "avx512bf16"
    if {"avx2", "fma", "f16c"} <= flags:
        return "avx2"
    return None


def ref_cpu_topk_attn_module(isa: str | None = None):
    """The reference extension module (``cpu_topk_attn``, ``set_cpu_attn_threads`` ...), or None."""
    isa = isa or ref_isa()
    if isa is None:
        return None
    if isa in _REF:
        return _REF[isa]
    path = HERE / "_ref" / f"jetfire_cpu_topk_attn_ref_{isa}.so"
    if not path.exists():
        _REF[isa] = None
        return None
    import torch  # noqa: F401  (the extension links against libtorch)
    try:
        C.CDLL("libcuda.so.1", mode=C.RTLD_GLOBAL)
    except OSError:
        stub = Path("/usr/local/cuda/lib64/stubs/libcuda.so")
        if stub.exists():  # no driver on this machine: the link-time stub satisfies the loader
            C.CDLL(str(stub), mode=C.RTLD_GLOBAL)
    try:
        spec = importlib.util.spec_from_file_location(path.name[:-3], str(path))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    except Exception as exc:  # pragma: no cover - depends on the host
        print(f"[oracle] reference extension failed to load: {exc}")
        mod = None
    _REF[isa] = mod
    return mod


_REF_GPU = {}


def ref_gpu_module(name: str):
    """The reference's GPU extension ``name`` (a key of ``build_oracle.REF_GPU``: ``int3_qk_scores``,
    ``int2_softmax_v``, ``int4_softmax_v``, ``int8tc_qk_scores``, ``int8tc_softmax_v_fused``,
    ``blend``) compiled from its unmodified source for sm_100, or None."""
    if name in _REF_GPU:
        return _REF_GPU[name]
    path = HERE / "_ref" / f"jetfire_{name}_ref.so"
    mod = None
    if path.exists():
        import torch  # noqa: F401  (the extension links against libtorch)
        try:
            spec = importlib.util.spec_from_file_location(path.name[:-3], str(path))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
        except Exception as exc:  # pragma: no cover - depends on the host
            print(f"[oracle] reference GPU extension {name} failed to load: {exc}")
            mod = None
    _REF_GPU[name] = mod
    return mod
