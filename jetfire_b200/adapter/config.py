"""Resolved configuration of the hot path (jetfire_vllm/adapter/config.py:34-60, 238-390).

Only the two paper modes are registered; one code path, no experiment knobs.  Environment
variables kept from the reference: ``JETFIRE_MODE``, ``JETFIRE_TOPK``, ``JETFIRE_GROUP_SIZE``,
``JETFIRE_CPU_ATTN_THREADS``, ``JETFIRE_MAX_BATCH_SIZE``.  Own: ``JETFIRE_SLOTS_I32``,
``JETFIRE_STREAM_ORDERED`` (decode steps queued on the stream without a host wait),
``JETFIRE_STREAM_SIGNAL`` (``flags`` | ``callbacks``: how such a step meets the host),
``JETFIRE_GPU_CORRECTION_SHARE`` (0..0.5: rows of the correction the GPU computes itself from the
mapped mirror over the host link, stream-ordered steps with flags only) and
``JETFIRE_NUMA_NODE`` (``auto`` | ``off`` | a node number: where the host mirrors and the
correction workers of this rank are placed).
"""
from __future__ import annotations

import os
from dataclasses import dataclass


@dataclass(frozen=True)
class QuantScheme:
    name: str
    k_nbits: int
    v_nbits: int
    k_asymmetric: bool = False
    v_asymmetric: bool = False


SYM_INT3K_SYM_INT2V = QuantScheme("SymInt3K_SymInt2V", 3, 2)
SYM_INT4K_SYM_INT4V = QuantScheme("SymInt4K_SymInt4V", 4, 4)
QUANT_SCHEMES = {s.name: s for s in (SYM_INT3K_SYM_INT2V, SYM_INT4K_SYM_INT4V)}

# paper mode table (jetfire_vllm/bench/artifact_performance.py:45): name -> (scheme, group size)
PAPER_MODES = {"k3v2": ("SymInt3K_SymInt2V", 64), "k4v4": ("SymInt4K_SymInt4V", 128)}
SCHEME_TO_KERNEL_MODE = {"SymInt3K_SymInt2V": "k3v2", "SymInt4K_SymInt4V": "k4v4"}

# top-k widths the release matrix offers (jetfire_vllm/adapter/release_policy.py:31-34),
# limited to what this library builds
SUPPORTED_TOP_K = (32, 64, 128, 256, 512, 1024, 2048, 4096)


NUMA_AUTO, NUMA_OFF = -2, -1   # the GPU's own node when the host has several / leave it to first touch


@dataclass(frozen=True)
class JetFireConfig:
    mode: str = "SymInt3K_SymInt2V"      # jetfire_vllm/adapter/config.py:166
    top_k: int = 256                      # :260
    group_size: int = 64                  # :261
    cpu_attn_threads: int = 32            # :179
    max_batch_size: int = 32
    enabled: bool = True
    slots_i32: bool = True                # selected slots cross to the host as int32 (the reference: int64)
    numa_node: int = NUMA_AUTO            # memory node of mirrors and workers: NUMA_AUTO, NUMA_OFF or a node
    stream_ordered: bool = True           # decode step queued on the stream without a host wait (capturable)
    stream_signal: str = "flags"          # how a stream-ordered step meets the host: "flags" or "callbacks"
    gpu_correction_share: float = 0.0     # fraction of the correction's rows the GPU computes from the mapped mirror

    @property
    def scheme(self) -> QuantScheme:
        return QUANT_SCHEMES[self.mode]

    @property
    def kernel_mode(self) -> str:
        return SCHEME_TO_KERNEL_MODE[self.mode]


_CONFIG: JetFireConfig | None = None


def _int_env(name: str, default: int) -> int:
    raw = os.environ.get(name)
    if raw is None or raw.strip() == "":
        return default
    try:
        return int(raw)
    except ValueError as exc:
        raise ValueError(f"{name} must be an integer, got {raw!r}") from exc


def _numa_env() -> int:
    raw = (os.environ.get("JETFIRE_NUMA_NODE") or "auto").strip().lower()
    if raw == "auto":
        return NUMA_AUTO
    if raw in ("off", "none", "-1"):
        return NUMA_OFF
    try:
        node = int(raw)
    except ValueError as exc:
        raise ValueError(f"JETFIRE_NUMA_NODE must be 'auto', 'off' or a node number, got {raw!r}") from exc
    if node < 0:
        raise ValueError(f"JETFIRE_NUMA_NODE must be 'auto', 'off' or a node number, got {raw!r}")
    return node


def get_jetfire_config() -> JetFireConfig:
    """Environment -> config, cached (jetfire_vllm/adapter/config.py:300-390)."""
    global _CONFIG
    if _CONFIG is not None:
        return _CONFIG
    mode = os.environ.get("JETFIRE_MODE", "SymInt3K_SymInt2V")
    group_default = 64
    if mode in PAPER_MODES:                      # accept the paper's short names too
        mode, group_default = PAPER_MODES[mode]
    elif mode == "SymInt4K_SymInt4V":
        group_default = 128
    if mode not in QUANT_SCHEMES:
        raise ValueError(f"JETFIRE_MODE={mode!r} is not built; choose one of {sorted(QUANT_SCHEMES)}")
    group = _int_env("JETFIRE_GROUP_SIZE", group_default)
    want = 64 if mode == "SymInt3K_SymInt2V" else 128
    if group != want:
        raise ValueError(f"{mode} is built for group size {want}, got JETFIRE_GROUP_SIZE={group}")
    top_k = _int_env("JETFIRE_TOPK", 256)
    if top_k not in SUPPORTED_TOP_K:
        raise ValueError(f"JETFIRE_TOPK={top_k} must be one of {SUPPORTED_TOP_K}")
    threads = _int_env("JETFIRE_CPU_ATTN_THREADS", 32)
    if threads <= 0:
        raise ValueError("JETFIRE_CPU_ATTN_THREADS must be positive")
    signal = (os.environ.get("JETFIRE_STREAM_SIGNAL") or "flags").strip().lower()
    if signal not in ("flags", "callbacks"):
        raise ValueError(f"JETFIRE_STREAM_SIGNAL must be 'flags' or 'callbacks', got {signal!r}")
    try:
        share = float(os.environ.get("JETFIRE_GPU_CORRECTION_SHARE") or 0.0)
    except ValueError as exc:
        raise ValueError("JETFIRE_GPU_CORRECTION_SHARE must be a number between 0 and 0.5") from exc
    if not 0.0 <= share <= 0.5:
        raise ValueError("JETFIRE_GPU_CORRECTION_SHARE must be a number between 0 and 0.5")
    _CONFIG = JetFireConfig(mode=mode, top_k=top_k, group_size=group, cpu_attn_threads=threads,
                            max_batch_size=_int_env("JETFIRE_MAX_BATCH_SIZE", 32),
                            slots_i32=_int_env("JETFIRE_SLOTS_I32", 1) != 0, numa_node=_numa_env(),
                            stream_ordered=_int_env("JETFIRE_STREAM_ORDERED", 1) != 0, stream_signal=signal,
                            gpu_correction_share=share)
    return _CONFIG


def reset_jetfire_config() -> None:
    global _CONFIG
    _CONFIG = None


def compute_inflate_ratio(scheme: QuantScheme, group_size: int = 128) -> float:
    """bf16 KV bytes / packed KV bytes (jetfire_vllm/adapter/config.py:409-425): 5.8x for
    K3V2 at group 64, 3.9x for K4V4 at group 128."""
    def bits(n):
        return n + 16.0 / group_size
    return 32.0 / (bits(scheme.k_nbits) + bits(scheme.v_nbits))
