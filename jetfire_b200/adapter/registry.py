"""Wiring into a running vLLM (jetfire_vllm/adapter/registry.py:19-61, :1859-1945 of JetFire, reduced
to what the decode hot path needs).

``ensure_jetfire_registered()`` puts the backend of ``jetfire_backend.py`` into vLLM's ``CUSTOM``
attention-backend slot, so that ``--attention-backend CUSTOM`` (``attention_backend="CUSTOM"``)
selects it -- the reference does the same with its own class path
(``register_backend(AttentionBackendEnum.CUSTOM, "jetfire_vllm.adapter.jetfire_backend.
JetFireAttentionBackend")``).  ``install_layer_stores()`` is the worker-side hook: once vLLM has
planned its KV cache (number of blocks, block size per layer group), it creates the packed cache
and host mirror of every attention layer with that geometry; the backend's
``do_kv_cache_update`` / ``forward`` then find the store by layer name.

Not built here (out of the hot path): the reference's patches of vLLM's memory planner, its
dummy native KV tensors, prefill activation chunking and scheduler changes.
"""
from __future__ import annotations

from .cache_store import JetFireCacheStore
from .config import JetFireConfig, get_jetfire_config
from .jetfire_backend import register_layer_store

JETFIRE_BACKEND_PATH = "jetfire_b200.adapter.jetfire_backend.JetFireAttentionBackend"
_REGISTERED = False


def ensure_jetfire_registered() -> bool:
    """Register the backend as vLLM's CUSTOM attention backend (idempotent).  Returns False when
    the configuration disables it; raises ImportError when vLLM's registry is not importable."""
    global _REGISTERED
    cfg = get_jetfire_config()
    if not cfg.enabled:
        return False
    if _REGISTERED:
        return True
    try:
        from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend
    except Exception as exc:  # pragma: no cover - depends on the installed vLLM
        raise ImportError(f"vLLM's attention-backend registry is not importable: {exc}") from exc
    register_backend(AttentionBackendEnum.CUSTOM, JETFIRE_BACKEND_PATH)
    _REGISTERED = True
    return True


def install_layer_stores(layers: dict, *, num_blocks: int, block_size: int = 16, device="cuda", dtype=None,
                         cfg: JetFireConfig | None = None, mirror_append: str = "mapped") -> dict:
    """``layers``: layer name -> object with ``num_kv_heads`` and ``head_size`` (vLLM's ``Attention``
    modules, or any stand-in).  Creates one ``JetFireCacheStore`` per layer with vLLM's planned
    ``num_blocks`` (the scheduler hands out block ids in [0, num_blocks), so the cache must cover
    them all) and registers it under the layer's name.  Layers whose geometry the decode path does
    not serve (head size other than 128, block size other than 16) are skipped and fall back to
    vLLM's native attention.  Returns name -> store for the layers that were installed."""
    import torch
    cfg = cfg or get_jetfire_config()
    dtype = dtype or torch.bfloat16
    out = {}
    for name, layer in layers.items():
        if int(getattr(layer, "head_size", 0)) != 128 or int(block_size) != 16:
            continue
        store = JetFireCacheStore(num_blocks=int(num_blocks), num_kv_heads=int(layer.num_kv_heads), head_dim=128,
                                  cfg=cfg, device=device, dtype=dtype, block_size=int(block_size),
                                  mirror_append=mirror_append)
        register_layer_store(name, store)
        out[name] = store
    return out
