"""Attention-backend shim (jetfire_vllm/adapter/jetfire_backend.py:66-229).

vLLM's classes are imported lazily and only here, so the rest of the package works without
vLLM.  ``JetFireAttentionImplMixin`` holds the routing (decode -> ``try_jetfire_decode``,
a step with decode and prefill sequences -> ``try_jetfire_mixed``, append ->
``JetFireCacheStore.write_slots``); ``make_backend()`` binds it to the vLLM FlashAttention
classes of the installed version, with a metadata builder that notes the scheduler's
decode/prefill split on the metadata, and returns the backend class to register as ``CUSTOM`` (``register_backend(AttentionBackendEnum.CUSTOM, ...)``, reference
jetfire_vllm/adapter/registry.py:19, :61).
"""
from __future__ import annotations

from .cache_store import JetFireCacheStore
from .config import get_jetfire_config
from .decode_path import try_jetfire_decode
from .mixed_batch import annotate_split_counts, try_jetfire_mixed

_STORES: dict[str, JetFireCacheStore] = {}


def get_layer_store(layer_name: str) -> JetFireCacheStore | None:
    return _STORES.get(layer_name)


def register_layer_store(layer_name: str, store: JetFireCacheStore) -> None:
    _STORES[layer_name] = store


class JetFireAttentionImplMixin:
    """forward / do_kv_cache_update with the reference's signatures."""

    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None,
                output_scale=None, output_block_scale=None):
        store = get_layer_store(getattr(layer, "layer_name", ""))
        if output is not None and attn_metadata is not None:
            done = try_jetfire_decode(impl=self, layer=layer, query=query, attn_metadata=attn_metadata,
                                      output=output, store=store, cfg=get_jetfire_config())
            if done is not None:
                return done
            if key is not None and value is not None:
                done = try_jetfire_mixed(impl=self, layer=layer, query=query, key=key, value=value,
                                         attn_metadata=attn_metadata, output=output, store=store,
                                         cfg=get_jetfire_config())
                if done is not None:
                    return done
        return super().forward(layer, query, key, value, kv_cache, attn_metadata, output=output,
                               output_scale=output_scale, output_block_scale=output_block_scale)

    def do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping) -> None:
        store = get_layer_store(getattr(layer, "layer_name", ""))
        if store is not None:
            n = int(slot_mapping.shape[0])
            store.write_slots(key[:n].view(n, store.num_kv_heads, store.head_dim),
                              value[:n].view(n, store.num_kv_heads, store.head_dim), slot_mapping)
        parent = getattr(super(), "do_kv_cache_update", None)
        if parent is not None:
            parent(layer, key, value, kv_cache, slot_mapping)


def make_backend():
    """Bind the mixin to the installed vLLM's FlashAttention backend.  Raises ImportError
    with a clear message when vLLM (or the expected classes) is unavailable."""
    try:
        from vllm.v1.attention.backends.flash_attn import (FlashAttentionBackend, FlashAttentionImpl,
                                                           FlashAttentionMetadataBuilder)
    except Exception as exc:  # pragma: no cover - depends on the installed vLLM
        raise ImportError(f"vLLM FlashAttention backend classes not importable: {exc}") from exc

    class JetFireAttentionImpl(JetFireAttentionImplMixin, FlashAttentionImpl):
        pass

    class JetFireAttentionMetadataBuilder(FlashAttentionMetadataBuilder):
        """FlashAttention's metadata plus the decode/prefill split of the step, taken from the
        host copies the scheduler already holds (jetfire_vllm/adapter/jetfire_backend.py:66-127)."""

        def build(self, common_prefix_len, common_attn_metadata, fast_build=False):
            metadata = super().build(common_prefix_len, common_attn_metadata, fast_build=fast_build)
            try:
                annotate_split_counts(metadata, common_attn_metadata.query_start_loc_cpu.tolist(),
                                      common_attn_metadata.seq_lens_cpu.tolist())
            except (AttributeError, ValueError):
                pass        # without the counts a mixed step is split from the device tensors
            return metadata

    class JetFireAttentionBackend(FlashAttentionBackend):
        @staticmethod
        def get_name() -> str:
            return "CUSTOM"

        @staticmethod
        def get_impl_cls():
            return JetFireAttentionImpl

        @staticmethod
        def get_builder_cls():
            return JetFireAttentionMetadataBuilder

    return JetFireAttentionBackend


_BACKEND = None


def __getattr__(name):
    """``JetFireAttentionBackend`` / ``JetFireAttentionImpl`` resolve lazily (the class path vLLM's
    registry is given, see ``registry.JETFIRE_BACKEND_PATH``), so importing this module does not
    import vLLM."""
    global _BACKEND
    if name in ("JetFireAttentionBackend", "JetFireAttentionImpl"):
        if _BACKEND is None:
            _BACKEND = make_backend()
        return _BACKEND if name == "JetFireAttentionBackend" else _BACKEND.get_impl_cls()
    raise AttributeError(name)
