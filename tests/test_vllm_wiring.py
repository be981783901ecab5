"""Import-level wiring against the vLLM that is installed (skipped where it is not, or where its
classes moved): the backend binds to vLLM's FlashAttention classes, keeps their method
signatures (the reference's own contract, jetfire_vllm/adapter/jetfire_backend.py:138-209 of
JetFire), registers as the CUSTOM attention backend and resolves back through vLLM's registry."""
import inspect

import pytest

pytest.importorskip("vllm", reason="vLLM is not installed")


def _vllm_classes():
    try:
        from vllm.v1.attention.backends.flash_attn import FlashAttentionBackend, FlashAttentionImpl
        from vllm.v1.attention.backends.registry import AttentionBackendEnum
    except Exception as exc:
        pytest.skip(f"this vLLM's attention classes are elsewhere: {exc}")
    return FlashAttentionBackend, FlashAttentionImpl, AttentionBackendEnum


@pytest.mark.timeout(600)
def test_backend_binds_registers_and_resolves():
    FlashAttentionBackend, FlashAttentionImpl, AttentionBackendEnum = _vllm_classes()
    from jetfire_b200.adapter import jetfire_backend as jb
    from jetfire_b200.adapter.registry import JETFIRE_BACKEND_PATH, ensure_jetfire_registered
    backend = jb.make_backend()
    impl = backend.get_impl_cls()
    assert backend.get_name() == "CUSTOM" and issubclass(backend, FlashAttentionBackend)
    assert issubclass(impl, FlashAttentionImpl) and issubclass(impl, jb.JetFireAttentionImplMixin)
    # same parameter names, in the same order, as the methods vLLM calls
    for meth in ("forward", "do_kv_cache_update"):
        theirs = list(inspect.signature(getattr(FlashAttentionImpl, meth)).parameters)
        mine = list(inspect.signature(getattr(jb.JetFireAttentionImplMixin, meth)).parameters)
        assert mine == theirs, f"{meth}: {mine} vs {theirs}"
    # the metadata builder is FlashAttention's, with the decode/prefill split noted on what it builds
    from vllm.v1.attention.backends.flash_attn import FlashAttentionMetadataBuilder
    builder = backend.get_builder_cls()
    assert issubclass(builder, FlashAttentionMetadataBuilder) and builder is not FlashAttentionMetadataBuilder
    assert (list(inspect.signature(builder.build).parameters)
            == list(inspect.signature(FlashAttentionMetadataBuilder.build).parameters))
    from vllm.v1.attention.backend import CommonAttentionMetadata
    assert "query_start_loc_cpu" in CommonAttentionMetadata.__dataclass_fields__
    assert isinstance(getattr(CommonAttentionMetadata, "seq_lens_cpu", None), property)
    assert ensure_jetfire_registered() is True
    assert ensure_jetfire_registered() is True            # idempotent
    resolved = AttentionBackendEnum.CUSTOM.get_class()
    assert resolved is jb.JetFireAttentionBackend and resolved.get_name() == "CUSTOM"
    assert JETFIRE_BACKEND_PATH.endswith("JetFireAttentionBackend")
