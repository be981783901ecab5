"""Host-side mirror of the pieces of JetFire's vLLM adapter that sit on the decode hot
path (jetfire_vllm/adapter/): configuration, the per-layer packed cache with its
full-precision host mirror, the decode orchestrator and the attention-backend shim."""
