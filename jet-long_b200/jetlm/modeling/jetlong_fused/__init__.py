from .modeling_qwen3_jetlong_fused import (  # noqa: F401
    Qwen3JetLongFusedForCausalLM,
    Qwen3JetLongFusedModel,
    Qwen3JetLongFusedRotaryEmbedding,
)
