"""xax_b200: the FP8 transformer inference forward path of codekansas/xax, rebuilt for B200.

Top-level names mirror the ones xax exports for this path (xax/__init__.py:19-61); FP8
utilities live in ``xax_b200.nn.fp8`` as they do in ``xax.nn.fp8``.  Imports are lazy so
that importing the package never needs a GPU; calling anything that computes does.
"""

from __future__ import annotations

import importlib

__version__ = "0.1.0"

NAME_MAP = {
    # xax.arch.attention
    "AttentionCache": "arch.attention", "Fp8ScalesCache": "arch.attention", "TransformerBlockCache": "arch.attention",
    "RMSNorm": "arch.attention", "RotaryEmbedding": "arch.attention", "SelfAttentionBlock": "arch.attention",
    "SwiGLU": "arch.attention", "TransformerBlock": "arch.attention", "apply_linear": "arch.attention",
    "can_use_cudnn_attention": "arch.attention", "Linear": "arch.attention", "Embedding": "arch.attention",
    "TransformerStack": "arch.attention", "Transformer": "arch.attention", "TransformerCache": "arch.attention",
    "CrossAttentionBlock": "arch.attention",
    # xax.arch.llm
    "LLM": "arch.llm", "LLMConfig": "arch.llm", "CrossAttentionLLM": "arch.llm", "llm_generate": "arch.llm", "llm_generate_jit": "arch.llm",
    "llm_generate_batch": "arch.llm", "llm_generate_stream": "arch.llm", "TokenSampler": "arch.llm",
    "tie_embedding_and_head": "arch.llm", "chunked_cross_entropy_loss": "arch.llm",
    "chunked_cross_entropy_acc": "arch.llm",
    "get_model_parallel_sharding_spec": "arch.llm", "DecodeState": "arch.llm",
    "build_pretrained_llm": "arch.hf", "hf_config_to_llm_config": "arch.hf", "load_hf_weights_into_llm": "arch.hf",
    # xax.nn.fp8 (not re-exported by xax at top level; offered here for convenience)
    "Fp8Linear": "nn.fp8", "Fp8Scales": "nn.fp8", "init_fp8_scales": "nn.fp8", "fp8_matmul": "nn.fp8",
    # xax.nn.lora
    "LoRALinear": "nn.lora", "loraize_linear": "nn.lora",
    # tensor parallelism
    "setup_model_parallel_mesh": "parallel", "TensorParallel": "parallel", "make_sharded_array": "parallel",
}

__all__ = sorted(NAME_MAP)


def __getattr__(name: str):
    mod = NAME_MAP.get(name)
    if mod is None:
        raise AttributeError(f"module 'xax_b200' has no attribute {name!r}")
    return getattr(importlib.import_module(f"{__name__}.{mod}"), name)
