"""The C ABI and the module API, as far as they can be checked without a GPU: the shared
library builds and loads, exports exactly the symbols include/xaxb200.h declares, the ctypes
table covers them, the package mirrors the reference's names / signatures / defaults, and
compute calls fail loudly instead of falling back."""

import inspect
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "xaxb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(xaxb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    from xax_b200 import _lib

    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes table and header disagree"
    assert lib.xaxb_status_string(0) == b"ok" and lib.xaxb_status_string(5) == b"device-side wait timed out"
    assert lib.xaxb_attn_decode_workspace_bytes(32, 32, 128, 8192) == 32 * 32 * 64 * 130 * 4


def test_header_cites_the_reference_for_every_kernel_entry():
    text = open(os.path.join(ROOT, "include", "xaxb200.h")).read()
    for entry in ("xaxb_quantize_current", "xaxb_quantize_delayed", "xaxb_gemm_fp8", "xaxb_gemm_bf16", "xaxb_rmsnorm",
                  "xaxb_silu_mul", "xaxb_embed", "xaxb_argmax", "xaxb_kv_append_rope", "xaxb_attn_decode",
                  "xaxb_attn_prefill"):
        head = text[:text.index(f"int {entry}(")]
        comment = head[head.rindex("/*"):]
        assert re.search(r"xax/(nn|arch)/\w+\.py:\d+", comment), entry


def test_no_cpu_fallback():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from xax_b200 import ops

    with pytest.raises((RuntimeError, ValueError)):
        ops.quantize_current(torch.zeros((4, 8), dtype=torch.bfloat16), 1)
    with pytest.raises((RuntimeError, ValueError)):
        ops.gemm_bf16(torch.zeros((4, 8), dtype=torch.bfloat16), torch.zeros((8, 8), dtype=torch.bfloat16))


def test_package_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "xax_b200")
    for d, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                src = open(os.path.join(d, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", src, flags=re.M), f
                assert "_work/" not in src, f


def test_module_api_matches_the_reference():
    """Names, keyword arguments and defaults of the hot-path API (xax/__init__.py:19-61,
    xax/nn/fp8.py, xax/arch/attention.py, xax/arch/llm.py)."""
    import xax_b200 as xax
    from xax_b200.nn import fp8

    for name in ("RMSNorm", "RotaryEmbedding", "SelfAttentionBlock", "SwiGLU", "TransformerBlock", "apply_linear",
                 "AttentionCache", "Fp8ScalesCache", "TransformerBlockCache", "LLM", "LLMConfig", "llm_generate",
                 "llm_generate_jit", "tie_embedding_and_head"):
        assert getattr(xax, name) is not None
    with pytest.raises(AttributeError):
        xax.NoSuchThing
    assert fp8.E4M3_MAX == 448.0 and fp8.E5M2_MAX == 57344.0 and fp8.AMAX_HISTORY_LENGTH == 1024
    for fn in ("get_fp8_max", "compute_scale", "compute_amax_history", "quantize", "dequantize", "quantize_dequantize",
               "Fp8Scales", "init_fp8_scales", "Fp8Linear", "fp8_matmul"):
        assert hasattr(fp8, fn)

    def params(f):
        return inspect.signature(f).parameters

    p = params(fp8.compute_scale)
    assert list(p)[:4] == ["amax", "scale", "fp8_max", "margin"] and p["margin"].default == 0
    assert params(fp8.init_fp8_scales)["history_length"].default == 1024
    p = params(fp8.Fp8Linear.__init__)
    assert list(p)[1:3] == ["in_features", "out_features"]
    assert p["use_bias"].default is True and p["use_fp8"].default is True and p["key"].kind == p["key"].KEYWORD_ONLY
    assert list(params(fp8.Fp8Linear.__call__))[1:3] == ["x", "scales"]
    assert [f for f in fp8.Fp8Scales.__dataclass_fields__] == ["input_scale", "input_amax_history", "kernel_scale",
                                                               "kernel_amax_history"]
    p = params(xax.RMSNorm.build)
    assert p["eps"].default == 1e-6
    p = params(xax.SwiGLU.build)
    assert p["hidden_dim"].default is None and p["use_bias"].default is False
    p = params(xax.RotaryEmbedding.build)
    assert p["base"].default == 10000.0 and p["style"].default == "interleaved" and p["beta_fast"].default == 32.0
    p = params(xax.SelfAttentionBlock.build)
    for k, v in dict(num_kv_heads=None, head_dim=None, use_bias=True, causal=False, context_length=None,
                     use_rotary_embeddings=False, rotary_base=10000.0, rotary_style="concatenated", rotary_factor=1.0,
                     use_qk_norm=False, qk_norm_eps=1e-6, use_attention_sinks=False, use_fp8=False).items():
        assert p[k].default == v, k
    assert list(params(xax.SelfAttentionBlock.forward))[1:5] == ["x_tn", "mask", "cache", "fp8_scales"]
    p = params(xax.TransformerBlock.build)
    assert list(p)[:3] == ["embed_dim", "num_heads", "ff_dim"]
    assert p["norm_type"].default == "layernorm" and p["feedforward_type"].default == "mlp" and p["norm_eps"].default == 1e-6
    assert list(params(xax.TransformerBlock.forward))[1:5] == ["x_tn", "context_sn", "mask", "cache"]
    assert list(params(xax.TransformerBlock.init_cache))[1:5] == ["max_len", "dtype", "context_sn", "fp8_history_length"]
    c = xax.LLMConfig(vocab_size=10, embed_dim=8, q_heads=2, kv_heads=1, head_dim=4, num_layers=1)
    assert (c.max_tsz, c.rope_theta, c.mlp_mult, c.mlp_hidden_dim, c.rms_eps, c.attention_bias, c.mlp_bias) == \
        (32768, 10000.0, 4, None, 1e-6, False, False)
    assert c.with_vocab(12).vocab_size == 12 and c.uses_yarn is False
    with pytest.raises(Exception):
        c.vocab_size = 3  # frozen
    p = params(xax.llm_generate_jit)
    assert list(p)[:8] == ["model", "tokens_t", "eos_id", "max_new_tokens", "context_tn", "temperature", "top_p", "key"]
    assert p["allowed_token_range"].default is None and p["min_new_tokens_before_eos"].default == 0
    assert params(xax.llm_generate)["max_new_tokens"].default == 20
    assert xax.can_use_cudnn_attention(__import__("torch").bfloat16, 128, 64) is True
    assert xax.can_use_cudnn_attention(__import__("torch").bfloat16, 128, 1) is False  # decode: seq_len % 64


def test_sharding_spec_matches_the_reference_rule():
    """xax/arch/llm.py:931-975."""
    from xax_b200.arch.llm import get_model_parallel_sharding_spec as spec

    for n in ("layers.0.self_attn.q_proj", "k_proj", "v_proj", "mlp.gate_proj", "up_proj"):
        assert spec((8, 4), n) == ("model", None)
    for n in ("self_attn.o_proj", "mlp.down_proj"):
        assert spec((8, 4), n) == (None, "model")
    assert spec((8, 4), "lm_head") == ("model", None)
    assert spec((8,), "q_proj") == () and spec((8, 4), "embed_tokens") == () and spec((8, 4), "norm") == ()


def test_unsupported_features_raise_clearly():
    import xax_b200 as xax

    sa = xax.SelfAttentionBlock.build(64, 2, key=0, context_length=8, use_attention_sinks=True, device="cpu")
    assert sa.local_window_size == 7 and sa.sinks.shape == (2,)  # :660, :652-654
    xblk = xax.TransformerBlock.build(64, 2, 128, key=0, cross_attention=True, causal=True, use_rotary_embeddings=True,
                                      norm_type="rmsnorm", feedforward_type="swiglu", device="cpu")
    assert type(xblk.cross_attn).__name__ == "CrossAttentionBlock" and xblk.cross_attn_norm is not None
    assert xblk.cross_attn.rotary_emb.style == "interleaved"  # the class default, as CrossAttentionBlock.build gets it
    with pytest.raises(ValueError, match="context_sn must be provided"):
        xblk.init_cache(max_len=8)
    with pytest.raises(ValueError):
        xax.TransformerBlock.build(64, 2, 128, key=0, device="cpu")  # layernorm / mlp defaults are not on the path
    with pytest.raises(ValueError, match="float8_e4m3fn only"):
        xax.Fp8Linear(8, 8, key=0, fp8_dtype=__import__("torch").float8_e5m2, device="cpu")
    blk = xax.TransformerBlock.build(64, 2, 128, key=0, num_kv_heads=1, head_dim=32, causal=True,
                                     use_rotary_embeddings=True, norm_type="rmsnorm", feedforward_type="swiglu",
                                     use_fp8=True, device="cpu")
    assert type(blk.self_attn.q_proj).__name__ == "Fp8Linear" and blk.self_attn.q_proj.bias is not None
    assert type(blk.feed_forward.gate).__name__ == "Linear"  # like the reference: use_fp8 leaves the SwiGLU plain
    with pytest.raises(ValueError):
        blk.self_attn.init_cache(None)
