"""Oracle restatement of the decode path of ``xax/arch/llm.py`` (test infrastructure;
parity unpinned -- see the package docstring)."""

from __future__ import annotations

from dataclasses import dataclass, replace

import numpy as np

from .attention import Embedding, Linear, RMSNorm, apply_linear, build_block
from .fp8 import bfloat16, f32, float32


@dataclass(frozen=True)
class LLMConfig:
    """xax/arch/llm.py:47-79 (fields used by the path)."""

    vocab_size: int
    embed_dim: int
    q_heads: int
    kv_heads: int
    head_dim: int
    num_layers: int
    max_tsz: int = 32768
    rope_theta: float = 10_000.0
    mlp_mult: int = 4
    mlp_hidden_dim: int | None = None
    rms_eps: float = 1e-6
    sliding_window_size: int | None = None
    layer_attention_types: tuple | None = None  # :113-120: layers whose type contains "sliding" get the window

    def with_vocab(self, vocab_size: int) -> "LLMConfig":
        return replace(self, vocab_size=vocab_size)


class LLM:
    """xax/arch/llm.py:82-324."""

    def __init__(self, embed, blocks, norm, lm_head, config):
        self.embed, self.blocks, self.norm, self.lm_head, self.config = embed, tuple(blocks), norm, lm_head, config

    @classmethod
    def build(cls, config: LLMConfig, rng, *, use_fp8=True, tie=True, std=0.02, dtype=bfloat16) -> "LLM":
        """Random-init model: N(0, std^2) weights, bf16, FP8 projections when ``use_fp8``."""
        embed = Embedding((rng.standard_normal((config.vocab_size, config.embed_dim), dtype=float32) * float32(std)).astype(dtype))
        width = config.mlp_hidden_dim or config.embed_dim * config.mlp_mult  # :109
        blocks = [
            build_block(rng, embed_dim=config.embed_dim, num_heads=config.q_heads, num_kv_heads=config.kv_heads,
                        head_dim=config.head_dim, ff_dim=width, rope_theta=config.rope_theta, norm_eps=config.rms_eps,
                        fp8_attn=use_fp8, fp8_mlp=use_fp8, std=std, dtype=dtype,
                        local_window_size=(config.sliding_window_size
                                           if config.layer_attention_types is not None
                                           and i < len(config.layer_attention_types)
                                           and "sliding" in config.layer_attention_types[i] else None))
            for i in range(config.num_layers)
        ]
        norm = RMSNorm.build(config.embed_dim, config.rms_eps, dtype)
        if tie:  # tie_embedding_and_head, :713-715
            head = Linear(embed.weight)
        else:
            head = Linear((rng.standard_normal((config.vocab_size, config.embed_dim), dtype=float32) * float32(std)).astype(dtype))
        return cls(embed, blocks, norm, head, config)

    def embed_tokens(self, tokens_t):  # :205-211
        return self.embed.weight[np.asarray(tokens_t)]

    def get_logits(self, hidden_td):  # :213-219
        return apply_linear(hidden_td, self.lm_head)

    def init_cache(self, max_len=None, dtype=bfloat16):  # :221-234
        return [b.init_cache(max_len, dtype) for b in self.blocks]

    def forward_hidden(self, tokens_t, *, caches=None):  # :252-285
        tokens_t = np.asarray(tokens_t)
        assert tokens_t.ndim == 1
        x = self.embed_tokens(tokens_t)
        if caches is None:
            for b in self.blocks:
                x, _ = b.forward(x, cache=None)
            return self.norm(x)
        out = []
        for b, c in zip(self.blocks, caches, strict=True):
            x, c = b.forward(x, cache=c)
            out.append(c)
        return self.norm(x), out

    def forward(self, tokens_t, *, caches=None):  # :304-324
        if caches is None:
            return self.get_logits(self.forward_hidden(tokens_t))
        x, caches = self.forward_hidden(tokens_t, caches=caches)
        return self.get_logits(x), caches


def greedy_token(logits_v) -> int:
    """xax/arch/llm.py:1466-1470: argmax of float32 logits, first index on ties."""
    return int(np.argmax(f32(logits_v)))


def llm_generate_greedy(model: LLM, tokens_t, eos_id: int, max_new_tokens: int):
    """xax/arch/llm.py:1492-1614 with temperature <= 0 (greedy), no context, no token
    range: prefill the cache with the prompt, then one token per iteration until max_len or
    EOS.  Returns (tokens[max_len] int32, final_len)."""
    tokens_t = np.asarray(tokens_t, dtype=np.int32)
    initial_len = tokens_t.shape[-1]
    max_len = initial_len + max_new_tokens
    if max_new_tokens <= 0:  # :1537-1538
        return tokens_t, initial_len
    padded = np.zeros(max_len, dtype=np.int32)
    padded[:initial_len] = tokens_t
    caches = model.init_cache(max_len, model.embed.weight.dtype)  # :1544-1545
    logits, caches = model.forward(tokens_t, caches=caches)  # :1574
    nxt = greedy_token(logits[-1])
    padded[initial_len] = nxt
    done = eos_id >= 0 and nxt == eos_id
    cur = initial_len + 1
    while cur < max_len and not done:  # :1586-1613
        logits, caches = model.forward(padded[cur - 1:cur], caches=caches)
        nxt = greedy_token(logits[-1])
        padded[cur] = nxt
        done = eos_id >= 0 and nxt == eos_id
        cur += 1
    return padded, cur
