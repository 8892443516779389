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


def chunked_cross_entropy(hidden_td, targets_t, head_weight, mask_t=None):
    """xax/arch/llm.py:718-887, loss and accuracy at once: the hidden states are cast to float32 and multiplied
    by the (bf16) head weight in float32, log_softmax in float32, masked mean.  Returns (loss, accuracy) float32.
    (The chunking of the reference changes memory use, not the value, apart from float32 summation order.)"""
    h = f32(np.asarray(hidden_td))
    w = f32(np.asarray(head_weight))
    targets_t = np.asarray(targets_t).astype(np.int64)
    T = h.shape[0]
    mask = np.ones((T,), dtype=bool) if mask_t is None else np.asarray(mask_t).astype(bool)
    logits = (h @ w.T).astype(float32)
    m = logits.max(axis=-1, keepdims=True)
    lse = (m[:, 0] + np.log(np.exp(logits - m, dtype=float32).sum(axis=-1, dtype=float32))).astype(float32)
    loss_t = (lse - logits[np.arange(T), targets_t]).astype(float32)
    correct = logits.argmax(axis=-1) == targets_t
    n = float32(mask.sum())
    if n == 0:
        return float32(0.0), float32(0.0)
    return float32(loss_t[mask].sum(dtype=float32) / n), float32(float32(correct[mask].sum()) / n)


class CrossAttentionLLM:
    """xax/arch/llm.py:362-623: an LLM with one cross-attention block (and its pre-norm) shared by all layers,
    applied after every transformer block."""

    def __init__(self, llm: LLM, cross_attn, cross_attn_norm):
        self.llm, self.cross_attn, self.cross_attn_norm, self.config = llm, cross_attn, cross_attn_norm, llm.config

    def init_cache(self, max_len=None, dtype=bfloat16, encoder_output_sn=None):  # :445-470
        cross = None if encoder_output_sn is None else self.cross_attn.init_cache(encoder_output_sn)
        return self.llm.init_cache(max_len, dtype), cross

    def _cross(self, x, encoder_output_sn, cross_cache):  # :537-545 / :551-559
        from .attention import promote, rnd

        norm_x = self.cross_attn_norm(x)
        out, new_cache = self.cross_attn.forward(norm_x, kv_sn=encoder_output_sn if cross_cache is None else None,
                                                 cache=cross_cache)
        return rnd(f32(x) + f32(out), promote(x.dtype, out.dtype)), new_cache

    def forward_hidden(self, tokens_t, *, encoder_output_sn=None, context_tn=None, caches=None, cross_cache=None):
        """:502-560."""
        from .attention import promote, rnd

        tokens_t = np.asarray(tokens_t)
        assert tokens_t.ndim == 1
        x = self.llm.embed_tokens(tokens_t)
        if context_tn is not None:  # :529-530
            context_tn = np.asarray(context_tn)
            x = rnd(f32(context_tn) + f32(x), promote(context_tn.dtype, x.dtype))
        if caches is None:
            for b in self.llm.blocks:
                x, _ = b.forward(x, cache=None)
                if encoder_output_sn is not None:
                    x, _ = self._cross(x, encoder_output_sn, None)
            return self.llm.norm(x)
        out, updated_cross = [], cross_cache
        for b, c in zip(self.llm.blocks, caches, strict=True):
            x, c = b.forward(x, cache=c)
            out.append(c)
            if cross_cache is not None or encoder_output_sn is not None:
                x, updated_cross = self._cross(x, encoder_output_sn, cross_cache)
        return self.llm.norm(x), out, updated_cross

    def forward(self, tokens_t, *, context_tn=None, encoder_output_sn=None, caches=None, cross_cache=None):
        """:594-623."""
        if caches is None:
            return self.llm.get_logits(self.forward_hidden(tokens_t, context_tn=context_tn,
                                                           encoder_output_sn=encoder_output_sn))
        x, caches_out, cross_out = self.forward_hidden(tokens_t, context_tn=context_tn, encoder_output_sn=encoder_output_sn,
                                                       caches=caches, cross_cache=cross_cache)
        return self.llm.get_logits(x), caches_out, cross_out


def greedy_token(logits_v) -> int:
    """xax/arch/llm.py:1466-1470: argmax of float32 logits, first index on ties."""
    return int(np.argmax(f32(logits_v)))


def apply_sampling_mask(logits_1v, generated_count: int, eos_id: int, min_new_tokens_before_eos: int = 0,
                        allowed_token_range=None):
    """xax/arch/llm.py:1547-1570: tokens outside the allowed range -- and EOS before
    ``min_new_tokens_before_eos`` tokens were generated -- get the most negative finite value of the
    logits' dtype."""
    logits_1v = np.asarray(logits_1v)
    ids = np.arange(logits_1v.shape[-1], dtype=np.int32)
    allow_eos = generated_count >= min_new_tokens_before_eos
    if allowed_token_range is None:
        allowed = np.ones_like(ids, dtype=bool)
        if eos_id >= 0 and not allow_eos:
            allowed &= ids != eos_id
    else:
        lo, hi = allowed_token_range
        if hi <= lo:
            raise ValueError("allowed_token_range must satisfy max_id > min_id.")
        allowed = (ids >= lo) & (ids < hi)
        if eos_id >= 0 and allow_eos:
            allowed |= ids == eos_id
    import ml_dtypes

    min_logit = np.asarray(ml_dtypes.finfo(logits_1v.dtype).min).astype(logits_1v.dtype)
    return np.where(allowed[None, :], logits_1v, min_logit)


def nucleus(logits_v, temperature: float, top_p: float):
    """xax/arch/llm.py:1472-1482 for one row: (token ids in sorted order, their probabilities, kept mask).
    Descending stable sort of logits / temperature, float32 softmax and cumulative sum over the sorted
    order, a token is dropped when its inclusive cumulative probability exceeds top_p, the first never."""
    scaled = (f32(logits_v) / float32(temperature)).astype(float32)
    order = np.argsort(-scaled, kind="stable")
    srt = scaled[order]
    e = np.exp(srt - srt[0], dtype=float32)
    probs = (e / e.sum(dtype=float32)).astype(float32)
    cum = np.cumsum(probs, dtype=float32)
    drop = cum > float32(top_p)
    drop[0] = False
    return order, probs, ~drop


def sample_next_token(logits_tv, temperature: float, top_p: float, uniforms=None):
    """xax/arch/llm.py:1446-1489 with the random draw restated as an inverse CDF: the reference draws with
    jax.random.categorical over the kept logits (same distribution, its own PRNG stream); here row t takes
    the token at quantile ``uniforms[t]`` of the kept tokens in sorted order.  Returns int32 (tsz, 1)."""
    logits_tv = np.asarray(logits_tv)
    out = np.zeros((logits_tv.shape[0], 1), np.int32)
    for t in range(logits_tv.shape[0]):
        if temperature <= 0:  # :1469-1470, :1489
            out[t, 0] = int(np.argmax(f32(logits_tv[t])))
            continue
        order, probs, keep = nucleus(logits_tv[t], temperature, top_p)
        p = np.where(keep, probs, 0.0).astype(np.float64)
        cdf = np.cumsum(p)
        j = int(np.searchsorted(cdf, float(uniforms[t]) * cdf[-1], side="right"))
        j = min(j, int(np.nonzero(keep)[0][-1]))
        out[t, 0] = int(order[j])
    return out


def llm_generate_sampled(model: LLM, tokens_t, eos_id: int, max_new_tokens: int, temperature: float, top_p: float,
                         uniforms, allowed_token_range=None, min_new_tokens_before_eos: int = 0):
    """xax/arch/llm.py:1492-1614 with sampling: ``uniforms[i]`` drives the draw of the i-th new token (the
    reference splits its PRNG key once per token instead).  Returns (tokens[max_len] int32, final_len)."""
    if min_new_tokens_before_eos < 0:
        raise ValueError("min_new_tokens_before_eos must be >= 0.")
    tokens_t = np.asarray(tokens_t, dtype=np.int32)
    initial_len = tokens_t.shape[-1]
    max_len = initial_len + max_new_tokens
    if max_new_tokens <= 0:
        return tokens_t, initial_len
    padded = np.zeros(max_len, dtype=np.int32)
    padded[:initial_len] = tokens_t
    caches = model.init_cache(max_len, model.embed.weight.dtype)
    logits, caches = model.forward(tokens_t, caches=caches)
    cur, done = initial_len, False
    last = logits[-1:]
    while True:
        masked = apply_sampling_mask(last, cur - initial_len, eos_id, min_new_tokens_before_eos, allowed_token_range)
        nxt = int(sample_next_token(masked, temperature, top_p, uniforms[cur - initial_len:cur - initial_len + 1])[0, 0])
        padded[cur] = nxt
        done = eos_id >= 0 and nxt == eos_id
        cur += 1
        if cur >= max_len or done:
            break
        last, caches = model.forward(padded[cur - 1:cur], caches=caches)
    return padded, cur


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
