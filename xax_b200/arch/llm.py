"""B200-native mirror of the decode path of ``xax/arch/llm.py``: ``LLMConfig``, ``LLM``,
``tie_embedding_and_head``, greedy ``llm_generate`` / ``llm_generate_jit`` and the
tensor-parallel placement rule ``get_model_parallel_sharding_spec``.

The reference generates one sequence at a time and leaves batching to ``jax.vmap``;
``llm_generate_batch`` is the batched loop (B prompts of equal length); the greedy decode step is
captured in a CUDA graph and replayed, a sampled one (temperature / top-p, token-range and EOS
masks) runs step by step because the random numbers and the EOS rule change per step.
Extra-token embeddings are outside the path this library covers and raise.
"""

from __future__ import annotations

from dataclasses import dataclass, replace

import torch

from .. import ops
from ..nn.fp8 import Fp8Linear
from .attention import BF16, Embedding, Linear, RMSNorm, SelfAttentionBlock, SwiGLU, TransformerBlock, apply_linear


@dataclass(frozen=True)
class LLMConfig:
    """xax/arch/llm.py:47-79 (same fields and defaults)."""

    vocab_size: int
    embed_dim: int
    q_heads: int
    kv_heads: int
    head_dim: int
    num_layers: int
    max_tsz: int = 32768
    rope_theta: float = 10_000.0
    dropout_rate: float = 0.0
    mlp_mult: int = 4
    mlp_hidden_dim: int | None = None
    rms_eps: float = 1e-6
    attention_bias: bool = False
    mlp_bias: bool = False
    rope_factor: float = 1.0
    rope_original_max_position_embeddings: int | None = None
    rope_beta_slow: float = 1.0
    rope_beta_fast: float = 32.0
    sliding_window_size: int | None = None
    layer_attention_types: tuple[str, ...] | None = None
    use_attention_sinks: bool = False
    use_qk_norm: bool = False

    def with_vocab(self, vocab_size: int) -> "LLMConfig":
        return replace(self, vocab_size=vocab_size)

    @property
    def uses_yarn(self) -> bool:
        return self.rope_factor > 1.0 and self.rope_original_max_position_embeddings is not None


def _randn(shape, std, gen, device):
    """N(0, std^2) bf16 weights generated on the device in slabs (no host copy of 8B-scale models)."""
    out = torch.empty(shape, dtype=BF16, device=device)
    flat = out.view(-1)
    step = 1 << 26
    for i in range(0, flat.numel(), step):
        n = min(step, flat.numel() - i)
        flat[i:i + n] = (torch.randn((n,), generator=gen, device=device, dtype=torch.float32) * std).to(BF16)
    return out


class LLM:
    """xax/arch/llm.py:82-324."""

    def __init__(self, embed: Embedding, blocks, norm: RMSNorm, lm_head: Linear, config: LLMConfig,
                 extra_embed=None, extra_lm_head=None, tied_extra_embed: bool = False):
        if extra_embed is not None or extra_lm_head is not None:
            raise ValueError("extra-token embeddings are outside the path this library covers")
        self.embed, self.blocks, self.norm, self.lm_head, self.config = embed, tuple(blocks), norm, lm_head, config
        self.extra_embed, self.extra_lm_head, self.tied_extra_embed = None, None, False

    @classmethod
    def build(cls, config: LLMConfig, *, extra_tokens: int | None = None, tied_extra_embed: bool = False, key=None,
              use_fp8: bool = False, init_std: float | None = None, device=None, tp_rank: int = 0,
              tp_size: int = 1) -> "LLM":
        """xax/arch/llm.py:96-203.  ``use_fp8`` (an extension: the reference hard-codes False,
        :155) makes q/k/v/out and gate/up/down Fp8Linear layers without bias, which is how the
        reference reaches an FP8 LLM (by swapping Fp8Linear into the module tree).
        ``init_std`` draws every weight from N(0, std^2) on the device instead of the
        reference's per-layer uniform init.  ``tp_rank`` / ``tp_size`` build only this rank's
        shard of each weight per get_model_parallel_sharding_spec (same seed on every rank)."""
        if extra_tokens is not None:
            raise ValueError("extra-token embeddings are outside the path this library covers")
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        seed = int(key or 0) if not isinstance(key, torch.Generator) else int(key.initial_seed())
        gen = torch.Generator(device=dev).manual_seed(seed)
        std = 0.02 if init_std is None else init_std
        H, D = config.embed_dim, config.head_dim
        width = config.mlp_hidden_dim or (H * config.mlp_mult)  # :109
        if config.q_heads % tp_size or config.kv_heads % tp_size or width % tp_size:
            raise ValueError(f"tp_size {tp_size} does not divide heads ({config.q_heads}/{config.kv_heads}) or MLP width {width}")

        def shard(w, name):
            dim = tp_shard_dim(name, w.dim())
            if tp_size == 1 or dim is None:
                return w
            n = w.shape[dim] // tp_size
            return w.narrow(dim, tp_rank * n, n).contiguous()

        def lin(o, i, name, bias):
            w = shard(_randn((o, i), std, gen, dev), name)
            if tp_shard_dim(name, 2) == 1 and tp_rank > 0:
                bias = False  # a row-parallel layer's bias is added once, by rank 0
            b = torch.zeros((w.shape[0],), dtype=BF16, device=dev) if bias else None
            if use_fp8:
                return Fp8Linear(w.shape[1], w.shape[0], weight=w, bias=b, use_bias=bias)
            return Linear(w.shape[1], w.shape[0], use_bias=bias, weight=w, bias=b)

        embed = Embedding(config.vocab_size, H, weight=_randn((config.vocab_size, H), std, gen, dev))
        blocks = []
        for i in range(config.num_layers):
            from .attention import RotaryEmbedding

            layer_window = None  # :113-120
            if config.layer_attention_types is not None and i < len(config.layer_attention_types):
                if "sliding" in config.layer_attention_types[i]:
                    layer_window = config.sliding_window_size

            attn = SelfAttentionBlock(
                lin(config.q_heads * D, H, "q_proj", config.attention_bias),
                lin(config.kv_heads * D, H, "k_proj", config.attention_bias),
                lin(config.kv_heads * D, H, "v_proj", config.attention_bias),
                lin(H, config.q_heads * D, "o_proj", config.attention_bias),
                RotaryEmbedding.build(D, config.rope_theta, "concatenated", config.rope_factor,
                                      config.rope_original_max_position_embeddings, config.rope_beta_slow,
                                      config.rope_beta_fast),
                RMSNorm.build(D, 1e-6, dev) if config.use_qk_norm else None,  # :123-141 leaves qk_norm_eps at its default
                RMSNorm.build(D, 1e-6, dev) if config.use_qk_norm else None,
                torch.zeros((config.q_heads // tp_size,), dtype=torch.float32, device=dev)
                if config.use_attention_sinks else None,
                local_window_size=layer_window,  # context_length = window + 1 (:131), local_window_size = that - 1 (:660)
                num_heads=config.q_heads // tp_size, num_kv_heads=config.kv_heads // tp_size, head_dim=D, causal=True,
                use_fp8=use_fp8)
            mlp = SwiGLU(lin(width, H, "gate_proj", config.mlp_bias), lin(width, H, "up_proj", config.mlp_bias),
                         lin(H, width, "down_proj", config.mlp_bias))
            blocks.append(TransformerBlock(attn, mlp, RMSNorm.build(H, config.rms_eps, dev),
                                           RMSNorm.build(H, config.rms_eps, dev), num_heads=config.q_heads // tp_size,
                                           head_dim=D, causal=True, use_fp8=False))
        norm = RMSNorm.build(H, config.rms_eps, dev)
        head_w = _randn((config.vocab_size, H), std, gen, dev)
        lm_head = Linear(H, config.vocab_size, use_bias=False, weight=head_w)
        m = cls(embed, blocks, norm, lm_head, config)
        m.tp_rank, m.tp_size = tp_rank, tp_size
        return m

    tp_rank = 0
    tp_size = 1

    # -- reference API (one sequence) -------------------------------------------------------------
    def embed_tokens(self, tokens_t: torch.Tensor) -> torch.Tensor:
        """xax/arch/llm.py:205-211."""
        return ops.embed(tokens_t.to(torch.int32).reshape(-1), self.embed.weight)

    def get_logits(self, hidden_td: torch.Tensor) -> torch.Tensor:
        """xax/arch/llm.py:213-219."""
        return apply_linear(hidden_td, self.lm_head)

    def init_cache(self, max_len: int | None = None, dtype=BF16, batch: int | None = None):
        """xax/arch/llm.py:221-234."""
        return [b.init_cache(max_len=max_len, dtype=dtype, batch=batch) for b in self.blocks]

    def forward_hidden(self, tokens_t: torch.Tensor, context_tn=None, *, caches=None, donate: bool = True):
        """xax/arch/llm.py:252-285 for one sequence of token ids (T,)."""
        if tokens_t.dim() != 1:
            raise ValueError(f"expected rank 1 tokens, got rank {tokens_t.dim()}")
        bc = None
        if caches is not None:
            bc = [{"k": c["self_attn"]["k"].unsqueeze(0), "v": c["self_attn"]["v"].unsqueeze(0),
                   "position": c["self_attn"]["position"].reshape(1)} for c in caches]
        ctx = None if context_tn is None else context_tn.reshape(1, *context_tn.shape)
        x, nc = self.forward_hidden_batch(tokens_t.reshape(1, -1), ctx, caches=bc, donate=donate)
        x = x[0]
        if caches is None:
            return x
        return x, [{"self_attn": {"k": c["k"][0], "v": c["v"][0], "position": c["position"].reshape(())}} for c in nc]

    def forward(self, tokens_t: torch.Tensor, context_tn=None, *, caches=None, donate: bool = True):
        """xax/arch/llm.py:304-324."""
        if caches is None:
            return self.get_logits(self.forward_hidden(tokens_t, context_tn))
        x, caches = self.forward_hidden(tokens_t, context_tn, caches=caches, donate=donate)
        return self.get_logits(x), caches

    # -- batched entry points (B sequences, T new tokens each) -------------------------------------
    def forward_hidden_batch(self, tokens_bt: torch.Tensor, context_btn=None, *, caches=None, donate: bool = True,
                             workspace=None, tp=None, advance: bool = True):
        """tokens_bt: int32 [B, T]; caches: list of batched attention caches
        ({"k","v": [B, max_len, Hkv, D], "position": [B]}) or None.  Returns hidden [B, T, H]
        (after the final norm) and the updated caches.  ``tp`` (a parallel.TensorParallel) runs
        the blocks with this rank's weight shards and all-reduces the row-parallel outputs."""
        B, T = tokens_bt.shape
        x = ops.embed(tokens_bt.to(torch.int32).reshape(-1), self.embed.weight)
        if context_btn is not None:  # x = context + embedding, :274-275
            x = (context_btn.reshape(B * T, -1).to(BF16) + x).to(BF16)
        out_caches = []
        x_q = None  # (q, inv_scale) of attn_norm(x) when the previous block's closing exchange made it
        for i, block in enumerate(self.blocks):
            c = None if caches is None else caches[i]
            if tp is None:
                x, nc = block.forward_tokens(x, B, T, cache=c, donate=donate, workspace=workspace, advance=advance)
            else:
                nxt = self.blocks[i + 1].attn_norm if T == 1 and i + 1 < len(self.blocks) else None
                x, nc, x_q = tp.block_forward_chain(block, x, B, T, cache=c, workspace=workspace, advance=advance,
                                                    x_q=x_q, next_norm=nxt)
            out_caches.append(nc)
        y, _ = ops.rmsnorm(x, self.norm.weight_bf16(), self.norm.eps)
        return y.reshape(B, T, -1), (out_caches if caches is not None else None)

    def forward_batch(self, tokens_bt: torch.Tensor, *, caches=None, donate: bool = True, last_only: bool = False):
        """Logits [B, T, V] (or [B, 1, V] for the last position only) and updated caches."""
        h, caches = self.forward_hidden_batch(tokens_bt, caches=caches, donate=donate)
        if last_only:
            h = h[:, -1:, :].contiguous()
        return self.get_logits(h), caches


def _head_weight(lm_head) -> torch.Tensor:
    w = getattr(lm_head, "weight", None)
    if not isinstance(w, torch.Tensor) or w.dim() != 2 or isinstance(lm_head, Fp8Linear) or getattr(lm_head, "bias", None) is not None:
        raise ValueError("the fused loss takes the head as a layer with a bf16 (vocab, hidden) weight and no bias "
                         "(model.lm_head); an arbitrary callable is outside the path this library covers")
    return w.to(BF16)


def chunked_cross_entropy_loss(hidden_td: torch.Tensor, targets_t: torch.Tensor, lm_head, mask_t=None,
                               chunk_size: int = 1) -> torch.Tensor:
    """xax/arch/llm.py:718-788: mean cross-entropy over the valid positions, float32 scalar, without ever
    holding the (seq, vocab) logits: they are reduced to (max, sum-exp, target logit) inside the head GEMM's
    epilogue, 256 vocabulary columns at a time, so ``chunk_size`` (the reference's way of bounding memory) is
    accepted and not needed.  ``lm_head``: the model's head layer (the reference takes its ``__call__``)."""
    if hidden_td.dim() != 2:
        raise ValueError(f"expected rank 2 hidden states (seq, hidden_dim), got rank {hidden_td.dim()}")
    result, _, _ = ops.lm_head_cross_entropy(hidden_td.to(BF16).contiguous(), _head_weight(lm_head), targets_t, mask_t)
    return result[0]


def chunked_cross_entropy_acc(hidden_td: torch.Tensor, targets_t: torch.Tensor, lm_head, mask_t=None,
                              chunk_size: int = 1) -> torch.Tensor:
    """xax/arch/llm.py:791-887: fraction of valid positions whose arg-max logit is the target, float32 scalar."""
    if hidden_td.dim() != 2:
        raise ValueError(f"expected rank 2 hidden states (seq, hidden_dim), got rank {hidden_td.dim()}")
    result, _, _ = ops.lm_head_cross_entropy(hidden_td.to(BF16).contiguous(), _head_weight(lm_head), targets_t, mask_t)
    return result[1]


class CrossAttentionLLM:
    """xax/arch/llm.py:362-623: an LLM plus ONE cross-attention block (no RoPE, as many heads as the LLM has
    query heads) and its pre-norm, shared by all layers and applied after every transformer block, so that
    the decoder attends to an encoder's output (text embeddings while generating audio tokens, say)."""

    def __init__(self, llm: LLM, cross_attn, cross_attn_norm: RMSNorm, config: LLMConfig):
        self.llm, self.cross_attn, self.cross_attn_norm, self.config = llm, cross_attn, cross_attn_norm, config

    @classmethod
    def build(cls, config: LLMConfig, *, key=None, extra_tokens: int | None = None, **llm_kwargs) -> "CrossAttentionLLM":
        """:376-412.  ``llm_kwargs`` go to ``LLM.build`` (use_fp8, init_std, device)."""
        seed = int(key or 0) if not isinstance(key, torch.Generator) else int(key.initial_seed())
        llm = LLM.build(config, extra_tokens=extra_tokens, key=seed * 2 + 1, **llm_kwargs)
        return cls.from_llm(llm, key=seed * 2 + 2)

    @classmethod
    def from_llm(cls, llm: LLM, *, key=None) -> "CrossAttentionLLM":
        """:414-443: wrap an existing (possibly pretrained) LLM; the cross-attention starts from a fresh init."""
        from .attention import CrossAttentionBlock

        dev = llm.embed.weight.device
        cross = CrossAttentionBlock.build(llm.config.embed_dim, llm.config.q_heads, key=key,
                                          use_rotary_embeddings=False, device=dev)
        return cls(llm, cross, RMSNorm.build(llm.config.embed_dim, eps=llm.config.rms_eps, device=dev), llm.config)

    def init_cache(self, max_len: int | None = None, dtype=BF16, encoder_output_sn=None):
        """:445-470: (self-attention caches per layer, cross-attention cache or None)."""
        self_caches = self.llm.init_cache(max_len=max_len, dtype=dtype)
        cross_cache = None
        if encoder_output_sn is not None:
            cross_cache, _ = self.cross_attn.init_cache(kv_sn=encoder_output_sn)
        return self_caches, cross_cache

    def _cross(self, x, encoder_output_sn, cross_cache):
        y, _ = ops.rmsnorm(x, self.cross_attn_norm.weight_bf16(), self.cross_attn_norm.eps)
        out, new_cache, _ = self.cross_attn.forward(y, kv_sn=encoder_output_sn if cross_cache is None else None,
                                                    cache=cross_cache, residual=x)  # x + cross_out in the GEMM
        return out, new_cache

    def forward_hidden(self, tokens_t: torch.Tensor, *, encoder_output_sn=None, context_tn=None, caches=None,
                       cross_cache=None):
        """:502-560: hidden states (after the final norm); with ``caches`` also the updated self-attention caches
        and cross-attention cache.  Every layer's cross-attention call gets the cache that came IN (its position
        therefore advances by the number of new tokens once per call of this method, not once per layer)."""
        if tokens_t.dim() != 1:
            raise ValueError(f"expected rank 1 tokens, got rank {tokens_t.dim()}")
        x = self.llm.embed_tokens(tokens_t)
        if context_tn is not None:  # :529-530
            x = (context_tn.to(BF16) + x).to(BF16)
        if caches is None:
            for block in self.llm.blocks:
                x, _ = block.forward(x, cache=None)
                if encoder_output_sn is not None:
                    x, _ = self._cross(x, encoder_output_sn, None)
            return self.llm.norm(x)
        caches_out = []
        updated_cross = cross_cache
        for block, cache in zip(self.llm.blocks, caches, strict=True):
            x, cache = block.forward(x, cache=cache)
            caches_out.append(cache)
            if cross_cache is not None or encoder_output_sn is not None:
                x, updated_cross = self._cross(x, encoder_output_sn, cross_cache)
        return self.llm.norm(x), caches_out, updated_cross

    def forward(self, tokens_t: torch.Tensor, *, context_tn=None, encoder_output_sn=None, caches=None, cross_cache=None):
        """:594-623: logits, and with ``caches`` the updated caches."""
        if caches is None:
            x = self.forward_hidden(tokens_t, context_tn=context_tn, encoder_output_sn=encoder_output_sn)
            return apply_linear(x, self.llm.lm_head)
        x, caches_out, cross_out = self.forward_hidden(tokens_t, context_tn=context_tn, encoder_output_sn=encoder_output_sn,
                                                       caches=caches, cross_cache=cross_cache)
        return apply_linear(x, self.llm.lm_head), caches_out, cross_out


def tie_embedding_and_head(model: LLM) -> LLM:
    """xax/arch/llm.py:713-715: the returned model's lm_head shares the embedding array."""
    tied = LLM(model.embed, model.blocks, model.norm,
               Linear(model.config.embed_dim, model.config.vocab_size, use_bias=False, weight=model.embed.weight),
               model.config)
    tied.tp_rank, tied.tp_size = model.tp_rank, model.tp_size
    return tied


# ---------------------------------------------------------------------------------------
# tensor-parallel placement (xax/arch/llm.py:931-975)

_COLUMN = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj")
_ROW = ("o_proj", "down_proj")


def tp_shard_dim(weight_name: str, ndim: int) -> int | None:
    """Which dimension of an (out, in) weight is split across tensor-parallel ranks: 0 for
    column-parallel (q/k/v/gate/up and lm_head), 1 for row-parallel (o/down), None = replicated
    (1-D tensors, embeddings, norms)."""
    if ndim != 2:
        return None
    if any(weight_name.endswith(n) for n in _COLUMN):
        return 0
    if any(weight_name.endswith(n) for n in _ROW):
        return 1
    if "lm_head" in weight_name:
        return 0
    return None


def get_model_parallel_sharding_spec(weight_shape: tuple[int, ...], weight_name: str, mesh=None) -> tuple:
    """xax/arch/llm.py:931-975, returned as a PartitionSpec-like tuple: ("model", None),
    (None, "model") or ()."""
    dim = tp_shard_dim(weight_name, len(weight_shape))
    if dim is None:
        return ()
    return ("model", None) if dim == 0 else (None, "model")


# ---------------------------------------------------------------------------------------
# generation


class TokenSampler:
    """Next-token choice of the generation loop (xax/arch/llm.py:1446-1489 and :1547-1570): the
    allowed-token-range and minimum-length masks, then arg-max (``temperature <= 0``) or a draw from the
    top-p nucleus of softmax(logits / temperature).

    ``key`` seeds the draws: a ``torch.Generator`` on the logits' device, an int seed, or None (seed 0,
    as the reference defaults to ``jax.random.key(0)``); ``uniforms`` (float32 [steps, rows] or [steps])
    overrides it with explicit numbers in [0, 1), one per row and step.  The reference draws through
    jax.random.categorical from its own PRNG stream; the distribution is the same, the stream is not."""

    def __init__(self, temperature: float, top_p: float, key=None, *, eos_id: int = -1, allowed_token_range=None,
                 min_new_tokens_before_eos: int = 0, uniforms: torch.Tensor | None = None):
        if allowed_token_range is not None and allowed_token_range[1] <= allowed_token_range[0]:
            raise ValueError("allowed_token_range must satisfy max_id > min_id.")  # :1525-1526
        if min_new_tokens_before_eos < 0:
            raise ValueError("min_new_tokens_before_eos must be >= 0.")  # :1527-1528
        self.temperature, self.top_p, self.key = float(temperature), float(top_p), key
        self.eos_id, self.range, self.min_new = int(eos_id), allowed_token_range, int(min_new_tokens_before_eos)
        self.uniforms = uniforms
        self.generated = 0  # tokens drawn so far per sequence (the loop's generated_count)
        self._gen: torch.Generator | None = None

    def _draw(self, rows: int, device) -> torch.Tensor | None:
        if self.temperature <= 0:
            return None
        if self.uniforms is not None:
            u = self.uniforms[self.generated]
            return u.reshape(-1).expand(rows).to(device=device, dtype=torch.float32).contiguous()
        if self._gen is None:
            if isinstance(self.key, torch.Generator):
                self._gen = self.key
            else:
                self._gen = torch.Generator(device=device).manual_seed(int(self.key or 0))
        return torch.rand((rows,), generator=self._gen, device=device, dtype=torch.float32)

    def __call__(self, logits_bv: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        rows = logits_bv.shape[0]
        ops.sample_top_p(logits_bv, self.temperature, self.top_p, self._draw(rows, logits_bv.device),
                         allowed_token_range=self.range, eos_id=self.eos_id,
                         allow_eos=self.generated >= self.min_new, out=out)
        self.generated += 1
        return out


def llm_generate_jit(model: LLM, tokens_t: torch.Tensor, eos_id: int, max_new_tokens: int, context_tn=None,
                     temperature: float = 0.0, top_p: float = 1.0, key=None, allowed_token_range=None,
                     min_new_tokens_before_eos: int = 0):
    """xax/arch/llm.py:1492-1614: prefill, then one token per step until max_len or EOS.  Returns
    (tokens[max_len] int32, final_len).  ``key``: see TokenSampler."""
    if allowed_token_range is not None and allowed_token_range[1] <= allowed_token_range[0]:
        raise ValueError("allowed_token_range must satisfy max_id > min_id.")
    if min_new_tokens_before_eos < 0:
        raise ValueError("min_new_tokens_before_eos must be >= 0.")
    if context_tn is not None:
        raise NotImplementedError("context embeddings are not on the path this library covers")
    tokens_t = tokens_t.to(torch.int32)
    initial_len = tokens_t.shape[-1]
    if max_new_tokens <= 0:  # :1537-1538
        return tokens_t, initial_len
    sampler = None
    if temperature > 0 or allowed_token_range is not None or (eos_id >= 0 and min_new_tokens_before_eos > 0):
        sampler = TokenSampler(temperature, top_p, key, eos_id=eos_id, allowed_token_range=allowed_token_range,
                               min_new_tokens_before_eos=min_new_tokens_before_eos)
    out, lens = llm_generate_batch(model, tokens_t.reshape(1, -1), max_new_tokens, eos_id=eos_id, sampler=sampler)
    return out[0], int(lens[0])


def llm_generate(model: LLM, tokens: list[int], eos_id: int | None, max_new_tokens: int = 20, *, context_tn=None,
                 temperature: float = 0.7, top_p: float = 0.9, key=None) -> list[int]:
    """xax/arch/llm.py:1419-1443."""
    dev = model.embed.weight.device
    toks, n = llm_generate_jit(model, torch.tensor(tokens, dtype=torch.int32, device=dev),
                               eos_id if eos_id is not None else -1, max_new_tokens, context_tn, temperature, top_p, key)
    return toks[:n].tolist()


def llm_generate_stream(model: LLM, tokens: list[int], eos_id: int | None, max_new_tokens: int = 256, *,
                        context_tn=None, temperature: float = 0.7, top_p: float = 0.9, key=None):
    """xax/arch/llm.py:1617-1693: yields the generated tokens one at a time (the prompt is not yielded) and
    stops at EOS, which is not yielded either."""
    if context_tn is not None:
        raise NotImplementedError("context embeddings are not on the path this library covers")
    if max_new_tokens <= 0:
        return
    dev = model.embed.weight.device
    prompt = torch.tensor(tokens, dtype=torch.int32, device=dev).reshape(1, -1)
    st = DecodeState(model, 1, prompt.shape[1] + max_new_tokens, sampler=TokenSampler(temperature, top_p, key))
    tok = int(st.prefill(prompt).item())
    if eos_id is not None and tok == eos_id:
        return
    yield tok
    for _ in range(max_new_tokens - 1):
        tok = int(st.step().item())
        if eos_id is not None and tok == eos_id:
            return
        yield tok


class DecodeState:
    """Device buffers of a batched greedy decode: caches, the current token per sequence, and
    one decode step captured in a CUDA graph.  All layers append at the same position, so they
    share one position vector that is advanced once per step."""

    def __init__(self, model: LLM, batch: int, max_len: int, tp=None, sampler=None):
        """``sampler`` (a TokenSampler) replaces the arg-max; its state lives on the host, so a decode
        step with a sampler is not captured in a graph."""
        if sampler is not None and tp is not None:
            raise ValueError("sampling over a vocabulary-sharded lm_head is outside the path this library covers")
        self.model, self.B, self.max_len, self.tp, self.sampler = model, batch, max_len, tp, sampler
        dev = model.embed.weight.device
        self.caches = [c["self_attn"] for c in model.init_cache(max_len, batch=batch)]
        self.positions = self.caches[0]["position"]
        for c in self.caches:
            c["position"] = self.positions
        a = model.blocks[0].self_attn
        self.workspace = ops.attn_decode_workspace(batch, a.num_heads, a.head_dim, max_len, dev)
        self.cur = torch.zeros((batch,), dtype=torch.int32, device=dev)  # token fed to the next step
        self.graph = None

    def _next_tokens(self, hidden_bh: torch.Tensor, out: torch.Tensor) -> None:
        if self.sampler is not None:
            self.sampler(self.model.get_logits(hidden_bh), out)
        elif self.tp is None:
            ops.argmax(self.model.get_logits(hidden_bh), out=out)
        else:
            self.tp.greedy_tokens(self.model, hidden_bh, out)

    def prefill(self, tokens_bt: torch.Tensor, chunk: int | None = None) -> torch.Tensor:
        """Run the prompt through the model (sequences in chunks of ``chunk`` to bound the
        activation memory), fill the caches, return the first generated token per sequence."""
        B, T = tokens_bt.shape
        chunk = chunk or B
        if self.sampler is not None:
            chunk = B  # one draw per step for the whole batch
        for b0 in range(0, B, chunk):
            b1 = min(B, b0 + chunk)
            sub = [{"k": c["k"][b0:b1], "v": c["v"][b0:b1], "position": self.positions[b0:b1]} for c in self.caches]
            h, _ = self.model.forward_hidden_batch(tokens_bt[b0:b1], caches=sub, workspace=None, tp=self.tp,
                                                   advance=False)
            self._next_tokens(h[:, -1, :].contiguous(), self.cur[b0:b1])
        ops.advance_positions(self.positions, T)
        return self.cur

    def step(self) -> torch.Tensor:
        """One greedy decode step for all sequences: consumes self.cur, appends one row to every
        layer's cache, advances the positions, writes the next tokens into self.cur."""
        h, _ = self.model.forward_hidden_batch(self.cur.reshape(self.B, 1), caches=self.caches,
                                               workspace=self.workspace, tp=self.tp, advance=False)
        ops.advance_positions(self.positions, 1)
        self._next_tokens(h.reshape(self.B, -1), self.cur)
        return self.cur

    def capture(self) -> None:
        """Capture one decode step in a CUDA graph (positions and tokens live on the device,
        so the same graph serves every step).  A warm-up step runs first on a side stream; its
        effects (one cache row that the real step rewrites, the position advance, the token)
        are rolled back."""
        if self.sampler is not None:
            raise ValueError("a decode step with a sampler cannot be captured (its random numbers and EOS rule "
                             "change per step); call step()")
        saved_pos = self.positions.clone()
        saved_cur = self.cur.clone()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self.step()
        torch.cuda.current_stream().wait_stream(s)
        self.positions.copy_(saved_pos)
        self.cur.copy_(saved_cur)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.step()
        self.positions.copy_(saved_pos)
        self.cur.copy_(saved_cur)
        self.graph = g

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        return self.cur

    def step_host(self, tokens_in: torch.Tensor, tokens_out: torch.Tensor) -> torch.Tensor:
        """One decode step driven from the host: ``tokens_in`` (pinned host int32 [B], the token
        each sequence consumes) is copied to the device, the step runs (graph replay when
        captured), and the produced tokens are copied into ``tokens_out`` (pinned host int32 [B])
        and returned once they have arrived."""
        self.cur.copy_(tokens_in, non_blocking=True)
        if self.graph is not None:
            self.graph.replay()
        else:
            self.step()
        tokens_out.copy_(self.cur, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return tokens_out


def _sample_next_token(logits_tv: torch.Tensor, temperature: float, top_p: float, key=None, num_samples: int = 1):
    """xax/arch/llm.py:1446-1489: next token for every row of logits (tsz, vocab), shape (tsz, num_samples).
    ``temperature <= 0`` is the arg-max in float32 (first index on ties) whatever ``num_samples`` -- as in
    the reference, whose final ``where`` broadcasts it; otherwise every sample is a draw from the top-p
    nucleus.  ``key``: a torch.Generator on the logits' device, an int seed, None (seed 0), or a float32
    tensor of explicit uniforms [tsz, num_samples]."""
    if logits_tv.dtype != BF16:
        raise ValueError("the logits of this path are bf16 (they are compared and exponentiated as float32)")
    logits = logits_tv.reshape(-1, logits_tv.shape[-1]).contiguous()
    rows = logits.shape[0]
    cols = []
    if isinstance(key, torch.Tensor):
        u_all = key.to(device=logits.device, dtype=torch.float32).reshape(rows, num_samples)
    else:
        gen = key if isinstance(key, torch.Generator) else torch.Generator(device=logits.device).manual_seed(int(key or 0))
        u_all = torch.rand((rows, num_samples), generator=gen, device=logits.device, dtype=torch.float32)
    for j in range(num_samples):
        cols.append(ops.sample_top_p(logits, temperature, top_p, u_all[:, j].contiguous() if temperature > 0 else None))
    return torch.stack(cols, dim=-1).reshape(*logits_tv.shape[:-1], num_samples)


def llm_generate_batch(model: LLM, tokens_bt: torch.Tensor, max_new_tokens: int, *, eos_id: int = -1,
                       use_graph: bool = True, prefill_chunk: int | None = None, tp=None, sampler=None):
    """Batched generation: the loop of xax/arch/llm.py:1572-1613 for B prompts of equal length, greedy
    unless ``sampler`` (a TokenSampler) is given.  Returns (tokens [B, max_len] int32, final lengths [B])."""
    tokens_bt = tokens_bt.to(torch.int32)
    B, T0 = tokens_bt.shape
    max_len = T0 + max_new_tokens
    out = torch.zeros((B, max_len), dtype=torch.int32, device=tokens_bt.device)
    out[:, :T0] = tokens_bt
    if max_new_tokens <= 0:
        return out, torch.full((B,), T0, dtype=torch.int64)
    st = DecodeState(model, B, max_len, tp=tp, sampler=sampler)
    use_graph = use_graph and sampler is None
    first = st.prefill(tokens_bt, prefill_chunk)
    out[:, T0] = first
    if max_new_tokens > 1:
        if use_graph:
            st.capture()
        for i in range(1, max_new_tokens):
            nxt = st.replay() if use_graph else st.step()
            out[:, T0 + i] = nxt
    from .. import _lib

    _lib.device_status()
    lens = torch.full((B,), max_len, dtype=torch.int64)
    if eos_id >= 0:  # the reference stops a sequence at its first EOS: trim afterwards
        gen = out[:, T0:].cpu()
        for b in range(B):
            hit = (gen[b] == eos_id).nonzero()
            if hit.numel():
                lens[b] = T0 + int(hit[0]) + 1
                out[b, lens[b]:] = 0
    return out, lens
