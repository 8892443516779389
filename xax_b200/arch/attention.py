"""B200-native mirror of the hot-path modules of ``xax/arch/attention.py``.

Same class names, fields, ``build`` keyword arguments and call signatures as the reference
for: ``apply_linear``, ``RMSNorm``, ``SwiGLU``, ``RotaryEmbedding``, ``SelfAttentionBlock``,
``TransformerBlock`` and the cache dictionaries.  Arrays are torch CUDA tensors (bf16
activations); every computation is one of the library's sm_100a kernels.

The reference is unbatched and batches with ``jax.vmap``; here every module also has a
``*_batch`` entry that takes ``B`` sequences of ``T`` tokens at once -- numerically the
vmapped reference: per-token activation scales inside attention projections
(xax/arch/attention.py:279), per-sequence scales inside the SwiGLU (xax/arch/attention.py:55).

Caches are donated: ``forward(..., cache=c)`` appends into ``c``'s buffers and returns a
cache sharing them (the reference donates at its jit boundary, xax/arch/llm.py:1446).
Pass ``donate=False`` to copy first.  QK-norm, sliding windows and attention sinks are built.
Outside the path: LayerNorm / MLP feed-forward variants of the block.
"""

from __future__ import annotations

import math
import warnings
from typing import Literal, NotRequired, TypedDict

import torch

from .. import ops
from ..nn.fp8 import Fp8Linear, Fp8Scales, init_fp8_scales
from ..nn.lora import LoRALinear

BF16 = torch.bfloat16


class Linear:
    """Stand-in for ``eqx.nn.Linear``: weight (out_features, in_features), optional bias."""

    def __init__(self, in_features: int, out_features: int, use_bias: bool = True, *, key=None, weight=None, bias=None,
                 dtype=BF16, device=None):
        self.in_features, self.out_features, self.use_bias = in_features, out_features, use_bias
        if weight is None:
            gen = key if isinstance(key, torch.Generator) else torch.Generator(device="cpu").manual_seed(int(key or 0))
            lim = 1.0 / math.sqrt(in_features)
            dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
            weight = ((torch.rand((out_features, in_features), generator=gen) * 2 - 1) * lim).to(dtype).to(dev)
            bias = ((torch.rand((out_features,), generator=gen) * 2 - 1) * lim).to(dtype).to(dev) if use_bias else None
        self.weight, self.bias = weight, bias

    def __call__(self, x):
        return apply_linear(x, self)


class Embedding:
    """Stand-in for ``eqx.nn.Embedding``: weight (num_embeddings, embedding_size)."""

    def __init__(self, num_embeddings: int, embedding_size: int, *, key=None, weight=None, dtype=BF16, device=None):
        if weight is None:
            gen = key if isinstance(key, torch.Generator) else torch.Generator(device="cpu").manual_seed(int(key or 0))
            dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
            weight = torch.randn((num_embeddings, embedding_size), generator=gen).to(dtype).to(dev)
        self.weight = weight
        self.num_embeddings, self.embedding_size = weight.shape

    def __call__(self, token):
        return ops.embed(torch.as_tensor(token, dtype=torch.int32, device=self.weight.device).reshape(-1), self.weight)[0]


def _weights_key(*layers):
    """Identity of the weights (and biases) a stacked operand was built from: reassigning or updating
    one of them in place makes the stacked copy stale."""
    out = []
    for m in layers:
        wq = m.weight_q_current()[0] if isinstance(m, Fp8Linear) and m.use_fp8 else None  # (re)made if stale
        for t in (m.weight, m.bias, wq):
            out.append(None if t is None else (t.data_ptr(), t._version))
    return tuple(out)


def apply_linear(x: torch.Tensor, linear, *, residual: torch.Tensor | None = None) -> torch.Tensor:
    """xax/arch/attention.py:30-69: dispatch on the layer type.  An Fp8Linear is applied to the
    whole tensor at once (one activation scale, scales dropped).  A leading batch dimension
    (rank 3) reproduces the vmapped reference: one activation scale per sequence."""
    if isinstance(linear, LoRALinear):  # :44-51: the frozen layer plus the low-rank residual
        if residual is not None:
            raise ValueError("a LoRA layer does not take a fused residual")
        return linear(x)
    if isinstance(linear, Fp8Linear):
        if x.dim() == 3 and linear.use_fp8:
            B, T, _ = x.shape
            x2 = x.reshape(B * T, -1).to(BF16).contiguous()
            xq, _, x_inv, _ = ops.quantize_current(x2, T)
            res2 = None if residual is None else residual.reshape(B * T, -1)
            return linear.forward_quantized(xq, x_inv, res2).reshape(B, T, -1)
        return linear(x, residual=residual)[0]
    if isinstance(linear, Linear):
        x2 = x.reshape(-1, x.shape[-1]).to(BF16).contiguous()
        res2 = None if residual is None else residual.reshape(-1, linear.out_features)
        return ops.gemm_bf16(x2, linear.weight, None, None, linear.bias, res2).reshape(*x.shape[:-1], -1)
    if isinstance(linear, Embedding):
        x2 = x.reshape(-1, x.shape[-1]).to(BF16).contiguous()
        return ops.gemm_bf16(x2, linear.weight).reshape(*x.shape[:-1], -1)
    raise ValueError(f"Unsupported linear layer type: {type(linear)}")


def _apply_linear_batched(layer, x: torch.Tensor, scales=None, residual=None):
    """xax/arch/attention.py:244-287: the layer applied to every row of x on its own.  Current
    scaling: every row gets its own scale (:279).  Delayed scaling: all rows are cast with the
    incoming scales and the updated scales of the LAST row are returned (:273-275).  ``residual`` (not in
    the reference's signature) is added in the GEMM's epilogue."""
    if isinstance(layer, Fp8Linear):
        flat = x.reshape(-1, x.shape[-1])
        if scales is not None and layer.use_fp8:
            out, _ = layer(flat, scales, residual=residual)  # shared incoming scales: same bytes row by row
            _, new_scales = layer(flat[-1:], scales)  # history slot 0 <- amax of the last row
            return out.reshape(*x.shape[:-1], -1), new_scales
        out, _ = layer(flat, per_row=True, residual=residual)
        return out.reshape(*x.shape[:-1], -1), None
    return apply_linear(x, layer, residual=residual), None  # :286


class RMSNorm:
    """xax/arch/attention.py:72-98.  ``build`` makes a float32 weight of ones like the
    reference; the kernel runs in bf16, so the weight is cast to bf16 at use (exact for ones)."""

    def __init__(self, weight: torch.Tensor, eps: float = 1e-6):
        self.weight, self.eps = weight, eps
        self._w16 = None

    @classmethod
    def build(cls, dim: int, eps: float = 1e-6, device=None) -> "RMSNorm":
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        return cls(torch.ones((dim,), dtype=torch.float32, device=dev), eps)

    def weight_bf16(self) -> torch.Tensor:
        if self._w16 is None or self._w16.device != self.weight.device:
            self._w16 = self.weight.to(BF16).contiguous()
        return self._w16

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        x2 = x.reshape(-1, x.shape[-1]).to(BF16).contiguous()
        y, _ = ops.rmsnorm(x2, self.weight_bf16(), self.eps)
        return y.reshape(x.shape)


class SwiGLU:
    """xax/arch/attention.py:101-147: down(silu(gate(x)) * up(x)).  ``build`` uses plain
    linears like the reference (:138-140); pass ``use_fp8=True`` (an extension) or swap
    Fp8Linear instances into ``gate`` / ``up`` / ``down`` for the FP8 MLP."""

    def __init__(self, gate, up, down):
        self.gate, self.up, self.down = gate, up, down
        self._fused = None
        self._fused_key = None

    @classmethod
    def build(cls, embed_dim: int, hidden_dim: int | None = None, *, key=None, use_bias: bool = False,
              use_fp8: bool = False, device=None) -> "SwiGLU":
        if hidden_dim is None:
            hidden_dim = embed_dim * 4
        seed = int(key or 0) if not isinstance(key, torch.Generator) else int(key.initial_seed())
        if use_fp8:
            mk = lambda i, o, k: Fp8Linear(i, o, key=k, use_bias=use_bias, device=device)  # noqa: E731
        else:
            mk = lambda i, o, k: Linear(i, o, use_bias=use_bias, key=k, device=device)  # noqa: E731
        return cls(mk(embed_dim, hidden_dim, seed + 1), mk(embed_dim, hidden_dim, seed + 2),
                   mk(hidden_dim, embed_dim, seed + 3))

    def is_fp8(self) -> bool:
        return all(isinstance(m, Fp8Linear) and m.use_fp8 for m in (self.gate, self.up, self.down))

    def fused_gate_up(self):
        """gate | up weights stacked into one [2F, H] operand so one GEMM reads x once."""
        key = _weights_key(self.gate, self.up)
        if self._fused is not None and self._fused_key != key:
            self._fused = None
        self._fused_key = key
        if self._fused is None:
            if self.is_fp8():
                gq, g_inv = self.gate.weight_q_current()
                uq, u_inv = self.up.weight_q_current()
                F = gq.shape[0]
                wq = torch.cat([gq.view(torch.uint8), uq.view(torch.uint8)], 0).view(torch.float8_e4m3fn)
                col = torch.cat([g_inv.expand(F), u_inv.expand(F)]).contiguous()
            else:
                wq = torch.cat([self.gate.weight, self.up.weight], 0).contiguous()
                col = None
            biases = [self.gate.bias, self.up.bias]
            bias = None if biases[0] is None else torch.cat(biases).contiguous()
            self._fused = (wq, col, bias)
        return self._fused

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if x.dim() not in (2, 3):
            raise ValueError(f"SwiGLU expects rank 2 or 3 input, got rank {x.dim()}")
        B, T = (1, x.shape[0]) if x.dim() == 2 else x.shape[:2]
        x2 = x.reshape(B * T, -1).to(BF16).contiguous()
        return self.forward_tokens(x2, B, T).reshape(x.shape)

    def forward_tokens(self, y: torch.Tensor, B: int, T: int, *, residual=None, y_q=None) -> torch.Tensor:
        """y: normalised activations [B*T, H].  One activation scale per sequence (T rows).
        ``y_q`` = (q, inv_scale) when the preceding RMSNorm already cast y."""
        wq, col, bias = self.fused_gate_up()
        F = self.gate.out_features
        if self.is_fp8():
            if y_q is None:
                q, _, inv, _ = ops.quantize_current(y, T)
            else:
                q, inv = y_q
            gu = ops.gemm_fp8(q, wq, inv, col, bias)
            if T == 1:
                _, (hq, _, h_inv) = ops.silu_mul(gu, F, want_h=False, quantize=True)
            else:
                amax = torch.zeros((B,), dtype=torch.float32, device=y.device)
                h, _ = ops.silu_mul(gu, F, group_amax=amax, group_rows=T)
                hq, _, h_inv = ops.quantize_with_amax(h, amax, T)
            return self.down.forward_quantized(hq, h_inv, residual)
        gu = ops.gemm_bf16(y, wq, None, None, bias)
        h, _ = ops.silu_mul(gu, F)
        return apply_linear(h, self.down, residual=residual)


def can_use_cudnn_attention(dtype, head_dim: int, seq_len: int, has_bias: bool = False) -> bool:
    """xax/arch/attention.py:150-179 (kept for API compatibility; this library never calls cuDNN)."""
    return dtype in (torch.float16, torch.bfloat16) and head_dim <= 128 and head_dim % 8 == 0 and seq_len % 64 == 0 \
        and not has_bias


class AttentionCache(TypedDict):
    k: torch.Tensor
    v: torch.Tensor
    position: torch.Tensor


class Fp8ScalesCache(TypedDict):
    q_proj: NotRequired[Fp8Scales]
    k_proj: NotRequired[Fp8Scales]
    v_proj: NotRequired[Fp8Scales]
    output_proj: NotRequired[Fp8Scales]


class TransformerBlockCache(TypedDict):
    self_attn: AttentionCache
    self_attn_fp8: NotRequired[Fp8ScalesCache]


def _make_linear(in_features, out_features, key, use_bias=True, use_fp8=False, compute_dtype=BF16, device=None):
    """xax/arch/attention.py:212-241 (an FP8 layer always gets a bias, like the reference)."""
    if use_fp8:
        return Fp8Linear(in_features, out_features, key=key, use_fp8=True, compute_dtype=compute_dtype, device=device)
    return Linear(in_features, out_features, use_bias=use_bias, key=key, device=device)


def _init_fp8_scales_cache(history_length: int) -> Fp8ScalesCache:
    """xax/arch/attention.py:290-304."""
    return {k: init_fp8_scales(history_length) for k in ("q_proj", "k_proj", "v_proj", "output_proj")}


RotaryEmbeddingStyle = Literal["concatenated", "interleaved"]


class RotaryEmbedding:
    """xax/arch/attention.py:310-526.  The kernels implement the "concatenated" (LLaMA) style
    that the LLM builds (xax/arch/llm.py:134) from cos/sin tables computed in the reference's
    op order and dtype (bf16 frequencies, positions and angles)."""

    def __init__(self, head_dim: int, base: float = 10000.0, style: RotaryEmbeddingStyle = "interleaved",
                 factor: float = 1.0, original_max_position_embeddings: int | None = None, beta_slow: float = 1.0,
                 beta_fast: float = 32.0):
        self.head_dim, self.base, self.style, self.factor = head_dim, base, style, factor
        self.original_max_position_embeddings = original_max_position_embeddings
        self.beta_slow, self.beta_fast = beta_slow, beta_fast
        self._tables: dict = {}

    @classmethod
    def build(cls, head_dim, base=10000.0, style="interleaved", factor=1.0, original_max_position_embeddings=None,
              beta_slow=1.0, beta_fast=32.0) -> "RotaryEmbedding":
        return cls(head_dim, base, style, factor, original_max_position_embeddings, beta_slow, beta_fast)

    @property
    def uses_yarn(self) -> bool:
        return self.factor > 1.0 and self.original_max_position_embeddings is not None

    def tables(self, length: int, device, any_style: bool = False):
        """(cos, sin) bf16 [>= length, head_dim / 2] on ``device`` (cached, grown on demand)."""
        if self.style != "concatenated" and not any_style:
            raise ValueError("the attention kernels implement the 'concatenated' RoPE style only")
        key = str(device)
        cur = self._tables.get(key)
        if cur is None or cur[0].shape[0] < length:
            n = max(length, 256)
            if self.uses_yarn:  # :401-441: interpolated frequencies, float32, attention scaling folded in
                cur = ops.rope_tables_yarn(self.head_dim, self.base, self.factor, self.original_max_position_embeddings,
                                           self.beta_slow, self.beta_fast, n, device)
            else:
                cur = ops.rope_tables(self.head_dim, self.base, n, device)
            self._tables[key] = cur
        return cur


    def _get_rotary_embeddings(self, positions: torch.Tensor, dtype=BF16):
        """xax/arch/attention.py:374-399: (cos, sin) [n, head_dim / 2] for integer positions [n]
        (rows of the table, which is built in the reference's bf16 op order)."""
        if dtype != BF16:
            raise ValueError("the tables are built for bf16 activations (the compute dtype of this path)")
        pos = positions.reshape(-1).to(torch.int64)
        n = int(pos.max().item()) + 1 if pos.numel() else 1
        cos, sin = self.tables(n, positions.device, any_style=True)
        return cos.index_select(0, pos), sin.index_select(0, pos)

    def apply_rotary_embeddings(self, x: torch.Tensor, positions: torch.Tensor | None = None) -> torch.Tensor:
        """xax/arch/attention.py:443-483: x (seq_len, heads, head_dim) or (batch, seq_len, heads,
        head_dim); positions (seq_len,) / (batch, seq_len) integers, default 0 .. seq_len-1."""
        if x.dim() == 4:
            bsz, seq_len = x.shape[:2]
            if positions is None:
                positions = torch.arange(seq_len, device=x.device, dtype=torch.int32)[None, :].expand(bsz, seq_len)
            return self._apply_rotary_4d(x, positions)
        if x.dim() != 3:
            raise ValueError(f"expected a 3-D or 4-D tensor, got shape {tuple(x.shape)}")
        seq_len, _, head_dim = x.shape
        assert head_dim == self.head_dim, f"Expected head_dim {self.head_dim}, got {head_dim}"  # :468
        if self.style not in ("concatenated", "interleaved"):
            raise ValueError(f"Unknown RoPE style: {self.style}. Use 'concatenated' or 'interleaved'.")  # :483
        if positions is None:
            positions = torch.arange(seq_len, device=x.device, dtype=torch.int32)
        pos = positions.reshape(-1).to(torch.int32).contiguous()
        n = int(pos.max().item()) + 1 if pos.numel() else 1
        cos, sin = self.tables(n, x.device, any_style=True)
        return ops.rope_apply(x.to(BF16).contiguous(), pos, cos, sin, interleaved=self.style == "interleaved")

    def _apply_rotary_4d(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """xax/arch/attention.py:485-508."""
        bsz, seq_len, heads, head_dim = x.shape
        assert head_dim == self.head_dim  # :488
        out = self.apply_rotary_embeddings(x.reshape(bsz * seq_len, heads, head_dim), positions.reshape(-1))
        return out.reshape(bsz, seq_len, heads, head_dim)


class SelfAttentionBlock:
    """xax/arch/attention.py:529-980 restricted to causal GQA self-attention with optional RoPE
    and a KV cache."""

    def __init__(self, q_proj, k_proj, v_proj, output_proj, rotary_emb, q_norm=None, k_norm=None, sinks=None, *,
                 num_heads: int, num_kv_heads: int, head_dim: int, causal: bool, local_window_size: int | None = None,
                 use_fp8: bool = False):
        # Attention sinks: the reference adds them to the logits as a bias of shape (1, heads, 1)
        # (:745-748, :893-896) -- one constant per head over all keys, which a softmax over keys
        # cancels.  They are kept (float32 [heads], zeros at build :652-654; no loader fills them) and
        # the kernels need nothing for them.
        self.q_proj, self.k_proj, self.v_proj, self.output_proj = q_proj, k_proj, v_proj, output_proj
        self.rotary_emb, self.q_norm, self.k_norm, self.sinks = rotary_emb, q_norm, k_norm, sinks
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.causal, self.local_window_size, self.use_fp8 = causal, local_window_size, use_fp8
        self._fused = None
        self._fused_key = None

    @classmethod
    def build(cls, embed_dim: int, num_heads: int, *, key=None, num_kv_heads: int | None = None,
              head_dim: int | None = None, use_bias: bool = True, causal: bool = False,
              context_length: int | None = None, use_rotary_embeddings: bool = False, rotary_base: float = 10000.0,
              rotary_style: RotaryEmbeddingStyle = "concatenated", rotary_factor: float = 1.0,
              rotary_original_max_position_embeddings: int | None = None, rotary_beta_slow: float = 1.0,
              rotary_beta_fast: float = 32.0, use_qk_norm: bool = False, qk_norm_eps: float = 1e-6,
              use_attention_sinks: bool = False, use_fp8: bool = False, compute_dtype=BF16,
              device=None) -> "SelfAttentionBlock":
        sinks = torch.zeros((num_heads,), dtype=torch.float32, device=device) if use_attention_sinks else None  # :652-654
        kv = num_kv_heads if num_kv_heads is not None else num_heads
        hd = head_dim if head_dim is not None else embed_dim // num_heads
        assert num_heads % kv == 0, "num_heads must be divisible by num_kv_heads"  # :620
        seed = int(key or 0) if not isinstance(key, torch.Generator) else int(key.initial_seed())
        qd, kd = num_heads * hd, kv * hd
        mk = lambda i, o, k: _make_linear(i, o, k, use_bias, use_fp8, compute_dtype, device)  # noqa: E731
        rope = RotaryEmbedding.build(hd, rotary_base, rotary_style, rotary_factor,
                                     rotary_original_max_position_embeddings, rotary_beta_slow,
                                     rotary_beta_fast) if use_rotary_embeddings else None
        qn = RMSNorm.build(hd, qk_norm_eps, device) if use_qk_norm else None  # :665-669
        kn = RMSNorm.build(hd, qk_norm_eps, device) if use_qk_norm else None
        return cls(mk(embed_dim, qd, seed + 1), mk(embed_dim, kd, seed + 2), mk(embed_dim, kd, seed + 3),
                   mk(qd, embed_dim, seed + 4), rope, qn, kn, sinks, num_heads=num_heads, num_kv_heads=kv, head_dim=hd,
                   causal=causal, local_window_size=None if context_length is None else context_length - 1,  # :660
                   use_fp8=use_fp8)

    @property
    def embed_dim(self) -> int:
        return self.head_dim * self.num_heads

    def _is_fp8(self) -> bool:
        return all(isinstance(m, Fp8Linear) and m.use_fp8 for m in (self.q_proj, self.k_proj, self.v_proj))

    def fused_qkv(self):
        """q | k | v weights stacked into one [(Hq + 2 Hkv) D, H] operand; per-column
        dequantisation multipliers keep each projection's own weight scale."""
        key = _weights_key(self.q_proj, self.k_proj, self.v_proj)
        if self._fused is not None and self._fused_key != key:
            self._fused = None
        self._fused_key = key
        if self._fused is None:
            projs = (self.q_proj, self.k_proj, self.v_proj)
            if self._is_fp8():
                qs = [p.weight_q_current() for p in projs]
                wq = torch.cat([q.view(torch.uint8) for q, _ in qs], 0).view(torch.float8_e4m3fn)
                col = torch.cat([inv.expand(q.shape[0]) for q, inv in qs]).contiguous()
            else:
                wq = torch.cat([p.weight for p in projs], 0).contiguous()
                col = None
            if all(p.bias is None for p in projs):
                bias = None
            else:
                bias = torch.cat([p.bias if p.bias is not None else
                                  torch.zeros((p.out_features,), dtype=BF16, device=p.weight.device)
                                  for p in projs]).contiguous()
            self._fused = (wq, col, bias)
        return self._fused

    def init_cache(self, max_len: int | None = None, dtype=None, batch: int | None = None, device=None) -> AttentionCache:
        """xax/arch/attention.py:775-794; ``batch`` adds a leading sequence dimension."""
        if max_len is None:
            max_len = self.local_window_size
        if max_len is None:
            raise ValueError("context_length or max_len must be set for caching")
        if dtype not in (None, BF16):
            raise ValueError("the KV cache is bfloat16")
        dev = self.q_proj.weight.device if device is None else device
        lead = () if batch is None else (batch,)
        shape = (*lead, max_len, self.num_kv_heads, self.head_dim)
        return {"k": torch.zeros(shape, dtype=BF16, device=dev), "v": torch.zeros(shape, dtype=BF16, device=dev),
                "position": torch.zeros(lead, dtype=torch.int32, device=dev)}

    def init_mask(self, seq_len: int, add_cache: bool = False, batch_dim: bool = False) -> torch.Tensor:
        """xax/arch/attention.py:796-824 (boolean mask; informational -- the kernels mask by position)."""
        if add_cache:
            raise ValueError("local_window_size must be set for caching")
        mask = torch.tril(torch.ones((seq_len, seq_len), dtype=torch.bool))
        return mask.reshape(1, 1, seq_len, seq_len) if batch_dim else mask

    # -- forward --------------------------------------------------------------------------------
    def forward(self, x_tn: torch.Tensor, *, mask=None, cache: AttentionCache | None = None, fp8_scales=None,
                donate: bool = True):
        """xax/arch/attention.py:826-980 for one sequence (T, H)."""
        if x_tn.dim() != 2:
            raise ValueError(f"expected rank 2 input, got rank {x_tn.dim()}")
        if mask is not None:
            self._require_builtin_mask(mask, x_tn.shape[0], cache)
        if fp8_scales is not None:
            raise ValueError("delayed scaling through the attention block is undefined in the reference "
                             "(its Fp8Scales is not a pytree); call Fp8Linear directly with scales")
        bc = None
        if cache is not None:
            bc = {"k": cache["k"].unsqueeze(0), "v": cache["v"].unsqueeze(0), "position": cache["position"].reshape(1)}
        out, nc = self.forward_tokens(x_tn, 1, x_tn.shape[0], cache=bc, donate=donate)
        return out, {"k": nc["k"][0], "v": nc["v"][0], "position": nc["position"].reshape(())}, None

    def _require_builtin_mask(self, mask: torch.Tensor, T: int, cache) -> None:
        """The reference hands an explicit mask to dot_product_attention in place of every built-in rule
        (xax/arch/attention.py:907-909).  The kernels mask by position, so an explicit mask is accepted when
        it is the mask they apply anyway -- filled cache rows that are causal for the query and inside the
        window, (T, max_len) with a cache and (T, T) without (any leading singleton dimensions) -- and
        refused otherwise."""
        if not self.causal:
            raise ValueError("the attention kernels are causal")
        start = int(cache["position"]) if cache is not None else 0
        S = cache["k"].shape[-3] if cache is not None else T
        if mask.numel() != T * S:
            raise ValueError(f"mask has {mask.numel()} elements, expected ({T}, {S})")
        qpos = torch.arange(T, device=mask.device)[:, None] + start
        kpos = torch.arange(S, device=mask.device)[None, :]
        want = kpos <= qpos
        if self.local_window_size is not None:
            want &= kpos >= qpos - self.local_window_size
        if not torch.equal(mask.reshape(T, S).to(torch.bool), want):
            raise ValueError("explicit masks other than the causal (and sliding-window) mask the kernels apply are "
                             "outside the path this library covers")

    def __call__(self, x_btd: torch.Tensor, positions_bt: torch.Tensor | None = None, *, key=None,
                 inference: bool = True) -> torch.Tensor:
        """xax/arch/attention.py:700-773: batched self-attention without a cache.  As there, every projection
        goes through ``apply_linear`` on the whole (batch, seq, dim) tensor -- an FP8 layer therefore uses ONE
        activation scale for the whole batch (:52-58) -- RoPE takes explicit positions (default 0 .. seq-1) and
        the causal mask goes by token index, not by position.  ``key`` and ``inference`` are unused, as in
        the reference."""
        if x_btd.dim() != 3:
            raise ValueError(f"expected rank 3 input (batch, seq_len, embed_dim), got rank {x_btd.dim()}")
        if not self.causal:
            raise ValueError("the attention kernels are causal")
        B, T, _ = x_btd.shape
        Hq, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        x2 = x_btd.reshape(B * T, -1).to(BF16).contiguous()
        projs = (self.q_proj, self.k_proj, self.v_proj)
        if self._is_fp8():  # the three layers quantise the same tensor the same way: do it once
            xq, _, x_inv, _ = ops.quantize_current(x2, B * T)
            q, k, v = (p.forward_quantized(xq, x_inv) for p in projs)
        else:
            q, k, v = (apply_linear(x2, p) for p in projs)
        if self.q_norm is not None:  # :739-742, per head
            q = self.q_norm(q.reshape(B * T * Hq, D)).reshape(B * T, Hq * D)
        if self.k_norm is not None:
            k = self.k_norm(k.reshape(B * T * Hkv, D)).reshape(B * T, Hkv * D)
        if self.rotary_emb is not None:  # :745-747
            if positions_bt is None:
                positions_bt = torch.arange(T, device=x2.device, dtype=torch.int32)[None, :].expand(B, T)
            pos = positions_bt.to(torch.int32).contiguous()
            q = self.rotary_emb.apply_rotary_embeddings(q.reshape(B, T, Hq, D), pos)
            k = self.rotary_emb.apply_rotary_embeddings(k.reshape(B, T, Hkv, D), pos)
        # the new keys and values ARE a cache of T rows per sequence whose queries start at row 0
        q3 = q.reshape(B * T, Hq, D).contiguous()
        kc, vc = k.reshape(B, T, Hkv, D).contiguous(), v.reshape(B, T, Hkv, D).contiguous()
        zero = torch.zeros((B,), dtype=torch.int32, device=x2.device)
        scale = 1.0 / math.sqrt(D)
        if self.local_window_size:  # :765 (a window of 0 counts as "none" there)
            ctx = ops.attn_prefill_window(q3, kc, vc, zero, B, T, self.local_window_size, scale=scale)
        else:
            ctx = ops.attn_prefill(q3, kc, vc, zero, B, T, scale=scale)
        out = apply_linear(ctx.reshape(B * T, Hq * D), self.output_proj)
        return out.reshape(B, T, -1)

    def forward_tokens(self, y: torch.Tensor, B: int, T: int, *, cache=None, donate: bool = True, y_q=None,
                       residual=None, workspace=None, advance: bool = True, reduce_amax=None, out=None,
                       peer_site=None):
        """y: [B*T, H] (normalised) activations of B sequences, T new tokens each.  Returns
        (attention output [B*T, H] (+ residual), updated batched cache).  ``advance=False``
        leaves cache["position"] untouched (a caller sharing one position vector between layers
        advances it once per step).  ``reduce_amax`` (tensor-parallel runs) is applied to the
        per-token amax of the row-parallel output projection's input; ``out`` is where the output
        projection writes (a buffer the other ranks can read, in tensor-parallel runs);
        ``peer_site`` routes the amax exchange of a decode step through peer memory, inside the
        attention merge pass (ops.attn_decode_cast_tp), instead of ``reduce_amax``."""
        if not self.causal:
            raise ValueError("the attention kernels are causal")
        Hq, Hkv, D = self.num_heads, self.num_kv_heads, self.head_dim
        dev = y.device
        if cache is None:  # no cache given: attend within the T new tokens, scratch cache
            cache = self.init_cache(T, batch=B, device=dev)
        elif not donate:
            cache = {"k": cache["k"].clone(), "v": cache["v"].clone(), "position": cache["position"].clone()}
        max_len = cache["k"].shape[1]
        wq, col, bias = self.fused_qkv()
        if self._is_fp8():  # per-token activation scales (vmapped layer, :279)
            if y_q is None:
                q, _, inv, _ = ops.quantize_current(y.to(BF16).contiguous(), 1)
            else:
                q, inv = y_q
            qkv = ops.gemm_fp8(q, wq, inv, col, bias)
        else:
            qkv = ops.gemm_bf16(y.to(BF16).contiguous(), wq, None, None, bias)
        if self.rotary_emb is None:
            raise ValueError("the attention kernels expect rotary embeddings (as the LLM builds them)")
        if self.q_norm is not None or self.k_norm is not None:  # QK-norm before RoPE (:864-867)
            nq, nk = self.q_norm, self.k_norm
            eps = (nq if nq is not None else nk).eps
            if nq is not None and nk is not None and nq.eps != nk.eps:
                raise ValueError("q_norm and k_norm must share one eps")
            ops.qk_norm(qkv, Hq, Hkv, D, None if nq is None else nq.weight_bf16(),
                        None if nk is None else nk.weight_bf16(), eps)
        cos, sin = self.rotary_emb.tables(max_len, dev)
        pos = cache["position"]
        scale = 1.0 / math.sqrt(D)
        op = self.output_proj
        op_fp8 = isinstance(op, Fp8Linear) and op.use_fp8
        win = self.local_window_size
        fits_cast = T == 1 and op_fp8 and win is None and Hq <= 64 and Hq * D <= 4096
        if T == 1 and D in (64, 128):
            # decode: RoPE, cache append, attention (and, where it fits, the per-token cast of its output with
            # the amax exchange over ranks) are one attention launch + one merge launch
            use_cast = fits_cast and (peer_site is not None or reduce_amax is None)
            attn, aq, _, a_inv = ops.attn_decode_append(qkv, cache["k"], cache["v"], pos, cos, sin, Hq, scale=scale,
                                                        window=win, want_out=not use_cast, cast=use_cast,
                                                        peer=peer_site if use_cast else None, workspace=workspace)
            if not use_cast:
                attn2 = attn.reshape(B, Hq * D)
                if op_fp8:
                    if reduce_amax is None:
                        aq, _, a_inv, _ = ops.quantize_current(attn2, 1)
                    else:
                        amax = ops.group_amax(attn2, 1)
                        reduce_amax(amax)
                        aq, _, a_inv = ops.quantize_with_amax(attn2, amax, 1)
            if op_fp8:
                out = op.forward_quantized(aq, a_inv, residual, out)
            else:
                out = apply_linear(attn2, op, residual=residual)
            if advance:
                ops.advance_positions(pos, T)  # new_position = p + seq_len (:888), on the device
            return out, {"k": cache["k"], "v": cache["v"], "position": pos}
        q_rot = ops.kv_append_rope(qkv, B, T, Hq, Hkv, D, pos, cos, sin, cache["k"], cache["v"])
        if fits_cast and peer_site is not None:
            aq, _, a_inv = ops.attn_decode_cast_tp(q_rot, cache["k"], cache["v"], pos, peer_site, scale=scale,
                                                   workspace=workspace)
            out = op.forward_quantized(aq, a_inv, residual, out)
            if advance:
                ops.advance_positions(pos, T)
            return out, {"k": cache["k"], "v": cache["v"], "position": pos}
        if fits_cast and reduce_amax is None:
            # decode: the per-token cast of the attention output happens inside the merge pass
            _, aq, _, a_inv = ops.attn_decode_cast(q_rot, cache["k"], cache["v"], pos, scale=scale, workspace=workspace)
            out = op.forward_quantized(aq, a_inv, residual, out)
            if advance:
                ops.advance_positions(pos, T)
            return out, {"k": cache["k"], "v": cache["v"], "position": pos}
        if win is not None:  # sliding window (:931-936): a query sees keys q - window .. q
            attn = (ops.attn_decode_window(q_rot, cache["k"], cache["v"], pos, win, scale=scale, workspace=workspace)
                    if T == 1 else ops.attn_prefill_window(q_rot, cache["k"], cache["v"], pos, B, T, win, scale=scale))
        elif T == 1:
            attn = ops.attn_decode(q_rot, cache["k"], cache["v"], pos, scale=scale, workspace=workspace)
        else:
            attn = ops.attn_prefill(q_rot, cache["k"], cache["v"], pos, B, T, scale=scale)
        attn2 = attn.reshape(B * T, Hq * D)
        if op_fp8:
            if reduce_amax is None:
                aq, _, a_inv, _ = ops.quantize_current(attn2, 1)
            else:
                amax = ops.group_amax(attn2, 1)
                reduce_amax(amax)
                aq, _, a_inv = ops.quantize_with_amax(attn2, amax, 1)
            out = op.forward_quantized(aq, a_inv, residual, out)
        else:
            out = apply_linear(attn2, op, residual=residual)
        if advance:
            ops.advance_positions(pos, T)  # new_position = p + seq_len (:888), on the device
        new_cache = {"k": cache["k"], "v": cache["v"], "position": pos}
        return out, new_cache


class CrossAttentionBlock:
    """xax/arch/attention.py:983-1205: queries from the decoder stream, keys and values from a context
    sequence; every query sees every context token (``is_causal=False``), as many kv heads as query heads.
    The cache holds the projected (and, with RoPE, rotated) context once; ``forward`` then only projects
    the queries.  Attention runs on the prefill kernel with its causal mask switched off
    (``ops.attn_cross``)."""

    def __init__(self, q_proj, k_proj, v_proj, output_proj, *, num_heads: int, head_dim: int, use_fp8: bool = False,
                 rotary_emb: RotaryEmbedding | None = None):
        self.q_proj, self.k_proj, self.v_proj, self.output_proj = q_proj, k_proj, v_proj, output_proj
        self.num_heads, self.head_dim, self.use_fp8, self.rotary_emb = num_heads, head_dim, use_fp8, rotary_emb

    @classmethod
    def build(cls, embed_dim: int, num_heads: int, *, key=None, use_rotary_embeddings: bool = False,
              rotary_base: float = 10000.0, use_fp8: bool = False, compute_dtype=BF16, device=None) -> "CrossAttentionBlock":
        """Same keyword arguments as the reference (:995-1047).  RoPE, when asked for, has the class default
        style of ``RotaryEmbedding.build`` ("interleaved"), as there (:1035)."""
        head_dim = embed_dim // num_heads
        assert head_dim * num_heads == embed_dim, "embed_dim must be divisible by num_heads"  # :1025
        seed = int(key or 0) if not isinstance(key, torch.Generator) else int(key.initial_seed())
        projs = [_make_linear(embed_dim, embed_dim, seed * 4 + i, use_fp8=use_fp8, compute_dtype=compute_dtype,
                              device=device) for i in range(4)]
        rotary = RotaryEmbedding.build(head_dim=head_dim, base=rotary_base) if use_rotary_embeddings else None
        return cls(*projs, num_heads=num_heads, head_dim=head_dim, use_fp8=use_fp8, rotary_emb=rotary)

    def _project_kv(self, kv_sn: torch.Tensor, fp8_scales):
        if kv_sn.dim() != 2:
            raise ValueError(f"expected rank 2 context (kv_seq_len, embed_dim), got rank {kv_sn.dim()}")
        S = kv_sn.shape[0]
        x = kv_sn.to(BF16).contiguous()
        k, new_k = _apply_linear_batched(self.k_proj, x, fp8_scales.get("k_proj") if fp8_scales else None)
        v, new_v = _apply_linear_batched(self.v_proj, x, fp8_scales.get("v_proj") if fp8_scales else None)
        k = k.reshape(S, self.num_heads, self.head_dim)
        v = v.reshape(S, self.num_heads, self.head_dim).contiguous()
        if self.rotary_emb is not None:  # :1090-1093: the context's positions are fixed, K is stored rotated
            k = self.rotary_emb.apply_rotary_embeddings(k, torch.arange(S, device=x.device, dtype=torch.int32))
        return k.contiguous(), v, new_k, new_v

    def init_cache(self, kv_sn: torch.Tensor, fp8_scales=None):
        """:1062-1108.  Returns (cache, updated FP8 scales or None)."""
        k, v, new_k, new_v = self._project_kv(kv_sn, fp8_scales)
        updated = None
        if fp8_scales is not None and self.use_fp8:
            updated = dict(fp8_scales)
            if new_k is not None:
                updated["k_proj"] = new_k
            if new_v is not None:
                updated["v_proj"] = new_v
        return {"k": k, "v": v, "position": torch.zeros((), dtype=torch.int32, device=k.device)}, updated

    def forward(self, q_tn: torch.Tensor, *, kv_sn=None, cache=None, fp8_scales=None, residual=None):
        """:1110-1205: (output (q_seq_len, embed_dim), cache, updated FP8 scales or None).  ``residual`` (an
        extension) is added to the output inside the output projection's GEMM."""
        if q_tn.dim() != 2:
            raise ValueError(f"expected rank 2 input (q_seq_len, embed_dim), got rank {q_tn.dim()}")
        T = q_tn.shape[0]
        H, D = self.num_heads, self.head_dim
        q, new_q = _apply_linear_batched(self.q_proj, q_tn.to(BF16).contiguous(),
                                         fp8_scales.get("q_proj") if fp8_scales else None)
        q = q.reshape(T, H, D)
        new_k = new_v = None
        if cache is not None:  # :1146-1149
            k, v, start = cache["k"], cache["v"], cache["position"]
        elif kv_sn is not None:  # :1150-1167
            k, v, new_k, new_v = self._project_kv(kv_sn, fp8_scales)
            start = torch.zeros((), dtype=torch.int32, device=q.device)
        else:
            raise ValueError("Either `cache` or `kv_sn` must be provided.")  # :1169
        if self.rotary_emb is not None:  # :1171-1173
            q = self.rotary_emb.apply_rotary_embeddings(
                q, torch.arange(T, device=q.device, dtype=torch.int32) + start.to(torch.int32))
        attn = ops.attn_cross(q.contiguous(), k.unsqueeze(0), v.unsqueeze(0), scale=1.0 / math.sqrt(D))
        out, new_o = _apply_linear_batched(self.output_proj, attn.reshape(T, H * D),
                                           fp8_scales.get("output_proj") if fp8_scales else None, residual=residual)
        updated = None
        if fp8_scales is not None and self.use_fp8:  # :1192-1202
            updated = {}
            for name, val in (("q_proj", new_q), ("k_proj", new_k), ("v_proj", new_v), ("output_proj", new_o)):
                if val is not None:
                    updated[name] = val
        new_cache = {"k": k, "v": v, "position": (start + T).to(torch.int32)}
        return out, new_cache, updated


class TransformerBlock:
    """xax/arch/attention.py:1214-1510: pre-norm block, x + attn(norm(x)), optionally x + cross_attn(norm(x),
    context), x + ffn(norm(x))."""

    def __init__(self, self_attn: SelfAttentionBlock, feed_forward: SwiGLU, attn_norm: RMSNorm, mlp_norm: RMSNorm, *,
                 num_heads: int, head_dim: int, causal: bool, use_fp8: bool = False, cross_attn=None,
                 cross_attn_norm=None, context_length: int | None = None):
        if (cross_attn is None) != (cross_attn_norm is None):
            raise ValueError("cross_attn and cross_attn_norm go together")
        self.self_attn, self.feed_forward, self.attn_norm, self.mlp_norm = self_attn, feed_forward, attn_norm, mlp_norm
        self.num_heads, self.head_dim, self.causal, self.use_fp8 = num_heads, head_dim, causal, use_fp8
        self.cross_attn, self.cross_attn_norm, self.context_length = cross_attn, cross_attn_norm, context_length

    @classmethod
    def build(cls, embed_dim: int, num_heads: int, ff_dim: int, *, key=None, num_kv_heads: int | None = None,
              head_dim: int | None = None, causal: bool = False, cross_attention: bool = False,
              context_length: int | None = None, use_rotary_embeddings: bool = False, rotary_base: float = 10000.0,
              rotary_style: RotaryEmbeddingStyle = "concatenated", rotary_factor: float = 1.0,
              rotary_original_max_position_embeddings: int | None = None, rotary_beta_slow: float = 1.0,
              rotary_beta_fast: float = 32.0, use_qk_norm: bool = False, qk_norm_eps: float = 1e-6,
              use_attention_sinks: bool = False, norm_type: str = "layernorm", norm_eps: float = 1e-6,
              feedforward_type: str = "mlp", use_fp8: bool = False, compute_dtype=BF16, fp8_mlp: bool | None = None,
              device=None) -> "TransformerBlock":
        """Same keyword arguments as the reference.  ``norm_type`` must be "rmsnorm" and
        ``feedforward_type`` "swiglu" (the LLM path).  Like the reference, ``use_fp8`` makes the
        four attention projections FP8 and leaves the SwiGLU on plain linears (:1354-1355);
        ``fp8_mlp=True`` (an extension) builds the SwiGLU from Fp8Linear too."""
        if norm_type != "rmsnorm" or feedforward_type != "swiglu":
            raise ValueError("only norm_type='rmsnorm' with feedforward_type='swiglu' is on the path this library covers")
        seed = int(key or 0) if not isinstance(key, torch.Generator) else int(key.initial_seed())
        hd = head_dim if head_dim is not None else embed_dim // num_heads
        attn = SelfAttentionBlock.build(
            embed_dim, num_heads, key=seed * 3 + 1, num_kv_heads=num_kv_heads, head_dim=head_dim, causal=causal,
            context_length=context_length, use_rotary_embeddings=use_rotary_embeddings, rotary_base=rotary_base,
            rotary_style=rotary_style, rotary_factor=rotary_factor,
            rotary_original_max_position_embeddings=rotary_original_max_position_embeddings,
            rotary_beta_slow=rotary_beta_slow, rotary_beta_fast=rotary_beta_fast, use_qk_norm=use_qk_norm,
            qk_norm_eps=qk_norm_eps, use_attention_sinks=use_attention_sinks, use_fp8=use_fp8,
            compute_dtype=compute_dtype, device=device)
        ff = SwiGLU.build(embed_dim, ff_dim, key=seed * 3 + 2, use_fp8=bool(fp8_mlp), device=device)
        cross = cross_norm = None
        if cross_attention:  # :1312-1322
            cross = CrossAttentionBlock.build(embed_dim, num_heads, key=seed * 3 + 3,
                                              use_rotary_embeddings=use_rotary_embeddings, rotary_base=rotary_base,
                                              use_fp8=use_fp8, compute_dtype=compute_dtype, device=device)
            cross_norm = RMSNorm.build(embed_dim, norm_eps, device)
        return cls(attn, ff, RMSNorm.build(embed_dim, norm_eps, device), RMSNorm.build(embed_dim, norm_eps, device),
                   num_heads=num_heads, head_dim=hd, causal=causal, use_fp8=use_fp8, cross_attn=cross,
                   cross_attn_norm=cross_norm, context_length=context_length)

    @property
    def embed_dim(self) -> int:
        return self.head_dim * self.num_heads

    def init_cache(self, max_len: int | None = None, dtype=None, context_sn=None, fp8_history_length: int | None = None,
                   batch: int | None = None) -> TransformerBlockCache:
        """xax/arch/attention.py:1384-1419."""
        cache: TransformerBlockCache = {"self_attn": self.self_attn.init_cache(max_len=max_len, dtype=dtype, batch=batch)}
        if self.cross_attn is not None:  # :1407-1411
            if context_sn is None:
                raise ValueError("context_sn must be provided if cross_attn is not None")
            cache["cross_attn"], _ = self.cross_attn.init_cache(kv_sn=context_sn)
        if fp8_history_length is not None:
            if self.self_attn.use_fp8:
                cache["self_attn_fp8"] = _init_fp8_scales_cache(fp8_history_length)
            if self.cross_attn is not None and self.cross_attn.use_fp8:
                cache["cross_attn_fp8"] = _init_fp8_scales_cache(fp8_history_length)
        return cache

    def init_mask(self, seq_len: int, add_cache: bool = False, batch_dim: bool = False) -> torch.Tensor:
        return self.self_attn.init_mask(seq_len, add_cache=add_cache, batch_dim=batch_dim)

    def __call__(self, x_tn, *, context_sn=None, mask=None, cache=None, donate: bool = True):
        return self.forward(x_tn, context_sn=context_sn, mask=mask, cache=cache, donate=donate)

    def forward(self, x_tn: torch.Tensor, *, context_sn=None, mask=None, cache: TransformerBlockCache | None = None,
                donate: bool = True):
        """xax/arch/attention.py:1443-1510 for one sequence (T, H)."""
        if x_tn.dim() != 2:
            raise ValueError(f"expected rank 2 input, got rank {x_tn.dim()}")
        if self.cross_attn is not None:
            return self._forward_with_cross_attention(x_tn, context_sn, mask, cache, donate)
        if mask is not None:  # accepted when it is the mask the kernels apply anyway
            self.self_attn._require_builtin_mask(mask, x_tn.shape[0], None if cache is None else cache["self_attn"])
        bc = None
        if cache is not None:
            a = cache["self_attn"]
            bc = {"k": a["k"].unsqueeze(0), "v": a["v"].unsqueeze(0), "position": a["position"].reshape(1)}
        x, nc = self.forward_tokens(x_tn.to(BF16).contiguous(), 1, x_tn.shape[0], cache=bc, donate=donate)
        out_cache: TransformerBlockCache = {
            "self_attn": {"k": nc["k"][0], "v": nc["v"][0], "position": nc["position"].reshape(())}}
        return x, out_cache

    def _forward_with_cross_attention(self, x_tn, context_sn, mask, cache, donate):
        """:1466-1508 with the cross-attention sub-block: the three sub-blocks one after the other, each a
        pre-norm residual branch.  (The fused kernel sequence of ``forward_tokens`` covers the decoder-only
        block; this path is module by module.)"""
        x = x_tn.to(BF16).contiguous()
        T = x.shape[0]
        attn = self.self_attn
        if mask is not None:
            attn._require_builtin_mask(mask, T, None if cache is None else cache["self_attn"])
        bc = None
        if cache is not None:
            a = cache["self_attn"]
            bc = {"k": a["k"].unsqueeze(0), "v": a["v"].unsqueeze(0), "position": a["position"].reshape(1)}
        y, _ = ops.rmsnorm(x, self.attn_norm.weight_bf16(), self.attn_norm.eps)
        x1, nc = attn.forward_tokens(y, 1, T, cache=bc, donate=donate, residual=x)
        out_cache: TransformerBlockCache = {
            "self_attn": {"k": nc["k"][0], "v": nc["v"][0], "position": nc["position"].reshape(())}}
        y, _ = ops.rmsnorm(x1, self.cross_attn_norm.weight_bf16(), self.cross_attn_norm.eps)
        x2, c_cache, _ = self.cross_attn.forward(y, kv_sn=context_sn, residual=x1,
                                                 cache=None if cache is None else cache.get("cross_attn"))
        out_cache["cross_attn"] = c_cache
        y, _ = ops.rmsnorm(x2, self.mlp_norm.weight_bf16(), self.mlp_norm.eps)
        x3 = self.feed_forward.forward_tokens(y, 1, T, residual=x2)
        return x3, out_cache

    def forward_tokens(self, x: torch.Tensor, B: int, T: int, *, cache=None, donate: bool = True, workspace=None,
                       advance: bool = True):
        """x: [B*T, H] bf16 residual stream of B sequences, T new tokens each; returns the new
        residual stream and the updated batched attention cache.  Kernel sequence:
        RMSNorm(+cast) -> QKV GEMM -> RoPE + cache append -> attention -> cast -> out-proj GEMM
        (+x) -> RMSNorm(+cast / amax) -> gate|up GEMM -> SiLU*up(+cast / amax) -> down GEMM (+x)."""
        attn, ff = self.self_attn, self.feed_forward
        wn = self.attn_norm.weight_bf16()
        if attn._is_fp8():
            _, yq = ops.rmsnorm(x, wn, self.attn_norm.eps, want_y=False, quantize=True)
            x1, new_cache = attn.forward_tokens(x, B, T, cache=cache, donate=donate, y_q=(yq[0], yq[2]), residual=x,
                                                workspace=workspace, advance=advance)
        else:
            y, _ = ops.rmsnorm(x, wn, self.attn_norm.eps)
            x1, new_cache = attn.forward_tokens(y, B, T, cache=cache, donate=donate, residual=x, workspace=workspace,
                                                advance=advance)
        wm = self.mlp_norm.weight_bf16()
        if ff.is_fp8():
            if T == 1:  # one token per sequence: the per-sequence scale is the per-token scale
                _, yq = ops.rmsnorm(x1, wm, self.mlp_norm.eps, want_y=False, quantize=True)
                x2 = ff.forward_tokens(x1, B, T, residual=x1, y_q=(yq[0], yq[2]))
            else:
                amax = torch.zeros((B,), dtype=torch.float32, device=x.device)
                y, _ = ops.rmsnorm(x1, wm, self.mlp_norm.eps, group_amax=amax, group_rows=T)
                q, _, inv = ops.quantize_with_amax(y, amax, T)
                x2 = ff.forward_tokens(y, B, T, residual=x1, y_q=(q, inv))
        else:
            y, _ = ops.rmsnorm(x1, wm, self.mlp_norm.eps)
            x2 = ff.forward_tokens(y, B, T, residual=x1)
        return x2, new_cache


class TransformerCache(TypedDict):
    """xax/arch/attention.py:1208-1211: {"layers": {"layer_<i>": TransformerBlockCache}}."""

    layers: dict[str, TransformerBlockCache]


class TransformerStack:
    """xax/arch/attention.py:1513-1654: a stack of transformer blocks with the reference's cache layout.

    The reference's ``build`` makes LayerNorm + GELU-MLP blocks (it leaves ``norm_type`` / ``feedforward_type``
    of TransformerBlock.build at their defaults); the kernels of this library cover the RMSNorm + SwiGLU
    block of the LLM path, so ``build`` takes the two keywords explicitly (an extension), defaults to what
    the kernels cover, and refuses the rest like TransformerBlock.build does.  Stacks can also be made from
    existing blocks through the constructor."""

    def __init__(self, layers, num_layers: int | None = None, causal: bool = True, use_fp8: bool = False):
        self.layers = tuple(layers)
        self.num_layers = len(self.layers) if num_layers is None else num_layers
        self.causal, self.use_fp8 = causal, use_fp8

    @classmethod
    def build(cls, embed_dim: int, num_heads: int, ff_dim: int, num_layers: int, *, key=None, causal: bool = False,
              cross_attention: bool = False, context_length: int | None = None, use_rotary_embeddings: bool = False,
              rotary_base: float = 10000.0, use_fp8: bool = False, compute_dtype=BF16, norm_type: str = "rmsnorm",
              feedforward_type: str = "swiglu", num_kv_heads: int | None = None, head_dim: int | None = None,
              norm_eps: float = 1e-6, fp8_mlp: bool | None = None, device=None) -> "TransformerStack":
        seed = int(key or 0) if not isinstance(key, torch.Generator) else int(key.initial_seed())
        layers = tuple(
            TransformerBlock.build(embed_dim, num_heads, ff_dim, key=seed * 1000 + i, num_kv_heads=num_kv_heads,
                                   head_dim=head_dim, causal=causal, cross_attention=cross_attention,
                                   context_length=context_length, use_rotary_embeddings=use_rotary_embeddings,
                                   rotary_base=rotary_base, norm_type=norm_type, norm_eps=norm_eps,
                                   feedforward_type=feedforward_type, use_fp8=use_fp8, compute_dtype=compute_dtype,
                                   fp8_mlp=fp8_mlp, device=device)
            for i in range(num_layers))
        return cls(layers, num_layers, causal, use_fp8)

    def init_cache(self, dtype=None, x_tn=None, fp8_history_length: int | None = None,
                   max_len: int | None = None) -> TransformerCache:
        """:1583-1602.  The reference sizes the cache from the blocks' ``context_length``; ``max_len`` (an
        extension) overrides it for blocks built without one."""
        return {"layers": {f"layer_{i}": layer.init_cache(max_len=max_len, dtype=dtype, context_sn=x_tn,
                                                          fp8_history_length=fp8_history_length)
                           for i, layer in enumerate(self.layers)}}

    def init_mask(self, seq_len: int, add_cache: bool = False, batch_dim: bool = False) -> torch.Tensor:
        return self.layers[0].init_mask(seq_len, add_cache=add_cache, batch_dim=batch_dim)  # :1604-1614

    def forward(self, x_tn: torch.Tensor, *, context_sn=None, mask=None, cache: TransformerCache | None = None,
                donate: bool = True):
        """:1616-1654: (output (seq_len, embed_dim), updated cache)."""
        if cache is None:
            cache = {"layers": {}}
        updated: TransformerCache = {"layers": {}}
        for i, layer in enumerate(self.layers):
            x_tn, updated["layers"][f"layer_{i}"] = layer.forward(x_tn, context_sn=context_sn, mask=mask,
                                                                   cache=cache["layers"].get(f"layer_{i}"), donate=donate)
        return x_tn, updated


class Transformer:
    """xax/arch/attention.py:1657-1912: token embedding, a TransformerStack, a final norm and an optional output
    projection, with ``encode`` / ``forward`` / ``predict_sequence`` / ``generate_sequence``.  The final norm is
    an RMSNorm here (the reference's is a LayerNorm; see TransformerStack); ``decode`` runs the stack with its
    cross-attention sub-blocks against an embedded context."""

    def __init__(self, token_embedding: Embedding, layers: TransformerStack, layer_norm: RMSNorm, embed_dim: int,
                 causal: bool, use_fp8: bool = False, output_layer=None, context_length: int | None = None):
        self.token_embedding, self.layers, self.layer_norm = token_embedding, layers, layer_norm
        self.embed_dim, self.causal, self.use_fp8 = embed_dim, causal, use_fp8
        self.output_layer, self.context_length = output_layer, context_length

    @classmethod
    def build(cls, vocab_size: int, embed_dim: int, num_heads: int, ff_dim: int, num_layers: int,
              output_size: int | None = None, *, key=None, causal: bool = False, cross_attention: bool = False,
              context_length: int | None = None, use_rotary_embeddings: bool = False, rotary_base: float = 10000.0,
              use_fp8: bool = False, compute_dtype=BF16, device=None, **stack_kwargs) -> "Transformer":
        seed = int(key or 0) if not isinstance(key, torch.Generator) else int(key.initial_seed())
        emb = Embedding(vocab_size, embed_dim, key=seed * 4 + 1, device=device)
        stack = TransformerStack.build(embed_dim, num_heads, ff_dim, num_layers, key=seed * 4 + 3, causal=causal,
                                       cross_attention=cross_attention, context_length=context_length,
                                       use_rotary_embeddings=use_rotary_embeddings, rotary_base=rotary_base,
                                       use_fp8=use_fp8, compute_dtype=compute_dtype, device=device, **stack_kwargs)
        out = None
        if output_size is not None:
            out = _make_linear(embed_dim, output_size, seed * 4 + 4, use_fp8=use_fp8, compute_dtype=compute_dtype,
                               device=device)
        return cls(emb, stack, RMSNorm.build(embed_dim, device=device), embed_dim, causal, use_fp8, out, context_length)

    def init_cache(self, dtype=None, x_tn=None, fp8_history_length: int | None = None,
                   max_len: int | None = None) -> TransformerCache:
        return self.layers.init_cache(dtype=dtype, x_tn=x_tn, fp8_history_length=fp8_history_length, max_len=max_len)

    def init_mask(self, seq_len: int, add_cache: bool = False, batch_dim: bool = False) -> torch.Tensor:
        return self.layers.init_mask(seq_len, add_cache=add_cache, batch_dim=batch_dim)

    def encode(self, x: torch.Tensor, *, mask=None, cache: TransformerCache | None = None):
        """:1765-1786: token ids (seq_len,) -> (normalised hidden states, updated cache)."""
        emb = ops.embed(x.to(torch.int32).reshape(-1), self.token_embedding.weight)
        h, updated = self.layers.forward(emb, mask=mask, cache=cache)
        return self.layer_norm(h), updated

    def decode(self, x_t: torch.Tensor, context_s: torch.Tensor, *, mask=None, cache: TransformerCache | None = None):
        """:1788-1818: token ids (seq_len,) and context token ids (context_len,), both looked up in the token
        embedding, through the stack with cross-attention -> (normalised hidden states, updated cache)."""
        table = self.token_embedding.weight
        emb = ops.embed(x_t.to(torch.int32).reshape(-1), table)
        ctx = ops.embed(context_s.to(torch.int32).reshape(-1), table)
        h, updated = self.layers.forward(emb, context_sn=ctx, mask=mask, cache=cache)
        return self.layer_norm(h), updated

    def forward(self, x: torch.Tensor, *, mask=None, cache: TransformerCache | None = None):
        """:1820-1842."""
        if x.dim() != 1:
            raise ValueError(f"expected rank 1 token ids, got rank {x.dim()}")
        out, updated = self.encode(x, mask=mask, cache=cache)
        if self.output_layer is not None:
            out, _ = _apply_linear_batched(self.output_layer, out)
        return out, updated

    def predict_sequence(self, x_seq: torch.Tensor) -> torch.Tensor:
        return self.forward(x_seq)[0]  # :1844-1846

    def generate_sequence(self, prompt_seq: torch.Tensor, max_len: int, temperature: float = 1.0,
                          top_k: int | None = None, key=None, jit_level: int | None = None) -> torch.Tensor:
        """:1848-1912: prime the cache with the prompt, then ``max_len`` steps, each feeding the last token and
        drawing the next from softmax(logits / temperature).  ``key``: a torch.Generator on the model's device or
        an int seed (default 0); the reference draws through jax.random.categorical from its own stream, the
        distribution is the same.  ``top_k`` is outside the path this library covers."""
        if top_k is not None:
            raise ValueError("top-k truncation is outside the path this library covers")
        if self.output_layer is None:
            raise ValueError("generate_sequence needs an output projection onto the vocabulary")
        dev = self.token_embedding.weight.device
        prompt_seq = prompt_seq.to(device=dev, dtype=torch.int32)
        n0 = prompt_seq.shape[0]
        out = torch.zeros((n0 + max_len,), dtype=torch.int32, device=dev)
        out[:n0] = prompt_seq
        cache = self.init_cache(max_len=n0 + max_len if self.context_length is None else None)
        # the prompt primes the cache; like the reference's scan, the first step then feeds the prompt's last
        # token once more (at cache row n0) and every later step the token drawn before it
        _, cache = self.encode(prompt_seq, cache=cache)
        gen = key if isinstance(key, torch.Generator) else torch.Generator(device=dev).manual_seed(int(key or 0))
        for pos in range(n0 - 1, n0 - 1 + max_len):
            logits, cache = self.forward(out[pos:pos + 1], cache=cache)
            u = torch.rand((1,), generator=gen, device=dev, dtype=torch.float32)
            out[pos + 1] = ops.sample_top_p(logits[-1:].to(BF16).contiguous(), float(temperature), 1.0, u)[0]
        return out
