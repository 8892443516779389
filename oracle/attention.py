"""Oracle restatement of the hot-path parts of ``xax/arch/attention.py`` (test
infrastructure; parity unpinned -- see the package docstring).

Unbatched, like the reference: ``forward`` takes one sequence ``(T, H)``; callers batch by
looping (the reference batches with ``jax.vmap``).
"""

from __future__ import annotations

import math

import numpy as np

from .fp8 import Fp8Linear, bfloat16, f32, float32, matmul_nt, promote, rnd


class Linear:
    """Stand-in for ``eqx.nn.Linear``: weight (out, in), optional bias."""

    def __init__(self, weight, bias=None):
        self.weight = np.asarray(weight)
        self.bias = None if bias is None else np.asarray(bias)
        self.out_features, self.in_features = self.weight.shape


class Embedding:
    """Stand-in for ``eqx.nn.Embedding``: weight (num_embeddings, dim)."""

    def __init__(self, weight):
        self.weight = np.asarray(weight)


class LoRALinear:
    """xax/nn/lora.py:14-97 (fields only; the forward is the LoRA branch of apply_linear)."""

    def __init__(self, weight_oi, bias_o, lora_a_ir, lora_b_ro, rank, alpha=16.0):
        self.weight_oi, self.lora_a_ir, self.lora_b_ro = np.asarray(weight_oi), np.asarray(lora_a_ir), np.asarray(lora_b_ro)
        self.bias_o = None if bias_o is None else np.asarray(bias_o)
        self.rank, self.alpha = rank, alpha

    @property
    def scaling(self):
        return self.alpha / self.rank


def apply_linear(x, linear):
    """xax/arch/attention.py:30-69."""
    x = np.asarray(x)
    if isinstance(linear, LoRALinear):  # :44-51
        dt = promote(x.dtype, linear.weight_oi.dtype)
        y = matmul_nt(x, linear.weight_oi, dt)
        if linear.bias_o is not None:
            y = rnd(f32(y) + f32(linear.bias_o), promote(dt, linear.bias_o.dtype))
        low = rnd(f32(x) @ f32(linear.lora_a_ir), promote(x.dtype, linear.lora_a_ir.dtype))
        delta = rnd(f32(low) @ f32(linear.lora_b_ro), promote(low.dtype, linear.lora_b_ro.dtype))
        delta = rnd(f32(delta) * float32(linear.scaling), delta.dtype)  # weak Python scalar keeps the dtype
        return rnd(f32(y) + f32(delta), promote(y.dtype, delta.dtype))
    if isinstance(linear, Fp8Linear):  # :52-58 -- whole tensor at once, scales dropped
        return linear(x)[0]
    if isinstance(linear, Linear):  # :59-64
        dt = promote(x.dtype, linear.weight.dtype)
        y = matmul_nt(x, linear.weight, dt)
        if linear.bias is not None:
            y = rnd(f32(y) + f32(linear.bias), promote(dt, linear.bias.dtype))
        return y
    if isinstance(linear, Embedding):  # :65-67
        return matmul_nt(x, linear.weight, promote(x.dtype, linear.weight.dtype))
    raise ValueError(f"Unsupported linear layer type: {type(linear)}")


def apply_linear_batched(layer, x, scales=None):
    """xax/arch/attention.py:244-287: the layer is vmapped over rows, so an Fp8Linear with
    current scaling quantises every row with its own scale."""
    x = np.asarray(x)
    if isinstance(layer, Fp8Linear):
        flat = x.reshape(-1, x.shape[-1])
        if scales is not None:  # :270-275: shared incoming scales, last row's update kept
            outs = []
            new_scales = None
            for row in flat:
                o, new_scales = layer(row, scales)
                outs.append(o)
            out = np.stack(outs)
        else:  # :276-280
            if layer.use_fp8:
                out = layer.call_rows(flat)[0]
            else:
                out = layer(flat)[0]
            new_scales = None
        return out.reshape(*x.shape[:-1], -1), new_scales
    return apply_linear(x, layer), None  # :286 (row-wise == batched for a plain linear)


class RMSNorm:
    """xax/arch/attention.py:72-98, every op rounded to the promoted dtype."""

    def __init__(self, weight, eps: float = 1e-6):
        self.weight = np.asarray(weight)
        self.eps = eps

    @classmethod
    def build(cls, dim: int, eps: float = 1e-6, dtype=float32) -> "RMSNorm":
        return cls(np.ones((dim,), dtype=dtype), eps)

    def __call__(self, x):
        x = np.asarray(x)
        dt = x.dtype
        sq = rnd(f32(x) * f32(x), dt)
        mean = rnd(np.mean(f32(sq), axis=-1, keepdims=True, dtype=float32), dt)
        eps = np.asarray(self.eps).astype(dt)  # weak scalar takes the array dtype
        norm = rnd(np.sqrt(f32(rnd(f32(mean) + f32(eps), dt))), dt)
        y = rnd(f32(x) / f32(norm), dt)
        odt = promote(dt, self.weight.dtype)
        return rnd(f32(y) * f32(self.weight), odt)


def silu(x):
    """jax.nn.silu = x * sigmoid(x), each op rounded to x's dtype."""
    x = np.asarray(x)
    sig = rnd(1.0 / (1.0 + np.exp(-f32(x))), x.dtype)
    return rnd(f32(x) * f32(sig), x.dtype)


class SwiGLU:
    """xax/arch/attention.py:101-147."""

    def __init__(self, gate, up, down):
        self.gate, self.up, self.down = gate, up, down

    def __call__(self, x):
        g = apply_linear(x, self.gate)
        u = apply_linear(x, self.up)
        sg = silu(g)
        hidden = rnd(f32(sg) * f32(u), promote(sg.dtype, u.dtype))
        return apply_linear(hidden, self.down)


class RotaryEmbedding:
    """xax/arch/attention.py:310-526 (YaRN branch :401-441 included for the table)."""

    def __init__(self, head_dim, base=10000.0, style="interleaved", factor=1.0,
                 original_max_position_embeddings=None, beta_slow=1.0, beta_fast=32.0):
        self.head_dim = head_dim
        self.base = base
        self.style = style
        self.factor = factor
        self.original_max_position_embeddings = original_max_position_embeddings
        self.beta_slow = beta_slow
        self.beta_fast = beta_fast

    @property
    def uses_yarn(self) -> bool:
        return self.factor > 1.0 and self.original_max_position_embeddings is not None

    def get_rotary_embeddings(self, positions, dtype):
        """:374-399.  ``positions`` int32; everything else in ``dtype`` -- including the
        positions themselves once they meet ``freqs`` (int32 * bf16 -> bf16)."""
        dim = self.head_dim // 2
        positions = np.asarray(positions)
        if self.uses_yarn:
            return self._yarn(positions, dtype, dim)
        i = np.arange(0, dim).astype(dtype)
        neg = rnd(-f32(i), dtype)
        logb = np.asarray(np.log(float32(self.base))).astype(dtype)  # weak f32 scalar -> dtype
        t = rnd(f32(neg) * f32(logb), dtype)
        t = rnd(f32(t) / f32(np.asarray(dim).astype(dtype)), dtype)
        freqs = rnd(np.exp(f32(t)), dtype)
        if np.issubdtype(positions.dtype, np.integer):
            pos = positions.astype(dtype)
            adt = dtype
        else:
            pos = positions
            adt = promote(positions.dtype, dtype)
        angles = rnd(f32(pos)[:, None] * f32(freqs)[None, :], adt)
        return rnd(np.cos(f32(angles)), adt), rnd(np.sin(f32(angles)), adt)

    def _yarn(self, positions, dtype, dim):
        """:401-441 -- float32 internally, cast at the end."""
        features = self.head_dim
        omp = self.original_max_position_embeddings
        low = (features * math.log(omp / (self.beta_fast * 2 * math.pi))) / (2 * math.log(self.base))
        high = (features * math.log(omp / (self.beta_slow * 2 * math.pi))) / (2 * math.log(self.base))
        low, high = max(low, 0), min(high, features - 1)
        timescale = (float32(self.base) ** (np.arange(0, features, 2, dtype=float32) / float32(features))).astype(float32)
        extra = (float32(1.0) / timescale).astype(float32)
        inter = (float32(1.0) / (float32(self.factor) * timescale)).astype(float32)
        high = high if low != high else (high + 0.001)
        idx = np.arange(dim, dtype=float32)
        interp = (1 - np.clip((idx - float32(low)) / float32(high - low), 0.0, 1.0)).astype(float32)
        freq = (inter * (1 - interp) + extra * interp).astype(float32)
        angles = (f32(positions)[:, None] * freq[None, :]).astype(float32)
        scaling = float32(0.1 * 1.0 * math.log(self.factor) + 1.0)
        return (np.cos(angles) * scaling).astype(dtype), (np.sin(angles) * scaling).astype(dtype)

    def apply_rotary_embeddings(self, x, positions=None):
        """:443-483, 3-D input (T, heads, head_dim)."""
        x = np.asarray(x)
        T = x.shape[0]
        if positions is None:
            positions = np.arange(T).astype(x.dtype)  # :471
        cos, sin = self.get_rotary_embeddings(positions, x.dtype)
        cos, sin = cos[:, None, :], sin[:, None, :]
        dt = promote(x.dtype, cos.dtype)

        def mul(a, b):
            return rnd(f32(a) * f32(b), dt)

        if self.style == "concatenated":  # :510-515
            h = x.shape[-1] // 2
            x1, x2 = x[..., :h], x[..., h:]
            a = rnd(f32(mul(x1, cos)) - f32(mul(x2, sin)), dt)
            b = rnd(f32(mul(x2, cos)) + f32(mul(x1, sin)), dt)
            return np.concatenate([a, b], axis=-1)
        if self.style == "interleaved":  # :517-526
            xe, xo = x[..., ::2], x[..., 1::2]
            re = rnd(f32(mul(xe, cos)) - f32(mul(xo, sin)), dt)
            ro = rnd(f32(mul(xe, sin)) + f32(mul(xo, cos)), dt)
            out = np.zeros(x.shape, dtype=dt)
            out[..., ::2] = re
            out[..., 1::2] = ro
            return out
        raise ValueError(f"Unknown RoPE style: {self.style}. Use 'concatenated' or 'interleaved'.")


def dot_product_attention(q, k, v, *, mask=None, is_causal=False, scale=None, local_window_size=None):
    """Documented behaviour of ``jax.nn.dot_product_attention``'s default path for
    q (T, Hq, D), k/v (S, Hkv, D): float32 logits * scale, masked positions get a large
    negative value, float32 softmax over keys, probabilities cast to the value dtype, P.V
    accumulated in float32 and rounded to the value dtype.  Query head h reads kv head
    h // (Hq // Hkv).  ``local_window_size`` = (left, right): query i sees keys i - left .. i + right."""
    q, k, v = np.asarray(q), np.asarray(k), np.asarray(v)
    T, Hq, D = q.shape
    S, Hkv, _ = k.shape
    G = Hq // Hkv
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    allow = np.ones((T, S), dtype=bool)
    if mask is not None:
        allow &= np.asarray(mask).reshape(T, S)
    if is_causal:
        allow &= np.tril(np.ones((T, S), dtype=bool))
    if local_window_size is not None:
        left, right = local_window_size
        qi, kj = np.arange(T)[:, None], np.arange(S)[None, :]
        allow &= (kj >= qi - left) & (kj <= qi + right)
    out = np.empty((T, Hq, D), dtype=v.dtype)
    neg = float32(-0.7 * np.finfo(np.float32).max)
    for h in range(Hq):
        g = h // G
        logits = (f32(q[:, h]) @ f32(k[:, g]).T).astype(float32) * float32(scale)
        logits = np.where(allow, logits, neg).astype(float32)
        m = logits.max(axis=-1, keepdims=True)
        e = np.exp(logits - m, dtype=float32)
        p = (e / e.sum(axis=-1, keepdims=True, dtype=float32)).astype(float32)
        p = p.astype(v.dtype)
        out[:, h] = rnd(f32(p) @ f32(v[:, g]), v.dtype)
    return out


class SelfAttentionBlock:
    """xax/arch/attention.py:529-980 restricted to the path: GQA, optional RoPE, causal,
    KV cache, optional QK-norm (:864-867) and sliding window (:931-936, :955); no sinks."""

    def __init__(self, q_proj, k_proj, v_proj, output_proj, rotary_emb, *, num_heads, num_kv_heads, head_dim,
                 causal=True, q_norm=None, k_norm=None, local_window_size=None):
        assert num_heads % num_kv_heads == 0  # :620
        self.q_proj, self.k_proj, self.v_proj, self.output_proj = q_proj, k_proj, v_proj, output_proj
        self.rotary_emb = rotary_emb
        self.q_norm, self.k_norm = q_norm, k_norm
        self.local_window_size = local_window_size
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.causal = causal

    def init_cache(self, max_len=None, dtype=bfloat16):
        """:775-794."""
        if max_len is None:
            raise ValueError("context_length or max_len must be set for caching")
        shape = (max_len, self.num_kv_heads, self.head_dim)
        return {"k": np.zeros(shape, dtype), "v": np.zeros(shape, dtype), "position": np.int32(0)}

    def call_batched(self, x_btd, positions_bt=None):
        """:700-773, ``__call__``: batched, no cache.  Every projection goes through apply_linear on the whole
        (batch, seq, dim) tensor (an FP8 layer: one activation scale for everything), RoPE takes explicit
        positions, the causal mask goes by token index."""
        x_btd = np.asarray(x_btd)
        assert x_btd.ndim == 3
        B, T, _ = x_btd.shape
        if positions_bt is None:
            positions_bt = np.broadcast_to(np.arange(T)[None, :], (B, T))
        q = apply_linear(x_btd, self.q_proj).reshape(B, T, self.num_heads, self.head_dim)
        k = apply_linear(x_btd, self.k_proj).reshape(B, T, self.num_kv_heads, self.head_dim)
        v = apply_linear(x_btd, self.v_proj).reshape(B, T, self.num_kv_heads, self.head_dim)
        if self.q_norm is not None:
            q = self.q_norm(q)
        if self.k_norm is not None:
            k = self.k_norm(k)
        outs = []
        for b in range(B):
            qb, kb = q[b], k[b]
            if self.rotary_emb is not None:
                pos = np.asarray(positions_bt[b]).astype(np.int32)
                qb = self.rotary_emb.apply_rotary_embeddings(qb, pos)
                kb = self.rotary_emb.apply_rotary_embeddings(kb, pos)
            lw = (self.local_window_size, 0) if self.local_window_size else None  # :765
            outs.append(dot_product_attention(qb, kb, v[b], is_causal=self.causal, local_window_size=lw).reshape(T, -1))
        return apply_linear(np.stack(outs), self.output_proj)

    def forward(self, x_tn, *, cache=None):
        """:826-980 (mask=None, fp8_scales=None)."""
        x_tn = np.asarray(x_tn)
        assert x_tn.ndim == 2
        q, _ = apply_linear_batched(self.q_proj, x_tn)  # :854-856
        k, _ = apply_linear_batched(self.k_proj, x_tn)
        v, _ = apply_linear_batched(self.v_proj, x_tn)
        T = x_tn.shape[0]
        q = q.reshape(T, self.num_heads, self.head_dim)
        k = k.reshape(T, self.num_kv_heads, self.head_dim)
        v = v.reshape(T, self.num_kv_heads, self.head_dim)
        if self.q_norm is not None:  # :864-867, per head, before RoPE
            q = self.q_norm(q)
        if self.k_norm is not None:
            k = self.k_norm(k)
        start = int(cache["position"]) if cache is not None else 0
        if self.rotary_emb is not None:  # :870-878
            positions = (np.arange(T) + start).astype(np.int32)
            q = self.rotary_emb.apply_rotary_embeddings(q, positions)
            k = self.rotary_emb.apply_rotary_embeddings(k, positions)
        if cache is not None:  # :880-888 (post-RoPE K stored)
            kc, vc = cache["k"].copy(), cache["v"].copy()
            kc[start:start + T] = k.astype(kc.dtype)
            vc[start:start + T] = v.astype(vc.dtype)
            k, v = kc, vc
            new_position = start + T
            S = k.shape[0]
            valid = np.arange(S) < new_position  # :917
            if self.causal:  # :919-926
                qpos = np.arange(T) + start
                allow = valid[None, :] & (np.arange(S)[None, :] <= qpos[:, None])
            else:
                allow = np.broadcast_to(valid[None, :], (T, S))
            if self.local_window_size is not None:  # :931-936: k_pos >= q_pos - window
                qpos = np.arange(T) + start
                allow = allow & (np.arange(S)[None, :] >= (qpos[:, None] - self.local_window_size))
            attn = dot_product_attention(q, k, v, mask=allow)
        else:
            new_position = T
            lw = (self.local_window_size, 0) if self.local_window_size is not None else None
            attn = dot_product_attention(q, k, v, is_causal=self.causal, local_window_size=lw)  # :949-957
        attn = attn.reshape(T, -1)
        out, _ = apply_linear_batched(self.output_proj, attn)  # :959-961
        return out, {"k": k, "v": v, "position": np.int32(new_position)}


class CrossAttentionBlock:
    """xax/arch/attention.py:983-1205: queries from x, keys / values from a context sequence, every query sees
    every context token (is_causal=False), as many kv heads as query heads.  RoPE, when enabled, is the class
    default style of RotaryEmbedding.build ("interleaved", :1035), keys at positions 0 .. S-1 (:1090-1093), queries
    at cache position + 0 .. T-1 (:1179-1181)."""

    def __init__(self, q_proj, k_proj, v_proj, output_proj, rotary_emb=None, *, num_heads, head_dim):
        self.q_proj, self.k_proj, self.v_proj, self.output_proj = q_proj, k_proj, v_proj, output_proj
        self.rotary_emb, self.num_heads, self.head_dim = rotary_emb, num_heads, head_dim

    def _project_kv(self, kv_sn):
        kv_sn = np.asarray(kv_sn)
        assert kv_sn.ndim == 2
        k, _ = apply_linear_batched(self.k_proj, kv_sn)  # :1082-1083
        v, _ = apply_linear_batched(self.v_proj, kv_sn)
        S = kv_sn.shape[0]
        k = k.reshape(S, self.num_heads, self.head_dim)
        v = v.reshape(S, self.num_heads, self.head_dim)
        if self.rotary_emb is not None:  # :1090-1093
            k = self.rotary_emb.apply_rotary_embeddings(k, np.arange(S).astype(np.int32))
        return k, v

    def init_cache(self, kv_sn):
        """:1062-1108 (fp8_scales=None)."""
        k, v = self._project_kv(kv_sn)
        return {"k": k, "v": v, "position": np.int32(0)}

    def forward(self, q_tn, *, kv_sn=None, cache=None):
        """:1110-1205 (fp8_scales=None)."""
        q_tn = np.asarray(q_tn)
        assert q_tn.ndim == 2
        q, _ = apply_linear_batched(self.q_proj, q_tn)  # :1135
        T = q_tn.shape[0]
        q = q.reshape(T, self.num_heads, self.head_dim)
        if cache is not None:  # :1146-1149
            k, v, start = cache["k"], cache["v"], int(cache["position"])
        elif kv_sn is not None:  # :1150-1167
            k, v = self._project_kv(kv_sn)
            start = 0
        else:
            raise ValueError("Either `cache` or `kv_sn` must be provided.")
        if self.rotary_emb is not None:  # :1171-1173
            q = self.rotary_emb.apply_rotary_embeddings(q, (np.arange(T) + start).astype(np.int32))
        attn = dot_product_attention(q, k, v, is_causal=False, scale=1.0 / math.sqrt(self.head_dim))  # :1176-1182
        out, _ = apply_linear_batched(self.output_proj, attn.reshape(T, -1))  # :1188-1189
        return out, {"k": k, "v": v, "position": np.int32(start + T)}


class TransformerBlock:
    """xax/arch/attention.py:1214-1510 (pre-norm: self-attention, optional cross-attention, feed-forward)."""

    def __init__(self, self_attn, feed_forward, attn_norm, mlp_norm, cross_attn=None, cross_attn_norm=None):
        self.self_attn, self.feed_forward = self_attn, feed_forward
        self.attn_norm, self.mlp_norm = attn_norm, mlp_norm
        self.cross_attn, self.cross_attn_norm = cross_attn, cross_attn_norm

    def init_cache(self, max_len=None, dtype=bfloat16, context_sn=None):
        cache = {"self_attn": self.self_attn.init_cache(max_len, dtype)}  # :1404-1405
        if self.cross_attn is not None:  # :1407-1411
            if context_sn is None:
                raise ValueError("context_sn must be provided if cross_attn is not None")
            cache["cross_attn"] = self.cross_attn.init_cache(context_sn)
        return cache

    def forward(self, x_tn, *, cache=None, context_sn=None):
        """:1443-1510."""
        x_tn = np.asarray(x_tn)
        norm_x = self.attn_norm(x_tn)  # :1468
        attn_out, attn_cache = self.self_attn.forward(norm_x, cache=None if cache is None else cache["self_attn"])
        x_tn = rnd(f32(x_tn) + f32(attn_out), promote(x_tn.dtype, attn_out.dtype))  # :1481
        new_cache = {"self_attn": attn_cache}
        if self.cross_attn is not None:  # :1483-1500
            norm_x = self.cross_attn_norm(x_tn)
            c_out, c_cache = self.cross_attn.forward(norm_x, kv_sn=context_sn,
                                                     cache=None if cache is None else cache.get("cross_attn"))
            new_cache["cross_attn"] = c_cache
            x_tn = rnd(f32(x_tn) + f32(c_out), promote(x_tn.dtype, c_out.dtype))
        norm_x = self.mlp_norm(x_tn)  # :1503
        ff = self.feed_forward(norm_x)  # :1507
        x_tn = rnd(f32(x_tn) + f32(ff), promote(x_tn.dtype, ff.dtype))  # :1508
        return x_tn, new_cache


def build_block(rng, *, embed_dim, num_heads, num_kv_heads, head_dim, ff_dim, rope_theta=10000.0, norm_eps=1e-6,
                fp8_attn=True, fp8_mlp=True, out_scale=1.0, std=0.02, dtype=bfloat16, attn_bias=False,
                use_qk_norm=False, qk_norm_eps=1e-6, local_window_size=None):
    """Random block with N(0, std^2) weights; output projections scaled by ``out_scale``.
    FP8 projections are Fp8Linear instances (as xax/arch/attention.py:233-240 builds for
    attention; for the MLP they are swapped into SwiGLU, which apply_linear accepts :52)."""

    def w(o, i, s=1.0):
        return (rng.standard_normal((o, i), dtype=float32) * float32(std * s)).astype(dtype)

    def lin(o, i, fp8, s=1.0, bias=False):
        b = np.zeros((o,), dtype) if bias else None
        return Fp8Linear(w(o, i, s), b) if fp8 else Linear(w(o, i, s), b)

    qd, kd = num_heads * head_dim, num_kv_heads * head_dim
    attn = SelfAttentionBlock(
        lin(qd, embed_dim, fp8_attn, bias=attn_bias), lin(kd, embed_dim, fp8_attn, bias=attn_bias),
        lin(kd, embed_dim, fp8_attn, bias=attn_bias), lin(embed_dim, qd, fp8_attn, out_scale, bias=attn_bias),
        RotaryEmbedding(head_dim, base=rope_theta, style="concatenated"),
        num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim, causal=True,
        local_window_size=local_window_size,
        # :665-669 builds ones; seeded weights around one make the test see them
        q_norm=RMSNorm((1 + 0.1 * rng.standard_normal(head_dim, dtype=float32)).astype(dtype), qk_norm_eps) if use_qk_norm else None,
        k_norm=RMSNorm((1 + 0.1 * rng.standard_normal(head_dim, dtype=float32)).astype(dtype), qk_norm_eps) if use_qk_norm else None)
    ff = SwiGLU(lin(ff_dim, embed_dim, fp8_mlp), lin(ff_dim, embed_dim, fp8_mlp),
                lin(embed_dim, ff_dim, fp8_mlp, out_scale))
    return TransformerBlock(attn, ff, RMSNorm.build(embed_dim, norm_eps, dtype), RMSNorm.build(embed_dim, norm_eps, dtype))
