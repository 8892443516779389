"""Test helpers: numpy(ml_dtypes) <-> torch conversions and error metrics."""

import ml_dtypes
import numpy as np
import torch

bf16 = ml_dtypes.bfloat16
e4m3 = ml_dtypes.float8_e4m3fn
e5m2 = ml_dtypes.float8_e5m2


def to_torch(a: np.ndarray, device="cuda") -> torch.Tensor:
    a = np.ascontiguousarray(a)
    if a.dtype == np.dtype(bf16):
        return torch.from_numpy(a.view(np.uint16).astype(np.int32)).to(torch.int16).view(torch.bfloat16).to(device)
    if a.dtype == np.dtype(e4m3):
        return torch.from_numpy(a.view(np.uint8).copy()).view(torch.float8_e4m3fn).to(device)
    if a.dtype == np.dtype(e5m2):
        return torch.from_numpy(a.view(np.uint8).copy()).view(torch.float8_e5m2).to(device)
    return torch.from_numpy(a).to(device)


def to_numpy(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16).view(bf16)
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy().view(e4m3)
    if t.dtype == torch.float8_e5m2:
        return t.view(torch.uint8).numpy().view(e5m2)
    return t.numpy()


def f32(a) -> np.ndarray:
    return np.asarray(a).astype(np.float32)


def rel_fro(a, b) -> float:
    """||a - b||_F / ||b||_F in float64."""
    a = np.asarray(a).astype(np.float64)
    b = np.asarray(b).astype(np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def cfg1_inputs(M=2048, K=2048, N=8192, seed=0):
    """benchmark config 1 distributions: x ~ N(0,1) with 0.1 % of entries x20, W ~ N(0, 0.02^2)
    stored (N, K), bias ~ N(0, 0.01^2); all bf16."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K)).astype(np.float32)
    x = np.where(rng.random((M, K)) < 1e-3, x * 20.0, x)
    w = (rng.standard_normal((K, N)) * 0.02).astype(np.float32).T.copy()
    b = (rng.standard_normal((N,)) * 0.01).astype(np.float32)
    return x.astype(bf16), w.astype(bf16), b.astype(bf16), rng


# ---------------------------------------------------------------------------------------
# oracle model -> device model (same weights), so both sides of a parity test share parameters


def _lin_from_oracle(o, device="cuda"):
    from xax_b200.arch.attention import Linear
    from xax_b200.nn.fp8 import Fp8Linear

    w = to_torch(o.weight, device)
    b = None if o.bias is None else to_torch(o.bias, device)
    if type(o).__name__ == "Fp8Linear":
        return Fp8Linear(w.shape[1], w.shape[0], weight=w, bias=b, use_bias=b is not None, use_fp8=o.use_fp8)
    return Linear(w.shape[1], w.shape[0], use_bias=b is not None, weight=w, bias=b)


def block_from_oracle(ob, device="cuda"):
    from xax_b200.arch.attention import RMSNorm, RotaryEmbedding, SelfAttentionBlock, SwiGLU, TransformerBlock

    a = ob.self_attn
    attn = SelfAttentionBlock(
        _lin_from_oracle(a.q_proj, device), _lin_from_oracle(a.k_proj, device), _lin_from_oracle(a.v_proj, device),
        _lin_from_oracle(a.output_proj, device),
        RotaryEmbedding.build(a.head_dim, a.rotary_emb.base, a.rotary_emb.style),
        None if getattr(a, "q_norm", None) is None else RMSNorm(to_torch(a.q_norm.weight, device), a.q_norm.eps),
        None if getattr(a, "k_norm", None) is None else RMSNorm(to_torch(a.k_norm.weight, device), a.k_norm.eps),
        num_heads=a.num_heads, num_kv_heads=a.num_kv_heads, head_dim=a.head_dim, causal=a.causal,
        local_window_size=getattr(a, "local_window_size", None))
    f = ob.feed_forward
    ff = SwiGLU(_lin_from_oracle(f.gate, device), _lin_from_oracle(f.up, device), _lin_from_oracle(f.down, device))
    return TransformerBlock(attn, ff, RMSNorm(to_torch(ob.attn_norm.weight, device), ob.attn_norm.eps),
                            RMSNorm(to_torch(ob.mlp_norm.weight, device), ob.mlp_norm.eps),
                            num_heads=a.num_heads, head_dim=a.head_dim, causal=a.causal)


def llm_from_oracle(om, device="cuda"):
    from xax_b200.arch.attention import Embedding, Linear, RMSNorm
    from xax_b200.arch.llm import LLM, LLMConfig

    c = om.config
    cfg = LLMConfig(vocab_size=c.vocab_size, embed_dim=c.embed_dim, q_heads=c.q_heads, kv_heads=c.kv_heads,
                    head_dim=c.head_dim, num_layers=c.num_layers, max_tsz=c.max_tsz, rope_theta=c.rope_theta,
                    mlp_mult=c.mlp_mult, mlp_hidden_dim=c.mlp_hidden_dim, rms_eps=c.rms_eps)
    ew = to_torch(om.embed.weight, device)
    embed = Embedding(ew.shape[0], ew.shape[1], weight=ew)
    tied = om.lm_head.weight is om.embed.weight
    hw = ew if tied else to_torch(om.lm_head.weight, device)
    head = Linear(hw.shape[1], hw.shape[0], use_bias=False, weight=hw)
    return LLM(embed, [block_from_oracle(b, device) for b in om.blocks],
               RMSNorm(to_torch(om.norm.weight, device), om.norm.eps), head, cfg)


def attn_setup(ops, B, T, Hq, Hkv, D, max_len, starts, theta, seed, rotated=True):
    """Seeded decode / prefill attention case shared by the kernel tests: K/V caches holding ``starts[b]``
    tokens per sequence (K stored rotated like the reference, or as projected when ``rotated`` is False), T
    new tokens per sequence appended through the device kernel (checked bit for bit against the oracle's
    rotation), and the oracle's attention output for the new tokens."""
    from oracle.attention import RotaryEmbedding

    rng = np.random.default_rng(seed)
    rope = RotaryEmbedding(D, theta, "concatenated")
    kc = np.zeros((B, max_len, Hkv, D), bf16)
    vc = np.zeros((B, max_len, Hkv, D), bf16)
    k_raw = np.zeros_like(kc)
    for b in range(B):
        n = starts[b]
        kr = rng.standard_normal((n, Hkv, D)).astype(np.float32).astype(bf16)
        k_raw[b, :n] = kr
        kc[b, :n] = rope.apply_rotary_embeddings(kr, np.arange(n, dtype=np.int32)) if n else kr
        vc[b, :n] = rng.standard_normal((n, Hkv, D)).astype(np.float32).astype(bf16)
    qkv = rng.standard_normal((B * T, (Hq + 2 * Hkv) * D)).astype(np.float32).astype(bf16)
    cos, sin = ops.rope_tables(D, theta, max_len, "cuda")
    pos = to_torch(np.asarray(starts, np.int32))
    kct, vct = to_torch(kc if rotated else k_raw), to_torch(vc)
    q_rot = ops.kv_append_rope(to_torch(qkv), B, T, Hq, Hkv, D, pos, cos, sin, kct, vct, store_rotated_k=rotated)
    # oracle: rotate q, k of the new tokens and append
    exp_out = np.zeros((B * T, Hq, D), bf16)
    from oracle.attention import dot_product_attention

    for b in range(B):
        rows = qkv[b * T:(b + 1) * T]
        q = rows[:, :Hq * D].reshape(T, Hq, D)
        k = rows[:, Hq * D:(Hq + Hkv) * D].reshape(T, Hkv, D)
        v = rows[:, (Hq + Hkv) * D:].reshape(T, Hkv, D)
        p = (np.arange(T) + starts[b]).astype(np.int32)
        qr, kr = rope.apply_rotary_embeddings(q, p), rope.apply_rotary_embeddings(k, p)
        kc[b, starts[b]:starts[b] + T] = kr
        vc[b, starts[b]:starts[b] + T] = v
        S = starts[b] + T
        allow = np.arange(S)[None, :] <= p[:, None]
        exp_out[b * T:(b + 1) * T] = dot_product_attention(qr, kc[b, :S], vc[b, :S], mask=allow)
        assert np.array_equal(to_numpy(q_rot)[b * T:(b + 1) * T].view(np.uint16), qr.view(np.uint16))
    if rotated:
        assert np.array_equal(to_numpy(kct).view(np.uint16), kc.view(np.uint16))
    assert np.array_equal(to_numpy(vct).view(np.uint16), vc.view(np.uint16))
    return q_rot, kct, vct, pos, cos, sin, exp_out
