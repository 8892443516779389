"""The parts of the module surface beside the cached forward: SelfAttentionBlock.__call__ (batched, no cache,
explicit RoPE positions), explicit masks, TransformerStack / Transformer and their cache layout."""

import numpy as np
import pytest
import torch

from helpers import bf16, block_from_oracle, f32, rel_fro, to_numpy, to_torch

pytestmark = pytest.mark.gpu
TOL = 1e-2


@pytest.fixture(scope="module", autouse=True)
def _status():
    yield
    from xax_b200 import _lib

    _lib.device_status()


@pytest.mark.parametrize("fp8,window", [(False, None), (True, None), (False, 40)])
def test_self_attention_call_batched_vs_oracle(fp8, window):
    """xax/arch/attention.py:700-773 against the oracle: (batch, seq, dim) in, one activation scale for the whole
    batch under FP8, positions given explicitly (a shifted and a strided sequence) and defaulted."""
    from oracle.attention import build_block

    rng = np.random.default_rng(7)
    ob = build_block(rng, embed_dim=256, num_heads=4, num_kv_heads=2, head_dim=64, ff_dim=512, rope_theta=1e4,
                     fp8_attn=fp8, fp8_mlp=False, std=0.05, local_window_size=window, attn_bias=True)
    attn_o, attn = ob.self_attn, block_from_oracle(ob).self_attn
    B, T = 3, 150
    x = rng.standard_normal((B, T, 256), dtype=np.float32).astype(bf16)
    pos = np.stack([np.arange(T), np.arange(T) + 500, np.arange(T) * 3]).astype(np.int32)
    for p in (None, pos):
        exp = attn_o.call_batched(x, p)
        got = attn(to_torch(x), None if p is None else to_torch(p))
        assert got.shape == (B, T, 256)
        err = rel_fro(f32(to_numpy(got)), f32(exp))
        assert err < (TOL if not fp8 else 2e-2), err  # two chained FP8 linears (see the stacked-FP8 note in test_modules_gpu)
    with pytest.raises(ValueError, match="rank 3"):
        attn(to_torch(x[0]))


def test_explicit_masks_are_accepted_when_they_are_the_builtin_mask():
    from oracle.attention import build_block

    rng = np.random.default_rng(8)
    ob = build_block(rng, embed_dim=128, num_heads=2, num_kv_heads=1, head_dim=64, ff_dim=256, fp8_attn=False,
                     fp8_mlp=False, std=0.05)
    blk = block_from_oracle(ob)
    T = 9
    x = to_torch(rng.standard_normal((T, 128), dtype=np.float32).astype(bf16))
    causal = torch.tril(torch.ones((T, T), dtype=torch.bool, device="cuda"))
    y0, _ = blk.forward(x)
    y1, _ = blk.forward(x, mask=causal)
    y2, _, _ = blk.self_attn.forward(blk.attn_norm(x), mask=causal.reshape(1, 1, T, T))
    assert torch.equal(y0, y1) and y2.shape == (T, 128)
    assert torch.equal(blk.self_attn.init_mask(T).cuda(), causal)
    # with a cache: (T, max_len), filled rows that are causal for the query
    cache = blk.init_cache(max_len=16)
    _, cache = blk.forward(x[:5], cache=cache)
    m = torch.zeros((4, 16), dtype=torch.bool, device="cuda")
    for i in range(4):
        m[i, :5 + i + 1] = True
    y3, c3 = blk.forward(x[5:], cache=cache, mask=m, donate=False)
    y4, _ = blk.forward(x[5:], cache=cache, donate=False)
    assert torch.equal(y3, y4) and int(c3["self_attn"]["position"]) == 9
    full = torch.ones((T, T), dtype=torch.bool, device="cuda")
    with pytest.raises(ValueError, match="explicit masks"):
        blk.forward(x, mask=full)


def test_transformer_stack_and_transformer():
    from xax_b200.arch.attention import Transformer, TransformerStack

    stack = TransformerStack.build(128, 2, 256, 3, key=1, causal=True, use_rotary_embeddings=True, context_length=33,
                                   num_kv_heads=1, head_dim=64)
    assert stack.num_layers == 3 and len(stack.layers) == 3
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((10, 128), generator=g, device="cuda").to(torch.bfloat16)
    cache = stack.init_cache()
    assert sorted(cache["layers"]) == ["layer_0", "layer_1", "layer_2"]
    assert cache["layers"]["layer_0"]["self_attn"]["k"].shape == (32, 1, 64)  # context_length - 1 rows (:660)
    y, c2 = stack.forward(x[:6], cache=cache)
    y2, c3 = stack.forward(x[6:], cache=c2)
    ref = x
    for layer in stack.layers:
        ref, _ = layer.forward(ref)
    got = torch.cat([y, y2])
    assert float((got.float() - ref.float()).norm() / ref.float().norm()) < 5e-3  # cached == one shot
    assert int(c3["layers"]["layer_2"]["self_attn"]["position"]) == 10
    y_nc, c_nc = stack.forward(x)  # no cache given: every layer attends within the tokens
    assert float((y_nc.float() - ref.float()).norm() / ref.float().norm()) < 5e-3
    with pytest.raises(ValueError, match="rmsnorm"):
        TransformerStack.build(128, 2, 256, 1, key=1, causal=True, use_rotary_embeddings=True, norm_type="layernorm")

    model = Transformer.build(96, 128, 2, 256, 2, output_size=96, key=3, causal=True, use_rotary_embeddings=True,
                              num_kv_heads=1, head_dim=64)
    toks = torch.tensor([5, 9, 33, 7], dtype=torch.int32, device="cuda")
    logits, _ = model.forward(toks)
    assert logits.shape == (4, 96) and torch.equal(model.predict_sequence(toks), logits)
    a = model.generate_sequence(toks, 6, temperature=0.8, key=11)
    b = model.generate_sequence(toks, 6, temperature=0.8, key=11)
    assert a.shape == (10,) and torch.equal(a, b) and torch.equal(a[:4], toks)
    assert int(a.max()) < 96 and int(a.min()) >= 0
    # a stack built without cross-attention ignores the context, as the reference's blocks do (:1483)
    h_dec, _ = model.decode(toks, toks)
    h_enc, _ = model.encode(toks)
    assert torch.equal(h_dec, h_enc)


def test_lora_branch_of_apply_linear_vs_oracle():
    """xax/arch/attention.py:44-51 with xax/nn/lora.py: y = x W^T + b + ((x A) B) * alpha / rank."""
    from oracle import attention as oattn
    from xax_b200.arch.attention import Linear, apply_linear
    from xax_b200.nn.lora import LoRALinear, loraize_linear

    rng = np.random.default_rng(12)
    I, O, R = 256, 136, 16
    w = (rng.standard_normal((O, I)) * 0.05).astype(np.float32).astype(bf16)
    b = (rng.standard_normal(O) * 0.1).astype(np.float32).astype(bf16)
    a = (rng.standard_normal((I, R)) / np.sqrt(I)).astype(np.float32).astype(bf16)
    bb = (rng.standard_normal((R, O)) * 0.3).astype(np.float32).astype(bf16)
    x = rng.standard_normal((3, 21, I), dtype=np.float32).astype(bf16)
    for bias in (b, None):
        exp = oattn.apply_linear(x, oattn.LoRALinear(w, bias, a, bb, R, alpha=8.0))
        layer = LoRALinear(to_torch(w), None if bias is None else to_torch(bias), to_torch(a), to_torch(bb), R, alpha=8.0)
        got = apply_linear(to_torch(x), layer)
        assert got.shape == (3, 21, O) and layer.scaling == 0.5
        assert rel_fro(f32(to_numpy(got)), f32(exp)) < 5e-3
    # a fresh LoRA layer (B = 0) equals its base layer (xax/nn/lora.py:63-64)
    base = Linear(I, O, use_bias=True, weight=to_torch(w), bias=to_torch(b))
    fresh = loraize_linear(base, 8, key=3)
    assert torch.equal(apply_linear(to_torch(x), fresh), apply_linear(to_torch(x), base))
    with pytest.raises(ValueError, match="rank"):
        loraize_linear(base, 0)


def test_dequantize_and_quantize_dequantize_match_oracle_bit_for_bit():
    """xax/nn/fp8.py:123-162: dequantize and the quantise -> dequantise round trip, bf16 and float32."""
    from oracle import fp8 as ofp8
    from xax_b200 import ops
    from xax_b200.nn import fp8

    rng = np.random.default_rng(13)
    x = (rng.standard_normal((37, 200)) * 3).astype(np.float32).astype(bf16)
    scale = ofp8.current_scale(x, ofp8.float8_e4m3fn, bf16)
    q = ofp8.quantize(x, ofp8.float8_e4m3fn, scale, bf16)
    got = fp8.dequantize(to_torch(q), torch.bfloat16, torch.tensor(float(f32(scale))))
    exp = ofp8.dequantize(q, bf16, scale)
    assert np.array_equal(to_numpy(got).view(np.uint16), exp.view(np.uint16))
    got32 = fp8.dequantize(to_torch(q), torch.float32, torch.tensor(float(f32(scale))))
    assert np.array_equal(to_numpy(got32), ofp8.dequantize(q, np.float32, f32(scale)))
    rt = fp8.quantize_dequantize(to_torch(x), torch.float8_e4m3fn, torch.tensor(float(f32(scale))), torch.bfloat16)
    assert np.array_equal(to_numpy(rt).view(np.uint16), ofp8.quantize_dequantize(x, ofp8.float8_e4m3fn, scale, bf16).view(np.uint16))
    # per-row scales through the functional layer
    qr, s_rows, _, _ = ops.quantize_current(to_torch(x[:, :192].copy()), 1)
    d = to_numpy(ops.dequantize(qr, s_rows))
    for r in range(5):
        e = ofp8.dequantize(to_numpy(qr)[r], bf16, to_numpy(s_rows)[r].astype(bf16))
        assert np.array_equal(d[r].view(np.uint16), e.view(np.uint16))
