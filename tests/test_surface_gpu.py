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
    with pytest.raises(ValueError, match="cross-attention"):
        model.decode(toks, toks)
