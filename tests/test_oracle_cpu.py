"""CPU tests of the oracle: the reference's own relational tests re-expressed against the
restatement (xax tests/nn/test_fp8.py, test_attention.py, test_llm.py), and the committed golden
fixtures.  No GPU."""

import os

import numpy as np
import pytest

from helpers import bf16, cfg1_inputs, e4m3, f32, rel_fro
from oracle import attention as oattn
from oracle import fp8 as ofp8
from oracle import llm as ollm

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def as_bf16(a):
    return np.ascontiguousarray(a).view(bf16)


# ---- xax tests/nn/test_fp8.py ----------------------------------------------------------------

@pytest.mark.parametrize("dt,mx", [(ofp8.float8_e4m3fn, 448.0), (ofp8.float8_e5m2, 57344.0)])
def test_get_fp8_max(dt, mx):  # :19-25
    v = ofp8.get_fp8_max(dt)
    assert np.isfinite(v) and v > 0 and float(v) == mx


def test_compute_scale():  # :28-44
    fp8_max, prev = np.float32(448.0), np.float32(2.5)
    assert np.isclose(ofp8.compute_scale(np.float32(100.0), prev, fp8_max), 4.48)
    for bad in (0.0, -1.0, np.inf, np.nan):
        assert ofp8.compute_scale(np.float32(bad), prev, fp8_max) == prev
    m0 = ofp8.compute_scale(np.float32(100.0), prev, fp8_max, margin=0)
    m1 = ofp8.compute_scale(np.float32(100.0), prev, fp8_max, margin=1)
    assert np.isclose(m1, m0 / 2)
    # delayed mode: bf16 fp8_max against a float32 amax promotes to float32
    assert ofp8.compute_scale(np.float32(3.0), prev, ofp8.get_fp8_max(e4m3, bf16)).dtype == np.float32


def test_amax_history():  # :47-53
    h = ofp8.compute_amax_history(np.array([1.0, -5.0, 3.0], np.float32), np.zeros(4, np.float32))
    assert h[0] == 5.0 and len(h) == 4
    # roll(-1) then slot 0: old slot 0 wraps to the end, old slot 1 is dropped
    h2 = ofp8.compute_amax_history(np.array([2.0], np.float32), np.array([10.0, 11.0, 12.0, 13.0], np.float32))
    assert h2.tolist() == [2.0, 12.0, 13.0, 10.0]
    assert np.isnan(ofp8.compute_amax_history(np.array([1.0, np.nan], np.float32), np.zeros(2, np.float32))[0])


@pytest.mark.parametrize("dt", [ofp8.float8_e4m3fn, ofp8.float8_e5m2])
def test_quantize_dequantize(dt):  # :56-78
    rng = np.random.default_rng(42)
    x = rng.standard_normal((16, 16)).astype(np.float32)
    fp8_max = ofp8.get_fp8_max(dt)
    scale = fp8_max / np.max(np.abs(x))
    r = ofp8.quantize_dequantize(x, dt, scale)
    assert r.shape == x.shape and np.mean(np.abs(r - x) / (np.abs(x) + 1e-6)) < 0.05
    xo = np.array([-5.0, -1.0, 0.0, 1.0, 5.0], np.float32)
    ro = ofp8.quantize_dequantize(xo, dt, fp8_max / 5.0)
    assert np.all(np.sign(ro) == np.sign(xo))
    q = ofp8.quantize(np.array([1000.0, -1000.0], np.float32), dt, np.float32(1.0))
    assert np.all(np.abs(f32(q)) <= fp8_max)


def test_bf16_intermediate_rounding_matters():
    """The product x*scale is rounded to bf16 before the e4m3 cast (compute dtype bf16); skipping
    that rounding changes ~2 % of the bytes, so the CUDA kernel must reproduce it."""
    x, _, _, _ = cfg1_inputs(M=64, K=512, N=8)
    s = ofp8.current_scale(x, e4m3, bf16)
    strict = ofp8.quantize(x, e4m3, s, bf16).view(np.uint8)
    loose = np.clip(f32(x) * f32(s), -448, 448).astype(e4m3).view(np.uint8)
    frac = np.mean(strict != loose)
    assert 0.002 < frac < 0.06


def test_fp8_scales_init_and_linear():  # :81-118
    s = ofp8.init_fp8_scales(16)
    assert s.input_scale == 1.0 and s.kernel_scale == 1.0 and s.input_amax_history.shape == (16,)
    rng = np.random.default_rng(0)
    layer = ofp8.Fp8Linear.random(32, 64, rng)
    x = rng.standard_normal((8, 32)).astype(np.float32).astype(bf16)
    out = layer.call_rows(x)[0]  # jax.vmap(layer)(x)
    assert out.shape == (8, 64)
    std = ofp8.Fp8Linear(layer.weight, layer.bias, use_fp8=False)
    o_std, sc = std(x)
    assert sc is None and np.allclose(f32(o_std), f32((f32(x) @ f32(layer.weight).T).astype(bf16)) + f32(layer.bias), atol=2e-2)
    assert np.allclose(f32(out), f32(o_std), atol=1.0, rtol=0.1)
    o1, new = layer(x[0], ofp8.init_fp8_scales(16))
    assert o1.shape == (64,) and np.any(new.input_amax_history != 0.0)
    # per-row call == calling the layer on each row (what vmap means)
    for r in range(3):
        assert np.array_equal(layer(x[r])[0].view(np.uint16), out[r].view(np.uint16))


@pytest.mark.parametrize("dt,atol", [(ofp8.float8_e4m3fn, 0.5), (ofp8.float8_e5m2, 1.0)])
def test_fp8_matmul(dt, atol):  # :121-135
    rng = np.random.default_rng(0)
    a = rng.standard_normal((4, 16)).astype(np.float32)
    b = rng.standard_normal((16, 8)).astype(np.float32)
    r = ofp8.fp8_matmul(a, b, fp8_dtype=dt)
    assert r.shape == (4, 8) and np.allclose(f32(r), a @ b, atol=atol, rtol=0.1)


def test_matmul_modes_agree_on_one_linear_and_drift_when_chained():
    x, w, b, _ = cfg1_inputs(M=64, K=512, N=256)
    layer = ofp8.Fp8Linear(w, b)
    a = layer(x)[0]
    ofp8.MATMUL_MODE = "fp8_gemm"
    try:
        g = layer(x)[0]
    finally:
        ofp8.MATMUL_MODE = "qdq"
    assert rel_fro(f32(g), f32(a)) < 1e-2


# ---- xax tests/nn/test_attention.py / test_llm.py --------------------------------------------

def _toy(use_fp8, dtype=bf16, std=0.3, seed=0):
    cfg = ollm.LLMConfig(vocab_size=256, embed_dim=64, q_heads=4, kv_heads=2, head_dim=16, num_layers=2, max_tsz=128)
    return ollm.LLM.build(cfg, np.random.default_rng(seed), use_fp8=use_fp8, std=std, dtype=dtype)


@pytest.mark.parametrize("chunks", [[1] * 8, [3, 2, 3], [8]])
def test_cached_forward_equals_full_forward(chunks):  # test_attention.py:10-102 (fp32, atol 1e-4)
    m = _toy(False, dtype=np.float32)
    toks = np.random.default_rng(1).integers(0, 256, 8)
    full = m.forward(toks)
    caches, outs, i = m.init_cache(8, np.float32), [], 0
    for n in chunks:
        lg, caches = m.forward(toks[i:i + n], caches=caches)
        outs.append(lg)
        i += n
    assert np.allclose(np.concatenate(outs), full, atol=1e-4)
    assert int(caches[0]["self_attn"]["position"]) == 8


def test_logits_shape_tying_and_greedy_loop():  # test_llm.py:20-112
    m = _toy(True)
    assert m.forward(np.array([1, 2, 3, 4, 5])).shape == (5, 256)
    assert m.lm_head.weight is m.embed.weight
    toks, n = ollm.llm_generate_greedy(m, [ord("h"), ord("i")], ord("!"), 3)
    assert n <= 5 and len(toks) == 5
    # the generate loop equals a hand-written cache-decode loop token for token
    prompt = np.array([11, 17, 23], np.int32)
    caches = m.init_cache(9, bf16)
    lg, caches = m.forward(prompt, caches=caches)
    seq = list(prompt) + [int(np.argmax(f32(lg[-1])))]
    while len(seq) < 9:
        lg, caches = m.forward(np.array(seq[-1:], np.int32), caches=caches)
        seq.append(int(np.argmax(f32(lg[-1]))))
    got, n = ollm.llm_generate_greedy(m, prompt, -1, 6)
    assert n == 9 and got.tolist() == seq
    assert ollm.llm_generate_greedy(m, prompt, -1, 0)[1] == 3


def test_rope_positions_are_rounded_to_bf16():
    """int32 positions meet bf16 frequencies: position 257 rotates like 256 (bf16 has 8 bits)."""
    rope = oattn.RotaryEmbedding(64, 10000.0, "concatenated")
    c, s = rope.get_rotary_embeddings(np.array([256, 257, 8191, 8192], np.int32), bf16)
    assert np.array_equal(c[0].view(np.uint16), c[1].view(np.uint16))
    assert np.array_equal(s[2].view(np.uint16), s[3].view(np.uint16))
    x = np.random.default_rng(0).standard_normal((4, 2, 64)).astype(np.float32).astype(bf16)
    y = rope.apply_rotary_embeddings(x, np.zeros(4, np.int32))
    assert np.array_equal(y.view(np.uint16), x.view(np.uint16))  # angle 0: identity
    yi = oattn.RotaryEmbedding(64, 10000.0, "interleaved").apply_rotary_embeddings(x, np.arange(4, dtype=np.int32))
    assert yi.shape == x.shape
    with pytest.raises(ValueError):
        oattn.RotaryEmbedding(64, style="bogus").apply_rotary_embeddings(x)


def test_gqa_groups_consecutive_query_heads():
    rng = np.random.default_rng(2)
    q = rng.standard_normal((3, 4, 16)).astype(np.float32)
    k = rng.standard_normal((5, 2, 16)).astype(np.float32)
    v = rng.standard_normal((5, 2, 16)).astype(np.float32)
    out = oattn.dot_product_attention(q, k, v)
    k4, v4 = np.repeat(k, 2, axis=1), np.repeat(v, 2, axis=1)  # heads 0,1 -> kv 0; 2,3 -> kv 1
    assert np.allclose(out, oattn.dot_product_attention(q, k4, v4), atol=1e-6)
    causal = oattn.dot_product_attention(q, k[:3], v[:3], is_causal=True)
    assert np.allclose(causal[0], np.broadcast_to(v[0][[0, 0, 1, 1]], (4, 16)), atol=1e-6)  # first query sees key 0 only


def test_init_cache_requires_max_len():
    m = _toy(False)
    with pytest.raises(ValueError):
        m.blocks[0].self_attn.init_cache(None)


# ---- golden fixtures --------------------------------------------------------------------------

def test_golden_fp8_linear():
    g = np.load(os.path.join(GOLD, "fp8_linear_cfg1_reduced.npz"))
    x, w, b = as_bf16(g["x"]), as_bf16(g["w"]), as_bf16(g["bias"])
    sc = ofp8.Fp8Scales(g["in_scale"], g["in_hist"], g["k_scale"], g["k_hist"])
    out, new = ofp8.Fp8Linear(w, b)(x, sc)
    assert np.array_equal(ofp8.quantize(x, e4m3, sc.input_scale, bf16).view(np.uint8), g["q_x"])
    assert np.array_equal(ofp8.quantize(w, e4m3, sc.kernel_scale, bf16).view(np.uint8), g["q_w"])
    assert np.array_equal(new.input_amax_history, g["new_in_hist"]) and new.input_scale == g["new_in_scale"]
    assert np.array_equal(new.kernel_amax_history, g["new_k_hist"]) and new.kernel_scale == g["new_k_scale"]
    assert np.array_equal(out.view(np.uint16), g["out_delayed"])
    assert np.array_equal(ofp8.Fp8Linear(w, b)(x)[0].view(np.uint16), g["out_current"])
    o, s, q = ofp8.Fp8Linear(w, b).call_rows(x)
    assert np.array_equal(o.view(np.uint16), g["out_rows"]) and np.array_equal(q.view(np.uint8), g["q_rows"])
    assert np.array_equal(s.view(np.uint16), g["row_scale"])


def test_golden_rope_and_attention():
    g = np.load(os.path.join(GOLD, "rope_decode_attention.npz"))
    rope = oattn.RotaryEmbedding(128, 500000.0, "concatenated")
    c, s = rope.get_rotary_embeddings(g["positions"], bf16)
    assert np.array_equal(c.view(np.uint16), g["cos"]) and np.array_equal(s.view(np.uint16), g["sin"])
    q, k, v = as_bf16(g["q"]), as_bf16(g["k_cache"]), as_bf16(g["v_cache"])
    for b, n in enumerate(g["lengths"]):
        qr = rope.apply_rotary_embeddings(q[b][None], np.array([n - 1], np.int32))
        out = oattn.dot_product_attention(qr, k[b, :n], v[b, :n])[0]
        assert np.array_equal(out.view(np.uint16), g["out"][b])


def test_golden_toy_llm():
    g = np.load(os.path.join(GOLD, "toy_llm_greedy.npz"))
    cfg = ollm.LLMConfig(vocab_size=256, embed_dim=64, q_heads=4, kv_heads=2, head_dim=64, num_layers=2, max_tsz=128,
                         mlp_hidden_dim=128)
    om = ollm.LLM.build(cfg, np.random.default_rng(0), use_fp8=False, std=0.3)
    toks, n = ollm.llm_generate_greedy(om, [11, 17, 23], -1, 6)
    assert np.array_equal(toks, g["tokens"]) and n == int(g["final_len"])
    assert np.array_equal(om.forward(np.array([11, 17, 23], np.int32)).view(np.uint16), g["prompt_logits"])


def test_hf_config_parsing_defaults_and_aliases():
    """hf_config_to_llm_config: the reference's defaults and alias names (xax/arch/llm.py:1027-1188)."""
    import pytest

    from xax_b200.arch.hf import hf_config_to_llm_config

    c = hf_config_to_llm_config({"n_embd": 512, "n_head": 8, "n_layer": 3, "vocab_size": 1000})
    assert (c.embed_dim, c.q_heads, c.kv_heads, c.head_dim, c.num_layers) == (512, 8, 4, 64, 3)
    assert c.mlp_hidden_dim == 2048 and c.mlp_mult == 4 and c.rope_theta == 10000.0 and c.rms_eps == 1e-6
    assert not c.attention_bias and not c.mlp_bias and not c.use_qk_norm and not c.uses_yarn
    q = hf_config_to_llm_config({"hidden_size": 1024, "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 128,
                                 "num_hidden_layers": 2, "vocab_size": 5, "intermediate_size": 3072, "model_type": "qwen3",
                                 "rope_theta": 1e6, "rms_norm_eps": 1e-6, "attention_bias": True,
                                 "rope_scaling": {"rope_type": "yarn", "factor": 4.0,
                                                  "original_max_position_embeddings": 32768}})
    assert q.head_dim == 128 and q.use_qk_norm and q.attention_bias and q.mlp_mult == 3
    assert q.uses_yarn and q.rope_factor == 4.0 and q.rope_original_max_position_embeddings == 32768
    assert q.rope_beta_slow == 1.0 and q.rope_beta_fast == 32.0
    with pytest.raises(ValueError, match="hidden_size"):
        hf_config_to_llm_config({"num_attention_heads": 8, "num_hidden_layers": 1, "vocab_size": 10})


def test_weight_quantisation_cache_changes_nothing():
    """oracle.fp8.CACHE_WEIGHT_QUANT computes the weight's scale / bytes once per layer: same outputs, both
    matmul executions, whole-tensor and per-row scaling."""
    from oracle import fp8 as ofp8

    rng = np.random.default_rng(21)
    w = (rng.standard_normal((48, 64)) * 0.05).astype(np.float32).astype(ofp8.bfloat16)
    x = rng.standard_normal((9, 64)).astype(np.float32).astype(ofp8.bfloat16)
    layer = ofp8.Fp8Linear(w, None)
    outs = {}
    for cache in (False, True):
        ofp8.CACHE_WEIGHT_QUANT = cache
        try:
            for mode in ("qdq", "fp8_gemm"):
                ofp8.MATMUL_MODE = mode
                for _ in range(2):
                    outs[(cache, mode)] = (layer(x)[0], layer.call_rows(x)[0])
        finally:
            ofp8.CACHE_WEIGHT_QUANT, ofp8.MATMUL_MODE = False, "qdq"
    for mode in ("qdq", "fp8_gemm"):
        for a, b in zip(outs[(False, mode)], outs[(True, mode)]):
            assert np.array_equal(np.asarray(a).view(np.uint16), np.asarray(b).view(np.uint16))


def test_sampling_restatement_properties():
    """xax/arch/llm.py:1446-1489 / :1547-1570 as restated in oracle.llm: the nucleus always holds the arg-max,
    shrinks to it as top_p -> 0, is everything at top_p = 1; masks use the most negative finite value; the
    quantile draw is monotone in u."""
    from oracle import llm as ollm

    rng = np.random.default_rng(22)
    lg = (rng.standard_normal((4, 300)) * 2).astype(np.float32).astype(ollm.bfloat16)
    order, probs, keep = ollm.nucleus(lg[0], 0.7, 0.9)
    assert order[0] == int(np.argmax(lg[0].astype(np.float32))) and keep[0]
    assert abs(float(probs.sum()) - 1.0) < 1e-4 and float(probs[keep].sum()) <= 0.9 + 1e-6
    assert not keep[int(keep.sum()):].any()  # a prefix of the sorted order
    assert ollm.nucleus(lg[0], 0.7, 1e-6)[2].sum() == 1 and ollm.nucleus(lg[0], 0.7, 1.0)[2].all()
    toks = [int(ollm.sample_next_token(lg[:1], 0.7, 0.9, np.array([u], np.float32))[0, 0]) for u in np.linspace(0, 0.999, 50)]
    ranks = [int(np.nonzero(order == t)[0][0]) for t in toks]
    assert ranks == sorted(ranks) and ranks[0] == 0
    assert np.array_equal(ollm.sample_next_token(lg, 0.0, 0.9)[:, 0], np.argmax(lg.astype(np.float32), -1))
    m = ollm.apply_sampling_mask(lg[:1], 1, 7, 3, (10, 20))  # EOS 7 not yet allowed: only 10..19 survive
    low = np.asarray(m.astype(np.float32))[0]
    assert (low[:10] == low[25]).all() and low[25] < -3e38 and 10 <= int(np.argmax(low)) < 20
    m2 = ollm.apply_sampling_mask(lg[:1], 3, 7, 3, (10, 20))
    assert float(m2.astype(np.float32)[0, 7]) == float(lg[0, 7].astype(np.float32))
    with pytest.raises(ValueError, match="max_id > min_id"):
        ollm.apply_sampling_mask(lg[:1], 0, -1, 0, (5, 5))
