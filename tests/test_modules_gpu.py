"""Module-level parity on the GPU: the xax-shaped API (Fp8Linear, TransformerBlock, LLM,
greedy generation) against the CPU oracle with shared weights and seeded inputs.

Tolerances: relative Frobenius error <= 1e-2 against the oracle's strict reference path;
greedy tokens equal on the toy model and >= 99 % top-1 agreement on the larger one."""

import numpy as np
import pytest
import torch

from helpers import (bf16, block_from_oracle, cfg1_inputs, e4m3, f32, llm_from_oracle, rel_fro, to_numpy, to_torch)

pytestmark = pytest.mark.gpu
TOL = 1e-2


@pytest.fixture(scope="module", autouse=True)
def _status():
    yield
    from xax_b200 import _lib

    _lib.device_status()


def test_fp8_linear_modes_vs_oracle():
    from oracle import fp8 as ofp8
    from xax_b200.nn.fp8 import Fp8Linear, Fp8Scales, init_fp8_scales

    x, w, b, rng = cfg1_inputs(M=96, K=512, N=256)
    ol = ofp8.Fp8Linear(w, b)
    layer = Fp8Linear(512, 256, weight=to_torch(w), bias=to_torch(b))
    # current scaling, whole tensor (apply_linear semantics)
    exp, _ = ol(x)
    out, sc = layer(to_torch(x))
    assert sc is None and out.shape == (96, 256)
    assert rel_fro(f32(to_numpy(out)), f32(exp)) < TOL
    # per-row (vmapped) semantics
    exp_r = ol.call_rows(x)[0]
    out_r, _ = layer(to_torch(x), per_row=True)
    assert rel_fro(f32(to_numpy(out_r)), f32(exp_r)) < TOL
    # a single vector, as the reference's own test calls it (tests/nn/test_fp8.py:112-118)
    s0 = init_fp8_scales(16)
    o1, ns = layer(to_torch(x[0]), scales=s0)
    e1, es = ol(x[0], ofp8.init_fp8_scales(16))
    assert o1.shape == (256,) and float(ns.input_amax_history.abs().max()) != 0.0
    assert np.array_equal(to_numpy(ns.input_amax_history), es.input_amax_history)
    assert np.array_equal(to_numpy(ns.kernel_amax_history), es.kernel_amax_history)
    assert to_numpy(ns.input_scale) == es.input_scale and to_numpy(ns.kernel_scale) == es.kernel_scale
    assert rel_fro(f32(to_numpy(o1)), f32(e1)) < 0.1  # unit scales: values underflow e4m3, loose like the reference
    # second call with the updated scales
    o2, ns2 = layer(to_torch(x), scales=ns)
    e2, es2 = ol(x, es)
    assert rel_fro(f32(to_numpy(o2)), f32(e2)) < TOL
    assert np.array_equal(to_numpy(ns2.input_amax_history), es2.input_amax_history)
    # FP8 disabled == plain matmul (tests/nn/test_fp8.py:99-105)
    plain = Fp8Linear(512, 256, weight=to_torch(w), bias=to_torch(b), use_fp8=False)
    op, sp = plain(to_torch(x))
    ep, _ = ofp8.Fp8Linear(w, b, use_fp8=False)(x)
    assert sp is None and rel_fro(f32(to_numpy(op)), f32(ep)) < 5e-3
    # FP8 close to plain, the reference's own loose bound (tests/nn/test_fp8.py:107-110)
    assert np.allclose(f32(to_numpy(out)), f32(to_numpy(op)), atol=1.0, rtol=0.1)


def test_fp8_free_functions():
    from oracle import fp8 as ofp8
    from xax_b200.nn import fp8

    rng = np.random.default_rng(42)
    x = rng.standard_normal((16, 16)).astype(np.float32).astype(bf16)
    scale = np.float32(448.0) / np.max(np.abs(f32(x)))
    q = fp8.quantize(to_torch(x), torch.float8_e4m3fn, torch.tensor(float(scale)), torch.bfloat16)
    assert np.array_equal(to_numpy(q).view(np.uint8), ofp8.quantize(x, e4m3, scale, bf16).view(np.uint8))
    r = fp8.quantize_dequantize(to_torch(x), torch.float8_e4m3fn, torch.tensor(float(scale)), torch.bfloat16)
    rel = np.abs(f32(to_numpy(r)) - f32(x)) / (np.abs(f32(x)) + 1e-6)
    assert rel.mean() < 0.05  # tests/nn/test_fp8.py:63-67
    big = fp8.quantize(torch.tensor([[1000.0, -1000.0] + [0.0] * 6], device="cuda"), torch.float8_e4m3fn,
                       torch.tensor(1.0))
    assert float(big.float().abs().max()) <= 448.0  # tests/nn/test_fp8.py:75-78
    h = fp8.compute_amax_history(torch.tensor([1.0, -5.0, 3.0, 0, 0, 0, 0, 0], device="cuda"),
                                 torch.zeros(4, device="cuda"))
    assert float(h[0]) == 5.0 and h.numel() == 4  # tests/nn/test_fp8.py:47-53
    with pytest.raises(ValueError, match="unsupported"):
        fp8.quantize(to_torch(x), torch.float16, torch.tensor(1.0))
    a = rng.standard_normal((4, 16)).astype(np.float32).astype(bf16)
    b = rng.standard_normal((16, 8)).astype(np.float32).astype(bf16)
    got = fp8.fp8_matmul(to_torch(a), to_torch(b))
    assert np.allclose(f32(to_numpy(got)), f32(a) @ f32(b), atol=0.5, rtol=0.1)  # tests/nn/test_fp8.py:121-135
    assert rel_fro(f32(to_numpy(got)), f32(ofp8.fp8_matmul(a, b))) < TOL


@pytest.mark.parametrize("fp8_attn,fp8_mlp,T,start", [(True, True, 160, 0), (True, False, 40, 0), (False, False, 130, 0),
                                                      (True, True, 1, 37)])
def test_transformer_block_vs_oracle(fp8_attn, fp8_mlp, T, start):
    """A reduced benchmark config 2: pre-norm block, GQA 8/2 heads x 64, SwiGLU, RoPE, prefill
    (and one decode step at a non-zero position) of B = 2 sequences."""
    from oracle.attention import build_block

    B, H, Hq, Hkv, D, F = 2, 256, 8, 2, 64, 640
    rng = np.random.default_rng(5)
    ob = build_block(rng, embed_dim=H, num_heads=Hq, num_kv_heads=Hkv, head_dim=D, ff_dim=F, rope_theta=10000.0,
                     norm_eps=1e-5, fp8_attn=fp8_attn, fp8_mlp=fp8_mlp, out_scale=1.0 / np.sqrt(2 * 22))
    blk = block_from_oracle(ob)
    x = rng.standard_normal((B, T, H)).astype(np.float32).astype(bf16)
    max_len = start + T + 3
    cache = blk.self_attn.init_cache(max_len, batch=B)
    ocaches = [ob.init_cache(max_len) for _ in range(B)]
    if start:  # warm the caches with `start` tokens first, on both sides
        x0 = rng.standard_normal((B, start, H)).astype(np.float32).astype(bf16)
        _, cache = blk.forward_tokens(to_torch(x0).reshape(B * start, H), B, start, cache=cache)
        for b in range(B):
            _, ocaches[b] = ob.forward(x0[b], cache=ocaches[b])
    out, cache = blk.forward_tokens(to_torch(x).reshape(B * T, H), B, T, cache=cache)
    got = to_numpy(out).reshape(B, T, H)
    for b in range(B):
        exp, oc = ob.forward(x[b], cache=ocaches[b])
        err = rel_fro(f32(got[b]), f32(exp))
        assert err < TOL, (b, err)
        n = start + T
        kerr = rel_fro(f32(to_numpy(cache["k"])[b, :n]), f32(oc["self_attn"]["k"][:n]))
        assert kerr < TOL, kerr
    assert to_numpy(cache["position"]).tolist() == [start + T] * B


def test_block_unbatched_api_and_donation():
    from oracle.attention import build_block

    H, Hq, Hkv, D, F, T = 128, 2, 1, 64, 256, 9
    rng = np.random.default_rng(9)
    ob = build_block(rng, embed_dim=H, num_heads=Hq, num_kv_heads=Hkv, head_dim=D, ff_dim=F, fp8_attn=True, fp8_mlp=True)
    blk = block_from_oracle(ob)
    x = rng.standard_normal((T, H)).astype(np.float32).astype(bf16)
    cache = blk.init_cache(max_len=16)
    assert cache["self_attn"]["k"].shape == (16, Hkv, D) and int(cache["self_attn"]["position"]) == 0
    y, c2 = blk.forward(to_torch(x), cache=cache, donate=False)
    assert int(cache["self_attn"]["position"]) == 0 and int(c2["self_attn"]["position"]) == T
    assert float(cache["self_attn"]["k"].float().abs().max()) == 0.0  # input cache untouched
    exp, _ = ob.forward(x, cache=ob.init_cache(16))
    assert rel_fro(f32(to_numpy(y)), f32(exp)) < TOL
    with pytest.raises(ValueError):
        blk.forward(to_torch(x).reshape(1, T, H))
    with pytest.raises(ValueError, match="max_len"):
        blk.self_attn.init_cache(None)


def _toy(use_fp8, std=0.2, dtype=bf16, seed=0, layers=2):
    from oracle import llm as ollm

    cfg = ollm.LLMConfig(vocab_size=256, embed_dim=64, q_heads=4, kv_heads=2, head_dim=64, num_layers=layers,
                         max_tsz=128, mlp_hidden_dim=128)
    om = ollm.LLM.build(cfg, np.random.default_rng(seed), use_fp8=use_fp8, std=std, dtype=dtype)
    return om, llm_from_oracle(om)


def test_llm_forward_shape_and_tying():
    from xax_b200.arch.llm import tie_embedding_and_head

    om, m = _toy(True)
    toks = torch.tensor([[1, 2, 3, 4, 5], [9, 8, 7, 6, 5]], dtype=torch.int32, device="cuda")
    logits, _ = m.forward_batch(toks)
    assert logits.shape == (2, 5, 256)  # xax tests/nn/test_llm.py:20-26
    tied = tie_embedding_and_head(m)
    assert tied.lm_head.weight is tied.embed.weight  # tests/nn/test_llm.py:29-32


def test_cached_decode_matches_full_forward():
    """xax tests/nn/test_attention.py:10-43 / 72-102: token-by-token and chunked (3+2+3) cached
    forward equal the one-shot forward (plain bf16 linears, so scales do not depend on T)."""
    om, m = _toy(False, std=0.3)
    toks = torch.tensor([5, 77, 130, 2, 9, 201, 33, 64], dtype=torch.int32, device="cuda")
    full = f32(to_numpy(m.forward(toks)))
    for chunks in ([1] * 8, [3, 2, 3]):
        caches = m.init_cache(8)
        outs, i = [], 0
        for n in chunks:
            lg, caches = m.forward(toks[i:i + n], caches=caches)
            outs.append(f32(to_numpy(lg)))
            i += n
        got = np.concatenate(outs)
        assert rel_fro(got, full) < 5e-3, chunks


def test_greedy_generation_matches_oracle():
    """xax tests/nn/test_llm.py:49-112: generation equals the cache-decode loop token for token
    (plain bf16 linears, as in the reference's own test; an FP8 model's greedy path is chaotic in
    the last bit of every GEMM, so for FP8 the tokens are compared teacher-forced below)."""
    from oracle import llm as ollm
    from xax_b200.arch.llm import llm_generate, llm_generate_batch, llm_generate_jit

    om, m = _toy(False, std=0.3)
    prompt = [11, 17, 23]
    exp, exp_len = ollm.llm_generate_greedy(om, prompt, -1, 6)
    toks, n = llm_generate_jit(m, torch.tensor(prompt, dtype=torch.int32, device="cuda"), -1, 6)
    assert n == exp_len and np.array_equal(toks.cpu().numpy(), exp)
    assert len(llm_generate(m, prompt, None, max_new_tokens=3)) == len(prompt) + 3  # tests/nn/test_llm.py:35-46
    # batched; graph replay and eager stepping agree
    pb = torch.tensor([prompt, [5, 6, 7]], dtype=torch.int32, device="cuda")
    g, _ = llm_generate_batch(m, pb, 6, use_graph=True)
    e, _ = llm_generate_batch(m, pb, 6, use_graph=False)
    assert torch.equal(g, e) and np.array_equal(g[0].cpu().numpy(), exp)
    exp2, _ = ollm.llm_generate_greedy(om, [5, 6, 7], -1, 6)
    assert np.array_equal(g[1].cpu().numpy(), exp2)
    # EOS stops the sequence (reference: done flag, :1582,1609)
    eos = int(exp[4])
    t2, n2 = llm_generate_jit(m, torch.tensor(prompt, dtype=torch.int32, device="cuda"), eos, 6)
    e2, en2 = ollm.llm_generate_greedy(om, prompt, eos, 6)
    assert n2 == en2 and np.array_equal(t2.cpu().numpy()[:n2], e2[:en2])


def test_fp8_greedy_graph_equals_eager_and_teacher_forced_tokens():
    from oracle import fp8 as ofp8
    from oracle import llm as ollm
    from xax_b200.arch.llm import llm_generate_batch

    om, m = _toy(True)
    pb = torch.tensor([[11, 17, 23], [5, 6, 7]], dtype=torch.int32, device="cuda")
    g, _ = llm_generate_batch(m, pb, 8, use_graph=True)
    e, _ = llm_generate_batch(m, pb, 8, use_graph=False)
    assert torch.equal(g, e)
    # teacher forcing: given the oracle's own token history, does the device pick the same next token?
    ofp8.MATMUL_MODE = "fp8_gemm"
    try:
        exp, _ = ollm.llm_generate_greedy(om, [11, 17, 23], -1, 8)
        full = f32(om.forward(exp[:-1]))
    finally:
        ofp8.MATMUL_MODE = "qdq"
    logits, _ = m.forward_batch(to_torch(exp[:-1].reshape(1, -1)))
    got = f32(to_numpy(logits))[0]
    agree = np.mean(np.argmax(got[2:], -1) == exp[3:])
    print(f"teacher-forced next-token agreement {agree:.2f}, logits rel err {rel_fro(got, full):.3e}")
    assert agree >= 0.75


def _oracle_pass(om, toks):
    """Oracle forward keeping every layer's input, the final residual stream and the logits."""
    B = toks.shape[0]
    layer_in, finals, logits = [[] for _ in om.blocks], [], []
    for b in range(B):
        x = om.embed_tokens(toks[b])
        for i, blk in enumerate(om.blocks):
            layer_in[i].append(x)
            x, _ = blk.forward(x)
        finals.append(x)
        logits.append(om.get_logits(om.norm(x)))
    return [np.stack(v) for v in layer_in], np.stack(finals), np.stack(logits)


def test_llm_reduced_cfg4_layerwise_and_logits():
    """Reduced benchmark config 4 (4 layers, hidden 512, 8/2 heads x 64, SwiGLU 1408, vocab 2048).

    Every FP8 cast is discontinuous, so two correct FP8 pipelines that differ in the last bit of
    one GEMM output drift apart over chained layers: the reference's own two executions of this
    model -- CPU "dequantise, bf16 matmul" and GPU "FP8 matmul" (xax/nn/fp8.py:3-11) -- differ by
    several per cent after one block and more at the logits (oracle against oracle, no GPU involved).
    Single linears and single attention calls meet 1e-2 against the strict oracle (test_kernels_gpu.py,
    test_baseline_shapes_gpu.py); here the stack is checked
      * layer by layer, each layer fed the activations of the oracle run with FP8-matmul semantics:
        no further from that execution than the reference's other execution (QDQ) of the same layer on
        the same input is (+25 %);
      * logits from the oracle's final hidden state: <= 1e-2 and >= 99 % top-1 agreement;
      * free-running logits against both oracle executions: no further from either than they are from
        each other (+25 %).
    The measured figures are printed for the record."""
    from oracle import fp8 as ofp8
    from oracle import llm as ollm

    cfg = ollm.LLMConfig(vocab_size=2048, embed_dim=512, q_heads=8, kv_heads=2, head_dim=64, num_layers=4,
                         mlp_hidden_dim=1408, rms_eps=1e-5)
    om = ollm.LLM.build(cfg, np.random.default_rng(1), use_fp8=True, std=0.05)
    m = llm_from_oracle(om)
    B, T = 2, 96
    toks = np.random.default_rng(2).integers(0, 2048, (B, T)).astype(np.int32)
    _, _, exp_qdq = _oracle_pass(om, toks)
    ofp8.MATMUL_MODE = "fp8_gemm"
    try:
        layer_in, finals, exp_fp8 = _oracle_pass(om, toks)
    finally:
        ofp8.MATMUL_MODE = "qdq"
    errs, refs = [], []
    for i, blk in enumerate(m.blocks):
        out, _ = blk.forward_tokens(to_torch(layer_in[i]).reshape(B * T, -1), B, T)
        nxt = layer_in[i + 1] if i + 1 < len(m.blocks) else finals
        errs.append(rel_fro(f32(to_numpy(out)).reshape(B, T, -1), f32(nxt)))
        qdq_out = np.stack([om.blocks[i].forward(layer_in[i][b])[0] for b in range(B)])  # QDQ execution, same input
        refs.append(rel_fro(f32(qdq_out), f32(nxt)))
    print("teacher-forced per-layer rel err vs FP8-matmul oracle:", [f"{e:.2e}" for e in errs],
          "| QDQ oracle vs FP8-matmul oracle, same layer, same input:", [f"{e:.2e}" for e in refs])
    h = m.norm(to_torch(finals).reshape(B * T, -1))
    got = f32(to_numpy(m.get_logits(h))).reshape(B, T, -1)
    head_err = rel_fro(got, f32(exp_fp8))
    head_top1 = np.mean(np.argmax(got, -1) == np.argmax(f32(exp_fp8), -1))
    print(f"lm_head on the oracle's final hidden state: rel err {head_err:.2e}, top-1 {head_top1:.4f}")
    assert head_err < TOL and head_top1 >= 0.99
    logits, _ = m.forward_batch(to_torch(toks))
    free = f32(to_numpy(logits))
    e_fp8, e_qdq = rel_fro(free, f32(exp_fp8)), rel_fro(free, f32(exp_qdq))
    agree = np.mean(np.argmax(free, -1) == np.argmax(f32(exp_fp8), -1))
    agree_oo = np.mean(np.argmax(f32(exp_qdq), -1) == np.argmax(f32(exp_fp8), -1))
    oo = rel_fro(f32(exp_fp8), f32(exp_qdq))
    print(f"free-running logits: {e_fp8:.3e} vs FP8-matmul oracle (top-1 {agree:.3f}), {e_qdq:.3e} vs QDQ oracle; "
          f"oracle vs oracle {oo:.3e} (top-1 {agree_oo:.3f})")
    for e, r in zip(errs, refs):
        assert e < 1.25 * r + 2e-3, (errs, refs)
    assert e_fp8 < 1.25 * oo and e_qdq < 1.25 * oo


def test_fp8_stack_greedy_64_steps_top1_agreement():
    """Greedy decoding of an FP8 stack over 64 new tokens against the oracle's loop (FP8-matmul execution).

    Two models of the reduced config-4 shape.  With independent random weights the logits are nearly flat
    (the top-1 margin is a fraction of the FP8 rounding noise), and no two executions -- the reference's own
    two included -- pick the same tokens for long: the figure is printed, and the bar is that the device
    agrees with the FP8-matmul oracle at least as often as the reference's QDQ execution does, minus 10
    points.  With the embedding tied to the head and the blocks' output projections scaled by 0.1 the residual
    stream carries the input token, the median top-1 margin is about ten times the rounding noise (margins of
    that order are what a trained model has), and the bar is the path's stated one: >= 99 % top-1 agreement,
    teacher-forced and free-running."""
    from oracle import fp8 as ofp8
    from oracle import llm as ollm
    from xax_b200.arch.llm import llm_generate_batch

    ofp8.CACHE_WEIGHT_QUANT = True
    try:
        for tied, bar in ((False, None), (True, 0.99)):
            cfg = ollm.LLMConfig(vocab_size=2048, embed_dim=512, q_heads=8, kv_heads=2, head_dim=64, num_layers=4,
                                 mlp_hidden_dim=1408, rms_eps=1e-5)
            om = ollm.LLM.build(cfg, np.random.default_rng(3), use_fp8=True, tie=tied, std=0.05)
            if tied:
                for blk in om.blocks:
                    for lin in (blk.self_attn.output_proj, blk.feed_forward.down):
                        lin.weight = (f32(lin.weight) * np.float32(0.1)).astype(bf16)
            m = llm_from_oracle(om)
            prompt = np.random.default_rng(4).integers(0, 2048, 16).astype(np.int32)
            n_new = 64
            ofp8.MATMUL_MODE = "fp8_gemm"
            try:
                exp, _ = ollm.llm_generate_greedy(om, prompt, -1, n_new)
                tf_logits = f32(om.forward(exp[:-1]))  # the oracle's logits along its own token history
            finally:
                ofp8.MATMUL_MODE = "qdq"
            qdq_logits = f32(om.forward(exp[:-1]))
            got, _ = llm_generate_batch(m, to_torch(prompt.reshape(1, -1)), n_new)
            got = got[0].cpu().numpy()
            free = float(np.mean(got[16:] == exp[16:]))
            first_diff = int(np.argmax(got != exp)) if (got != exp).any() else len(exp)
            dev_logits, _ = m.forward_batch(to_torch(exp[:-1].reshape(1, -1)))
            dev_logits = f32(to_numpy(dev_logits))[0]
            tf = float(np.mean(np.argmax(dev_logits[15:], -1) == exp[16:]))
            tf_ref = float(np.mean(np.argmax(qdq_logits[15:], -1) == exp[16:]))
            srt = np.sort(tf_logits[15:], axis=-1)
            margin = float(np.median(srt[:, -1] - srt[:, -2]))
            noise = float(np.sqrt(np.mean((dev_logits[15:] - tf_logits[15:]) ** 2)))
            print(f"greedy 64 steps, tied={tied}: free-running top-1 {free:.3f} (first difference at token {first_diff} of "
                  f"{len(exp)}), teacher-forced top-1 {tf:.3f} (reference QDQ vs FP8-matmul execution: {tf_ref:.3f}); "
                  f"median top-1 margin {margin:.3e}, rms logit difference {noise:.3e}")
            if bar is None:
                assert tf >= tf_ref - 0.10, (tf, tf_ref)
            else:
                assert tf >= bar and free >= bar, (tf, free)
    finally:
        ofp8.CACHE_WEIGHT_QUANT = False


@pytest.mark.parametrize("style", ["concatenated", "interleaved"])
def test_rotary_embedding_methods_match_oracle_bit_for_bit(style):
    """RotaryEmbedding.apply_rotary_embeddings / _apply_rotary_4d / _get_rotary_embeddings, both styles,
    default and explicit positions (position 257 rounds to 256 in bf16, there and here)."""
    from oracle import attention as oattn
    from xax_b200.arch.attention import RotaryEmbedding

    rng = np.random.default_rng(5)
    T, H, D = 300, 3, 64
    x = bf16(rng.standard_normal((T, H, D), dtype=np.float32))
    orope = oattn.RotaryEmbedding(D, base=10000.0, style=style)
    rope = RotaryEmbedding.build(D, base=10000.0, style=style)
    exp = orope.apply_rotary_embeddings(x)
    got = rope.apply_rotary_embeddings(to_torch(x))
    assert np.array_equal(to_numpy(got).view(np.uint16), np.asarray(exp).view(np.uint16))
    pos = np.array([0, 1, 255, 256, 257, 258, 1000, 7], dtype=np.int32)
    exp_p = orope.apply_rotary_embeddings(x[:8], pos.astype(x.dtype))
    got_p = rope.apply_rotary_embeddings(to_torch(x[:8]), torch.from_numpy(pos).cuda())
    assert np.array_equal(to_numpy(got_p).view(np.uint16), np.asarray(exp_p).view(np.uint16))
    # 4-D: (batch, seq, heads, head_dim) with per-sequence positions
    x4 = x[:24].reshape(2, 12, H, D)
    pos4 = np.stack([np.arange(12), np.arange(100, 112)]).astype(np.int32)
    got4 = rope.apply_rotary_embeddings(to_torch(x4), torch.from_numpy(pos4).cuda())
    exp4 = np.stack([np.asarray(orope.apply_rotary_embeddings(x4[b], pos4[b].astype(x.dtype))) for b in range(2)])
    assert np.array_equal(to_numpy(got4).view(np.uint16), exp4.view(np.uint16))
    cos, sin = rope._get_rotary_embeddings(torch.from_numpy(pos).cuda())
    ecos, esin = orope.get_rotary_embeddings(pos.astype(x.dtype), x.dtype)
    assert np.array_equal(to_numpy(cos).view(np.uint16), np.asarray(ecos).view(np.uint16))
    assert np.array_equal(to_numpy(sin).view(np.uint16), np.asarray(esin).view(np.uint16))


def test_apply_linear_batched_and_greedy_sampling_helper():
    """_apply_linear_batched (per-row current scaling; delayed scaling keeps the last row's update) and
    _sample_next_token's greedy branch (the sampling branch: test_sampling_gpu.py)."""
    from oracle import attention as oattn
    from oracle import fp8 as ofp8
    from xax_b200.arch.attention import _apply_linear_batched
    from xax_b200.arch.llm import _sample_next_token
    from xax_b200.nn.fp8 import Fp8Linear, init_fp8_scales

    x, w, b, rng = cfg1_inputs(M=24, K=256, N=128)
    ol = ofp8.Fp8Linear(w, b)
    layer = Fp8Linear(256, 128, weight=to_torch(w), bias=to_torch(b))
    x3 = x.reshape(2, 12, 256)
    exp, es = oattn.apply_linear_batched(ol, x3)
    got, gs = _apply_linear_batched(layer, to_torch(x3))
    assert es is None and gs is None and got.shape == (2, 12, 128)
    assert rel_fro(f32(to_numpy(got)), f32(exp)) < TOL
    s0 = ofp8.init_fp8_scales(16)
    s0 = ofp8.Fp8Scales(np.float32(4.0), s0.input_amax_history, np.float32(2000.0), s0.kernel_amax_history)
    g0 = init_fp8_scales(16)
    g0 = type(g0)(torch.tensor(4.0, device="cuda"), g0.input_amax_history, torch.tensor(2000.0, device="cuda"),
                  g0.kernel_amax_history)
    exp_d, es_d = oattn.apply_linear_batched(ol, x3, s0)
    got_d, gs_d = _apply_linear_batched(layer, to_torch(x3), g0)
    assert rel_fro(f32(to_numpy(got_d)), f32(exp_d)) < TOL
    assert np.array_equal(to_numpy(gs_d.input_amax_history), es_d.input_amax_history)  # the LAST row's amax
    assert to_numpy(gs_d.input_scale) == es_d.input_scale and to_numpy(gs_d.kernel_scale) == es_d.kernel_scale
    logits = bf16(rng.standard_normal((5, 1000), dtype=np.float32))
    logits[2, 10] = logits[2, 900] = 50.0  # tie: first index wins
    tok = _sample_next_token(to_torch(logits), 0.0, 0.9)
    assert tok.shape == (5, 1) and np.array_equal(to_numpy(tok)[:, 0], np.argmax(f32(logits), axis=-1))


def _write_hf_checkpoint(om, path, *, prefix="model.", transpose_o=False, tied=True, qk_norm=False):
    """The oracle model's weights under HuggingFace names (seeded synthetic tensors, no published model)."""
    import json

    from safetensors.torch import save_file

    c = om.config
    st = {f"{prefix}embed_tokens.weight": to_torch(om.embed.weight, "cpu")}
    for i, b in enumerate(om.blocks):
        a, f = b.self_attn, b.feed_forward
        for name, lin in (("q_proj", a.q_proj), ("k_proj", a.k_proj), ("v_proj", a.v_proj), ("o_proj", a.output_proj)):
            w = to_torch(lin.weight, "cpu")
            st[f"{prefix}layers.{i}.self_attn.{name}.weight"] = w.t().contiguous() if (transpose_o and name == "q_proj") else w
        for name, lin in (("gate_proj", f.gate), ("up_proj", f.up), ("down_proj", f.down)):
            st[f"{prefix}layers.{i}.mlp.{name}.weight"] = to_torch(lin.weight, "cpu")
        st[f"{prefix}layers.{i}.input_layernorm.weight"] = to_torch(b.attn_norm.weight, "cpu")
        st[f"{prefix}layers.{i}.post_attention_layernorm.weight"] = to_torch(b.mlp_norm.weight, "cpu")
    st[f"{prefix}norm.weight"] = to_torch(om.norm.weight, "cpu")
    if not tied:
        st["lm_head.weight"] = to_torch(om.lm_head.weight, "cpu")
    if qk_norm:
        g = np.random.default_rng(99)
        for i in range(len(om.blocks)):
            for n in ("q_norm", "k_norm"):
                st[f"model.layers.{i}.self_attn.{n}.weight"] = to_torch(
                    bf16(1 + 0.1 * g.standard_normal(c.head_dim, dtype=np.float32)), "cpu")
    save_file({k: v.contiguous() for k, v in st.items()}, str(path / "model.safetensors"))
    cfg = {"hidden_size": c.embed_dim, "num_attention_heads": c.q_heads, "num_key_value_heads": c.kv_heads,
           "num_hidden_layers": c.num_layers, "vocab_size": c.vocab_size, "intermediate_size": c.mlp_hidden_dim,
           "rope_theta": c.rope_theta, "rms_norm_eps": c.rms_eps, "head_dim": c.head_dim,
           "model_type": "qwen3" if qk_norm else "llama"}
    (path / "config.json").write_text(json.dumps(cfg))
    return st


@pytest.mark.parametrize("use_fp8,tied,prefix", [(True, True, "model."), (False, False, "")])
def test_pretrained_checkpoint_round_trip(tmp_path, use_fp8, tied, prefix):
    """A synthetic checkpoint in the HuggingFace naming scheme loads into the same model as handing the
    tensors over directly: logits equal bit for bit (tied and untied head, both name prefixes, a
    transposed projection)."""
    from oracle import llm as ollm
    from xax_b200.arch.hf import build_pretrained_llm, hf_config_to_llm_config, load_hf_config

    cfg = ollm.LLMConfig(vocab_size=256, embed_dim=128, q_heads=4, kv_heads=2, head_dim=64, num_layers=2, max_tsz=128,
                         mlp_hidden_dim=256, rope_theta=500000.0, rms_eps=1e-5)
    om = ollm.LLM.build(cfg, np.random.default_rng(3), use_fp8=use_fp8, tie=tied, std=0.2)
    _write_hf_checkpoint(om, tmp_path, prefix=prefix, transpose_o=True, tied=tied)
    parsed = hf_config_to_llm_config(load_hf_config(str(tmp_path)))
    assert (parsed.embed_dim, parsed.q_heads, parsed.kv_heads, parsed.head_dim, parsed.mlp_hidden_dim) == (128, 4, 2, 64, 256)
    assert parsed.rope_theta == 500000.0 and parsed.rms_eps == 1e-5 and not parsed.use_qk_norm
    loaded = build_pretrained_llm(str(tmp_path), use_fp8=use_fp8)
    direct = llm_from_oracle(om)
    toks = torch.tensor([[1, 2, 3, 4, 5, 6], [9, 8, 7, 6, 5, 4]], dtype=torch.int32, device="cuda")
    l1, _ = loaded.forward_batch(toks)
    l2, _ = direct.forward_batch(toks)
    assert torch.equal(l1, l2)
    assert (loaded.lm_head.weight is loaded.embed.weight) == tied


@pytest.mark.parametrize("fp8", [False, True])
def test_qk_norm_block_vs_oracle_prefill_and_decode(fp8):
    """QK-norm (xax/arch/attention.py:864-867) before RoPE: one block, prefill of 40 tokens then two cached
    decode steps, against the oracle with the same seeded norm weights."""
    from oracle import attention as oattn

    rng = np.random.default_rng(11)
    ob = oattn.build_block(rng, embed_dim=256, num_heads=4, num_kv_heads=2, head_dim=64, ff_dim=512, rope_theta=1e6,
                           norm_eps=1e-6, fp8_attn=fp8, fp8_mlp=fp8, std=0.05, use_qk_norm=True)
    blk = block_from_oracle(ob)
    assert blk.self_attn.q_norm is not None and blk.self_attn.k_norm is not None
    x = bf16(rng.standard_normal((42, 256), dtype=np.float32))
    cache_o = ob.init_cache(64)
    cache = blk.init_cache(64)
    exp, cache_o = ob.forward(x[:40], cache=cache_o)
    got, cache = blk.forward(to_torch(x[:40]), cache=cache)
    # normalised q and k sharpen the softmax, which amplifies the one-step e4m3 flips that separate any two
    # executions of chained FP8 linears (2e-2 between the reference's own two executions of two linears)
    assert rel_fro(f32(to_numpy(got)), f32(exp)) < (TOL if not fp8 else 3e-2)
    for t in (40, 41):
        exp, cache_o = ob.forward(x[t:t + 1], cache=cache_o)
        got, cache = blk.forward(to_torch(x[t:t + 1]), cache=cache)
        assert rel_fro(f32(to_numpy(got)), f32(exp)) < (TOL if not fp8 else 3e-2)
    # the cache holds normalised, rotated keys: compare the rows written so far
    kc = f32(to_numpy(cache["self_attn"]["k"]))[:42]
    assert rel_fro(kc, f32(cache_o["self_attn"]["k"])[:42]) < 5e-3


def test_pretrained_checkpoint_with_qk_norm(tmp_path):
    """A qwen3-style checkpoint (model_type qwen3, q_norm / k_norm weights per layer) loads with QK-norm on,
    and the norm weights change the logits."""
    from oracle import llm as ollm
    from xax_b200.arch.hf import build_pretrained_llm

    # embed_dim / q_heads = 64: the shared cross-attention block derives its head size from that quotient
    cfg = ollm.LLMConfig(vocab_size=256, embed_dim=256, q_heads=4, kv_heads=2, head_dim=64, num_layers=2, max_tsz=128,
                         mlp_hidden_dim=256, rope_theta=1e6, rms_eps=1e-6)
    om = ollm.LLM.build(cfg, np.random.default_rng(4), use_fp8=False, tie=True, std=0.2)
    st = _write_hf_checkpoint(om, tmp_path, qk_norm=True)
    m = build_pretrained_llm(str(tmp_path), use_fp8=False)
    a0 = m.blocks[0].self_attn
    assert m.config.use_qk_norm and a0.q_norm is not None and a0.k_norm is not None and a0.q_norm.eps == 1e-6
    assert torch.equal(a0.q_norm.weight.cpu(), st["model.layers.0.self_attn.q_norm.weight"])
    toks = torch.tensor([[1, 2, 3, 4, 5, 6]], dtype=torch.int32, device="cuda")
    l_qk, _ = m.forward_batch(toks)
    l_plain, _ = llm_from_oracle(om).forward_batch(toks)
    assert l_qk.shape == l_plain.shape and not torch.equal(l_qk, l_plain)
    # use_cross_attention wraps the loaded model with a freshly initialised shared cross-attention block (:706-708)
    with pytest.raises(ValueError, match="key is required"):
        build_pretrained_llm(str(tmp_path), use_fp8=False, use_cross_attention=True)
    x = build_pretrained_llm(str(tmp_path), use_fp8=False, use_cross_attention=True, key=5)
    assert type(x).__name__ == "CrossAttentionLLM" and x.cross_attn.num_heads == 4 and x.cross_attn.rotary_emb is None
    enc = torch.randn((9, 256), device="cuda").to(torch.bfloat16)
    out = x.forward(toks[0], encoder_output_sn=enc)
    assert out.shape == (6, 256) and bool(torch.isfinite(out.float()).all())
    assert torch.equal(x.forward(toks[0]), m.forward(toks[0]))  # without an encoder output: the plain model


def test_yarn_tables_match_oracle_and_feed_the_block():
    """YaRN (xax/arch/attention.py:401-441): tables bit-equal to the oracle's float32 computation, applied
    through the same kernels."""
    from oracle import attention as oattn
    from xax_b200.arch.attention import RotaryEmbedding

    kw = dict(base=1e6, style="concatenated", factor=4.0, original_max_position_embeddings=64, beta_slow=1.0, beta_fast=32.0)
    orope = oattn.RotaryEmbedding(64, **kw)
    rope = RotaryEmbedding.build(64, **kw)
    assert rope.uses_yarn
    pos = np.arange(300, dtype=np.int32)
    ecos, esin = orope.get_rotary_embeddings(pos, bf16(np.zeros(1)).dtype)
    cos, sin = rope.tables(300, "cuda")
    assert np.array_equal(to_numpy(cos)[:300].view(np.uint16), np.asarray(ecos).view(np.uint16))
    assert np.array_equal(to_numpy(sin)[:300].view(np.uint16), np.asarray(esin).view(np.uint16))
    x = bf16(np.random.default_rng(2).standard_normal((300, 2, 64), dtype=np.float32))
    exp = orope.apply_rotary_embeddings(x, pos)
    got = rope.apply_rotary_embeddings(to_torch(x))
    assert np.array_equal(to_numpy(got).view(np.uint16), np.asarray(exp).view(np.uint16))


@pytest.mark.parametrize("window,fp8", [(5, False), (100, False), (130, False), (300, True)])
def test_sliding_window_block_vs_oracle(window, fp8):
    """Sliding-window attention (xax/arch/attention.py:931-936: keys q - window .. q): chunked prefill of 400
    tokens (150 + 250, so later queries' windows start inside, and beyond, the first KV tile) and three cached
    decode steps, against the oracle."""
    from oracle import attention as oattn

    rng = np.random.default_rng(window)
    ob = oattn.build_block(rng, embed_dim=256, num_heads=4, num_kv_heads=2, head_dim=64, ff_dim=512, rope_theta=1e4,
                           fp8_attn=fp8, fp8_mlp=fp8, std=0.05, local_window_size=window)
    blk = block_from_oracle(ob)
    assert blk.self_attn.local_window_size == window
    x = bf16(rng.standard_normal((403, 256), dtype=np.float32))
    cache_o, cache = ob.init_cache(448), blk.init_cache(448)
    tol = TOL if not fp8 else 3e-2
    for lo, hi in ((0, 150), (150, 400), (400, 401), (401, 402), (402, 403)):
        exp, cache_o = ob.forward(x[lo:hi], cache=cache_o)
        got, cache = blk.forward(to_torch(x[lo:hi]), cache=cache)
        assert rel_fro(f32(to_numpy(got)), f32(exp)) < tol, (lo, hi)
    # and the kernels alone: windowed decode equals full decode when the window covers everything
    from xax_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(1)
    kc = torch.randn((3, 700, 2, 64), generator=g, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn((3, 700, 2, 64), generator=g, device="cuda", dtype=torch.bfloat16)
    q = torch.randn((3, 4, 64), generator=g, device="cuda", dtype=torch.bfloat16)
    pos = torch.tensor([0, 333, 699], dtype=torch.int32, device="cuda")
    assert torch.equal(ops.attn_decode_window(q, kc, vc, pos, 10_000), ops.attn_decode(q, kc, vc, pos))


def test_llm_with_sliding_and_full_attention_layers():
    """layer_attention_types (xax/arch/llm.py:113-120): a "sliding_attention" layer gets the window, a
    "full_attention" layer does not; sinks ride along (a per-head constant on the logits, which the softmax
    cancels).  Prefill + cached decode of a bf16 model against the oracle."""
    from oracle import llm as ollm
    from xax_b200.arch.llm import LLM, LLMConfig

    types = ("sliding_attention", "full_attention")
    ocfg = ollm.LLMConfig(vocab_size=256, embed_dim=128, q_heads=4, kv_heads=2, head_dim=64, num_layers=2, max_tsz=256,
                          mlp_hidden_dim=256, sliding_window_size=20, layer_attention_types=types)
    om = ollm.LLM.build(ocfg, np.random.default_rng(8), use_fp8=False, tie=True, std=0.05)
    m = llm_from_oracle(om)
    assert [b.self_attn.local_window_size for b in m.blocks] == [20, None]
    toks = np.random.default_rng(1).integers(0, 256, 70).astype(np.int32)
    exp = om.forward(toks)
    got = m.forward(torch.from_numpy(toks).cuda())
    assert rel_fro(f32(to_numpy(got)), f32(exp)) < TOL
    # LLM.build wires the same structure from the config
    cfg = LLMConfig(vocab_size=256, embed_dim=128, q_heads=4, kv_heads=2, head_dim=64, num_layers=2, mlp_hidden_dim=256,
                    sliding_window_size=20, layer_attention_types=types, use_attention_sinks=True)
    built = LLM.build(cfg, key=0, use_fp8=False)
    assert [b.self_attn.local_window_size for b in built.blocks] == [20, None]
    assert built.blocks[0].self_attn.sinks.shape == (4,)
