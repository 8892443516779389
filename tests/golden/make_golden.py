"""Regenerates the golden fixtures in this directory from the CPU oracle.

    python tests/golden/make_golden.py

The reference (JAX) cannot run in this environment and its own tests hold no golden values
for this path, so these vectors pin the ORACLE (oracle/), not the reference: they keep the
oracle from drifting unnoticed and give the GPU tests byte-level targets that do not need the
oracle's code at hand.  Inputs are seeded NumPy draws with the benchmark's distributions at
reduced sizes.
"""

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

from helpers import bf16, cfg1_inputs, e4m3  # noqa: E402
from oracle import attention as oattn  # noqa: E402
from oracle import fp8 as ofp8  # noqa: E402
from oracle import llm as ollm  # noqa: E402


def u16(a):
    return np.ascontiguousarray(a).view(np.uint16)


def fp8_linear_cfg1_reduced():
    """benchmark config 1 at M=64, K=256, N=128: delayed scaling with a 16-deep pre-filled history."""
    x, w, b, rng = cfg1_inputs(M=64, K=256, N=128, seed=0)
    hist = np.zeros(16, np.float32)
    for _ in range(16):
        d = rng.standard_normal(x.shape).astype(np.float32)
        hist = ofp8.compute_amax_history(np.where(rng.random(d.shape) < 1e-3, d * 20, d).astype(bf16), hist)
    fp8_max = ofp8.get_fp8_max(e4m3, bf16)
    khist = np.full(16, np.float32(ofp8.amax_of(w)), np.float32)
    sc = ofp8.Fp8Scales(ofp8.compute_scale(np.max(hist), np.float32(1), fp8_max), hist,
                        ofp8.compute_scale(np.max(khist), np.float32(1), fp8_max), khist)
    out, new = ofp8.Fp8Linear(w, b)(x, sc)
    out_cur, _ = ofp8.Fp8Linear(w, b)(x)
    out_rows, row_scale, q_rows = ofp8.Fp8Linear(w, b).call_rows(x)
    np.savez_compressed(
        os.path.join(HERE, "fp8_linear_cfg1_reduced.npz"),
        x=u16(x), w=u16(w), bias=u16(b), in_scale=sc.input_scale, in_hist=hist, k_scale=sc.kernel_scale, k_hist=khist,
        q_x=ofp8.quantize(x, e4m3, sc.input_scale, bf16).view(np.uint8),
        q_w=ofp8.quantize(w, e4m3, sc.kernel_scale, bf16).view(np.uint8),
        new_in_hist=new.input_amax_history, new_in_scale=new.input_scale, new_k_hist=new.kernel_amax_history,
        new_k_scale=new.kernel_scale, out_delayed=u16(out), out_current=u16(out_cur), out_rows=u16(out_rows),
        row_scale=u16(row_scale), q_rows=q_rows.view(np.uint8))


def rope_and_decode_attention():
    """RoPE table rows (theta 5e5, D=128) and a reduced benchmark config 3: B=3, 8q/2kv heads."""
    rope = oattn.RotaryEmbedding(128, 500000.0, "concatenated")
    pos = np.array([0, 1, 2, 255, 256, 257, 513, 1023, 4097, 8191], np.int32)
    cos, sin = rope.get_rotary_embeddings(pos, bf16)
    rng = np.random.default_rng(3)
    B, Hq, Hkv, D, lens = 3, 8, 2, 128, [70, 129, 300]
    max_len = 320
    k = np.zeros((B, max_len, Hkv, D), bf16)
    v = np.zeros((B, max_len, Hkv, D), bf16)
    q = rng.standard_normal((B, Hq, D)).astype(np.float32).astype(bf16)
    out = np.zeros((B, Hq, D), bf16)
    for b, n in enumerate(lens):
        kr = rng.standard_normal((n, Hkv, D)).astype(np.float32).astype(bf16)
        k[b, :n] = rope.apply_rotary_embeddings(kr, np.arange(n, dtype=np.int32))
        v[b, :n] = rng.standard_normal((n, Hkv, D)).astype(np.float32).astype(bf16)
        qr = rope.apply_rotary_embeddings(q[b][None], np.array([n - 1], np.int32))
        out[b] = oattn.dot_product_attention(qr, k[b, :n], v[b, :n])[0]
    np.savez_compressed(os.path.join(HERE, "rope_decode_attention.npz"), positions=pos, cos=u16(cos), sin=u16(sin),
                        q=u16(q), k_cache=u16(k), v_cache=u16(v), lengths=np.array(lens, np.int32), out=u16(out))


def toy_llm_greedy():
    """2-layer GQA toy model (the reference's test config with head_dim 64), bf16 linears:
    greedy tokens and the logits of the prompt."""
    cfg = ollm.LLMConfig(vocab_size=256, embed_dim=64, q_heads=4, kv_heads=2, head_dim=64, num_layers=2, max_tsz=128,
                         mlp_hidden_dim=128)
    om = ollm.LLM.build(cfg, np.random.default_rng(0), use_fp8=False, std=0.3)
    toks, n = ollm.llm_generate_greedy(om, [11, 17, 23], -1, 6)
    logits = om.forward(np.array([11, 17, 23], np.int32))
    np.savez_compressed(os.path.join(HERE, "toy_llm_greedy.npz"), tokens=toks, final_len=np.int32(n),
                        prompt_logits=u16(logits))


if __name__ == "__main__":
    fp8_linear_cfg1_reduced()
    rope_and_decode_attention()
    toy_llm_greedy()
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))
