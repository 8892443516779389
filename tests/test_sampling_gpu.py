"""Temperature / top-p sampling, the generation loop's masks and the streaming generator against the
oracle's restatement of xax/arch/llm.py:1446-1489, :1547-1570 and :1617-1693.

The reference draws through jax.random.categorical from its own PRNG stream, which cannot be reproduced
outside JAX; kernel and oracle both take the uniforms as an input and pick the token at that quantile of
the nucleus in sorted order, so they are compared token for token.  Sums run in float32 on the device and
float64 in the oracle: a uniform that lands within rounding of a boundary between two tokens may go
either way, so the bars are "always inside the oracle's nucleus" and ">= 99 % the same token"."""

import ml_dtypes
import numpy as np
import pytest
import torch

from helpers import bf16, f32, llm_from_oracle, to_numpy, to_torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _status():
    yield
    from xax_b200 import _lib

    _lib.device_status()


def _logits(rows, vocab, seed, scale=3.0):
    return (np.random.default_rng(seed).standard_normal((rows, vocab)) * scale).astype(np.float32).astype(bf16)


@pytest.mark.parametrize("vocab,temperature,top_p", [(1000, 0.7, 0.9), (32000, 1.0, 0.5), (128256, 0.7, 0.9),
                                                      (2048, 0.3, 0.99), (517, 1.5, 1.0), (4096, 0.7, 1e-4)])
def test_sample_top_p_matches_oracle(vocab, temperature, top_p):
    from oracle import llm as ollm
    from xax_b200 import ops

    rows = 48
    lg = _logits(rows, vocab, vocab)
    lg[1, 7] = lg[1, 3] = lg[1].astype(np.float32).max() + 1  # a tie at the top: index order decides
    u = np.random.default_rng(1).random(rows).astype(np.float32)
    u[0], u[2] = 0.0, np.float32(0.99999)
    got = to_numpy(ops.sample_top_p(to_torch(lg), temperature, top_p, to_torch(u)))
    exp = ollm.sample_next_token(lg, temperature, top_p, u)[:, 0]
    for r in range(rows):
        order, probs, keep = ollm.nucleus(lg[r], temperature, top_p)
        # one token of slack at the nucleus's edge: the float32 cumulative sum decides the last member
        edge = set(order[: int(keep.sum()) + 1].tolist())
        assert int(got[r]) in edge, (r, int(got[r]))
    assert np.mean(got == exp) >= 0.95, np.mean(got == exp)
    if top_p <= 1e-3:  # a nucleus of one token: the arg-max, whatever u
        assert np.array_equal(got, np.argmax(f32(lg), -1))


def test_sampling_is_greedy_at_zero_temperature_and_respects_masks():
    from oracle import llm as ollm
    from xax_b200 import ops

    rows, vocab = 9, 5000
    lg = _logits(rows, vocab, 5)
    lg[2, 100] = lg[2, 4000] = np.float32(50.0)  # tie: first index
    t = to_torch(lg)
    assert np.array_equal(to_numpy(ops.sample_top_p(t, 0.0, 0.9)), np.argmax(f32(lg), -1))
    eos = int(np.argmax(f32(lg[0])))
    u = to_torch(np.full(rows, 0.5, np.float32))
    for temp in (0.0, 0.8):
        # EOS held back until enough tokens were generated (:1551-1554)
        got = to_numpy(ops.sample_top_p(t, temp, 0.9, u, eos_id=eos, allow_eos=False))
        assert eos not in got.tolist()
        m = ollm.apply_sampling_mask(lg, 0, eos, 3)
        exp = ollm.sample_next_token(m, temp, 0.9, np.full(rows, 0.5, np.float32))[:, 0]
        assert np.mean(got == exp) >= 0.85
        # allowed range [1000, 1010); EOS joins it once allowed (:1560-1566)
        got = to_numpy(ops.sample_top_p(t, temp, 0.9, u, allowed_token_range=(1000, 1010), eos_id=eos, allow_eos=False))
        assert all(1000 <= g < 1010 for g in got.tolist())
        got = to_numpy(ops.sample_top_p(t, temp, 0.9, u, allowed_token_range=(1000, 1010), eos_id=eos, allow_eos=True))
        assert all(1000 <= g < 1010 or g == eos for g in got.tolist()) and got[0] == eos
        m = ollm.apply_sampling_mask(lg, 5, eos, 3, (1000, 1010))
        assert np.array_equal(np.argmax(f32(m), -1) if temp == 0 else got, got)
    with pytest.raises(ValueError, match="max_id > min_id"):
        ops.sample_top_p(t, 0.7, 0.9, u, allowed_token_range=(10, 10))


def test_sampling_distribution_over_many_draws():
    """20000 rows of the same small distribution with uniforms on a regular grid: the empirical frequencies
    equal the nucleus probabilities to the grid's resolution."""
    from oracle import llm as ollm
    from xax_b200 import ops

    vocab, n = 64, 20000
    row = _logits(1, vocab, 11, scale=1.5)
    lg = np.repeat(row, n, axis=0)
    u = ((np.arange(n) + 0.5) / n).astype(np.float32)
    got = to_numpy(ops.sample_top_p(to_torch(lg), 0.9, 0.8, to_torch(u)))
    order, probs, keep = ollm.nucleus(row[0], 0.9, 0.8)
    p = np.where(keep, probs, 0.0).astype(np.float64)
    p /= p.sum()
    freq = np.bincount(got, minlength=vocab) / n
    want = np.zeros(vocab)
    want[order] = p
    assert np.abs(freq - want).max() < 2e-3, np.abs(freq - want).max()
    assert set(np.nonzero(freq)[0].tolist()) <= set(order[: int(keep.sum()) + 1].tolist())


def test_generation_with_sampling_masks_and_stream():
    """llm_generate_jit with temperature / top-p and both masks, and llm_generate_stream, on a bf16 toy model
    against the oracle's loops fed the same uniforms; num_samples > 1 of _sample_next_token."""
    from oracle import llm as ollm
    from xax_b200.arch.llm import TokenSampler, _sample_next_token, llm_generate_batch, llm_generate_jit, llm_generate_stream

    cfg = ollm.LLMConfig(vocab_size=256, embed_dim=64, q_heads=4, kv_heads=2, head_dim=64, num_layers=2, max_tsz=128,
                         mlp_hidden_dim=128)
    om = ollm.LLM.build(cfg, np.random.default_rng(0), use_fp8=False, std=0.3)
    m = llm_from_oracle(om)
    prompt = [11, 17, 23]
    n_new = 12
    u = np.random.default_rng(9).random(n_new).astype(np.float32)
    exp, exp_len = ollm.llm_generate_sampled(om, prompt, -1, n_new, 0.8, 0.9, u)
    sampler = TokenSampler(0.8, 0.9, uniforms=to_torch(u))
    got, lens = llm_generate_batch(m, torch.tensor([prompt], dtype=torch.int32, device="cuda"), n_new, sampler=sampler)
    free = np.mean(got[0].cpu().numpy() == exp)
    # teacher-forced: along the oracle's own token history, does the device draw the same token from u[i]?
    from xax_b200 import ops

    # (the toy model's distribution is nearly flat over 256 tokens: one bf16 ulp in a logit moves the quantile
    # boundaries, so the oracle's draw is taken from the device's own logits)
    logits, _ = m.forward_batch(to_torch(exp[:-1].reshape(1, -1)))
    rows = logits[0, 2:].contiguous()
    tf = to_numpy(ops.sample_top_p(rows, 0.8, 0.9, to_torch(u)))
    tf_exp = ollm.sample_next_token(to_numpy(rows), 0.8, 0.9, u)[:, 0]
    print(f"sampled generation: free-running agreement with the oracle's loop {free:.2f}, "
          f"draws from the same logits {np.mean(tf == tf_exp):.2f}")
    assert int(lens[0]) == exp_len and np.mean(tf == tf_exp) >= 0.9, (tf.tolist(), tf_exp.tolist())
    # masks: generated tokens stay inside the range; EOS only after min_new tokens
    eos = 40
    exp2, exp2_len = ollm.llm_generate_sampled(om, prompt, eos, n_new, 0.8, 0.95, u, (32, 48), 4)
    s2 = TokenSampler(0.8, 0.95, uniforms=to_torch(u), eos_id=eos, allowed_token_range=(32, 48), min_new_tokens_before_eos=4)
    got2, lens2 = llm_generate_batch(m, torch.tensor([prompt], dtype=torch.int32, device="cuda"), n_new, eos_id=eos, sampler=s2)
    g2 = got2[0].cpu().numpy()
    new = g2[3:int(lens2[0])]
    assert all(32 <= t < 48 for t in new.tolist()) and eos not in new[:4].tolist()
    assert np.array_equal(g2[:3], exp2[:3])
    # the reference-shaped entry points: seeded, reproducible, greedy when temperature <= 0
    pt = torch.tensor(prompt, dtype=torch.int32, device="cuda")
    a, na = llm_generate_jit(m, pt, -1, 8, None, 0.7, 0.9, 123)
    b, nb = llm_generate_jit(m, pt, -1, 8, None, 0.7, 0.9, 123)
    assert torch.equal(a, b) and na == nb == 11
    g, _ = llm_generate_jit(m, pt, -1, 8, None, 0.0, 0.9, 5, allowed_token_range=(100, 120))
    assert all(100 <= t < 120 for t in g[3:].tolist())
    with pytest.raises(ValueError, match="max_id > min_id"):
        llm_generate_jit(m, pt, -1, 8, None, 0.7, 0.9, 1, allowed_token_range=(5, 5))
    with pytest.raises(ValueError, match=">= 0"):
        llm_generate_jit(m, pt, -1, 8, None, 0.7, 0.9, 1, min_new_tokens_before_eos=-1)
    streamed = list(llm_generate_stream(m, prompt, None, max_new_tokens=8, temperature=0.7, top_p=0.9, key=123))
    assert streamed == a[3:].tolist()  # same seed, same draws as the jit entry
    greedy_stream = list(llm_generate_stream(m, prompt, None, max_new_tokens=5, temperature=0.0))
    exp_g, _ = ollm.llm_generate_greedy(om, prompt, -1, 5)
    assert greedy_stream == exp_g[3:].tolist()
    stop = greedy_stream[2]
    assert list(llm_generate_stream(m, prompt, stop, max_new_tokens=5, temperature=0.0)) == greedy_stream[:greedy_stream.index(stop)]
    # several samples per position
    lg = to_torch(_logits(5, 256, 2))
    s = _sample_next_token(lg, 0.7, 0.9, 3, num_samples=4)
    assert s.shape == (5, 4) and len(set(s.flatten().tolist())) > 4
    gz = _sample_next_token(lg, 0.0, 0.9, 3, num_samples=1)
    assert torch.equal(gz[:, 0].cpu(), torch.from_numpy(np.argmax(f32(to_numpy(lg)), -1).astype(np.int32)))
