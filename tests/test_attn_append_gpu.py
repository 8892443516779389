"""Decode attention with the cache append fused in (xaxb_attn_decode_append) against the two separate calls it
replaces (xaxb_kv_append_rope, then xaxb_attn_decode / _cast / _window): outputs, e4m3 bytes, scales and the
cache rows written must be bit-identical -- the fused path is the one the model's decode step runs.  Positions
sit at the places where the new token's row changes tile or chunk: 0, 1, 126, 127, 128, 129, a chunk owned by
another CTA of the sequence, the last row of the cache."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bf16(shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def _case(B, Hq, Hkv, D, max_len, positions, seed):
    qkv = _bf16((B, (Hq + 2 * Hkv) * D), seed)
    kc = _bf16((B, max_len, Hkv, D), seed + 1)
    vc = _bf16((B, max_len, Hkv, D), seed + 2)
    pos = torch.tensor(positions, dtype=torch.int32, device="cuda")
    return qkv, kc, vc, pos


POSITIONS = [0, 1, 126, 127, 128, 129, 255, 256, 700, 1023]


@pytest.mark.parametrize("Hq,Hkv,D", [(8, 2, 128), (4, 4, 128), (16, 1, 128), (8, 4, 64), (32, 8, 128)])
def test_fused_append_equals_append_then_attention(Hq, Hkv, D):
    from xax_b200 import _lib, ops

    B, max_len = len(POSITIONS), 1024
    qkv, kc, vc, pos = _case(B, Hq, Hkv, D, max_len, POSITIONS, Hq * 100 + D)
    cos, sin = ops.rope_tables(D, 500000.0, max_len, "cuda")
    # the two separate calls, on copies of the caches
    kc_a, vc_a = kc.clone(), vc.clone()
    q_rot = ops.kv_append_rope(qkv, B, 1, Hq, Hkv, D, pos, cos, sin, kc_a, vc_a)
    want = ops.attn_decode(q_rot, kc_a, vc_a, pos)
    # fused
    kc_b, vc_b = kc.clone(), vc.clone()
    got, _, _, _ = ops.attn_decode_append(qkv, kc_b, vc_b, pos, cos, sin, Hq)
    _lib.device_status()
    assert torch.equal(got, want)
    assert torch.equal(kc_b, kc_a) and torch.equal(vc_b, vc_a)
    # only the new rows changed
    changed = (kc_b != kc).any(dim=(2, 3))
    for b, p in enumerate(POSITIONS):
        rows = changed[b].nonzero().flatten().tolist()
        assert rows == [p]


def test_fused_append_with_cast_window_and_unrotated_cache():
    from xax_b200 import _lib, ops

    Hq, Hkv, D = 32, 8, 128
    B, max_len = len(POSITIONS), 1024
    qkv, kc, vc, pos = _case(B, Hq, Hkv, D, max_len, POSITIONS, 7)
    cos, sin = ops.rope_tables(D, 500000.0, max_len, "cuda")

    kc_a, vc_a = kc.clone(), vc.clone()
    q_rot = ops.kv_append_rope(qkv, B, 1, Hq, Hkv, D, pos, cos, sin, kc_a, vc_a)
    w_out, w_q, w_s, w_i = ops.attn_decode_cast(q_rot, kc_a, vc_a, pos, want_out=True)
    kc_b, vc_b = kc.clone(), vc.clone()
    g_out, g_q, g_s, g_i = ops.attn_decode_append(qkv, kc_b, vc_b, pos, cos, sin, Hq, want_out=True, cast=True)
    assert torch.equal(g_out, w_out) and torch.equal(g_q.view(torch.uint8), w_q.view(torch.uint8))
    assert torch.equal(g_s, w_s) and torch.equal(g_i, w_i)
    assert torch.equal(kc_b, kc_a) and torch.equal(vc_b, vc_a)

    for window in (0, 5, 127, 128, 300):
        want = ops.attn_decode_window(q_rot, kc_a, vc_a, pos, window)
        kc_b, vc_b = kc.clone(), vc.clone()
        got, _, _, _ = ops.attn_decode_append(qkv, kc_b, vc_b, pos, cos, sin, Hq, window=window)
        assert torch.equal(got, want), window
        assert torch.equal(kc_b, kc_a) and torch.equal(vc_b, vc_a)

    # K stored as projected, rotated on load: the new key is stored un-rotated too
    kc_a, vc_a = kc.clone(), vc.clone()
    q_rot = ops.kv_append_rope(qkv, B, 1, Hq, Hkv, D, pos, cos, sin, kc_a, vc_a, store_rotated_k=False)
    want = ops.attn_decode(q_rot, kc_a, vc_a, pos, k_is_rotated=False, cos=cos, sin=sin)
    kc_b, vc_b = kc.clone(), vc.clone()
    got, _, _, _ = ops.attn_decode_append(qkv, kc_b, vc_b, pos, cos, sin, Hq, k_is_rotated=False)
    _lib.device_status()
    assert torch.equal(got, want)
    assert torch.equal(kc_b, kc_a) and torch.equal(vc_b, vc_a)


def test_fused_append_many_sequences_ragged_contexts():
    """The benchmark's decode shape at a reduced batch: several CTAs per (sequence, kv head), the new token in a
    chunk that another CTA than the first one owns."""
    from xax_b200 import _lib, ops

    Hq, Hkv, D, B, max_len = 32, 8, 128, 24, 4096
    g = torch.Generator().manual_seed(5)
    positions = torch.randint(0, max_len, (B,), generator=g).tolist()
    positions[0], positions[1] = max_len - 1, 2048
    qkv, kc, vc, pos = _case(B, Hq, Hkv, D, max_len, positions, 11)
    cos, sin = ops.rope_tables(D, 500000.0, max_len, "cuda")
    kc_a, vc_a = kc.clone(), vc.clone()
    q_rot = ops.kv_append_rope(qkv, B, 1, Hq, Hkv, D, pos, cos, sin, kc_a, vc_a)
    want = ops.attn_decode(q_rot, kc_a, vc_a, pos)
    got, _, _, _ = ops.attn_decode_append(qkv, kc, vc, pos, cos, sin, Hq)
    _lib.device_status()
    assert torch.equal(got, want)
    assert torch.equal(kc, kc_a) and torch.equal(vc, vc_a)


def test_fused_append_checks_its_arguments():
    from xax_b200 import ops

    Hq, Hkv, D, B, max_len = 8, 2, 128, 2, 256
    qkv, kc, vc, pos = _case(B, Hq, Hkv, D, max_len, [3, 4], 1)
    cos, sin = ops.rope_tables(D, 10000.0, max_len, "cuda")
    with pytest.raises(ValueError):
        ops.attn_decode_append(qkv[:, :-8].contiguous(), kc, vc, pos, cos, sin, Hq)  # row too short for the heads
    with pytest.raises(ValueError):
        ops.attn_decode_append(qkv, kc, vc, pos, cos[:100], sin[:100], Hq)  # tables shorter than the cache
    with pytest.raises(ValueError):
        ops.attn_decode_append(qkv.float(), kc, vc, pos, cos, sin, Hq)
