"""The allocation-free decode-attention entry point (xaxb_attn_decode_static) against the
regular one.  Collected last on purpose: a run that stops at the first failure has then
already run every other test.

Some users of this library cannot give it scratch memory -- an XLA/JAX custom-call handler
only sees the buffers declared for the call, a latency-critical serving loop may forbid
cudaMalloc (it synchronises the device), an embedding application may keep the allocator to
itself.  For them the library carries its own fixed scratch array; this test checks that the
variant using it returns what the workspace variant returns, also on a second call that finds
the first call's leftovers in the array, and that oversize shapes are refused."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(B, Hq, Hkv, D, max_len, lengths, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    kc = torch.randn((B, max_len, Hkv, D), generator=g, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn((B, max_len, Hkv, D), generator=g, device="cuda", dtype=torch.bfloat16)
    q = torch.randn((B, Hq, D), generator=g, device="cuda", dtype=torch.bfloat16)
    pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device="cuda")
    return q, kc, vc, pos


def test_static_scratch_variant_matches_workspace_variant_twice():
    from xax_b200 import _lib, ops

    cap = _lib.load().xaxb_attn_decode_static_capacity_bytes()
    assert cap == 16 << 20
    cases = [
        (4, 8, 2, 128, 1024, [1000, 130, 1, 513], 1),   # long sequences first ...
        (3, 8, 4, 64, 300, [37, 300, 129], 2),          # ... then a smaller call that finds their leftovers
    ]
    for B, Hq, Hkv, D, max_len, lengths, seed in cases:
        q, kc, vc, pos = _case(B, Hq, Hkv, D, max_len, lengths, seed)
        assert _lib.load().xaxb_attn_decode_workspace_bytes(B, Hq, D, max_len) <= cap
        ref = ops.attn_decode(q, kc, vc, pos)
        got = ops.attn_decode_static(q, kc, vc, pos)
        torch.cuda.synchronize()
        # same kernels, same inputs: bit-identical; the suite's attention tolerance as the formal bar
        err = (got.float() - ref.float()).norm() / ref.float().norm()
        assert float(err) <= 5e-3, float(err)
        assert torch.equal(got, ref)
    _lib.device_status()


def test_static_scratch_variant_refuses_oversize_shapes():
    from xax_b200 import _lib, ops

    B, Hq, Hkv, D, max_len = 64, 32, 8, 128, 8192  # needs 545 MB of scratch
    assert _lib.load().xaxb_attn_decode_workspace_bytes(B, Hq, D, max_len) > (16 << 20)
    q = torch.zeros((B, Hq, D), dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros((B, 128, Hkv, D), dtype=torch.bfloat16, device="cuda")  # never read: the call is refused
    kc = kc.as_strided((B, max_len, Hkv, D), (0, 0, D, 1))
    pos = torch.zeros((B,), dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="built-in"):
        ops.attn_decode_static(q, kc, kc, pos, scale=1.0 / math.sqrt(D))
