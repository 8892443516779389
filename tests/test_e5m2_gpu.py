"""float8_e5m2 through the free functions of the FP8 module (xax/nn/fp8.py:97-162, :347-378; the reference's
tests/nn/test_fp8.py parametrises quantize_dequantize and fp8_matmul over both formats): bytes and scales
bit-exact against the oracle in the bf16 compute dtype, the matmul within the tolerance of the e4m3 path and
within the reference test's own bounds."""

import numpy as np
import pytest
import torch

from helpers import bf16, e4m3, e5m2, f32, rel_fro, to_numpy, to_torch

pytestmark = pytest.mark.gpu

TOL = 1e-2


@pytest.fixture(scope="module")
def ofp8():
    from oracle import fp8

    return fp8


def _same_bytes(got, exp):
    """Equal bytes; where the oracle has a NaN the kernel must have the same NaN byte (0x7E / 0xFE)."""
    assert np.array_equal(got, exp), np.flatnonzero(got != exp)[:8]


def test_e5m2_quantize_given_scale_bit_exact(ofp8):
    from xax_b200 import ops

    rng = np.random.default_rng(0)
    x = (rng.standard_normal((64, 256)) * np.exp(rng.uniform(-12, 12, (64, 256)))).astype(np.float32)
    x[0, :10] = [0.0, -0.0, 1e-40, -1e-39, np.inf, -np.inf, np.nan, 57344.0, 60000.0, -61440.0]
    x[1, :4] = [1.52e-5, 7.6e-6, 6.1e-5, -3.05e-5]  # around the smallest e5m2 subnormals
    xb = x.astype(bf16)
    for scale in (1.0, 0.37, 1024.0, 3.1e-3):
        s = np.float32(scale)
        q, sc, inv = ops.quantize_e5m2(to_torch(xb), scale=to_torch(np.asarray([s], np.float32)))
        with np.errstate(invalid="ignore", over="ignore"):
            exp = ofp8.quantize(xb, e5m2, s, bf16)
        _same_bytes(to_numpy(q).view(np.uint8), exp.view(np.uint8))
        assert np.all(to_numpy(sc) == f32(np.asarray(s).astype(bf16)))
        assert np.all(to_numpy(inv) == np.float32(1.0) / f32(np.asarray(s).astype(bf16)))


@pytest.mark.parametrize("group_rows", [None, 1, 8])
def test_e5m2_current_scaling_bit_exact(ofp8, group_rows):
    from xax_b200 import ops

    rng = np.random.default_rng(1)
    x = rng.standard_normal((32, 512)).astype(np.float32)
    x = np.where(rng.random(x.shape) < 1e-2, x * 30, x)
    x[5] = 0.0  # an all-zero row: the 1e-12 floor of the divisor applies
    xb = x.astype(bf16)
    q, sc, _ = ops.quantize_e5m2(to_torch(xb), group_rows=group_rows)
    g = 32 if group_rows is None else group_rows
    qn, scn = to_numpy(q).view(np.uint8), to_numpy(sc)
    for r0 in range(0, 32, g):
        blk = xb[r0:r0 + g]
        exp_scale = ofp8.current_scale(blk, e5m2, bf16)
        assert np.all(scn[r0:r0 + g] == f32(exp_scale))
        _same_bytes(qn[r0:r0 + g], ofp8.quantize(blk, e5m2, exp_scale, bf16).view(np.uint8))


def test_e5m2_dequantize_and_round_trip(ofp8):
    from xax_b200 import ops
    from xax_b200.nn import fp8

    q = np.arange(256, dtype=np.uint8).reshape(1, 256).repeat(8, axis=0).view(e5m2)  # every byte, NaN and inf too
    for scale in (1.0, 0.37, 448.0):
        s = np.asarray([scale], np.float32)
        for dt, odt in ((torch.bfloat16, bf16), (torch.float32, np.float32)):
            got = to_numpy(ops.dequantize_e5m2(to_torch(q), to_torch(s), dt))
            with np.errstate(invalid="ignore", over="ignore"):
                exp = ofp8.dequantize(q, odt, s[0])
            assert np.array_equal(np.isnan(f32(got)), np.isnan(f32(exp)))
            ok = ~np.isnan(f32(exp))
            assert np.array_equal(f32(got)[ok], f32(exp)[ok])
    # the relation the reference's test checks (tests/nn/test_fp8.py:56-67): mean relative error below 5 %
    rng = np.random.default_rng(42)
    x = rng.standard_normal((16, 16)).astype(np.float32)
    scale = np.float32(57344.0 / np.abs(x).max())
    back = fp8.quantize_dequantize(to_torch(x), torch.float8_e5m2, torch.tensor(float(scale)))
    assert back.shape == (16, 16)
    rel = np.abs(to_numpy(back.float()) - x) / (np.abs(x) + 1e-6)
    assert rel.mean() < 0.05
    with np.errstate(invalid="ignore"):
        exp = ofp8.quantize_dequantize(x.astype(bf16), e5m2, scale, bf16)
    assert np.array_equal(to_numpy(fp8.quantize_dequantize(to_torch(x.astype(bf16)), torch.float8_e5m2,
                                                           torch.tensor(float(scale)), torch.bfloat16)).view(np.uint16),
                          exp.view(np.uint16))


@pytest.mark.parametrize("M,K,N", [(4, 16, 8), (130, 512, 264), (512, 1024, 768)])
def test_e5m2_fp8_matmul(ofp8, M, K, N):
    from xax_b200.nn import fp8

    rng = np.random.default_rng(M)
    a = rng.standard_normal((M, K)).astype(np.float32).astype(bf16)
    b = rng.standard_normal((K, N)).astype(np.float32).astype(bf16)
    got = f32(to_numpy(fp8.fp8_matmul(to_torch(a), to_torch(b), fp8_dtype=torch.float8_e5m2)))
    assert got.shape == (M, N)
    exp = f32(ofp8.fp8_matmul(a, b, bf16, e5m2))
    assert rel_fro(got, exp) < TOL
    if K == 16:  # the reference test's own bound for e5m2 (tests/nn/test_fp8.py:121-135)
        assert np.allclose(got, f32(a) @ f32(b), atol=1.0, rtol=0.1)


@pytest.mark.parametrize("fa,fb", [(e5m2, e5m2), (e4m3, e5m2), (e5m2, e4m3)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 512), (100, 264, 1040), (512, 768, 1024), (64, 4096, 2048)])
def test_gemm_mixed_fp8_formats_exact(fa, fb, M, N, K):
    """Small integers are exact in both formats and their dot products in float32: every kernel variant the
    shapes select (single-CTA, CTA-pair, split-K) must reproduce the integer result for every format pair."""
    from xax_b200 import ops

    rng = np.random.default_rng(N + K)
    a = rng.integers(-3, 4, (M, K)).astype(np.float32)
    b = rng.integers(-3, 4, (N, K)).astype(np.float32)
    got = f32(to_numpy(ops.gemm_fp8_formats(to_torch(a.astype(fa)), to_torch(b.astype(fb)))))
    exp = f32((a @ b.T).astype(bf16))
    assert np.array_equal(got, exp)


def test_e5m2_arguments_are_checked():
    from xax_b200 import ops
    from xax_b200.nn import fp8

    x = torch.zeros((4, 16), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        ops.quantize_e5m2(x, group_rows=3)
    with pytest.raises(ValueError):
        ops.quantize_e5m2(x.float())
    with pytest.raises(ValueError):
        ops.gemm_fp8_formats(x, x)
    with pytest.raises(ValueError, match="float8_e4m3fn only"):
        fp8.Fp8Linear(16, 16, key=0, fp8_dtype=torch.float8_e5m2)
