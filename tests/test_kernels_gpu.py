"""Parity of each CUDA kernel (through the C ABI) against the CPU oracle on seeded inputs.

Bars: e4m3 bytes, amax, scales, history bit-exact; GEMM / attention within a relative
Frobenius error of 1e-2 of the oracle's strict reference path and 2e-3 of a float32
restatement of the kernel's own formula."""

import math

import numpy as np
import pytest
import torch

from helpers import attn_setup as _attn_setup
from helpers import bf16, cfg1_inputs, e4m3, f32, rel_fro, to_numpy, to_torch

pytestmark = pytest.mark.gpu

TOL_REF = 1e-2      # vs the oracle's QDQ / strict-bf16 path (the stated tolerance of the path)
TOL_SELF = 2e-3     # vs a float32 restatement of the kernel's own arithmetic


@pytest.fixture(scope="module")
def ops():
    from xax_b200 import _lib, ops as o

    yield o
    _lib.device_status()


@pytest.fixture(scope="module")
def ofp8():
    from oracle import fp8

    return fp8


# ---------------------------------------------------------------------------------------
# kernel 1


@pytest.mark.parametrize("rows,cols,group", [(1, 8, 1), (3, 24, 1), (64, 2048, 1), (7, 4096, 1), (16, 512, 16),
                                             (6, 64, 3), (2048, 2048, 2048), (256, 5632, 64)])
def test_quantize_current_bit_exact(ops, ofp8, rows, cols, group):
    rng = np.random.default_rng(rows * 131 + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    x = np.where(rng.random((rows, cols)) < 1e-3, x * 20.0, x).astype(bf16)
    q, scale, inv, amax = ops.quantize_current(to_torch(x), group)
    xg = x.reshape(rows // group, group * cols)
    exp_amax = np.max(np.abs(f32(xg)), axis=1)
    floor = f32(np.asarray(1e-12).astype(bf16))
    exp_scale = (np.float32(448.0) / np.maximum(exp_amax, floor)).astype(bf16)
    exp_q = ofp8.quantize(xg, e4m3, exp_scale[:, None], bf16).reshape(rows, cols)
    assert np.array_equal(to_numpy(amax), exp_amax)
    assert np.array_equal(to_numpy(scale), np.repeat(f32(exp_scale), group))
    assert np.array_equal(to_numpy(inv), np.repeat(np.float32(1.0) / f32(exp_scale), group))
    assert np.array_equal(to_numpy(q).view(np.uint8), exp_q.view(np.uint8))


def test_quantize_special_values(ops, ofp8):
    """zeros, -0, subnormals, values that clip, infinities; a NaN row poisons only its row."""
    x = np.zeros((4, 16), dtype=np.float32)
    x[0, :6] = [0.0, -0.0, 1e-40, -1e-39, 3.0, -7.5]
    x[1, :4] = [np.inf, -np.inf, 1.0, -1.0]
    x[2, :3] = [np.nan, 1.0, -2.0]
    x[3, :] = 0.0  # all-zero row: amax floor 1e-12 applies
    xb = x.astype(bf16)
    q, scale, _, amax = ops.quantize_current(to_torch(xb), 1)
    qn = to_numpy(q).view(np.uint8)
    for r in (0, 1, 3):
        exp_scale = ofp8.current_scale(xb[r], e4m3, bf16)
        with np.errstate(invalid="ignore"):
            exp = ofp8.quantize(xb[r], e4m3, exp_scale, bf16).view(np.uint8)
        got = qn[r]
        nan_exp = (exp & 0x7F) == 0x7F
        assert np.array_equal(got[~nan_exp], exp[~nan_exp]), r
        assert np.all((got[nan_exp] & 0x7F) == 0x7F), r  # NaN stays NaN (sign is not pinned)
        assert to_numpy(scale)[r] == f32(exp_scale) or (np.isnan(to_numpy(scale)[r]) and np.isnan(f32(exp_scale)))
    assert np.isnan(to_numpy(amax)[2]) and np.isnan(to_numpy(scale)[2])
    assert np.all((qn[2] & 0x7F) == 0x7F)


@pytest.mark.parametrize("scale", [1.0, 0.37, 300.0, 3.0e-3, 1.0e30])
def test_quantize_delayed_special_values(ops, ofp8, scale):
    """The delayed-scaling cast (packed bf16 multiply / clip) on zeros, -0, bf16 subnormals, values that clip,
    infinities and NaN, and on random values of every magnitude: the bytes the oracle gives."""
    rng = np.random.default_rng(7)
    x = (rng.standard_normal((32, 256)) * np.exp(rng.uniform(-40, 40, (32, 256)))).astype(np.float32)
    x[0, :12] = [0.0, -0.0, 1e-40, -1e-39, 3.0, -7.5, np.inf, -np.inf, np.nan, 448.0, -449.0, 1e38]
    xb = x.astype(bf16)
    s_in = np.asarray(scale, np.float32)
    hist = np.zeros(16, np.float32)
    q, _, _, inv = ops.quantize_delayed(to_torch(xb), to_torch(s_in), to_torch(hist))
    with np.errstate(invalid="ignore", over="ignore"):
        exp = ofp8.quantize(xb, e4m3, s_in, bf16).view(np.uint8)
    got = to_numpy(q).view(np.uint8)
    nan_exp = (exp & 0x7F) == 0x7F
    assert np.array_equal(got[~nan_exp], exp[~nan_exp])
    assert np.all((got[nan_exp] & 0x7F) == 0x7F)  # NaN stays NaN (sign is not pinned)


@pytest.mark.parametrize("hist_len", [16, 1024])
def test_quantize_delayed_matches_oracle(ops, ofp8, hist_len):
    """benchmark config 1's scaling: history pre-filled from seeded draws, quantise with the
    incoming scale, new history / scale bit-exact."""
    x, w, _, rng = cfg1_inputs(M=256, K=512, N=128)
    hist = np.zeros(hist_len, np.float32)
    for _ in range(min(hist_len, 16)):
        d = rng.standard_normal((256, 512)).astype(np.float32)
        d = np.where(rng.random(d.shape) < 1e-3, d * 20, d).astype(bf16)
        hist = ofp8.compute_amax_history(d, hist)
    scale_in = ofp8.compute_scale(np.max(hist), np.float32(1.0), ofp8.get_fp8_max(e4m3, bf16))
    q, new_hist, new_scale, inv = ops.quantize_delayed(to_torch(x), to_torch(np.asarray(scale_in, np.float32)),
                                                       to_torch(hist))
    exp_hist = ofp8.compute_amax_history(x, hist)
    exp_scale = ofp8.compute_scale(np.max(exp_hist), scale_in, ofp8.get_fp8_max(e4m3, bf16))
    exp_q = ofp8.quantize(x, e4m3, scale_in, bf16)
    assert np.array_equal(to_numpy(new_hist), exp_hist)
    assert to_numpy(new_scale) == exp_scale
    assert np.array_equal(to_numpy(q).view(np.uint8), exp_q.view(np.uint8))
    assert to_numpy(inv)[0] == np.float32(1.0) / f32(np.asarray(scale_in).astype(bf16))


def test_quantize_delayed_invalid_amax_keeps_scale(ops):
    x = torch.zeros((8, 64), dtype=torch.bfloat16, device="cuda")
    scale_in = torch.tensor(2.5, device="cuda")
    hist = torch.zeros(16, device="cuda")
    _, new_hist, new_scale, _ = ops.quantize_delayed(x, scale_in, hist)
    assert float(new_scale) == 2.5 and float(new_hist.abs().max()) == 0.0
    hist[3] = float("inf")
    _, _, new_scale, _ = ops.quantize_delayed(x, scale_in, hist)
    assert float(new_scale) == 2.5


# ---------------------------------------------------------------------------------------
# kernel 2


def _gemm_inputs(M, N, K, seed):
    rng = np.random.default_rng(seed)
    a = (rng.standard_normal((M, K)) * 40).astype(np.float32).astype(e4m3)
    b = (rng.standard_normal((N, K)) * 40).astype(np.float32).astype(e4m3)
    return a, b, rng


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (128, 32, 256), (256, 512, 2048), (64, 4096, 2048),
                                   (100, 264, 1040), (1, 8, 16), (333, 776, 528), (2048, 1024, 512)])
def test_gemm_fp8_exact_small_integers(ops, M, N, K):
    """Integer-valued e4m3 operands with exactly representable sums: the tensor-core path
    must equal integer arithmetic exactly (no scaling, no bias)."""
    rng = np.random.default_rng(M + N + K)
    a = rng.integers(-4, 5, (M, K)).astype(np.float32).astype(e4m3)
    b = rng.integers(-4, 5, (N, K)).astype(np.float32).astype(e4m3)
    # shrink to keep |sum| <= 256 so the bf16 output is exact
    a[:, 16:] = 0
    out = ops.gemm_fp8(to_torch(a), to_torch(b))
    exp = (f32(a) @ f32(b).T)
    assert np.abs(exp).max() <= 256
    assert np.array_equal(f32(to_numpy(out)), exp)


@pytest.mark.parametrize("M,N,K,row_mode,col_mode,use_bias,use_res", [
    (256, 512, 1024, "scalar", "scalar", True, False),
    (192, 384, 2048, "row", "vec", True, True),
    (64, 2048, 2048, "row", None, False, True),
    (130, 520, 272, None, None, False, False),
])
def test_gemm_fp8_epilogue_variants(ops, M, N, K, row_mode, col_mode, use_bias, use_res):
    a, b, rng = _gemm_inputs(M, N, K, 7)
    rm = {"scalar": np.array([0.013], np.float32), "row": rng.uniform(0.005, 0.02, M).astype(np.float32), None: None}[row_mode]
    cm = {"scalar": np.array([0.021], np.float32), "vec": rng.uniform(0.01, 0.03, N).astype(np.float32), None: None}[col_mode]
    bias = (rng.standard_normal(N) * 0.5).astype(bf16) if use_bias else None
    res = rng.standard_normal((M, N)).astype(bf16) if use_res else None
    t = lambda v: None if v is None else to_torch(v)  # noqa: E731
    out = ops.gemm_fp8(to_torch(a), to_torch(b), t(rm), t(cm), t(bias), t(res))
    chk = ops.gemm_fp8_check(to_torch(a), to_torch(b), t(rm), t(cm), t(bias), t(res))
    exp = (f32(a).astype(np.float64) @ f32(b).astype(np.float64).T)
    if rm is not None:
        exp = exp * (rm[:, None] if rm.size > 1 else rm[0])
    if cm is not None:
        exp = exp * (cm[None, :] if cm.size > 1 else cm[0])
    if bias is not None:
        exp = exp + f32(bias)
    if res is not None:
        exp = exp + f32(res)
    assert rel_fro(f32(to_numpy(out)), exp) < TOL_SELF
    assert rel_fro(f32(to_numpy(chk)), exp) < TOL_SELF
    # the two GPU implementations differ only by summation order and one bf16 rounding
    assert rel_fro(f32(to_numpy(out)), f32(to_numpy(chk))) < TOL_SELF


@pytest.mark.parametrize("M,N,K,bn,split", [(128, 4096, 4096, 128, 4), (64, 768, 2048, 256, 8), (1, 512, 1024, 64, 2),
                                             (100, 1000, 1792, 32, 4), (128, 2048, 14336, 128, 2),
                                             (77, 264, 528, 64, 8), (128, 6144, 4096, 0, 0)])
def test_gemm_fp8_split_k_cluster_variants(ops, M, N, K, bn, split):
    """The split-K kernel (thread-block cluster, partial tiles summed through distributed shared
    memory) against the CUDA-core kernel, for forced (tile width, split) plans and the automatic
    plan; two runs must agree bit for bit (fixed summation order)."""
    from xax_b200 import _lib

    a, b, rng = _gemm_inputs(M, N, K, 21)
    rm = to_torch(rng.uniform(0.005, 0.02, M).astype(np.float32))
    cm = to_torch(rng.uniform(0.01, 0.03, N).astype(np.float32))
    bias = to_torch((rng.standard_normal(N) * 0.5).astype(bf16))
    res = to_torch(rng.standard_normal((M, N)).astype(bf16))
    at, bt = to_torch(a), to_torch(b)
    chk = ops.gemm_fp8_check(at, bt, rm, cm, bias, res)
    lib = _lib.load()
    assert lib.xaxb_gemm_force_plan(bn, split) == 0
    try:
        out1 = ops.gemm_fp8(at, bt, rm, cm, bias, res)
        out2 = ops.gemm_fp8(at, bt, rm, cm, bias, res)
    finally:
        lib.xaxb_gemm_force_plan(0, 0)
    assert torch.equal(out1, out2)
    assert rel_fro(f32(to_numpy(out1)), f32(to_numpy(chk))) < TOL_SELF
    _lib.device_status()


@pytest.mark.parametrize("M,N,K,fp8", [(256, 256, 128, True), (512, 768, 1024, True), (300, 520, 272, True),
                                           (1024, 2048, 2048, True), (129, 256, 4096, True), (512, 512, 512, False),
                                           (2048, 8192, 2048, True)])
def test_gemm_cta_pair_kernel(ops, M, N, K, fp8):
    """The CTA-pair kernels (tcgen05.mma.cta_group::2; 256 x 256, 256 x 224 and 256 x 192 tiles) against the
    single-CTA kernel on the same inputs, with every epilogue term; integer-valued operands make all exact."""
    from xax_b200 import _lib

    rng = np.random.default_rng(M + N)
    if fp8:
        a = to_torch(rng.integers(-3, 4, (M, K)).astype(np.float32).astype(e4m3))
        b = to_torch(rng.integers(-3, 4, (N, K)).astype(np.float32).astype(e4m3))
        f = ops.gemm_fp8
    else:
        a = to_torch(rng.integers(-3, 4, (M, K)).astype(np.float32).astype(bf16))
        b = to_torch(rng.integers(-3, 4, (N, K)).astype(np.float32).astype(bf16))
        f = ops.gemm_bf16
    rm = to_torch(rng.uniform(0.005, 0.02, M).astype(np.float32))
    cm = to_torch(rng.uniform(0.01, 0.03, N).astype(np.float32))
    bias = to_torch((rng.standard_normal(N) * 0.5).astype(bf16))
    res = to_torch(rng.standard_normal((M, N)).astype(bf16))
    lib = _lib.load()
    outs = {}
    for bn in (256, 512, 448, 384, 0):  # 0: the width the library picks by itself
        assert lib.xaxb_gemm_force_plan(bn, 1 if bn else 0) == 0
        try:
            outs[bn] = f(a, b, rm, cm, bias, res)
        finally:
            lib.xaxb_gemm_force_plan(0, 0)
    _lib.device_status()
    for bn in (512, 448, 384, 0):
        assert torch.equal(outs[256], outs[bn]), bn


@pytest.mark.parametrize("M,N,K", [(128, 256, 512), (200, 1000, 1088), (64, 32000, 2048)])
def test_gemm_bf16(ops, M, N, K):
    rng = np.random.default_rng(3)
    a = rng.standard_normal((M, K)).astype(np.float32).astype(bf16)
    b = (rng.standard_normal((N, K)) * 0.05).astype(np.float32).astype(bf16)
    out = ops.gemm_bf16(to_torch(a), to_torch(b))
    exp = f32(a).astype(np.float64) @ f32(b).astype(np.float64).T
    assert rel_fro(f32(to_numpy(out)), exp) < TOL_SELF


def test_fp8_linear_cfg1_reduced_vs_oracle(ops, ofp8):
    """Reduced benchmark config 1 (M=256, K=2048, N=512), delayed scaling: quantised bytes exact,
    output within 1e-2 of the oracle's QDQ path."""
    x, w, bias, rng = cfg1_inputs(M=256, K=2048, N=512)
    layer = ofp8.Fp8Linear(w, bias)
    sc = ofp8.init_fp8_scales(16)
    hist = sc.input_amax_history
    for _ in range(16):
        d = rng.standard_normal(x.shape).astype(np.float32)
        hist = ofp8.compute_amax_history(np.where(rng.random(d.shape) < 1e-3, d * 20, d).astype(bf16), hist)
    fp8_max = ofp8.get_fp8_max(e4m3, bf16)
    khist = np.full(16, f32(ofp8.amax_of(w)), np.float32)
    sc = ofp8.Fp8Scales(ofp8.compute_scale(np.max(hist), np.float32(1), fp8_max), hist,
                        ofp8.compute_scale(np.max(khist), np.float32(1), fp8_max), khist)
    exp_out, exp_sc = layer(x, sc)

    xq, nh, ns, xinv = ops.quantize_delayed(to_torch(x), to_torch(np.asarray(sc.input_scale)), to_torch(hist))
    wq, wh, ws, winv = ops.quantize_delayed(to_torch(w), to_torch(np.asarray(sc.kernel_scale)), to_torch(khist))
    out = ops.gemm_fp8(xq, wq, xinv, winv, to_torch(bias))
    assert np.array_equal(to_numpy(xq).view(np.uint8), ofp8.quantize(x, e4m3, sc.input_scale, bf16).view(np.uint8))
    assert np.array_equal(to_numpy(wq).view(np.uint8), ofp8.quantize(w, e4m3, sc.kernel_scale, bf16).view(np.uint8))
    assert np.array_equal(to_numpy(nh), exp_sc.input_amax_history) and to_numpy(ns) == exp_sc.input_scale
    assert np.array_equal(to_numpy(wh), exp_sc.kernel_amax_history) and to_numpy(ws) == exp_sc.kernel_scale
    err = rel_fro(f32(to_numpy(out)), f32(exp_out))
    assert err < TOL_REF, err


# ---------------------------------------------------------------------------------------
# small ops


@pytest.mark.parametrize("rows,dim", [(5, 64), (64, 2048), (3, 4096)])
def test_rmsnorm_and_fused_cast(ops, ofp8, rows, dim):
    from oracle.attention import RMSNorm

    rng = np.random.default_rng(dim)
    x = (rng.standard_normal((rows, dim)) * 3).astype(np.float32).astype(bf16)
    w = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32).astype(bf16)
    exp = RMSNorm(w, 1e-5)(x)
    y, (q, scale, inv) = ops.rmsnorm(to_torch(x), to_torch(w), 1e-5, quantize=True)
    got = to_numpy(y)
    # only the float32 summation order of the mean may differ: allow 1 bf16 ulp on few elements
    mism = np.mean(got.view(np.uint16) != exp.view(np.uint16))
    assert mism < 0.01, mism
    assert rel_fro(f32(got), f32(exp)) < 1e-3
    # the fused cast must be exactly the stand-alone cast of the kernel's own y
    q2, s2, i2, _ = ops.quantize_current(y, 1)
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(scale, s2) and torch.equal(inv, i2)


def test_silu_mul_and_group_amax(ops):
    from oracle.attention import silu

    rng = np.random.default_rng(5)
    rows, dim = 12, 704
    gu = (rng.standard_normal((rows, 2 * dim)) * 2).astype(np.float32).astype(bf16)
    sg = silu(gu[:, :dim])
    exp = (f32(sg) * f32(gu[:, dim:])).astype(bf16)
    amax = torch.zeros(3, device="cuda")
    h, (q, scale, inv) = ops.silu_mul(to_torch(gu), dim, quantize=True, group_amax=amax, group_rows=4)
    got = to_numpy(h)
    assert np.mean(got.view(np.uint16) != exp.view(np.uint16)) < 0.01
    assert rel_fro(f32(got), f32(exp)) < 1e-3
    q2, s2, _, _ = ops.quantize_current(h, 1)
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(scale, s2)
    exp_amax = np.abs(f32(got)).reshape(3, -1).max(axis=1)
    assert np.array_equal(to_numpy(amax), exp_amax)
    q3, s3, _ = ops.quantize_with_amax(h, amax, 4)
    q4, s4, _, _ = ops.quantize_current(h, 4)
    assert torch.equal(q3.view(torch.uint8), q4.view(torch.uint8)) and torch.equal(s3, s4)


@pytest.mark.parametrize("rows,dim", [(5, 14336), (3, 5632), (130, 2048), (2, 4096)])
def test_silu_mul_row_spread_over_a_cluster(ops, rows, dim):
    """Wide rows are spread over a thread-block cluster; the fused cast must still equal the
    stand-alone cast of the kernel's own h, and h the oracle's."""
    from oracle.attention import silu

    rng = np.random.default_rng(dim)
    gu = (rng.standard_normal((rows, 2 * dim)) * 2).astype(np.float32).astype(bf16)
    exp = (f32(silu(gu[:, :dim])) * f32(gu[:, dim:])).astype(bf16)
    amax = torch.zeros(rows, device="cuda")
    h, (q, scale, inv) = ops.silu_mul(to_torch(gu), dim, quantize=True, group_amax=amax, group_rows=1)
    got = to_numpy(h)
    assert np.mean(got.view(np.uint16) != exp.view(np.uint16)) < 0.01
    q2, s2, i2, a2 = ops.quantize_current(h, 1)
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(scale, s2) and torch.equal(inv, i2)
    assert torch.equal(amax, a2)
    _, (q3, s3, _) = ops.silu_mul(to_torch(gu), dim, want_h=False, quantize=True)
    assert torch.equal(q3.view(torch.uint8), q.view(torch.uint8)) and torch.equal(s3, scale)


def test_embed_and_argmax(ops):
    rng = np.random.default_rng(1)
    table = rng.standard_normal((1000, 256)).astype(np.float32).astype(bf16)
    toks = rng.integers(0, 1000, 77).astype(np.int32)
    x = ops.embed(to_torch(toks), to_torch(table))
    assert np.array_equal(to_numpy(x).view(np.uint16), table[toks].view(np.uint16))
    logits = rng.standard_normal((9, 32003)).astype(np.float32).astype(bf16)
    logits[2, 100] = logits[2, 31000] = np.float32(9.0)  # tie: first index wins
    got = to_numpy(ops.argmax(to_torch(logits)))
    assert np.array_equal(got, np.argmax(f32(logits), axis=-1).astype(np.int32))


def test_rope_table_matches_oracle(ops):
    from oracle.attention import RotaryEmbedding

    for D, base, n in [(128, 500000.0, 8192), (64, 10000.0, 1024)]:
        cos, sin = ops.rope_tables(D, base, n)
        ec, es = RotaryEmbedding(D, base, "concatenated").get_rotary_embeddings(np.arange(n, dtype=np.int32), bf16)
        assert np.array_equal(to_numpy(cos).view(np.uint16), ec.view(np.uint16))
        assert np.array_equal(to_numpy(sin).view(np.uint16), es.view(np.uint16))


# ---------------------------------------------------------------------------------------
# kernel 3


@pytest.fixture(params=[1, 11, 13], ids=["chunk-walk", "one-chunk-per-cta", "three-chunks-per-cta"])
def decode_variant(request):
    """Run a test with the decode-attention kernel's own choice of chunks per CTA (1, the default) and with
    n chunks per CTA forced (10 + n)."""
    from xax_b200 import _lib

    lib = _lib.load()
    assert lib.xaxb_attn_decode_force_variant(request.param) == 0
    yield request.param
    lib.xaxb_attn_decode_force_variant(0)
    _lib.device_status()


@pytest.mark.parametrize("Hq,Hkv,D,starts", [
    (8, 2, 128, [0, 62, 63, 64, 127, 128, 300, 1000]),
    (32, 8, 128, [511, 2047, 4000]),
    (32, 4, 64, [5, 129, 640, 767]),
    (4, 4, 128, [10, 200]),
    (16, 1, 128, [700] * 40),
])
def test_attn_decode_vs_oracle(ops, decode_variant, Hq, Hkv, D, starts):
    B, max_len = len(starts), max(starts) + 1 + 37
    theta = 500000.0 if D == 128 else 10000.0
    q_rot, kc, vc, pos, cos, sin, exp = _attn_setup(ops, B, 1, Hq, Hkv, D, max_len, starts, theta, 11)
    out = ops.attn_decode(q_rot, kc, vc, pos)
    chk = ops.attn_check(q_rot, kc, vc, pos, B, 1)
    assert rel_fro(f32(to_numpy(chk)), f32(exp)) < TOL_SELF
    err = rel_fro(f32(to_numpy(out)), f32(exp))
    assert err < TOL_REF, err
    assert rel_fro(f32(to_numpy(out)), f32(to_numpy(chk))) < 5e-3


@pytest.mark.parametrize("Hq,Hkv,D,starts", [(32, 8, 128, [0, 127, 128, 700]), (32, 4, 64, [5, 300]), (8, 2, 128, [64])])
def test_attn_decode_fused_cast_equals_separate_cast(ops, decode_variant, Hq, Hkv, D, starts):
    B, max_len = len(starts), max(starts) + 9
    q_rot, kc, vc, pos, cos, sin, exp = _attn_setup(ops, B, 1, Hq, Hkv, D, max_len, starts, 10000.0, 23)
    out = ops.attn_decode(q_rot, kc, vc, pos)
    o2, q, rs, ri = ops.attn_decode_cast(q_rot, kc, vc, pos, want_out=True)
    assert torch.equal(o2, out)
    q_ref, s_ref, i_ref, _ = ops.quantize_current(out.reshape(B, Hq * D), 1)
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8)) and torch.equal(rs, s_ref) and torch.equal(ri, i_ref)
    _, q3, _, _ = ops.attn_decode_cast(q_rot, kc, vc, pos)
    assert torch.equal(q3.view(torch.uint8), q.view(torch.uint8))


def test_attn_decode_rotate_on_load(ops, decode_variant):
    starts = [0, 100, 129, 515]
    B, Hq, Hkv, D = 4, 8, 2, 128
    max_len = 700
    q_rot, kc_raw, vc, pos, cos, sin, exp = _attn_setup(ops, B, 1, Hq, Hkv, D, max_len, starts, 500000.0, 13,
                                                        rotated=False)
    out = ops.attn_decode(q_rot, kc_raw, vc, pos, k_is_rotated=False, cos=cos, sin=sin)
    err = rel_fro(f32(to_numpy(out)), f32(exp))
    assert err < TOL_REF, err


@pytest.mark.parametrize("B,T,Hq,Hkv,D,start", [(2, 128, 4, 2, 128, 0), (1, 300, 8, 2, 128, 0), (2, 77, 8, 4, 64, 0),
                                                (2, 5, 4, 2, 128, 3), (1, 200, 4, 1, 128, 131)])
def test_attn_prefill_vs_oracle(ops, B, T, Hq, Hkv, D, start):
    """Prefill from an empty cache and chunked prefill (non-zero start: the reference's
    3+2+3 chunk test shape, xax tests/nn/test_attention.py:72-102)."""
    max_len = start + T + 19
    q_rot, kc, vc, pos, cos, sin, exp = _attn_setup(ops, B, T, Hq, Hkv, D, max_len, [start] * B, 10000.0, 17)
    out = ops.attn_prefill(q_rot, kc, vc, pos, B, T)
    chk = ops.attn_check(q_rot, kc, vc, pos, B, T)
    assert rel_fro(f32(to_numpy(chk)), f32(exp)) < TOL_SELF
    err = rel_fro(f32(to_numpy(out)), f32(exp))
    assert err < TOL_REF, err


def test_cache_overflow_is_reported(ops):
    from xax_b200 import _lib

    B, T, Hq, Hkv, D, max_len = 1, 4, 2, 1, 64, 6
    qkv = torch.zeros((B * T, (Hq + 2 * Hkv) * D), dtype=torch.bfloat16, device="cuda")
    cos, sin = ops.rope_tables(D, 10000.0, max_len, "cuda")
    kc = torch.zeros((B, max_len, Hkv, D), dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    pos = torch.tensor([3], dtype=torch.int32, device="cuda")
    ops.kv_append_rope(qkv, B, T, Hq, Hkv, D, pos, cos, sin, kc, vc)
    with pytest.raises(ValueError, match="overflow"):
        _lib.device_status()
