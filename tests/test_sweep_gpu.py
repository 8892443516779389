"""Seeded random sweeps: the tensor-core kernels against the CUDA-core kernels of the same contract
(xaxb_gemm_fp8_check, xaxb_attn_check) over shapes nobody picked by hand -- odd sizes, ragged
lengths, every epilogue combination, every group size."""

import numpy as np
import pytest
import torch

from helpers import bf16, e4m3, f32, rel_fro, to_numpy, to_torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from xax_b200 import ops as o

    return o


def test_gemm_random_shapes_against_cuda_core_kernel(ops):
    from xax_b200 import _lib

    rng = np.random.default_rng(2024)
    for case in range(40):
        M = int(rng.choice([1, 7, 64, 128, 129, 200, 256, 300, 513, 1000]))
        N = int(rng.integers(1, 160)) * 8
        K = int(rng.integers(1, 130)) * 16
        a = to_torch((rng.standard_normal((M, K)) * 30).astype(np.float32).astype(e4m3))
        b = to_torch((rng.standard_normal((N, K)) * 30).astype(np.float32).astype(e4m3))
        rm = to_torch(rng.uniform(0.005, 0.02, M).astype(np.float32)) if rng.random() < 0.7 else None
        cm = to_torch(rng.uniform(0.01, 0.03, N).astype(np.float32)) if rng.random() < 0.7 else None
        bias = to_torch((rng.standard_normal(N) * 0.5).astype(bf16)) if rng.random() < 0.5 else None
        res = to_torch(rng.standard_normal((M, N)).astype(bf16)) if rng.random() < 0.5 else None
        out = ops.gemm_fp8(a, b, rm, cm, bias, res)
        chk = ops.gemm_fp8_check(a, b, rm, cm, bias, res)
        err = rel_fro(f32(to_numpy(out)), f32(to_numpy(chk)))
        assert err < 2e-3, (case, M, N, K, err)
    _lib.device_status()


def test_decode_attention_random_shapes_against_cuda_core_kernel(ops):
    from xax_b200 import _lib

    rng = np.random.default_rng(77)
    g = torch.Generator(device="cuda").manual_seed(5)
    for case in range(24):
        D = int(rng.choice([64, 128]))
        Hkv = int(rng.choice([1, 2, 3, 4]))
        G = int(rng.choice([1, 2, 3, 4, 5, 8, 16]))
        Hq = Hkv * G
        if Hq * D > 4096:
            continue
        B = int(rng.integers(1, 9))
        max_len = int(rng.choice([130, 257, 700, 1300]))
        lens = rng.integers(1, max_len + 1, B)
        kc = torch.randn((B, max_len, Hkv, D), generator=g, device="cuda", dtype=torch.bfloat16)
        vc = torch.randn((B, max_len, Hkv, D), generator=g, device="cuda", dtype=torch.bfloat16)
        q = torch.randn((B, Hq, D), generator=g, device="cuda", dtype=torch.bfloat16)
        pos = to_torch((lens - 1).astype(np.int32))
        out = ops.attn_decode(q, kc, vc, pos)
        chk = ops.attn_check(q, kc, vc, pos, B, 1)
        err = rel_fro(f32(to_numpy(out)), f32(to_numpy(chk)).reshape(B, Hq, D))
        assert err < 5e-3, (case, B, Hq, Hkv, D, lens.tolist(), err)
        # the fused per-token cast agrees with casting the bf16 output
        _, qq, rs, ri = ops.attn_decode_cast(q, kc, vc, pos)
        q_ref, s_ref, i_ref, _ = ops.quantize_current(out.reshape(B, Hq * D), 1)
        assert torch.equal(qq.view(torch.uint8), q_ref.view(torch.uint8)) and torch.equal(rs, s_ref), case
    _lib.device_status()


def test_prefill_attention_random_shapes_against_cuda_core_kernel(ops):
    from xax_b200 import _lib

    rng = np.random.default_rng(31)
    g = torch.Generator(device="cuda").manual_seed(6)
    for case in range(12):
        D = int(rng.choice([64, 128]))
        Hkv = int(rng.choice([1, 2, 4]))
        Hq = Hkv * int(rng.choice([1, 2, 4]))
        B = int(rng.integers(1, 4))
        T = int(rng.choice([1, 5, 128, 129, 300]))
        start = rng.integers(0, 200, B)
        max_len = int(start.max()) + T + int(rng.integers(0, 50))
        kc = torch.randn((B, max_len, Hkv, D), generator=g, device="cuda", dtype=torch.bfloat16)
        vc = torch.randn((B, max_len, Hkv, D), generator=g, device="cuda", dtype=torch.bfloat16)
        q = torch.randn((B * T, Hq, D), generator=g, device="cuda", dtype=torch.bfloat16)
        pos = to_torch(start.astype(np.int32))
        out = ops.attn_prefill(q, kc, vc, pos, B, T)
        chk = ops.attn_check(q, kc, vc, pos, B, T)
        err = rel_fro(f32(to_numpy(out)), f32(to_numpy(chk)))
        assert err < 5e-3, (case, B, T, Hq, Hkv, D, start.tolist(), err)
    _lib.device_status()
