"""The all-reduce fused into the row-parallel GEMM's epilogue (xaxb_gemm_fp8_push + xaxb_tp_push_sum_rmsnorm),
checked on ONE GPU: the "ranks" are buffers on the same device and run one after the other in one stream --
both GEMMs push into both buffers, then each buffer's consumer runs.  By then every piece has arrived, so no
kernel ever waits for a kernel that is not already finished (which is the only way several ranks may share a
GPU); the protocol, the addressing of the slots, the arrival counters and the running totals are the same
as across GPUs.  The multi-GPU test (test_tp_gpu.py) covers the NVLink side.
"""

import ctypes

import numpy as np
import pytest
import torch

from helpers import bf16, e4m3, to_torch

pytestmark = pytest.mark.gpu


def _up(n, a=4096):
    return (n + a - 1) // a * a


class _FakeRanks:
    """`world` buffers on one device laid out like PeerExchange's push region: two (counter, staging) pairs."""

    def __init__(self, world, rows, cols):
        from xax_b200 import _lib

        lib = _lib.load()
        self.world, self.rows, self.cols = world, rows, cols
        self.slot = _up(rows * cols * 2)
        self.flag = [0, 4096]
        self.data = [8192, 8192 + world * self.slot]
        total = self.data[1] + world * self.slot
        self.bufs = [torch.zeros(total, dtype=torch.uint8, device="cuda") for _ in range(world)]
        self.ptrs = (ctypes.c_void_p * world)(*[b.data_ptr() for b in self.bufs])
        self.totals = [torch.zeros((2, lib.xaxb_tp_push_totals_bytes() // 4), dtype=torch.int32, device="cuda")
                       for _ in range(world)]

    def push(self, rank, parity, xq, wq, x_inv, w_inv, bias, residual):
        from xax_b200 import ops

        ops.gemm_fp8_push(xq, wq, x_inv, w_inv, bias, residual, self.ptrs, rank, self.world,
                          self.data[parity] + rank * self.slot, self.flag[parity])

    def consume(self, rank, parity, weight=None, eps=0.0):
        from xax_b200 import ops

        base = self.bufs[rank].data_ptr()
        return ops.tp_push_sum_rmsnorm(base + self.data[parity], self.slot, base + self.flag[parity],
                                       self.totals[rank][parity].data_ptr(), self.world, self.rows, self.cols, "cuda",
                                       weight, eps)


@pytest.mark.parametrize("world,M,N,K", [(2, 128, 4096, 2048), (2, 128, 4096, 7168), (4, 128, 4096, 1024),
                                         (8, 128, 4096, 512), (8, 128, 4096, 1792), (3, 5, 512, 256), (2, 77, 1032, 528)])
def test_pushed_partial_outputs_sum_like_separate_gemms(world, M, N, K):
    from xax_b200 import _lib, ops

    rng = np.random.default_rng(world * 1000 + K)
    fake = _FakeRanks(world, M, N)
    lib = _lib.load()
    # The order in which float32 partial sums over K are added depends on the tile plan (how K is split over
    # a cluster), and the pushing GEMM picks its plan from the kernels that can push.  Both sides of the
    # comparison run under the same forced plan, so equality is bit for bit.
    assert lib.xaxb_gemm_force_plan(64, 2) == 0
    try:
        _push_exchanges(fake, rng, world, M, N, K)
    finally:
        lib.xaxb_gemm_force_plan(0, 0)
    # the counters hold exactly the pieces announced: world * M * N / 8 per exchange on each pair
    for r in range(world):
        c0 = int(fake.bufs[r][0:4].view(torch.int32).item())
        c1 = int(fake.bufs[r][4096:4100].view(torch.int32).item())
        assert c0 == 2 * world * M * N // 8 and c1 == world * M * N // 8


def _push_exchanges(fake, rng, world, M, N, K):
    from xax_b200 import _lib, ops

    w_norm = to_torch((1 + 0.1 * rng.standard_normal(N)).astype(np.float32).astype(bf16))
    for exchange in range(3):  # pairs 0, 1, 0: alternation and the running totals
        parity = exchange & 1
        parts = []
        for r in range(world):
            a = to_torch((rng.standard_normal((M, K)) * 30).astype(np.float32).astype(e4m3))
            b = to_torch((rng.standard_normal((N, K)) * 30).astype(np.float32).astype(e4m3))
            rm = to_torch(rng.uniform(0.005, 0.02, M).astype(np.float32))
            cm = to_torch(rng.uniform(0.01, 0.03, 1).astype(np.float32))
            res = to_torch(rng.standard_normal((M, N)).astype(np.float32).astype(bf16)) if r == 0 else None
            fake.push(r, parity, a, b, rm, cm, None, res)
            parts.append(ops.gemm_fp8(a, b, rm, cm, None, res))  # the same GEMM with a local output
        # what every rank must compute: float32 sum in rank order, one rounding to bf16
        acc = torch.zeros((M, N), dtype=torch.float32, device="cuda")
        for p in parts:
            acc += p.float()
        want = acc.to(torch.bfloat16)
        use_norm = exchange != 1
        outs = [fake.consume(r, parity, w_norm if use_norm else None, 1e-5) for r in range(world)]
        _lib.device_status()
        for x, q, scale, inv in outs:
            assert torch.equal(x, want)
            if use_norm:  # bit for bit what RMSNorm + per-token cast of the summed rows gives
                _, (q_ref, s_ref, i_ref) = ops.rmsnorm(want, w_norm, 1e-5, want_y=False, quantize=True)
                assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))
                assert torch.equal(scale, s_ref) and torch.equal(inv, i_ref)
            else:
                assert q is None


def test_push_with_the_library_own_plan_matches_within_rounding():
    """Without a forced plan the pushing GEMM and the plain GEMM may split K differently: the sums then agree to
    float32 summation order, i.e. a bf16 ulp here and there."""
    from xax_b200 import _lib, ops

    world, M, N, K = 4, 128, 4096, 3584
    rng = np.random.default_rng(3)
    fake = _FakeRanks(world, M, N)
    acc = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    for r in range(world):
        a = to_torch((rng.standard_normal((M, K)) * 30).astype(np.float32).astype(e4m3))
        b = to_torch((rng.standard_normal((N, K)) * 30).astype(np.float32).astype(e4m3))
        rm = to_torch(rng.uniform(0.005, 0.02, M).astype(np.float32))
        fake.push(r, 0, a, b, rm, None, None, None)
        acc += ops.gemm_fp8(a, b, rm, None, None, None).float()
    x, _, _, _ = fake.consume(0, 0)
    _lib.device_status()
    want = acc.to(torch.bfloat16).float()
    assert float((x.float() - want).norm() / want.norm()) < 2e-3


def test_push_arguments_are_checked():
    from xax_b200 import ops

    fake = _FakeRanks(2, 128, 256)
    a = torch.zeros((200, 128), dtype=torch.float8_e4m3fn, device="cuda")
    b = torch.zeros((256, 128), dtype=torch.float8_e4m3fn, device="cuda")
    with pytest.raises(ValueError):  # more than 128 rows: outside the decode path the push covers
        fake.push(0, 0, a, b, None, None, None, None)
    with pytest.raises(ValueError):
        ops.gemm_fp8_push(a[:128], b, None, None, None, None, fake.ptrs, 2, 2, fake.data[0], fake.flag[0])  # rank >= world
