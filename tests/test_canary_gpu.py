"""Out-of-bounds writes, looked for without a memory checker: every output the functional layer allocates is
placed between two guard bands filled with a known pattern, the kernels run on small and ragged shapes (rows
and columns that do not fill a tile, sequence ends inside a chunk, a single row), and the bands must come
back untouched.  Reads past an input cannot be seen this way; the TMA loads clip them by construction and the
plain loads are bounded by the same extents as the stores checked here."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

GUARD = 4096  # bytes on either side of every allocation
PATTERN = 0xA5


class _Guarded:
    """Stands in for the ``torch`` module inside xax_b200.ops: ``empty`` / ``empty_like`` / ``zeros`` hand out
    views into larger byte buffers with guard bands; everything else is torch's."""

    def __init__(self):
        self.bands = []

    def __getattr__(self, name):
        return getattr(torch, name)

    def _alloc(self, shape, dtype, device, zero=False):
        shape = tuple(shape) if isinstance(shape, (tuple, list, torch.Size)) else (shape,)
        n = int(np.prod(shape)) if len(shape) else 1
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        pad = (-nbytes) % 256
        buf = torch.full((GUARD + nbytes + pad + GUARD,), PATTERN, dtype=torch.uint8, device=device)
        body = buf[GUARD:GUARD + nbytes]
        if zero:
            body.zero_()
        self.bands.append((buf, nbytes))
        return body.view(dtype).view(shape)

    def empty(self, *shape, dtype=torch.float32, device=None, **kw):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
            shape = shape[0]
        return self._alloc(shape, dtype, device)

    def zeros(self, *shape, dtype=torch.float32, device=None, **kw):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
            shape = shape[0]
        return self._alloc(shape, dtype, device, zero=True)

    def empty_like(self, t, **kw):
        return self._alloc(t.shape, t.dtype, t.device)

    def check(self):
        torch.cuda.synchronize()
        for buf, nbytes in self.bands:
            lo, hi = buf[:GUARD], buf[GUARD + nbytes + ((-nbytes) % 256):]
            assert bool((lo == PATTERN).all()), "a kernel wrote below an output buffer"
            assert bool((hi == PATTERN).all()), "a kernel wrote past an output buffer"
        n = len(self.bands)
        self.bands = []
        return n


@pytest.fixture()
def guarded(monkeypatch):
    from xax_b200 import _lib, ops

    g = _Guarded()
    monkeypatch.setattr(ops, "torch", g)
    yield g
    monkeypatch.undo()
    _lib.device_status()


def _bf16(shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def test_row_kernels_stay_inside_their_outputs(guarded):
    from xax_b200 import ops

    for rows, cols in ((1, 8), (3, 24), (5, 4096), (130, 264), (7, 14336)):
        x = _bf16((rows, cols), rows + cols)
        ops.quantize_current(x, 1)
        ops.quantize_current(x, rows)
        w = torch.ones((cols,), dtype=torch.bfloat16, device="cuda")
        ops.rmsnorm(x, w, 1e-5, quantize=True)
        q, s, inv, _ = ops.quantize_current(x, 1)
        ops.dequantize(q, s)
        scale = torch.tensor(3.0, device="cuda")
        hist = torch.zeros(16, device="cuda")
        ops.quantize_delayed(x, scale, hist)
    for rows, dim in ((1, 8), (5, 704), (3, 5632), (2, 14336)):
        gu = _bf16((rows, 2 * dim), dim)
        ops.silu_mul(gu, dim, quantize=True)
    table = _bf16((100, 64), 1)
    toks = torch.tensor([0, 99, 5], dtype=torch.int32, device="cuda")
    ops.embed(toks, table)
    logits = _bf16((3, 1000), 2)
    ops.argmax(logits)
    ops.sample_top_p(logits, 0.7, 0.9, torch.tensor([0.1, 0.5, 0.9], device="cuda"))
    assert guarded.check() > 20


def test_gemms_stay_inside_their_outputs(guarded):
    from xax_b200 import _lib, ops

    lib = _lib.load()
    g = torch.Generator(device="cuda").manual_seed(0)
    for M, N, K in ((1, 8, 16), (100, 264, 1040), (128, 4096, 512), (77, 1032, 528), (333, 776, 528), (129, 256, 4096)):
        a = torch.randn((M, K), generator=g, device="cuda").to(torch.float8_e4m3fn)
        b = torch.randn((N, K), generator=g, device="cuda").to(torch.float8_e4m3fn)
        for bn, split in ((0, 0), (32, 1), (64, 2), (128, 4), (256, 1), (512, 1)):
            if split > 1 and M > 128:
                continue
            assert lib.xaxb_gemm_force_plan(bn, split) == 0
            try:
                ops.gemm_fp8(a, b)
            finally:
                lib.xaxb_gemm_force_plan(0, 0)
        ops.gemm_bf16(a.to(torch.bfloat16), b.to(torch.bfloat16))
    assert guarded.check() > 20


def test_attention_kernels_stay_inside_their_outputs(guarded):
    from xax_b200 import ops

    for B, T, Hq, Hkv, D, starts, max_len in ((2, 1, 8, 2, 128, [0, 130], 140), (3, 1, 4, 4, 64, [5, 127, 128], 200),
                                              (2, 77, 8, 4, 64, [0, 0], 90), (1, 130, 4, 1, 128, [3, 3], 140)):
        qkv = _bf16((B * T, (Hq + 2 * Hkv) * D), B + T)
        kc = torch.zeros((B, max_len, Hkv, D), dtype=torch.bfloat16, device="cuda")
        vc = torch.zeros_like(kc)
        pos = torch.tensor(starts[:B], dtype=torch.int32, device="cuda")
        cos, sin = ops.rope_tables(D, 10000.0, max_len, "cuda")
        q_rot = ops.kv_append_rope(qkv, B, T, Hq, Hkv, D, pos, cos, sin, kc, vc)
        if T == 1:
            ops.attn_decode(q_rot, kc, vc, pos)
            ops.attn_decode_cast(q_rot, kc, vc, pos, want_out=True)
            ops.attn_decode_window(q_rot, kc, vc, pos, 17)
            ops.attn_decode(q_rot, kc, vc, pos, k_is_rotated=False, cos=cos, sin=sin)
        else:
            ops.attn_prefill(q_rot, kc, vc, pos, B, T)
            ops.attn_prefill_window(q_rot, kc, vc, pos, B, T, 9)
        ops.rope_apply(q_rot, pos.repeat_interleave(T) if T > 1 else pos, cos, sin)
    assert guarded.check() > 15
