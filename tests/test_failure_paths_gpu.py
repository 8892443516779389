"""Failure paths that must end in a status code, never in a hang or a fault.

  * a device-side wait whose flag nobody raises runs out after the (shortened) limit, records
    XAXB_DEVICE_TIMEOUT with the waiting site, and leaves the context usable;
  * a decode-attention position outside the cache is clamped, reported as XAXB_CACHE_OVERFLOW, and
    gives a finite output.

Nothing here faults, traps or spins without bound: the "missing peer" is a second buffer on the
same GPU that simply never gets its flag written, and the wait limit is set to 50 ms for the call.
"""

import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_wait_runs_out_and_context_stays_usable():
    from xax_b200 import _lib, ops

    lib = _lib.load()
    ctx = _lib.ctx()
    _lib.device_status()  # start from a clean status word
    sync = int(lib.xaxb_tp_sync_bytes())
    box = int(lib.xaxb_tp_max_inbox_bytes())
    total = sync + box
    mine = torch.zeros(total, dtype=torch.uint8, device="cuda")
    silent = torch.zeros(total, dtype=torch.uint8, device="cuda")  # stands for a rank that never shows up
    peers = (ctypes.c_void_p * 2)(mine.data_ptr(), silent.data_ptr())
    vals = torch.arange(8, dtype=torch.float32, device="cuda")
    out = torch.empty_like(vals)
    assert lib.xaxb_set_wait_limit_ms(ctx, 0, 50) == 0
    try:
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        rc = lib.xaxb_tp_allreduce_max_f32(ctx, _lib.stream_ptr(), peers, 0, 2, sync, 0, vals.data_ptr(), out.data_ptr(), 8)
        t1.record()
        assert rc == 0
        site = ctypes.c_int(0)
        status = lib.xaxb_ctx_status(ctx, _lib.stream_ptr(), ctypes.byref(site))
        assert status == _lib.DEVICE_TIMEOUT and site.value == 42, (status, site.value)
        ms = t0.elapsed_time(t1)
        assert 40.0 <= ms < 2000.0, ms  # gave up at the 50 ms limit, not at the 10 s default
    finally:
        assert lib.xaxb_set_wait_limit_ms(ctx, 0, 0) == 0
    # the status word was cleared by the read, and ordinary work runs
    _lib.device_status()
    x = torch.randn((4, 64), device="cuda").to(torch.bfloat16)
    q, scale, _, amax = ops.quantize_current(x, 1)
    _lib.device_status()
    assert torch.equal(amax, x.float().abs().amax(dim=1))
    # the silent rank's inbox did receive this rank's values (pushed before the wait)
    got = silent[sync:sync + 2 * 8 * 1024 * 4].view(torch.float32)  # float32 [2 parities][8 ranks][1024 slots]
    assert torch.equal(got.view(2, 8, 1024)[1, 0, :8].cpu(), vals.cpu()) or \
        torch.equal(got.view(2, 8, 1024)[0, 0, :8].cpu(), vals.cpu())


def test_decode_position_outside_the_cache_is_reported_not_nan():
    from xax_b200 import _lib, ops

    _lib.device_status()
    B, Hq, Hkv, D, max_len = 3, 4, 2, 128, 256
    g = torch.Generator(device="cuda").manual_seed(3)
    kc = torch.randn((B, max_len, Hkv, D), generator=g, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn((B, max_len, Hkv, D), generator=g, device="cuda", dtype=torch.bfloat16)
    q = torch.randn((B, Hq, D), generator=g, device="cuda", dtype=torch.bfloat16)
    good = torch.tensor([10, 200, 255], dtype=torch.int32, device="cuda")
    ref = ops.attn_decode(q, kc, vc, good)
    _lib.device_status()
    for bad_value, same_as in ((-5, 0), (max_len + 40, max_len - 1)):
        pos = good.clone()
        pos[1] = bad_value
        out = ops.attn_decode(q, kc, vc, pos)
        with pytest.raises(ValueError, match="overflow"):
            _lib.device_status()
        assert bool(torch.isfinite(out.float()).all())
        assert torch.equal(out[0], ref[0]) and torch.equal(out[2], ref[2])  # the other sequences are untouched
        clamped = good.clone()
        clamped[1] = same_as
        assert torch.equal(out, ops.attn_decode(q, kc, vc, clamped))
        _lib.device_status()
    # the fused-cast variant shares the clamp
    pos = good.clone()
    pos[0] = -1
    _, qq, rs, _ = ops.attn_decode_cast(q, kc, vc, pos)
    with pytest.raises(ValueError, match="overflow"):
        _lib.device_status()
    assert bool(torch.isfinite(rs).all()) and not bool(torch.isnan(qq.float()).any())


def test_attention_wrappers_reject_wrong_dtypes_and_views():
    from xax_b200 import ops

    B, Hq, Hkv, D, max_len = 2, 4, 2, 64, 128
    kc = torch.zeros((B, max_len, Hkv, D), device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    q = torch.zeros((B, Hq, D), device="cuda", dtype=torch.bfloat16)
    pos = torch.zeros((B,), dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="positions"):
        ops.attn_decode(q, kc, vc, pos.to(torch.int64))
    with pytest.raises(ValueError, match="contiguous"):
        ops.attn_decode(q, kc.transpose(1, 2).contiguous().transpose(1, 2), vc, pos)
    with pytest.raises(ValueError, match="bfloat16"):
        ops.attn_decode(q.float(), kc, vc, pos)
    with pytest.raises(ValueError, match="match"):
        ops.attn_decode(q[:1].contiguous(), kc, vc, pos)
    assert np.isfinite(ops.attn_decode(q, kc, vc, pos).float().cpu().numpy()).all()
