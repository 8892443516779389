"""Functional layer over the C ABI: torch tensors in, torch tensors out.

torch is used for device memory and streams only; every computation on the path is one of
the library's sm_100a kernels.  All functions run on the current CUDA stream and do not
synchronise.
"""

from __future__ import annotations

import math

import numpy as np
import torch

from . import _lib
from ._lib import check, ptr

E4M3 = torch.float8_e4m3fn
BF16 = torch.bfloat16


def _c():
    return _lib.ctx(), _lib.stream_ptr(), _lib.load()


def _req(t: torch.Tensor, dtype, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU fallback)")
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    return t if t.is_contiguous() else t.contiguous()


# ---------------------------------------------------------------------------------------
# kernel 1


def quantize_current(x: torch.Tensor, group_rows: int = 1):
    """x[rows, cols] bf16 -> (q e4m3, scale[rows] f32, inv_scale[rows] f32, amax[groups] f32).

    group_rows = 1: a scale per row (per token); group_rows = rows: one scale per tensor."""
    x = _req(x, BF16, "x")
    rows, cols = x.shape
    ctx, st, lib = _c()
    q = torch.empty((rows, cols), dtype=E4M3, device=x.device)
    scale = torch.empty((rows,), dtype=torch.float32, device=x.device)
    inv = torch.empty((rows,), dtype=torch.float32, device=x.device)
    amax = torch.empty((rows // max(group_rows, 1),), dtype=torch.float32, device=x.device)
    check(lib.xaxb_quantize_current(ctx, st, ptr(x), rows, cols, group_rows, ptr(q), ptr(scale), ptr(inv), ptr(amax)),
          "quantize_current")
    return q, scale, inv, amax


def quantize_with_amax(x: torch.Tensor, group_amax: torch.Tensor, group_rows: int):
    x = _req(x, BF16, "x")
    rows, cols = x.shape
    ctx, st, lib = _c()
    q = torch.empty((rows, cols), dtype=E4M3, device=x.device)
    scale = torch.empty((rows,), dtype=torch.float32, device=x.device)
    inv = torch.empty((rows,), dtype=torch.float32, device=x.device)
    check(lib.xaxb_quantize_with_amax(ctx, st, ptr(x), rows, cols, group_rows, ptr(group_amax), ptr(q), ptr(scale),
                                      ptr(inv)), "quantize_with_amax")
    return q, scale, inv


def dequantize(q: torch.Tensor, scale: torch.Tensor, out_dtype=BF16) -> torch.Tensor:
    """q e4m3 [rows, cols] / scale (one float32 value, or one per row) -> bf16 or float32 [rows, cols]."""
    q = _req(q, E4M3, "q")
    scale = _req(scale, torch.float32, "scale").reshape(-1)
    rows, cols = q.shape
    if scale.numel() not in (1, rows):
        raise ValueError(f"dequantize: scale has {scale.numel()} elements, expected 1 or {rows}")
    if out_dtype not in (BF16, torch.float32):
        raise ValueError("dequantize: output must be bfloat16 or float32")
    ctx, st, lib = _c()
    out = torch.empty((rows, cols), dtype=out_dtype, device=q.device)
    check(lib.xaxb_dequantize(ctx, st, ptr(q), rows, cols, ptr(scale), 0 if scale.numel() == 1 else 1,
                              1 if out_dtype == BF16 else 0, ptr(out)), "dequantize")
    return out


_DELAYED_SCRATCH: dict = {}


def quantize_delayed(x: torch.Tensor, scale_in: torch.Tensor, history: torch.Tensor, *, cast: bool = True):
    """Delayed scaling: returns (q or None, new_history, new_scale, inv_scale_used)."""
    x = _req(x, BF16, "x")
    x2 = x.reshape(-1, x.shape[-1])
    rows, cols = x2.shape
    scale_in = _req(scale_in, torch.float32, "scale_in")
    history = _req(history, torch.float32, "history")
    ctx, st, lib = _c()
    q = torch.empty((rows, cols), dtype=E4M3, device=x.device) if cast else None
    new_hist = torch.empty_like(history)
    new_scale = torch.empty((), dtype=torch.float32, device=x.device)
    inv = torch.empty((1,), dtype=torch.float32, device=x.device)
    # the kernel needs 8 zero bytes and leaves them zero: one scratch per (device, stream), made once
    key = (x.device.index, st)
    scratch = _DELAYED_SCRATCH.get(key)
    if scratch is None:
        scratch = _DELAYED_SCRATCH[key] = torch.zeros((2,), dtype=torch.float32, device=x.device)
    check(lib.xaxb_quantize_delayed(ctx, st, ptr(x2), rows, cols, ptr(scale_in), ptr(history), history.numel(), ptr(q),
                                    ptr(new_hist), ptr(new_scale), ptr(inv), ptr(scratch)), "quantize_delayed")
    return q, new_hist, new_scale, inv


# ---------------------------------------------------------------------------------------
# kernel 2


def _mul_arg(m, n_expected: int, name: str):
    if m is None:
        return None, 0
    if m.dtype != torch.float32 or not m.is_cuda:
        raise ValueError(f"{name} must be a float32 CUDA tensor")
    if m.numel() == 1:
        return m, 0
    if m.numel() != n_expected:
        raise ValueError(f"{name} has {m.numel()} elements, expected 1 or {n_expected}")
    return m.contiguous(), 1


def _gemm(fn_name, a, b, row_mul, col_mul, bias, residual, out):
    ctx, st, lib = _c()
    M, K = a.shape
    N, Kb = b.shape
    if K != Kb:
        raise ValueError(f"gemm: inner dimensions differ ({K} vs {Kb})")
    if a.stride(1) != 1 or b.stride(1) != 1:
        raise ValueError("gemm: operands must be K-contiguous")
    if out is None:
        out = torch.empty((M, N), dtype=BF16, device=a.device)
    row_mul, rs = _mul_arg(row_mul, M, "row_mul")
    col_mul, cs = _mul_arg(col_mul, N, "col_mul")
    ldr = residual.stride(0) if residual is not None else 0
    fn = getattr(lib, fn_name)
    check(fn(ctx, st, ptr(a), a.stride(0), ptr(b), b.stride(0), M, N, K, ptr(row_mul), rs, ptr(col_mul), cs,
             ptr(bias), ptr(residual), ldr, ptr(out), out.stride(0)), fn_name)
    return out


def gemm_fp8(a_q, b_q, row_mul=None, col_mul=None, bias=None, residual=None, out=None):
    """bf16( (a_q @ b_q.T) * row_mul[:, None] * col_mul[None, :] + bias + residual )."""
    if a_q.dtype != E4M3 or b_q.dtype != E4M3:
        raise ValueError("gemm_fp8 needs float8_e4m3fn operands")
    return _gemm("xaxb_gemm_fp8", a_q, b_q, row_mul, col_mul, bias, residual, out)


E5M2 = torch.float8_e5m2


def gemm_fp8_formats(a_q, b_q, row_mul=None, col_mul=None, bias=None, residual=None, out=None):
    """gemm_fp8 for operands that are float8_e4m3fn or float8_e5m2, in any combination."""
    for t in (a_q, b_q):
        if t.dtype not in (E4M3, E5M2):
            raise ValueError("gemm_fp8_formats needs float8_e4m3fn / float8_e5m2 operands")
    ctx, st, lib = _c()
    M, K = a_q.shape
    N, Kb = b_q.shape
    if K != Kb:
        raise ValueError(f"gemm: inner dimensions differ ({K} vs {Kb})")
    if a_q.stride(1) != 1 or b_q.stride(1) != 1:
        raise ValueError("gemm: operands must be K-contiguous")
    if out is None:
        out = torch.empty((M, N), dtype=BF16, device=a_q.device)
    row_mul, rs = _mul_arg(row_mul, M, "row_mul")
    col_mul, cs = _mul_arg(col_mul, N, "col_mul")
    ldr = residual.stride(0) if residual is not None else 0
    check(lib.xaxb_gemm_fp8_formats(ctx, st, ptr(a_q), a_q.stride(0), int(a_q.dtype == E5M2), ptr(b_q), b_q.stride(0),
                                    int(b_q.dtype == E5M2), M, N, K, ptr(row_mul), rs, ptr(col_mul), cs, ptr(bias),
                                    ptr(residual), ldr, ptr(out), out.stride(0)), "gemm_fp8_formats")
    return out


def quantize_e5m2(x: torch.Tensor, *, scale=None, group_rows: int | None = None):
    """x bf16 [rows, cols] -> (q float8_e5m2, scale float32 [rows], inv_scale float32 [rows]).  With ``scale`` (one
    float32 value) every element is multiplied by it; without, groups of ``group_rows`` rows (default: all rows)
    get the current scale 57344 / max|x| of the group."""
    x = _req(x, BF16, "x")
    rows, cols = x.shape
    ctx, st, lib = _c()
    q = torch.empty((rows, cols), dtype=E5M2, device=x.device)
    sc = torch.empty((rows,), dtype=torch.float32, device=x.device)
    inv = torch.empty((rows,), dtype=torch.float32, device=x.device)
    if scale is not None:
        scale = _req(scale, torch.float32, "scale").reshape(-1)
        if scale.numel() != 1:
            raise ValueError("quantize_e5m2: scale must hold one value")
        check(lib.xaxb_quantize_e5m2(ctx, st, ptr(x), rows, cols, rows, ptr(scale), None, ptr(q), ptr(sc), ptr(inv)),
              "quantize_e5m2")
    else:
        g = rows if group_rows is None else int(group_rows)
        if g <= 0 or rows % g:
            raise ValueError(f"quantize_e5m2: group_rows {g} must divide rows {rows}")
        amax = group_amax(x, g)
        check(lib.xaxb_quantize_e5m2(ctx, st, ptr(x), rows, cols, g, None, ptr(amax), ptr(q), ptr(sc), ptr(inv)),
              "quantize_e5m2")
    return q, sc, inv


def dequantize_e5m2(q: torch.Tensor, scale: torch.Tensor, out_dtype=BF16) -> torch.Tensor:
    """dequantize for float8_e5m2 bytes."""
    q = _req(q, E5M2, "q")
    scale = _req(scale, torch.float32, "scale").reshape(-1)
    rows, cols = q.shape
    if scale.numel() not in (1, rows):
        raise ValueError(f"dequantize: scale has {scale.numel()} elements, expected 1 or {rows}")
    if out_dtype not in (BF16, torch.float32):
        raise ValueError("dequantize: output must be bfloat16 or float32")
    ctx, st, lib = _c()
    out = torch.empty((rows, cols), dtype=out_dtype, device=q.device)
    check(lib.xaxb_dequantize_e5m2(ctx, st, ptr(q), rows, cols, ptr(scale), 0 if scale.numel() == 1 else 1,
                                   1 if out_dtype == BF16 else 0, ptr(out)), "dequantize_e5m2")
    return out


def lm_head_cross_entropy(hidden, weight, targets, mask=None):
    """Cross-entropy loss and accuracy of hidden bf16 [T, H] against targets int [T] under the head weight bf16
    [V, H], without materialising the [T, V] logits (they are reduced inside the GEMM's epilogue).  ``mask``:
    bool / uint8 [T], True = counted.  Returns (result float32 [3] = mean loss, accuracy, count; row_loss float32
    [T]; row_pred int32 [T])."""
    hidden = _req(hidden, BF16, "hidden")
    weight = _req(weight, BF16, "weight")
    if hidden.dim() != 2 or weight.dim() != 2 or hidden.shape[1] != weight.shape[1]:
        raise ValueError(f"lm_head_cross_entropy: hidden [T, H] and weight [V, H] expected, got {tuple(hidden.shape)}, "
                         f"{tuple(weight.shape)}")
    T, H = hidden.shape
    V = weight.shape[0]
    targets = targets.to(device=hidden.device, dtype=torch.int32).contiguous()
    if targets.shape != (T,):
        raise ValueError(f"lm_head_cross_entropy: targets must be [T] = [{T}], got {tuple(targets.shape)}")
    if mask is not None:
        mask = mask.to(device=hidden.device).reshape(-1).to(torch.uint8).contiguous()
        if mask.shape != (T,):
            raise ValueError(f"lm_head_cross_entropy: mask must be [T] = [{T}]")
    ctx, st, lib = _c()
    nws = int(lib.xaxb_lm_head_cross_entropy_workspace_bytes(T, V))
    ws = torch.empty((nws // 4,), dtype=torch.float32, device=hidden.device)
    row_loss = torch.empty((T,), dtype=torch.float32, device=hidden.device)
    row_pred = torch.empty((T,), dtype=torch.int32, device=hidden.device)
    result = torch.empty((3,), dtype=torch.float32, device=hidden.device)
    check(lib.xaxb_lm_head_cross_entropy(ctx, st, ptr(hidden), hidden.stride(0), ptr(weight), weight.stride(0), T, V, H,
                                         ptr(targets), ptr(mask), ptr(ws), nws, ptr(row_loss), ptr(row_pred), ptr(result)),
          "lm_head_cross_entropy")
    return result, row_loss, row_pred


def gemm_fp8_push(a_q, b_q, row_mul, col_mul, bias, residual, peer_ptrs, rank: int, world: int, slot_offset: int,
                  flag_offset: int):
    """gemm_fp8 whose epilogue writes the bf16 output into this rank's slot of every rank's staging buffer and
    counts the pieces in on every rank (xaxb_gemm_fp8_push); M <= 128.  Nothing is returned: the consumer is
    tp_push_sum_rmsnorm on each rank."""
    if a_q.dtype != E4M3 or b_q.dtype != E4M3:
        raise ValueError("gemm_fp8_push needs float8_e4m3fn operands")
    ctx, st, lib = _c()
    M, K = a_q.shape
    N, Kb = b_q.shape
    if K != Kb or a_q.stride(1) != 1 or b_q.stride(1) != 1:
        raise ValueError("gemm_fp8_push: operands must be K-contiguous with equal inner dimensions")
    row_mul, rs = _mul_arg(row_mul, M, "row_mul")
    col_mul, cs = _mul_arg(col_mul, N, "col_mul")
    ldr = residual.stride(0) if residual is not None else 0
    check(lib.xaxb_gemm_fp8_push(ctx, st, ptr(a_q), a_q.stride(0), ptr(b_q), b_q.stride(0), M, N, K, ptr(row_mul), rs,
                                 ptr(col_mul), cs, ptr(bias), ptr(residual), ldr, peer_ptrs, rank, world, slot_offset,
                                 flag_offset), "gemm_fp8_push")


def tp_push_sum_rmsnorm(staging_ptr: int, slot_stride: int, counter_ptr: int, totals_ptr: int, world: int, rows: int,
                        cols: int, device, weight=None, eps: float = 0.0):
    """Consumer of gemm_fp8_push on this rank: sum of the `world` staged partial outputs (local reads only) into
    x bf16 [rows, cols]; with ``weight`` also RMSNorm + per-token e4m3 cast.  Returns (x, q, scale, inv_scale)
    (the last three None without a weight)."""
    ctx, st, lib = _c()
    x = torch.empty((rows, cols), dtype=BF16, device=device)
    q = scale = inv = None
    if weight is not None:
        weight = _req(weight, BF16, "weight")
        q = torch.empty((rows, cols), dtype=E4M3, device=device)
        scale = torch.empty((rows,), dtype=torch.float32, device=device)
        inv = torch.empty((rows,), dtype=torch.float32, device=device)
    check(lib.xaxb_tp_push_sum_rmsnorm(ctx, st, staging_ptr, slot_stride, counter_ptr, totals_ptr, world, rows, cols,
                                       ptr(x), ptr(weight), float(eps), ptr(q), ptr(scale), ptr(inv)),
          "tp_push_sum_rmsnorm")
    return x, q, scale, inv


def gemm_fp8_check(a_q, b_q, row_mul=None, col_mul=None, bias=None, residual=None, out=None):
    return _gemm("xaxb_gemm_fp8_check", a_q, b_q, row_mul, col_mul, bias, residual, out)


def gemm_bf16(a, b, row_mul=None, col_mul=None, bias=None, residual=None, out=None):
    if a.dtype != BF16 or b.dtype != BF16:
        raise ValueError("gemm_bf16 needs bfloat16 operands")
    return _gemm("xaxb_gemm_bf16", a, b, row_mul, col_mul, bias, residual, out)


# ---------------------------------------------------------------------------------------
# small ops


def rmsnorm(x, weight, eps, *, want_y=True, quantize=False, group_amax=None, group_rows=0):
    """Returns (y or None, (q, scale, inv_scale) or None)."""
    x = _req(x, BF16, "x")
    weight = _req(weight, BF16, "weight")
    rows, dim = x.shape
    ctx, st, lib = _c()
    y = torch.empty_like(x) if want_y else None
    q = scale = inv = None
    if quantize:
        q = torch.empty((rows, dim), dtype=E4M3, device=x.device)
        scale = torch.empty((rows,), dtype=torch.float32, device=x.device)
        inv = torch.empty((rows,), dtype=torch.float32, device=x.device)
    check(lib.xaxb_rmsnorm(ctx, st, ptr(x), ptr(weight), float(eps), rows, dim, ptr(y), ptr(q), ptr(scale), ptr(inv),
                           ptr(group_amax), group_rows), "rmsnorm")
    return y, ((q, scale, inv) if quantize else None)


def silu_mul(gate_up, dim, *, want_h=True, quantize=False, group_amax=None, group_rows=0):
    """gate_up[rows, 2*dim] bf16 (gate | up) -> (h or None, (q, scale, inv_scale) or None)."""
    gate_up = _req(gate_up, BF16, "gate_up")
    rows, ld = gate_up.shape
    ctx, st, lib = _c()
    h = torch.empty((rows, dim), dtype=BF16, device=gate_up.device) if want_h else None
    q = scale = inv = None
    if quantize:
        q = torch.empty((rows, dim), dtype=E4M3, device=gate_up.device)
        scale = torch.empty((rows,), dtype=torch.float32, device=gate_up.device)
        inv = torch.empty((rows,), dtype=torch.float32, device=gate_up.device)
    check(lib.xaxb_silu_mul(ctx, st, ptr(gate_up), None, ld, rows, dim, ptr(h), ptr(q), ptr(scale), ptr(inv),
                            ptr(group_amax), group_rows), "silu_mul")
    return h, ((q, scale, inv) if quantize else None)


def embed(tokens, table):
    table = _req(table, BF16, "table")
    tokens = _req(tokens, torch.int32, "tokens").reshape(-1)
    ctx, st, lib = _c()
    x = torch.empty((tokens.numel(), table.shape[1]), dtype=BF16, device=table.device)
    check(lib.xaxb_embed(ctx, st, ptr(tokens), tokens.numel(), ptr(table), table.shape[0], table.shape[1], ptr(x)),
          "embed")
    return x


def argmax(logits, out=None, max_out=None):
    logits = _req(logits, BF16, "logits")
    rows, vocab = logits.shape
    ctx, st, lib = _c()
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    check(lib.xaxb_argmax(ctx, st, ptr(logits), rows, vocab, logits.stride(0), ptr(out), ptr(max_out)), "argmax")
    return out


def sample_top_p(logits, temperature: float, top_p: float, uniforms=None, *, allowed_token_range=None, eos_id: int = -1,
                 allow_eos: bool = True, out=None):
    """One token per row of bf16 logits [rows, vocab]: arg-max when ``temperature <= 0``, else the token at
    quantile ``uniforms[r]`` of the top-p nucleus of softmax(logits / temperature); ``allowed_token_range``
    (min, max) and the EOS rule mask tokens first (see xaxb_sample_top_p)."""
    logits = _req(logits, BF16, "logits")
    rows, vocab = logits.shape
    if temperature > 0:
        if uniforms is None:
            raise ValueError("sample_top_p: sampling needs one uniform per row")
        uniforms = _req(uniforms, torch.float32, "uniforms")
        if uniforms.numel() != rows:
            raise ValueError(f"sample_top_p: {uniforms.numel()} uniforms for {rows} rows")
    lo, hi = (-1, -1) if allowed_token_range is None else (int(allowed_token_range[0]), int(allowed_token_range[1]))
    if allowed_token_range is not None and hi <= lo:
        raise ValueError("allowed_token_range must satisfy max_id > min_id.")
    ctx, st, lib = _c()
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    check(lib.xaxb_sample_top_p(ctx, st, ptr(logits), rows, vocab, logits.stride(0), float(temperature), float(top_p),
                                ptr(uniforms), lo, hi, int(eos_id), 1 if allow_eos else 0, ptr(out)), "sample_top_p")
    return out


def argmax_merge(part_max, part_idx, slice_cols: int, out):
    """Global arg-max from per-slice (max, index) pairs [parts, rows]."""
    parts, rows = part_max.shape
    ctx, st, lib = _c()
    check(lib.xaxb_argmax_merge(ctx, st, ptr(part_max), ptr(part_idx), parts, rows, slice_cols, ptr(out)),
          "argmax_merge")
    return out


def tp_allreduce_sum(peer_ptrs, rank: int, world: int, data_offset: int, sync_offset: int, rows: int, cols: int, out):
    """Sum of every rank's bf16 [rows, cols] partial output (at ``data_offset`` of its symmetric
    buffer) into the local tensor ``out``.  ``peer_ptrs``: ctypes array of ``world`` mappings."""
    ctx, st, lib = _c()
    check(lib.xaxb_tp_allreduce_sum_bf16(ctx, st, peer_ptrs, rank, world, data_offset, sync_offset, rows, cols,
                                         ptr(out)), "tp_allreduce_sum")
    return out


def tp_allreduce_sum_rmsnorm(peer_ptrs, rank: int, world: int, data_offset: int, sync_offset: int, rows: int, cols: int,
                             weight, eps: float):
    """tp_allreduce_sum followed by RMSNorm and the per-token e4m3 cast, in one kernel.  Returns
    (x bf16 [rows, cols], q e4m3 [rows, cols], scale [rows], inv_scale [rows])."""
    ctx, st, lib = _c()
    dev = weight.device
    x = torch.empty((rows, cols), dtype=BF16, device=dev)
    q = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=dev)
    scale = torch.empty((rows,), dtype=torch.float32, device=dev)
    inv = torch.empty((rows,), dtype=torch.float32, device=dev)
    check(lib.xaxb_tp_allreduce_sum_rmsnorm(ctx, st, peer_ptrs, rank, world, data_offset, sync_offset, rows, cols,
                                            ptr(x), ptr(_req(weight, BF16, "weight")), float(eps), ptr(q), ptr(scale),
                                            ptr(inv)), "tp_allreduce_sum_rmsnorm")
    return x, q, scale, inv


def tp_argmax(peer_ptrs, rank: int, world: int, inbox_offset: int, sync_offset: int, part_max, part_idx, slice_cols: int,
              out):
    """Global arg-max (int32 [rows] into ``out``) from every rank's (max, local index) of its vocabulary slice."""
    ctx, st, lib = _c()
    check(lib.xaxb_tp_argmax(ctx, st, peer_ptrs, rank, world, inbox_offset, sync_offset, ptr(part_max), ptr(part_idx),
                             part_max.numel(), slice_cols, ptr(out)), "tp_argmax")
    return out


def tp_allreduce_max(peer_ptrs, rank: int, world: int, inbox_offset: int, sync_offset: int, values, out=None):
    """Element-wise maximum over ranks of a float32 vector of at most 1024 values."""
    ctx, st, lib = _c()
    if out is None:
        out = values
    check(lib.xaxb_tp_allreduce_max_f32(ctx, st, peer_ptrs, rank, world, inbox_offset, sync_offset, ptr(values),
                                        ptr(out), values.numel()), "tp_allreduce_max")
    return out


def group_amax(x, group_rows: int = 1, out=None):
    """max|x| per group of rows, float32 [rows / group_rows]."""
    x = _req(x, BF16, "x")
    rows, cols = x.shape
    ctx, st, lib = _c()
    if out is None:
        out = torch.empty((rows // group_rows,), dtype=torch.float32, device=x.device)
    check(lib.xaxb_group_amax(ctx, st, ptr(x), rows, cols, group_rows, ptr(out)), "group_amax")
    return out


# ---------------------------------------------------------------------------------------
# kernel 3


def rope_tables(head_dim: int, base: float, length: int, device=None):
    """cos/sin tables [length, head_dim/2] bf16 for positions 0..length-1, built on the host
    in the reference's op order and dtype (xax/arch/attention.py:390-397 with bf16
    activations): bf16 frequencies, positions converted to bf16, bf16 angles."""
    import ml_dtypes

    bf = ml_dtypes.bfloat16
    f32 = np.float32

    def rb(a):
        return np.asarray(a, dtype=f32).astype(bf)

    dim = head_dim // 2
    i = np.arange(0, dim).astype(bf)
    t = rb(rb(-i.astype(f32)).astype(f32) * np.asarray(np.log(f32(base))).astype(bf).astype(f32))
    t = rb(t.astype(f32) / f32(dim))
    freqs = rb(np.exp(t.astype(f32)))
    pos = np.arange(length, dtype=np.int32).astype(bf)
    ang = rb(pos.astype(f32)[:, None] * freqs.astype(f32)[None, :])
    cos = rb(np.cos(ang.astype(f32)))
    sin = rb(np.sin(ang.astype(f32)))

    def to_torch(a):
        tt = torch.from_numpy(a.view(np.uint16).astype(np.int32)).to(torch.int16).view(BF16)
        return tt.to(device) if device is not None else tt

    return to_torch(cos), to_torch(sin)


def rope_tables_yarn(head_dim: int, base: float, factor: float, original_max_position_embeddings: int, beta_slow: float,
                     beta_fast: float, length: int, device=None):
    """cos/sin tables [length, head_dim/2] bf16 with YaRN frequency interpolation and attention
    scaling (xax/arch/attention.py:401-441): float32 throughout, cast to bf16 at the end."""
    import math

    import ml_dtypes

    f32 = np.float32
    dim = head_dim // 2
    omp = original_max_position_embeddings
    low = (head_dim * math.log(omp / (beta_fast * 2 * math.pi))) / (2 * math.log(base))
    high = (head_dim * math.log(omp / (beta_slow * 2 * math.pi))) / (2 * math.log(base))
    low, high = max(low, 0), min(high, head_dim - 1)
    timescale = (f32(base) ** (np.arange(0, head_dim, 2, dtype=f32) / f32(head_dim))).astype(f32)
    extra = (f32(1.0) / timescale).astype(f32)
    inter = (f32(1.0) / (f32(factor) * timescale)).astype(f32)
    high = high if low != high else (high + 0.001)
    idx = np.arange(dim, dtype=f32)
    interp = (1 - np.clip((idx - f32(low)) / f32(high - low), 0.0, 1.0)).astype(f32)
    freq = (inter * (1 - interp) + extra * interp).astype(f32)
    angles = (np.arange(length, dtype=f32)[:, None] * freq[None, :]).astype(f32)
    scaling = f32(0.1 * 1.0 * math.log(factor) + 1.0)
    cos = (np.cos(angles) * scaling).astype(ml_dtypes.bfloat16)
    sin = (np.sin(angles) * scaling).astype(ml_dtypes.bfloat16)

    def to_torch(a):
        tt = torch.from_numpy(a.view(np.uint16).astype(np.int32)).to(torch.int16).view(BF16)
        return tt.to(device) if device is not None else tt

    return to_torch(cos), to_torch(sin)


def qk_norm(qkv, Hq: int, Hkv: int, D: int, q_weight, k_weight, eps: float):
    """RMSNorm over head_dim of the query and key heads of the fused projection output, in place."""
    qkv = _req(qkv, BF16, "qkv")
    rows, ld = qkv.shape
    ctx, st, lib = _c()
    check(lib.xaxb_qk_norm(ctx, st, ptr(qkv), ld, rows, Hq, Hkv, D, ptr(q_weight), ptr(k_weight), float(eps)), "qk_norm")
    return qkv


def rope_apply(x, positions, cos, sin, *, interleaved: bool = False):
    """Rotary embedding of x bf16 [rows, heads, D] at int32 positions [rows]."""
    x = _req(x, BF16, "x")
    rows, heads, D = x.shape
    out = torch.empty_like(x)
    ctx, st, lib = _c()
    check(lib.xaxb_rope_apply(ctx, st, ptr(x), rows, heads, D, ptr(positions), ptr(cos), ptr(sin), cos.shape[0],
                              1 if interleaved else 0, ptr(out)), "rope_apply")
    return out


def kv_append_rope(qkv, B, T, Hq, Hkv, D, positions, cos, sin, k_cache, v_cache, *, store_rotated_k=True, q_rot=None):
    """RoPE on q and k of the fused projection output, K/V written into the cache at
    positions[b] .. +T-1.  Returns q_rot [B*T, Hq, D]."""
    qkv = _req(qkv, BF16, "qkv")
    for name, t in (("k_cache", k_cache), ("v_cache", v_cache)):
        if not t.is_cuda or t.dtype != BF16 or not t.is_contiguous() or tuple(t.shape[::2]) != (B, Hkv):
            raise ValueError(f"kv_append_rope: {name} must be a contiguous bfloat16 CUDA tensor [B, max_len, Hkv, D]")
    if not positions.is_cuda or positions.dtype != torch.int32 or not positions.is_contiguous() or positions.numel() != B:
        raise ValueError("kv_append_rope: positions must be a contiguous int32 CUDA tensor [B]")
    ctx, st, lib = _c()
    if q_rot is None:
        q_rot = torch.empty((B * T, Hq, D), dtype=BF16, device=qkv.device)
    max_len = k_cache.shape[1]
    check(lib.xaxb_kv_append_rope(ctx, st, ptr(qkv), qkv.stride(0), B, T, Hq, Hkv, D, ptr(positions), ptr(cos), ptr(sin),
                                  cos.shape[0], ptr(q_rot), ptr(k_cache), ptr(v_cache), max_len,
                                  1 if store_rotated_k else 0), "kv_append_rope")
    return q_rot


def _attn_args(q_rot, k_cache, v_cache, positions, rows_per_seq: int = 1):
    """Checks shared by the attention wrappers: bf16 contiguous q [B * rows_per_seq, Hq, D] and caches
    [B, max_len, Hkv, D], int32 contiguous positions [B], all on one CUDA device.  The kernels read raw
    pointers, so a wrong dtype or a strided view would be read as something else without any error."""
    if q_rot.dim() != 3 or k_cache.dim() != 4 or v_cache.shape != k_cache.shape:
        raise ValueError(f"attention: q must be [rows, Hq, D] and both caches [B, max_len, Hkv, D], got "
                         f"{tuple(q_rot.shape)}, {tuple(k_cache.shape)}, {tuple(v_cache.shape)}")
    for name, t in (("q_rot", q_rot), ("k_cache", k_cache), ("v_cache", v_cache)):
        if not t.is_cuda or t.dtype != BF16 or not t.is_contiguous():
            raise ValueError(f"attention: {name} must be a contiguous bfloat16 CUDA tensor")
    B = k_cache.shape[0]
    if not positions.is_cuda or positions.dtype != torch.int32 or not positions.is_contiguous() or \
            positions.numel() != B:
        raise ValueError(f"attention: positions must be a contiguous int32 CUDA tensor with one entry per sequence ({B})")
    if q_rot.shape[0] != B * rows_per_seq or q_rot.shape[2] != k_cache.shape[3]:
        raise ValueError(f"attention: q {tuple(q_rot.shape)} does not match caches {tuple(k_cache.shape)} "
                         f"with {rows_per_seq} query rows per sequence")


def attn_decode_workspace(B, Hq, D, max_len, device):
    n = _lib.load().xaxb_attn_decode_workspace_bytes(B, Hq, D, max_len)
    return torch.empty((n // 4,), dtype=torch.float32, device=device)


def attn_decode(q_rot, k_cache, v_cache, positions, *, scale=None, k_is_rotated=True, cos=None, sin=None,
                workspace=None, out=None):
    """One query token per sequence; attends to cache rows 0 .. positions[b]."""
    _attn_args(q_rot, k_cache, v_cache, positions)
    B, Hq, D = q_rot.shape
    _, max_len, Hkv, _ = k_cache.shape
    ctx, st, lib = _c()
    if workspace is None:
        workspace = attn_decode_workspace(B, Hq, D, max_len, q_rot.device)
    if out is None:
        out = torch.empty_like(q_rot)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    check(lib.xaxb_attn_decode(ctx, st, ptr(q_rot), ptr(k_cache), ptr(v_cache), ptr(positions), B, Hq, Hkv, D,
                               max_len, float(scale), 1 if k_is_rotated else 0, ptr(cos), ptr(sin),
                               0 if cos is None else cos.shape[0], ptr(out), ptr(workspace),
                               workspace.numel() * 4), "attn_decode")
    return out


def attn_decode_window(q_rot, k_cache, v_cache, positions, window: int, *, scale=None, workspace=None, out=None):
    """attn_decode with a sliding window: the query at position q attends to keys q - window .. q."""
    _attn_args(q_rot, k_cache, v_cache, positions)
    B, Hq, D = q_rot.shape
    _, max_len, Hkv, _ = k_cache.shape
    ctx, st, lib = _c()
    if workspace is None:
        workspace = attn_decode_workspace(B, Hq, D, max_len, q_rot.device)
    if out is None:
        out = torch.empty_like(q_rot)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    check(lib.xaxb_attn_decode_window(ctx, st, ptr(q_rot), ptr(k_cache), ptr(v_cache), ptr(positions), B, Hq, Hkv, D,
                                      max_len, float(scale), int(window), ptr(out), ptr(workspace),
                                      workspace.numel() * 4), "attn_decode_window")
    return out


def attn_prefill_window(q_rot, k_cache, v_cache, positions, B, T, window: int, *, scale=None, out=None):
    """attn_prefill with a sliding window."""
    _attn_args(q_rot, k_cache, v_cache, positions, T)
    _, Hq, D = q_rot.shape
    _, max_len, Hkv, _ = k_cache.shape
    ctx, st, lib = _c()
    if out is None:
        out = torch.empty_like(q_rot)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    check(lib.xaxb_attn_prefill_window(ctx, st, ptr(q_rot), ptr(k_cache), ptr(v_cache), ptr(positions), B, T, Hq, Hkv, D,
                                       max_len, float(scale), int(window), ptr(out)), "attn_prefill_window")
    return out


def attn_decode_cast(q_rot, k_cache, v_cache, positions, *, scale=None, k_is_rotated=True, cos=None, sin=None,
                     workspace=None, want_out=False):
    """Decode attention whose output row [Hq*D] per sequence is cast to e4m3 with a per-token
    scale inside the merge pass.  Returns (out bf16 or None, q e4m3 [B, Hq*D], row_scale, row_inv_scale)."""
    _attn_args(q_rot, k_cache, v_cache, positions)
    B, Hq, D = q_rot.shape
    _, max_len, Hkv, _ = k_cache.shape
    ctx, st, lib = _c()
    if workspace is None:
        workspace = attn_decode_workspace(B, Hq, D, max_len, q_rot.device)
    out = torch.empty_like(q_rot) if want_out else None
    q = torch.empty((B, Hq * D), dtype=E4M3, device=q_rot.device)
    rs = torch.empty((B,), dtype=torch.float32, device=q_rot.device)
    ri = torch.empty((B,), dtype=torch.float32, device=q_rot.device)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    check(lib.xaxb_attn_decode_cast(ctx, st, ptr(q_rot), ptr(k_cache), ptr(v_cache), ptr(positions), B, Hq, Hkv, D,
                                    max_len, float(scale), 1 if k_is_rotated else 0, ptr(cos), ptr(sin),
                                    0 if cos is None else cos.shape[0], ptr(out), ptr(q), ptr(rs), ptr(ri),
                                    ptr(workspace), workspace.numel() * 4), "attn_decode_cast")
    return out, q, rs, ri


def attn_decode_cast_tp(q_rot, k_cache, v_cache, positions, peer, *, scale=None, workspace=None):
    """attn_decode_cast for this rank's heads of a tensor-parallel model: the per-token scale comes
    from the amax over ALL ranks' heads, exchanged inside the merge pass.  ``peer`` = (ctypes table of
    peer mappings, rank, world, inbox offset, flag offset).  Returns (q e4m3 [B, Hq*D], scale, inv_scale)."""
    _attn_args(q_rot, k_cache, v_cache, positions)
    B, Hq, D = q_rot.shape
    _, max_len, Hkv, _ = k_cache.shape
    ctx, st, lib = _c()
    if workspace is None:
        workspace = attn_decode_workspace(B, Hq, D, max_len, q_rot.device)
    q = torch.empty((B, Hq * D), dtype=E4M3, device=q_rot.device)
    rs = torch.empty((B,), dtype=torch.float32, device=q_rot.device)
    ri = torch.empty((B,), dtype=torch.float32, device=q_rot.device)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    ptrs, rank, world, inbox, sync = peer
    check(lib.xaxb_attn_decode_cast_tp(ctx, st, ptr(q_rot), ptr(k_cache), ptr(v_cache), ptr(positions), B, Hq, Hkv,
                                       D, max_len, float(scale), 1, None, None, 0, ptr(q), ptr(rs), ptr(ri),
                                       ptr(workspace), workspace.numel() * 4, ptrs, rank, world, inbox, sync),
          "attn_decode_cast_tp")
    return q, rs, ri


def attn_decode_append(qkv, k_cache, v_cache, positions, cos, sin, Hq: int, *, scale=None, k_is_rotated=True,
                       window=None, want_out=True, cast=False, peer=None, workspace=None):
    """A decode step's cache append and attention as one call: ``qkv`` [B, (Hq + 2 Hkv) * D] is the fused
    projection's output for the new token of every sequence (not yet in the cache); the query is rotated
    inside the attention kernel, the new key / value are written to cache row positions[b] by it.  Same
    results, bit for bit, as kv_append_rope followed by attn_decode / attn_decode_cast / attn_decode_window /
    attn_decode_cast_tp.  Returns (out bf16 [B, Hq, D] or None, q e4m3 [B, Hq*D] or None, scale, inv_scale)."""
    if qkv.dim() != 2 or k_cache.dim() != 4 or v_cache.shape != k_cache.shape:
        raise ValueError(f"attention: qkv must be [B, (Hq + 2 Hkv) * D] and both caches [B, max_len, Hkv, D], got "
                         f"{tuple(qkv.shape)}, {tuple(k_cache.shape)}, {tuple(v_cache.shape)}")
    B, max_len, Hkv, D = k_cache.shape
    for name, t in (("qkv", qkv), ("k_cache", k_cache), ("v_cache", v_cache), ("cos", cos), ("sin", sin)):
        if not t.is_cuda or t.dtype != BF16 or not t.is_contiguous():
            raise ValueError(f"attention: {name} must be a contiguous bfloat16 CUDA tensor")
    if not positions.is_cuda or positions.dtype != torch.int32 or not positions.is_contiguous() or \
            positions.numel() != B:
        raise ValueError(f"attention: positions must be a contiguous int32 CUDA tensor with one entry per sequence ({B})")
    if qkv.shape[0] != B or qkv.shape[1] < (Hq + 2 * Hkv) * D:
        raise ValueError(f"attention: qkv {tuple(qkv.shape)} does not hold {Hq} + 2 x {Hkv} heads of {D} for {B} sequences")
    if cos.shape != sin.shape or cos.dim() != 2 or cos.shape[1] != D // 2 or cos.shape[0] < max_len:
        raise ValueError("attention: cos / sin must be [table_len >= max_len, D/2]")
    if peer is not None and not cast:
        raise ValueError("attention: the exchange over ranks goes with the cast output")
    ctx, st, lib = _c()
    dev = qkv.device
    if workspace is None:
        workspace = attn_decode_workspace(B, Hq, D, max_len, dev)
    out = torch.empty((B, Hq, D), dtype=BF16, device=dev) if want_out else None
    q = rs = ri = None
    if cast:
        q = torch.empty((B, Hq * D), dtype=E4M3, device=dev)
        rs = torch.empty((B,), dtype=torch.float32, device=dev)
        ri = torch.empty((B,), dtype=torch.float32, device=dev)
    elif not want_out:
        raise ValueError("attention: nothing to compute (neither out nor the cast output wanted)")
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    ptrs, rank, world, inbox, sync = peer if peer is not None else (None, 0, 1, 0, 0)
    check(lib.xaxb_attn_decode_append(ctx, st, ptr(qkv), qkv.stride(0), ptr(k_cache), ptr(v_cache), ptr(positions), B,
                                      Hq, Hkv, D, max_len, float(scale), 1 if k_is_rotated else 0, ptr(cos), ptr(sin),
                                      cos.shape[0], -1 if window is None else int(window), ptr(out), ptr(q), ptr(rs),
                                      ptr(ri), ptr(workspace), workspace.numel() * 4, ptrs, rank, world, inbox, sync),
          "attn_decode_append")
    return out, q, rs, ri


def silu_mul_cast_tp(gate_up, dim: int, peer):
    """silu(gate) * up of this rank's slice of the hidden width, cast per row with the amax over all
    ranks (exchanged inside the kernel).  gate_up: bf16 [rows, 2*dim] (gate | up).  Returns
    (q e4m3 [rows, dim], scale, inv_scale)."""
    gate_up = _req(gate_up, BF16, "gate_up")
    rows, ld = gate_up.shape
    ctx, st, lib = _c()
    q = torch.empty((rows, dim), dtype=E4M3, device=gate_up.device)
    rs = torch.empty((rows,), dtype=torch.float32, device=gate_up.device)
    ri = torch.empty((rows,), dtype=torch.float32, device=gate_up.device)
    ptrs, rank, world, inbox, sync = peer
    check(lib.xaxb_silu_mul_cast_tp(ctx, st, ptr(gate_up), None, ld, rows, dim, ptr(q), ptr(rs), ptr(ri), ptrs, rank,
                                    world, inbox, sync), "silu_mul_cast_tp")
    return q, rs, ri


def attn_decode_static(q_rot, k_cache, v_cache, positions, *, scale=None, k_is_rotated=True, cos=None, sin=None,
                       out=None):
    """Decode attention for callers that can hand over no scratch memory: identical to
    ``attn_decode`` except that the partial results live in an array inside the library (16 MiB
    per GPU).  Shapes needing more raise; calls must not overlap on the GPU."""
    B, Hq, D = q_rot.shape
    _, max_len, Hkv, _ = k_cache.shape
    ctx, st, lib = _c()
    need, have = lib.xaxb_attn_decode_workspace_bytes(B, Hq, D, max_len), lib.xaxb_attn_decode_static_capacity_bytes()
    if need > have:  # refused on the shape alone, before anything is looked at or read
        raise ValueError(f"attn_decode_static: B={B} Hq={Hq} D={D} max_len={max_len} needs {need} bytes of scratch, the "
                         f"built-in array holds {have}; use attn_decode with a caller-provided workspace")
    _attn_args(q_rot, k_cache, v_cache, positions)
    if out is None:
        out = torch.empty_like(q_rot)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    rc = lib.xaxb_attn_decode_static(ctx, st, ptr(q_rot), ptr(k_cache), ptr(v_cache), ptr(positions), B, Hq, Hkv, D,
                                     max_len, float(scale), 1 if k_is_rotated else 0, ptr(cos), ptr(sin),
                                     0 if cos is None else cos.shape[0], ptr(out))
    if rc == _lib.WORKSPACE_TOO_SMALL:
        raise ValueError(f"attn_decode_static: {lib.xaxb_last_error().decode()}")
    check(rc, "attn_decode_static")
    return out


def attn_prefill(q_rot, k_cache, v_cache, positions, B, T, *, scale=None, out=None):
    """Causal attention of T new tokens per sequence (already in the cache) against the cache."""
    _attn_args(q_rot, k_cache, v_cache, positions, T)
    _, Hq, D = q_rot.shape
    _, max_len, Hkv, _ = k_cache.shape
    ctx, st, lib = _c()
    if out is None:
        out = torch.empty_like(q_rot)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    check(lib.xaxb_attn_prefill(ctx, st, ptr(q_rot), ptr(k_cache), ptr(v_cache), ptr(positions), B, T, Hq, Hkv, D,
                                max_len, float(scale), ptr(out)), "attn_prefill")
    return out


def attn_cross(q, k, v, kv_lens=None, *, scale=None, out=None):
    """Cross-attention: q bf16 [B*T, Hq, D] (or [T, Hq, D] with B = 1) against k, v bf16 [B, S, Hkv, D]; every
    query of sequence b sees rows 0 .. kv_lens[b]-1 (default: all S).  Returns bf16 like q."""
    if k.dim() != 4 or v.shape != k.shape or q.dim() != 3:
        raise ValueError(f"attention: q must be [rows, Hq, D] and k, v [B, S, Hkv, D], got {tuple(q.shape)}, "
                         f"{tuple(k.shape)}, {tuple(v.shape)}")
    B, S, Hkv, D = k.shape
    if kv_lens is None:
        kv_lens = torch.full((B,), S, dtype=torch.int32, device=k.device)
    _attn_args(q, k, v, kv_lens, q.shape[0] // max(B, 1))
    if q.shape[0] % B:
        raise ValueError("attention: the query rows must divide evenly over the sequences")
    T = q.shape[0] // B
    Hq = q.shape[1]
    ctx, st, lib = _c()
    if out is None:
        out = torch.empty_like(q)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    check(lib.xaxb_attn_cross(ctx, st, ptr(q), ptr(k), ptr(v), ptr(kv_lens), B, T, Hq, Hkv, D, S, float(scale), ptr(out)),
          "attn_cross")
    return out


def attn_check(q_rot, k_cache, v_cache, positions, B, T, *, scale=None):
    _attn_args(q_rot, k_cache, v_cache, positions, T)
    _, Hq, D = q_rot.shape
    _, max_len, Hkv, _ = k_cache.shape
    ctx, st, lib = _c()
    out = torch.empty_like(q_rot)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    check(lib.xaxb_attn_check(ctx, st, ptr(q_rot), ptr(k_cache), ptr(v_cache), ptr(positions), B, T, Hq, Hkv, D,
                              max_len, float(scale), ptr(out)), "attn_check")
    return out


def advance_positions(positions, delta: int):
    ctx, st, lib = _c()
    check(lib.xaxb_advance_positions(ctx, st, ptr(positions), positions.numel(), int(delta)), "advance_positions")
    return positions
