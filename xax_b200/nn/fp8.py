"""B200-native mirror of ``xax/nn/fp8.py``: same names, arguments and results, computed by the
library's sm_100a kernels on torch CUDA tensors (torch supplies memory and streams only).

Differences from the reference, all deliberate:
  * the quantise -> dequantise -> bf16 matmul pattern (xax/nn/fp8.py:335-339), which exists so
    that XLA can pattern-match an FP8 GEMM, is executed as what it stands for: e4m3 bytes go
    straight into an e4m3 x e4m3 tensor-core GEMM whose epilogue applies 1/(sx*sw), the bias
    and the bf16 cast.  The e4m3 bytes, amax, history and scales are bit-identical to the
    reference's; the output differs from the QDQ formulation by ~4e-3 relative;
  * the weight is quantised once per (weight, scale) and cached instead of on every call
    (xax/nn/fp8.py:336);
  * ``float8_e5m2`` is served by the free functions (``quantize``, ``dequantize``, ``quantize_dequantize``,
    ``fp8_matmul``: what the reference's tests exercise in both formats); ``Fp8Linear`` itself, i.e. the
    transformer path, takes ``float8_e4m3fn`` only.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import ops

# xax/nn/fp8.py:30-34
E4M3_MAX = float(torch.finfo(torch.float8_e4m3fn).max)
E5M2_MAX = float(torch.finfo(torch.float8_e5m2).max)
AMAX_HISTORY_LENGTH = 1024


def _dev(device=None):
    return torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)


def _only_e4m3(fp8_dtype) -> None:
    if fp8_dtype != torch.float8_e4m3fn:
        raise ValueError(f"unsupported fp8 dtype {fp8_dtype}: the fused sm_100a kernels of the linear layer implement "
                         "float8_e4m3fn only")


def _fp8_format(fp8_dtype) -> None:
    if fp8_dtype not in (torch.float8_e4m3fn, torch.float8_e5m2):
        raise ValueError(f"unsupported fp8 dtype {fp8_dtype}: float8_e4m3fn or float8_e5m2")


def get_fp8_max(fp8_dtype: torch.dtype, compute_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """xax/nn/fp8.py:37-47."""
    return torch.tensor(float(torch.finfo(fp8_dtype).max), dtype=compute_dtype)


def compute_scale(amax: torch.Tensor, scale: torch.Tensor, fp8_max: torch.Tensor, margin: int = 0) -> torch.Tensor:
    """xax/nn/fp8.py:50-79 (scalar bookkeeping, not on the hot path: the delayed-scaling
    kernel computes the same expression on the device)."""
    amax = torch.as_tensor(amax)
    scale = torch.as_tensor(scale).to(amax.device)
    fp8_max = torch.as_tensor(fp8_max).to(amax.device)
    sf = (fp8_max / amax) / (2**margin)
    sf = torch.where(amax > 0, sf, scale.to(sf.dtype))
    return torch.where(torch.isfinite(amax), sf, scale.to(sf.dtype))


@dataclass
class Fp8Scales:
    """xax/nn/fp8.py:165-175."""

    input_scale: torch.Tensor
    input_amax_history: torch.Tensor
    kernel_scale: torch.Tensor
    kernel_amax_history: torch.Tensor


def init_fp8_scales(history_length: int = AMAX_HISTORY_LENGTH, compute_dtype: torch.dtype = torch.float32,
                    device=None) -> Fp8Scales:
    """xax/nn/fp8.py:178-196."""
    d = _dev(device)
    return Fp8Scales(
        input_scale=torch.ones((), dtype=compute_dtype, device=d),
        input_amax_history=torch.zeros((history_length,), dtype=compute_dtype, device=d),
        kernel_scale=torch.ones((), dtype=compute_dtype, device=d),
        kernel_amax_history=torch.zeros((history_length,), dtype=compute_dtype, device=d),
    )


def compute_amax_history(x: torch.Tensor, amax_history: torch.Tensor) -> torch.Tensor:
    """xax/nn/fp8.py:82-94 via the delayed-scaling kernel (state update only)."""
    x2 = x.to(torch.bfloat16).reshape(-1, x.shape[-1]) if x.dim() > 1 else x.to(torch.bfloat16).reshape(1, -1)
    x2 = _pad_cols(x2)
    one = torch.ones((), dtype=torch.float32, device=x.device)
    _, new_hist, _, _ = ops.quantize_delayed(x2, one, amax_history.to(torch.float32), cast=False)
    return new_hist.to(amax_history.dtype)


def _pad_cols(x2: torch.Tensor) -> torch.Tensor:
    """The kernels read 8 bf16 at a time; zero padding changes neither amax nor the bytes kept."""
    pad = (-x2.shape[-1]) % 8
    return torch.nn.functional.pad(x2, (0, pad)) if pad else x2


def quantize(x: torch.Tensor, fp8_dtype: torch.dtype, scale: torch.Tensor,
             compute_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """xax/nn/fp8.py:97-120 for a scalar scale.  The kernels implement the bf16 compute dtype
    that Fp8Linear uses; x is cast to bf16 first."""
    _fp8_format(fp8_dtype)
    if torch.as_tensor(scale).numel() != 1:
        raise ValueError("quantize: the kernel path takes a scalar scale")
    shape = x.shape
    x2 = x.to(torch.bfloat16).reshape(-1, shape[-1]) if x.dim() > 1 else x.to(torch.bfloat16).reshape(1, -1)
    cols = x2.shape[-1]
    x2 = _pad_cols(x2)
    s = torch.as_tensor(scale, dtype=torch.float32, device=x.device).reshape(())
    if fp8_dtype == torch.float8_e5m2:
        q, _, _ = ops.quantize_e5m2(x2.contiguous(), scale=s)
        return q[:, :cols].reshape(shape)
    hist = torch.zeros((1,), dtype=torch.float32, device=x.device)
    q, _, _, _ = ops.quantize_delayed(x2, s, hist)
    return q[:, :cols].reshape(shape)


def dequantize(x: torch.Tensor, compute_dtype: torch.dtype, scale: torch.Tensor) -> torch.Tensor:
    """xax/nn/fp8.py:123-138 for a scalar scale: compute_dtype(x) / compute_dtype(scale).  The linear layer
    never materialises the dequantised tensor; this is the free function."""
    _fp8_format(x.dtype)
    shape = x.shape
    x2 = x.reshape(-1, shape[-1]) if x.dim() > 1 else x.reshape(1, -1)
    cols = x2.shape[-1]
    pad = (-cols) % 8
    if pad:
        x2 = torch.nn.functional.pad(x2.view(torch.uint8), (0, pad)).view(x.dtype)
    s = torch.as_tensor(scale, dtype=torch.float32, device=x.device).reshape(-1)
    if s.numel() != 1:
        raise ValueError("dequantize: the kernel path takes a scalar scale")
    deq = ops.dequantize_e5m2 if x.dtype == torch.float8_e5m2 else ops.dequantize
    return deq(x2.contiguous(), s, compute_dtype)[:, :cols].reshape(shape)


def quantize_dequantize(x, fp8_dtype, scale, compute_dtype=torch.float32):
    """xax/nn/fp8.py:141-162."""
    return dequantize(quantize(x, fp8_dtype, scale, compute_dtype), compute_dtype, scale)


class Fp8Linear:
    """xax/nn/fp8.py:199-344.  ``weight`` is (out_features, in_features) like the reference."""

    def __init__(self, in_features: int, out_features: int, *, key=None, use_bias: bool = True, use_fp8: bool = True,
                 compute_dtype: torch.dtype = torch.bfloat16, fp8_dtype: torch.dtype = torch.float8_e4m3fn,
                 weight: torch.Tensor | None = None, bias: torch.Tensor | None = None, device=None):
        if compute_dtype != torch.bfloat16:
            raise ValueError("the sm_100a kernels compute in bfloat16 only")
        if use_fp8:
            _only_e4m3(fp8_dtype)
        self.in_features, self.out_features = in_features, out_features
        self.use_fp8, self.compute_dtype, self.fp8_dtype = use_fp8, compute_dtype, fp8_dtype
        d = _dev(device)
        if weight is None:  # U(+-1/sqrt(in)), xax/nn/fp8.py:251-269
            gen = key if isinstance(key, torch.Generator) else torch.Generator(device="cpu").manual_seed(int(key or 0))
            bound = 1.0 / math.sqrt(in_features)
            weight = ((torch.rand((out_features, in_features), generator=gen) * 2 - 1) * bound).to(compute_dtype).to(d)
            bias = ((torch.rand((out_features,), generator=gen) * 2 - 1) * bound).to(compute_dtype).to(d) if use_bias else None
        self.weight = weight
        self.bias = bias
        self._wq_current = None  # (q, inv_scale) under current scaling
        self._wq_delayed = None  # (scale tensor, its version, q, inv_scale, weight key)
        self._wq_key = None      # _weight_key() the current-scaling copy was made from

    # -- weight quantisation (cached) ----------------------------------------------------------
    def _weight_key(self):
        """Identity of the weight the cached e4m3 copies were made from: a new tensor assigned to
        ``weight`` or an in-place update of it (torch bumps ``_version``) makes them stale."""
        w = self.weight
        return (w.data_ptr(), w._version, tuple(w.shape))

    def invalidate(self) -> None:
        """Drop the cached e4m3 weights (loaders that overwrite ``weight`` behind torch's back call this)."""
        self._wq_current = None
        self._wq_delayed = None
        self._wq_key = None

    def set_weight_q_current(self, q: torch.Tensor, inv_scale: torch.Tensor) -> None:
        """Install e4m3 bytes made elsewhere for the current weight (tensor-parallel ranks quantise their
        slice with the amax of the whole weight, which this layer cannot know on its own)."""
        self._wq_current = (q, inv_scale)
        self._wq_key = self._weight_key()

    def weight_q_current(self):
        """e4m3 weight and its dequantisation multiplier 1/sw under current scaling."""
        key = self._weight_key()
        if self._wq_current is None or self._wq_key != key:
            w = self.weight.to(torch.bfloat16)
            q, _, inv, _ = ops.quantize_current(w, group_rows=w.shape[0])
            self._wq_current = (q, inv[:1].clone())
            self._wq_delayed = None
            self._wq_key = key
        return self._wq_current

    def _weight_q_delayed(self, scales: Fp8Scales):
        ks = scales.kernel_scale
        c = self._wq_delayed
        key = self._weight_key()
        w = self.weight.to(torch.bfloat16)
        if c is not None and c[0] is ks and c[1] == ks._version and c[4] == key:
            q, inv = c[2], c[3]
            _, new_hist, new_scale, _ = ops.quantize_delayed(w, ks, scales.kernel_amax_history, cast=False)
        else:
            q, new_hist, new_scale, inv = ops.quantize_delayed(w, ks, scales.kernel_amax_history)
            self._wq_delayed = (ks, ks._version, q, inv, key)
        return q, inv, new_hist, new_scale

    # -- forward --------------------------------------------------------------------------------
    def __call__(self, x: torch.Tensor, scales: Fp8Scales | None = None, *, per_row: bool = False, residual=None):
        """Returns (out, updated scales or None).  ``per_row`` gives every row its own current
        scale -- what the reference computes when the layer is vmapped over rows
        (xax/arch/attention.py:279); ``residual`` is added in the GEMM epilogue."""
        shape = x.shape
        x2 = x.reshape(-1, shape[-1]) if x.dim() != 2 else x
        if x2.shape[-1] != self.in_features:
            raise ValueError(f"expected last dimension {self.in_features}, got {x2.shape[-1]}")
        res2 = None if residual is None else residual.reshape(-1, self.out_features)
        if not self.use_fp8:  # xax/nn/fp8.py:288-293
            out = ops.gemm_bf16(x2.to(torch.bfloat16).contiguous(), self.weight, None, None, self.bias, res2)
            return out.reshape(*shape[:-1], self.out_features), None
        x2 = x2.to(self.compute_dtype).contiguous()
        updated = None
        if scales is not None:  # delayed scaling, xax/nn/fp8.py:299-326
            xq, in_hist, in_scale, x_inv = ops.quantize_delayed(x2, scales.input_scale, scales.input_amax_history)
            wq, w_inv, k_hist, k_scale = self._weight_q_delayed(scales)
            updated = Fp8Scales(in_scale, in_hist, k_scale, k_hist)
        else:  # current scaling, xax/nn/fp8.py:327-332
            xq, _, x_inv, _ = ops.quantize_current(x2, 1 if per_row else x2.shape[0])
            wq, w_inv = self.weight_q_current()
        out = ops.gemm_fp8(xq, wq, x_inv, w_inv, self.bias, res2)
        return out.reshape(*shape[:-1], self.out_features), updated

    def forward_quantized(self, xq: torch.Tensor, x_inv: torch.Tensor, residual=None, out=None):
        """GEMM on activations that an upstream kernel (RMSNorm / SiLU*up) already cast.  ``out`` may be a
        tensor to write into, or a tensor-parallel push target (an object with ``push_gemm``): the epilogue
        then writes the partial output to every rank's staging buffer and the target is returned."""
        wq, w_inv = self.weight_q_current()
        if out is not None and hasattr(out, "push_gemm"):
            return out.push_gemm(xq, wq, x_inv, w_inv, self.bias, residual)
        return ops.gemm_fp8(xq, wq, x_inv, w_inv, self.bias, residual, out)


def fp8_matmul(a: torch.Tensor, b: torch.Tensor, compute_dtype: torch.dtype = torch.bfloat16,
               fp8_dtype: torch.dtype = torch.float8_e4m3fn) -> torch.Tensor:
    """xax/nn/fp8.py:347-378: a @ b with per-tensor current scaling of both operands."""
    _fp8_format(fp8_dtype)
    a2 = a.to(torch.bfloat16).reshape(-1, a.shape[-1]).contiguous()
    bt = b.to(torch.bfloat16).t().contiguous()  # (N, K), K-contiguous
    if fp8_dtype == torch.float8_e5m2:
        aq, _, a_inv = ops.quantize_e5m2(a2)
        bq, _, b_inv = ops.quantize_e5m2(bt)
        out = ops.gemm_fp8_formats(aq, bq, a_inv, b_inv[:1])
        return out.reshape(*a.shape[:-1], b.shape[-1])
    aq, _, a_inv, _ = ops.quantize_current(a2, a2.shape[0])
    bq, _, b_inv, _ = ops.quantize_current(bt, bt.shape[0])
    out = ops.gemm_fp8(aq, bq, a_inv, b_inv[:1])
    return out.reshape(*a.shape[:-1], b.shape[-1])
