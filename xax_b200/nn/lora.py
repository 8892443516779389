"""B200-native mirror of the inference side of ``xax/nn/lora.py``: ``LoRALinear`` (a frozen linear layer plus
a low-rank residual scaled by alpha / rank), ``LoRALinear.from_linear`` and ``loraize_linear``.  The forward runs as
three bf16 tensor-core GEMMs; dropout exists only in training and is refused here (``inference`` must be True)."""

from __future__ import annotations

import math

import torch

from .. import ops

BF16 = torch.bfloat16


class LoRALinear:
    """xax/nn/lora.py:14-97.  ``weight_oi`` (out, in), ``bias_o`` (out) or None, ``lora_a_ir`` (in, rank),
    ``lora_b_ro`` (rank, out); the residual is (x @ A) @ B * (alpha / rank).  ``rank`` must be a multiple of 8
    (the GEMM kernels read 16 bytes at a time)."""

    def __init__(self, weight_oi, bias_o, lora_a_ir, lora_b_ro, rank: int, alpha: float = 16.0, dropout_rate: float = 0.0):
        if rank < 1:
            raise ValueError("rank must be at least 1")  # :54-55
        if rank % 8 or lora_a_ir.shape != (weight_oi.shape[1], rank) or lora_b_ro.shape != (rank, weight_oi.shape[0]):
            raise ValueError(f"LoRA factors must be (in, rank) and (rank, out) with rank a multiple of 8, got "
                             f"{tuple(lora_a_ir.shape)} and {tuple(lora_b_ro.shape)} for rank {rank}")
        self.weight_oi, self.bias_o, self.lora_a_ir, self.lora_b_ro = weight_oi, bias_o, lora_a_ir, lora_b_ro
        self.rank, self.alpha, self.dropout_rate = rank, alpha, dropout_rate
        self._t = None  # K-contiguous copies of the two factors, keyed on their identity

    @classmethod
    def from_linear(cls, linear, rank: int, *, alpha: float = 16.0, dropout_rate: float = 0.0, key=None) -> "LoRALinear":
        """:34-74: A ~ N(0, 1) / sqrt(in), B = 0 (so the layer starts out equal to ``linear``)."""
        if rank < 1:
            raise ValueError("rank must be at least 1")
        w = linear.weight
        gen = key if isinstance(key, torch.Generator) else torch.Generator(device="cpu").manual_seed(int(key or 0))
        a = (torch.randn((w.shape[1], rank), generator=gen) / math.sqrt(float(w.shape[1]))).to(w.dtype).to(w.device)
        b = torch.zeros((rank, w.shape[0]), dtype=w.dtype, device=w.device)
        return cls(w, linear.bias, a, b, rank, alpha, dropout_rate)

    @property
    def scaling(self) -> float:
        return self.alpha / self.rank  # :76-79

    @property
    def in_features(self) -> int:
        return self.weight_oi.shape[1]

    @property
    def out_features(self) -> int:
        return self.weight_oi.shape[0]

    def factors_t(self):
        """(A^T [rank, in], B^T [out, rank]) bf16, K-contiguous for the GEMM kernels (cached)."""
        key = (self.lora_a_ir.data_ptr(), self.lora_a_ir._version, self.lora_b_ro.data_ptr(), self.lora_b_ro._version)
        if self._t is None or self._t[0] != key:
            self._t = (key, self.lora_a_ir.to(BF16).t().contiguous(), self.lora_b_ro.to(BF16).t().contiguous())
        return self._t[1], self._t[2]

    def __call__(self, x_bi: torch.Tensor, *, key=None, inference: bool = True) -> torch.Tensor:
        """:81-97 without dropout: x @ W^T + bias + ((x @ A) @ B) * scaling."""
        if self.dropout_rate > 0.0 and not inference:
            raise ValueError("LoRA dropout is a training feature; this library runs inference (pass inference=True)")
        x2 = x_bi.reshape(-1, x_bi.shape[-1]).to(BF16).contiguous()
        a_t, b_t = self.factors_t()
        scale = torch.full((1,), self.scaling, dtype=torch.float32, device=x2.device)
        low = ops.gemm_bf16(x2, a_t)                           # x @ A          [rows, rank]
        delta = ops.gemm_bf16(low, b_t, None, scale)           # (.. @ B) * s   [rows, out]
        y = ops.gemm_bf16(x2, self.weight_oi.to(BF16), None, None,
                          None if self.bias_o is None else self.bias_o.to(BF16), delta)
        return y.reshape(*x_bi.shape[:-1], self.out_features)


def loraize_linear(linear, rank: int, *, alpha: float = 16.0, dropout_rate: float = 0.0, key=None) -> LoRALinear:
    """xax/nn/lora.py:100-119."""
    return LoRALinear.from_linear(linear, rank, alpha=alpha, dropout_rate=dropout_rate, key=key)
