"""ctypes binding of the C ABI declared in ``include/xaxb200.h``.

The library is loaded on first use.  There is no CPU fallback: if the shared library is
missing, or no sm_100 GPU is present, the call raises.
"""

from __future__ import annotations

import ctypes
import threading
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_void_p

from . import _build

_lock = threading.Lock()
_lib: ctypes.CDLL | None = None
_ctxs: dict[int, c_void_p] = {}

OK = 0
BAD_ARGUMENT = 1
UNSUPPORTED = 2
WORKSPACE_TOO_SMALL = 3
LAUNCH_FAILED = 4
DEVICE_TIMEOUT = 5
CACHE_OVERFLOW = 6

_P = c_void_p
_I64 = c_int64
_F = c_float
_I = c_int

# name -> (restype, argtypes); mirrors include/xaxb200.h one to one
SIGNATURES: dict[str, tuple] = {
    "xaxb_ctx_create": (_I, [_I, POINTER(_P)]),
    "xaxb_ctx_destroy": (_I, [_P]),
    "xaxb_ctx_status": (_I, [_P, _P, POINTER(_I)]),
    "xaxb_num_sms": (_I, [_P]),
    "xaxb_status_string": (c_char_p, [_I]),
    "xaxb_last_error": (c_char_p, []),
    "xaxb_set_programmatic_launch": (_I, [_I]),
    "xaxb_programmatic_launch_enabled": (_I, []),
    "xaxb_launch_count": (ctypes.c_longlong, [_I]),
    "xaxb_set_wait_limit_ms": (_I, [_P, _I, _I]),
    "xaxb_quantize_current": (_I, [_P, _P, _P, _I64, _I64, _I64, _P, _P, _P, _P]),
    "xaxb_quantize_delayed": (_I, [_P, _P, _P, _I64, _I64, _P, _P, _I, _P, _P, _P, _P, _P]),
    "xaxb_dequantize": (_I, [_P, _P, _P, _I64, _I64, _P, _I, _I, _P]),
    "xaxb_quantize_with_amax": (_I, [_P, _P, _P, _I64, _I64, _I64, _P, _P, _P, _P]),
    "xaxb_quantize_e5m2": (_I, [_P, _P, _P, _I64, _I64, _I64, _P, _P, _P, _P, _P]),
    "xaxb_dequantize_e5m2": (_I, [_P, _P, _P, _I64, _I64, _P, _I, _I, _P]),
    "xaxb_gemm_fp8_formats": (_I, [_P, _P, _P, _I64, _I, _P, _I64, _I, _I64, _I64, _I64, _P, _I, _P, _I, _P, _P, _I64,
                                   _P, _I64]),
    "xaxb_gemm_fp8": (_I, [_P, _P, _P, _I64, _P, _I64, _I64, _I64, _I64, _P, _I, _P, _I, _P, _P, _I64, _P, _I64]),
    "xaxb_gemm_bf16": (_I, [_P, _P, _P, _I64, _P, _I64, _I64, _I64, _I64, _P, _I, _P, _I, _P, _P, _I64, _P, _I64]),
    "xaxb_gemm_force_plan": (_I, [_I, _I]),
    "xaxb_gemm_set_prefetch": (_I, [_I]),
    "xaxb_gemm_fp8_check": (_I, [_P, _P, _P, _I64, _P, _I64, _I64, _I64, _I64, _P, _I, _P, _I, _P, _P, _I64, _P, _I64]),
    "xaxb_rmsnorm": (_I, [_P, _P, _P, _P, _F, _I64, _I64, _P, _P, _P, _P, _P, _I64]),
    "xaxb_silu_mul": (_I, [_P, _P, _P, _P, _I64, _I64, _I64, _P, _P, _P, _P, _P, _I64]),
    "xaxb_embed": (_I, [_P, _P, _P, _I64, _P, _I64, _I64, _P]),
    "xaxb_argmax": (_I, [_P, _P, _P, _I64, _I64, _I64, _P, _P]),
    "xaxb_argmax_merge": (_I, [_P, _P, _P, _P, _I64, _I64, _I64, _P]),
    "xaxb_sample_top_p": (_I, [_P, _P, _P, _I64, _I64, _I64, _F, _F, _P, c_int32, c_int32, c_int32, _I, _P]),
    "xaxb_group_amax": (_I, [_P, _P, _P, _I64, _I64, _I64, _P]),
    "xaxb_kv_append_rope": (_I, [_P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _P, _P, _P, _I64, _P, _P, _P, _I64, _I]),
    "xaxb_attn_decode_workspace_bytes": (_I64, [_I64, _I64, _I64, _I64]),
    "xaxb_attn_decode": (_I, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _F, _I, _P, _P, _I64, _P, _P, _I64]),
    "xaxb_attn_decode_window": (_I, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _F, _I64, _P, _P, _I64]),
    "xaxb_attn_decode_force_variant": (_I, [_I]),
    "xaxb_attn_decode_cast": (_I, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _F, _I, _P, _P, _I64, _P, _P, _P,
                                   _P, _P, _I64]),
    "xaxb_attn_decode_static_capacity_bytes": (_I64, []),
    "xaxb_attn_decode_static": (_I, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _F, _I, _P, _P, _I64, _P]),
    "xaxb_attn_prefill": (_I, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _F, _P]),
    "xaxb_attn_prefill_window": (_I, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _F, _I64, _P]),
    "xaxb_attn_check": (_I, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _F, _P]),
    "xaxb_qk_norm": (_I, [_P, _P, _P, _I64, _I64, _I64, _I64, _I64, _P, _P, _F]),
    "xaxb_rope_apply": (_I, [_P, _P, _P, _I64, _I64, _I64, _P, _P, _P, _I64, _I, _P]),
    "xaxb_advance_positions": (_I, [_P, _P, _P, _I64, c_int32]),
    "xaxb_tp_sync_bytes": (_I64, []),
    "xaxb_tp_max_inbox_bytes": (_I64, []),
    "xaxb_tp_allreduce_sum_bf16": (_I, [_P, _P, _P, _I, _I, _I64, _I64, _I64, _I64, _P]),
    "xaxb_tp_allreduce_sum_rmsnorm": (_I, [_P, _P, _P, _I, _I, _I64, _I64, _I64, _I64, _P, _P, _F, _P, _P, _P]),
    "xaxb_silu_mul_cast_tp": (_I, [_P, _P, _P, _P, _I64, _I64, _I64, _P, _P, _P, _P, _I, _I, _I64, _I64]),
    "xaxb_attn_decode_cast_tp": (_I, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _F, _I, _P, _P, _I64, _P, _P,
                                      _P, _P, _I64, _P, _I, _I, _I64, _I64]),
    "xaxb_lm_head_cross_entropy_workspace_bytes": (_I64, [_I64, _I64]),
    "xaxb_lm_head_cross_entropy": (_I, [_P, _P, _P, _I64, _P, _I64, _I64, _I64, _I64, _P, _P, _P, _I64, _P, _P, _P]),
    "xaxb_attn_cross": (_I, [_P, _P, _P, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _I64, _F, _P]),
    "xaxb_attn_decode_append": (_I, [_P, _P, _P, _I64, _P, _P, _P, _I64, _I64, _I64, _I64, _I64, _F, _I, _P, _P, _I64,
                                     _I64, _P, _P, _P, _P, _P, _I64, _P, _I, _I, _I64, _I64]),
    "xaxb_gemm_fp8_push": (_I, [_P, _P, _P, _I64, _P, _I64, _I64, _I64, _I64, _P, _I, _P, _I, _P, _P, _I64, _P, _I, _I,
                                _I64, _I64]),
    "xaxb_tp_push_totals_bytes": (_I64, []),
    "xaxb_tp_push_sum_rmsnorm": (_I, [_P, _P, _P, _I64, _P, _P, _I, _I64, _I64, _P, _P, _F, _P, _P, _P]),
    "xaxb_tp_argmax_inbox_bytes": (_I64, []),
    "xaxb_tp_argmax": (_I, [_P, _P, _P, _I, _I, _I64, _I64, _P, _P, _I64, _I64, _P]),
    "xaxb_tp_allreduce_max_f32": (_I, [_P, _P, _P, _I, _I, _I64, _I64, _P, _P, _I64]),
}


class XaxbError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


def load() -> ctypes.CDLL:
    """Load (building first if the sources changed and nvcc is present) the shared library."""
    global _lib
    with _lock:
        if _lib is None:
            if not _build.is_current():
                try:
                    _build.build()
                except Exception as e:  # noqa: BLE001
                    if not _build.LIB_PATH.exists():
                        raise RuntimeError(
                            "libxaxb200.so is missing and could not be built; run "
                            "`python -m xax_b200._build` (needs nvcc). There is no CPU fallback."
                        ) from e
            lib = ctypes.CDLL(str(_build.LIB_PATH))
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


def ctx(device: int | None = None) -> c_void_p:
    """The per-device context handle (created on first use)."""
    import torch

    if not torch.cuda.is_available():
        raise RuntimeError("xax_b200 needs a CUDA device (sm_100a); there is no CPU fallback")
    if device is None:
        device = torch.cuda.current_device()
    lib = load()
    with _lock:
        if device not in _ctxs:
            h = c_void_p()
            rc = lib.xaxb_ctx_create(int(device), ctypes.byref(h))
            if rc != OK:
                raise XaxbError(rc, f"xaxb_ctx_create: {lib.xaxb_last_error().decode()}")
            _ctxs[device] = h
        return _ctxs[device]


def stream_ptr() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream


def check(rc: int, what: str) -> None:
    """Map a status code to the exception the reference would raise for the same condition."""
    if rc == OK:
        return
    lib = load()
    msg = f"{what}: {lib.xaxb_status_string(rc).decode()}"
    detail = lib.xaxb_last_error().decode()
    if detail:
        msg += f" ({detail})"
    if rc in (BAD_ARGUMENT, UNSUPPORTED, CACHE_OVERFLOW):
        raise ValueError(msg)
    raise XaxbError(rc, msg)


def device_status(device: int | None = None) -> None:
    """Synchronise the current stream and raise if a device-side wait gave up or a kernel
    recorded an error."""
    lib = load()
    site = c_int(0)
    rc = lib.xaxb_ctx_status(ctx(device), stream_ptr(), ctypes.byref(site))
    if rc != OK:
        check(rc, f"device status (site {site.value})")


def ptr(t) -> int | None:
    """Device pointer of a torch tensor (None passes NULL)."""
    return None if t is None else t.data_ptr()
