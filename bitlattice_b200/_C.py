"""ctypes binding of ``libbitlattice_b200.so`` (declared in ``include/bitlattice_b200.h``).

The library is the only implementation of the arithmetic in this package: there is no Python or CPU fallback. Loading
fails loudly when the shared object is missing, and every non-zero status becomes a ``RuntimeError`` carrying the
library's message (the reference raises the same type from ``TORCH_CHECK``).
"""
from __future__ import annotations

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libbitlattice_b200.so")

F32, BF16, F16 = 0, 1, 2
SF_ROWMAJOR, SF_BLOCKED = 0, 1
DTYPE = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}

_c = ctypes
_P = _c.c_void_p
_SIGNATURES = {
    "bl_version": (_c.c_int, []),
    "bl_last_error": (_c.c_char_p, []),
    "bl_nvfp4_step_quantized": (_c.c_int, [_P, _P, _P, _P, _P, _P, _c.c_int64, _c.c_int64, _c.c_uint64, _c.c_int,
                                           _c.c_int, _c.c_double, _c.c_double, _c.c_int, _c.c_uint32, _c.c_uint32,
                                           _c.c_int, _c.c_int, _c.c_int, _c.c_double, _c.c_int, _P]),
    "bl_update_scratch_bytes": (_c.c_size_t, [_c.c_int64, _c.c_int64, _c.c_int, _c.c_double]),
    "bl_nvfp4_lattice_update": (_c.c_int, [_P, _P, _P, _P, _P, _c.c_int, _c.c_int64, _c.c_int64, _c.c_uint64, _c.c_int,
                                           _c.c_int, _c.c_double, _c.c_double, _c.c_int, _c.c_uint32, _c.c_uint32,
                                           _c.c_int, _c.c_int, _c.c_int, _c.c_double, _c.c_int, _c.c_double, _P,
                                           _c.c_size_t, _c.c_int, _P]),
    "bl_direction": (_c.c_int, [_P, _c.c_int, _c.c_int64, _c.c_int64, _c.c_int, _c.c_double, _P, _P, _c.c_size_t,
                                _c.c_int, _P]),
    "bl_nvfp4_dequantize": (_c.c_int, [_P, _P, _P, _c.c_int64, _c.c_int64, _P, _c.c_int, _c.c_int, _P]),
    "bl_nvfp4_amax": (_c.c_int, [_P, _c.c_int, _c.c_int64, _P, _c.c_int, _P]),
    "bl_nvfp4_quantize": (_c.c_int, [_P, _c.c_int, _c.c_int64, _c.c_int64, _P, _c.c_int64, _c.c_uint32, _P, _P,
                                     _c.c_int, _c.c_int, _P]),
    "bl_nvfp4_quantize_t": (_c.c_int, [_P, _c.c_int, _c.c_int64, _c.c_int64, _P, _c.c_int64, _c.c_uint32, _P, _P, _P,
                                       _P, _P, _c.c_int, _c.c_int, _P]),
    "bl_nvfp4_requantize_t": (_c.c_int, [_P, _P, _P, _c.c_int64, _c.c_int64, _P, _P, _P, _c.c_int, _c.c_int, _P]),
    "bl_blocked_scale_bytes": (_c.c_size_t, [_c.c_int64, _c.c_int64]),
    "bl_nvfp4_scales_to_blocked": (_c.c_int, [_P, _c.c_int64, _c.c_int64, _P, _c.c_int, _P]),
    "bl_nvfp4_gemm": (_c.c_int, [_P, _P, _P, _P, _P, _P, _c.c_int64, _c.c_int64, _c.c_int64, _P, _c.c_int,
                                 _c.c_int64, _c.c_int, _P]),
    "bl_nvfp4_gemm_status": (_c.c_int, [_c.POINTER(_c.c_int), _c.c_int]),
}

_lib = None


def exported_symbols() -> list[str]:
    """Names this binding expects the library to export (every function of the public header)."""
    return sorted(_SIGNATURES)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m bitlattice_b200.csrc.build` "
                              "(there is no fallback implementation)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def ptr(t: torch.Tensor | None):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def stream_of(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def device_of(t: torch.Tensor) -> int:
    if not t.is_cuda:
        raise RuntimeError("bitlattice_b200 kernels need CUDA tensors (there is no CPU path)")
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def check(status: int) -> None:
    if status != 0:
        raise RuntimeError(lib().bl_last_error().decode("utf-8", "replace"))


def call(name: str, *args) -> None:
    check(getattr(lib(), name)(*args))
