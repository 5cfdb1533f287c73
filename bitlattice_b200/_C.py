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
    "bl_update_many_scratch_bytes": (_c.c_size_t, [_c.c_int, _P, _P, _c.c_int, _c.c_double]),
    "bl_nvfp4_lattice_update_many": (_c.c_int, [_c.c_int, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _c.c_int, _c.c_int,
                                                _c.c_int, _c.c_double, _c.c_double, _c.c_int, _c.c_int, _c.c_int,
                                                _c.c_double, _c.c_int, _c.c_double, _P, _c.c_size_t, _c.c_int, _P,
                                                _c.POINTER(_c.c_int)]),
    "bl_update_shards_scratch_bytes": (_c.c_size_t, [_c.c_int, _P, _P, _c.c_int]),
    "bl_update_shard_stats": (_c.c_int, [_c.c_int, _P, _P, _P, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_double, _P,
                                         _c.c_size_t, _P, _P, _c.c_int, _P, _c.POINTER(_c.c_int)]),
    "bl_nvfp4_lattice_update_shards": (_c.c_int, [_c.c_int, _P, _P, _P, _P, _P, _P, _P, _c.c_int, _c.c_int, _P, _P, _P,
                                                  _P, _c.c_int, _c.c_int, _c.c_int, _c.c_double, _c.c_double, _c.c_int,
                                                  _c.c_int, _c.c_int, _c.c_double, _c.c_int, _c.c_double, _P,
                                                  _c.c_size_t, _c.c_int, _P, _c.POINTER(_c.c_int)]),
    "bl_update_select": (_c.c_int, [_c.c_int]),
    "bl_update_fixed_scratch_capacity": (_c.c_size_t, []),
    "bl_nvfp4_lattice_update_fixed_scratch": (_c.c_int, [_P, _P, _P, _P, _P, _c.c_int, _c.c_int64, _c.c_int64,
                                                         _c.c_uint64, _c.c_int, _c.c_int, _c.c_double, _c.c_double,
                                                         _c.c_int, _c.c_uint32, _c.c_uint32, _c.c_int, _c.c_int,
                                                         _c.c_int, _c.c_double, _c.c_int, _c.c_double, _c.c_int, _P]),
    "bl_direction": (_c.c_int, [_P, _c.c_int, _c.c_int64, _c.c_int64, _c.c_int, _c.c_double, _P, _P, _c.c_size_t,
                                _c.c_int, _P]),
    "bl_nvfp4_dequantize": (_c.c_int, [_P, _P, _P, _c.c_int64, _c.c_int64, _P, _c.c_int, _c.c_int, _P]),
    "bl_nvfp4_amax": (_c.c_int, [_P, _c.c_int, _c.c_int64, _P, _c.c_int, _P]),
    "bl_nvfp4_quantize": (_c.c_int, [_P, _c.c_int, _c.c_int64, _c.c_int64, _P, _c.c_int64, _c.c_uint32, _P, _P,
                                     _c.c_int, _c.c_int, _P]),
    "bl_nvfp4_amax_quantize": (_c.c_int, [_P, _c.c_int, _c.c_int64, _c.c_int64, _P, _c.c_int64, _c.c_uint32, _P, _P,
                                          _c.c_int, _c.c_int, _P]),
    "bl_nvfp4_quantize_4over6": (_c.c_int, [_P, _c.c_int, _c.c_int64, _c.c_int64, _P, _c.c_int, _P, _P, _c.c_int,
                                            _c.c_int, _P]),
    "bl_nvfp4_quantize_general": (_c.c_int, [_P, _c.c_int, _c.c_int64, _c.c_int64, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                             _c.c_int, _c.c_int64, _c.c_int64, _P, _c.c_int, _P, _P, _P, _P, _c.c_int,
                                             _P, _P, _P, _c.c_int, _P]),
    "bl_fp4_fold_scales": (_c.c_int, [_P, _c.c_int64, _c.c_int64, _P, _P, _c.c_int, _P, _P, _c.c_int, _P]),
    "bl_nvfp4_quantize_t": (_c.c_int, [_P, _c.c_int, _c.c_int64, _c.c_int64, _P, _c.c_int64, _c.c_uint32, _P, _P, _P,
                                       _P, _P, _c.c_int, _c.c_int, _P]),
    "bl_nvfp4_requantize_t": (_c.c_int, [_P, _P, _P, _c.c_int64, _c.c_int64, _P, _P, _P, _c.c_int, _c.c_int, _P]),
    "bl_blocked_scale_bytes": (_c.c_size_t, [_c.c_int64, _c.c_int64]),
    "bl_nvfp4_scales_to_blocked": (_c.c_int, [_P, _c.c_int64, _c.c_int64, _P, _c.c_int, _P]),
    "bl_nvfp4_assemble_gathered": (_c.c_int, [_P, _c.c_int64, _c.c_int, _c.c_int64, _c.c_int64, _c.c_int64, _c.c_int64,
                                              _c.c_int64, _c.c_int64, _P, _P, _P, _P, _c.c_int, _P]),
    "bl_nvfp4_gemm": (_c.c_int, [_P, _P, _P, _P, _P, _P, _c.c_int64, _c.c_int64, _c.c_int64, _P, _c.c_int,
                                 _c.c_int64, _c.c_int, _P]),
    "bl_nvfp4_gemm_accumulate": (_c.c_int, [_P, _P, _P, _P, _P, _P, _c.c_int64, _c.c_int64, _c.c_int64, _P, _c.c_int,
                                            _c.c_int64, _c.c_int, _P]),
    "bl_nvfp4_gemm_status": (_c.c_int, [_c.POINTER(_c.c_int), _c.c_int]),
    "bl_nvfp4_gemm_status_async": (_c.c_int, [_P, _c.c_int, _P]),
    "bl_selftest_bounded_wait": (_c.c_int, [_c.POINTER(_c.c_int), _c.POINTER(_c.c_int), _P, _c.c_int]),
    "bl_selftest_mma_peak": (_c.c_int, [_c.c_int, _c.c_int, _c.POINTER(_c.c_float), _c.POINTER(_c.c_double), _P,
                                        _c.c_int]),
    "bl_nvfp4_gemm_select": (_c.c_int, [_c.c_int]),
    "bl_swiglu_fwd": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int64, _c.c_int, _c.c_void_p]),
    "bl_swiglu_bwd": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int64,
                                  _c.c_int, _c.c_void_p]),
    "bl_selftest_division": (_c.c_int, [_c.c_uint64, _c.c_uint32, _c.POINTER(_c.c_uint64), _c.c_int]),
}

_lib = None


def exported_symbols() -> list[str]:
    """Names this binding expects the library to export (every function of the public header)."""
    return sorted(_SIGNATURES)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python bitlattice_b200/csrc/build.py` "
                              "(there is no fallback implementation)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def ptr(t: torch.Tensor | None):
    """Device address as a plain int (ctypes converts it for a void* parameter), None for an absent tensor."""
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_of(t: torch.Tensor):
    """The current CUDA stream of the tensor's device as a raw handle. These wrappers run a few hundred times per
    training step, so the handle comes from torch's raw query where it exists instead of a Stream object."""
    index = t.device.index
    if _raw_stream is not None and index is not None:
        return _raw_stream(index)
    return torch.cuda.current_stream(t.device).cuda_stream


def device_of(t: torch.Tensor) -> int:
    if not t.is_cuda:
        raise RuntimeError("bitlattice_b200 kernels need CUDA tensors (there is no CPU path)")
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def check(status: int) -> None:
    if status != 0:
        raise RuntimeError(lib().bl_last_error().decode("utf-8", "replace"))


# kernels each entry point launches (memsets not counted); the lattice update launches 3 when it needs column
# statistics, the transposed quantizer 2 without a scale bound
KERNELS_PER_CALL = {"bl_nvfp4_step_quantized": 1, "bl_nvfp4_lattice_update": 1, "bl_nvfp4_lattice_update_many": 0,
                    "bl_nvfp4_lattice_update_fixed_scratch": 1, "bl_direction": 1,
                    "bl_update_shard_stats": 0, "bl_nvfp4_lattice_update_shards": 0,
                    "bl_nvfp4_dequantize": 1, "bl_nvfp4_amax": 1, "bl_nvfp4_quantize": 1, "bl_nvfp4_quantize_t": 1,
                    "bl_nvfp4_quantize_4over6": 1, "bl_nvfp4_amax_quantize": 2, "bl_nvfp4_quantize_general": 2, "bl_fp4_fold_scales": 1,
                    "bl_nvfp4_requantize_t": 1, "bl_nvfp4_scales_to_blocked": 1, "bl_nvfp4_gemm": 1, "bl_nvfp4_gemm_accumulate": 1,
                    "bl_nvfp4_assemble_gathered": 1,
                    "bl_swiglu_fwd": 1, "bl_swiglu_bwd": 1}


class Counters:
    """Launch accounting for benchmarks: ``launches`` counts this library's kernels; with ``timed`` set to a set of
    entry-point names, every call of one of them is bracketed by CUDA events on its stream (``events[name]``)."""

    launches = 0
    timed: set | None = None
    events: dict = {}

    @classmethod
    def reset(cls, timed=None) -> None:
        cls.launches, cls.timed, cls.events = 0, (set(timed) if timed else None), {}

    @classmethod
    def elapsed_ms(cls, name: str) -> tuple[float, int]:
        """(total milliseconds, calls) of a timed entry point; synchronize the device first."""
        ev = cls.events.get(name, [])
        return sum(a.elapsed_time(b) for a, b in ev), len(ev)


def call(name: str, *args, extra_kernels: int = 0) -> None:
    fn = getattr(lib(), name)
    if Counters.timed is not None and name in Counters.timed:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        check(fn(*args))
        b.record()
        Counters.events.setdefault(name, []).append((a, b))
    else:
        check(fn(*args))
    Counters.launches += KERNELS_PER_CALL.get(name, 0) + extra_kernels
