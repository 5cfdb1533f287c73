"""TEST INFRASTRUCTURE: numpy/ctypes front end of the CPU oracle in ``bl_oracle.c``.

The oracle restates the reference's pure-PyTorch arithmetic for the NVFP4 linear layer and the lattice update
(``bitlattice/reference.py``, ``bitlattice/fp4ref.py``, ``bitlattice/backend.py``; the C file cites line ranges per
function). It is the checker of the CUDA path and the timed CPU baseline, never a code path of the product: nothing
under ``bitlattice_b200/`` imports it.

All arrays are C-contiguous numpy arrays: fp32 values, uint8 code / scale / phase bytes.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libbl_oracle.so")
_lib = None

ROUNDING = {"sr": 0, "strat": 1, "rtn": 2}
RULE = {"fixed": 0, "fit": 1, "fit_latent": 2}
DIRECTION = {"raw": 0, "sign": 1, "colnorm": 2}
PANEL_ROWS = 128


def build(force: bool = False) -> str:
    """Compile ``bl_oracle.c`` (gcc, OpenMP when available) into ``oracle/_build``; returns the library path."""
    src = os.path.join(_HERE, "bl_oracle.c")
    if not force and os.path.exists(_LIB_PATH) and os.path.getmtime(_LIB_PATH) >= os.path.getmtime(src):
        return _LIB_PATH
    os.makedirs(os.path.dirname(_LIB_PATH), exist_ok=True)
    base = ["gcc", "-O2", "-fPIC", "-shared", "-std=c11", "-ffp-contract=off", "-fno-fast-math",
            "-fvisibility=hidden", "-o", _LIB_PATH, src, "-lm"]
    try:
        subprocess.run(base[:1] + ["-fopenmp"] + base[1:], check=True, capture_output=True)
    except (subprocess.CalledProcessError, FileNotFoundError):
        subprocess.run(base, check=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        L = ctypes.CDLL(build())
        c = ctypes
        u8p, f32p, u16p = c.POINTER(c.c_uint8), c.POINTER(c.c_float), c.POINTER(c.c_uint16)
        L.blo_hash_uniform.restype = c.c_float
        L.blo_hash_uniform.argtypes = [c.c_uint64, c.c_uint32, c.c_uint32]
        L.blo_rounding_u.restype = c.c_float
        L.blo_rounding_u.argtypes = [c.c_uint64, c.c_int, c.c_uint32, c.c_uint32, c.c_int, c.c_int]
        L.blo_e4m3_decode.restype = c.c_float
        L.blo_e4m3_decode.argtypes = [c.c_uint8]
        L.blo_e4m3_encode.restype = c.c_uint8
        L.blo_e4m3_encode.argtypes = [c.c_float]
        L.blo_amax.argtypes = [f32p, c.c_int64, f32p]
        L.blo_global_from_amax.restype = c.c_float
        L.blo_global_from_amax.argtypes = [c.c_float]
        L.blo_global_from_bound.restype = c.c_float
        L.blo_global_from_bound.argtypes = [c.c_float]
        L.blo_quantize_rows.argtypes = [f32p, c.c_int64, c.c_int64, c.c_float, c.c_int, c.c_uint32, c.c_uint32, u8p,
                                        u8p]
        L.blo_global_fos.argtypes = [c.c_float]
        L.blo_global_fos.restype = c.c_float
        L.blo_quantize_rows_fos.argtypes = [f32p, c.c_int64, c.c_int64, c.c_float, c.c_int, u8p, u8p]
        L.blo_quantize_t.argtypes = [f32p, c.c_int64, c.c_int64, f32p, c.c_float, c.c_int, c.c_uint32, c.c_uint32,
                                     u8p, u8p]
        L.blo_requantize_t.argtypes = [u8p, u8p, c.c_float, c.c_int64, c.c_int64, u8p, u8p]
        L.blo_dequantize.argtypes = [u8p, u8p, c.c_float, c.c_int64, c.c_int64, c.c_int, f32p]
        L.blo_to_blocked.argtypes = [u8p, c.c_int64, c.c_int64, u8p]
        L.blo_direction.argtypes = [f32p, c.c_int64, c.c_int64, c.c_int, c.c_float, f32p, f32p]
        L.blo_lattice_step.argtypes = [u8p, u8p, u8p, u8p, c.c_float, f32p, c.c_int64, c.c_int64, c.c_uint64, c.c_int,
                                       c.c_int, c.c_float, c.c_float, c.c_int, c.c_uint32, c.c_uint32, c.c_int,
                                       c.c_int, c.c_int, c.c_double]
        L.blo_gemm_nt.argtypes = [u8p, u8p, c.c_float, u8p, u8p, c.c_float, c.c_int64, c.c_int64, c.c_int64, f32p]
        L.blo_gemm_bf16_nt.argtypes = [u16p, u16p, c.c_int64, c.c_int64, c.c_int64, f32p]
        L.blo_num_threads.restype = c.c_int
        L.blo_set_num_threads.argtypes = [c.c_int]
        _lib = L
    return _lib


def _p(a: np.ndarray, ct):
    return a.ctypes.data_as(ctypes.POINTER(ct)) if a is not None else None


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint8)


def num_threads() -> int:
    return int(lib().blo_num_threads())


def set_num_threads(n: int) -> None:
    lib().blo_set_num_threads(int(n))


def hash_uniform(n: int, seed: int, step: int, offset: int = 0) -> np.ndarray:
    L = lib()
    return np.array([L.blo_hash_uniform(offset + i, seed & 0xFFFFFFFF, step & 0xFFFFFFFF) for i in range(n)],
                    dtype=np.float32)


def e4m3_encode(s) -> np.ndarray:
    L = lib()
    flat = _f32(s).reshape(-1)
    return np.array([L.blo_e4m3_encode(float(v)) for v in flat], dtype=np.uint8).reshape(np.shape(s))


def e4m3_decode(b) -> np.ndarray:
    L = lib()
    flat = _u8(b).reshape(-1)
    return np.array([L.blo_e4m3_decode(int(v)) for v in flat], dtype=np.float32).reshape(np.shape(b))


def amax(x) -> float:
    x = _f32(x)
    out = np.zeros(1, np.float32)
    lib().blo_amax(_p(x, ctypes.c_float), x.size, _p(out, ctypes.c_float))
    return float(out[0])


def global_from_amax(a: float) -> float:
    return float(lib().blo_global_from_amax(float(a)))


def global_from_bound(b: float) -> float:
    return float(lib().blo_global_from_bound(float(b)))


def quantize_rows(x, g: float | None = None, mode: str = "rtn", seed: int = 0, step: int = 0):
    """x [rows, cols] -> (codes [rows, cols/2], scale bytes [rows, cols/16], global). ``g`` None: from the amax."""
    x = _f32(x)
    rows, cols = x.shape
    if g is None:
        g = global_from_amax(amax(x))
    codes = np.empty((rows, cols // 2), np.uint8)
    scales = np.empty((rows, cols // 16), np.uint8)
    lib().blo_quantize_rows(_p(x, ctypes.c_float), rows, cols, np.float32(g), 0 if mode == "rtn" else 1,
                            seed & 0xFFFFFFFF, step & 0xFFFFFFFF, _p(codes, ctypes.c_uint8), _p(scales, ctypes.c_uint8))
    return codes, scales, np.float32(g)


def quantize_rows_fos(x, g: float | None = None, select: str = "mse"):
    """Four-over-six round-to-nearest quantizer of the forward activations (bitlattice/fp4ref.py:103-135 with
    four_over_six=True): x [rows, cols] -> (codes, scale bytes, global). ``g`` None: amax / (6 * 256)."""
    x = _f32(x)
    rows, cols = x.shape
    if g is None:
        g = lib().blo_global_fos(np.float32(amax(x)))
    codes = np.empty((rows, cols // 2), np.uint8)
    scales = np.empty((rows, cols // 16), np.uint8)
    lib().blo_quantize_rows_fos(_p(x, ctypes.c_float), rows, cols, np.float32(g), 1 if select == "mae" else 0,
                                _p(codes, ctypes.c_uint8), _p(scales, ctypes.c_uint8))
    return codes, scales, np.float32(g)


def quantize_t(x, H=None, g: float = 1.0, mode: str = "rtn", seed: int = 0, step: int = 0):
    """x [M, K] -> NVFP4 of x^T (optionally rotated along M): (codes [K, M/2], scale bytes [K, M/16])."""
    x = _f32(x)
    M, K = x.shape
    Hc = _f32(H) if H is not None else None
    codes = np.empty((K, M // 2), np.uint8)
    scales = np.empty((K, M // 16), np.uint8)
    lib().blo_quantize_t(_p(x, ctypes.c_float), M, K, _p(Hc, ctypes.c_float), np.float32(g),
                         0 if mode == "rtn" else 1, seed & 0xFFFFFFFF, step & 0xFFFFFFFF, _p(codes, ctypes.c_uint8),
                         _p(scales, ctypes.c_uint8))
    return codes, scales


def requantize_t(codes, scales, g: float):
    codes, scales = _u8(codes), _u8(scales)
    N, K = codes.shape[0], codes.shape[1] * 2
    oc = np.empty((K, N // 2), np.uint8)
    os_ = np.empty((K, N // 16), np.uint8)
    lib().blo_requantize_t(_p(codes, ctypes.c_uint8), _p(scales, ctypes.c_uint8), np.float32(g), N, K,
                           _p(oc, ctypes.c_uint8), _p(os_, ctypes.c_uint8))
    return oc, os_


def dequantize(codes, scales, g: float, order: int = 0) -> np.ndarray:
    codes, scales = _u8(codes), _u8(scales)
    rows, cols = codes.shape[0], codes.shape[1] * 2
    out = np.empty((rows, cols), np.float32)
    lib().blo_dequantize(_p(codes, ctypes.c_uint8), _p(scales, ctypes.c_uint8), np.float32(g), rows, cols, order,
                         _p(out, ctypes.c_float))
    return out


def to_blocked(scales) -> np.ndarray:
    scales = _u8(scales)
    rows, cols = scales.shape
    out = np.empty(((rows + 127) // 128) * ((cols + 3) // 4) * 512, np.uint8)
    lib().blo_to_blocked(_p(scales, ctypes.c_uint8), rows, cols, _p(out, ctypes.c_uint8))
    return out


def direction(G, kind: str, clip: float = 1.0):
    """fp32 direction D [rows, cols] and (rho, divisor) for 'raw', 'sign' or 'colnorm'."""
    G = _f32(G)
    rows, cols = G.shape
    D = np.empty_like(G)
    stats = np.zeros(2, np.float32)
    lib().blo_direction(_p(G, ctypes.c_float), rows, cols, DIRECTION[kind], np.float32(clip), _p(D, ctypes.c_float),
                        _p(stats, ctypes.c_float))
    return D, (float(stats[0]), float(stats[1]))


def hadamard16() -> np.ndarray:
    """diag(s) H / 4 with the reference's fixed sign vector (bitlattice/backend.py:365-372)."""
    h = np.ones((1, 1), np.float32)
    for _ in range(4):
        h = np.block([[h, h], [h, -h]])
    s = np.array([1, -1, 1, -1, -1, 1, -1, 1, -1, -1, 1, 1, -1, -1, -1, 1], np.float32)
    return (s[:, None] * h / 4.0).astype(np.float32)


def phase_container(bits: int) -> int:
    return 0 if bits == 0 else 1 if bits == 1 else 2 if bits == 2 else 4 if bits <= 4 else 8


def lattice_step(codes, phase, scales, g: float, D, *, lr: float, weight_decay: float = 0.0, phase_bits: int = 2,
                 rounding: str = "sr", seed: int = 0, step: int = 1, scale_rule: str = "fit", trust: float = 0.01,
                 trust_lr: float = 1.0, strata: int = 16, offset: int = 0):
    """One update; returns new (codes, phase, scale bytes). ``phase``: packed bytes [rows, cols*cb/8] or None."""
    codes = _u8(codes).copy()
    rows, cols = codes.shape[0], codes.shape[1] * 2
    pcb = phase_container(phase_bits)
    ph = _u8(phase).copy() if phase_bits else np.zeros(1, np.uint8)
    sc_in = _u8(scales)
    sc_out = np.empty_like(sc_in)
    D = _f32(D).reshape(rows, cols)
    if rounding == "strat":
        bits = max(1, (strata - 1).bit_length())
        k = 1 << bits
        v, j = step % k, 0
        for _ in range(bits):
            j = (j << 1) | (v & 1)
            v >>= 1
    else:
        j, k = 0, 1
    kappa = trust if trust_lr <= 0 else min(trust, trust_lr * lr)
    decay = np.float32(1.0 - lr * weight_decay)
    lib().blo_lattice_step(_p(codes, ctypes.c_uint8), _p(ph, ctypes.c_uint8), _p(sc_in, ctypes.c_uint8),
                           _p(sc_out, ctypes.c_uint8), np.float32(g), _p(D, ctypes.c_float), rows, cols, offset,
                           phase_bits, max(pcb, 1), np.float32(lr), decay, ROUNDING[rounding], seed & 0xFFFFFFFF,
                           step & 0xFFFFFFFF, j, k, RULE[scale_rule], float(kappa))
    return codes, (ph if phase_bits else None), sc_out


def gemm_nt(a_codes, a_scales, ga: float, b_codes, b_scales, gb: float) -> np.ndarray:
    a_codes, a_scales, b_codes, b_scales = _u8(a_codes), _u8(a_scales), _u8(b_codes), _u8(b_scales)
    M, K = a_codes.shape[0], a_codes.shape[1] * 2
    N = b_codes.shape[0]
    out = np.empty((M, N), np.float32)
    lib().blo_gemm_nt(_p(a_codes, ctypes.c_uint8), _p(a_scales, ctypes.c_uint8), np.float32(ga),
                      _p(b_codes, ctypes.c_uint8), _p(b_scales, ctypes.c_uint8), np.float32(gb), M, N, K,
                      _p(out, ctypes.c_float))
    return out


def gemm_bf16_nt(a_bits, b_bits) -> np.ndarray:
    """a [M, K], b [N, K] as uint16 bf16 bit patterns -> fp32 a @ b^T."""
    a = np.ascontiguousarray(a_bits, dtype=np.uint16)
    b = np.ascontiguousarray(b_bits, dtype=np.uint16)
    M, K = a.shape
    N = b.shape[0]
    out = np.empty((M, N), np.float32)
    lib().blo_gemm_bf16_nt(_p(a, ctypes.c_uint16), _p(b, ctypes.c_uint16), M, N, K, _p(out, ctypes.c_float))
    return out
