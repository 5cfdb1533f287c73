"""TEST INFRASTRUCTURE: numpy restatement of the reference's general NVFP4 quantizer (``bitlattice/fp4ref.py:103-150``:
round to nearest with ties to the even code, stochastic rounding, MS-EDEN, four-over-six block scales, the randomized
128-point Hadamard rotation; ``csrc/nvfp4.cu:553-600`` is the operator it twins) and of the scale folding of deferred
weight gradients (``bitlattice/backend.py:665-700``, ``csrc/fold.cu:12-33``).

The reference forms the rotation as a matrix product and its sums with torch reductions, whose summation order is
not defined; its own tests therefore allow 2e-3 of the codes and scales to differ between its kernel and fp4ref
(``tests/test_nvfp4.py:45-47``). This restatement pins one order, the one the CUDA kernels of this repository use, so
that kernel and oracle agree bit for bit, and is itself checked against fixtures written by ``fp4ref.quantize`` with
the reference's 2e-3 criterion:

  rotation   x * signs, then the fast Walsh-Hadamard butterflies with strides 1, 2, 4, ..., 64 (pairs (i, i + h) with
             bit h of i clear: a + b to i, a - b to i + h), then every element times fp32(1 / sqrt(128))
  4/6 error  per block of 16: four sequential sums over elements 4q .. 4q + 3 (ascending), then (s0 + s1) + (s2 + s3)
  MS-EDEN    <x, x> and <x, x_rtn> per 128: sequential sums over elements 4q .. 4q + 3, then a pairwise tree over the
             32 partial sums (neighbours first)
Everything is float32 arithmetic, one rounding per operation (no fused multiply-add).
"""
from __future__ import annotations

import numpy as np

F = np.float32
LEVELS = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
INV_SQRT128 = np.float32(0.08838834764831845)


# ---------------------------------------------------------------------------------------------- counter hash, E4M3

def hash_u(idx, seed: int, step: int) -> np.ndarray:
    """u in [0, 1) of bitlattice/reference.py:22-30 for an array of element indices (truncated to 32 bits)."""
    with np.errstate(over="ignore"):
        key = np.uint32((seed & 0xFFFFFFFF) * 0x9E3779B1 + (step & 0xFFFFFFFF) * 0x85EBCA77 & 0xFFFFFFFF)
        x = (np.asarray(idx).astype(np.uint64) & np.uint64(0xFFFFFFFF)).astype(np.uint32)
        x = x * np.uint32(0x27D4EB2F) + key
        x = (x ^ (x >> np.uint32(16))) * np.uint32(0x7FEB352D)
        x = (x ^ (x >> np.uint32(15))) * np.uint32(0x846CA68B)
        x = x ^ (x >> np.uint32(16))
    return (x >> np.uint32(8)).astype(np.float32) * np.float32(2.0 ** -24)


def _e4m3_table() -> np.ndarray:
    v = np.zeros(127, dtype=np.float64)
    for b in range(127):
        e, m = b >> 3, b & 7
        v[b] = (m / 8.0) * 2.0 ** -6 if e == 0 else (1.0 + m / 8.0) * 2.0 ** (e - 7)
    return v.astype(np.float32)


E4M3 = _e4m3_table()                       # value of code b, b = 0 .. 0x7E (448)


def e4m3_encode(v) -> np.ndarray:
    """clamp to [2^-9, 448], round to nearest even -> code byte (bitlattice/fp4ref.py:57-58)."""
    x = np.clip(np.asarray(v, dtype=np.float32), F(2.0 ** -9), F(448.0))
    hi = np.searchsorted(E4M3, x, side="left")                 # first code with value >= x
    hi = np.clip(hi, 1, 126)
    lo = hi - 1
    dlo = x.astype(np.float64) - E4M3[lo].astype(np.float64)
    dhi = E4M3[hi].astype(np.float64) - x.astype(np.float64)
    pick_hi = (dhi < dlo) | ((dhi == dlo) & ((hi & 1) == 0))
    return np.where(pick_hi, hi, lo).astype(np.uint8)


def e4m3_decode(b) -> np.ndarray:
    return E4M3[np.asarray(b, dtype=np.int64)]


def e4m3_sr(v, u) -> np.ndarray:
    """Stochastic rounding of positive values to E4M3 codes (bitlattice/fp4ref.py:81-88)."""
    v = np.clip(np.asarray(v, dtype=np.float32), F(2.0 ** -9), F(448.0))
    b = e4m3_encode(v).astype(np.int64)
    lo = E4M3[b]
    down = lo > v
    b = np.where(down, np.maximum(b - 1, 1), b)
    lo = E4M3[b]
    hb = np.minimum(b + 1, 0x7E)
    hi = E4M3[hb]
    with np.errstate(invalid="ignore", divide="ignore"):
        p = np.where(hi > lo, (v - lo) / np.where(hi > lo, hi - lo, F(1.0)), F(0.0)).astype(np.float32)
    return np.where(u < p, hb, b).astype(np.uint8)


# ---------------------------------------------------------------------------------------------- E2M1

def nearest_even(q) -> np.ndarray:
    """Code (sign in bit 3, never -0) of the E2M1 level nearest to q, ties to the even code, saturating
    (bitlattice/fp4ref.py:61-68)."""
    a = np.abs(q)
    mids = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]
    idx = np.zeros(q.shape, dtype=np.int64)
    for i, m in enumerate(mids):
        idx += (a >= F(m)) if i % 2 else (a > F(m))
    return (idx | np.where((q < 0) & (idx > 0), 8, 0)).astype(np.uint8)


def stochastic(q, u) -> np.ndarray:
    """Code of q rounded stochastically between its E2M1 neighbours (bitlattice/fp4ref.py:71-78)."""
    a = np.minimum(np.abs(q), F(6.0))
    lo_i = np.clip(np.searchsorted(LEVELS, a, side="right") - 1, 0, 7)
    lo, hi = LEVELS[lo_i], LEVELS[np.minimum(lo_i + 1, 7)]
    up = (lo_i < 7) & (u * (hi - lo) < a - lo)
    idx = lo_i + up
    return (idx | np.where((q < 0) & (idx > 0), 8, 0)).astype(np.uint8)


def level(codes) -> np.ndarray:
    c = np.asarray(codes, dtype=np.int64)
    return np.where(c & 8, -LEVELS[c & 7], LEVELS[c & 7]).astype(np.float32)


def pack(codes) -> np.ndarray:
    c = np.asarray(codes, dtype=np.uint8)
    return (c[..., 0::2] | (c[..., 1::2] << 4)).astype(np.uint8)


def unpack(packed, cols: int) -> np.ndarray:
    p = np.asarray(packed, dtype=np.uint8)
    out = np.empty(p.shape[:-1] + (cols,), dtype=np.uint8)
    out[..., 0::2] = p & 15
    out[..., 1::2] = p >> 4
    return out


# ---------------------------------------------------------------------------------------------- rotation

def signs128(rotate_seed: int) -> np.ndarray:
    """The +-1 vector of the rotation (bitlattice/fp4ref.py:31-34)."""
    u = hash_u(np.arange(128), rotate_seed, 0x5151)
    return np.where(u < F(0.5), F(-1.0), F(1.0)).astype(np.float32)


def fwht128(v) -> np.ndarray:
    """Butterflies with strides 1 .. 64 over the last axis (length 128), then the normalisation."""
    v = np.asarray(v, dtype=np.float32)
    lead = v.shape[:-1]
    h = 1
    while h < 128:
        w = v.reshape(lead + (128 // (2 * h), 2, h))
        a, b = w[..., 0, :], w[..., 1, :]
        v = np.stack([a + b, a - b], axis=-2).reshape(lead + (128,))
        h *= 2
    return (v * INV_SQRT128).astype(np.float32)


def rht128(x, rotate_seed: int) -> np.ndarray:
    x = np.asarray(x, dtype=np.float32)
    r, c = x.shape
    return fwht128(x.reshape(r, c // 128, 128) * signs128(rotate_seed)).reshape(r, c)


# ---------------------------------------------------------------------------------------------- the quantizer

def _tree(s) -> np.ndarray:
    """Pairwise sum over the last axis (a power of two), neighbours first."""
    while s.shape[-1] > 1:
        s = (s[..., 0::2] + s[..., 1::2]).astype(np.float32)
    return s[..., 0]


def _lane_sums(e) -> np.ndarray:
    """[..., n] -> [..., n / 4]: sequential sums over groups of four consecutive elements."""
    g = e.reshape(e.shape[:-1] + (e.shape[-1] // 4, 4))
    s = g[..., 0]
    for i in range(1, 4):
        s = (s + g[..., i]).astype(np.float32)
    return s


def pow2_up(g: np.float32) -> np.float32:
    b = np.array([g], dtype=np.float32).view(np.uint32)
    if b[0] & np.uint32(0x7FFFFF):
        b[0] = (b[0] & np.uint32(0x7F800000)) + np.uint32(0x00800000)
    return b.view(np.float32)[0]


def weight_values(codes, scales, g) -> np.ndarray:
    """Dense fp32 values of an NVFP4 matrix as the packed-input quantizer forms them: (level * block scale) * global
    (tests/test_nvfp4.py:96-99)."""
    rows, half = codes.shape
    lv = level(unpack(codes, half * 2)).reshape(rows, half // 8, 16)
    sc = e4m3_decode(scales).reshape(rows, half // 8, 1)
    return ((lv * sc).astype(np.float32) * F(g)).astype(np.float32).reshape(rows, half * 2)


def quantize(x, *, transpose: bool = False, mode: str = "rtn", four_over_six: bool = False, select: str = "mse",
             rotate: bool = False, seed: int = 0, rotate_seed: int | None = None, given=None, pow2: bool = False):
    """x [R, C] fp32 (already the dense values; see weight_values for NVFP4 input). Returns (codes [rows, cols] uint8,
    scale bytes [rows, cols / 16], global fp32) of x or x^T, blocks of 16 along the last dimension."""
    y = np.ascontiguousarray(np.asarray(x, dtype=np.float32).T if transpose else np.asarray(x, dtype=np.float32))
    rows, cols = y.shape
    if rotate:
        y = rht128(y, seed if rotate_seed is None else rotate_seed)
    top = F(1536.0) if four_over_six else F(2688.0)
    if given is not None:
        g = F(given)
    else:
        g = np.maximum(np.abs(y).max() / top, F(1e-12)).astype(np.float32)
        if pow2:
            g = pow2_up(g)
    b = y.reshape(rows, cols // 16, 16)
    amax = np.abs(b).max(-1)

    def candidate(div):
        sb = e4m3_encode(((amax / F(div)).astype(np.float32) / g).astype(np.float32))
        t = (e4m3_decode(sb) * g).astype(np.float32)
        with np.errstate(divide="ignore"):
            inv = np.where(t > 0, F(1.0) / np.where(t > 0, t, F(1.0)), F(0.0)).astype(np.float32)
        c = nearest_even((b * inv[..., None]).astype(np.float32))
        return sb, t, inv, c

    sb, t, inv, codes = candidate(6.0)
    if four_over_six:
        sb4, t4, inv4, c4 = candidate(4.0)

        def err(c, tt):
            e = ((level(c) * tt[..., None]).astype(np.float32) - b).astype(np.float32)
            e = np.abs(e) if select == "mae" else (e * e).astype(np.float32)
            s = _lane_sums(e)
            return ((s[..., 0] + s[..., 1]).astype(np.float32) + (s[..., 2] + s[..., 3]).astype(np.float32)).astype(np.float32)

        pick4 = err(c4, t4) < err(codes, t)
        sb = np.where(pick4, sb4, sb)
        t = np.where(pick4, t4, t)
        inv = np.where(pick4, inv4, inv)
        codes = np.where(pick4[..., None], c4, codes)
    if mode == "sr":
        u = hash_u(np.arange(rows * cols), seed, 0).reshape(rows, cols // 16, 16)
        codes = stochastic((b * inv[..., None]).astype(np.float32), u)
    elif mode == "eden":
        xr = (level(codes) * t[..., None]).astype(np.float32)
        bb = b.reshape(rows, cols // 128, 128)
        rr = xr.reshape(rows, cols // 128, 128)
        num = _tree(_lane_sums((bb * bb).astype(np.float32)))
        den = _tree(_lane_sums((bb * rr).astype(np.float32)))
        with np.errstate(divide="ignore", invalid="ignore"):
            S = np.where(den != 0, num / np.where(den != 0, den, F(1.0)), F(1.0)).astype(np.float32)
        S = np.repeat(S, 8, axis=-1)
        u = hash_u(np.arange(rows * (cols // 16)), seed ^ 0x9E3779B9, 0).reshape(rows, cols // 16)
        sb = e4m3_sr((e4m3_decode(sb) * S).astype(np.float32), u)
    elif mode != "rtn":
        raise ValueError(mode)
    return codes.reshape(rows, cols).astype(np.uint8), sb.astype(np.uint8), np.float32(g)


def dequantize(codes, sb, g) -> np.ndarray:
    rows, cols = codes.shape
    return (level(codes).reshape(rows, cols // 16, 16)
            * (e4m3_decode(sb) * F(g)).astype(np.float32)[..., None]).reshape(rows, cols)


# ---------------------------------------------------------------------------------------------- folding

def fold_scales(scale_bytes, f) -> tuple[np.ndarray, int]:
    """Block scales times a power of two f <= 1, rounded to E4M3 (round to nearest even, no clamp from below: values
    under the smallest subnormal's half become 0); also the number of non-zero products below E4M3's smallest normal
    2^-6 when f != 1 (bitlattice/backend.py:690-697)."""
    v = (e4m3_decode(scale_bytes) * F(f)).astype(np.float32)
    rounded = int(((v > 0) & (v < F(2.0 ** -6)) & (F(f) != 1)).sum())
    x = np.clip(v, F(0.0), F(448.0))
    hi = np.clip(np.searchsorted(E4M3, x, side="left"), 1, 126)
    lo = hi - 1
    dlo = x.astype(np.float64) - E4M3[lo].astype(np.float64)
    dhi = E4M3[hi].astype(np.float64) - x.astype(np.float64)
    pick_hi = (dhi < dlo) | ((dhi == dlo) & ((hi & 1) == 0))
    return np.where(pick_hi, hi, lo).astype(np.uint8), rounded
