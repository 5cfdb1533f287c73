"""GEMM back end of NVFP4 lattice linear layers on B200: operand quantization + the block-scaled FP4 GEMM.

Mirrors the NVIDIA-recipe part of the reference's ``bitlattice/backend.py`` (same names, argument meaning and tensor
layouts): round-to-nearest activations, stochastically rounded gradients, a 16-point Hadamard rotation of the
weight-gradient operands, the transposed weight re-quantized once per weight version for the input gradient, the layer
input saved as transposed NVFP4. Where the reference calls ``torch.ops.bitlattice.*`` quantizers and
``torch._scaled_mm`` (cuBLASLt), this module calls the kernels of ``libbitlattice_b200.so``; block scales are produced
directly in the GEMM's tiled layout and the per-tensor scales are applied in the GEMM epilogue.

Not built (the reference's other recipes): MS-EDEN / 128-point rotations, delayed scales, deferred
weight gradients, MXFP8. Asking for them raises.
"""
from __future__ import annotations

import itertools
import weakref
from collections import OrderedDict
from dataclasses import astuple, dataclass
from functools import cache
from typing import NamedTuple

import torch

from . import _ops
from . import formats as F
from .tensor import wait_for_update

__all__ = ["FP4_RECIPES", "Fp4Operand", "Fp4Recipe", "as_recipe", "clear_shared", "drop_cached", "fp4_backward", "fp4_dgrad", "fp4_wgrad",
           "fp4_forward_saving", "fp4_mm", "fp4_supported", "fp4_unfit", "is_nvfp4", "nvfp4_linear", "quantize_fp4",
           "rht_last", "set_sr_seed", "to_blocked", "weight_operand", "weight_t_operand"]


@dataclass(frozen=True)
class Fp4Recipe:
    """Quantization of the GEMM operands (reference: bitlattice/backend.py:57-121). Built: the default values (the
    NVIDIA NVFP4 training recipe) and ``activations='4over6'`` (four-over-six block scales for the forward input,
    criterion ``select``), everything else as in the NVIDIA recipe. The 128-point rotation, MS-EDEN gradients and
    delayed scales are not."""

    activations: str = "rtn"
    gradients: str = "sr"
    rotation: int = 16
    rotate_dgrad: bool = False
    backward_4over6: bool = False
    select: str = "mse"
    dgrad_weight: str = "requantize"
    dgrad_scale: str = "current"
    scale_source: str = "current"
    scale_margin: float = 2.0

    def __post_init__(self):
        if self.activations not in ("rtn", "4over6"):
            raise ValueError("activations must be 'rtn' or '4over6'")
        if self.select not in ("mse", "mae"):
            raise ValueError("select must be 'mse' or 'mae'")
        if astuple(self)[1:5] + astuple(self)[6:] != _NVIDIA[1:5] + _NVIDIA[6:]:
            raise ValueError("only the 'nvidia' and '4over6' FP4 recipes (stochastically rounded gradients, 16-point "
                             "rotation) are built; the quartet2 recipes (128-point rotation, MS-EDEN, cached or "
                             "delayed scales) are not")

    @property
    def legacy(self) -> bool:
        """True for the NVIDIA recipe."""
        return astuple(self) == _NVIDIA


_NVIDIA = ("rtn", "sr", 16, False, False, "mse", "requantize", "current", "current", 2.0)

FP4_RECIPES: dict[str, Fp4Recipe] = {"nvidia": Fp4Recipe(), "4over6": Fp4Recipe(activations="4over6")}


def as_recipe(r) -> Fp4Recipe:
    if isinstance(r, Fp4Recipe):
        return r
    if r not in FP4_RECIPES:
        raise ValueError(f"unknown FP4 recipe {r!r}; built: {sorted(FP4_RECIPES)}")
    return FP4_RECIPES[r]


def is_nvfp4(fmt) -> bool:
    """NVFP4 storage layout: E2M1 values, E4M3 scales per 16 elements, a per-tensor global scale."""
    sc = getattr(fmt, "scale", None)
    return (getattr(fmt, "kind", None) == "table" and fmt.bits == 4 and sc is not None and sc.group == 16
            and sc.dtype == "e4m3" and sc.global_scale and fmt.levels == F.get("nvfp4").levels)


@cache
def fp4_supported(device_index: int) -> bool:
    """tcgen05 block-scaled FP4 MMAs exist on compute capability 10.x (the kernels are built for sm_100a only)."""
    return torch.cuda.is_available() and torch.cuda.get_device_capability(device_index)[0] == 10


def fp4_unfit(w, device_index: int | None, backward: bool) -> str | None:
    """Why the lattice weight ``w`` cannot use the NVFP4 GEMMs (None: it can); reference: backend.py:191-207."""
    if not is_nvfp4(w.fmt):
        return f"format {w.fmt.name} is not NVFP4-layout"
    if getattr(w, "hi_idx", None) is not None:
        return "it keeps high-precision columns"
    if w.dim() != 2:
        return "the weight is not a matrix"
    if w.shape[1] % 32:
        return f"in_features {w.shape[1]} is not a multiple of 32"
    if w.shape[0] % (32 if backward else 16):
        return f"out_features {w.shape[0]} is not a multiple of {32 if backward else 16}"
    if device_index is None:
        return "the weight is not on a CUDA device"
    if not fp4_supported(device_index):
        return f"GPU {device_index} has no tcgen05 FP4 tensor cores (sm_100a)"
    return None


class Fp4Operand(NamedTuple):
    """A [rows, cols] matrix in NVFP4: packed E2M1 codes, E4M3 block scales along cols, fp32 global scale.
    ``blocked``: the scales are a flat uint8 buffer in the GEMM's 128x4-tiled layout."""

    packed: torch.Tensor
    scales: torch.Tensor
    global_scale: torch.Tensor
    blocked: bool = False
    rotate_seed: int = -1


_sr_counter = itertools.count(1)


def set_sr_seed(start: int) -> None:
    """Restart the process-wide counter the stochastic-rounding seeds come from (reference: backend.py:234). Ranks of
    an N-sharded layer call this with the same value so their draws agree."""
    global _sr_counter
    _sr_counter = itertools.count(int(start))


def _seed() -> int:
    return next(_sr_counter) & 0x7FFFFFFF


def to_blocked(s: torch.Tensor) -> torch.Tensor:
    """[rows, cols] block scales -> the 128x4-tiled layout of block-scaled GEMMs (reference: backend.py:179-188)."""
    return _ops.to_blocked(s.view(torch.uint8) if s.dtype != torch.uint8 else s)


def quantize_fp4(x2: torch.Tensor, stochastic: bool = False, blocked: bool = True) -> Fp4Operand:
    """NVFP4 quantization along the last dimension of a contiguous 2-D tensor: round to nearest, or stochastic rounding
    with a fresh seed per call (reference: backend.py:237-244). One amax pass, one quantization pass."""
    am = _ops.amax_global(x2)
    g = am[1:2]
    seed = _seed() if stochastic else -1
    packed, scales = _ops.quantize_nvfp4(x2, g, seed, 0, blocked=blocked)
    return Fp4Operand(packed, scales, g, blocked)


def _act_operand(x2: torch.Tensor, recipe: Fp4Recipe) -> Fp4Operand:
    """Forward operand of the activations under ``recipe`` (reference: backend.py `_act_operand`)."""
    if recipe.activations != "4over6":
        return quantize_fp4(x2)
    g = _ops.amax_global(x2)[3:4]
    packed, scales = _ops.quantize_nvfp4_4over6(x2, g, recipe.select, blocked=True)
    return Fp4Operand(packed, scales, g, True)


def fp4_mm(a: Fp4Operand, b: Fp4Operand, out_dtype: torch.dtype = torch.bfloat16,
           add_to: torch.Tensor | None = None) -> torch.Tensor:
    """A B^T for NVFP4 operands A [M, K], B [N, K] (K: multiple of 32), fp32 accumulation in tensor memory,
    ``out_dtype`` output, both per-tensor scales applied in the epilogue (reference: backend.py:280-290).
    ``add_to`` [M, N]: the product is added to it in the GEMM's epilogue (same bits as ``add_to + product``) and it is
    returned: how the input gradients of projections sharing an input are summed without a pass of their own."""
    sa = a.scales if a.blocked else to_blocked(a.scales)
    sb = b.scales if b.blocked else to_blocked(b.scales)
    ga, gb = a.global_scale, b.global_scale
    return _ops.nvfp4_gemm(a.packed, sa, ga if ga.dtype == torch.float32 else ga.float(), b.packed, sb,
                           gb if gb.dtype == torch.float32 else gb.float(), out_dtype, out=add_to,
                           accumulate=add_to is not None)


# per-weight operands, kept while the weight is unchanged (the role of the reference's backend.py:293-342)

class _WeightOperands:
    """Derived GEMM operands of weights (re-tiled scales, the re-quantized transpose), valid for one weight version
    (``_bl_version``, bumped by the optimizer), bounded by bytes with least-recently-used eviction. Weights are held
    weakly, so an entry never keeps a parameter alive and a recycled ``id`` is detected."""

    def __init__(self, limit_bytes: int):
        self.limit = limit_bytes
        self.used = 0
        self.entries: OrderedDict = OrderedDict()      # (id(weight), kind) -> (version, weakref, operand, bytes)

    def get(self, w, kind: str, make):
        key, version = (id(w), kind), getattr(w, "_bl_version", 0)
        entry = self.entries.get(key)
        if entry is not None:
            if entry[0] == version and entry[1]() is w:
                self.entries.move_to_end(key)
                return entry[2]
            self._remove(key)
        wait_for_update(w)                              # an update issued on another stream finishes before we read
        operand = make()
        nbytes = sum(t.numel() * t.element_size() for t in operand if isinstance(t, torch.Tensor))
        self.entries[key] = (version, weakref.ref(w), operand, nbytes)
        self.used += nbytes
        while self.used > self.limit and len(self.entries) > 1:
            self._remove(next(iter(self.entries)))
        return operand

    def _remove(self, key) -> None:
        self.used -= self.entries.pop(key)[3]

    def drop(self, w) -> None:
        for key in [k for k in self.entries if k[0] == id(w)]:
            self._remove(key)

    def clear(self) -> None:
        self.entries.clear()
        self.used = 0


OPERAND_CACHE_BYTES = 768 << 20
_OPERANDS = _WeightOperands(OPERAND_CACHE_BYTES)


def _cached(w, kind: str, make):
    return _OPERANDS.get(w, kind, make)


def drop_cached(w) -> None:
    """Forget the cached operands of ``w`` (the optimizer changed it: old versions are never used again)."""
    _OPERANDS.drop(w)


def weight_operand(w) -> Fp4Operand:
    """W [N, K] as a GEMM operand (scales re-tiled once per weight version)."""
    return _cached(w, "w", lambda: Fp4Operand(w.packed, to_blocked(w.scales), w.global_scale.float(), True))


def weight_t_operand(w) -> Fp4Operand:
    """W^T [K, N] re-quantized along N from the NVFP4 codes, for the input gradient (once per weight version)."""
    def make():
        packed, scales, g = _ops.requantize_nvfp4_t(w.packed, w.scales, w.global_scale, blocked=True)
        return Fp4Operand(packed, scales, g, True)
    return _cached(w, "wt", make)


@cache
def _hadamard16(device: torch.device, dtype: torch.dtype) -> torch.Tensor:
    """Orthogonal 16x16 matrix diag(s) H / 4 with the reference's fixed sign vector (backend.py:365-372; the signs
    are what torch.Generator().manual_seed(0x5EED) draws there)."""
    h = torch.ones(1, 1)
    for _ in range(4):
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    s = torch.tensor([1, -1, 1, -1, -1, 1, -1, 1, -1, -1, 1, 1, -1, -1, -1, 1], dtype=torch.float32)
    return (s[:, None] * h / 4.0).to(device, dtype)


def rht_last(x: torch.Tensor) -> torch.Tensor:
    """The 16-point rotation over consecutive blocks of the last dimension (dense; for checks)."""
    r, c = x.shape
    return (x.view(r, c // 16, 16) @ _hadamard16(x.device, x.dtype)).view(r, c)


def _pad_rows(x2: torch.Tensor, multiple: int) -> torch.Tensor:
    pad = (-x2.shape[0]) % multiple
    return torch.nn.functional.pad(x2, (0, 0, 0, pad)) if pad else x2


# one quantization per input shared by its consumers (q / k / v, gate / up); reference: backend.py:471-499

_SHARED: OrderedDict = OrderedDict()
_SHARED_MAX = 4


def _shared(x: torch.Tensor, recipe: Fp4Recipe, kind: str, make):
    key = (id(x), x._version, recipe, kind, tuple(x.shape))
    hit = _SHARED.get(key)
    if hit is not None and hit[0]() is x:
        _SHARED.move_to_end(key)
        return hit[1]
    val = make()
    _SHARED[key] = (weakref.ref(x, lambda _, k=key: _SHARED.pop(k, None)), val)
    while len(_SHARED) > _SHARED_MAX:
        _SHARED.popitem(last=False)
    return val


def clear_shared() -> None:
    _SHARED.clear()


def _input_operands(x: torch.Tensor, recipe: Fp4Recipe, row: bool = True):
    """Forward operand of x and its rotated transposed operand for the weight gradient (reference:
    backend.py:519-546, legacy branch): the global scale of x bounds the rotated one by a factor 4."""
    K = x.shape[-1]
    x2 = _pad_rows(x.reshape(-1, K), 32).contiguous()
    xq = _act_operand(x2, recipe)
    # |x H/4| <= 4 max|x| for the orthogonal 16 x 16 rotation: the row-wise per-tensor scale bounds the rotated one
    # (brought back to the 448 convention when the row operand used 256; reference: backend.py:541-544)
    bound = xq.global_scale * (4.0 * (256.0 / 448.0 if recipe.activations == "4over6" else 1.0))
    xt = Fp4Operand(*_ops.quantize_nvfp4_t(x2, _hadamard16(x2.device, torch.float32), -1, 0, bound, blocked=True), True)
    return (xq if row else None), xt


def nvfp4_linear(x: torch.Tensor, w, bias: torch.Tensor | None = None, recipe: Fp4Recipe = Fp4Recipe()
                 ) -> torch.Tensor:
    """y = Q(x) W^T (+ bias) with x quantized to NVFP4 on the fly; W must be an NVFP4 LatticeTensor."""
    K = x.shape[-1]
    M = x.numel() // K
    xq = _shared(x, recipe, "fwd", lambda: _act_operand(_pad_rows(x.reshape(-1, K), 16).contiguous(), recipe))
    y = fp4_mm(xq, weight_operand(w), x.dtype)[:M]
    if bias is not None:
        y += bias.to(y.dtype)
    return y.reshape(*x.shape[:-1], w.shape[0])


def fp4_forward_saving(x: torch.Tensor, w, bias, recipe: Fp4Recipe = Fp4Recipe()):
    """Forward of 'fp4_all': returns (y, saved), saved = x^T (rotated, NVFP4) for the weight gradient."""
    K = x.shape[-1]
    M = x.numel() // K
    xq, xt = _shared(x, recipe, "fwd+t", lambda: _input_operands(x, recipe))
    y = fp4_mm(xq, weight_operand(w), x.dtype)[:M]
    if bias is not None:
        y += bias.to(y.dtype)
    return y.reshape(*x.shape[:-1], w.shape[0]), xt


def fp4_dgrad(gy: torch.Tensor, w, recipe: Fp4Recipe = Fp4Recipe(), add_to: torch.Tensor | None = None):
    """gx = Q_sr(gy) Q(W^T)^T; also returns the padded 2-D gradient and its operand for fp4_wgrad. ``add_to``: the
    padded [Mp, K] buffer of an earlier projection's input gradient, to which this one is added in the epilogue (the
    padded buffer is then what is returned)."""
    N = gy.shape[-1]
    g2 = gy.reshape(-1, N)
    g2p = _pad_rows(g2, 32).contiguous()
    gq = quantize_fp4(g2p, stochastic=True)
    if add_to is not None:
        return fp4_mm(gq, weight_t_operand(w), gy.dtype, add_to=add_to), g2p, gq
    return fp4_mm(gq, weight_t_operand(w), gy.dtype)[:g2.shape[0]], g2p, gq


def fp4_wgrad(g2p: torch.Tensor, gq: Fp4Operand | None, xt: Fp4Operand, w, recipe: Fp4Recipe = Fp4Recipe()):
    """gw = Q_sr(rot(gy^T)) Q(rot(x^T))^T for the padded 2-D gradient ``g2p``; ``gq`` (its row operand, if the input
    gradient was computed) supplies the bound of the rotated operand's per-tensor scale."""
    seed = _seed()
    bound = gq.global_scale * 4.0 if gq is not None else None
    gt = Fp4Operand(*_ops.quantize_nvfp4_t(g2p, _hadamard16(g2p.device, torch.float32), seed, 0, bound,
                                           blocked=True), True)
    return fp4_mm(gt, xt, w.dtype)


def fp4_backward(gy: torch.Tensor, w, xt: Fp4Operand | None, need_x: bool, need_w: bool,
                 recipe: Fp4Recipe = Fp4Recipe()):
    """Input and weight gradients of y = x W^T on FP4 tensor cores (reference: backend.py:592-626):
    gx = Q_sr(gy) Q(W^T)^T, gw = Q_sr(rot(gy^T)) Q(rot(x^T))^T; the rotations cancel in the product."""
    gx = gw = gq = g2p = None
    if need_x:
        gx, g2p, gq = fp4_dgrad(gy, w, recipe)
    if need_w:
        if g2p is None:
            g2p = _pad_rows(gy.reshape(-1, gy.shape[-1]), 32).contiguous()
        gw = fp4_wgrad(g2p, gq, xt, w, recipe)
    return gx, gw
