"""GEMM back end of NVFP4 lattice linear layers on B200: operand quantization + the block-scaled FP4 GEMM.

Mirrors the NVFP4 part of the reference's ``bitlattice/backend.py`` (same names, argument meaning and tensor layouts).
The NVIDIA recipe: round-to-nearest activations, stochastically rounded gradients, a 16-point Hadamard rotation of the
weight-gradient operands, the transposed weight re-quantized once per weight version for the input gradient, the layer
input saved as transposed NVFP4. The quartet2 recipes: four-over-six activations, MS-EDEN (or stochastic) gradients,
a randomized 128-point rotation of the token axis of the weight-gradient GEMM and of the output-feature axis of the
input-gradient GEMM, the rotated W^T re-quantized per backward or cached per weight version (with a current or a
bounded per-tensor scale), and deferred weight gradients (operands with power-of-two per-tensor scales kept per
micro-batch, folded and multiplied in one GEMM). Where the reference calls ``torch.ops.bitlattice.*`` quantizers and
``torch._scaled_mm`` (cuBLASLt), this module calls the kernels of ``libbitlattice_b200.so``; block scales are produced
directly in the GEMM's tiled layout and the per-tensor scales are applied in the GEMM epilogue.

Not built: seeds mixed with a device epoch for CUDA-graph replay, MXFP8. Asking for them raises. The reference's one-read kernel for both layouts of an operand
(``nvfp4_quantize2``) is two calls of the general quantizer here: same results, one more read.
"""
from __future__ import annotations

import contextlib
import itertools
import os
import weakref
from collections import OrderedDict
from dataclasses import astuple, dataclass
from functools import cache
from typing import NamedTuple

import torch

from . import _ops
from . import formats as F
from .tensor import wait_for_update

__all__ = ["FP4_RECIPES", "Fp4Operand", "Fp4Recipe", "as_recipe", "clear_shared", "defer_wgrad", "drop_cached",
           "flush_wgrad", "fold_rounded", "fp4_backward", "fp4_dgrad", "fp4_wgrad", "fp4_forward_saving", "fp4_mm",
           "fp4_supported", "fp4_unfit", "is_nvfp4", "nvfp4_linear", "pending_wgrad", "quantize_fp4", "rht_last",
           "set_sr_seed", "to_blocked", "weight_operand", "weight_t_operand", "weight_t_rotated_operand"]


_CHOICES = {"activations": ("rtn", "4over6"), "gradients": ("sr", "eden"), "rotation": (16, 128),
            "select": ("mse", "mae"), "dgrad_weight": ("requantize", "cached"), "dgrad_scale": ("current", "bound"),
            "scale_source": ("current", "delayed")}


@dataclass(frozen=True)
class Fp4Recipe:
    """How the three GEMMs of a layer get their NVFP4 operands (field names, values and error messages are the
    reference's, bitlattice/backend.py:57-121).

    Forward: ``activations`` -- plain round to nearest, or '4over6' (every block picks the better of two block scales,
    judged by ``select``). Backward: ``gradients`` -- the output gradient stochastically rounded ('sr'), or MS-EDEN
    ('eden': nearest codes with block scales that are rounded stochastically so that the product stays unbiased;
    only with the 128-point rotation); ``backward_4over6`` extends the two-candidate block scales to the backward
    operands. ``rotation`` is the size of the randomized Hadamard block applied along the token axis of both
    weight-gradient operands; ``rotate_dgrad`` rotates the output-feature axis of both input-gradient operands the
    same way. With ``rotate_dgrad`` the rotated W^T is made anew in every backward ('requantize') or once per weight
    version ('cached'), its per-tensor scale then coming from a pass over the rotated weight ('current') or from the
    bound sqrt(128) * W.global_scale ('bound'). ``scale_source='delayed'`` takes the per-tensor scales of the rotated
    operands from the maximum the same layer saw one call earlier, times ``scale_margin``, which saves the amax pass
    (the first call is exact; later values beyond the range saturate)."""

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
        for name, allowed in _CHOICES.items():
            if getattr(self, name) not in allowed:
                raise ValueError(f"{name} must be {' or '.join(repr(v) if isinstance(v, str) else str(v) for v in allowed)}")
        if self.gradients == "eden" and self.rotation != 128:
            raise ValueError("MS-EDEN gradients need rotation=128")
        bound_ok = self.dgrad_weight == "cached" and self.rotate_dgrad and self.rotation == 128
        if self.dgrad_scale == "bound" and not bound_ok:
            raise ValueError("dgrad_scale='bound' needs cached weights and the 128-element dgrad rotation")
        if not self.scale_margin >= 1.0:
            raise ValueError("scale_margin must be >= 1")

    @property
    def legacy(self) -> bool:
        """True for the NVIDIA recipe."""
        return astuple(self) == _NVIDIA

    @property
    def packed_exchange(self) -> bool:
        """True when the operands are those of the NVIDIA recipe up to the forward activations' block scales: what the
        multi-GPU layers that exchange packed operands are written for."""
        return astuple(self)[1:5] + astuple(self)[6:] == _NVIDIA[1:5] + _NVIDIA[6:]

    @property
    def simple_backward(self) -> bool:
        """Backward operands of the NVIDIA recipe: stochastic rounding, 16-point rotation, single block scales."""
        return self.rotation == 16 and self.gradients == "sr" and not self.backward_4over6


_NVIDIA = ("rtn", "sr", 16, False, False, "mse", "requantize", "current", "current", 2.0)
_QUARTET2 = dict(activations="4over6", gradients="eden", rotation=128, rotate_dgrad=True)

FP4_RECIPES: dict[str, Fp4Recipe] = {"nvidia": Fp4Recipe(), "4over6": Fp4Recipe(activations="4over6")}
for _name, _extra in (("quartet2", {}), ("quartet2_4o6", dict(backward_4over6=True)),
                      ("quartet2_fast", dict(dgrad_weight="cached")),
                      ("quartet2_delayed", dict(dgrad_weight="cached", scale_source="delayed")),
                      ("quartet2_bound", dict(dgrad_weight="cached", dgrad_scale="bound"))):
    FP4_RECIPES[_name] = Fp4Recipe(**_QUARTET2, **_extra)


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
    seed = _seed() if stochastic else -1
    packed, scales, am = _ops.amax_quantize_nvfp4(x2, seed, 0, blocked=blocked)
    return Fp4Operand(packed, scales, am[1:2], blocked)


def _act_operand(x2: torch.Tensor, recipe: Fp4Recipe) -> Fp4Operand:
    """Forward operand of the activations under ``recipe`` (reference: backend.py `_act_operand`)."""
    if recipe.activations != "4over6":
        return quantize_fp4(x2)
    g = _ops.amax_global(x2)[3:4]
    packed, scales = _ops.quantize_nvfp4_4over6(x2, g, recipe.select, blocked=True)
    return Fp4Operand(packed, scales, g, True)


NVTX = bool(os.environ.get("BL_NVTX"))       # name the GEMMs and the update in profiler timelines (off by default)


@contextlib.contextmanager
def nvtx(name: str):
    """An NVTX range around a piece of the hot path when BL_NVTX is set in the environment (else nothing)."""
    if not NVTX:
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


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
        self.kinds: dict = {}                           # id(weight) -> kinds present (drop() without a scan)

    def get(self, w, kind: str, make):
        opt = getattr(w, "_bl_pending", None)
        if opt is not None:                             # an update held back by its optimizer goes out first (it
            opt._flush_pending()                        # bumps the version)
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
        self.kinds.setdefault(key[0], set()).add(kind)
        self.used += nbytes
        while self.used > self.limit and len(self.entries) > 1:
            self._remove(next(iter(self.entries)))
        return operand

    def _remove(self, key) -> None:
        self.used -= self.entries.pop(key)[3]
        kinds = self.kinds.get(key[0])
        if kinds is not None:
            kinds.discard(key[1])
            if not kinds:
                del self.kinds[key[0]]

    def drop(self, w) -> None:
        for kind in tuple(self.kinds.get(id(w), ())):
            self._remove((id(w), kind))

    def clear(self) -> None:
        self.entries.clear()
        self.kinds.clear()
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


def weight_t_rotated_operand(w, four_over_six: bool = False, seed: int | None = None,
                             scale_source: str = "current") -> Fp4Operand:
    """W^T [K, N] rotated along N (128-blocks) and re-quantized from the codes once per weight version (round to
    nearest); the rotation seed (``rotate_seed`` of the result) is fixed per version, or ``seed`` (then not cached).
    ``scale_source='bound'``: per-tensor scale sqrt(128) * W.global_scale instead of an amax pass over the rotated
    weight (reference: bitlattice/backend.py:345-362)."""
    if scale_source not in ("current", "bound"):
        raise ValueError("scale_source must be 'current' or 'bound'")

    def make(seed):
        # |W H_128| <= sqrt(128) * 6 * 448 * W.global_scale; block scales still use the current block maxima
        given = ((w.global_scale.float() * (128 ** 0.5) * (448.0 / 256.0 if four_over_six else 1.0)).reshape(1)
                 if scale_source == "bound" else None)
        return _q(None, mode="rtn", four_over_six=four_over_six, rotate_seed=seed, seed=0, w=w, given=given)
    if seed is not None:
        return make(seed)
    ver = getattr(w, "_bl_version", 0)
    seed = (id(w) * 2654435761 + ver * 40503 + 1) & 0x7FFFFFFF
    return _cached(w, ("wt128_4o6" if four_over_six else "wt128") + "_" + scale_source, lambda: make(seed))


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


def _pad_to(recipe: Fp4Recipe) -> int:
    return 128 if recipe.rotation == 128 else 32


def _q(x2: torch.Tensor | None, *, transpose: bool = False, mode: str = "rtn", four_over_six: bool = False,
       recipe: Fp4Recipe | None = None, rotate_seed: int = -1, seed: int = 0, w=None, pow2: bool = False,
       given: torch.Tensor | None = None, amax_out: torch.Tensor | None = None) -> Fp4Operand:
    """NVFP4 operand from the general quantizer: rows of x2 (or of x2^T), optionally rotated (128) with
    ``rotate_seed``; ``w``: an NVFP4 weight given by its codes (transposed re-quantization); ``pow2``: per-tensor scale
    rounded up to a power of two (reference: bitlattice/backend.py:398-416)."""
    select = recipe.select if recipe is not None else "mse"
    rot = rotate_seed >= 0
    if w is not None:
        wait_for_update(w)
        packed, scales, g = _ops.nvfp4_quantize_general(
            w.packed, transpose=True, mode=mode, four_over_six=four_over_six, select=select, rotate=rot, seed=seed,
            rotate_seed=rotate_seed if rot else -1, given=given, pow2=pow2, w_scales=w.scales,
            w_global=w.global_scale.float().reshape(1), blocked=True)
    else:
        packed, scales, g = _ops.nvfp4_quantize_general(
            x2, transpose=transpose, mode=mode, four_over_six=four_over_six, select=select, rotate=rot, seed=seed,
            rotate_seed=rotate_seed if rot else -1, given=given, pow2=pow2, blocked=True, amax_out=amax_out)
    return Fp4Operand(packed, scales, g, True, rotate_seed)


def _site(w, role: str) -> dict:
    """Per-weight state of an operand site (delayed scales): the amax its row and column operands saw last."""
    sites = w.__dict__.setdefault("_bl_sites", {})
    return sites.setdefault(role, {})


def _q2(x2: torch.Tensor, row: dict | None, col: dict | None, recipe: Fp4Recipe, site: dict | None = None):
    """Row and column (x2^T) operands of x2; ``row`` / ``col``: keyword arguments of ``_q`` for that side, or None.

    Delayed scales (``scale_source='delayed'``, reference: bitlattice/backend.py:419-443): ``site`` remembers, per
    side, the largest magnitude the quantizer saw in the previous call. Once every side asked for has such a record,
    its per-tensor scale is record * margin / (6 * top) -- rounded up to a power of two where the side wants one --
    and no amax pass runs; until then the call is exact. Every call leaves its own maxima in the record. (The
    reference makes both layouts in one kernel from one read; here the general quantizer runs once per side.)"""
    sides = (row, col)
    delayed = recipe.scale_source == "delayed" and site is not None
    scale = [None, None]
    seen = None
    if delayed:
        record, have = site.get("amax"), site.get("known", (False, False))
        if record is not None and all(have[i] for i, kw in enumerate(sides) if kw is not None):
            for i, kw in enumerate(sides):
                if kw is None:
                    continue
                top = 256.0 if kw.get("four_over_six") else 448.0
                g = (record[i:i + 1] * (recipe.scale_margin / (6.0 * top))).clamp_min(1e-30)    # stays on the device
                scale[i] = torch.exp2(torch.ceil(torch.log2(g))) if kw.get("pow2") else g
        seen = torch.zeros(2, dtype=torch.float32, device=x2.device)
    out = [None, None]
    for i, kw in enumerate(sides):
        if kw is not None:
            out[i] = _q(x2, transpose=i == 1, recipe=recipe, given=scale[i],
                        amax_out=None if seen is None else seen[i:i + 1], **kw)
    if delayed:
        record, have = site.get("amax"), site.get("known", (False, False))
        if record is not None and None in sides:                # a side that did not run keeps its old maximum
            seen = torch.cat([(seen if kw is not None else record)[i:i + 1] for i, kw in enumerate(sides)])
        site["amax"] = seen
        site["known"] = tuple(h or kw is not None for h, kw in zip(have, sides))
    return out[0], out[1]


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


def _input_operands(x: torch.Tensor, recipe: Fp4Recipe, row: bool = True, site: dict | None = None):
    """Forward operand of x (None with ``row=False``) and its rotated transposed operand for the weight gradient
    (reference: bitlattice/backend.py:519-557)."""
    K = x.shape[-1]
    x2 = _pad_rows(x.reshape(-1, K), _pad_to(recipe)).contiguous()
    if recipe.rotation == 16:
        xq = _act_operand(x2, recipe)
        # |x H/4| <= 4 max|x| for the orthogonal 16 x 16 rotation: the row-wise per-tensor scale bounds the rotated
        # one (brought back to the 448 convention when the row operand used 256; reference: backend.py:541-544)
        bound = xq.global_scale * (4.0 * (256.0 / 448.0 if recipe.activations == "4over6" else 1.0))
        xt = Fp4Operand(*_ops.quantize_nvfp4_t(x2, _hadamard16(x2.device, torch.float32), -1, 0, bound, blocked=True),
                        True)
        return (xq if row else None), xt
    mode = "eden" if recipe.gradients == "eden" else "rtn"
    fos = recipe.backward_4over6 or (mode == "rtn" and recipe.activations == "4over6")
    rseed, seed = _seed(), _seed()
    # the weight-gradient operands get power-of-two per-tensor scales: micro-batches can then be concatenated exactly
    # into one GEMM (deferred weight gradients)
    col = dict(mode=mode, four_over_six=fos, rotate_seed=rseed, seed=seed, pow2=True)
    if K % 128 == 0:
        return _q2(x2, dict(four_over_six=recipe.activations == "4over6") if row else None, col, recipe, site)
    xt = _q(x2, transpose=True, recipe=recipe, **col)
    return (_act_operand(x2, recipe) if row else None), xt


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
    xq, xt = _shared(x, recipe, "fwd+t", lambda: _input_operands(x, recipe, site=_site(w, "x")))
    with nvtx("bl.fwd_gemm"):
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
    with nvtx("bl.dgrad_gemm"):
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
    with nvtx("bl.wgrad_gemm"):
        return fp4_mm(gt, xt, w.dtype)


def _rotated_weight_t(w, recipe: Fp4Recipe, mode: str, seed: int | None) -> Fp4Operand:
    """The W^T operand of a rotated input-gradient GEMM: the per-version cache ('cached' recipes, ``seed`` None), or
    a fresh quantization with the rotation ``seed`` -- MS-EDEN when the gradient is (both factors unbiased), else
    round to nearest."""
    if seed is None:
        return weight_t_rotated_operand(w, recipe.backward_4over6, scale_source=recipe.dgrad_scale)
    return _q(None, mode="eden" if mode == "eden" else "rtn", four_over_six=recipe.backward_4over6, recipe=recipe,
              rotate_seed=seed, seed=_seed(), w=w)


def fp4_backward(gy: torch.Tensor, w, xt: Fp4Operand | None, need_x: bool, need_w: bool,
                 recipe: Fp4Recipe = Fp4Recipe(), *, wt: Fp4Operand | None = None, keep: list | None = None):
    """Input and weight gradients of y = x W^T on FP4 tensor cores (reference: bitlattice/backend.py:560-634).

    NVIDIA-recipe operands: gx = Q_sr(gy) Q(W^T)^T and gw = Q_sr(rot16(gy^T)) Q(rot16(x^T))^T. The 128-rotation
    recipes quantize the output gradient twice as well: along N, rotated with the signs of the W^T operand it meets,
    and along the tokens, rotated with the signs of the saved x^T; each rotation cancels in its product. Layers whose
    N is not a multiple of 128 cannot rotate along N and fall back to the unrotated input-gradient operands.

    ``wt``: the rotated W^T operand to use instead of the per-version cache; ``keep``: a list that receives the
    weight-gradient operands (g^T, x^T) instead of their product. Both need a recipe with cached rotated weights and
    N in multiples of 128."""
    N = gy.shape[-1]
    rotated_dgrad = recipe.rotation == 128 and recipe.rotate_dgrad and N % 128 == 0
    if wt is not None or keep is not None:
        if not (rotated_dgrad and recipe.dgrad_weight == "cached" and (xt is None or xt.rotate_seed >= 0)):
            raise RuntimeError("explicit W^T / kept operands need a 'quartet2_fast'-like recipe and output features "
                               "in multiples of 128")
    if recipe.simple_backward and not _defer_wgrad[0]:
        gx = gw = gq = g2p = None
        if need_x:
            gx, g2p, gq = fp4_dgrad(gy, w, recipe)
        if need_w:
            if g2p is None:
                g2p = _pad_rows(gy.reshape(-1, N), 32).contiguous()
            gw = fp4_wgrad(g2p, gq, xt, w, recipe)
        return gx, gw

    g2 = gy.reshape(-1, N)
    M = g2.shape[0]
    g2p = _pad_rows(g2, _pad_to(recipe)).contiguous()
    fos = recipe.backward_4over6
    mode = "eden" if recipe.gradients == "eden" else "sr"
    rotated_wgrad = need_w and xt.rotate_seed >= 0
    gx = gw = rows = cols = None

    # ---- the operands of the output gradient
    both_rotated = N % 128 == 0 and (rotated_wgrad or not need_w) and (rotated_dgrad or not need_x)
    if need_x and rotated_dgrad:
        cached = recipe.dgrad_weight == "cached"
        if wt is None and cached:
            wt = _rotated_weight_t(w, recipe, mode, None)
        r = wt.rotate_seed if wt is not None else _seed()
        rows = dict(mode=mode, four_over_six=fos, rotate_seed=r, seed=_seed())
    if rotated_wgrad:
        cols = dict(mode=mode, four_over_six=fos, rotate_seed=xt.rotate_seed, seed=_seed(), pow2=True)
    if both_rotated:                   # one site for both layouts of gy (delayed scales live there)
        gq, gt = _q2(g2p, rows, cols, recipe, _site(w, "g"))
    else:
        gq = _q(g2p, recipe=recipe, **rows) if rows is not None else None
        gt = _q(g2p, transpose=True, recipe=recipe, **cols) if cols is not None else None

    # ---- input gradient
    if need_x:
        if rotated_dgrad:
            if wt is None:
                wt = _rotated_weight_t(w, recipe, mode, rows["rotate_seed"])
            gx = fp4_mm(gq, wt, gy.dtype)[:M]
            gq = None                                  # rotated: its per-tensor scale says nothing about g^T
        else:
            gq = (_q(g2p, mode="sr", four_over_six=True, recipe=recipe, seed=_seed()) if fos
                  else quantize_fp4(g2p, stochastic=True))
            gx = fp4_mm(gq, weight_t_operand(w), gy.dtype)[:M]

    # ---- weight gradient
    if need_w:
        if not rotated_wgrad:          # the saved x^T carries the 16-point rotation: so must g^T
            if _defer_wgrad[0]:
                name = getattr(w, "_bl_name", None) or f"weight {tuple(w.shape)}"
                raise RuntimeError(f"{name}: deferred weight gradients need a recipe with the 128-element rotation "
                                   "(e.g. 'quartet2_fast'); this layer's recipe rotates by 16 and its weight-gradient "
                                   "operands cannot be folded")
            bound = gq.global_scale * (4.0 * (256.0 / 448.0 if fos else 1.0)) if gq is not None else None
            gt = Fp4Operand(*_ops.quantize_nvfp4_t(g2p, _hadamard16(g2p.device, torch.float32), _seed(), 0, bound,
                                                   blocked=True), True)
            return gx, fp4_mm(gt, xt, w.dtype)
        if keep is not None:
            keep.append((gt, xt))
        else:
            gw = _weight_grad(w, gt, xt)
    return gx, gw


# ---- deferred weight gradients (the role of bitlattice/backend.py:637-746)
# Under gradient accumulation every micro-batch's backward would run its own weight-gradient GEMM and add a full-size
# result into .grad. Inside ``defer_wgrad()`` the 128-rotation recipes only remember the quantized operand pairs
# (g^T, x^T); their per-tensor scales are powers of two by construction, so ``flush_wgrad`` can bring the pieces to the
# largest scale by shifting the exponents of their block scales (exact unless a block scale leaves E4M3's normal
# range; those are counted), lay the micro-batches side by side along the token axis and multiply once.

_defer_wgrad = [0]                               # nesting depth of defer_wgrad()
_PENDING: OrderedDict = OrderedDict()            # id(parameter) -> (weak reference, list of operand pairs)
_FOLD_ROUNDED: dict = {}                         # device -> int64 [1]: block scales that were rounded while folding
_PIECES: dict = {}                               # (tile counts of the pieces, device) -> int32 piece of every column tile


@contextlib.contextmanager
def defer_wgrad():
    """While active, FP4 layers of the 128-rotation recipes keep their weight-gradient operands for ``flush_wgrad``
    instead of multiplying them."""
    _defer_wgrad[0] += 1
    try:
        yield
    finally:
        _defer_wgrad[0] -= 1


def _weight_grad(w, gt: Fp4Operand, xt: Fp4Operand):
    """g^T x now, or -- deferred -- nothing yet."""
    if _defer_wgrad[0] == 0:
        return fp4_mm(gt, xt, w.dtype)
    held = _PENDING.get(id(w))
    if held is None or held[0]() is not w:
        held = _PENDING[id(w)] = (weakref.ref(w), [])
    held[1].append((gt, xt))
    return None


def _concat(ops: list) -> Fp4Operand:
    """One operand [rows, K_1 + ... + K_n] from operands [rows, K_j] whose per-tensor scales are powers of two and
    whose block scales are tiled: the largest per-tensor scale serves all, the block scales of the others are
    multiplied by their 2^-k in place (``bl_fp4_fold_scales``)."""
    if len(ops) == 1:
        return ops[0]
    rows = ops[0].packed.shape[0]
    row_tiles = (rows + 127) // 128
    dev = ops[0].packed.device
    tiled = [o.scales.view(torch.uint8).view(row_tiles, -1, 512) for o in ops]
    widths = tuple(t.shape[1] for t in tiled)
    piece = _PIECES.get((widths, dev))
    if piece is None:
        piece = _PIECES[(widths, dev)] = torch.repeat_interleave(
            torch.arange(len(widths), dtype=torch.int32), torch.tensor(widths)).to(dev)
    counter = _FOLD_ROUNDED.get(dev)
    if counter is None:
        counter = _FOLD_ROUNDED[dev] = torch.zeros(1, dtype=torch.int64, device=dev)
    scales = torch.cat(tiled, 1).contiguous()
    g_all = torch.cat([o.global_scale.reshape(1).float() for o in ops])
    g_max = _ops.fp4_fold_scales(scales.view(-1), row_tiles, piece, g_all, counter)
    return Fp4Operand(torch.cat([o.packed for o in ops], 1), scales.view(-1), g_max, True)


def fold_rounded(reset: bool = False) -> int:
    """How many block scales had to be rounded so far when deferred operands of unequal magnitude were folded (0: every
    deferred gradient was exactly the product of its operands). Reads device counters: synchronizes."""
    total = sum(int(c.item()) for c in _FOLD_ROUNDED.values())
    if reset:
        for c in _FOLD_ROUNDED.values():
            c.zero_()
    return total


def pending_wgrad() -> list:
    """The parameters whose weight gradients are waiting in ``flush_wgrad``'s queue."""
    alive = (ref() for ref, _ in _PENDING.values())
    return [p for p in alive if p is not None]


def flush_wgrad(params=None, optimizer=None) -> int:
    """One weight-gradient GEMM per parameter over everything deferred for it (all parameters, or ``params``), added
    to ``.grad``; a ``fused_backward`` optimizer then updates the parameter right away. Returns how many parameters
    received a gradient."""
    wanted = list(_PENDING) if params is None else [id(p) for p in params if id(p) in _PENDING]
    done = 0
    for key in wanted:
        ref, pairs = _PENDING.pop(key)
        p = ref()
        if p is None or not pairs:
            continue
        gw = fp4_mm(_concat([g for g, _ in pairs]), _concat([x for _, x in pairs]), p.dtype)
        pairs.clear()
        if p.grad is None:
            p.grad = gw
        else:
            p.grad.add_(gw)
        if getattr(optimizer, "fused_backward", False):
            optimizer._on_grad(p)
        done += 1
    return done
