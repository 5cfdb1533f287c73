"""Operator layer: the call sites of the reference's ``torch.ops.bitlattice.*`` operators (``bitlattice/_ops.py``,
schemas in the reference's ``csrc/bindings.cpp:75-134``) bound to the C ABI of ``libbitlattice_b200.so``.

Function names and argument meaning follow the reference so the layers above (tensor, backend, optimizer) read the
same; tensors are allocated here with torch and handed to the library as raw pointers on the current CUDA stream.
There is no CPU or PyTorch fallback: an input that is not a contiguous CUDA tensor of a supported shape raises.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _C
from . import formats as F

HAVE_EXT = True            # the library is mandatory; importing this package fails without it (see _C.lib)

_ROUNDING = {"sr": 0, "strat": 1, "rtn": 2}
_RULE = {"fixed": 0, "fit": 1, "fit_latent": 2}
_DIRECTION = {"raw": 0, "sign": 1, "colnorm": 2}


def _require(t: torch.Tensor, name: str, dtype=None) -> torch.Tensor:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (this build has no CPU path)")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"{name} must be {dtype}, got {t.dtype}")
    return t


def _bytes(t: torch.Tensor) -> torch.Tensor:
    return t if t.dtype == torch.uint8 else t.view(torch.uint8)


def _is_nvfp4(fmt) -> bool:
    fmt = F.get(fmt)
    sc = fmt.scale
    return fmt.kind == "table" and fmt.bits == 4 and sc.group == 16 and sc.dtype == "e4m3" and sc.global_scale


def cuda_ok(fmt, rows: int, cols: int, device) -> bool:
    """Whether the kernels take this tensor: NVFP4 on a CUDA device with rows made of 16-element groups."""
    return torch.device(device).type == "cuda" and _is_nvfp4(fmt) and cols % 16 == 0


def phase_container(phase_bits: int) -> int:
    return 0 if phase_bits == 0 else 1 if phase_bits == 1 else 2 if phase_bits == 2 else 4 if phase_bits <= 4 else 8


def phase_numel(n: int) -> int:
    return math.ceil(n / 8) * 8


def bitrev(v: int, bits: int) -> int:
    r = 0
    for _ in range(bits):
        r = (r << 1) | (v & 1)
        v >>= 1
    return r


def strat_args(rounding: str, step: int, strata: int) -> tuple[int, int]:
    if rounding != "strat":
        return 0, 1
    bits = max(1, (strata - 1).bit_length())
    k = 1 << bits
    return bitrev(step % k, bits), k


def kappa(trust: float, trust_lr: float, lr: float) -> float:
    return trust if trust_lr <= 0 else min(trust, trust_lr * lr)


# ------------------------------------------------------------------------------------------------ storage <-> dense

def dequantize(packed, scales, global_scale, zeros, fmt, rows: int, cols: int, dtype=torch.bfloat16):
    """Dense [rows, cols] tensor of the represented values (reference: bitlattice/_ops.py:55-61)."""
    if zeros is not None or not _is_nvfp4(fmt):
        raise RuntimeError("only NVFP4 tensors (no zero points) are built")
    _require(packed, "packed", torch.uint8)
    _require(scales, "scales")
    _require(global_scale, "global_scale", torch.float32)
    if dtype not in _C.DTYPE:
        raise RuntimeError(f"dequantize to {dtype} is not built (float32, bfloat16, float16 are)")
    out = torch.empty(rows, cols, dtype=dtype, device=packed.device)
    _C.call("bl_nvfp4_dequantize", _C.ptr(packed), _C.ptr(scales), _C.ptr(global_scale), rows, cols, _C.ptr(out),
            _C.DTYPE[dtype], _C.device_of(packed), _C.stream_of(packed))
    return out


# ------------------------------------------------------------------------------------------------ lattice update

def step_quantized(packed, phase, scales, global_scale, zeros, D, fmt, rows: int, cols: int, *, lr: float,
                   weight_decay: float, phase_bits: int, phase_cb: int, rounding: str, seed: int, step: int,
                   strata: int, scale_rule: str, trust: float, trust_lr: float, offset: int = 0,
                   inplace_scales: bool = False) -> torch.Tensor:
    """In-place update of ``packed`` (and ``phase``) given the fp32 direction ``D``; returns the new scales tensor
    (reference: bitlattice/_ops.py:76-86), or, with ``inplace_scales``, writes them into ``scales`` itself."""
    if zeros is not None or not _is_nvfp4(fmt):
        raise RuntimeError("only NVFP4 tensors (no zero points) are built")
    _require(packed, "packed", torch.uint8)
    _require(scales, "scales")
    _require(global_scale, "global_scale", torch.float32)
    Df = D.reshape(-1).float().contiguous()
    _require(Df, "D")
    if Df.numel() != rows * cols:
        raise RuntimeError("D: float32 [rows*cols]")
    if phase_bits > 0:
        _require(phase, "phase", torch.uint8)
    new_scales = scales if inplace_scales else torch.empty_like(scales)
    j, k = strat_args(rounding, step, strata)
    _C.call("bl_nvfp4_step_quantized", _C.ptr(packed), _C.ptr(phase) if phase_bits > 0 else None, _C.ptr(scales),
            _C.ptr(new_scales), _C.ptr(global_scale), _C.ptr(Df), rows, cols, int(offset) & 0xFFFFFFFFFFFFFFFF,
            phase_bits, phase_cb, float(lr), float(1.0 - lr * weight_decay), _ROUNDING[rounding],
            int(seed) & 0xFFFFFFFF, int(step) & 0xFFFFFFFF, j, k, _RULE[scale_rule],
            float(kappa(trust, trust_lr, lr)), _C.device_of(packed), _C.stream_of(packed))
    return new_scales


_scratch: dict = {}


def _scratch_for(device: torch.device, nbytes: int) -> torch.Tensor | None:
    """The scratch buffer (column statistics of the fused update) of the calling stream: one per (device, current
    stream), growing on demand. Kernels of one stream run in order, so they can share a buffer; callers on different
    streams of a device (two optimizers, a user stream beside autograd's) each get their own and never race on the
    statistics. A buffer that is outgrown is released to torch's allocator by the stream that used it, which only
    hands the memory out again behind that stream's work."""
    if nbytes == 0:
        return None
    key = (device, _C._raw_stream(device.index) if _C._raw_stream is not None and device.index is not None
           else torch.cuda.current_stream(device).cuda_stream)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        with torch.cuda.device(device):
            buf = _scratch[key] = torch.empty(nbytes, dtype=torch.uint8, device=device)
    return buf


def update_scratch_bytes(rows: int, cols: int, direction: str, clip: float) -> int:
    return int(_C.lib().bl_update_scratch_bytes(rows, cols, _DIRECTION[direction], float(clip)))


def lattice_update(packed, phase, scales, global_scale, zeros, G, fmt, rows: int, cols: int, *, lr: float,
                   weight_decay: float, phase_bits: int, phase_cb: int, rounding: str, seed: int, step: int,
                   strata: int, scale_rule: str, trust: float, trust_lr: float, direction: str, clip: float = 1.0,
                   offset: int = 0, scratch: torch.Tensor | None = None) -> None:
    """Direction + lattice step in one pass over the gradient ``G`` (bf16 / fp16 / fp32), everything in place,
    scales included (reference: torch.ops.bitlattice.lattice_update, csrc/update.cpp:30-53)."""
    if zeros is not None or not _is_nvfp4(fmt):
        raise RuntimeError("only NVFP4 tensors (no zero points) are built")
    if direction not in _DIRECTION:
        raise RuntimeError(f"direction {direction!r} is outside this build (raw, sign, colnorm are built)")
    _require(packed, "packed", torch.uint8)
    _require(scales, "scales")
    _require(global_scale, "global_scale", torch.float32)
    _require(G, "gradient")
    if G.dtype not in _C.DTYPE or G.numel() != rows * cols:
        raise RuntimeError("gradient: bf16, fp16 or fp32 with rows*cols elements")
    if phase_bits > 0:
        _require(phase, "phase", torch.uint8)
    need = update_scratch_bytes(rows, cols, direction, clip)
    if scratch is None:
        scratch = _scratch_for(packed.device, need)
    j, k = strat_args(rounding, step, strata)
    _C.call("bl_nvfp4_lattice_update", _C.ptr(packed), _C.ptr(phase) if phase_bits > 0 else None, _C.ptr(scales),
            _C.ptr(global_scale), _C.ptr(G), _C.DTYPE[G.dtype], rows, cols, int(offset) & 0xFFFFFFFFFFFFFFFF,
            phase_bits, phase_cb, float(lr), float(1.0 - lr * weight_decay), _ROUNDING[rounding],
            int(seed) & 0xFFFFFFFF, int(step) & 0xFFFFFFFF, j, k, _RULE[scale_rule],
            float(kappa(trust, trust_lr, lr)), _DIRECTION[direction], float(clip), _C.ptr(scratch),
            scratch.numel() if scratch is not None else 0, _C.device_of(packed), _C.stream_of(packed),
            extra_kernels=2 if need else 0)


def update_select(route: str = "auto") -> None:
    """Send every later lattice update of this process through the general route of the update kernel ("general") or
    hand the choice back ("auto": the fast route where it applies). Identical results; for tests and experiments."""
    _C.call("bl_update_select", {"auto": 0, "general": 1}[route])


def update_many_scratch_bytes(shapes, direction: str, clip: float) -> int:
    """Scratch with which ``lattice_update_many`` runs tensors of the given (rows, cols) in the fewest launches."""
    n = len(shapes)
    if n == 0:
        return 0
    rows = (ctypes.c_int64 * n)(*[int(r) for r, _ in shapes])
    cols = (ctypes.c_int64 * n)(*[int(c) for _, c in shapes])
    return int(_C.lib().bl_update_many_scratch_bytes(n, rows, cols, _DIRECTION[direction], float(clip)))


class UpdatePlan:
    """The per-tensor arguments of ``lattice_update_many`` that do not change from step to step (shapes, offsets,
    seeds, the weights' and the phase buffers' addresses), validated and marshalled once: a step then only fills in the
    gradients' addresses and the step counters. ``items`` as for ``lattice_update_many`` (``grad`` / ``step`` are read
    for validation only). The plan keeps the tensors alive; build a new one when a parameter's storage is replaced
    (``stale`` tells)."""

    def __init__(self, items, fmt, phase_bits: int):
        if not _is_nvfp4(fmt):
            raise RuntimeError("only NVFP4 tensors (no zero points) are built")
        n = self.n = len(items)
        self.phase_bits = phase_bits
        self.gdtype = items[0]["grad"].dtype
        for it in items:
            _require(it["packed"], "packed", torch.uint8)
            _require(it["scales"], "scales")
            _require(it["global_scale"], "global_scale", torch.float32)
            if phase_bits > 0:
                _require(it["phase"], "phase", torch.uint8)
        self.tensors = [(it["packed"], it["phase"] if phase_bits > 0 else None, it["scales"], it["global_scale"])
                        for it in items]
        self.numel = [int(it["rows"]) * int(it["cols"]) for it in items]
        self.shapes = [(int(it["rows"]), int(it["cols"])) for it in items]
        self.rows = (ctypes.c_int64 * n)(*[int(it["rows"]) for it in items])
        self.cols = (ctypes.c_int64 * n)(*[int(it["cols"]) for it in items])
        self.offset = (ctypes.c_uint64 * n)(*[int(it["offset"]) & 0xFFFFFFFFFFFFFFFF for it in items])
        self.seed = (ctypes.c_uint32 * n)(*[int(it["seed"]) & 0xFFFFFFFF for it in items])
        self.addr = [tuple(t.data_ptr() if t is not None else 0 for t in ts) for ts in self.tensors]
        col = lambda k: (ctypes.c_void_p * n)(*[a[k] or None for a in self.addr])
        self.packed, self.phase, self.scales, self.gs = col(0), (col(1) if phase_bits > 0 else None), col(2), col(3)
        self.grad = (ctypes.c_void_p * n)()
        self.step = (ctypes.c_uint32 * n)()
        self.strat_j = (ctypes.c_int * n)()
        self.device = items[0]["packed"]
        self.scratch_need: dict = {}

    def stale(self, tensors) -> bool:
        """True when one of ``tensors`` (per parameter: packed, phase or None, scales, global_scale) is not the
        storage the plan was built for."""
        return any(tuple(t.data_ptr() if t is not None else 0 for t in ts) != a for ts, a in zip(tensors, self.addr))

    def scratch_bytes(self, direction: str, clip: float) -> int:
        key = (direction, float(clip))
        need = self.scratch_need.get(key)
        if need is None:
            need = self.scratch_need[key] = update_many_scratch_bytes(self.shapes, direction, clip)
        return need


def lattice_update_many(items, fmt, *, lr: float, weight_decay: float, phase_bits: int, phase_cb: int, rounding: str,
                        strata: int, scale_rule: str, trust: float, trust_lr: float, direction: str, clip: float = 1.0,
                        scratch: torch.Tensor | None = None, plan: UpdatePlan | None = None, grads=None,
                        steps=None) -> None:
    """``lattice_update`` for many tensors of one parameter group in one library call: the library packs them into
    batches of up to 40 and runs each batch as one chain of launches (statistics, their reduction, the update), so
    small shards are not paced by launches. ``items``: dicts with packed, phase (or None), scales, global_scale, grad,
    rows, cols, offset, seed, step; all gradients of one dtype, everything on one device. With a ``plan``
    (:class:`UpdatePlan`) ``items`` is ignored and only ``grads`` (contiguous tensors of the plan's gradient dtype)
    and ``steps`` are read."""
    if direction not in _DIRECTION:
        raise RuntimeError(f"direction {direction!r} is outside this build (raw, sign, colnorm are built)")
    if plan is None:
        if len(items) == 0:
            return
        plan = UpdatePlan(items, fmt, phase_bits)
        grads = [it["grad"] for it in items]
        steps = [it["step"] for it in items]
    n = plan.n
    gdtype = plan.gdtype
    if gdtype not in _C.DTYPE:
        raise RuntimeError("gradient: bf16, fp16 or fp32 with rows*cols elements")
    grad, step, sj = plan.grad, plan.step, plan.strat_j
    strat_k = 1
    for i in range(n):
        G = grads[i]
        if G.dtype != gdtype or G.numel() != plan.numel[i] or not G.is_cuda or not G.is_contiguous():
            raise RuntimeError("gradient: a contiguous CUDA tensor of the group's dtype with rows*cols elements")
        grad[i] = G.data_ptr()
        step[i] = int(steps[i]) & 0xFFFFFFFF
        if rounding == "strat":
            sj[i], strat_k = strat_args(rounding, steps[i], strata)
    if rounding != "strat":
        strat_k = strat_args(rounding, steps[0], strata)[1]
    dev = plan.device
    if scratch is None:
        scratch = _scratch_for(dev.device, plan.scratch_bytes(direction, clip))
    launches = ctypes.c_int(0)
    _C.call("bl_nvfp4_lattice_update_many", n, plan.packed, plan.phase, plan.scales, plan.gs, grad, plan.rows,
            plan.cols, plan.offset, plan.seed, step, sj, _C.DTYPE[gdtype], phase_bits, phase_cb, float(lr),
            float(1.0 - lr * weight_decay), _ROUNDING[rounding], strat_k, _RULE[scale_rule],
            float(kappa(trust, trust_lr, lr)), _DIRECTION[direction], float(clip), _C.ptr(scratch),
            scratch.numel() if scratch is not None else 0, _C.device_of(dev), _C.stream_of(dev),
            ctypes.byref(launches))
    _C.Counters.launches += launches.value


def lattice_update_shards(items, fmt, world: int, rank: int, exchange, *, lr: float, weight_decay: float,
                          phase_bits: int, phase_cb: int, rounding: str, strata: int, scale_rule: str, trust: float,
                          trust_lr: float, direction: str, clip: float = 1.0, plan: UpdatePlan | None = None,
                          grads=None, steps=None) -> None:
    """The fused update of row shards whose direction normalises over the whole weight (colnorm; raw and sign with
    clip < 1): together the ``world`` owners of the shards reproduce the unsharded update bit for bit. ``items`` (or
    ``plan``, ``grads``, ``steps``) as for ``lattice_update_many``; every tensor is owner ``rank``'s shard, rows
    [rank * rows, (rank + 1) * rows) of a weight of ``world * rows`` rows (rows a multiple of 128; ``offset`` = the RNG
    index of the shard's first element). Between the statistics and the update ``exchange(blocks)`` is called once
    with an fp32 tensor [world, n] of which this owner has filled row ``rank``; on return every row must hold its
    owner's sums (an in-place all-gather, issued on the current stream)."""
    if direction not in _DIRECTION:
        raise RuntimeError(f"direction {direction!r} is outside this build (raw, sign, colnorm are built)")
    if plan is None:
        if len(items) == 0:
            return
        plan = UpdatePlan(items, fmt, phase_bits)
        grads = [it["grad"] for it in items]
        steps = [it["step"] for it in items]
    n, gdtype = plan.n, plan.gdtype
    if gdtype not in _C.DTYPE:
        raise RuntimeError("gradient: bf16, fp16 or fp32 with rows*cols elements")
    grad, step, sj = plan.grad, plan.step, plan.strat_j
    strat_k = 1
    for i in range(n):
        G = grads[i]
        if G.dtype != gdtype or G.numel() != plan.numel[i] or not G.is_cuda or not G.is_contiguous():
            raise RuntimeError("gradient: a contiguous CUDA tensor of the group's dtype with rows*cols elements")
        grad[i] = G.data_ptr()
        step[i] = int(steps[i]) & 0xFFFFFFFF
        if rounding == "strat":
            sj[i], strat_k = strat_args(rounding, steps[i], strata)
    if rounding != "strat":
        strat_k = strat_args(rounding, steps[0], strata)[1]
    dev = plan.device
    need = plan.scratch_need.get(("shards", world))
    if need is None:
        need = plan.scratch_need[("shards", world)] = int(_C.lib().bl_update_shards_scratch_bytes(n, plan.rows, plan.cols,
                                                                                                  world))
    scratch = _scratch_for(dev.device, need)
    where, block, launches = ctypes.c_uint64(0), ctypes.c_uint64(0), ctypes.c_int(0)
    _C.call("bl_update_shard_stats", n, grad, plan.rows, plan.cols, world, rank, _C.DTYPE[gdtype], _DIRECTION[direction],
            float(clip), _C.ptr(scratch), scratch.numel(), ctypes.byref(where), ctypes.byref(block), _C.device_of(dev),
            _C.stream_of(dev), ctypes.byref(launches))
    _C.Counters.launches += launches.value
    if world > 1:
        exchange(scratch[where.value:where.value + world * block.value].view(torch.float32).view(world, -1))
    _C.call("bl_nvfp4_lattice_update_shards", n, plan.packed, plan.phase, plan.scales, plan.gs, grad, plan.rows,
            plan.cols, world, rank, plan.offset, plan.seed, step, sj, _C.DTYPE[gdtype], phase_bits, phase_cb, float(lr),
            float(1.0 - lr * weight_decay), _ROUNDING[rounding], strat_k, _RULE[scale_rule],
            float(kappa(trust, trust_lr, lr)), _DIRECTION[direction], float(clip), _C.ptr(scratch), scratch.numel(),
            _C.device_of(dev), _C.stream_of(dev), ctypes.byref(launches))
    _C.Counters.launches += launches.value


def direction(G, kind: str, r=None, c=None, k: int = 1, beta2: float = 0.95, block=0, ns_steps: int = 5,
              ns_dtype: str = "bf16", sinkhorn_iters: int = 2, clip: float = 1.0, **unused) -> torch.Tensor:
    """Update direction as float32 [rows, cols], RMS clipped to ``clip`` (reference: bitlattice/_ops.py:110-144).
    'raw', 'sign' and 'colnorm' are built."""
    if kind not in _DIRECTION:
        raise RuntimeError(f"direction {kind!r} is outside this build (raw, sign, colnorm are built)")
    G2 = G.reshape(1, -1) if G.dim() == 1 else G.reshape(G.shape[0], -1)
    G2 = _require(G2.contiguous(), "gradient")
    if G2.dtype not in _C.DTYPE:
        G2 = G2.float()
    rows, cols = G2.shape
    D = torch.empty(rows, cols, dtype=torch.float32, device=G2.device)
    scratch = _scratch_for(G2.device, update_scratch_bytes(rows, cols, kind, clip))
    _C.call("bl_direction", _C.ptr(G2), _C.DTYPE[G2.dtype], rows, cols, _DIRECTION[kind], float(clip), _C.ptr(D),
            _C.ptr(scratch), scratch.numel() if scratch is not None else 0, _C.device_of(G2), _C.stream_of(G2),
            extra_kernels=2 if scratch is not None else 0)
    return D


# ------------------------------------------------------------------------------------------------ operand quantizers

def blocked_scale_bytes(rows: int, cols16: int) -> int:
    """Bytes of the 128x4-tiled scale layout (== bl_blocked_scale_bytes of the library; tests compare the two)."""
    return ((rows + 127) // 128) * ((cols16 + 3) // 4) * 512


def amax_global(x: torch.Tensor) -> torch.Tensor:
    """fp32 [4]: [0] = max|x|, [1] = the per-tensor NVFP4 scale max(amax/(6*448), 1e-12)
    (reference: bitlattice/backend.py:240-241), [3] = max(amax/(6*256), 1e-12), the per-tensor scale of the
    four-over-six recipe."""
    _require(x, "x")
    out = torch.empty(4, dtype=torch.float32, device=x.device)
    _C.call("bl_nvfp4_amax", _C.ptr(x), _C.DTYPE[x.dtype], x.numel(), _C.ptr(out), _C.device_of(x), _C.stream_of(x))
    return out


def _scale_buffer(rows: int, cols16: int, blocked: bool, device) -> torch.Tensor:
    if blocked:
        return torch.empty(blocked_scale_bytes(rows, cols16), dtype=torch.uint8, device=device)
    return torch.empty(rows, cols16, dtype=torch.uint8, device=device)


def quantize_nvfp4(x: torch.Tensor, global_scale: torch.Tensor, seed: int = -1, step: int = 0, blocked: bool = False):
    """x [rows, cols] -> (packed [rows, cols/2] uint8, scales). ``blocked``: scales in the GEMM's 128x4-tiled layout
    (flat uint8), else float8_e4m3fn [rows, cols/16] (reference: torch.ops.bitlattice.quantize_nvfp4)."""
    _require(x, "x")
    _require(global_scale, "global_scale", torch.float32)
    if x.dtype not in _C.DTYPE:
        raise RuntimeError("x must be bf16, fp16 or fp32")
    cols = x.shape[-1]
    rows = x.numel() // cols
    packed = torch.empty(rows, cols // 2, dtype=torch.uint8, device=x.device)
    scales = _scale_buffer(rows, cols // 16, blocked, x.device)
    _C.call("bl_nvfp4_quantize", _C.ptr(x), _C.DTYPE[x.dtype], rows, cols, _C.ptr(global_scale), int(seed),
            int(step) & 0xFFFFFFFF, _C.ptr(packed), _C.ptr(scales), int(blocked), _C.device_of(x), _C.stream_of(x))
    return packed, scales if blocked else scales.view(torch.float8_e4m3fn)


def amax_quantize_nvfp4(x: torch.Tensor, seed: int = -1, step: int = 0, blocked: bool = False):
    """``amax_global`` and ``quantize_nvfp4`` against the scale it finds, enqueued by one library call: returns
    (packed, scales, amax [4]); the per-tensor scale is ``amax[1:2]``."""
    _require(x, "x")
    if x.dtype not in _C.DTYPE:
        raise RuntimeError("x must be bf16, fp16 or fp32")
    cols = x.shape[-1]
    rows = x.numel() // cols
    am = torch.empty(4, dtype=torch.float32, device=x.device)
    packed = torch.empty(rows, cols // 2, dtype=torch.uint8, device=x.device)
    scales = _scale_buffer(rows, cols // 16, blocked, x.device)
    _C.call("bl_nvfp4_amax_quantize", _C.ptr(x), _C.DTYPE[x.dtype], rows, cols, _C.ptr(am), int(seed),
            int(step) & 0xFFFFFFFF, _C.ptr(packed), _C.ptr(scales), int(blocked), _C.device_of(x), _C.stream_of(x))
    return packed, scales if blocked else scales.view(torch.float8_e4m3fn), am


def quantize_nvfp4_4over6(x: torch.Tensor, global_scale: torch.Tensor, select: str = "mse", blocked: bool = False):
    """The four-over-six round-to-nearest quantizer of forward activations: every block keeps the better of "maximum
    mapped to 6" and "maximum mapped to 4" (``select``: 'mse' or 'mae'). ``global_scale``: amax / (6 * 256), i.e.
    ``amax_global(x)[3:4]`` (reference: torch.ops.bitlattice.nvfp4_quantize with four_over_six; Python twin
    bitlattice/fp4ref.py:103-135)."""
    _require(x, "x")
    _require(global_scale, "global_scale", torch.float32)
    if x.dtype not in _C.DTYPE:
        raise RuntimeError("x must be bf16, fp16 or fp32")
    if select not in ("mse", "mae"):
        raise ValueError("select must be 'mse' or 'mae'")
    cols = x.shape[-1]
    rows = x.numel() // cols
    packed = torch.empty(rows, cols // 2, dtype=torch.uint8, device=x.device)
    scales = _scale_buffer(rows, cols // 16, blocked, x.device)
    _C.call("bl_nvfp4_quantize_4over6", _C.ptr(x), _C.DTYPE[x.dtype], rows, cols, _C.ptr(global_scale),
            1 if select == "mae" else 0, _C.ptr(packed), _C.ptr(scales), int(blocked), _C.device_of(x), _C.stream_of(x))
    return packed, scales if blocked else scales.view(torch.float8_e4m3fn)


Q_MODES = {"rtn": 0, "sr": 1, "eden": 2}


def nvfp4_quantize_general(x: torch.Tensor, *, transpose: bool = False, mode: str = "rtn", four_over_six: bool = False,
                           select: str = "mse", rotate: bool = False, seed: int = 0, rotate_seed: int = -1,
                           given: torch.Tensor | None = None, pow2: bool = False, w_scales: torch.Tensor | None = None,
                           w_global: torch.Tensor | None = None, blocked: bool = False,
                           amax_out: torch.Tensor | None = None):
    """The general quantizer of the 128-rotation recipes (reference: torch.ops.bitlattice.nvfp4_quantize; Python twin
    bitlattice/fp4ref.py:103-150): x [R, C] dense, or the packed codes of an NVFP4 matrix with ``w_scales`` /
    ``w_global`` (transposed only) -> (packed, scales, global [1]) of x or x^T; ``mode`` 'rtn' | 'sr' | 'eden';
    ``rotate``: randomized 128-point Hadamard rotation along the quantized dimension with ``rotate_seed`` (< 0:
    ``seed``); ``given``: the per-tensor scale to use; ``pow2``: the computed per-tensor scale rounded up to a power
    of two; ``amax_out`` fp32 [1]: receives max|rotated x| (given scale or not)."""
    _require(x, "x")
    if x.dim() != 2:
        raise RuntimeError("x must be a contiguous 2-D CUDA tensor")
    if mode not in Q_MODES:
        raise ValueError("mode must be 'rtn', 'sr' or 'eden'")
    if select not in ("mse", "mae"):
        raise ValueError("select must be 'mse' or 'mae'")
    packed_in = w_scales is not None
    if packed_in:
        _require(w_scales, "w_scales")
        _require(w_global, "w_global", torch.float32)
        R, C = x.shape[0], x.shape[1] * 2
        dtype = 0
    else:
        if x.dtype not in _C.DTYPE:
            raise RuntimeError("x must be bf16, fp16 or fp32")
        R, C = x.shape
        dtype = _C.DTYPE[x.dtype]
    if given is not None:
        _require(given, "given", torch.float32)
    rows, cols = (C, R) if transpose else (R, C)
    packed = torch.empty(rows, cols // 2, dtype=torch.uint8, device=x.device)
    scales = _scale_buffer(rows, cols // 16, blocked, x.device)
    out = torch.empty(2, dtype=torch.float32, device=x.device)           # [0]: the per-tensor scale, [1]: amax scratch
    _C.call("bl_nvfp4_quantize_general", _C.ptr(x), dtype, R, C, int(transpose), Q_MODES[mode], int(four_over_six),
            1 if select == "mae" else 0, int(rotate), int(seed), int(rotate_seed),
            _C.ptr(given) if given is not None else None, int(pow2),
            _C.ptr(_bytes(w_scales)) if packed_in else None, _C.ptr(w_global) if packed_in else None, _C.ptr(packed),
            _C.ptr(scales), int(blocked), _C.ptr(out), _C.ptr(out[1:]),
            _C.ptr(_require(amax_out, "amax_out", torch.float32)) if amax_out is not None else None,
            _C.device_of(x), _C.stream_of(x))
    return packed, scales if blocked else scales.view(torch.float8_e4m3fn), out[:1]


def fp4_fold_scales(scales: torch.Tensor, row_tiles: int, piece: torch.Tensor, g: torch.Tensor, rounded: torch.Tensor
                    ) -> torch.Tensor:
    """In place: the blocked scale bytes ``scales`` (row_tiles x len(piece) tiles of 512 bytes) of operands
    concatenated along K are brought to the common per-tensor scale max(g); ``piece`` int32: the piece of every column
    tile, ``g`` fp32: the pieces' power-of-two scales, ``rounded`` int64 [1]: counter of inexact products. Returns
    max(g) [1] (reference: torch.ops.bitlattice.fp4_fold_scales)."""
    _require(scales, "scales", torch.uint8)
    _require(piece, "piece", torch.int32)
    _require(g, "g", torch.float32)
    _require(rounded, "rounded", torch.int64)
    g_max = torch.empty(1, dtype=torch.float32, device=scales.device)
    _C.call("bl_fp4_fold_scales", _C.ptr(scales), int(row_tiles), piece.numel(), _C.ptr(piece), _C.ptr(g), g.numel(),
            _C.ptr(g_max), _C.ptr(rounded), _C.device_of(scales), _C.stream_of(scales))
    return g_max


def quantize_nvfp4_t(x: torch.Tensor, hadamard: torch.Tensor | None, seed: int = -1, step: int = 0,
                     global_scale: torch.Tensor | None = None, blocked: bool = False):
    """x [M, K] -> NVFP4 of x^T (rotated by ``hadamard`` along M): (packed [K, M/2], scales, global [1])
    (reference: torch.ops.bitlattice.quantize_nvfp4_t)."""
    _require(x, "x")
    if x.dim() != 2:
        raise RuntimeError("x must be a contiguous 2-D CUDA tensor")
    if x.dtype not in _C.DTYPE:
        raise RuntimeError("x must be bf16, fp16 or fp32")
    M, K = x.shape
    if hadamard is not None:
        _require(hadamard, "hadamard", torch.float32)
        if hadamard.numel() != 256:
            raise RuntimeError("hadamard must be a contiguous fp32 [16, 16] tensor")
    packed = torch.empty(K, M // 2, dtype=torch.uint8, device=x.device)
    scales = _scale_buffer(K, M // 16, blocked, x.device)
    gout = torch.empty(1, dtype=torch.float32, device=x.device)
    bound = amax = None
    if global_scale is not None:
        bound = global_scale
        if bound.dtype != torch.float32 or bound.numel() != 1 or not bound.is_contiguous():
            bound = bound.to(torch.float32).reshape(1).contiguous()
        _require(bound, "global_scale")
    else:
        amax = torch.empty(4, dtype=torch.float32, device=x.device)
    _C.call("bl_nvfp4_quantize_t", _C.ptr(x), _C.DTYPE[x.dtype], M, K, _C.ptr(hadamard), int(seed),
            int(step) & 0xFFFFFFFF, _C.ptr(bound), _C.ptr(amax), _C.ptr(packed), _C.ptr(scales), _C.ptr(gout),
            int(blocked), _C.device_of(x), _C.stream_of(x), extra_kernels=0 if bound is not None else 1)
    return packed, scales if blocked else scales.view(torch.float8_e4m3fn), gout


def requantize_nvfp4_t(packed: torch.Tensor, scales: torch.Tensor, global_scale: torch.Tensor, blocked: bool = False):
    """NVFP4 W [N, K] -> NVFP4 of W^T: (packed [K, N/2], scales, global [1])
    (reference: torch.ops.bitlattice.requantize_nvfp4_t)."""
    _require(packed, "packed", torch.uint8)
    _require(scales, "scales")
    g = global_scale
    if g.dtype != torch.float32 or g.numel() != 1 or not g.is_contiguous():
        g = g.to(torch.float32).reshape(1).contiguous()
    _require(g, "global_scale")
    N, K = packed.shape[0], packed.shape[1] * 2
    out = torch.empty(K, N // 2, dtype=torch.uint8, device=packed.device)
    osc = _scale_buffer(K, N // 16, blocked, packed.device)
    gout = torch.empty(1, dtype=torch.float32, device=packed.device)
    _C.call("bl_nvfp4_requantize_t", _C.ptr(packed), _C.ptr(scales), _C.ptr(g), N, K, _C.ptr(out), _C.ptr(osc),
            _C.ptr(gout), int(blocked), _C.device_of(packed), _C.stream_of(packed))
    return out, osc if blocked else osc.view(torch.float8_e4m3fn), gout


def to_blocked(scales: torch.Tensor) -> torch.Tensor:
    """[rows, cols16] scale bytes -> flat 128x4-tiled layout (reference: bitlattice/backend.py:179-188)."""
    _require(scales, "scales")
    rows, cols16 = scales.shape
    out = torch.empty(blocked_scale_bytes(rows, cols16), dtype=torch.uint8, device=scales.device)
    _C.call("bl_nvfp4_scales_to_blocked", _C.ptr(scales), rows, cols16, _C.ptr(out), _C.device_of(scales),
            _C.stream_of(scales))
    return out


def assemble_gathered(recv: torch.Tensor, n: int, K: int, offsets):
    """recv [p, bytes] uint8: the all-gathered per-rank buffers holding, at byte ``offsets`` = (codes, blocked scales,
    transposed codes, transposed row-major scales), the pieces of a weight's row shard [n, K]. Returns the operands of
    the full weight, ((codes [p*n, K/2], blocked scales), (W^T codes [K, p*n/2], blocked scales)), in one launch."""
    _require(recv, "recv", torch.uint8)
    p = recv.shape[0]
    dev = recv.device
    codes = torch.empty(p * n, K // 2, dtype=torch.uint8, device=dev)
    sf = torch.empty(p * blocked_scale_bytes(n, K // 16), dtype=torch.uint8, device=dev)
    tcodes = torch.empty(K, p * n // 2, dtype=torch.uint8, device=dev)
    tsf = torch.empty(blocked_scale_bytes(K, p * n // 16), dtype=torch.uint8, device=dev)
    _C.call("bl_nvfp4_assemble_gathered", _C.ptr(recv), recv.stride(0), p, n, K, *[int(o) for o in offsets],
            _C.ptr(codes), _C.ptr(sf), _C.ptr(tcodes), _C.ptr(tsf), _C.device_of(recv), _C.stream_of(recv))
    return (codes, sf), (tcodes, tsf)


# ------------------------------------------------------------------------------------------------ GEMM

def nvfp4_gemm(a_packed, a_sf, a_global, b_packed, b_sf, b_global, out_dtype=torch.bfloat16,
               out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """(A B^T) * ga * gb for NVFP4 A [M, K], B [N, K] with blocked scales; fp32 accumulation on FP4 tensor cores
    (reference: bitlattice/backend.py:280-290). ``accumulate``: add the product to ``out`` (the bits of
    ``out + product`` as an add of two tensors of out's type)."""
    _require(a_packed, "a_packed", torch.uint8)
    _require(b_packed, "b_packed", torch.uint8)
    _require(a_sf, "a_sf")
    _require(b_sf, "b_sf")
    M, K = a_packed.shape[0], a_packed.shape[1] * 2
    N = b_packed.shape[0]
    if b_packed.shape[1] * 2 != K:
        raise RuntimeError(f"operand K mismatch: {K} vs {b_packed.shape[1] * 2}")
    if a_sf.numel() < blocked_scale_bytes(M, K // 16) or b_sf.numel() < blocked_scale_bytes(N, K // 16):
        raise RuntimeError("scale buffers are smaller than the blocked layout of their operands")
    ga = _require(a_global, "a_global", torch.float32)
    gb = _require(b_global, "b_global", torch.float32)
    if out is None:
        if accumulate:
            raise RuntimeError("accumulate needs the tensor to add to (out=)")
        out = torch.empty(M, N, dtype=out_dtype, device=a_packed.device)
    elif out.shape != (M, N) or not out.is_cuda or out.stride(1) != 1:
        raise RuntimeError(f"out must be a CUDA tensor [{M}, {N}] with unit column stride")
    _C.call("bl_nvfp4_gemm_accumulate" if accumulate else "bl_nvfp4_gemm", _C.ptr(a_packed), _C.ptr(a_sf), _C.ptr(ga), _C.ptr(b_packed), _C.ptr(b_sf), _C.ptr(gb),
            M, N, K, _C.ptr(out), _C.DTYPE[out.dtype], out.stride(0), _C.device_of(a_packed), _C.stream_of(a_packed))
    return out


def swiglu_fwd(g: torch.Tensor, u: torch.Tensor) -> torch.Tensor:
    """a = T(T(silu(g)) * u), the bits of ``F.silu(g) * u`` under autograd (reference:
    torch.ops.bitlattice.swiglu_fwd)."""
    _require(g, "g")
    _require(u, "u", g.dtype)
    if g.dtype not in (torch.bfloat16, torch.float16) or g.shape != u.shape:
        raise RuntimeError("swiglu: g and u must be bf16 or fp16 tensors of one shape")
    a = torch.empty_like(g)
    if g.numel():
        _C.call("bl_swiglu_fwd", _C.ptr(g), _C.ptr(u), _C.ptr(a), _C.DTYPE[g.dtype], g.numel(), _C.device_of(g),
                _C.stream_of(g))
    return a


def swiglu_bwd(g: torch.Tensor, u: torch.Tensor, da: torch.Tensor):
    """(dg, du) of swiglu_fwd for the upstream gradient ``da`` (reference: torch.ops.bitlattice.swiglu_bwd)."""
    _require(g, "g")
    _require(u, "u", g.dtype)
    _require(da, "da", g.dtype)
    if g.dtype not in (torch.bfloat16, torch.float16) or g.shape != u.shape or g.shape != da.shape:
        raise RuntimeError("swiglu: g, u and da must be bf16 or fp16 tensors of one shape")
    dg, du = torch.empty_like(g), torch.empty_like(g)
    if g.numel():
        _C.call("bl_swiglu_bwd", _C.ptr(g), _C.ptr(u), _C.ptr(da), _C.ptr(dg), _C.ptr(du), _C.DTYPE[g.dtype], g.numel(),
                _C.device_of(g), _C.stream_of(g))
    return dg, du


GEMM_KERNELS = {"auto": 0, "tile": 1, "persistent": 2, "pair": 3}


def gemm_select(kernel: str = "auto") -> None:
    """Force one of the GEMM kernels for every later nvfp4_gemm call of this process ("tile": 128 x 128 tiles,
    "persistent": 128 x 256 tiles with one CTA per SM, "pair": 256 x 256 tiles on pairs of SMs), or hand the choice
    back to the library ("auto"). All kernels give identical results; this exists for tests and experiments."""
    _C.call("bl_nvfp4_gemm_select", GEMM_KERNELS[kernel])


def gemm_status_async(host_flag: torch.Tensor, device: int, stream=None) -> None:
    """Enqueue, behind the work already on the current stream of ``device``, a copy of the GEMM kernels' error flag
    (not cleared) into ``host_flag``: a pinned int32 CPU tensor, to be read after that stream has passed the copy."""
    if host_flag.dtype != torch.int32 or host_flag.is_cuda or not host_flag.is_pinned():
        raise RuntimeError("gemm_status_async needs a pinned int32 host tensor")
    st = stream if stream is not None else torch.cuda.current_stream(device).cuda_stream
    _C.call("bl_nvfp4_gemm_status_async", host_flag.data_ptr(), int(device), st)


def selftest_bounded_wait(device: int = 0) -> tuple[int, int]:
    """(recorded code, kernel-returned marker) of the give-up path of the kernels' bounded waits run in isolation:
    (9, 2) when a wait that expires records its code and the kernel still runs to its end."""
    st, ret = ctypes.c_int(0), ctypes.c_int(0)
    scratch = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", device))
    _C.call("bl_selftest_bounded_wait", ctypes.byref(st), ctypes.byref(ret), scratch.data_ptr(), int(device))
    return st.value, ret.value


def mma_peak_tflops(device: int = 0, iters: int = 4096, mma_n: int = 256) -> float:
    """The tensor-pipe ceiling for block-scaled FP4 on this GPU: TFLOP/s of a kernel that only issues MMAs (no loads,
    no scale copies, no epilogue), a few hundred microseconds of work per call, timed with CUDA events."""
    ms, flops = ctypes.c_float(0.0), ctypes.c_double(0.0)
    scratch = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", device))
    _C.call("bl_selftest_mma_peak", int(iters), int(mma_n), ctypes.byref(ms), ctypes.byref(flops), scratch.data_ptr(),
            int(device))
    return flops.value / (ms.value * 1e-3) / 1e12


def gemm_status(device: int = 0) -> int:
    """Device-side error code of the GEMM kernels since the last call (0: none); synchronizes the device."""
    st = ctypes.c_int(0)
    _C.call("bl_nvfp4_gemm_status", ctypes.byref(st), int(device))
    return st.value
