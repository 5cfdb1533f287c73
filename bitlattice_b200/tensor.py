"""LatticeTensor: a torch.Tensor subclass holding a weight as NVFP4 storage.

Mirror of the reference's ``bitlattice/tensor.py`` for the linear-layer path: the logical tensor (shape, dtype) is what
PyTorch code sees; the storage is ``packed`` E2M1 codes, ``scales`` (E4M3 per 16 elements) and ``global_scale``
(fp32 [1]) in exactly the reference's layout, so checkpoints and optimizer state interchange. ``F.linear`` with a
LatticeTensor weight goes through :class:`_LatticeLinear`; any other operator sees the dequantized weight.

Quantization and dequantization run on the GPU kernels of this package (there is no CPU path): ``from_float`` needs a
CUDA tensor. Only ``method="rtn"`` is built (the reference's default ``"mse"`` search is a set-up time choice outside
the hot path); high-precision columns (``keep``) and zero points are not part of NVFP4 and are not built.
"""
from __future__ import annotations

import torch
from torch.utils._pytree import tree_map

from . import _ops
from . import formats as F

__all__ = ["LatticeTensor", "is_lattice", "to_parameter", "wait_for_update"]

_PARTS = ("packed", "scales", "global_scale")
# torch's own "no override" implementation of __torch_function__ (what nn.Parameter uses): attribute reads such as
# .shape or .grad on a lattice parameter happen dozens of times per layer call and should cost what they cost on a
# plain tensor
_plain_torch_function = torch._C._disabled_torch_function_impl


def is_lattice(t) -> bool:
    return isinstance(t, LatticeTensor)


def wait_for_update(t) -> None:
    """Make the current stream wait for the last update of ``t`` that an optimizer issued on another stream
    (``Lattice(overlap=True)`` leaves its event in ``t._bl_updated``), after having an optimizer that still holds the
    update back (``hook_flush='reader'``: ``t._bl_pending``) issue it. Every reader of the storage calls this first,
    so an update that is pending or still running beside the caller's stream is never raced, whatever the order of
    calls."""
    opt = getattr(t, "_bl_pending", None)
    if opt is not None:                  # its update has not been issued yet (an optimizer collecting gradients)
        opt._flush_pending()
    ev = getattr(t, "_bl_updated", None)
    if ev is not None:
        torch.cuda.current_stream(t.packed.device).wait_event(ev)


class LatticeTensor(torch.Tensor):
    packed: torch.Tensor
    scales: torch.Tensor
    global_scale: torch.Tensor
    fmt: F.Format

    @staticmethod
    def __new__(cls, packed, scales, global_scale, zeros, fmt, shape, dtype=torch.bfloat16, hi_idx=None, hi_val=None,
                requires_grad=False):
        if zeros is not None or hi_idx is not None or hi_val is not None:
            raise ValueError("zero points and high-precision columns are not part of the NVFP4 path")
        t = torch.Tensor._make_wrapper_subclass(cls, torch.Size(shape), dtype=dtype, device=packed.device,
                                                requires_grad=requires_grad)
        t.packed, t.scales, t.global_scale = packed, scales, global_scale
        t.zeros = t.hi_idx = t.hi_val = None
        t.fmt = F.get(fmt)
        t.compute = None                 # a bitlattice_b200.Compute, or None: exact
        return t

    def __init__(self, *args, **kwargs):
        super().__init__()

    # construction

    @classmethod
    def from_float(cls, w: torch.Tensor, fmt="nvfp4", method: str = "rtn", keep: float = 0.0,
                   dtype: torch.dtype | None = None, **unused) -> "LatticeTensor":
        """Quantize a dense CUDA tensor: per-tensor scale amax/(6*448), E4M3 group scales amax16/6/global, codes by
        round to nearest with ties to the lower level (== reference.quantize(w, "nvfp4", "rtn"))."""
        fmt = F.get(fmt)
        if method != "rtn":
            raise NotImplementedError(f"quantization method {method!r} is outside this build; use method='rtn'")
        if keep:
            raise NotImplementedError("high-precision columns (keep > 0) are outside this build")
        if not w.is_cuda:
            raise RuntimeError("LatticeTensor.from_float needs a CUDA tensor (this build has no CPU path)")
        w2 = (w.detach().reshape(1, -1) if w.dim() == 1 else w.detach().reshape(w.shape[0], -1)).float().contiguous()
        am = _ops.amax_global(w2)
        g = am[1:2].clone()
        packed, scales = _ops.quantize_nvfp4(w2, g, -1, 0)
        logical = dtype or (w.dtype if w.dtype.is_floating_point else torch.bfloat16)
        return cls(packed, scales, g, None, fmt, w.shape, logical)

    # views of the storage

    @property
    def rows(self) -> int:
        return 1 if self.dim() == 1 else self.shape[0]

    @property
    def cols(self) -> int:
        return self.numel() // self.rows

    def parts(self) -> dict:
        return {k: getattr(self, k) for k in _PARTS}

    def dequantize(self, dtype: torch.dtype | None = None) -> torch.Tensor:
        dtype = dtype or self.dtype
        wait_for_update(self)
        kd = dtype if dtype in (torch.float32, torch.bfloat16, torch.float16) else torch.float32
        w = _ops.dequantize(self.packed, self.scales, self.global_scale, None, self.fmt, self.rows, self.cols, kd)
        return w.to(dtype).reshape(self.shape)

    def storage_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.parts().values())

    def __repr__(self, *, tensor_contents=None) -> str:
        return (f"LatticeTensor(shape={tuple(self.shape)}, format={self.fmt.name}, dtype={self.dtype}, "
                f"device={self.device})")

    def __tensor_flatten__(self):
        return list(_PARTS), (self.fmt, tuple(self.shape), self.dtype)

    @staticmethod
    def __tensor_unflatten__(inner, ctx, outer_size, outer_stride):
        fmt, shape, dtype = ctx
        return LatticeTensor(inner["packed"], inner["scales"], inner["global_scale"], None, fmt, shape, dtype)

    def _map(self, fn, shape=None, dtype=None, shares_storage: bool = False) -> "LatticeTensor":
        """A LatticeTensor over ``fn`` of every part. The side attributes travel with it: a row shard stays a row
        shard (``_bl_row_offset``, ``_bl_rows_total``: the optimizer's RNG offset and the checkpoint writer's gather depend
        on them), and a
        result that shares the storage (detach, alias: what ``nn.Parameter(t)`` is made of) also keeps the weight
        version and the event of an update still running on another stream."""
        t = LatticeTensor(fn(self.packed), fn(self.scales), fn(self.global_scale), None, self.fmt,
                          shape or self.shape, dtype or self.dtype)
        t.compute = self.compute
        keep = (("_bl_row_offset", "_bl_rows_total", "_bl_version", "_bl_updated", "_bl_pending") if shares_storage
                else ("_bl_row_offset", "_bl_rows_total"))
        for name in keep:
            if name in self.__dict__:
                setattr(t, name, self.__dict__[name])
        return t

    # operator interception

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if func is torch.nn.functional.linear:
            x, w = args[0], args[1]
            b = args[2] if len(args) > 2 else kwargs.get("bias")
            if isinstance(w, LatticeTensor) and not isinstance(x, LatticeTensor):
                return _LatticeLinear.apply(x, w, b)
        return _plain_torch_function(func, types, args, kwargs)     # everything else: as for a plain tensor

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        """Operators that act on the storage itself are handled part by part (``_STORAGE_OPS``); every other operator
        sees the dequantized weight."""
        kwargs = kwargs or {}
        handler = _STORAGE_OPS.get(func)
        if handler is not None:
            return handler(*args, **kwargs)
        dense = lambda t: t.dequantize() if isinstance(t, LatticeTensor) else t      # noqa: E731
        return func(*tree_map(dense, args), **tree_map(dense, kwargs))


def _view_of(t: LatticeTensor) -> LatticeTensor:
    """detach / alias: the same storage under a new tensor object (what ``nn.Parameter(t)`` is made of)."""
    return t._map(lambda part: part, shares_storage=True)


def _clone(t: LatticeTensor, **unused) -> LatticeTensor:
    wait_for_update(t)
    return t._map(torch.clone)


def _to_copy(t: LatticeTensor, *, device=None, dtype=None, **unused) -> LatticeTensor:
    """``.to(device)`` moves the parts; a floating dtype only changes the logical dtype (the storage has none)."""
    wait_for_update(t)
    target = t.device if device is None else device
    logical = dtype if (dtype is not None and dtype.is_floating_point) else t.dtype
    return t._map(lambda part: part.to(target), dtype=logical)


def _copy_into(dst: LatticeTensor, src, *unused, **unused_kw) -> LatticeTensor:
    """``dst.copy_(src)``: parts are copied when ``src`` is stored in the same format, else ``src`` (dense, or a lattice
    tensor of another format) is quantized into ``dst``'s format first. Bumps the weight version."""
    wait_for_update(dst)                       # an update still running on another stream finishes first
    if isinstance(src, LatticeTensor):
        wait_for_update(src)
    same_format = isinstance(src, LatticeTensor) and src.fmt == dst.fmt
    if not same_format:
        values = src.dequantize(torch.float32) if isinstance(src, LatticeTensor) else src
        src = LatticeTensor.from_float(values.to(dst.device), dst.fmt, method="rtn", dtype=dst.dtype)
    dst._bl_version = getattr(dst, "_bl_version", 0) + 1          # derived GEMM operands are stale now
    for name in _PARTS:
        mine, theirs = getattr(dst, name), getattr(src, name)
        if mine.shape == theirs.shape:
            mine.copy_(theirs)
        else:
            setattr(dst, name, theirs.to(dst.device).clone())
    return dst


_aten = torch.ops.aten
_STORAGE_OPS = {
    _aten.detach.default: _view_of,
    _aten.alias.default: _view_of,
    _aten.clone.default: _clone,
    _aten._to_copy.default: _to_copy,
    _aten.copy_.default: _copy_into,
    _aten.is_same_size.default: lambda a, b: a.shape == b.shape,
}


class _LatticeLinear(torch.autograd.Function):
    """y = x W^T + b for a lattice weight. The compute policy decides the route when the layer is called
    (reference: bitlattice/tensor.py:204-288):

      exact    the weight is dequantized; forward and both gradients are dense GEMMs in the activations' dtype
      fp4      forward on the FP4 tensor cores, gradients as for 'exact'
      fp4_all  forward and both gradients on the FP4 tensor cores; instead of x the layer saves the quantized,
               rotated x^T that the weight gradient needs
    """

    @staticmethod
    def forward(ctx, x, w: LatticeTensor, bias):
        from . import backend
        from .compute_policy import route
        policy, setting = route(x, w)
        recipe = setting.nvfp4
        wants_gw = ctx.needs_input_grad[1]
        # backward may run on another thread, after the caller's compute(...) block has ended: keep what was chosen
        ctx.w, ctx.policy, ctx.recipe, ctx.bias_grad = w, policy, recipe, bias is not None and ctx.needs_input_grad[2]
        if policy != "fp4_all":
            ctx.save_for_backward(x if wants_gw else None)
            if policy == "fp4":
                return backend.nvfp4_linear(x, w, bias, recipe)
            return torch.nn.functional.linear(x, w.dequantize(x.dtype), bias)
        ctx.x_like = (x.shape, x.dtype)
        if not wants_gw:
            ctx.save_for_backward()
            return backend.nvfp4_linear(x, w, bias, recipe)
        y, xt = backend.fp4_forward_saving(x, w, bias, recipe)
        ctx.xt_flags = (xt.blocked, xt.rotate_seed)
        ctx.save_for_backward(xt.packed, xt.scales, xt.global_scale)
        return y

    @staticmethod
    def backward(ctx, gy):
        w = ctx.w
        wants_gx, wants_gw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        g2 = gy.reshape(-1, gy.shape[-1])
        gb = g2.sum(0) if ctx.bias_grad else None
        if ctx.policy == "fp4_all":
            from . import backend
            shape, dtype = ctx.x_like
            xt = backend.Fp4Operand(*ctx.saved_tensors, *ctx.xt_flags) if ctx.saved_tensors else None
            gx, gw = backend.fp4_backward(gy, w, xt, wants_gx, wants_gw and xt is not None, ctx.recipe)
            if gx is not None:
                gx = gx.to(dtype).reshape(shape)
            if gw is not None:
                gw = gw.to(w.dtype)
            return gx, gw, gb
        (x,) = ctx.saved_tensors
        gx = gy @ w.dequantize(gy.dtype) if wants_gx else None
        gw = (g2.t() @ x.reshape(-1, x.shape[-1])).to(w.dtype) if (wants_gw and x is not None) else None
        return gx, gw, gb


def to_parameter(t: LatticeTensor, requires_grad: bool = True) -> torch.nn.Parameter:
    return torch.nn.Parameter(t, requires_grad=requires_grad)


def _register_safe_globals() -> None:
    """Allow torch.load(weights_only=True) of state dicts containing LatticeTensor."""
    add = getattr(torch.serialization, "add_safe_globals", None)
    if add is not None:
        add([LatticeTensor, F.TableFormat, F.ScaleSpec])


_register_safe_globals()
