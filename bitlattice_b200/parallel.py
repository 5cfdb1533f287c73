"""Column-parallel (N-sharded) NVFP4 linear layers over one process per GPU.

The reference has no tensor parallelism (its multi-GPU code splits layers, ``bitlattice/parallel.py`` and
``bitlattice/pipeline.py``); this module is the B200 design for the same layer: a weight ``W [N, K]`` is split by rows,
rank r holding rows ``[r*N/p, (r+1)*N/p)`` of codes, scales and optimizer phase, with the per-tensor scale replicated.

    forward   x is sharded along tokens [M/p, K]  --all-gather-->  x [M, K];   y_r = x W_r^T   [M, N/p]
    dgrad     gx_partial_r = gy_r W_r  [M, K]     --reduce-scatter (sum)-->   gx [M/p, K]
    wgrad     gw_r = gy_r^T x  [N/p, K]           local
    update    lattice update of shard r           local: no communication; ``_bl_row_offset`` makes the shard draw
                                                  the random numbers of the unsharded weight

The two collectives are NCCL's (``torch.distributed``) over NVLink; gathered activations land in local HBM before any
kernel reads them. ``gloo`` works for CPU tests of the bookkeeping. With ``group=None`` or a world of one the layer
degenerates to the plain lattice linear.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .tensor import LatticeTensor

__all__ = ["ColumnParallelLinear", "column_parallel_linear", "shard_bounds", "shard_rows", "world"]


def world(group=None) -> tuple[int, int]:
    """(rank, size) of ``group``; (0, 1) when torch.distributed is not initialised."""
    if not (dist.is_available() and dist.is_initialized()):
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


def shard_bounds(n: int, rank: int, size: int, multiple: int = 32) -> tuple[int, int]:
    """Rows [lo, hi) of rank ``rank`` when ``n`` rows are split evenly over ``size`` ranks. Shards must keep the
    layer's alignment (out_features a multiple of 32 for the FP4 backward, bitlattice/backend.py:201 of the
    reference), so ``n`` has to be a multiple of ``size * multiple``."""
    if n % (size * multiple):
        raise ValueError(f"{n} rows cannot be split over {size} ranks in multiples of {multiple}")
    per = n // size
    return rank * per, (rank + 1) * per


def shard_rows(w: LatticeTensor, rank: int, size: int) -> LatticeTensor:
    """The row shard of ``w`` owned by ``rank``: a LatticeTensor [N/size, K] sharing nothing with ``w`` (codes and
    scales copied), same per-tensor scale, ``_bl_row_offset`` = first global row."""
    lo, hi = shard_bounds(w.shape[0], rank, size)
    t = LatticeTensor(w.packed[lo:hi].clone(), w.scales[lo:hi].clone(), w.global_scale.clone(), None, w.fmt,
                      (hi - lo, *w.shape[1:]), w.dtype)
    t.compute = w.compute
    t._bl_row_offset = lo
    return t


def _all_gather_rows(x: torch.Tensor, group) -> torch.Tensor:
    rank, size = world(group)
    if size == 1:
        return x
    out = torch.empty(size * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out


def _reduce_scatter_rows(x: torch.Tensor, group) -> torch.Tensor:
    rank, size = world(group)
    if size == 1:
        return x
    if x.shape[0] % size:
        raise ValueError(f"{x.shape[0]} rows cannot be scattered over {size} ranks")
    out = torch.empty(x.shape[0] // size, *x.shape[1:], dtype=x.dtype, device=x.device)
    if x.device.type == "cpu":                       # gloo has no reduce_scatter_tensor: reduce, then take the slice
        full = x.contiguous().clone()
        dist.all_reduce(full, group=group)
        out.copy_(full[rank * out.shape[0]:(rank + 1) * out.shape[0]])
        return out
    dist.reduce_scatter_tensor(out, x.contiguous(), op=dist.ReduceOp.SUM, group=group)
    return out


class ColumnParallelLinear(torch.autograd.Function):
    """y_r = all_gather(x) W_r^T with the matching backward; ``linear`` is the local layer (F.linear: the lattice
    route of the weight's compute policy)."""

    @staticmethod
    def forward(ctx, x_shard, w, group, linear):
        ctx.group, ctx.linear = group, linear
        x = _all_gather_rows(x_shard, group)
        ctx.rows = x_shard.shape[0]
        with torch.enable_grad():
            xin = x.detach().requires_grad_(x_shard.requires_grad)
            y = linear(xin, w)
        ctx.xin, ctx.y = xin, y
        ctx.w = w
        return y.detach()

    @staticmethod
    def backward(ctx, gy):
        inputs = [t for t in (ctx.xin, ctx.w) if t.requires_grad]
        grads = torch.autograd.grad(ctx.y, inputs, gy, allow_unused=True) if inputs else ()
        it = iter(grads)
        gx_partial = next(it) if ctx.xin.requires_grad else None
        gw = next(it) if ctx.w.requires_grad else None
        gx = _reduce_scatter_rows(gx_partial, ctx.group) if gx_partial is not None else None
        return gx, gw, None, None


def column_parallel_linear(x_shard: torch.Tensor, w: torch.Tensor, group=None, linear=None) -> torch.Tensor:
    """Token-sharded input [M/p, K], row-sharded weight [N/p, K] -> feature-sharded output [M, N/p]."""
    linear = linear or torch.nn.functional.linear
    if world(group)[1] == 1:
        return linear(x_shard, w)
    return ColumnParallelLinear.apply(x_shard, w, group, linear)
