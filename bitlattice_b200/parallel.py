"""Column-parallel (N-sharded) NVFP4 linear layers over one process per GPU.

The reference has no tensor parallelism (its multi-GPU code splits layers, ``bitlattice/parallel.py`` and
``bitlattice/pipeline.py``); this module is the B200 design for the same layer: a weight ``W [N, K]`` is split by rows,
rank r holding rows ``[r*N/p, (r+1)*N/p)`` of codes, scales and optimizer phase, with the per-tensor scale replicated.

    forward   x is sharded along tokens [M/p, K]  --all-gather-->  x [M, K];   y_r = x W_r^T   [M, N/p]
    dgrad     gx_partial_r = gy_r W_r  [M, K]     --reduce-scatter (sum)-->   gx [M/p, K]
    wgrad     gw_r = gy_r^T x  [N/p, K]           local
    update    lattice update of shard r           local: no communication; ``_bl_row_offset`` makes the shard draw
                                                  the random numbers of the unsharded weight

On the FP4 routes each rank quantizes only its own token shard (after an all-reduce of one float, the shard maxima,
so that every rank derives the same per-tensor scale) and the ranks all-gather the packed operands instead of the
bf16 activations: 0.5625 bytes per element instead of 2, and the quantization work shrinks with the world size.

How close to the one-GPU step: the forward shard is the matching columns of the unsharded output bit for bit. By
default a rank quantizes its gradient columns as a tensor of their own (own maximum, own rounding draws), so the
gradients agree with the unsharded layer's statistically. With ``MATCH_UNSHARDED`` the gradient columns take the scale
and the transposed operand's rounding draws of the unsharded gradient: the weight-gradient shard is then the rows of
the unsharded weight gradient bit for bit, and with ``Lattice(shard_group=...)`` (colnorm statistics of the whole
weight) the updated shard is the rows of the one-GPU step's updated weight. The input gradient, a sum of per-rank
partial products, keeps its own rounding either way.

The collectives are NCCL's (``torch.distributed``) over NVLink; gathered operands land in local HBM before any
kernel reads them. ``gloo`` works for CPU tests of the bookkeeping. With ``group=None`` or a world of one the layer
degenerates to the plain lattice linear.

A second exchange pattern over the SAME storage (weights and optimizer state sharded along N, communication-free
update) is ``token_parallel_linear(s)``: every rank keeps its tokens and runs the whole layer on them against the
all-gathered packed weight, and the weight-gradient partials are reduce-scattered to the shard owners,

    forward   W_r codes + scales  --all-gather (0.5625 B/weight)-->  W [N, K];      y = x_r W^T   [M/p, N]
    dgrad     re-quantized W_r^T  --all-gather-->  W^T [K, N];                       gx_r = gy_r W  [M/p, K]
    wgrad     gw_partial_r = gy_r^T x_r  [N, K]    --reduce-scatter (sum)-->          gw [N/p, K]
    update    as above

which moves weight-sized instead of activation-sized messages (about 3.1 N K bytes per layer and step -- 1.125 N K
of packed operands gathered, 2 N K of bf16 partials scattered -- against 3.1 M K): the better choice when a step has
more tokens M than the weight has rows N. A rank's layer is exactly the single-GPU layer on
its tokens -- its own per-tensor scales and stochastic-rounding draws, i.e. the ranks are the micro-batches of the
reference's gradient accumulation (``Lattice.accumulate``: the gradient is the sum over micro-batches in the
weight's dtype).
"""
from __future__ import annotations

import weakref
from collections import OrderedDict

import torch
import torch.distributed as dist

from .tensor import LatticeTensor, wait_for_update

__all__ = ["ColumnParallelFp4Linear", "ColumnParallelLinear", "GatheredWeights", "SharedInputFp4Linears",
           "TokenParallelFp4Linear", "TokenParallelLinear", "column_parallel_linear", "column_parallel_linears",
           "gathered_input_operands", "shard_bounds", "shard_rows", "shared_input_linears", "token_parallel_linear",
           "token_parallel_linears", "world"]


# Column blocks of K the column-parallel backward splits its input-gradient GEMMs into, each block's reduce-scatter
# running under the GEMMs that follow (same bits as the unsplit backward). 1: not split -- the default, because at two
# GPUs the split measured slower (3301 against 3497 TFLOP/s on the 8B-class stack: four times the launches on a
# quarter of the columns each, while the reduce-scatter already hides under the weight-gradient GEMMs).
COLUMN_BLOCKS = 1


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
    t._bl_rows_total = w.rows
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


def _gather_cat(local: torch.Tensor, group, size: int) -> torch.Tensor:
    """all-gather of equally shaped contiguous tensors, stacked along a new leading dimension"""
    out = torch.empty(size, *local.shape, dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, local.contiguous(), group=group)
    return out


class _PendingTransposed:
    """The rotated transposed operand of the gathered input while its all-gathers are in flight; ``get`` waits for
    them (once), permutes the shards into place and re-tiles the scales."""

    def __init__(self, works, codes, scales, g, K, cols):
        self.works, self.codes, self.scales, self.g, self.K, self.cols = works, codes, scales, g, K, cols
        self.operand = None

    def get(self):
        if self.operand is None:
            from . import _ops, backend
            for w in self.works:
                w.wait()
            # shards are column slices of the transposed operand: [p, K, m] -> [K, p * m]
            tpf = self.codes.permute(1, 0, 2).reshape(self.K, self.cols // 2)
            tsf = self.scales.permute(1, 0, 2).reshape(self.K, self.cols // 16)
            self.operand = backend.Fp4Operand(tpf, _ops.to_blocked(tsf.contiguous()), self.g, True)
            self.works = self.codes = self.scales = None
        return self.operand


def gathered_input_operands(x_shard: torch.Tensor, group, want_t: bool):
    """NVFP4 GEMM operands of the full input x [M, K] from this rank's token shard [M/p, K] (M/p a multiple of 128):
    the row operand Q(x) and, if asked, the rotated transposed operand Q(rot(x^T)) for the weight gradient, returned as
    an object whose ``get()`` yields it: its all-gathers run asynchronously, so they overlap the forward GEMMs. Codes
    and scales equal those of the unsharded quantization bit for bit: the per-tensor scale comes from the maximum over
    all shards, blocks of 16 never straddle shards, and 128-row scale tiles are whole."""
    from . import _ops, backend
    rank, size = world(group)
    K = x_shard.shape[-1]
    x2 = x_shard.reshape(-1, K).contiguous()
    rows = x2.shape[0]
    amax = _ops.amax_global(x2)[0:1].clone()
    dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
    g = _ops.amax_global(amax)[1:2]                       # the scale rule applied to the global maximum
    packed, sf = _ops.quantize_nvfp4(x2, g, -1, 0, blocked=True)
    xq = backend.Fp4Operand(_gather_cat(packed, group, size).view(size * rows, K // 2),
                            _gather_cat(sf, group, size).view(-1), g, True)
    xt = None
    if want_t:
        tp, ts, tg = _ops.quantize_nvfp4_t(x2, backend._hadamard16(x2.device, torch.float32), -1, 0, g * 4.0,
                                           blocked=False)
        ts = ts.view(torch.uint8)
        codes = torch.empty(size, *tp.shape, dtype=tp.dtype, device=tp.device)
        scales = torch.empty(size, *ts.shape, dtype=ts.dtype, device=ts.device)
        works = [dist.all_gather_into_tensor(codes, tp, group=group, async_op=True),
                 dist.all_gather_into_tensor(scales, ts.contiguous(), group=group, async_op=True)]
        xt = _PendingTransposed(works, codes, scales, tg, K, size * rows)
    return xq, xt


# With MATCH_UNSHARDED the column-parallel backward quantizes its gradient columns exactly as the unsharded layer
# quantizes them: the per-tensor scale comes from the maximum over ALL columns (one all-reduce(MAX) of a float) and the
# transposed operand draws the unsharded tensor's stochastic-rounding numbers (the hash index of element (m, n) is
# n * M + m with the GLOBAL column n). The weight-gradient shard is then, bit for bit, the rows of the unsharded
# weight gradient, and with ``Lattice(shard_group=...)`` so is the update: an N-GPU step leaves the weights a one-GPU
# step leaves. (The input gradient is a sum of per-rank partial products and keeps its own rounding.) Off by default:
# it costs a small collective per projection and backward pass.
MATCH_UNSHARDED = False

_HASH_INDEX_MUL = 0x27D4EB2F                        # the counter hash: h = index * this + key(seed, step)
_HASH_STEP_INV = pow(0x85EBCA77, -1, 1 << 32)       # key(seed, step) = seed * 0x9E3779B1 + step * 0x85EBCA77


def _matching_gradient_operands(g2p: torch.Tensor, group, need_rows: bool):
    """(row operand or None, transposed rotated operand) of this rank's gradient columns ``g2p`` [M, N / p] with the
    per-tensor scale and the transposed operand's rounding draws of the unsharded gradient [M, N]."""
    from . import _ops, backend
    rank, size = world(group)
    am = _ops.amax_global(g2p)
    if size > 1:
        dist.all_reduce(am, op=dist.ReduceOp.MAX, group=group)      # every entry grows with the maximum
    g = am[1:2]
    s_rows, s_t = backend._seed(), backend._seed()                  # the unsharded order: rows, then transposed
    gq = None
    if need_rows:
        gq = backend.Fp4Operand(*_ops.quantize_nvfp4(g2p, g, seed=s_rows, blocked=True), g, True)
    M, cols = g2p.shape
    # index offset of this rank's first column, carried by the step counter: key(seed, step') = key(seed, 0) + offset * mul
    step = (rank * cols * M * _HASH_INDEX_MUL * _HASH_STEP_INV) & 0xFFFFFFFF
    gt = backend.Fp4Operand(*_ops.quantize_nvfp4_t(g2p, backend._hadamard16(g2p.device, torch.float32), s_t, step,
                                                   g * 4.0, blocked=True), True)
    return gq, gt


class ColumnParallelFp4Linear(torch.autograd.Function):
    """The 'fp4_all' route of the column-parallel layer for one or more weights that read the same input (q/k/v,
    gate/up): shard-local quantization and one packed all-gather for all of them; in the backward the partial input
    gradients of all weights are summed locally, reduce-scattered once, and that collective runs while the weight
    gradients are computed."""

    @staticmethod
    def forward(ctx, x_shard, group, recipe, *weights):
        from . import backend
        need_w = any(ctx.needs_input_grad[3:])
        kind = f"cp:{id(group)}:{'fwd+t' if need_w else 'fwd'}"
        xq, xt = backend._shared(x_shard, recipe, kind, lambda: gathered_input_operands(x_shard, group, need_w))
        ctx.group, ctx.weights, ctx.recipe, ctx.xt = group, weights, recipe, xt
        ctx.x_meta = (x_shard.shape, x_shard.dtype)
        return tuple(backend.fp4_mm(xq, backend.weight_operand(w), x_shard.dtype) for w in weights)

    @staticmethod
    def backward(ctx, *gys):
        from . import _ops, backend
        shape, dtype = ctx.x_meta
        rank, size = world(ctx.group)
        need_x = ctx.needs_input_grad[0]
        live = [(w, gy) for w, gy in zip(ctx.weights, gys) if gy is not None]
        K = ctx.weights[0].shape[1]
        rows = live[0][1].numel() // live[0][1].shape[-1] if live else 0
        matching = MATCH_UNSHARDED and need_x and ctx.recipe.legacy and rows % 32 == 0
        blocks = COLUMN_BLOCKS if (need_x and live and rows % (32 * size) == 0 and K % (COLUMN_BLOCKS * 128) == 0
                                   and rows * K >= (1 << 24) and not matching) else 1
        staged, gx_sum, gx_out, works, parts = {}, None, None, [], []
        if need_x and blocks > 1:
            # The input-gradient partial [M, K] is formed in column blocks of K: for every block the GEMMs of all
            # projections (the first writes, the others add in their epilogues), then its reduce-scatter is started
            # and runs under the GEMMs of the next blocks and under the weight-gradient GEMMs. A column block of the
            # product needs the matching rows of W^T: a contiguous slice of its codes and of its tiled scales.
            for w, gy in live:
                g2p = gy.reshape(-1, gy.shape[-1]).contiguous()
                staged[id(w)] = (g2p, backend.quantize_fp4(g2p, stochastic=True))
            Kb = K // blocks
            for b in range(blocks):
                buf = torch.empty(rows, Kb, dtype=dtype, device=live[0][1].device)
                for n, (w, gy) in enumerate(live):
                    gq, wt = staged[id(w)][1], backend.weight_t_operand(w)
                    tile_bytes = wt.scales.numel() // (K // 128)                # tiled scales of 128 rows of W^T
                    _ops.nvfp4_gemm(gq.packed, gq.scales, gq.global_scale, wt.packed[b * Kb:(b + 1) * Kb],
                                    wt.scales[b * (Kb // 128) * tile_bytes:(b + 1) * (Kb // 128) * tile_bytes],
                                    wt.global_scale, dtype, out=buf, accumulate=n > 0)
                part = torch.empty(rows // size, Kb, dtype=dtype, device=buf.device)
                works.append((dist.reduce_scatter_tensor(part, buf, op=dist.ReduceOp.SUM, group=ctx.group,
                                                         async_op=True), buf))
                parts.append(part)
        else:
            for w, gy in live:
                if matching:
                    g2p = gy.reshape(-1, gy.shape[-1]).contiguous()
                    gq, gt = _matching_gradient_operands(g2p, ctx.group, True)
                    gx = backend.fp4_mm(gq, backend.weight_t_operand(w), gy.dtype, add_to=gx_sum)
                    gx_sum = gx if gx_sum is None else gx_sum
                    staged[id(w)] = (g2p, gq, gt)
                    continue
                if need_x:
                    # the partial input gradients of the projections are summed in the GEMM's epilogue (same bits as
                    # adding the tensors) whenever the rows need no padding; otherwise by a dense add
                    if gx_sum is not None and rows % 32 == 0 and gx_sum.shape[0] == rows and gx_sum.is_contiguous():
                        _, g2p, gq = backend.fp4_dgrad(gy, w, ctx.recipe, add_to=gx_sum)
                    else:
                        gx, g2p, gq = backend.fp4_dgrad(gy, w, ctx.recipe)
                        gx_sum = gx if gx_sum is None else gx_sum.add_(gx)
                else:
                    g2p, gq = backend._pad_rows(gy.reshape(-1, gy.shape[-1]), 32).contiguous(), None
                staged[id(w)] = (g2p, gq)
            if gx_sum is not None:
                gx_sum = gx_sum.to(dtype).contiguous()
                gx_out = torch.empty(gx_sum.shape[0] // size, gx_sum.shape[1], dtype=dtype, device=gx_sum.device)
                works.append((dist.reduce_scatter_tensor(gx_out, gx_sum, op=dist.ReduceOp.SUM, group=ctx.group,
                                                         async_op=True), gx_sum))
        gws = []
        for i, (w, gy) in enumerate(zip(ctx.weights, gys)):
            st = staged.get(id(w)) if gy is not None else None
            if st is None or not ctx.needs_input_grad[3 + i] or ctx.xt is None:
                gws.append(None)
                continue
            if len(st) == 3:                          # operands quantized as the unsharded layer quantizes them
                gws.append(backend.fp4_mm(st[2], ctx.xt.get(), w.dtype))
            else:
                gws.append(backend.fp4_wgrad(st[0], st[1], ctx.xt.get(), w, ctx.recipe).to(w.dtype))
        for work, _ in works:
            work.wait()
        if parts:
            gx_out = torch.cat(parts, 1)
        if gx_out is not None:
            gx_out = gx_out.reshape(shape)
        return (gx_out, None, None, *gws)


class SharedInputFp4Linears(torch.autograd.Function):
    """Several 'fp4_all' layers on one input in one process (q/k/v, gate/up; what the column-parallel function does
    without its collectives): one quantization of the input for all of them, and in the backward the input gradients
    of the projections are summed in the epilogue of their GEMMs (``fp4_dgrad(add_to=)``, the bits of adding the
    tensors in the order of ``weights``) instead of by autograd's accumulation, which costs a pass over the gradient
    per extra projection."""

    @staticmethod
    def forward(ctx, x, recipe, *weights):
        from . import backend
        K = x.shape[-1]
        M = x.numel() // K
        if any(ctx.needs_input_grad[2:]):
            xq, xt = backend._shared(x, recipe, "fwd+t",
                                     lambda: backend._input_operands(x, recipe, site=backend._site(weights[0], "x")))
        else:
            xq, xt = backend._shared(x, recipe, "fwd", lambda: backend._act_operand(
                backend._pad_rows(x.reshape(-1, K), 16).contiguous(), recipe)), None
        ctx.weights, ctx.recipe, ctx.xt = weights, recipe, xt
        ctx.x_meta = (x.shape, x.dtype)
        return tuple(backend.fp4_mm(xq, backend.weight_operand(w), x.dtype)[:M].reshape(*x.shape[:-1], w.shape[0])
                     for w in weights)

    @staticmethod
    def backward(ctx, *gys):
        from . import backend
        shape, dtype = ctx.x_meta
        M = 1
        for d in shape[:-1]:
            M *= d
        staged, gx_sum = [], None
        for w, gy in zip(ctx.weights, gys):
            if gy is None:
                staged.append(None)
                continue
            if ctx.needs_input_grad[0]:
                if gx_sum is not None and M % 32 == 0 and gx_sum.is_contiguous():
                    _, g2p, gq = backend.fp4_dgrad(gy, w, ctx.recipe, add_to=gx_sum)
                else:
                    gx, g2p, gq = backend.fp4_dgrad(gy, w, ctx.recipe)
                    gx_sum = gx if gx_sum is None else gx_sum.add_(gx)
            else:
                g2p, gq = backend._pad_rows(gy.reshape(-1, gy.shape[-1]), 32).contiguous(), None
            staged.append((g2p, gq))
        gws = []
        for i, (w, st) in enumerate(zip(ctx.weights, staged)):
            if st is None or not ctx.needs_input_grad[2 + i] or ctx.xt is None:
                gws.append(None)
                continue
            gws.append(backend.fp4_wgrad(st[0], st[1], ctx.xt, w, ctx.recipe).to(w.dtype))
        gx = gx_sum.to(dtype).reshape(shape) if gx_sum is not None else None
        return (gx, None, *gws)


def shared_input_linears(x: torch.Tensor, weights) -> tuple:
    """``F.linear(x, w)`` for every weight. When all of them take the 'fp4_all' route with the NVIDIA-recipe operands
    they run as one function that quantizes the input once and sums their input gradients in the GEMM epilogues."""
    weights = tuple(weights)
    if len(weights) > 1 and x.is_cuda and all(isinstance(w, LatticeTensor) and w.dim() == 2 for w in weights):
        from .compute_policy import route
        routes = [route(x, w) for w in weights]
        recipe = routes[0][1].nvfp4
        if all(r[0] == "fp4_all" and r[1].nvfp4 == recipe for r in routes) and recipe.packed_exchange:
            return SharedInputFp4Linears.apply(x, recipe, *weights)
    return tuple(torch.nn.functional.linear(x, w) for w in weights)


def _fp4_all_route(x_shard: torch.Tensor, w):
    """The NVFP4 recipe when the layer would take the 'fp4_all' route and the shard shapes allow packed gathering."""
    if not (isinstance(w, LatticeTensor) and x_shard.is_cuda and x_shard.dim() == 2):
        return None
    from .compute_policy import route
    policy, comp = route(x_shard, w)
    if policy != "fp4_all" or not comp.nvfp4.packed_exchange or x_shard.shape[0] % 128 or x_shard.shape[1] % 64:
        return None                             # (the 128-rotation recipes take the generic route: local layers)
    return comp.nvfp4


def column_parallel_linear(x_shard: torch.Tensor, w: torch.Tensor, group=None, linear=None) -> torch.Tensor:
    """Token-sharded input [M/p, K], row-sharded weight [N/p, K] -> feature-sharded output [M, N/p]."""
    if world(group)[1] == 1:
        return (linear or torch.nn.functional.linear)(x_shard, w)
    if linear is None:
        recipe = _fp4_all_route(x_shard, w)
        if recipe is not None:
            return ColumnParallelFp4Linear.apply(x_shard, group, recipe, w)[0]
    return ColumnParallelLinear.apply(x_shard, w, group, linear or torch.nn.functional.linear)


def column_parallel_linears(x_shard: torch.Tensor, weights, group=None) -> tuple:
    """Several column-parallel layers on one input (q/k/v, gate/up): the outputs of column_parallel_linear for each
    weight. On the 'fp4_all' route they share one quantization and one all-gather of the input, and their input
    gradients leave through a single reduce-scatter -- call backward on all outputs together
    (``torch.autograd.backward(outputs, grads)``) to get that."""
    weights = tuple(weights)
    if world(group)[1] > 1:
        recipes = [_fp4_all_route(x_shard, w) for w in weights]
        if all(r is not None for r in recipes) and all(r == recipes[0] for r in recipes):
            return ColumnParallelFp4Linear.apply(x_shard, group, recipes[0], *weights)
    else:
        return shared_input_linears(x_shard, weights)
    return tuple(column_parallel_linear(x_shard, w, group) for w in weights)


# ------------------------------------------------------------------------------------ token-parallel, gathered weights

class _GatheredEntry:
    __slots__ = ("version", "ref", "batch", "spans", "meta", "row", "t", "nbytes")


class _GatherBatch:
    """One all-gather carrying every piece (codes, tiled scales, transposed codes and scales) of the weights of one
    ``prefetch`` call: each rank sends a single packed buffer, so a group of projections costs one collective; one
    kernel per weight (``_ops.assemble_gathered``) cuts the stacked buffers back into the two GEMM operands."""

    def __init__(self, pieces, group, size):
        send = torch.cat([t.reshape(-1) for t in pieces])                   # one launch; piece sizes are multiples of 16 bytes
        self.recv = torch.empty(size, send.numel(), dtype=torch.uint8, device=send.device)
        self.work = dist.all_gather_into_tensor(self.recv, send, group=group, async_op=True)
        self.send = send

    def buffers(self) -> torch.Tensor:
        """The gathered buffers [p, bytes], after the current stream has been made to wait for them."""
        if self.work is not None:
            self.work.wait()
            self.work = self.send = None
        return self.recv


class _Coalesced:
    """Several collectives of one kind issued as a single NCCL group (one launch, one host call); ``wait`` makes the
    current stream wait for all of them. Falls back to one call per collective on backends without the fast path."""

    def __init__(self, fn, pairs, group, **kw):
        self.works = []
        if len(pairs) > 1 and pairs[0][0].is_cuda and hasattr(dist, "_coalescing_manager"):
            with dist._coalescing_manager(group, async_ops=True) as cm:
                for out, inp in pairs:
                    fn(out, inp, group=group, **kw)
            self.works.append(cm)
        else:
            self.works = [fn(out, inp, group=group, async_op=True, **kw) for out, inp in pairs]
        self.keep = pairs                                   # inputs stay alive until the wait

    def wait(self) -> None:
        for w in self.works:
            w.wait()
        self.works, self.keep = [], None


class GatheredWeights:
    """GEMM operands of the full weight assembled from the ranks' row shards: W [N, K] for the forward and the
    re-quantized W^T [K, N] for the input gradient, valid for one weight version (``_bl_version``). The all-gather runs
    asynchronously, one collective for all the weights of a ``prefetch`` call; prefetching the weights needed next
    lets it finish under other work. Entries are dropped least recently used beyond ``limit_bytes``; weights are held
    weakly."""

    def __init__(self, group=None, limit_bytes: int = 4 << 30):
        self.group, self.limit, self.used = group, limit_bytes, 0
        self.entries: OrderedDict = OrderedDict()

    def _remove(self, key) -> None:
        self.used -= self.entries.pop(key).nbytes

    def clear(self) -> None:
        self.entries.clear()
        self.used = 0

    def _current(self, w):
        e = self.entries.get(id(w))
        if e is not None:
            if e.version == getattr(w, "_bl_version", 0) and e.ref() is w:
                self.entries.move_to_end(id(w))
                return e
            self._remove(id(w))
        return None

    def prefetch(self, weights) -> None:
        """Start the gather of every weight of ``weights`` whose current version is not here yet."""
        from . import _ops, backend
        todo = [w for w in weights if self._current(w) is None]
        if not todo:
            return
        size = world(self.group)[1]
        pieces, made, off = [], [], 0
        for w in todo:
            n, K = w.shape
            if n % 128 or K % 64:
                raise ValueError(f"a [{n}, {K}] shard cannot be gathered as packed operands (rows % 128, cols % 64)")
            wait_for_update(w)                                 # an update on another stream finishes before we read
            local = backend.weight_operand(w)                  # 128-row scale tiles are whole: shards concatenate
            # W_r^T [K, n] is a column slice of W^T: its pieces arrive as [p, K, n/2] and [p, K, n/16] and the
            # assembly kernel puts them side by side on first use
            tp, ts, tg = _ops.requantize_nvfp4_t(w.packed, w.scales, w.global_scale, blocked=False)
            parts = [w.packed, local.scales.view(torch.uint8), tp, ts.view(torch.uint8)]
            e = _GatheredEntry()
            e.version, e.ref = getattr(w, "_bl_version", 0), weakref.ref(w)
            e.spans = []
            for t in parts:
                e.spans.append(off)                            # byte offset of the piece in every rank's buffer
                off += t.numel()
            e.meta = (n, K, w.global_scale.float(), tg)
            e.row = e.t = None
            e.nbytes = 2 * sum(t.numel() for t in parts) * size
            pieces += parts
            made.append((w, e))
        batch = _GatherBatch(pieces, self.group, size)
        for w, e in made:
            e.batch = batch
            self.entries[id(w)] = e
            self.used += e.nbytes
        while self.used > self.limit and len(self.entries) > len(made):
            self._remove(next(iter(self.entries)))

    def _entry(self, w) -> _GatheredEntry:
        e = self._current(w)
        if e is None:
            self.prefetch((w,))
            e = self.entries[id(w)]
        return e

    def _assembled(self, w) -> _GatheredEntry:
        from . import _ops, backend
        e = self._entry(w)
        if e.row is None:
            n, K, g, tg = e.meta
            (codes, sf), (tcodes, tsf) = _ops.assemble_gathered(e.batch.buffers(), n, K, e.spans)
            e.row = backend.Fp4Operand(codes, sf, g, True)
            e.t = backend.Fp4Operand(tcodes, tsf, tg, True)
            e.batch = None                                      # the gathered buffer goes with the last weight cut out
        return e

    def operand(self, w):
        """W [N, K] of the current version as a GEMM operand."""
        return self._assembled(w).row

    def t_operand(self, w):
        """W^T [K, N], re-quantized along N, of the current version as a GEMM operand."""
        return self._assembled(w).t


class TokenParallelFp4Linear(torch.autograd.Function):
    """The 'fp4_all' route of one or more N-sharded weights that read the same input, on this rank's tokens: the plain
    layer's quantizers and GEMMs against the gathered weight operands; the weight-gradient partials leave through
    asynchronous reduce-scatters that run under the input-gradient GEMMs."""

    @staticmethod
    def forward(ctx, x, gathered, recipe, *weights):
        from . import backend
        need_w = any(ctx.needs_input_grad[3:])
        K = x.shape[-1]
        M = x.numel() // K
        if need_w:
            xq, xt = backend._shared(x, recipe, "fwd+t", lambda: backend._input_operands(x, recipe))
        else:
            xq = backend._shared(x, recipe, "fwd", lambda: backend._act_operand(
                backend._pad_rows(x.reshape(-1, K), 16).contiguous(), recipe))
            xt = None
        ctx.gathered, ctx.weights, ctx.recipe, ctx.xt = gathered, weights, recipe, xt
        ctx.x_meta = (x.shape, x.dtype)
        size = world(gathered.group)[1]
        return tuple(backend.fp4_mm(xq, gathered.operand(w), x.dtype)[:M].reshape(*x.shape[:-1], size * w.shape[0])
                     for w in weights)

    @staticmethod
    def backward(ctx, *gys):
        from . import backend
        shape, dtype = ctx.x_meta
        group = ctx.gathered.group
        size = world(group)[1]
        need_x = ctx.needs_input_grad[0]
        staged, gws, pairs = [], [], []
        for i, (w, gy) in enumerate(zip(ctx.weights, gys)):
            need_w = gy is not None and ctx.needs_input_grad[3 + i] and ctx.xt is not None
            if gy is None or not (need_x or need_w):
                staged.append(None)
                gws.append(None)
                continue
            N = gy.shape[-1]
            g2 = gy.reshape(-1, N)
            g2p = backend._pad_rows(g2, 32).contiguous()
            gq = backend.quantize_fp4(g2p, stochastic=True) if need_x else None
            staged.append((gq, g2.shape[0]))
            if not need_w:
                gws.append(None)
                continue
            part = backend.fp4_wgrad(g2p, gq, ctx.xt, w, ctx.recipe).to(w.dtype).contiguous()      # [N, K]
            out = torch.empty(N // size, part.shape[1], dtype=part.dtype, device=part.device)
            pairs.append((out, part))
            gws.append(out)
        # the partials of all weights leave as one NCCL group and are summed while the input gradients are computed
        work = _Coalesced(dist.reduce_scatter_tensor, pairs, group, op=dist.ReduceOp.SUM) if pairs else None
        gx = None
        if need_x:
            for w, st in zip(ctx.weights, staged):
                if st is None:
                    continue
                wt = ctx.gathered.t_operand(w)
                if gx is not None and st[1] % 32 == 0 and gx.shape[0] == st[1] and gx.is_contiguous():
                    backend.fp4_mm(st[0], wt, dtype, add_to=gx)        # summed in the epilogue: no pass of its own
                else:
                    gi = backend.fp4_mm(st[0], wt, dtype)[:st[1]]
                    gx = gi if gx is None else gx.add_(gi)
            if gx is not None:
                gx = gx.reshape(shape)
        if work is not None:
            work.wait()
        return (gx, None, None, *gws)


def _gather_weight_rows(w, group, requires_grad: bool):
    """The full weight from the ranks' row shards as a fresh leaf: a dense tensor, or a LatticeTensor built from the
    gathered parts."""
    if not isinstance(w, LatticeTensor):
        return _all_gather_rows(w.detach(), group).requires_grad_(requires_grad)
    wait_for_update(w)                         # an update still running on another stream finishes first
    packed = _all_gather_rows(w.packed, group)
    scales = _all_gather_rows(w.scales.view(torch.uint8), group).view(w.scales.dtype)
    full = LatticeTensor(packed, scales, w.global_scale, None, w.fmt, (packed.shape[0], *w.shape[1:]), w.dtype,
                         requires_grad=requires_grad)
    full.compute = w.compute
    return full


class TokenParallelLinear(torch.autograd.Function):
    """y = x_r all_gather(W)^T on this rank's tokens with the matching backward (the weight gradient is
    reduce-scattered to the shard owners); ``linear`` is the local layer."""

    @staticmethod
    def forward(ctx, x, w, group, linear):
        wf = _gather_weight_rows(w, group, w.requires_grad)
        with torch.enable_grad():
            xin = x.detach().requires_grad_(x.requires_grad)
            y = linear(xin, wf)
        ctx.group, ctx.xin, ctx.wf, ctx.y = group, xin, wf, y
        return y.detach()

    @staticmethod
    def backward(ctx, gy):
        inputs = [t for t in (ctx.xin, ctx.wf) if t.requires_grad]
        grads = torch.autograd.grad(ctx.y, inputs, gy, allow_unused=True) if inputs else ()
        it = iter(grads)
        gx = next(it) if ctx.xin.requires_grad else None
        gw = next(it) if ctx.wf.requires_grad else None
        if gw is not None:
            gw = _reduce_scatter_rows(gw, ctx.group)
        return gx, gw, None, None


def token_parallel_linear(x: torch.Tensor, w: torch.Tensor, gathered: GatheredWeights | None = None, group=None,
                          linear=None) -> torch.Tensor:
    """This rank's tokens [M/p, K], row-sharded weight [N/p, K] -> this rank's outputs [M/p, N]. ``gathered`` keeps the
    gathered operands of the FP4 route between calls (and carries the process group). The ranks are independent
    micro-batches: give each its own stochastic-rounding stream (``backend.set_sr_seed`` with a rank-dependent
    start), or their rounding errors are drawn from the same numbers."""
    return token_parallel_linears(x, (w,), gathered, group, linear)[0]


def token_parallel_linears(x: torch.Tensor, weights, gathered: GatheredWeights | None = None, group=None,
                           linear=None) -> tuple:
    """Several token-parallel layers on one input (q/k/v, gate/up). On the 'fp4_all' route they share one quantization
    of the input; call backward on all outputs together so that the reduce-scatters of their weight gradients run
    under the input-gradient GEMMs."""
    weights = tuple(weights)
    if gathered is not None:
        group = gathered.group
    fn = linear or torch.nn.functional.linear
    if world(group)[1] == 1:
        return shared_input_linears(x, weights) if linear is None else tuple(fn(x, w) for w in weights)
    if linear is None and x.is_cuda and all(isinstance(w, LatticeTensor) for w in weights):
        from .compute_policy import route
        routes = [route(x, w) for w in weights]
        if all(r[0] == "fp4_all" for r in routes) and all(r[1].nvfp4 == routes[0][1].nvfp4 for r in routes) \
                and routes[0][1].nvfp4.packed_exchange \
                and all(w.shape[0] % 128 == 0 and w.shape[1] % 64 == 0 for w in weights):
            if gathered is None:
                gathered = GatheredWeights(group)
            return TokenParallelFp4Linear.apply(x, gathered, routes[0][1].nvfp4, *weights)
    return tuple(TokenParallelLinear.apply(x, w, group, fn) for w in weights)
