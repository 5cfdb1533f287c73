"""Lattice optimizer for NVFP4 weights: every weight is updated directly in its storage format, without master
weights (mirror of the reference's ``bitlattice/optim/lattice.py`` for the part on the hot path).

One step of a parameter W with gradient G:
    D = direction(G), RMS-clipped
    t = latent(W, phase) * (1 - lr*wd) - lr*D
    refit the group scales inside the trust region, then project t back to (code, phase) with unbiased rounding.
For the directions sign, colnorm and raw, direction, scale refit and projection run as ONE pass over codes, phase and
gradient on the GPU (``bl_nvfp4_lattice_update``): the fp32 direction is never materialised and no row tiling is
needed. The other directions of the reference (Newton-Schulz ``muon`` / ``muon_block``, ``factored``, ``sinkhorn``,
neuron-wise normalisation) write D first (``optim/directions.py``) and hand it to the same kernel
(``bl_nvfp4_step_quantized``). Momentum (fp32, bf16, int8, fp8, nvfp4, ternary) replaces the gradient by its running
average.

Same constructor, option names, presets, validation errors, per-parameter seeds (``seed + 7919 * index``), step
counters and state layout (``state[p]["phase"]``: uint8 [rows, cols * container_bits / 8]; factored ``r`` / ``c`` /
``k``; momentum ``m`` / ``mb`` / ``m8`` + ``m8s`` / ``m4p`` + ``m4s`` + ``m4g`` / ``mq`` + ``ms``) as the reference, so optimizer state interchanges.
Not built, and refused with NotImplementedError: NVFP4-format momentum, row-sparse gradients, native-format
(non-lattice) parameters and host-memory state.

``overlap=True`` (reference: lattice.py:225-253 hands each update to a worker thread that issues it on a side stream)
is built without the thread: the hook itself issues the update on a per-device side stream that waits for the
gradient's event, so the caller's stream goes on with the rest of the backward pass while the update runs; ``wait()``
(called by ``step()``) makes the current stream wait for the update streams. A second Python thread would only take
turns with the first one on the interpreter lock.
"""
from __future__ import annotations

import contextlib
import threading
import weakref
from typing import Any

import torch

from .. import _ops
from ..backend import nvtx as _nvtx
from . import directions as D_
from ..packing import packed_cols
from ..tensor import LatticeTensor

__all__ = ["DEFAULTS", "DIRECTIONS", "MOMENTA", "ROUNDINGS", "SCALE_RULES", "Lattice", "defer_fused_updates"]

# windows in which no fused update is applied, across all optimizers and autograd threads (reference: lattice.py:33-45)
_deferred = 0
_deferred_lock = threading.Lock()


def defer_fused_updates(delta: int) -> None:
    """Open (+1) or close (-1) a window in which fused optimizers apply no update: gradients arriving meanwhile are
    summed in ``.grad`` and applied by the next arrival outside every window, or by ``step()``."""
    global _deferred
    with _deferred_lock:
        _deferred = max(0, _deferred + delta)


DIRECTIONS = ("muon_block", "muon", "factored", "sinkhorn", "colnorm", "sign", "raw")
FUSED_DIRECTIONS = ("colnorm", "sign", "raw")        # computed inside the update kernel; the others write D first
MOMENTA = ("none", "fp32", "ternary", "bf16", "int8", "fp8", "nvfp4")
ROUNDINGS = ("sr", "strat", "rtn")
SCALE_RULES = ("fit", "fit_latent", "fixed")

DEFAULTS: dict[str, Any] = dict(
    lr=3e-3, direction="muon_block", vector_direction="factored", phase_bits=2, rounding="sr", scale_rule="fit",
    momentum="none", beta1=0.9, beta2=0.95, weight_decay=0.0, clip=1.0, block=512, ns_steps=5, ns_dtype="bf16",
    ns_coeffs="muon", ns_algo="auto", sinkhorn_iters=2, trust=0.01, trust_lr=1.0, strata=16, tile_elems=1 << 24,
    normalize="none", row_beta=0.95, row_eps=1e-8,
)


def _validate(g: dict) -> None:
    """Same checks, same exception types as the reference (lattice.py:62-76); then what this build leaves out."""
    for key, allowed in (("direction", DIRECTIONS), ("vector_direction", DIRECTIONS), ("momentum", MOMENTA),
                         ("rounding", ROUNDINGS), ("scale_rule", SCALE_RULES)):
        if g[key] not in allowed:
            raise ValueError(f"{key}={g[key]!r}; expected one of {allowed}")
    if not 0 <= g["phase_bits"] <= 8:
        raise ValueError("phase_bits must be in [0, 8]")
    if g["vector_direction"] in ("muon", "muon_block"):
        raise ValueError("vector_direction cannot be a matrix direction")
    if g["normalize"] not in ("none", "row"):
        raise ValueError("normalize must be 'none' or 'row'")
    if g["ns_dtype"] not in ("bf16", "fp16", "fp32"):
        raise ValueError("ns_dtype must be 'bf16', 'fp16' or 'fp32'")
    if g["ns_coeffs"] not in ("muon", "polar_express"):
        raise ValueError("ns_coeffs must be 'muon' or 'polar_express'")
    if g["ns_algo"] not in ("auto", "standard", "gram"):
        raise ValueError("ns_algo must be 'auto', 'standard' or 'gram'")
    for p in g["params"]:
        if not isinstance(p, LatticeTensor):
            raise NotImplementedError("only NVFP4 LatticeTensor parameters are built; native-format parameters "
                                      f"(shape {tuple(p.shape)}, {p.dtype}) need the reference's native step")
        if not _ops.cuda_ok(p.fmt, p.rows, p.cols, p.packed.device):
            raise RuntimeError(f"parameter of shape {tuple(p.shape)} on {p.packed.device}: the update kernels need an "
                               "NVFP4 weight on a CUDA device with rows made of 16-element groups")


class Lattice(torch.optim.Optimizer):
    """The Lattice optimizer (reference: bitlattice/optim/lattice.py:125-145).

    ``params``          an iterable of LatticeTensor parameters or param-group dicts (any key of ``DEFAULTS`` per group)
    ``fused_backward``  apply each parameter's update as soon as its gradient is accumulated and free the gradient
                        (the step then only advances); peak memory holds one gradient
    ``hook_batch``      with ``fused_backward``: gradients are collected until this many are ready (or the backward
                        pass ends) and their updates go to the GPU as one batch; 1 updates every parameter on its
                        own. Same results; fewer, larger launches, and up to ``hook_batch`` gradients held
    ``hook_flush``      when an incomplete batch goes out: 'backward' -- at the end of the backward pass that produced
                        it; 'reader' -- when the batch fills up, at ``step()`` / ``synchronize()``, or as soon as
                        anything in this package reads one of its weights (GEMM operands, dequantize, copies, save):
                        batches then fill across several backward calls. Code that reads ``p.packed`` itself
                        between backward and step must use 'backward'
    ``seed``            base of the per-parameter RNG seeds: parameter number i uses (seed + 7919 * i) mod 2^32
    ``shard_group``     the process group (True: the default group) whose ranks own the row shards of the sharded
                        weights, in rank order and of equal size. Directions that normalise over the whole weight
                        (colnorm; raw and sign with clip < 1) then exchange their 128-row panel sums (weights / 32
                        bytes per step) and every shard receives exactly the update of its rows in the unsharded
                        weight. None: such a direction treats every shard as a weight of its own, without
                        communication. The directions computed outside the update kernel (muon, muon_block, factored,
                        sinkhorn, normalize='row') always work on the shard they are given
    A parameter that is a row shard of a larger weight sets ``p._bl_row_offset`` to its first global row (and
    ``p._bl_rows_total`` to the rows of the whole weight): the update then draws the random numbers of the unsharded
    tensor (as the reference's row tiles do, csrc/update.cpp:50).
    """

    def __init__(self, params, preset: str | None = None, *, lr: float = DEFAULTS["lr"], state: str = "gpu",
                 fused_backward: bool = False, seed: int = 0, weight_decay: float = 0.0, overlap: bool = False,
                 hook_batch: int = 1, hook_flush: str = "backward", shard_group=None, **options):
        from .presets import PRESETS
        if preset is not None:
            if preset not in PRESETS:
                raise KeyError(f"unknown preset {preset!r}; known: {sorted(PRESETS)}")
            options = {**PRESETS[preset], **options}
        options.pop("head_momentum", None)
        unknown = set(options) - set(DEFAULTS)
        if unknown:
            raise TypeError(f"unknown options {sorted(unknown)}")
        if isinstance(params, torch.nn.Module):
            params = [p for p in params.parameters() if p.requires_grad]
        defaults = {**DEFAULTS, **options, "lr": lr, "weight_decay": options.get("weight_decay", weight_decay)}
        super().__init__(params, defaults)
        if state not in ("gpu", "ram", "auto"):
            raise ValueError("state must be 'gpu', 'ram' or 'auto'")
        if state != "gpu":
            raise NotImplementedError("optimizer state in host memory is outside this build (state='gpu' is built)")
        for g in self.param_groups:
            _validate(g)
        self.state_placement = "gpu"
        self.seed = int(seed)
        self.fused_backward = fused_backward
        self.overlap = bool(overlap)
        self.shard_group = shard_group
        self._update_streams: dict = {}
        self._scratch: dict = {}
        self._plans: dict = {}            # (phase bits, ids of a batch of parameters) -> _ops.UpdatePlan
        self._gemm_flags: dict = {}                 # device -> (pinned int32 [1], event after its last async copy)
        self._gens: dict = {}                       # device -> torch.Generator of the bf16 / int8 momentum rounding
        self._pid = {}
        for g in self.param_groups:
            for p in g["params"]:
                self._pid[p] = len(self._pid)
        self._group_of = {p: g for g in self.param_groups for p in g["params"]}
        self._done: set = set()
        self._defer = 0
        self.hook_batch = max(1, int(hook_batch))
        if hook_flush not in ("backward", "reader"):
            raise ValueError("hook_flush must be 'backward' or 'reader'")
        self.hook_flush = hook_flush
        self._pending: list = []                    # parameters whose gradient is ready and whose update is not issued
        self._pending_lock = threading.Lock()
        self._hooks = []
        if fused_backward:
            for p in self._pid:
                if p.requires_grad:
                    self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad))

    # fused backward: the hook runs on the autograd thread that accumulated the gradient

    def _on_grad(self, p: torch.Tensor) -> None:
        if p.grad is None or self._defer or _deferred:
            return
        if self.hook_batch > 1:
            with self._pending_lock:
                self._pending.append(p)
                first, full = len(self._pending) == 1, len(self._pending) >= self.hook_batch
            self._done.add(p)
            if self.hook_flush == "reader":
                p._bl_pending = self                 # readers of the weight have the batch issued first
            elif first:                              # whatever is left when the backward pass ends goes out then
                torch.autograd.Variable._execution_engine.queue_callback(self._flush_pending)
            if full:
                self._flush_pending()
            return
        if self.overlap and p.is_cuda:
            self._update_aside(p, self._group_of[p])
        else:
            with torch.no_grad():
                self._update(p, self._group_of[p])
        p.grad = None
        self._done.add(p)

    def _flush_pending(self) -> None:
        """Issue the updates of the parameters collected by the hooks (``hook_batch``), batched per parameter group."""
        with self._pending_lock:
            ps, self._pending = self._pending, []
        if not ps:
            return
        with torch.no_grad():
            for g in self.param_groups:
                mine = [p for p in ps if self._group_of[p] is g]
                if mine:
                    self._apply(mine, g)
        for p in ps:
            p.grad = None
            if self.hook_flush == "reader":
                p._bl_pending = None

    def _apply(self, todo: list, g: dict) -> None:
        """Update the parameters ``todo`` of group ``g`` from their gradients: those that can share a library call
        (same device, gradient dtype, fused direction, no momentum) in one batch, the others one by one."""
        batch = [p for p in todo if self._batchable(p, g, todo[0])]
        if len(batch) > 1:
            # the tensors of the group in one library call: small shards are paced by the GPU, not the interpreter
            if self.overlap:
                side = self._update_stream(batch[0].device)
                side.wait_stream(torch.cuda.current_stream(batch[0].device))
                with torch.cuda.device(batch[0].device), torch.cuda.stream(side):
                    self._update_many(batch, g)
                    self._mark_updated(batch, side)
                for p in batch:
                    p.grad.record_stream(side)
            else:
                with torch.cuda.device(batch[0].device):
                    self._update_many(batch, g)
            batched = {id(p) for p in batch}
            todo = [p for p in todo if id(p) not in batched]
        for p in todo:
            if self.overlap and p.is_cuda:
                self._update_aside(p, g)
            else:
                with torch.cuda.device(p.device):
                    self._update(p, g)

    def _update_stream(self, device: torch.device) -> torch.cuda.Stream:
        s = self._update_streams.get(device)
        if s is None:
            s = self._update_streams[device] = torch.cuda.Stream(device=device)
        return s

    def _update_aside(self, p: torch.Tensor, g: dict) -> None:
        """Issue the update of ``p`` on the device's update stream, behind everything the caller's stream holds so far
        (the gradient is complete there)."""
        G = p.grad
        side = self._update_stream(p.device)
        side.wait_stream(torch.cuda.current_stream(p.device))
        with torch.cuda.device(p.device), torch.cuda.stream(side), torch.no_grad():
            self._update(p, g, G)
            self._mark_updated((p,), side)
        G.record_stream(side)                        # the gradient's memory is reused only after the update has run

    @staticmethod
    def _mark_updated(ps, side) -> None:
        """Leave the event readers of the storage wait for (``tensor.wait_for_update``)."""
        ev = torch.cuda.Event()
        ev.record(side)
        for p in ps:
            p._bl_updated = ev

    @staticmethod
    def _invalidate(p: torch.Tensor) -> None:
        p._bl_version = getattr(p, "_bl_version", 0) + 1          # derived GEMM operands of the old version are stale
        from ..backend import drop_cached
        drop_cached(p)

    def wait(self) -> None:
        """Make the current stream of every device wait (on the GPU) for the updates issued so far on the update
        streams (``overlap``); without ``overlap`` updates are issued on the caller's stream and there is nothing to
        wait for."""
        for dev, s in self._update_streams.items():
            torch.cuda.current_stream(dev).wait_stream(s)

    def synchronize(self) -> None:
        self._flush_pending()
        for dev in {p.device for p in self._pid if p.is_cuda}:
            torch.cuda.synchronize(dev)
        self.check_gemm_status(wait=True)

    # The GEMM kernels bound every wait; one that expires leaves a partial output and a sticky flag on the device
    # (bl_nvfp4_gemm_status). Gradients computed from such an output must not be trained on, so the optimizer watches
    # the flag: every step() enqueues an asynchronous copy of it into pinned host memory behind the step's work and
    # the next step() -- or synchronize() / state_dict() -- reads the copy and raises. No host synchronisation is
    # added to the step.

    def _watch_gemm_status(self) -> None:
        for dev in {p.device for p in self._pid if p.is_cuda}:
            entry = self._gemm_flags.get(dev)
            if entry is None:
                entry = self._gemm_flags[dev] = (torch.zeros(1, dtype=torch.int32).pin_memory(), torch.cuda.Event())
            flag, ev = entry
            with torch.cuda.device(dev):
                _ops.gemm_status_async(flag, dev.index if dev.index is not None else torch.cuda.current_device())
                ev.record(torch.cuda.current_stream(dev))

    def check_gemm_status(self, wait: bool = False) -> None:
        """Raise if a GEMM kernel of an earlier step gave up on a bounded wait (its output, and any update applied
        from it, is invalid). ``wait``: block until the copies enqueued by the last ``step()`` have arrived. The
        device flag is cleared when the error is raised; weights updated from the failed step are not restored."""
        for dev, (flag, ev) in self._gemm_flags.items():
            if wait:
                ev.synchronize()
            elif not ev.query():
                continue
            code = int(flag.item())
            if code:
                flag.zero_()
                _ops.gemm_status(dev.index if dev.index is not None else torch.cuda.current_device())   # clears it
                raise RuntimeError(f"an NVFP4 GEMM kernel on {dev} gave up on a bounded wait (code {code}: 1 operand "
                                   "loads, 2 MMA issue, 3 epilogue, 4 accumulator hand-over); outputs since then are "
                                   "partial and updates applied from them are invalid")

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self.check_gemm_status()                   # a failed GEMM of an earlier step: raise before updating further
        self._flush_pending()
        for g in self.param_groups:
            todo = [p for p in g["params"] if p not in self._done and p.grad is not None]
            if todo:
                self._apply(todo, g)
                if self.fused_backward:
                    for p in todo:
                        p.grad = None
        self._done.clear()
        self.wait()
        self._watch_gemm_status()
        return loss

    _matrix: dict = {}             # id(parameter) -> whether it counts as a matrix (shape reads of a tensor subclass
                                   # are slow and these run for every parameter of every step)

    @staticmethod
    def _kind(p, g: dict) -> str:
        """The direction of ``p``: matrices use ``direction``, vectors ``vector_direction`` (reference: lattice.py:472-473)."""
        matrix = Lattice._matrix.get(id(p))
        if matrix is None or matrix[0]() is not p:
            matrix = Lattice._matrix[id(p)] = (weakref.ref(p), p.dim() >= 2 and min(p.shape[0], p.numel() // p.shape[0]) > 1)
        return g["direction"] if matrix[1] else g["vector_direction"]

    @staticmethod
    def _fused(p, g: dict) -> bool:
        """Whether the direction of ``p`` is computed inside the update kernel."""
        return Lattice._kind(p, g) in FUSED_DIRECTIONS and g["normalize"] != "row"

    @staticmethod
    def _batchable(p, g: dict, first) -> bool:
        if g["momentum"] != "none" or g["normalize"] == "row":
            return False
        kind = Lattice._kind(p, g)
        if kind not in FUSED_DIRECTIONS or (p is not first and kind != Lattice._kind(first, g)):
            return False
        G = p.grad
        return (p.is_cuda and p.device == first.device and (p.fmt is first.fmt or p.fmt == first.fmt) and not G.is_sparse
                and G.dtype == first.grad.dtype and G.dtype in (torch.bfloat16, torch.float16, torch.float32)
                and G.is_contiguous())

    @staticmethod
    def _is_shard(p) -> bool:
        return getattr(p, "_bl_rows_total", p.rows) != p.rows

    def _whole_weight(self, g: dict, kind: str) -> bool:
        """Whether row shards are updated with the statistics of their whole weights (``shard_group``)."""
        return self.shard_group is not None and not (kind == "sign" and g["clip"] >= 1.0)

    def _shard_world(self):
        import torch.distributed as dist
        group = None if self.shard_group is True else self.shard_group
        return dist.get_world_size(group), dist.get_rank(group), group

    def _exchange(self, blocks: torch.Tensor) -> None:
        """The all-gather, in place, of the owners' panel sums (``_ops.lattice_update_shards``): row r of ``blocks``
        is rank r's."""
        import torch.distributed as dist
        _, rank, group = self._shard_world()
        dist.all_gather_into_tensor(blocks.view(-1), blocks[rank], group=group)

    def _check_shards(self, ps) -> tuple[int, int]:
        """(world, rank) after checking that every parameter of ``ps`` is this rank's equal share of its weight."""
        world, rank, _ = self._shard_world()
        for p in ps:
            row0 = int(getattr(p, "_bl_row_offset", 0))
            if p._bl_rows_total != world * p.rows or row0 != rank * p.rows:
                raise RuntimeError(f"shard_group: rank {rank} of {world} holds rows [{row0}, {row0 + p.rows}) of "
                                   f"{p._bl_rows_total}; equal row shards in rank order are built")
        return world, rank

    def _update_many(self, ps, g: dict) -> None:
        bits = g["phase_bits"]
        cb = _ops.phase_container(bits)
        kind = self._kind(ps[0], g)
        shards = None
        if self._whole_weight(g, kind):
            mine = [p for p in ps if self._is_shard(p)]
            if mine and len(mine) < len(ps):          # shards and whole weights: each kind in a call of its own
                self._update_many(mine, g)
                return self._update_many([p for p in ps if not self._is_shard(p)], g)
            if mine:
                shards = self._check_shards(ps)
        state, invalidate = self.state, self._invalidate
        steps, grads, tensors = [], [], []
        for p in ps:
            invalidate(p)
            st = state[p]
            step = st["step"] = st.get("step", 0) + 1
            steps.append(step)
            if bits and "phase" not in st:
                st["phase"] = torch.zeros(p.rows, packed_cols(p.cols, cb), dtype=torch.uint8, device=p.packed.device)
            grads.append(p.grad)
            tensors.append((p.packed, st["phase"] if bits else None, p.scales, p.global_scale))
        # shapes, offsets, seeds and the weights' addresses are marshalled once per set of parameters
        key = (bits, tuple(map(id, ps)))
        plan = self._plans.get(key)
        if plan is None or plan.gdtype != grads[0].dtype or plan.stale(tensors):
            items = [dict(packed=t[0], phase=t[1], scales=t[2], global_scale=t[3], grad=G, rows=p.rows, cols=p.cols,
                          offset=int(getattr(p, "_bl_row_offset", 0)) * p.cols,
                          seed=(self.seed + 7919 * self._pid[p]) & 0xFFFFFFFF, step=s)
                     for p, t, G, s in zip(ps, tensors, grads, steps)]
            plan = self._plans[key] = _ops.UpdatePlan(items, ps[0].fmt, bits)
        common = dict(lr=g["lr"], weight_decay=g["weight_decay"], phase_bits=bits, phase_cb=cb, rounding=g["rounding"],
                      strata=g["strata"], scale_rule=g["scale_rule"], trust=g["trust"], trust_lr=g["trust_lr"],
                      direction=kind, clip=g["clip"], plan=plan, grads=grads, steps=steps)
        if shards is not None:                       # statistics of the whole weights, exchanged among the owners
            with _nvtx("bl.lattice_update"):
                _ops.lattice_update_shards(None, ps[0].fmt, *shards, self._exchange, **common)
            return
        scratch = None
        if self.overlap:                             # updates that run beside the caller's stream: a buffer of their own
            need = plan.scratch_bytes(kind, g["clip"])
            dev = ps[0].device
            scratch = self._scratch.get(dev)
            if need and (scratch is None or scratch.numel() < need):
                scratch = self._scratch[dev] = torch.empty(need, dtype=torch.uint8, device=dev)
        with _nvtx("bl.lattice_update"):
            _ops.lattice_update_many(None, ps[0].fmt, scratch=scratch, **common)

    @contextlib.contextmanager
    def accumulate(self):
        """Gradient accumulation with ``fused_backward``: inside the context gradients are summed in ``.grad`` and no
        update is applied; the next backward pass outside the context applies the update with the total."""
        self._defer += 1
        try:
            yield
        finally:
            self._defer -= 1

    def state_dict(self):
        self.synchronize()
        return super().state_dict()

    def zero_grad(self, set_to_none: bool = True):
        self._flush_pending()                        # updates still held back need their gradients
        super().zero_grad(set_to_none=True)

    def remove_hooks(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks.clear()

    def _update(self, p: LatticeTensor, g: dict, G: torch.Tensor | None = None) -> None:
        self._invalidate(p)
        st = self.state[p]
        st["step"] = st.get("step", 0) + 1
        seed = (self.seed + 7919 * self._pid[p]) & 0xFFFFFFFF
        G = p.grad if G is None else G
        if G.is_sparse:
            raise NotImplementedError("row-sparse gradients are outside this build")
        rows, cols = p.rows, p.cols
        bits = g["phase_bits"]
        cb = _ops.phase_container(bits)
        if bits and "phase" not in st:
            st["phase"] = torch.zeros(rows, packed_cols(cols, cb), dtype=torch.uint8, device=p.packed.device)
        G2 = G.reshape(rows, cols)
        if g["momentum"] != "none":
            # an exponential average of the gradient, kept in the chosen format between steps, takes the gradient's place
            G2 = D_.momentum(G2, st, g["momentum"], g["beta1"], self.seed, self._pid[p], self._gens)
        if G2.dtype not in (torch.bfloat16, torch.float16, torch.float32):
            G2 = G2.float()
        matrix = p.dim() >= 2 and min(rows, cols) > 1
        kind = self._kind(p, g)
        common = dict(lr=g["lr"], weight_decay=g["weight_decay"], phase_bits=bits, phase_cb=cb, rounding=g["rounding"],
                      seed=seed, step=st["step"], strata=g["strata"], scale_rule=g["scale_rule"], trust=g["trust"],
                      trust_lr=g["trust_lr"], offset=int(getattr(p, "_bl_row_offset", 0)) * cols)
        if not self._fused(p, g):
            # directions outside the update kernel: D is written out, then the kernel takes it as given
            r = c = None
            if kind == "factored":
                if "r" not in st:
                    st["r"] = torch.zeros(rows, device=G2.device)
                    st["c"] = torch.zeros(cols, device=G2.device)
                    st["k"] = 0
                st["k"] += 1
                r, c = st["r"], st["c"]
            row = {}
            if g["normalize"] == "row" and matrix and kind != "factored":       # factored is adaptive already
                if "nv" not in st:
                    st["nv"] = torch.zeros(rows, device=G2.device)
                row = dict(row_state=st["nv"], row_k=st["step"], row_beta=g["row_beta"], row_eps=g["row_eps"])
            D = D_.direction(G2, kind, r, c, st.get("k", 1), g["beta2"], g["block"], g["ns_steps"], g["ns_dtype"],
                             g["sinkhorn_iters"], g["clip"], g["ns_coeffs"], g["ns_algo"], **row)
            _ops.step_quantized(p.packed, st.get("phase") if bits else None, p.scales, p.global_scale, None, D, p.fmt,
                                rows, cols, inplace_scales=True, **common)
            return
        if self._whole_weight(g, kind) and self._is_shard(p):
            item = dict(packed=p.packed, phase=st.get("phase") if bits else None, scales=p.scales,
                        global_scale=p.global_scale, grad=G2.contiguous(), rows=rows, cols=cols,
                        offset=common["offset"], seed=seed, step=st["step"])
            shared = {k: v for k, v in common.items() if k not in ("seed", "step", "offset")}
            with _nvtx("bl.lattice_update"):
                _ops.lattice_update_shards([item], p.fmt, *self._check_shards([p]), self._exchange, direction=kind,
                                           clip=g["clip"], **shared)
            return
        scratch = None
        if self.overlap:                             # column statistics of updates that run beside the caller's stream
            need = _ops.update_scratch_bytes(rows, cols, kind, g["clip"])
            scratch = self._scratch.get(p.device)
            if need and (scratch is None or scratch.numel() < need):
                scratch = self._scratch[p.device] = torch.empty(need, dtype=torch.uint8, device=p.device)
        with _nvtx("bl.lattice_update"):
            _ops.lattice_update(p.packed, st.get("phase") if bits else None, p.scales, p.global_scale, None,
                                G2.contiguous(), p.fmt, rows, cols, direction=kind, clip=g["clip"], scratch=scratch,
                                **common)

    def state_bits(self) -> dict[str, float]:
        """Logical optimizer state in bits, by component (phase and, with momentum='fp32', the fp32 average)."""
        out = {"phase": 0.0, "factors": 0.0, "momentum": 0.0}
        for g in self.param_groups:
            for p in g["params"]:
                out["phase"] += p.numel() * g["phase_bits"]
                mode = g["momentum"]
                if mode == "nvfp4" and p.shape[-1] % 16:
                    mode = "int8"
                out["momentum"] += p.numel() * {"none": 0, "fp32": 32, "bf16": 16, "int8": 8 + 32 / D_.MOM_BLOCK,
                                                "fp8": 8 + 32 / D_.MOM_BLOCK, "ternary": 8, "nvfp4": 4.5}[mode]
                if not self._fused(p, g):
                    kind = g["direction"] if p.dim() >= 2 else g["vector_direction"]
                    if kind == "factored":
                        out["factors"] += 32 * (p.rows + p.cols)
        out["total"] = sum(out.values())
        return out

    def state_bytes(self) -> int:
        return sum(v.numel() * v.element_size() for st in self.state.values() for v in st.values()
                   if torch.is_tensor(v))
