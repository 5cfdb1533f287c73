#!/usr/bin/env python
"""Benchmark of the NVFP4 hot path on B200: linear forward + dgrad + wgrad on FP4 tensor cores with the lattice
update fused into backward, over an 8B-class decoder linear stack.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Workload ("cfg4_8b_linear_stack"): `--layers` decoder layers (default 36) of {q, o: 4096x4096; k, v: 1024x4096;
gate, up: 12288x4096; down: 4096x12288} NVFP4 weights, `--tokens` tokens (default 16 x 4096), bf16 activations
~ N(0,1), upstream gradients ~ N(0, 1e-2^2), weights ~ N(0, 0.02^2), all synthetic and seeded. One step = for every
linear: y = F.linear(x, W) under compute("fp4_all"), y.backward(gy) -> dgrad + wgrad, and the lattice update of W
(colnorm direction, 4-bit phase, stochastic projection, scale refit with trust region 0.1) from the gradient hook.
With N > 1 every weight (codes, scales, optimizer phase) is sharded along N (rows) over the ranks and the update is
local (colnorm normalises every shard on its own; `--whole-colnorm 1` has the ranks exchange their panel sums so that
the shards receive the unsharded update bit for bit); total work is fixed (strong scaling). Two exchange patterns over that storage (`--parallel`):
  column  activations all-gathered (packed), input gradients reduce-scattered, each rank computes its N/p columns;
  token   packed weights all-gathered, weight-gradient partials reduce-scattered, each rank computes its M/p tokens;
  auto    (default) the one that moves fewer bytes for the workload: `token` when a step has more tokens than the
          weights have rows (65,536 tokens against 1024-12288 rows here). The line then also carries the other
          pattern's throughput from a short run (`other_parallelism`).

After the step measurements the lattice update alone is timed over the whole weight set (the 8B-class update workload:
one distinct bf16 gradient ~ N(0, 1e-3^2) per parameter, resident in HBM, every rank its shards, nothing else on the
GPU): `update.value` is its whole-job HBM GB/s. Then, on the same GPU, the GEMM kernel is timed against cuBLASLt
(`torch._scaled_mm`, the reference's Blackwell GEMM) on the workload's GEMM shapes (`vs_cublaslt`), the 32B-class GEMM
sweep runs (`gemm_sweep_32b`: hidden 5120 / intermediate 25600, N-sharded over the ranks) and an MMA-only kernel
measures the tensor-pipe ceiling the roofline fractions are quoted against (`roofline.peak`).

Prints one JSON line (rank 0). `value` is whole-job TFLOP/s with inputs resident in HBM; `e2e` is the same step with
the step's inputs copied from pinned host memory and a checksum read back inside the timed region. `cpu_baseline` and
`--impl reference` time the reference's own CPU path (its Python package staged by oracle/stage_reference.py when a
checkout was present at build time, else the C restatement in oracle/) on a bounded sample and extrapolate to the
workload: GEMM time by flops, update time by weights.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYER = (("q", 4096, 4096), ("k", 1024, 4096), ("v", 1024, 4096), ("o", 4096, 4096),
         ("gate", 12288, 4096), ("up", 12288, 4096), ("down", 4096, 12288))
# the four distinct activations of a decoder layer: q/k/v read one tensor, gate/up another (their quantization is
# shared, as in the reference's fused blocks); o and down have inputs of their own
INPUT_OF = {"q": "attn_in", "k": "attn_in", "v": "attn_in", "o": "o_in", "gate": "mlp_in", "up": "mlp_in",
            "down": "down_in"}
INPUT_WIDTH = {"attn_in": 4096, "o_in": 4096, "mlp_in": 4096, "down_in": 12288}
GROUPS = (("q", "k", "v"), ("o",), ("gate", "up"), ("down",))
INDEX = {n: i for i, (n, _, _) in enumerate(LAYER)}
SHAPE = {n: (N, K) for n, N, K in LAYER}
OPT = dict(lr=3e-3, direction="colnorm", phase_bits=4, rounding="sr", scale_rule="fit", trust=0.1, trust_lr=0.0,
           seed=1234)
BYTES_PER_WEIGHT = 4.125      # codes r+w 1.0, 4-bit phase r+w 1.0, bf16 gradient 2.0, E4M3 scales r+w 0.125
# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) from ncu captures of small cases, scaled by the units a
# launch processes (the summaries of those captures are kept with the other profiles of this repository):
#   update of one layer's seven matrices as a batch (192.9 M weights), colnorm: update_kernel 771.3 MB +
#     colstats_kernel 394.4 MB + finalize_kernel 6.0 MB
#   gemm_pair_kernel 8192 x 12288 x K 4096 (the down projection's input-gradient GEMM at 8192 tokens, the captured
#     launch closest in shape to the workload's): 169.0 MB for 0.825 TFLOP (operands stream from L2, the output is
#     written)
NCU_UPDATE_BYTES_PER_WEIGHT = (771.3e6 + 394.4e6 + 6.0e6) / 192937984
NCU_GEMM_BYTES_PER_FLOP = 169.0e6 / (2.0 * 8192 * 12288 * 4096)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=16 * 4096)
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--cpu-tokens", type=int, default=4096, help="tokens of the bounded CPU sample")
    ap.add_argument("--extras", type=int, default=1, choices=[0, 1],
                    help="1: after the step measurements also run the cuBLASLt comparison, the 32B-class GEMM sweep and "
                         "the MMA-only ceiling; 0: skip them")
    ap.add_argument("--parallel", default="auto", choices=["auto", "column", "token"],
                    help="exchange pattern of the N-sharded weights at N > 1")
    ap.add_argument("--overlap", type=int, default=1, choices=[0, 1],
                    help="1: the optimizer issues its updates on a side stream (Lattice(overlap=True)); 0: in line")
    ap.add_argument("--hook-batch", type=int, default=7,
                    help="gradients the optimizer's backward hooks collect before their updates go out as one batch "
                         "(Lattice(hook_batch=...)); 7 = the projections of one layer, 1 = every parameter on its own")
    ap.add_argument("--whole-colnorm", type=int, default=0, choices=[0, 1],
                    help="N > 1: 1 = the colnorm statistics cover the whole weight (Lattice(shard_group=...): the ranks "
                         "exchange their 128-row panel sums and reproduce the unsharded update bit for bit); 0 = every "
                         "row shard is normalised on its own, without communication")
    ap.add_argument("--match-unsharded", type=int, default=0, choices=[0, 1],
                    help="N > 1, column-parallel: 1 = gradient columns are quantized with the unsharded tensor's scale "
                         "and rounding draws (parallel.MATCH_UNSHARDED), which with --whole-colnorm 1 leaves the weights "
                         "of the one-GPU step")
    ap.add_argument("--kernel-summary", default=None, metavar="FILE",
                    help="after the measurements, run 2 more steps under torch.profiler on rank 0 and write per-kernel "
                         "launch counts and device time (text) to FILE")
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class Clocks:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------------- CPU arm

FULL_FLOPS = lambda tokens, layers: sum(6.0 * tokens * N * K for _, N, K in LAYER) * layers      # noqa: E731
FULL_WEIGHTS = lambda layers: sum(N * K for _, N, K in LAYER) * layers                            # noqa: E731


def _host_threads() -> int:
    """All host threads this process may use (torch.distributed.run exports OMP_NUM_THREADS=1 to its workers: the
    thread counts are set explicitly, after import)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def _reference_package():
    """The reference's own Python package when oracle/stage_reference.py staged it at build time, else None."""
    ref = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.isfile(os.path.join(ref, "bitlattice", "__init__.py")):
        return None
    if ref not in sys.path:
        sys.path.insert(0, ref)
    try:
        import bitlattice
        return bitlattice
    except Exception as ex:                          # a dependency of the package missing on this machine
        sys.stderr.write(f"staged reference package not importable ({type(ex).__name__}: {ex}); timing the C port\n")
        return None


class CpuSample:
    """One q-projection (4096 x 4096 NVFP4 weight) on `tokens` tokens on the host cores: exact-route forward + dgrad +
    wgrad (dequantize to bf16, bf16 GEMMs) and one lattice update with the workload's optimizer settings. `step()`
    returns (seconds of the three GEMMs, seconds of the update). kind 'reference': the reference's own
    F.linear / backward / bitlattice.optim.Lattice.step(); kind 'port': the C restatement of the same arithmetic."""

    N = K = 4096

    def __init__(self, tokens: int):
        import torch
        self.tokens = tokens
        self.threads = _host_threads()
        torch.set_num_threads(self.threads)
        self.torch = torch
        g = torch.Generator().manual_seed(0)
        w = torch.randn(self.N, self.K, generator=g) * 0.02
        self.x = torch.randn(tokens, self.K, generator=g).to(torch.bfloat16)
        self.gy = (torch.randn(tokens, self.N, generator=g) * 1e-2).to(torch.bfloat16)
        rb = _reference_package()
        if rb is not None:
            self.kind = "reference"
            self.p = torch.nn.Parameter(rb.LatticeTensor.from_float(w, "nvfp4", method="rtn", dtype=torch.bfloat16))
            self.opt = rb.optim.Lattice([self.p], **OPT)
        else:
            import numpy as np
            import oracle
            oracle.set_num_threads(self.threads)
            self.kind, self.np, self.oracle = "port", np, oracle
            self.codes, self.scales, self.gs = oracle.quantize_rows(w.numpy(), None, "rtn")
            self.phase = np.zeros((self.N, self.K // 2), np.uint8)
            self.nstep = 0
        self.flops = 6.0 * tokens * self.N * self.K
        self.weights = self.N * self.K

    def describe(self) -> str:
        how = ("the reference's own Python package on CPU: F.linear exact route + backward, bitlattice.optim.Lattice.step()"
               if self.kind == "reference" else "C restatement of the reference's CPU path (oracle/bl_oracle.c)")
        return (f"one q-projection 4096x4096 at {self.tokens} tokens, fwd+dgrad+wgrad + colnorm lattice update, {how}; "
                "extrapolated to the workload: GEMM seconds by flops, update seconds by weights")

    def step(self):
        torch = self.torch
        if self.kind == "reference":
            x = self.x.clone().requires_grad_(True)
            t0 = time.perf_counter()
            y = torch.nn.functional.linear(x, self.p)
            y.backward(self.gy)
            t1 = time.perf_counter()
            self.opt.step()
            self.opt.zero_grad()
            t2 = time.perf_counter()
            return t1 - t0, t2 - t1
        np, oracle = self.np, self.oracle
        bits = lambda t: t.contiguous().view(torch.int16).numpy().view(np.uint16)      # noqa: E731
        t0 = time.perf_counter()
        wd = torch.from_numpy(oracle.dequantize(self.codes, self.scales, self.gs)).to(torch.bfloat16)
        y = oracle.gemm_bf16_nt(bits(self.x), bits(wd))                                  # [M, N]
        gx = oracle.gemm_bf16_nt(bits(self.gy), bits(wd.t()))                            # [M, K]
        gw = oracle.gemm_bf16_nt(bits(self.gy.t()), bits(self.x.t()))                    # [N, K]
        del y, gx
        t1 = time.perf_counter()
        G = torch.from_numpy(gw).to(torch.bfloat16).float().numpy()
        D, _ = oracle.direction(G, "colnorm", 1.0)
        self.nstep += 1
        self.codes, self.phase, self.scales = oracle.lattice_step(
            self.codes, self.phase, self.scales, self.gs, D, lr=OPT["lr"], phase_bits=4, rounding="sr",
            seed=OPT["seed"], step=self.nstep, scale_rule="fit", trust=0.1, trust_lr=0.0)
        t2 = time.perf_counter()
        return t1 - t0, t2 - t1

    def extrapolate(self, t_gemm: float, t_update: float, tokens: int, layers: int):
        """Seconds of one full workload step on these host cores and the two factors used."""
        fg = FULL_FLOPS(tokens, layers) / self.flops
        fu = FULL_WEIGHTS(layers) / self.weights
        return t_gemm * fg + t_update * fu, fg, fu


def cpu_baseline(a, steps: int, warmup: int) -> dict:
    """Times `steps` sample steps after `warmup`, returns the JSON fields of the CPU arm."""
    smp = CpuSample(a.cpu_tokens)
    for _ in range(warmup):
        smp.step()
    ts = [smp.step() for _ in range(max(steps, 1))]
    tg = sum(t[0] for t in ts) / len(ts)
    tu = sum(t[1] for t in ts) / len(ts)
    full_s, fg, fu = smp.extrapolate(tg, tu, a.tokens, a.layers)
    val = FULL_FLOPS(a.tokens, a.layers) / full_s / 1e12
    return {"value": val, "unit": "TFLOP/s", "cores": smp.threads, "kind": smp.kind, "sample": smp.describe(),
            "sample_gemm_s": tg, "sample_update_s": tu, "sample_gemm_tflops": smp.flops / tg / 1e12,
            "sample_update_mweights_per_s": smp.weights / tu / 1e6, "extrapolation": {"gemm_by_flops": fg,
                                                                                       "update_by_weights": fu},
            "ms_per_step_extrapolated": full_s * 1e3, "ms_per_sample_step": (tg + tu) * 1e3}


def run_reference(a):
    """`--impl reference`: the reference's own CPU implementation of the path on this machine's host cores (all of
    them), each step a bounded sample of the workload. Rank 0 alone works; the other ranks exit at once."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cb = cpu_baseline(a, a.steps, max(a.warmup, 0))
    print(json.dumps({
        "impl": "reference", "metric": "nvfp4_linear_fwd_bwd_tflops", "value": cb["value"], "unit": "TFLOP/s",
        "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup, "ms_per_step": cb["ms_per_sample_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16 (CPU exact route: dequantize to bf16, fp32 accumulate)", "data": "synthetic",
        "config": {"workload": "cfg4_8b_linear_stack", "layers": a.layers, "tokens": a.tokens,
                   "sample": cb["sample"], "update": OPT},
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------------------------------- GPU arm

def run_ours(a):
    import torch
    import torch.distributed as dist
    import bitlattice_b200 as bl
    from bitlattice_b200 import _C, backend
    from bitlattice_b200.parallel import GatheredWeights, column_parallel_linears, shard_rows, token_parallel_linears

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    # backward (and the update hooks) on the calling thread: with a few hundred launches per layer the hand-over to
    # autograd's device thread and back costs more host time than it hides
    torch.autograd.set_multithreading_enabled(False)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    M = a.tokens
    assert M % (world * 128) == 0, "tokens must split evenly over the ranks in multiples of 128"
    Ms = M // world

    # weights: every rank draws the full matrix from the same seed, quantizes it (one per-tensor scale) and keeps
    # its row shard
    params, meta = [], []
    for layer in range(a.layers):
        for i, (name, N, K) in enumerate(LAYER):
            gen = torch.Generator(device=dev).manual_seed(1000 * layer + i)
            wd = torch.randn(N, K, device=dev, generator=gen) * 0.02
            w = bl.LatticeTensor.from_float(wd, "nvfp4", method="rtn", dtype=torch.bfloat16)
            del wd
            if world > 1:
                w = shard_rows(w, rank, world)
            p = torch.nn.Parameter(w)
            params.append(p)
            meta.append((name, N, K))
    group = dist.group.WORLD if world > 1 else None
    shard_group = group if a.whole_colnorm else None
    if a.match_unsharded:
        from bitlattice_b200 import parallel
        parallel.MATCH_UNSHARDED = True
    opt = bl.Lattice(params, fused_backward=True, overlap=bool(a.overlap), hook_batch=a.hook_batch, hook_flush="reader",
                     shard_group=shard_group, **OPT)
    flops = sum(6.0 * M * N * K for _, N, K in meta)
    weights = sum(N * K for _, N, K in meta)
    # bytes crossing NVLink per step and rank, to pick the pattern: activations (column) against weights (token)
    moved = {"column": sum(3.125 * M * K for _, N, K in meta), "token": sum(3.125 * N * K for _, N, K in meta)}
    mode = a.parallel if a.parallel != "auto" else min(moved, key=moved.get)
    backend.set_sr_seed(1 + (rank << 20))               # ranks draw different stochastic-rounding streams
    copy_stream = torch.cuda.Stream(device=dev)
    order = [[params[li * len(LAYER) + INDEX[n]] for n in names] for li in range(a.layers) for names in GROUPS]

    def measure(mode, steps, warmup, clocks=None, summary_to=None):
        """Warm up, time `steps` steps with inputs resident in HBM, then the same end to end from pinned host memory."""
        # inputs: this rank's tokens of x per distinct K; gy as the layer's output is laid out under `mode`
        gen = torch.Generator(device=dev).manual_seed(7 + rank)
        xs = {name: torch.randn(Ms, K, device=dev, generator=gen).to(torch.bfloat16) for name, K in INPUT_WIDTH.items()}
        gshape = (lambda N: (M, N // world)) if mode == "column" else (lambda N: (Ms, N))
        gys = {N: (torch.randn(*gshape(N), device=dev, generator=gen) * 1e-2).to(torch.bfloat16)
               for N in (4096, 1024, 12288)}
        host = {k: v.cpu().pin_memory() for k, v in {**{("x", name): t for name, t in xs.items()},
                                                     **{("g", N): t for N, t in gys.items()}}.items()}
        h2d_bytes = sum(t.numel() * t.element_size() for t in host.values())
        gathered = GatheredWeights(group, limit_bytes=1 << 30) if mode == "token" and world > 1 else None

        # End to end, the inputs of step i + 1 are copied from pinned host memory on a second stream while step i
        # computes (two sets of device buffers); the first step's copy has nothing to hide behind.
        sets = [(xs, gys)]

        def copy_in(k):
            while len(sets) <= k:
                sets.append(({n: torch.empty_like(t) for n, t in xs.items()},
                             {n: torch.empty_like(t) for n, t in gys.items()}))
            with torch.cuda.stream(copy_stream):
                for name, t in sets[k][0].items():
                    t.copy_(host[("x", name)], non_blocking=True)
                for N, t in sets[k][1].items():
                    t.copy_(host[("g", N)], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copy_stream)
            return ev

        def step(from_host: bool, bufs=None):
            cur_x, cur_g = bufs or sets[0]
            check = torch.zeros((), device=dev)
            with bl.compute("fp4_all"):
                for li in range(a.layers):
                    xin = {name: t.detach().requires_grad_(True) for name, t in cur_x.items()}
                    for gi, names in enumerate(GROUPS):    # forward + backward of the projections sharing an input
                        ps = order[li * len(GROUPS) + gi]
                        if gathered is not None:
                            # the next group's weights are gathered while this group computes (after the last
                            # group: the first group of the next step; the gather waits for that group's update)
                            gathered.prefetch(order[(li * len(GROUPS) + gi + 1) % len(order)])
                            ys = token_parallel_linears(xin[INPUT_OF[names[0]]], ps, gathered)
                        else:
                            ys = column_parallel_linears(xin[INPUT_OF[names[0]]], ps, group)
                        torch.autograd.backward(ys, [cur_g[SHAPE[n][0]] for n in names])
                    if from_host:
                        check = check + xin["attn_in"].grad[0, :8].float().sum()
            opt.step()
            return float(check.item()) if from_host else 0.0      # the device -> host read of the step's result

        def run_steps(n, from_host):
            if not from_host:
                for _ in range(n):
                    step(False)
                return
            ev = copy_in(0)
            for i in range(n):
                torch.cuda.current_stream().wait_event(ev)
                if i + 1 < n:
                    ev = copy_in((i + 1) % 2)               # safe: step i - 1, the last user of that set, has ended
                step(True, sets[i % 2])

        def timed(n, from_host):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            run_steps(n, from_host)
            e.record()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            t = torch.tensor([s.elapsed_time(e)], device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t.item() / 1e3

        for _ in range(warmup):
            step(False)
        if clocks is not None:
            clocks.start()
        _C.Counters.reset(timed={"bl_nvfp4_gemm", "bl_nvfp4_gemm_accumulate", "bl_nvfp4_lattice_update",
                                 "bl_nvfp4_lattice_update_many"})
        secs = timed(steps, False)
        r = {"secs": secs, "steps": steps, "launches": _C.Counters.launches, "h2d_bytes": h2d_bytes}
        g1, g2 = _C.Counters.elapsed_ms("bl_nvfp4_gemm"), _C.Counters.elapsed_ms("bl_nvfp4_gemm_accumulate")
        r["gemm_ms"], r["gemm_calls"] = g1[0] + g2[0], g1[1] + g2[1]      # every GEMM launch, accumulating ones too
        u1, u2 = _C.Counters.elapsed_ms("bl_nvfp4_lattice_update"), _C.Counters.elapsed_ms("bl_nvfp4_lattice_update_many")
        r["upd_ms"], r["upd_calls"] = u1[0] + u2[0], u1[1] + u2[1]
        _C.Counters.reset()
        r["clocks"] = clocks.stop() if clocks is not None else None
        run_steps(2, True)
        r["e2e_steps"] = max(2, min(steps, 5))
        r["e2e_secs"] = timed(r["e2e_steps"], True)
        if summary_to:
            kernel_summary(lambda: run_steps(2, False), summary_to)
        return r

    def kernel_summary(run, path):
        """Per-kernel launch counts and device time of `run()` from torch.profiler (CUPTI), written by rank 0. Times
        under a profiler are for shares and overlap, never for throughput."""
        from torch.profiler import ProfilerActivity, profile
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            run()
            torch.cuda.synchronize()
        if rank != 0:
            return
        rows, spans = {}, []
        for e in prof.events():
            if e.device_type != torch.autograd.DeviceType.CUDA:
                continue
            n, d = rows.get(e.name, (0, 0.0))
            rows[e.name] = (n + 1, d + e.time_range.elapsed_us())
            spans.append((e.time_range.start, e.time_range.end, e.name.startswith("nccl")))
        if not spans:
            return
        t0, t1 = min(s[0] for s in spans), max(s[1] for s in spans)
        busy, end = 0.0, t0                                   # union of the non-NCCL kernels' intervals
        for a0, a1, comm in sorted(spans):
            if comm:
                continue
            if a1 > end:
                busy += a1 - max(a0, end)
                end = a1
        with open(path, "w") as f:
            f.write(f"window {(t1 - t0) / 1e3:.2f} ms, 2 steps of {a.layers} layers, rank 0 of {world}; compute "
                    f"kernels busy {busy / 1e3:.2f} ms ({100 * busy / (t1 - t0):.1f} %)\n")
            for name, (n, d) in sorted(rows.items(), key=lambda kv: -kv[1][1]):
                f.write(f"{name[:90]:90s} n={n:5d} total {d / 1e3:9.3f} ms  avg {d / n:8.1f} us\n")

    def update_only(passes, warm):
        """The 8B-class update workload: the lattice update alone over the whole weight set (every rank its shards),
        one distinct bf16 gradient ~ N(0, 1e-3^2) per parameter resident in HBM (so that no matrix finds a gradient in
        L2 that an earlier one pulled in), nothing else on the GPU. Returns seconds per pass (max over ranks)."""
        plain = bl.Lattice(params, fused_backward=False, shard_group=shard_group, **OPT)         # in-line updates, own phase state
        gen = torch.Generator(device=dev).manual_seed(99 + rank)
        with torch.no_grad():
            for p in params:
                p.grad = (torch.randn(*p.shape, device=dev, generator=gen) * 1e-3).to(torch.bfloat16)

            def run(n):
                if world > 1:
                    dist.barrier()
                torch.cuda.synchronize()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                for _ in range(n):
                    plain.step()
                e.record()
                torch.cuda.synchronize()
                t = torch.tensor([s.elapsed_time(e)], device=dev)
                if world > 1:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                return t.item() / 1e3 / n
            run(warm)
            _C.Counters.reset()
            secs = run(passes)
            launches = _C.Counters.launches // passes
            for p in params:
                p.grad = None
        return secs, launches

    def extras():
        """Measurements beside the step, on this rank's GPU: the GEMM against cuBLASLt on the workload's shapes (this
        rank's tokens), the 32B-class sweep on this rank's N-shard, and the MMA-only ceiling (a burst, and the average
        over about a second of back-to-back calls: the figure for a kernel timed inside a long step)."""
        import kernel_bench as kb
        out = {}
        burst = max(bl._ops.mma_peak_tflops(local, 16384) for _ in range(3))
        t0, vals = time.perf_counter(), []
        while time.perf_counter() - t0 < 1.0:
            vals.append(bl._ops.mma_peak_tflops(local, 16384))
        out["mma_only"] = {"burst": burst, "sustained": sum(vals[len(vals) // 2:]) / max(len(vals) - len(vals) // 2, 1),
                           "unit": "TFLOP/s", "calls": len(vals)}
        shapes = [tuple(Ms if d == 65536 else d for d in shp) for shp in kb.CFG4_GEMMS]
        out["vs_cublaslt"] = {k: {kk: (round(vv, 3) if isinstance(vv, float) else vv) for kk, vv in r.items()}
                              for k, r in kb.gemm_vs_cublaslt(shapes, reps=10).items()}
        sweep = kb.gemm32b_sweep(world=world)
        out["gemm_sweep_32b"] = {k: {kk: round(vv, 1) for kk, vv in r.items()} for k, r in sweep.items()}
        return out

    res = measure(mode, a.steps, max(a.warmup, 3), Clocks(local) if rank == 0 else None, a.kernel_summary)
    other = None
    if world > 1 and a.parallel == "auto":
        other_mode = "column" if mode == "token" else "token"
        other = measure(other_mode, max(2, a.steps // 2), 3)     # the other exchange pattern over the same storage
    upd_alone, upd_launches = update_only(3, 3)
    backend._OPERANDS.clear()
    torch.cuda.empty_cache()
    extra = extras() if a.extras else None
    status = bl._ops.gemm_status(local)
    if world > 1:
        dist.barrier()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = measured_peaks()
    per_step = res["secs"] / a.steps
    proxy_peak = 4.0 * peaks["bf16_sustained"]
    mma = extra["mma_only"] if extra else None
    fp4_peak = mma["sustained"] if mma else proxy_peak
    gemm_ms, upd_ms = res["gemm_ms"], res["upd_ms"]
    gemm_flops_rank = a.steps * flops / world                     # this rank's share of the contraction work
    gemm_tf = gemm_flops_rank / (gemm_ms / 1e3) / 1e12 if gemm_ms else None
    upd_bytes_rank = a.steps * weights * BYTES_PER_WEIGHT / world
    upd_gbs = upd_bytes_rank / (upd_ms / 1e3) / 1e9 if upd_ms else None
    upd_alone_gbs = weights * BYTES_PER_WEIGHT / upd_alone / 1e9
    names = {"column": "N-sharded weights, column-parallel compute: packed activations all-gathered, input gradients "
                       "reduce-scattered",
             "token": "N-sharded weights, token-parallel compute: packed weights all-gathered, weight-gradient "
                      "partials reduce-scattered"}
    out = {
        "metric": "nvfp4_linear_fwd_bwd_tflops", "value": flops / per_step / 1e12, "unit": "TFLOP/s",
        "n_gpus": world, "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": per_step * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3, fp32 acc)",
        "data": "synthetic",
        "config": {"workload": "cfg4_8b_linear_stack", "layers": a.layers, "tokens": M,
                   "linears_per_layer": [f"{n}:{N}x{K}" for n, N, K in LAYER],
                   "activations_per_layer": "4 distinct (q/k/v share one, gate/up share one, o and down their own)",
                   "update": OPT,
                   "parallelism": f"x{world}: {names[mode]}" if world > 1 else "single GPU",
                   "nvlink_bytes_per_step_per_rank": {k: v * (world - 1) / world for k, v in moved.items()}
                   if world > 1 else None,
                   "gradient_quantization": ("as the unsharded layer (column-parallel)" if a.match_unsharded and world > 1
                                             else "per rank"),
                   "colnorm": ("whole weight (panel sums exchanged among the shard owners)" if shard_group is not None
                               else "per row shard (no communication)") if world > 1 else "whole weight",
                   "l2": "inputs larger than L2 (weights, activations and gradients of a step exceed 126 MB)",
                   "host": "one Python thread per rank (autograd multithreading off)",
                   "updates": ("side stream (overlap=True)" if a.overlap else "in line") +
                              (f", issued {a.hook_batch} parameters at a time" if a.hook_batch > 1 else "")},
        "e2e": {"value": flops / (res["e2e_secs"] / res["e2e_steps"]) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": res["h2d_bytes"], "d2h_bytes_per_step": 4, "steps": res["e2e_steps"]},
        "gpu_launches": res["launches"],
        "gemm_error_flag": status,
        "clocks": res["clocks"],
        "whole_step": {"frac_of_mma_only_peak": flops / world / per_step / 1e12 / fp4_peak,
                       "frac_of_nominal": flops / world / per_step / 1e12 / 9000.0,
                       "note": "per-GPU whole-step TFLOP/s (GEMMs, quantizers, update) against the tensor ceilings"},
        "roofline": {"bound": "tensor", "kernel": "gemm_pair_kernel (tcgen05 mxf4nvf4, cta_group::2, 256x256 tiles)",
                     "achieved": gemm_tf, "peak": fp4_peak, "unit": "TFLOP/s",
                     "frac": gemm_tf / fp4_peak if gemm_tf else None,
                     "traffic": NCU_GEMM_BYTES_PER_FLOP * gemm_flops_rank / max(res["gemm_calls"], 1),
                     "traffic_note": "bytes per average launch, scaled by flops from the ncu capture of a small case",
                     "launches": res["gemm_calls"],
                     "peak_note": ("measured on this GPU in this run: a kernel that only issues block-scaled FP4 MMAs "
                                   "(no loads, scale copies or epilogue), averaged over about a second of back-to-back "
                                   f"calls; burst {mma['burst']:.0f}" if mma else
                                   f"4 x bf16 sustained cuBLAS ({peaks['source']}); the MMA-only ceiling was not run")
                                  + f"; 4 x bf16 sustained cuBLAS ({peaks['source']}) {proxy_peak:.0f}; nominal dense "
                                    "FP4 9000",
                     "frac_of_4x_bf16_sustained": gemm_tf / proxy_peak if gemm_tf else None,
                     "frac_of_nominal": gemm_tf / 9000.0 if gemm_tf else None},
        # the update alone over the whole weight set (the 8B-class update workload): whole-job GB/s = all ranks' bytes
        # / time; `in_step` is the same kernel timed inside the step, where (with overlap) it shares the GPU with the GEMMs
        "update": {"metric": "lattice_update_hbm_gbs", "value": upd_alone_gbs, "unit": "GB/s", "n_gpus": world,
                   "per_gpu": upd_alone_gbs / world, "ms_per_pass": upd_alone * 1e3, "weights": weights,
                   "launches_per_pass": upd_launches,
                   "gradients": "one distinct bf16 tensor per parameter (none shared, none resident in L2)",
                   "bytes_per_weight": BYTES_PER_WEIGHT, "workload": f"cfg3: {a.layers} x 7 NVFP4 matrices, colnorm, 4-bit "
                   "phase, sr, scale refit (trust 0.1), sharded along N",
                   "in_step": {"value": upd_gbs, "unit": "GB/s per GPU", "calls": res["upd_calls"]},
                   "roofline": {"bound": "hbm", "achieved": upd_alone_gbs / world, "peak": peaks["hbm"],
                                "unit": "GB/s", "frac": upd_alone_gbs / world / peaks["hbm"],
                                "traffic": NCU_UPDATE_BYTES_PER_WEIGHT * weights / world,
                                "traffic_note": "bytes per pass and GPU (update, column statistics and their "
                                                "reduction), scaled by weights from the ncu capture of one "
                                                "layer's seven matrices updated as a batch",
                                "peak_note": f"per GPU against copy bandwidth ({peaks['source']}); nominal 8000"}},
    }
    if extra:
        out["vs_cublaslt"] = extra["vs_cublaslt"]
        out["gemm_sweep_32b"] = {"unit": "TFLOP/s per GPU", "sharding": f"N / {world}", "peak": fp4_peak,
                                 "cases": extra["gemm_sweep_32b"]}
        out["mma_only"] = mma
    if other is not None:
        out["other_parallelism"] = {"parallelism": names[other_mode], "steps": other["steps"], "warmup": 3,
                                    "value": flops / (other["secs"] / other["steps"]) / 1e12, "unit": "TFLOP/s",
                                    "ms_per_step": other["secs"] / other["steps"] * 1e3,
                                    "e2e": flops / (other["e2e_secs"] / other["e2e_steps"]) / 1e12,
                                    "gemm_tflops_per_gpu": (other["steps"] * flops / world / (other["gemm_ms"] / 1e3)
                                                            / 1e12 if other["gemm_ms"] else None)}
    if world == 1:
        out["cpu_baseline"] = cpu_baseline(a, 3, 1)
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)
