"""Per-kernel timings of the library on one GPU, next to the library kernels the reference would call.

    python kernel_bench.py [gemm] [gemm32b] [mma_peak] [quant] [update] [swiglu]

CUDA events on the current stream, 3 warm-up calls, inputs larger than L2 where the shape allows. Prints one line per
case: GEMM TFLOP/s for each of this library's kernels and for ``torch._scaled_mm`` on the same NVFP4 operands
(cuBLASLt, what the reference's ``fp4_mm`` runs, bitlattice/backend.py:267-290) with the relative difference of the
two outputs; quantizer microseconds per tensor; update GB/s on the algorithmic 3.125 + cb/4 bytes per weight; SwiGLU
GB/s on its 6 (forward) and 10 (backward) bytes per element.
"""
from __future__ import annotations

import sys

import torch

import os

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from bitlattice_b200 import _ops  # noqa: E402
from bitlattice_b200.backend import _hadamard16  # noqa: E402

DEV = "cuda"


def timeit(fn, reps=10, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(reps):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / reps * 1e-3


def _operand(rows, K, gen):
    codes = torch.randint(0, 256, (rows, K // 2), device=DEV, dtype=torch.uint8, generator=gen)
    sf = torch.randint(40, 72, (rows, K // 16), device=DEV, dtype=torch.uint8, generator=gen)
    return codes, _ops.to_blocked(sf)


CFG4_GEMMS = [(65536, 4096, 4096), (65536, 1024, 4096), (65536, 12288, 4096), (65536, 4096, 12288),
              (4096, 4096, 65536), (1024, 4096, 65536), (12288, 4096, 65536)]


def scaled_mm(a, asf, b, bsf):
    """torch._scaled_mm (cuBLASLt) on NVFP4 operands with blocked scales: the reference's Blackwell GEMM
    (bitlattice/backend.py:267-290)."""
    fp4 = torch.float4_e2m1fn_x2
    return torch._scaled_mm(a.view(fp4), b.view(fp4).t(), scale_a=asf.view(torch.float8_e4m3fn),
                            scale_b=bsf.view(torch.float8_e4m3fn), out_dtype=torch.bfloat16)


def gemm_vs_cublaslt(shapes=CFG4_GEMMS, reps=10, kernels=("auto",)):
    """For each (M, N, K): TFLOP/s of this library's GEMM (per kernel in ``kernels``) and of cuBLASLt on the same
    operands, the ratio auto / cuBLASLt, and whether the two outputs are bit-identical."""
    gen = torch.Generator(device=DEV).manual_seed(0)
    one = torch.ones(1, device=DEV)
    rows = {}
    for M, N, K in shapes:
        a, asf = _operand(M, K, gen)
        b, bsf = _operand(N, K, gen)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        r = {}
        try:
            for kern in kernels:
                _ops.gemm_select(kern)
                t = timeit(lambda: _ops.nvfp4_gemm(a, asf, one, b, bsf, one, out=out), reps=reps)
                r[kern] = 2 * M * N * K / t / 1e12
        finally:
            _ops.gemm_select("auto")
        try:
            y = scaled_mm(a, asf, b, bsf)
            t2 = timeit(lambda: scaled_mm(a, asf, b, bsf), reps=reps)
            r["cublaslt"] = 2 * M * N * K / t2 / 1e12
            r["identical"] = bool(torch.equal(y, out))
            r["ratio"] = r[kernels[0]] / r["cublaslt"]
        except Exception as ex:                       # the torch build may lack the NVFP4 path
            r["cublaslt"] = None
            r["error"] = str(ex)[:80]
        rows[f"{M}x{N}x{K}"] = r
        del a, asf, b, bsf, out
    return rows


def gemm():
    shapes = [(8192, 3072, 1024), (8192, 1024, 3072), (8192, 8192, 8192), (16384, 12288, 4096)] + CFG4_GEMMS
    for name, r in gemm_vs_cublaslt(shapes, kernels=("pair", "persistent", "tile")).items():
        msg = f"gemm {name}: pair {r['pair']:.0f} persistent {r['persistent']:.0f} tile {r['tile']:.0f}"
        if r.get("cublaslt"):
            msg += f" | torch._scaled_mm {r['cublaslt']:.0f} TFLOP/s, identical bits: {r['identical']}"
        else:
            msg += f" | torch._scaled_mm unavailable: {r.get('error')}"
        print(msg + "  (TFLOP/s)", flush=True)
    print("gemm error flag", _ops.gemm_status(0))


def gemm32b_sweep(world=1, tokens=(1024, 4096, 16384, 65536), reps=5, with_cublaslt=False):
    """The 32B-class sweep (hidden 5120, intermediate 25600): for (K, N) in {(5120, 25600), (25600, 5120),
    (5120, 5120)} and M tokens, the three GEMMs of a linear layer whose weight is sharded along N over ``world`` GPUs
    (this GPU's shard: N / world rows): forward [M, N/p] = A[M, K] W^T, input gradient [M, K] contracting over N/p,
    weight gradient [N/p, K] contracting over M. Returns {case: {fwd, dgrad, wgrad, all: TFLOP/s per GPU}}."""
    gen = torch.Generator(device=DEV).manual_seed(0)
    one = torch.ones(1, device=DEV)
    res = {}
    for K, N in ((5120, 25600), (25600, 5120), (5120, 5120)):
        n = N // world
        for M in tokens:
            x, xsf = _operand(M, K, gen)
            w, wsf = _operand(n, K, gen)
            gq, gsf = _operand(M, n, gen)
            wt, wtsf = _operand(K, n, gen)
            gt, gtsf = _operand(n, M, gen)
            xt, xtsf = _operand(K, M, gen)
            cases = {"fwd": (x, xsf, w, wsf, M, n, K), "dgrad": (gq, gsf, wt, wtsf, M, K, n),
                     "wgrad": (gt, gtsf, xt, xtsf, n, K, M)}
            r, total_t = {}, 0.0
            for name, (a, asf, b, bsf, m_, n_, k_) in cases.items():
                out = torch.empty(m_, n_, dtype=torch.bfloat16, device=DEV)
                t = timeit(lambda: _ops.nvfp4_gemm(a, asf, one, b, bsf, one, out=out), reps=reps)
                r[name] = 2.0 * m_ * n_ * k_ / t / 1e12
                total_t += t
                if with_cublaslt:
                    try:
                        t2 = timeit(lambda: scaled_mm(a, asf, b, bsf), reps=reps)
                        r[name + "_cublaslt"] = 2.0 * m_ * n_ * k_ / t2 / 1e12
                    except Exception:
                        r[name + "_cublaslt"] = None
                del out
            r["all"] = 6.0 * M * n * K / total_t / 1e12
            res[f"K{K}_N{N}_M{M}"] = r
            del x, xsf, w, wsf, gq, gsf, wt, wtsf, gt, gtsf, xt, xtsf
    return res


def gemm32b():
    for case, r in gemm32b_sweep(with_cublaslt=True).items():
        print(f"gemm32b {case}: fwd {r['fwd']:.0f} ({r.get('fwd_cublaslt') or 0:.0f}) dgrad {r['dgrad']:.0f} "
              f"({r.get('dgrad_cublaslt') or 0:.0f}) wgrad {r['wgrad']:.0f} ({r.get('wgrad_cublaslt') or 0:.0f}) "
              f"all three {r['all']:.0f} TFLOP/s (cuBLASLt in brackets)", flush=True)
    print("gemm error flag", _ops.gemm_status(0))


def mma_peak():
    """The tensor-pipe ceiling: MMAs only, no loads / scale copies / epilogue (bl_selftest_mma_peak)."""
    for n in (256, 128):
        vals = [_ops.mma_peak_tflops(0, iters, n) for iters in (1024, 4096, 16384, 16384, 16384)]
        print(f"mma-only block-scaled FP4 (128 x {n} x 64 MMAs on resident tiles), TFLOP/s per call: " +
              ", ".join(f"{v:.0f}" for v in vals), flush=True)
    vals = [_ops.mma_peak_tflops(0, iters, 1256) for iters in (1024, 4096, 16384, 16384, 16384)]
    print("the same with the 12 scale copies of every k-tile issued in order before its MMAs, TFLOP/s per call: " +
          ", ".join(f"{v:.0f}" for v in vals), flush=True)


def quant():
    H = _hadamard16(torch.device(DEV), torch.float32)
    for M, K in [(65536, 4096), (65536, 12288), (65536, 1024)]:
        x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
        am = _ops.amax_global(x)
        g = am[1:2]
        cases = [("amax", lambda: _ops.amax_global(x)),
                 ("rows rtn", lambda: _ops.quantize_nvfp4(x, g, blocked=True)),
                 ("rows 4over6", lambda: _ops.quantize_nvfp4_4over6(x, am[3:4], "mse", blocked=True)),
                 ("rows sr", lambda: _ops.quantize_nvfp4(x, g, seed=3, blocked=True)),
                 ("transposed rtn", lambda: _ops.quantize_nvfp4_t(x, H, -1, 0, g * 4, blocked=True)),
                 ("transposed sr", lambda: _ops.quantize_nvfp4_t(x, H, 5, 0, g * 4, blocked=True))]
        for name, fn in cases:
            t = timeit(fn, reps=5)
            print(f"quantize {M}x{K} bf16 {name}: {t * 1e6:.0f} us, {M * K * 2 / t / 1e9:.0f} GB/s of input", flush=True)


def update():
    gen = torch.Generator(device=DEV).manual_seed(0)
    for rows, cols in [(12288, 4096), (4096, 12288), (4096, 4096), (1024, 4096)]:
        codes = torch.randint(0, 256, (rows, cols // 2), device=DEV, dtype=torch.uint8, generator=gen)
        phase = torch.zeros(rows, cols // 2, device=DEV, dtype=torch.uint8)
        scales = torch.randint(40, 72, (rows, cols // 16), device=DEV, dtype=torch.uint8, generator=gen)
        gs = torch.full((1,), 1e-3, device=DEV)
        G = (torch.randn(rows, cols, device=DEV, generator=gen) * 1e-3).to(torch.bfloat16)
        for direction in ("sign", "colnorm", "raw"):
            for rule in ("fit", "fixed"):
                kw = dict(lr=3e-3, weight_decay=0.0, phase_bits=4, phase_cb=4, rounding="sr", seed=1, step=1, strata=16,
                          scale_rule=rule, trust=0.1, trust_lr=0.0, direction=direction)
                t = timeit(lambda: _ops.lattice_update(codes, phase, scales, gs, None, G, "nvfp4", rows, cols, **kw),
                           reps=20, warm=5)
                print(f"update {rows}x{cols} {direction} {rule}: {t * 1e6:.1f} us, {rows * cols * 4.125 / t / 1e9:.0f} "
                      f"GB/s (4.125 B/weight)", flush=True)


def swiglu():
    for M, I in [(65536, 12288), (8192, 3072)]:
        g = torch.randn(M, I, device=DEV).to(torch.bfloat16)
        u, da = torch.randn_like(g), torch.randn_like(g)
        t = timeit(lambda: _ops.swiglu_fwd(g, u), reps=5)
        print(f"swiglu forward {M}x{I}: {t * 1e6:.0f} us, {6 * M * I / t / 1e9:.0f} GB/s", flush=True)
        t = timeit(lambda: _ops.swiglu_bwd(g, u, da), reps=5)
        print(f"swiglu backward {M}x{I}: {t * 1e6:.0f} us, {10 * M * I / t / 1e9:.0f} GB/s", flush=True)


def recipes():
    """The general quantizer of the 128-rotation recipes (amax pass + quantization pass per call) and one linear
    layer, forward + backward, under every FP4 recipe (65,536 tokens, 4096 -> 4096)."""
    import bitlattice_b200 as bl
    x = torch.randn(65536, 4096, device=DEV).to(torch.bfloat16)
    for name, kw in [("rows rtn 4/6", dict(four_over_six=True)),
                     ("rows eden rotated", dict(mode="eden", rotate=True, seed=1)),
                     ("rows sr rotated", dict(mode="sr", rotate=True, seed=1)),
                     ("transposed eden rotated", dict(mode="eden", rotate=True, seed=1, transpose=True, pow2=True))]:
        t = timeit(lambda: _ops.nvfp4_quantize_general(x, blocked=True, **kw))
        print(f"general quantizer 65536x4096 bf16 {name}: {t * 1e6:.0f} us, {x.numel() * 2 / t / 1e9:.0f} GB/s of input",
              flush=True)
    w = torch.nn.Parameter(bl.LatticeTensor.from_float(torch.randn(4096, 4096, device=DEV) * 0.02, "nvfp4",
                                                       method="rtn", dtype=torch.bfloat16))
    gy = (torch.randn(65536, 4096, device=DEV) * 1e-2).to(torch.bfloat16)
    for name in bl.backend.FP4_RECIPES:
        def step():
            xi = x.detach().requires_grad_(True)
            with bl.compute(bl.Compute("nvfp4", nvfp4=name)):
                torch.nn.functional.linear(xi, w).backward(gy)
            w.grad = None
        t = timeit(step, reps=5)
        print(f"linear 65536 x 4096 -> 4096 fwd+bwd, recipe {name}: {t * 1e3:.2f} ms, "
              f"{6.0 * 65536 * 4096 * 4096 / t / 1e12:.0f} TFLOP/s", flush=True)
    print("gemm error flag", _ops.gemm_status(0), flush=True)


if __name__ == "__main__":
    which = sys.argv[1:] or ["mma_peak", "gemm", "gemm32b", "quant", "update", "swiglu", "recipes"]
    for name in which:
        {"gemm": gemm, "gemm32b": gemm32b, "mma_peak": mma_peak, "quant": quant, "update": update,
         "swiglu": swiglu, "recipes": recipes}[name]()
