"""Per-kernel timings of the library on one GPU, next to the library kernels the reference would call.

    python -m bitlattice_b200.kernel_bench [gemm] [quant] [update] [swiglu]

CUDA events on the current stream, 3 warm-up calls, inputs larger than L2 where the shape allows. Prints one line per
case: GEMM TFLOP/s for each of this library's kernels and for ``torch._scaled_mm`` on the same NVFP4 operands
(cuBLASLt, what the reference's ``fp4_mm`` runs, bitlattice/backend.py:267-290) with the relative difference of the
two outputs; quantizer microseconds per tensor; update GB/s on the algorithmic 3.125 + cb/4 bytes per weight; SwiGLU
GB/s on its 6 (forward) and 10 (backward) bytes per element.
"""
from __future__ import annotations

import sys

import torch

from . import _ops
from .backend import _hadamard16

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


def gemm():
    gen = torch.Generator(device=DEV).manual_seed(0)
    one = torch.ones(1, device=DEV)
    shapes = [(8192, 3072, 1024), (8192, 1024, 3072), (8192, 8192, 8192), (16384, 12288, 4096), (65536, 4096, 4096),
              (65536, 1024, 4096), (65536, 12288, 4096), (65536, 4096, 12288), (4096, 4096, 65536),
              (12288, 4096, 65536)]
    for M, N, K in shapes:
        a, asf = _operand(M, K, gen)
        b, bsf = _operand(N, K, gen)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        msg = f"gemm {M}x{N}x{K}:"
        try:
            for kern in ("pair", "persistent", "tile"):
                _ops.gemm_select(kern)
                t = timeit(lambda: _ops.nvfp4_gemm(a, asf, one, b, bsf, one, out=out))
                msg += f" {kern} {2 * M * N * K / t / 1e12:.0f}"
        finally:
            _ops.gemm_select("auto")
        try:
            fp4 = torch.float4_e2m1fn_x2
            f = lambda: torch._scaled_mm(a.view(fp4), b.view(fp4).t(), scale_a=asf.view(torch.float8_e4m3fn),  # noqa: E731
                                         scale_b=bsf.view(torch.float8_e4m3fn), out_dtype=torch.bfloat16)
            y = f()
            t2 = timeit(f)
            err = ((y.float() - out.float()).norm() / out.float().norm()).item()
            msg += f" | torch._scaled_mm {2 * M * N * K / t2 / 1e12:.0f} TFLOP/s, relative difference {err:.1e}"
        except Exception as ex:                       # the torch build may lack the NVFP4 path
            msg += f" | torch._scaled_mm unavailable: {str(ex)[:80]}"
        print(msg + "  (TFLOP/s)", flush=True)
    print("gemm error flag", _ops.gemm_status(0))


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


if __name__ == "__main__":
    which = sys.argv[1:] or ["gemm", "quant", "update", "swiglu"]
    for name in which:
        {"gemm": gemm, "quant": quant, "update": update, "swiglu": swiglu}[name]()
