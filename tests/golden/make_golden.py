"""Generates the golden fixtures in this folder from the reference's own pure-PyTorch functions.

Run where the reference checkout is importable (it is read-only, so no bytecode is written):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference [file names ...]

Every array below is an OUTPUT OF THE REFERENCE (bitlattice.reference, bitlattice.fp4ref, bitlattice._ops CPU
fallbacks, bitlattice.optim.Lattice on CPU) on seeded inputs; the inputs are stored next to them. The oracle and the
host logic of this repository are checked against these files, which travel with the repository.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("BITLATTICE_REFERENCE", "")
sys.dont_write_bytecode = True
sys.path.insert(0, REF)

import bitlattice as bl  # noqa: E402
from bitlattice import _ops, formats as F, fp4ref, reference as R  # noqa: E402
from bitlattice.packing import pack  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
FMT = F.get("nvfp4")


def gen(seed):
    return torch.Generator().manual_seed(seed)


def u8(t):
    return t.contiguous().view(torch.uint8).numpy().copy()


def values_to_codes(vals: torch.Tensor) -> torch.Tensor:
    """Signed E2M1 levels -> packed codes (zero is +0), low nibble first."""
    mag = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    m = torch.bucketize(vals.abs(), mag, right=True) - 1
    code = torch.where((vals < 0) & (m > 0), m + 8, m)
    return pack(code, 4)


def hash_cases():
    out = {}
    for i, (n, seed, step, off) in enumerate([(64, 0, 0, 0), (64, 7, 3, 0), (64, 0xFFFFFFFF, 12345, 1 << 33),
                                              (64, 1234 + 7919, 1, 4096 * 1024)]):
        out[f"u{i}"] = R.hash_uniform(n, seed, step, "cpu", off).numpy()
        out[f"args{i}"] = np.array([n, seed, step, off], dtype=np.int64)
    for mode in ("sr", "strat", "rtn"):
        out[f"round_{mode}"] = R.rounding_u(64, 11, 5, "cpu", mode, 16).numpy()
    return out


def e4m3_cases():
    v = torch.cat([torch.logspace(-12, 3, 400, base=10.0), torch.tensor([2.0 ** -9, 2.0 ** -6, 448.0, 500.0, 1e-30]),
                   torch.arange(1, 257).float() * 2.0 ** -10 * 1.5])
    enc = R.encode_scales(v, FMT.scale)
    return {"v": v.numpy(), "bytes": u8(enc), "decoded": enc.float().numpy()}


def quantize_cases():
    out = {}
    x = torch.randn(32, 128, generator=gen(1)).to(torch.bfloat16).float()
    # edge cases: an all-zero block, exact ties at every midpoint (block maximum 6 -> scale exactly 1 * g)
    x[0, :16] = 0.0
    q0 = R.quantize(x, FMT, "rtn")
    g = q0.global_scale.item()
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    x[1, :16] = ties * g * 1.0            # block scale encodes to 1.0 exactly when amax/6/g == 1
    q = R.quantize(x, FMT, "rtn")
    out["rtn_x"] = x.numpy()
    out["rtn_codes"], out["rtn_scales"], out["rtn_g"] = q.packed.numpy(), u8(q.scales), q.global_scale.numpy()
    out["rtn_deq_f32"] = R.dequantize(q, FMT, torch.float32).numpy()
    out["rtn_deq_bf16"] = R.dequantize(q, FMT, torch.bfloat16).view(torch.int16).numpy()
    # given global scale (as for the transposed re-quantization)
    q2 = R.quantize(x * 0.5, FMT, "rtn", global_scale=q.global_scale)
    out["rtng_codes"], out["rtng_scales"] = q2.packed.numpy(), u8(q2.scales)
    # stochastic rounding of a small-magnitude gradient
    gy = (torch.randn(32, 128, generator=gen(2)) * 1e-2).to(torch.bfloat16).float()
    for seed in (1, 77):
        vals, s, gg = fp4ref.quantize(gy, mode="sr", seed=seed)
        out[f"sr{seed}_codes"] = values_to_codes(vals).numpy()
        out[f"sr{seed}_scales"] = u8(s.to(torch.float8_e4m3fn))
        out[f"sr{seed}_g"] = gg.reshape(1).numpy()
    out["sr_x"] = gy.numpy()
    # blocked scale layout
    sc = torch.randint(0, 127, (200, 9), generator=gen(3), dtype=torch.uint8)
    out["blk_in"] = sc.numpy()
    out["blk_out"] = bl.backend.to_blocked(sc).numpy()
    return out


def fos_cases():
    """Four-over-six round-to-nearest quantizer of the forward activations (the '4over6' recipe): fp4ref.quantize
    with four_over_six=True, both selection criteria, bf16-valued and fp32-valued inputs, an all-zero block."""
    out = {}
    x = torch.randn(64, 256, generator=gen(11)).to(torch.bfloat16).float()
    x[0, :16] = 0.0
    xf = torch.randn(48, 128, generator=gen(12)) * 3.0
    for tag, inp in (("bf", x), ("f32", xf)):
        out[f"{tag}_x"] = inp.numpy()
        for select in ("mse", "mae"):
            vals, s, g = fp4ref.quantize(inp, mode="rtn", four_over_six=True, select=select)
            out[f"{tag}_{select}_codes"] = values_to_codes(vals).numpy()
            out[f"{tag}_{select}_scales"] = u8(s.to(torch.float8_e4m3fn))
            out[f"{tag}_{select}_g"] = g.reshape(1).numpy()
    return out


def general_cases():
    """The general quantizer (fp4ref.quantize): rows and transposed, round to nearest / stochastic / MS-EDEN, with and
    without four-over-six, with and without the 128-point rotation (MS-EDEN always rotated), on the input
    distribution of the reference's own kernel test (tests/test_nvfp4.py:22-27: per-row log-normal magnitudes, one
    outlier column, bf16). Stored: packed codes of the returned levels, scale bytes, global scale. Also the rotation
    itself and the E4M3 stochastic rounding on a value grid."""
    out = {}
    g = gen(0)
    x = torch.randn(128, 256, generator=g) * torch.exp(torch.randn(128, 1, generator=g))
    x[:, 3] *= 25
    x = x.to(torch.bfloat16).float()
    out["x"] = x.numpy()
    for transpose in (False, True):
        src = x.t().contiguous() if transpose else x
        for mode in ("rtn", "sr", "eden"):
            for fos in (False, True):
                for rotate in ((True,) if mode == "eden" else (False, True)):
                    vals, s, gg = fp4ref.quantize(src, mode=mode, four_over_six=fos, seed=11, rotate=rotate,
                                                  rotate_seed=21)
                    tag = f"{'t' if transpose else 'r'}_{mode}_{int(fos)}_{int(rotate)}"
                    out[tag + "_codes"] = values_to_codes(vals).numpy()
                    out[tag + "_scales"] = u8(s.to(torch.float8_e4m3fn))
                    out[tag + "_g"] = gg.reshape(1).numpy()
    out["rht_seed21"] = fp4ref.rht128(x[:8], 21).numpy()
    out["signs_seed21"] = fp4ref.hadamard_signs(21).numpy()
    v = torch.cat([torch.logspace(-10, 9.5, 300, base=2.0), torch.tensor([2.0 ** -9, 448.0, 500.0, 1e-4])])
    u = fp4ref.uniform_u(v.numel(), 5, "cpu")
    out["sr_e4m3_v"], out["sr_e4m3_u"] = v.numpy(), u.numpy()
    out["sr_e4m3_out"] = u8(fp4ref._sr_e4m3(v, u).to(torch.float8_e4m3fn))
    return out


def rotate_t(x: torch.Tensor, H: torch.Tensor) -> torch.Tensor:
    """x [M, K] -> rotated x^T [K, M]: every 16-block along M times H, summed sequentially over i (the order of
    csrc/act_quant.cu:110-116; products by +-0.25 are exact, so this equals the kernel's fmaf chain)."""
    xt = x.t().contiguous()
    K, M = xt.shape
    b = xt.view(K, M // 16, 16)
    acc = torch.zeros(K, M // 16, 16)
    for i in range(16):
        acc = acc + b[:, :, i:i + 1] * H[i].view(1, 1, 16)
    return acc.view(K, M)


def transposed_cases():
    out = {}
    H = bl.backend._hadamard16(torch.device("cpu"), torch.float32)
    out["H16"] = H.numpy()
    x = torch.randn(64, 96, generator=gen(4)).to(torch.bfloat16).float()
    gx = (x.abs().amax() / (6.0 * 448.0)).clamp_min(1e-12).reshape(1)
    bound = gx * 4.0
    out["t_x"], out["t_bound"] = x.numpy(), bound.numpy()
    for name, rot in (("rot", rotate_t(x, H)), ("plain", x.t().contiguous())):
        q = R.quantize(rot, FMT, "rtn", global_scale=bound)
        out[f"t_{name}_rtn_codes"], out[f"t_{name}_rtn_scales"] = q.packed.numpy(), u8(q.scales)
        vals, s, _ = fp4ref.quantize(rot, mode="sr", seed=9, global_scale=bound)
        out[f"t_{name}_sr_codes"] = values_to_codes(vals).numpy()
        out[f"t_{name}_sr_scales"] = u8(s.to(torch.float8_e4m3fn))
    # transposed re-quantization of an NVFP4 weight, values formed as (level * scale) * global
    w = torch.randn(64, 128, generator=gen(5)) * 0.02
    q = R.quantize(w, FMT, "rtn")
    raw = R.unpack(q.packed, 4, q.cols)
    lv = R.rank_level(FMT, R.raw_to_rank(FMT, raw))
    wd = lv * R.expand_groups(q.scales.float(), q.rows, q.cols, FMT.scale) * q.global_scale
    qt = R.quantize(wd.t().contiguous(), FMT, "rtn", global_scale=q.global_scale)
    out["w"], out["w_codes"], out["w_scales"], out["w_g"] = w.numpy(), q.packed.numpy(), u8(q.scales), \
        q.global_scale.numpy()
    out["wt_codes"], out["wt_scales"] = qt.packed.numpy(), u8(qt.scales)
    return out


def step_cases():
    out = {}
    w = torch.randn(16, 128, generator=gen(6)) * 0.02
    q = R.quantize(w, FMT)                                   # default method 'mse', as the reference's kernel test
    out["codes"], out["scales"], out["g"] = q.packed.numpy(), u8(q.scales), q.global_scale.numpy()
    D = torch.randn(16, 128, generator=gen(7))
    out["D"] = D.numpy()
    lr = 0.3 * R.effective_scales(q.scales, FMT.scale, q.global_scale).float().mean().item()
    out["lr"] = np.array([lr], dtype=np.float64)
    names = []
    for bits in (0, 1, 2, 3, 4, 8):
        half = 1 << max(bits - 1, 0)
        phase = torch.randint(-half, half, (16, 128), generator=gen(8 + bits), dtype=torch.int8) if bits else None
        cb = _ops.phase_container(bits)
        if bits:
            out[f"phase_in_b{bits}"] = pack(phase.to(torch.int32) & ((1 << bits) - 1), cb).numpy()
        for rule in ("fixed", "fit", "fit_latent"):
            for rounding, trust_lr in (("sr", 1.0), ("strat", 0.0), ("rtn", 0.0)):
                if rounding != "sr" and bits not in (0, 4):
                    continue
                kw = dict(lr=lr, weight_decay=0.01, phase_bits=bits, rounding=rounding, seed=7, step=3,
                          scale_rule=rule, trust=0.1 if trust_lr == 0.0 else 0.01, trust_lr=trust_lr)
                packed, scales, code = R.lattice_step_quantized(q, FMT, phase, D, **kw)
                key = f"b{bits}_{rule}_{rounding}"
                names.append(key)
                out[key + "_codes"] = packed.numpy()
                out[key + "_scales"] = u8(scales)
                if bits:
                    out[key + "_phase"] = pack(code.to(torch.int32) & ((1 << bits) - 1), cb).numpy()
    out["names"] = np.array(names)
    return out


def direction_cases():
    out = {}
    G = (torch.randn(300, 64, generator=gen(20)) * 1e-3).to(torch.bfloat16)
    G[5, 7] = 0.0
    out["G"] = G.float().numpy()
    for kind in ("raw", "sign", "colnorm"):
        for clip in (1.0, 0.25):
            out[f"{kind}_clip{clip}"] = _ops.direction(G, kind, clip=clip).numpy()
    big = torch.randn(40, 64, generator=gen(21)).to(torch.bfloat16) * 3.0
    out["G_big"] = big.float().numpy()
    out["raw_big"] = _ops.direction(big, "raw", clip=1.0).numpy()
    return out


def optimizer_cases():
    """bl.optim.Lattice on CPU: two steps per configuration, per-parameter seeds and step counters included."""
    out = {}
    names = []
    for direction, bits, rule, trust_lr in (("sign", 4, "fit", 1.0), ("raw", 2, "fit", 0.0), ("sign", 0, "fixed", 1.0),
                                            ("sign", 8, "fit_latent", 0.0)):
        ws = [torch.randn(32, 64, generator=gen(30)) * 0.02, torch.randn(16, 128, generator=gen(31)) * 0.02]
        ps = [torch.nn.Parameter(bl.LatticeTensor.from_float(w, "nvfp4", method="rtn", dtype=torch.bfloat16))
              for w in ws]
        key = f"{direction}_b{bits}_{rule}"
        names.append(key)
        for i, p in enumerate(ps):
            out[f"{key}_p{i}_codes0"], out[f"{key}_p{i}_scales0"] = p.packed.numpy().copy(), u8(p.scales)
            out[f"{key}_p{i}_g"] = p.global_scale.numpy().copy()
        opt = bl.optim.Lattice(ps, lr=3e-3, direction=direction, phase_bits=bits, scale_rule=rule, seed=1234,
                               trust=0.1, trust_lr=trust_lr)
        for s in range(2):
            for i, p in enumerate(ps):
                G = (torch.randn(p.shape, generator=gen(40 + 2 * s + i)) * 1e-2).to(torch.bfloat16)
                out[f"{key}_p{i}_G{s}"] = G.float().numpy()
                p.grad = G
            opt.step()
        for i, p in enumerate(ps):
            out[f"{key}_p{i}_codes"], out[f"{key}_p{i}_scales"] = p.packed.numpy().copy(), u8(p.scales)
            if bits:
                out[f"{key}_p{i}_phase"] = opt.state[p]["phase"].numpy().copy()
    out["names"] = np.array(names)
    return out


def momentum_cases():
    """bl.optim.Lattice on CPU with momentum='fp32' (lattice.py:396-405): three steps, so that the averaged gradient
    differs from every single one; the final momentum buffers are stored too."""
    out = {}
    names = []
    for direction, bits, rule in (("sign", 4, "fit"), ("raw", 2, "fixed")):
        ws = [torch.randn(32, 64, generator=gen(50)) * 0.02, torch.randn(16, 128, generator=gen(51)) * 0.02]
        ps = [torch.nn.Parameter(bl.LatticeTensor.from_float(w, "nvfp4", method="rtn", dtype=torch.bfloat16))
              for w in ws]
        key = f"{direction}_b{bits}_{rule}"
        names.append(key)
        for i, p in enumerate(ps):
            out[f"{key}_p{i}_codes0"], out[f"{key}_p{i}_scales0"] = p.packed.numpy().copy(), u8(p.scales)
            out[f"{key}_p{i}_g"] = p.global_scale.numpy().copy()
        opt = bl.optim.Lattice(ps, lr=3e-3, direction=direction, phase_bits=bits, scale_rule=rule, seed=4321,
                               trust=0.1, trust_lr=0.0, momentum="fp32", beta1=0.9)
        for s in range(3):
            for i, p in enumerate(ps):
                G = (torch.randn(p.shape, generator=gen(60 + 2 * s + i)) * 1e-2).to(torch.bfloat16)
                out[f"{key}_p{i}_G{s}"] = G.float().numpy()
                p.grad = G
            opt.step()
        for i, p in enumerate(ps):
            out[f"{key}_p{i}_codes"], out[f"{key}_p{i}_scales"] = p.packed.numpy().copy(), u8(p.scales)
            out[f"{key}_p{i}_phase"] = opt.state[p]["phase"].numpy().copy()
            out[f"{key}_p{i}_m"] = opt.state[p]["m"].numpy().copy()
    out["names"] = np.array(names)
    return out


def directions2_cases():
    """The reference's other directions on CPU (bitlattice/_ops.py:110-144 fallbacks -> reference.py:398-499): whole-
    matrix and blocked Newton-Schulz in fp32 (standard and Gram iteration, both coefficient sets), the factored
    direction over two steps with its running state, sinkhorn, and the neuron-wise normalisation over two steps."""
    out = {}
    G = (torch.randn(96, 160, generator=gen(70)) * 1e-3).to(torch.bfloat16)
    G2 = (torch.randn(96, 160, generator=gen(71)) * 1e-3).to(torch.bfloat16)
    out["G"], out["G2"] = G.float().numpy(), G2.float().numpy()
    kw = dict(ns_steps=5, ns_dtype="fp32", clip=1.0)
    out["muon"] = _ops.direction(G, "muon", **kw).numpy()
    out["muon_tall"] = _ops.direction(G.t().contiguous(), "muon", **kw).numpy()
    out["muon_block32"] = _ops.direction(G, "muon_block", block=32, **kw).numpy()
    out["muon_band32_gram_pe"] = _ops.direction(G, "muon_block", block=(32, None), ns_coeffs="polar_express",
                                                ns_algo="gram", **kw).numpy()
    out["muon_block64x48"] = _ops.direction(G, "muon_block", block=(64, 48), ns_algo="standard", **kw).numpy()
    out["sinkhorn"] = _ops.direction(G, "sinkhorn", sinkhorn_iters=2, clip=0.5).numpy()
    r, c = torch.zeros(96), torch.zeros(160)
    out["factored_1"] = _ops.direction(G, "factored", r, c, 1, 0.95, clip=1.0).numpy()
    out["factored_2"] = _ops.direction(G2, "factored", r, c, 2, 0.95, clip=1.0).numpy()
    out["factored_r"], out["factored_c"] = r.numpy().copy(), c.numpy().copy()
    v = torch.zeros(96)
    out["normuon_1"] = _ops.direction(G, "muon", row_state=v, row_k=1, **kw).numpy()
    out["normuon_2"] = _ops.direction(G2, "muon", row_state=v, row_k=2, **kw).numpy()
    out["normuon_v"] = v.numpy().copy()
    return out


def momentum2_cases():
    """bl.optim.Lattice on CPU with the deterministic low-precision momenta (lattice.py:396-431): 'ternary' (hash-based
    stochastic rounding) and 'fp8' (round to nearest), three steps with the sign direction; final weights, phase and
    momentum state."""
    out = {}
    for mode in ("ternary", "fp8"):
        ws = [torch.randn(32, 64, generator=gen(80)) * 0.02, torch.randn(16, 128, generator=gen(81)) * 0.02]
        ps = [torch.nn.Parameter(bl.LatticeTensor.from_float(w, "nvfp4", method="rtn", dtype=torch.bfloat16))
              for w in ws]
        for i, p in enumerate(ps):
            out[f"{mode}_p{i}_codes0"], out[f"{mode}_p{i}_scales0"] = p.packed.numpy().copy(), u8(p.scales)
            out[f"{mode}_p{i}_g"] = p.global_scale.numpy().copy()
        opt = bl.optim.Lattice(ps, lr=3e-3, direction="sign", phase_bits=4, scale_rule="fit", seed=777, trust=0.1,
                               trust_lr=0.0, momentum=mode, beta1=0.9)
        for s in range(3):
            for i, p in enumerate(ps):
                G = (torch.randn(p.shape, generator=gen(90 + 2 * s + i)) * 1e-2).to(torch.bfloat16)
                out[f"{mode}_p{i}_G{s}"] = G.float().numpy()
                p.grad = G
            opt.step()
        for i, p in enumerate(ps):
            st = opt.state[p]
            out[f"{mode}_p{i}_codes"], out[f"{mode}_p{i}_scales"] = p.packed.numpy().copy(), u8(p.scales)
            out[f"{mode}_p{i}_phase"] = st["phase"].numpy().copy()
            if mode == "ternary":
                out[f"{mode}_p{i}_mq"], out[f"{mode}_p{i}_ms"] = st["mq"].numpy().copy(), st["ms"].numpy().copy()
            else:
                out[f"{mode}_p{i}_m8"], out[f"{mode}_p{i}_m8s"] = u8(st["m8"]), st["m8s"].numpy().copy()
    return out


def presets_cases():
    """bl.optim.Lattice on CPU under presets whose directions are written out before the step ('balanced': factored;
    'stateless': sinkhorn, no phase; 'muon' with fp32 Newton-Schulz on 32 x 32 blocks): two steps; final weights."""
    out = {}
    for name, extra in (("balanced", {}), ("stateless", {}), ("muon", dict(block=32, ns_dtype="fp32"))):
        ws = [torch.randn(64, 96, generator=gen(100)) * 0.02]
        ps = [torch.nn.Parameter(bl.LatticeTensor.from_float(w, "nvfp4", method="rtn", dtype=torch.bfloat16))
              for w in ws]
        out[f"{name}_codes0"], out[f"{name}_scales0"] = ps[0].packed.numpy().copy(), u8(ps[0].scales)
        out[f"{name}_g"] = ps[0].global_scale.numpy().copy()
        opt = bl.optim.Lattice(ps, name, lr=3e-3, seed=55, trust=0.1, trust_lr=0.0, **extra)
        for s in range(2):
            G = (torch.randn(64, 96, generator=gen(110 + s)) * 1e-2).to(torch.bfloat16)
            out[f"{name}_G{s}"] = G.float().numpy()
            ps[0].grad = G
            opt.step()
        out[f"{name}_codes"], out[f"{name}_scales"] = ps[0].packed.numpy().copy(), u8(ps[0].scales)
        if "phase" in opt.state[ps[0]]:
            out[f"{name}_phase"] = opt.state[ps[0]]["phase"].numpy().copy()
    return out


def linear_cases():
    """'exact' route forward / backward of one layer (the GEMM oracle), config-1-like but small."""
    M, K, N = 48, 128, 64
    w = torch.randn(N, K, generator=gen(50)) * 0.02
    x = torch.randn(M, K, generator=gen(51)).to(torch.bfloat16)
    gy = (torch.randn(M, N, generator=gen(52)) * 1e-2).to(torch.bfloat16)
    p = torch.nn.Parameter(bl.LatticeTensor.from_float(w, "nvfp4", method="rtn", dtype=torch.bfloat16))
    xi = x.clone().requires_grad_(True)
    y = torch.nn.functional.linear(xi, p)
    y.backward(gy)
    return {"w": w.numpy(), "x": x.float().numpy(), "gy": gy.float().numpy(), "codes": p.packed.numpy(),
            "scales": u8(p.scales), "g": p.global_scale.numpy(), "y": y.detach().float().numpy(),
            "gx": xi.grad.float().numpy(), "gw": p.grad.float().numpy()}


def main():
    torch.set_num_threads(4)
    for name, fn in (("hash", hash_cases), ("e4m3", e4m3_cases), ("quantize", quantize_cases),
                     ("transposed", transposed_cases), ("step", step_cases), ("direction", direction_cases),
                     ("optimizer", optimizer_cases), ("linear", linear_cases), ("fos", fos_cases),
                     ("momentum", momentum_cases), ("directions2", directions2_cases),
                     ("momentum2", momentum2_cases), ("presets", presets_cases), ("general", general_cases)):
        if len(sys.argv) > 2 and name not in sys.argv[2:]:
            continue                                   # optional: names of the files to (re)generate
        data = fn()
        path = os.path.join(OUT, f"{name}.npz")
        np.savez_compressed(path, **data)
        print(f"{name}: {len(data)} arrays, {os.path.getsize(path) / 1024:.1f} KiB")


if __name__ == "__main__":
    main()
