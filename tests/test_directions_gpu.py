"""Directions that are written out before the update (Newton-Schulz, factored, sinkhorn, neuron-wise normalisation),
low-precision momentum and the optimizer presets, against fixtures produced by the reference's CPU implementation
(tests/golden/make_golden.py: directions2, momentum2, presets).

Tolerances: these directions are chains of fp32 matrix products and reductions whose summation order differs between
the CPU library that produced the fixtures and the GPU's; the reference's own tests compare kernel and Python
directions on ONE device with rtol 1e-4 (tests/test_kernels.py:143-165). Across devices the error of an element is
proportional to the magnitude of the entries it was summed from, not to its own, so the bound here is
|got - ref| <= 1e-4 |ref| + 2e-5 max|ref| (measured: 4e-6 max|ref|); bf16 Newton-Schulz against the fp32 fixture:
0.1 max|ref| (measured 0.05). Hash-based ('ternary') and
round-to-nearest ('fp8') momentum involve no such reduction beyond exact maxima: weights, phase and momentum state are
compared bit for bit. Whole optimizer runs under a preset may differ in the few weights whose target sits within that
tolerance of a rounding boundary: at most 0.5 % of the codes (the reference's bound for order-dependent sums,
tests/test_kernels.py:61-69)."""
import numpy as np
import pytest
import torch

from conftest import golden

import bitlattice_b200 as bl
from bitlattice_b200.optim import directions as D

pytestmark = pytest.mark.gpu
DEV = "cuda"


def close(got: torch.Tensor, ref: np.ndarray, rtol=1e-4, atol=2e-5):
    got = got.float().cpu().numpy()
    return bool(np.all(np.abs(got - ref) <= rtol * np.abs(ref) + atol * np.abs(ref).max()))


def lattice_from(codes, scales, g, shape):
    return bl.LatticeTensor(torch.from_numpy(codes.copy()).to(DEV),
                            torch.from_numpy(scales.copy()).to(DEV).view(torch.float8_e4m3fn),
                            torch.from_numpy(g.copy()).to(DEV), None, "nvfp4", shape, torch.bfloat16)


def test_newton_schulz_directions_match_reference_golden():
    g = golden("directions2")
    G = torch.from_numpy(g["G"]).to(DEV, torch.bfloat16)
    kw = dict(ns_steps=5, ns_dtype="fp32", clip=1.0)
    assert close(D.direction(G, "muon", **kw), g["muon"])
    assert close(D.direction(G.t().contiguous(), "muon", **kw), g["muon_tall"])
    assert close(D.direction(G, "muon_block", block=32, **kw), g["muon_block32"])
    assert close(D.direction(G, "muon_block", block=(32, None), ns_coeffs="polar_express", ns_algo="gram", **kw),
                 g["muon_band32_gram_pe"])
    assert close(D.direction(G, "muon_block", block=(64, 48), ns_algo="standard", **kw), g["muon_block64x48"])
    half = D.direction(G, "muon", ns_steps=5, ns_dtype="bf16", clip=1.0)          # the default dtype: looser
    assert close(half, g["muon"], atol=0.1) and half.dtype == torch.float32


def test_factored_sinkhorn_and_row_normalised_directions_match_reference_golden():
    g = golden("directions2")
    G = torch.from_numpy(g["G"]).to(DEV, torch.bfloat16)
    G2 = torch.from_numpy(g["G2"]).to(DEV, torch.bfloat16)
    assert close(D.direction(G, "sinkhorn", sinkhorn_iters=2, clip=0.5), g["sinkhorn"])
    r, c = torch.zeros(96, device=DEV), torch.zeros(160, device=DEV)
    assert close(D.direction(G, "factored", r, c, 1, 0.95, clip=1.0), g["factored_1"])
    assert close(D.direction(G2, "factored", r, c, 2, 0.95, clip=1.0), g["factored_2"])
    assert close(r, g["factored_r"]) and close(c, g["factored_c"])
    v = torch.zeros(96, device=DEV)
    kw = dict(ns_steps=5, ns_dtype="fp32", clip=1.0)
    assert close(D.direction(G, "muon", row_state=v, row_k=1, **kw), g["normuon_1"])
    assert close(D.direction(G2, "muon", row_state=v, row_k=2, **kw), g["normuon_2"])
    assert close(v, g["normuon_v"])


@pytest.mark.parametrize("mode", ["ternary", "fp8"])
def test_deterministic_low_precision_momentum_matches_reference_bit_for_bit(mode):
    g = golden("momentum2")
    shapes = [(32, 64), (16, 128)]
    ps = [torch.nn.Parameter(lattice_from(g[f"{mode}_p{i}_codes0"], g[f"{mode}_p{i}_scales0"], g[f"{mode}_p{i}_g"], s))
          for i, s in enumerate(shapes)]
    opt = bl.Lattice(ps, lr=3e-3, direction="sign", phase_bits=4, scale_rule="fit", seed=777, trust=0.1, trust_lr=0.0,
                     momentum=mode, beta1=0.9)
    for s in range(3):
        for i, p in enumerate(ps):
            p.grad = torch.from_numpy(g[f"{mode}_p{i}_G{s}"]).to(DEV, torch.bfloat16)
        opt.step()
    for i, p in enumerate(ps):
        st = opt.state[p]
        assert np.array_equal(p.packed.cpu().numpy(), g[f"{mode}_p{i}_codes"])
        assert np.array_equal(p.scales.view(torch.uint8).cpu().numpy(), g[f"{mode}_p{i}_scales"])
        assert np.array_equal(st["phase"].cpu().numpy(), g[f"{mode}_p{i}_phase"])
        if mode == "ternary":
            assert np.array_equal(st["mq"].cpu().numpy(), g[f"{mode}_p{i}_mq"])
            assert np.array_equal(st["ms"].cpu().numpy(), g[f"{mode}_p{i}_ms"])
        else:
            assert np.array_equal(st["m8"].view(torch.uint8).cpu().numpy(), g[f"{mode}_p{i}_m8"])
            assert np.array_equal(st["m8s"].cpu().numpy(), g[f"{mode}_p{i}_m8s"])


@pytest.mark.parametrize("mode", ["bf16", "int8"])
def test_generator_rounded_momentum_keeps_its_average(mode):
    """'bf16' and 'int8' momentum round with torch's device generator (as the reference does on the GPU, where its
    draws differ from the CPU's): the stored average follows the fp32 one within the format's resolution, the state
    has the reference's names and types, and equal seeds give equal runs."""
    def run():
        w = bl.LatticeTensor.from_float((torch.randn(32, 256, generator=torch.Generator().manual_seed(0)) * 0.02).to(DEV),
                                        "nvfp4", method="rtn", dtype=torch.bfloat16)
        p = torch.nn.Parameter(w)
        opt = bl.Lattice([p], lr=3e-3, direction="sign", phase_bits=4, seed=5, momentum=mode, beta1=0.9)
        m = torch.zeros(32, 256)
        for s in range(4):
            G = (torch.randn(32, 256, generator=torch.Generator().manual_seed(10 + s)) * 1e-2).to(torch.bfloat16)
            p.grad = G.to(DEV)
            opt.step()
            m = 0.9 * m + 0.1 * G.float()
        return p, opt, m
    p, opt, m = run()
    st = opt.state[p]
    got = D.load_momentum(st, mode, torch.empty(32, 256, device=DEV)).cpu()
    tol = 2.0 ** -7 * m.abs().max() if mode == "bf16" else 4 * m.abs().max() / 127
    assert (got - m).abs().max() <= tol
    assert ("mb" in st and st["mb"].dtype == torch.bfloat16) if mode == "bf16" else st["m8"].dtype == torch.int8
    p2, _, _ = run()
    assert torch.equal(p.packed, p2.packed)


def test_nvfp4_momentum_is_the_general_quantizer_of_the_average():
    """momentum='nvfp4' (reference: bitlattice/optim/lattice.py:419-423,455-458; needs the reference's CUDA
    extension, so no fixture): the stored average is the stochastically rounded four-over-six NVFP4 of the fp32
    average, with the seed (seed + 7919 pid + 104729 step) & 0x7FFFFFFF, and the next step starts from its values."""
    from oracle import fp4_general as G
    w = bl.LatticeTensor.from_float((torch.randn(32, 256, generator=torch.Generator().manual_seed(0)) * 0.02).to(DEV),
                                    "nvfp4", method="rtn", dtype=torch.bfloat16)
    p = torch.nn.Parameter(w)
    opt = bl.Lattice([p], lr=3e-3, direction="sign", phase_bits=4, seed=5, momentum="nvfp4", beta1=0.9)
    m = np.zeros((32, 256), np.float32)
    for s in range(1, 4):
        grad = (torch.randn(32, 256, generator=torch.Generator().manual_seed(10 + s)) * 1e-2).to(torch.bfloat16)
        p.grad = grad.to(DEV)
        opt.step()
        m = (m * np.float32(0.9)).astype(np.float32) + (grad.float().numpy() * np.float32(1 - 0.9)).astype(np.float32)
        codes, sb, g = G.quantize(m, mode="sr", four_over_six=True, seed=(5 + 104729 * s) & 0x7FFFFFFF)
        st = opt.state[p]
        assert np.array_equal(st["m4p"].cpu().numpy(), G.pack(codes))
        assert np.array_equal(st["m4s"].view(torch.uint8).cpu().numpy(), sb) and float(st["m4g"].item()) == float(g)
        m = G.dequantize(codes, sb, g).astype(np.float32)
    assert opt.state_bits()["momentum"] == 4.5 * p.numel()


@pytest.mark.parametrize("name,extra", [("balanced", {}), ("stateless", {}), ("muon", dict(block=32, ns_dtype="fp32"))])
def test_presets_follow_the_reference_optimizer(name, extra):
    g = golden("presets")
    p = torch.nn.Parameter(lattice_from(g[f"{name}_codes0"], g[f"{name}_scales0"], g[f"{name}_g"], (64, 96)))
    opt = bl.Lattice([p], name, lr=3e-3, seed=55, trust=0.1, trust_lr=0.0, **extra)
    for s in range(2):
        p.grad = torch.from_numpy(g[f"{name}_G{s}"]).to(DEV, torch.bfloat16)
        opt.step()
    codes = p.packed.cpu().numpy()
    lo, hi = codes & 15, codes >> 4
    rlo, rhi = g[f"{name}_codes"] & 15, g[f"{name}_codes"] >> 4
    differing = ((lo != rlo).sum() + (hi != rhi).sum()) / (2 * codes.size)
    assert differing <= 0.005, differing
    assert (p.scales.view(torch.uint8).cpu().numpy() != g[f"{name}_scales"]).mean() <= 0.02
    assert not np.array_equal(codes, g[f"{name}_codes0"])
    if name == "stateless":
        assert "phase" not in opt.state[p]
