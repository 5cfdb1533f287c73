"""Oracle parity at the shapes of the benchmark configurations (the other GPU tests use small and ragged shapes):

  single layer      M = 256, K = N = 1024 end to end: every GEMM operand bit for bit, the three outputs within bf16
                    rounding of the oracle's contraction, then one sign / 4-bit lattice update bit for bit;
  pair kernel       a GEMM large enough for the library to choose its 256 x 256 CTA-pair kernel by itself;
  8B-class update   the fused column-normalised update at 1024 x 4096 and 12288 x 4096 (many row panels, grid-stride
                    passes over the rows, a multi-block reduction of the statistics);
  32B-class GEMMs   K = 5120 with N = 25600 and K = 25600 with N = 5120 (20 and 100 k-tiles; 100 column tiles, not a
                    multiple of the pair kernel's tile groups), as plain GEMMs and as one layer through F.linear.

Tolerances: codes, scale bytes and phase bytes are compared with array_equal; GEMM outputs must lie within one bf16
ulp (2^-8 relative) plus 2e-5 of the largest magnitude of the oracle's double-precision contraction.
"""
import functools

import numpy as np
import pytest
import torch

import bitlattice_b200 as bl
import oracle
from bitlattice_b200 import _ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def gen(seed):
    return torch.Generator().manual_seed(seed)


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)) if isinstance(a, np.ndarray) else a
    if dtype is not None:
        t = t.to(dtype)
    return t.to(DEV).contiguous()


def host(t):
    t = t.detach().cpu().contiguous()
    return t.view(torch.uint8).numpy() if t.dtype == torch.float8_e4m3fn else t.numpy()


def within_bf16(got, ref):
    got = got.detach().float().cpu().numpy()
    return bool(np.all(np.abs(got - ref) <= 2.0 ** -8 * np.abs(ref) + 2e-5 * np.abs(ref).max()))


def layer_against_oracle(M, K, N, seeds=(0, 1, 2), sr_seed=1):
    """One F.linear forward + backward under 'fp4_all' against the oracle's operands and contractions; returns the
    parameter, the oracle's weight parts and the weight gradient."""
    wd = torch.randn(N, K, generator=gen(seeds[0])) * 0.02
    x = torch.randn(M, K, generator=gen(seeds[1])).to(torch.bfloat16)
    gy = (torch.randn(M, N, generator=gen(seeds[2])) * 1e-2).to(torch.bfloat16)
    p = torch.nn.Parameter(bl.LatticeTensor.from_float(wd.to(DEV), "nvfp4", method="rtn", dtype=torch.bfloat16))
    H = oracle.hadamard16()
    wc, ws, wg = oracle.quantize_rows(wd.numpy(), None, "rtn")
    assert np.array_equal(host(p.packed), wc) and np.array_equal(host(p.scales), ws)
    xc, xs, xg = oracle.quantize_rows(x.float().numpy(), None, "rtn")
    xtg = oracle.global_from_bound(float(np.float32(xg) * np.float32(4.0)))
    xtc, xts = oracle.quantize_t(x.float().numpy(), H, xtg, "rtn")
    gc, gs, gg = oracle.quantize_rows(gy.float().numpy(), None, "sr", seed=sr_seed)
    gtg = oracle.global_from_bound(float(np.float32(gg) * np.float32(4.0)))
    gtc, gts = oracle.quantize_t(gy.float().numpy(), H, gtg, "sr", seed=sr_seed + 1)
    wtc, wts = oracle.requantize_t(wc, ws, wg)

    bl.backend.set_sr_seed(sr_seed)
    xi = x.to(DEV).requires_grad_(True)
    with bl.compute("fp4_all"):
        y = torch.nn.functional.linear(xi, p)
        saved = y.grad_fn.saved_tensors
        assert np.array_equal(host(saved[0]), xtc), "saved x^T codes"
        assert np.array_equal(host(saved[1]), oracle.to_blocked(xts)), "saved x^T scales"
        assert host(saved[2])[0] == np.float32(xtg)
        # the operands of the backward GEMMs, produced exactly as the backward pass produces them
        g2 = gy.to(DEV)
        bl.backend.set_sr_seed(sr_seed)
        gq = bl.backend.quantize_fp4(g2, stochastic=True)
        assert np.array_equal(host(gq.packed), gc), "SR gradient codes"
        assert np.array_equal(host(gq.scales), oracle.to_blocked(gs)), "SR gradient scales"
        gt = _ops.quantize_nvfp4_t(g2, bl.backend._hadamard16(g2.device, torch.float32), sr_seed + 1, 0,
                                   gq.global_scale * 4.0, blocked=True)
        assert np.array_equal(host(gt[0]), gtc), "rotated transposed SR gradient codes"
        assert np.array_equal(host(gt[1]), oracle.to_blocked(gts)), "rotated transposed SR gradient scales"
        bl.backend.set_sr_seed(sr_seed)
        y.backward(g2)
    wt = bl.backend.weight_t_operand(p)
    assert np.array_equal(host(wt.packed), wtc) and np.array_equal(host(wt.scales), oracle.to_blocked(wts))
    assert within_bf16(y, oracle.gemm_nt(xc, xs, xg, wc, ws, wg)), "y"
    assert within_bf16(xi.grad, oracle.gemm_nt(gc, gs, gg, wtc, wts, wg)), "gx"
    assert within_bf16(p.grad, oracle.gemm_nt(gtc, gts, gtg, xtc, xts, xtg)), "gw"
    assert _ops.gemm_status(0) == 0
    return p, (wc, ws, wg)


def test_single_layer_config_end_to_end():
    """M = 256, K = N = 1024: forward, dgrad, wgrad, then one lattice update (sign, 4-bit phase, lr 3e-3, fixed seed)."""
    p, (wc, ws, wg) = layer_against_oracle(256, 1024, 1024)
    opt = bl.Lattice([p], lr=3e-3, direction="sign", phase_bits=4, seed=1234)
    gw = p.grad.clone()
    opt.step()
    D, _ = oracle.direction(gw.float().cpu().numpy(), "sign", 1.0)
    rc, rp, rs = oracle.lattice_step(wc, np.zeros((1024, 512), np.uint8), ws, wg, D, lr=3e-3, phase_bits=4,
                                     rounding="sr", seed=1234, step=1, scale_rule="fit", trust=0.01, trust_lr=1.0)
    assert np.array_equal(host(p.packed), rc)
    assert np.array_equal(host(p.scales), rs)
    assert np.array_equal(host(opt.state[p]["phase"]), rp)


def _random_operand(rows, K, seed, scale):
    x = (torch.randn(rows, K, generator=gen(seed)) * scale).numpy()
    codes, sf, g = oracle.quantize_rows(x, None, "rtn")
    return codes, sf, float(g)


@functools.lru_cache(maxsize=4)
def _gemm_case(M, N, K):
    ac, asf, ga = _random_operand(M, K, 20, 1.0)
    bc, bsf, gb = _random_operand(N, K, 21, 0.02)
    return ac, asf, ga, bc, bsf, gb, oracle.gemm_nt(ac, asf, ga, bc, bsf, gb)


def _gemm_vs_oracle(M, N, K, kernel="auto"):
    ac, asf, ga, bc, bsf, gb, ref = _gemm_case(M, N, K)
    _ops.gemm_select(kernel)
    try:
        y = _ops.nvfp4_gemm(dev(ac), _ops.to_blocked(dev(asf)), dev(np.array([ga], np.float32)), dev(bc),
                            _ops.to_blocked(dev(bsf)), dev(np.array([gb], np.float32)))
    finally:
        _ops.gemm_select("auto")
    assert _ops.gemm_status(0) == 0
    assert within_bf16(y, ref)


def test_pair_kernel_sized_gemm_matches_oracle():
    """4096 x 4096 x 1024: 256 tiles of 256 x 256, which the library gives to its CTA-pair kernel by itself."""
    _gemm_vs_oracle(4096, 4096, 1024)


@pytest.mark.parametrize("N,K", [(25600, 5120), (5120, 25600), (5120, 5120)])
@pytest.mark.parametrize("kernel", ["auto", "pair"])
def test_32b_class_gemm_shapes_match_oracle(N, K, kernel):
    _gemm_vs_oracle(256, N, K, kernel)


def test_32b_class_layer_end_to_end():
    """hidden 5120 -> intermediate 25600 at 128 tokens: the forward, dgrad and wgrad GEMMs with their real K and N
    (the weight-gradient GEMM contracts over the tokens)."""
    layer_against_oracle(128, 5120, 25600, seeds=(3, 4, 5), sr_seed=7)


@pytest.mark.parametrize("rows,cols", [(1024, 4096), (12288, 4096), (4096, 12288)])
def test_fused_colnorm_update_at_8b_class_shapes(rows, cols):
    """The benchmark's update settings (colnorm, 4-bit phase, sr, scale refit with trust 0.1, bf16 gradients
    ~ N(0, 1e-3^2)) on whole matrices of the 8B-class stack, two steps in a row (the second starts from the phase the
    first one left), codes / phase / scale bytes against the oracle."""
    w = (torch.randn(rows, cols, generator=gen(30)) * 0.02).numpy()
    codes, scales, g = oracle.quantize_rows(w, None, "rtn")
    kw = dict(lr=3e-3, weight_decay=0.0, phase_bits=4, rounding="sr", seed=1234, scale_rule="fit", trust=0.1,
              trust_lr=0.0)
    phase = np.zeros((rows, cols // 2), np.uint8)
    packed, ph, sc = dev(codes), dev(phase), dev(scales)
    gs = dev(np.array([g], np.float32))
    for step in (1, 2):
        G = (torch.randn(rows, cols, generator=gen(30 + step)) * 1e-3).to(torch.bfloat16)
        D, _ = oracle.direction(G.float().numpy(), "colnorm", 1.0)
        codes, phase, scales = oracle.lattice_step(codes, phase, scales, g, D, step=step, **kw)
        _ops.lattice_update(packed, ph, sc, gs, None, dev(G), "nvfp4", rows, cols, phase_cb=4, strata=16,
                            direction="colnorm", clip=1.0, step=step, **kw)
        assert np.array_equal(host(sc), scales), f"scales, step {step}"
        assert np.array_equal(host(packed), codes), f"codes, step {step}"
        assert np.array_equal(host(ph), phase), f"phase, step {step}"
