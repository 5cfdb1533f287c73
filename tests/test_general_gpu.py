"""The general NVFP4 quantizer (bl_nvfp4_quantize_general) and the scale folding (bl_fp4_fold_scales) through the C ABI
against the numpy oracle (oracle/fp4_general.py, bit for bit: both use the same pinned summation orders) and against
the fixtures written by the reference's fp4ref.quantize (tests/golden/general.npz) with the reference's own criterion
between its kernel and fp4ref (tests/test_nvfp4.py:45-47: per-tensor scale within 1e-6, fewer than 2e-3 of the codes
and scale bytes different; exact where no summation order enters)."""
import os

import numpy as np
import pytest
import torch

import bitlattice_b200 as bl
from bitlattice_b200 import _ops
from oracle import fp4_general as G

pytestmark = pytest.mark.gpu
DEV = "cuda"
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "general.npz"))
CASES = [(t, m, f, r) for t in (False, True) for m in ("rtn", "sr", "eden") for f in (False, True)
         for r in ((True,) if m == "eden" else (False, True))]


def host(t):
    t = t.detach().cpu().contiguous()
    return t.view(torch.uint8).numpy() if t.dtype == torch.float8_e4m3fn else t.numpy()


def run(x, **kw):
    packed, scales, g = _ops.nvfp4_quantize_general(x, **kw)
    torch.cuda.synchronize()
    return host(packed), host(scales), float(g.item())


@pytest.mark.parametrize("transpose,mode,fos,rotate", CASES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_kernel_equals_oracle_and_reference(transpose, mode, fos, rotate, dtype):
    x = torch.from_numpy(GOLD["x"]).to(DEV).to(dtype)
    packed, sb, g = run(x, transpose=transpose, mode=mode, four_over_six=fos, rotate=rotate, seed=11, rotate_seed=21)
    codes, osb, og = G.quantize(GOLD["x"], transpose=transpose, mode=mode, four_over_six=fos, rotate=rotate, seed=11,
                                rotate_seed=21)
    assert g == float(og)
    assert np.array_equal(sb, osb)
    assert np.array_equal(packed, G.pack(codes))
    tag = f"{'t' if transpose else 'r'}_{mode}_{int(fos)}_{int(rotate)}"
    ref_g = float(GOLD[tag + "_g"][0])
    assert abs(g - ref_g) <= 1e-6 * ref_g
    lim = 0.0 if (not rotate and not fos and mode != "eden") else 2e-3
    assert (sb != GOLD[tag + "_scales"]).mean() <= lim
    assert (G.unpack(packed, codes.shape[1]) != G.unpack(GOLD[tag + "_codes"], codes.shape[1])).mean() <= lim


@pytest.mark.parametrize("select", ["mse", "mae"])
def test_mae_selection_given_scale_and_pow2(select):
    g0 = torch.Generator().manual_seed(3)
    x = (torch.randn(256, 384, generator=g0) * torch.exp(torch.randn(256, 1, generator=g0))).to(torch.bfloat16)
    xf = x.float().numpy()
    for kw in (dict(mode="eden", rotate=True, four_over_six=True, select=select, seed=5, rotate_seed=9, pow2=True),
               dict(mode="rtn", four_over_six=True, select=select),
               dict(mode="sr", rotate=True, seed=7, transpose=True, pow2=True)):
        packed, sb, g = run(x.to(DEV), **kw)
        codes, osb, og = G.quantize(xf, **kw)
        assert g == float(og) and np.array_equal(sb, osb) and np.array_equal(packed, G.pack(codes)), kw
        if kw.get("pow2"):
            assert np.log2(g) == np.round(np.log2(g))
    given = torch.tensor([0.0123], device=DEV)
    packed, sb, g = run(x.to(DEV), mode="rtn", rotate=True, seed=1, given=given)
    codes, osb, og = G.quantize(xf, mode="rtn", rotate=True, seed=1, given=np.float32(0.0123))
    assert g == float(np.float32(0.0123)) and np.array_equal(sb, osb) and np.array_equal(packed, G.pack(codes))


@pytest.mark.parametrize("shape", [(128, 272 - 16), (256, 512), (384, 160)])
@pytest.mark.parametrize("rotate,fos,mode", [(False, False, "rtn"), (True, False, "rtn"), (True, True, "eden")])
def test_packed_weight_input_equals_dense_input(shape, rotate, fos, mode):
    """An NVFP4 weight re-quantized transposed from its codes equals the quantization of its dense values formed as
    (level * scale) * global (reference: tests/test_nvfp4.py:88-103)."""
    N, K = shape                                              # K a multiple of 32, N a multiple of 128
    w = bl.LatticeTensor.from_float(torch.randn(N, K, generator=torch.Generator().manual_seed(0)).to(DEV) * 0.05,
                                    "nvfp4", method="rtn")
    codes, scales, gw = host(w.packed), host(w.scales), float(w.global_scale.item())
    dense = G.weight_values(codes, scales, gw)
    kw = dict(transpose=True, mode=mode, four_over_six=fos, rotate=rotate, seed=11)
    packed, sb, g = run(w.packed, w_scales=w.scales, w_global=w.global_scale.float(), **kw)
    ocodes, osb, og = G.quantize(dense, **kw)
    assert g == float(og) and np.array_equal(sb, osb) and np.array_equal(packed, G.pack(ocodes))
    p2, s2, g2 = run(torch.from_numpy(dense).to(DEV), **kw)
    assert g2 == g and np.array_equal(p2, packed) and np.array_equal(s2, sb)


def test_observed_amax_with_and_without_a_given_scale():
    """amax_out receives the maximum of the rotated values whether the per-tensor scale is computed (the amax pass
    found it) or given (the quantization pass observes it): the 'seen' amax of delayed scales."""
    x = torch.from_numpy(GOLD["x"]).to(DEV).to(torch.bfloat16)
    for transpose in (False, True):
        src = GOLD["x"].T if transpose else GOLD["x"]
        want = np.abs(G.rht128(np.ascontiguousarray(src), 21)).max()
        for given in (None, torch.tensor([0.02], device=DEV)):
            seen = torch.zeros(1, device=DEV)
            _ops.nvfp4_quantize_general(x, transpose=transpose, mode="eden", rotate=True, seed=11, rotate_seed=21,
                                        given=given, amax_out=seen)
            assert float(seen.item()) == float(want)


@pytest.mark.parametrize("shape,transpose", [((37, 80), False), ((144, 72), True), ((208, 130), True), ((5, 16), False),
                                             ((16, 5), True)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ragged_shapes_without_rotation(shape, transpose, dtype):
    """Shapes that are not made of whole tiles (rows not a multiple of 64, quantized dimension not a multiple of 128,
    source rows of odd length that take the scalar staging path): every mode without the rotation against the
    oracle."""
    g0 = torch.Generator().manual_seed(sum(shape))
    x = (torch.randn(*shape, generator=g0) * 3.0).to(dtype)
    xf = x.float().numpy()
    for kw in (dict(mode="rtn"), dict(mode="sr", seed=3), dict(mode="rtn", four_over_six=True, select="mae")):
        packed, sb, g = run(x.to(DEV), transpose=transpose, **kw)
        codes, osb, og = G.quantize(xf, transpose=transpose, **kw)
        assert g == float(og) and np.array_equal(sb, osb) and np.array_equal(packed, G.pack(codes)), kw


def test_blocked_scale_layout_and_ragged_rows():
    x = torch.randn(200, 256, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(DEV)
    p0, s0, g0 = _ops.nvfp4_quantize_general(x, mode="eden", rotate=True, seed=3)
    p1, s1, g1 = _ops.nvfp4_quantize_general(x, mode="eden", rotate=True, seed=3, blocked=True)
    assert torch.equal(p0, p1) and torch.equal(g0, g1)
    assert torch.equal(_ops.to_blocked(s0.view(torch.uint8)), s1)


def test_eden_is_unbiased_and_tighter_than_sr():
    """The statistical property the reference tests (tests/test_nvfp4.py:62-78): averaged over seeds, MS-EDEN has
    about half the error of stochastic rounding and a smaller bias."""
    g0 = torch.Generator().manual_seed(0)
    x = (torch.randn(64, 256, generator=g0) * torch.exp(torch.randn(64, 1, generator=g0))).to(torch.bfloat16)
    xf = x.float().numpy()
    res = {}
    for mode in ("sr", "eden"):
        acc, mse = 0.0, 0.0
        for sd in range(48):
            packed, sb, g = run(x.to(DEV), mode=mode, rotate=True, seed=sd * 13 + 1)
            d = G.dequantize(G.unpack(packed, 256), sb, g)
            back = (G.fwht128(d.reshape(64, 2, 128)) * G.signs128(sd * 13 + 1)).reshape(64, 256)   # inverse rotation
            acc = acc + back
            mse += float(((back - xf) ** 2).mean())
        res[mode] = (float(np.linalg.norm(acc / 48 - xf) / np.linalg.norm(xf)), mse / 48)
    assert res["eden"][1] < 0.6 * res["sr"][1]
    assert res["eden"][0] < res["sr"][0]


def test_fold_scales_matches_oracle():
    gen = torch.Generator().manual_seed(5)
    row_tiles, widths = 3, (2, 1, 3)
    tiles_per_row = sum(widths)
    sc = torch.randint(0, 0x7F, (row_tiles * tiles_per_row * 512,), generator=gen, dtype=torch.uint8)
    g = torch.tensor([2.0 ** -3, 2.0 ** -9, 2.0 ** -5])
    piece = torch.tensor([j for j, w in enumerate(widths) for _ in range(w)], dtype=torch.int32)
    rounded = torch.zeros(1, dtype=torch.int64, device=DEV)
    dev_sc = sc.to(DEV)
    g_max = _ops.fp4_fold_scales(dev_sc, row_tiles, piece.to(DEV), g.to(DEV), rounded)
    assert float(g_max.item()) == 2.0 ** -3
    want = sc.numpy().reshape(row_tiles, tiles_per_row, 512).copy()
    count = 0
    for t in range(tiles_per_row):
        f = float(g[piece[t]] / g.max())
        if f != 1.0:
            want[:, t], n = G.fold_scales(want[:, t], f)
            count += n
    assert np.array_equal(host(dev_sc).reshape(row_tiles, tiles_per_row, 512), want)
    assert int(rounded.item()) == count and count > 0
