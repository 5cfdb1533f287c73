"""The 128-rotation FP4 recipes (quartet2, quartet2_4o6, quartet2_fast, quartet2_delayed, quartet2_bound) and deferred weight gradients
end to end through F.linear, with the criteria of the reference's own tests (tests/test_backend.py:159-201,318-334):
outputs and gradients within 0.25 relative of the exact route, MS-EDEN gradients unbiased (the mean over repeated
backward passes at most 0.35 of one pass's error), deferred weight gradients equal to the accumulated ones within
0.25. The quantizer underneath is compared bit for bit with its oracle in tests/test_general_gpu.py; here the
operands of one backward pass are additionally rebuilt with the oracle from the seeds the layer drew."""
import numpy as np
import pytest
import torch

import bitlattice_b200 as bl
from bitlattice_b200 import backend
from oracle import fp4_general as G

pytestmark = pytest.mark.gpu
DEV = "cuda"
RECIPES = ("nvidia", "4over6", "quartet2", "quartet2_4o6", "quartet2_fast", "quartet2_delayed", "quartet2_bound")


def _C(policy, recipe="nvidia"):
    if policy == "exact":
        return bl.Compute()
    return bl.Compute("nvfp4", backward=policy.endswith("_all"), nvfp4=recipe)


def _weight(n=128, k=256, seed=4):
    g = torch.Generator().manual_seed(seed)
    return bl.LatticeTensor.from_float((torch.randn(n, k, generator=g) * 0.05).to(DEV), "nvfp4", method="rtn",
                                       dtype=torch.bfloat16)


def _grads(x, w, gy, policy, recipe):
    p = torch.nn.Parameter(w.detach())
    xi = x.clone().requires_grad_(True)
    with bl.compute(_C(policy, recipe)):
        y = torch.nn.functional.linear(xi, p)
    y.backward(gy)
    return y.detach().float(), xi.grad.float(), p.grad.float()


def rel(a, b):
    return ((a - b).norm() / b.norm()).item()


@pytest.mark.parametrize("recipe", RECIPES)
@pytest.mark.parametrize("M", [5, 96, 512])
def test_recipes_gradients_close_to_exact(recipe, M):
    g = torch.Generator().manual_seed(4)
    x = torch.randn(M, 256, generator=g).to(torch.bfloat16).to(DEV)
    w = _weight()
    gy = torch.randn(M, 128, generator=g).to(torch.bfloat16).to(DEV)
    ref = _grads(x, w, gy, "exact", "nvidia")
    got = _grads(x, w, gy, "fp4_all", recipe)
    for name, r, v in zip(("y", "dx", "dw"), ref, got):
        assert rel(v, r) < 0.25, (recipe, name, rel(v, r))
    assert bl._ops.gemm_status(0) == 0


@pytest.mark.parametrize("recipe", ["quartet2", "quartet2_4o6"])
def test_eden_recipes_are_unbiased(recipe):
    g = torch.Generator().manual_seed(8)
    M = 256
    x = torch.randn(M, 256, generator=g).to(torch.bfloat16).to(DEV)
    w = _weight(seed=8)
    gy = torch.randn(M, 128, generator=g).to(torch.bfloat16).to(DEV)
    _, rdx, rdw = _grads(x, w, gy, "exact", "nvidia")
    n, sdx, sdw, one = 48, 0, 0, None
    for _ in range(n):
        _, dx, dw = _grads(x, w, gy, "fp4_all", recipe)
        sdx, sdw = sdx + dx, sdw + dw
        if one is None:
            one = (rel(dx, rdx), rel(dw, rdw))
    assert rel(sdx / n, rdx) < 0.35 * one[0], (rel(sdx / n, rdx), one)
    assert rel(sdw / n, rdw) < 0.35 * one[1], (rel(sdw / n, rdw), one)


def _host(t):
    t = t.detach().cpu().contiguous()
    return t.view(torch.uint8).numpy() if t.dtype == torch.float8_e4m3fn else t.numpy()


def _unblock(buf, rows, cols16):
    """Row-major scale bytes from the GEMM's 128 x 4 tiled layout."""
    r, c = np.meshgrid(np.arange(rows), np.arange(cols16), indexing="ij")
    nc = (cols16 + 3) // 4
    at = ((r >> 7) * nc + (c >> 2)) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (c & 3)
    return _host(buf)[at]


def test_quartet2_fast_operands_follow_the_oracle():
    """One forward + backward under 'quartet2_fast' with a known seed counter: every operand the layer builds is what
    the oracle gives for the seeds drawn in the reference's order (forward: rotation seed, then draw seed of the saved
    x^T; backward: draw seeds of the row and of the column operand of the output gradient; the cached W^T uses its
    per-version rotation seed), and the three GEMM results equal the oracle operands' products within bf16 rounding."""
    M, K, N = 256, 256, 128
    g = torch.Generator().manual_seed(21)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    gy = (torch.randn(M, N, generator=g) * 0.1).to(torch.bfloat16)
    w = _weight(N, K, seed=22)
    p = torch.nn.Parameter(w.detach())
    recipe = backend.FP4_RECIPES["quartet2_fast"]
    backend.set_sr_seed(100)
    xi = x.to(DEV).requires_grad_(True)
    with bl.compute(_C("fp4_all", "quartet2_fast")):
        y = torch.nn.functional.linear(xi, p)
        saved = y.grad_fn.saved_tensors
        y.backward(gy.to(DEV))
    xf, gf = x.float().numpy(), gy.float().numpy()
    # forward: x rows, four-over-six round to nearest; saved x^T: MS-EDEN, rotation seed 100, draw seed 101
    xc, xs, xg = G.quantize(xf, four_over_six=True)
    xtc, xts, xtg = G.quantize(xf, transpose=True, mode="eden", rotate=True, rotate_seed=100, seed=101, pow2=True)
    assert np.array_equal(_host(saved[0]), G.pack(xtc)) and np.array_equal(_unblock(saved[1], K, M // 16), xts)
    assert float(saved[2].item()) == float(xtg)
    wt = backend.weight_t_rotated_operand(p)
    wv = G.weight_values(_host(p.packed), _host(p.scales), float(p.global_scale.item()))
    wtc, wts, wtg = G.quantize(wv, transpose=True, rotate=True, rotate_seed=wt.rotate_seed)
    assert np.array_equal(_host(wt.packed), G.pack(wtc)) and np.array_equal(_unblock(wt.scales, K, N // 16), wts)
    # backward: seeds 102 (rows of gy, rotated with W^T's seed) and 103 (gy^T, rotated with x^T's seed)
    gc, gs, gg = G.quantize(gf, mode="eden", rotate=True, rotate_seed=wt.rotate_seed, seed=102)
    gtc, gts, gtg = G.quantize(gf, transpose=True, mode="eden", rotate=True, rotate_seed=100, seed=103, pow2=True)
    want_y = G.dequantize(xc, xs, xg) @ wv.T
    want_gx = G.dequantize(gc, gs, gg) @ G.dequantize(wtc, wts, wtg).T
    want_gw = G.dequantize(gtc, gts, gtg) @ G.dequantize(xtc, xts, xtg).T

    def close(got, want):
        got = got.detach().float().cpu().numpy()
        return bool(np.all(np.abs(got - want) <= 2.0 ** -7 * np.abs(want) + 1e-4 * np.abs(want).max()))
    assert close(y, want_y) and close(xi.grad, want_gx) and close(p.grad, want_gw)


@pytest.mark.parametrize("recipe", ["quartet2", "quartet2_fast"])
def test_deferred_weight_gradients_match_accumulated(recipe):
    g = torch.Generator().manual_seed(12)
    w = _weight(seed=12)
    xs = [(torch.randn(128, 256, generator=g) * s).to(torch.bfloat16).to(DEV) for s in (1.0, 3.0, 0.5)]
    gys = [torch.randn(128, 128, generator=g).to(torch.bfloat16).to(DEV) for _ in xs]
    ref = sum(_grads(x, w, gy, "exact", "nvidia")[2] for x, gy in zip(xs, gys))
    p = torch.nn.Parameter(w.detach())
    backend.fold_rounded(reset=True)
    with bl.compute(_C("fp4_all", recipe)):
        with backend.defer_wgrad():
            for x, gy in zip(xs, gys):
                torch.nn.functional.linear(x.clone().requires_grad_(True), p).backward(gy)
        assert p.grad is None and backend.pending_wgrad() == [p]
        assert backend.flush_wgrad() == 1
    assert rel(p.grad.float(), ref) < 0.25
    assert not backend.pending_wgrad()
    assert backend.fold_rounded() >= 0


def test_delayed_scales_follow_the_previous_call():
    """'quartet2_delayed' (reference: tests/test_backend.py:298-316): the first call of a layer computes its
    per-tensor scales, later calls take them from the amax the previous call saw times the margin -- also when the
    new input exceeds it within the margin -- and stay within 0.25 of the exact gradients. The kept amax is the one
    the oracle finds for the rotated operands, and a given scale is the previous amax * margin / (6 * 448), rounded
    up to a power of two for the weight-gradient side."""
    g = torch.Generator().manual_seed(11)
    w = _weight(seed=11)
    p = torch.nn.Parameter(w.detach())
    rels, seen_x = [], []
    backend.set_sr_seed(500)
    for i, scale in enumerate((1.0, 1.0, 1.0, 1.5)):
        x = (torch.randn(256, 256, generator=g) * scale).to(torch.bfloat16).to(DEV)
        gy = torch.randn(256, 128, generator=g).to(torch.bfloat16).to(DEV)
        _, rdx, rdw = _grads(x, w, gy, "exact", "nvidia")
        p.grad = None
        xi = x.clone().requires_grad_(True)
        with bl.compute(_C("fp4_all", "quartet2_delayed")):
            y = torch.nn.functional.linear(xi, p)
            xt_global = float(y.grad_fn.saved_tensors[2].item())
            y.backward(gy)
        rels.append(max(rel(xi.grad.float(), rdx), rel(p.grad.float(), rdw)))
        amax = p._bl_sites["x"]["amax"].cpu().numpy()
        xf = x.float().cpu().numpy()
        assert amax[0] == np.abs(xf).max()                                   # row side: not rotated
        rot = G.rht128(np.ascontiguousarray(xf.T), 500 + 4 * i)              # the call's first seed rotates x^T
        assert amax[1] == np.abs(rot).max()
        if seen_x:                                                           # the scale came from the previous amax
            want = np.float32(seen_x[-1][1]) * np.float32(2.0 / (6.0 * 448.0))      # MS-EDEN side: no four-over-six
            assert xt_global == float(G.pow2_up(np.float32(want)))
        seen_x.append(amax)
    assert p._bl_sites["x"]["known"] == (True, True) and p._bl_sites["g"]["known"] == (True, True)
    assert max(rels) < 0.25, rels


def test_deferred_weight_gradients_with_delayed_scales():
    g = torch.Generator().manual_seed(14)
    w = _weight(seed=14)
    p = torch.nn.Parameter(w.detach())
    for step in range(3):                              # the first step is exact; later ones use delayed scales
        xs = [(torch.randn(128, 256, generator=g) * s).to(torch.bfloat16).to(DEV) for s in (1.0, 1.3)]
        gys = [torch.randn(128, 128, generator=g).to(torch.bfloat16).to(DEV) for _ in xs]
        ref = sum(_grads(x, w, gy, "exact", "nvidia")[2] for x, gy in zip(xs, gys))
        p.grad = None
        with bl.compute(_C("fp4_all", "quartet2_delayed")):
            with backend.defer_wgrad():
                for x, gy in zip(xs, gys):
                    torch.nn.functional.linear(x.clone().requires_grad_(True), p).backward(gy)
            for _, items in backend._PENDING.values():   # the operands to concatenate: power-of-two scales
                for gt, xt in items:
                    for gs in (gt.global_scale, xt.global_scale):
                        assert torch.equal(gs, torch.exp2(torch.round(torch.log2(gs))))
            backend.flush_wgrad()
        assert rel(p.grad.float(), ref) < 0.25, step


def test_deferred_weight_gradients_need_the_128_rotation():
    w = _weight()
    p = torch.nn.Parameter(w.detach())
    x = torch.randn(128, 256, device=DEV, dtype=torch.bfloat16).requires_grad_(True)
    with bl.compute("fp4_all"), backend.defer_wgrad():
        y = torch.nn.functional.linear(x, p)
        with pytest.raises(RuntimeError, match="128-element rotation"):
            y.backward(torch.ones_like(y))


def test_optimizer_update_renews_the_cached_rotated_weight():
    p = torch.nn.Parameter(_weight())
    opt = bl.Lattice([p], lr=1e-2, direction="sign", phase_bits=4)
    x = torch.randn(128, 256, device=DEV, dtype=torch.bfloat16)
    with bl.compute("quartet2_fast"):
        torch.nn.functional.linear(x, p).float().square().mean().backward()
        first = backend.weight_t_rotated_operand(p)
        assert backend.weight_t_rotated_operand(p) is first
        opt.step()
        second = backend.weight_t_rotated_operand(p)
    assert second is not first and second.rotate_seed != first.rotate_seed
