"""The SwiGLU glue and the SwiGLU MLP block benchmark configuration (hidden 1024, intermediate 3072,
8192 tokens): gate/up -> SwiGLU -> down with NVFP4 weights, all nine GEMMs on the FP4 tensor cores."""
import pytest
import torch

import bitlattice_b200 as bl
from bitlattice_b200 import _ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm()).item()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(64, 1000), (3, 7), (8192, 3072)])
def test_swiglu_matches_autograd(dtype, shape):
    """The reference's own pin (tests/test_fused_block.py:120-130): forward and du equal autograd's bits; dg within 1 %
    of the largest gradient (ATen contracts silu_backward into fused multiply-adds, the kernel does not)."""
    gen = torch.Generator(device=DEV).manual_seed(5)
    g = torch.randn(*shape, device=DEV, generator=gen).to(dtype) * 3
    u = torch.randn(*shape, device=DEV, generator=gen).to(dtype)
    da = torch.randn(*shape, device=DEV, generator=gen).to(dtype)
    gr, ur = g.clone().requires_grad_(True), u.clone().requires_grad_(True)
    a = torch.nn.functional.silu(gr) * ur
    a.backward(da)
    assert torch.equal(_ops.swiglu_fwd(g, u), a.detach())
    dg, du = _ops.swiglu_bwd(g, u, da)
    assert torch.equal(du, ur.grad)
    assert (dg.float() - gr.grad.float()).abs().max().item() <= 1e-2 * gr.grad.float().abs().max().item()
    # and through the autograd function
    g2, u2 = g.clone().requires_grad_(True), u.clone().requires_grad_(True)
    bl.swiglu(g2, u2).backward(da)
    assert torch.equal(u2.grad, du) and torch.equal(g2.grad, dg)


def test_swiglu_rejects_bad_arguments():
    g = torch.zeros(4, 8, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="one shape"):
        _ops.swiglu_fwd(g, torch.zeros(4, 9, device=DEV, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="bf16 or fp16"):
        _ops.swiglu_fwd(g.float(), g.float())
    with pytest.raises(RuntimeError, match="CUDA"):
        _ops.swiglu_fwd(g.cpu(), g.cpu())


def test_swiglu_mlp_block_on_fp4_tensor_cores():
    """Config 2 at full size against the same block on the exact route. What passes one FP4 layer (the weight
    gradient of down) stays within the reference's single-layer bound (0.25 relative, tests/test_backend.py:91-94);
    what passes two independent ones (the output, the input gradient, the weight gradients of gate and up) within
    sqrt(2) times it. Two runs with the same stochastic-rounding seed agree bit for bit; one lattice step moves every
    weight."""
    H, I, M = 1024, 3072, 8192
    gen = torch.Generator(device=DEV).manual_seed(0)
    ws = {n: bl.LatticeTensor.from_float(torch.randn(*s, device=DEV, generator=gen) * 0.02, "nvfp4", method="rtn",
                                         dtype=torch.bfloat16)
          for n, s in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I)))}
    x = torch.randn(M, H, device=DEV, generator=gen).to(torch.bfloat16)
    gy = (torch.randn(M, H, device=DEV, generator=gen) * 1e-2).to(torch.bfloat16)

    def block(route, seed):
        bl.backend.set_sr_seed(seed)
        ps = {n: torch.nn.Parameter(w) for n, w in ws.items()}
        xin = x.clone().requires_grad_(True)
        with bl.compute(route):
            g = torch.nn.functional.linear(xin, ps["gate"])
            u = torch.nn.functional.linear(xin, ps["up"])
            y = torch.nn.functional.linear(bl.swiglu(g, u), ps["down"])
            y.backward(gy)
        return y.detach(), xin.grad, {n: p.grad for n, p in ps.items()}, ps

    y_e, gx_e, gw_e, _ = block("exact", 1)
    y_a, gx_a, gw_a, ps = block("fp4_all", 1)
    y_b, gx_b, gw_b, _ = block("fp4_all", 1)
    assert _ops.gemm_status(0) == 0
    one, two = 0.25, 0.25 * 2 ** 0.5
    assert rel(y_a, y_e) < two, rel(y_a, y_e)
    assert rel(gx_a, gx_e) < two, rel(gx_a, gx_e)
    for n in gw_e:
        assert rel(gw_a[n], gw_e[n]) < (one if n == "down" else two), (n, rel(gw_a[n], gw_e[n]))
        assert torch.equal(gw_a[n], gw_b[n])
    assert torch.equal(y_a, y_b) and torch.equal(gx_a, gx_b)

    opt = bl.Lattice(list(ps.values()), lr=3e-3, direction="sign", phase_bits=4, seed=1234)
    before = {n: p.packed.clone() for n, p in ps.items()}
    opt.step()
    for n, p in ps.items():
        assert (p.packed != before[n]).any(), n
