"""The reference-facing Python layer on the GPU: LatticeTensor, the linear autograd function under the compute
policy, and the Lattice optimizer, against golden vectors of the reference and the CPU oracle."""
import numpy as np
import pytest
import torch

from conftest import golden

import bitlattice_b200 as bl
import oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


def gen(seed):
    return torch.Generator().manual_seed(seed)


def rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm()).item()


def lattice_from(codes, scales, g, shape, dtype=torch.bfloat16):
    return bl.LatticeTensor(torch.from_numpy(np.ascontiguousarray(codes)).to(DEV),
                            torch.from_numpy(np.ascontiguousarray(scales)).to(DEV).view(torch.float8_e4m3fn),
                            torch.from_numpy(np.ascontiguousarray(g)).to(DEV), None, "nvfp4", shape, dtype)


def test_from_float_and_dequantize_match_reference_golden():
    g = golden("linear")
    w = bl.LatticeTensor.from_float(torch.from_numpy(g["w"]).to(DEV), "nvfp4", method="rtn", dtype=torch.bfloat16)
    assert np.array_equal(w.packed.cpu().numpy(), g["codes"])
    assert np.array_equal(w.scales.view(torch.uint8).cpu().numpy(), g["scales"])
    assert w.global_scale.cpu().numpy()[0] == g["g"][0]
    q = golden("quantize")
    t = lattice_from(q["rtn_codes"], q["rtn_scales"], q["rtn_g"], (32, 128))
    assert np.array_equal(t.dequantize(torch.float32).cpu().numpy(), q["rtn_deq_f32"])
    assert np.array_equal(t.dequantize().view(torch.int16).cpu().numpy(), q["rtn_deq_bf16"])


def test_exact_route_matches_reference_golden():
    """Tolerance: the reference values come from bf16 matmuls on the CPU, these from bf16 matmuls on the GPU; both
    round the same exact products differently -> relative Frobenius error below 1e-2."""
    g = golden("linear")
    p = torch.nn.Parameter(lattice_from(g["codes"], g["scales"], g["g"], (64, 128)))
    x = torch.from_numpy(g["x"]).to(DEV, torch.bfloat16).requires_grad_(True)
    y = torch.nn.functional.linear(x, p)
    y.backward(torch.from_numpy(g["gy"]).to(DEV, torch.bfloat16))
    assert rel(y.detach().cpu(), torch.from_numpy(g["y"])) < 1e-2
    assert rel(x.grad.cpu(), torch.from_numpy(g["gx"])) < 1e-2
    assert rel(p.grad.cpu(), torch.from_numpy(g["gw"])) < 1e-2
    assert p.grad.dtype == torch.bfloat16 and p.grad.shape == (64, 128)


@pytest.mark.parametrize("M", [1, 7, 256])
def test_fp4_linear_matches_quantized_reference(M):
    """The reference's own bound (tests/test_backend.py:23-32): rel < 1e-2 against dequant(quant(x)) @ dequant(W)^T."""
    x = torch.randn(M, 512, generator=gen(1)).to(torch.bfloat16)
    w = bl.LatticeTensor.from_float((torch.randn(384, 512, generator=gen(2)) * 0.05).to(DEV), "nvfp4", method="rtn",
                                    dtype=torch.bfloat16)
    xc, xs, xg = oracle.quantize_rows(x.float().numpy(), None, "rtn")
    ref = oracle.dequantize(xc, xs, xg) @ w.dequantize(torch.float32).cpu().numpy().T
    with bl.compute("fp4"):
        y = torch.nn.functional.linear(x.to(DEV), torch.nn.Parameter(w))
    assert y.shape == (M, 384) and rel(y.cpu(), torch.from_numpy(ref)) < 1e-2
    assert bl._ops.gemm_status(0) == 0


def test_four_over_six_recipe_forward_and_backward():
    """The '4over6' recipe: the forward follows dequant(Q_4over6(x)) @ dequant(W)^T within the reference's forward bound
    (1e-2), is at least as close to the exact layer as the NVIDIA recipe on Gaussian inputs, and the backward stays
    within the 0.25 bound of the exact route."""
    x = torch.randn(512, 512, generator=gen(1)).to(torch.bfloat16)
    w = bl.LatticeTensor.from_float((torch.randn(384, 512, generator=gen(2)) * 0.05).to(DEV), "nvfp4", method="rtn",
                                    dtype=torch.bfloat16)
    W = w.dequantize(torch.float32).cpu()
    xc, xs, xg = oracle.quantize_rows_fos(x.float().numpy(), None, "mse")
    ref = torch.from_numpy(oracle.dequantize(xc, xs, xg)) @ W.T
    exact = x.float() @ W.T
    gy = (torch.randn(512, 384, generator=gen(3)) * 1e-2).to(DEV, torch.bfloat16)
    errs = {}
    for name in ("nvidia", "4over6"):
        p = torch.nn.Parameter(w)
        xin = x.to(DEV).requires_grad_(True)
        with bl.compute(bl.Compute("nvfp4", nvfp4=name)):
            y = torch.nn.functional.linear(xin, p)
            y.backward(gy)
        errs[name] = rel(y.cpu(), exact)
        if name == "4over6":
            assert rel(y.cpu(), ref) < 1e-2
        assert rel(xin.grad.cpu(), gy.float().cpu() @ W) < 0.25
        assert rel(p.grad.cpu(), gy.float().cpu().T @ x.float()) < 0.25
    assert errs["4over6"] <= errs["nvidia"] * 1.02, errs
    assert bl._ops.gemm_status(0) == 0
    with pytest.raises(ValueError, match="scale_source"):
        bl.backend.Fp4Recipe(scale_source="sometimes")


@pytest.mark.parametrize("M", [5, 96, 512])
def test_fp4_all_gradients_close_to_exact(M):
    """The reference's bound (tests/test_backend.py:77-94): y, dx, dw within 0.25 relative error of the exact route."""
    x = torch.randn(M, 256, generator=gen(3)).to(DEV, torch.bfloat16)
    w = bl.LatticeTensor.from_float((torch.randn(128, 256, generator=gen(4)) * 0.05).to(DEV), "nvfp4", method="rtn")
    gy = torch.randn(M, 128, generator=gen(5)).to(DEV, torch.bfloat16)
    out = {}
    for pol in ("exact", "fp4_all"):
        p = torch.nn.Parameter(w.detach().clone())
        xi = x.clone().requires_grad_(True)
        with bl.compute(pol):
            y = torch.nn.functional.linear(xi, p)
        y.backward(gy)
        out[pol] = (y.detach(), xi.grad, p.grad)
    for name, r, got in zip(("y", "dx", "dw"), out["exact"], out["fp4_all"]):
        assert got.shape == r.shape and rel(got, r) < 0.25, (name, rel(got, r))
    assert bl._ops.gemm_status(0) == 0


def test_fp4_all_operands_are_bit_exact_and_outputs_follow_them():
    """Every operand of the three GEMMs equals the oracle's quantization (codes and scale bytes), and each GEMM
    output equals the oracle's contraction of those operands within bf16 rounding."""
    M, K, N = 96, 256, 128
    x = torch.randn(M, K, generator=gen(6)).to(torch.bfloat16)
    gy = (torch.randn(M, N, generator=gen(7)) * 1e-2).to(torch.bfloat16)
    wd = (torch.randn(N, K, generator=gen(8)) * 0.02)
    w = bl.LatticeTensor.from_float(wd.to(DEV), "nvfp4", method="rtn", dtype=torch.bfloat16)
    wc, ws, wg = oracle.quantize_rows(wd.numpy(), None, "rtn")
    assert np.array_equal(w.packed.cpu().numpy(), wc)
    H = oracle.hadamard16()
    # oracle operands
    xc, xs, xg = oracle.quantize_rows(x.float().numpy(), None, "rtn")
    xtg = oracle.global_from_bound(float(np.float32(xg) * np.float32(4.0)))
    xtc, xts = oracle.quantize_t(x.float().numpy(), H, xtg, "rtn")
    bl.backend.set_sr_seed(100)
    gc, gs, gg = oracle.quantize_rows(gy.float().numpy(), None, "sr", seed=100)
    wtc, wts = oracle.requantize_t(wc, ws, wg)
    gtg = oracle.global_from_bound(float(np.float32(gg) * np.float32(4.0)))
    gtc, gts = oracle.quantize_t(gy.float().numpy(), H, gtg, "sr", seed=101)
    y_ref = oracle.gemm_nt(xc, xs, xg, wc, ws, wg)
    gx_ref = oracle.gemm_nt(gc, gs, gg, wtc, wts, wg)
    gw_ref = oracle.gemm_nt(gtc, gts, gtg, xtc, xts, xtg)
    # product
    p = torch.nn.Parameter(w)
    xi = x.to(DEV).requires_grad_(True)
    with bl.compute("fp4_all"):
        y = torch.nn.functional.linear(xi, p)
        xt = y.grad_fn.saved_tensors
        assert np.array_equal(xt[0].cpu().numpy(), xtc)
        assert np.array_equal(xt[1].cpu().numpy(), oracle.to_blocked(xts))
        assert xt[2].cpu().numpy()[0] == np.float32(xtg)
        y.backward(gy.to(DEV))
    wt = bl.backend.weight_t_operand(p)
    assert np.array_equal(wt.packed.cpu().numpy(), wtc) and np.array_equal(wt.scales.cpu().numpy(),
                                                                            oracle.to_blocked(wts))
    for name, got, ref in (("y", y, y_ref), ("gx", xi.grad, gx_ref), ("gw", p.grad, gw_ref)):
        got = got.detach().float().cpu().numpy()
        assert np.all(np.abs(got - ref) <= 2.0 ** -8 * np.abs(ref) + 2e-5 * np.abs(ref).max()), name
    assert bl._ops.gemm_status(0) == 0


def test_cached_weight_operands_follow_updates():
    lin_w = bl.LatticeTensor.from_float((torch.randn(128, 256, generator=gen(9)) * 0.05).to(DEV), "nvfp4", method="rtn",
                                        dtype=torch.bfloat16)
    p = torch.nn.Parameter(lin_w)
    x = torch.randn(64, 256, generator=gen(10)).to(DEV, torch.bfloat16)
    opt = bl.Lattice([p], lr=5e-2, direction="sign", phase_bits=2)
    with bl.compute("fp4_all"):
        y1 = torch.nn.functional.linear(x, p)
        y1.float().square().mean().backward()
        opt.step()
        opt.zero_grad()
        y2 = torch.nn.functional.linear(x, p)
        bl.backend._OPERANDS.clear()
        y3 = torch.nn.functional.linear(x, p)
    assert not torch.equal(y1, y2)
    assert torch.equal(y2, y3)


# ------------------------------------------------------------------------------------------------ optimizer

def _golden_opt_names():
    return [str(n) for n in golden("optimizer")["names"]]


@pytest.mark.parametrize("key", _golden_opt_names())
def test_optimizer_matches_reference_golden(key):
    """Two steps of bl.optim.Lattice over two parameters reproduce the reference's CPU run bit for bit: codes, scale
    bytes and phase bytes (this pins the per-parameter seeds, step counters and state layout too)."""
    g = golden("optimizer")
    direction, bits, rule = key.split("_")[0], int(key.split("_")[1][1:]), key.split("_", 2)[2]
    trust_lr = {"sign_b4_fit": 1.0, "raw_b2_fit": 0.0, "sign_b0_fixed": 1.0, "sign_b8_fit_latent": 0.0}[key]
    shapes = [(32, 64), (16, 128)]
    ps = [torch.nn.Parameter(lattice_from(g[f"{key}_p{i}_codes0"], g[f"{key}_p{i}_scales0"], g[f"{key}_p{i}_g"], s))
          for i, s in enumerate(shapes)]
    opt = bl.optim.Lattice(ps, lr=3e-3, direction=direction, phase_bits=bits, scale_rule=rule, seed=1234, trust=0.1,
                           trust_lr=trust_lr)
    for s in range(2):
        for i, p in enumerate(ps):
            p.grad = torch.from_numpy(g[f"{key}_p{i}_G{s}"]).to(DEV, torch.bfloat16)
        opt.step()
    for i, p in enumerate(ps):
        assert np.array_equal(p.scales.view(torch.uint8).cpu().numpy(), g[f"{key}_p{i}_scales"]), (key, i)
        assert np.array_equal(p.packed.cpu().numpy(), g[f"{key}_p{i}_codes"]), (key, i)
        if bits:
            assert np.array_equal(opt.state[p]["phase"].cpu().numpy(), g[f"{key}_p{i}_phase"]), (key, i)
    assert opt.state_bits()["phase"] == bits * sum(p.numel() for p in ps)


@pytest.mark.parametrize("key", [str(n) for n in golden("momentum")["names"]])
def test_fp32_momentum_matches_reference_golden(key):
    """Three steps with momentum='fp32': codes, scale bytes, phase bytes and the momentum buffer itself equal the
    reference's CPU run bit for bit (the average is one rounded multiply and one fused multiply-add per element on both
    sides)."""
    g = golden("momentum")
    direction, bits, rule = key.split("_")[0], int(key.split("_")[1][1:]), key.split("_", 2)[2]
    shapes = [(32, 64), (16, 128)]
    ps = [torch.nn.Parameter(lattice_from(g[f"{key}_p{i}_codes0"], g[f"{key}_p{i}_scales0"], g[f"{key}_p{i}_g"], s))
          for i, s in enumerate(shapes)]
    opt = bl.optim.Lattice(ps, lr=3e-3, direction=direction, phase_bits=bits, scale_rule=rule, seed=4321, trust=0.1,
                           trust_lr=0.0, momentum="fp32", beta1=0.9)
    for s in range(3):
        for i, p in enumerate(ps):
            p.grad = torch.from_numpy(g[f"{key}_p{i}_G{s}"]).to(DEV, torch.bfloat16)
        opt.step()
    for i, p in enumerate(ps):
        assert np.array_equal(opt.state[p]["m"].cpu().numpy(), g[f"{key}_p{i}_m"]), (key, i)
        assert np.array_equal(p.scales.view(torch.uint8).cpu().numpy(), g[f"{key}_p{i}_scales"]), (key, i)
        assert np.array_equal(p.packed.cpu().numpy(), g[f"{key}_p{i}_codes"]), (key, i)
        assert np.array_equal(opt.state[p]["phase"].cpu().numpy(), g[f"{key}_p{i}_phase"]), (key, i)
    assert opt.state_bits()["momentum"] == 32 * sum(p.numel() for p in ps)


def _make_params(seed=11):
    return [torch.nn.Parameter(bl.LatticeTensor.from_float((torch.randn(s, generator=gen(seed + i)) * 0.05).to(DEV),
                                                           "nvfp4", method="rtn", dtype=torch.bfloat16))
            for i, s in enumerate([(64, 128), (32, 256)])]


def _run(ps, opt, steps, micro=1, accumulate=False):
    for s in range(steps):
        for m in range(micro):
            last = m == micro - 1
            ctx = opt.accumulate() if (accumulate and not last) else torch.autograd.profiler.record_function("step")
            with ctx:
                loss = 0
                for i, p in enumerate(ps):
                    x = torch.randn(16, p.shape[1], generator=gen(100 + 10 * s + m)).to(DEV, torch.bfloat16)
                    loss = loss + torch.nn.functional.linear(x, p).float().square().mean()
                loss.backward()
        opt.step()
        opt.zero_grad()


def test_fused_backward_matches_step():
    """Reference identity (tests/test_optim.py:60-71): applying updates from the gradient hooks equals step()."""
    a, b = _make_params(), _make_params()
    o1 = bl.Lattice(a, lr=5e-3, direction="colnorm", phase_bits=4, seed=3)
    o2 = bl.Lattice(b, lr=5e-3, direction="colnorm", phase_bits=4, seed=3, fused_backward=True)
    _run(a, o1, 3)
    _run(b, o2, 3)
    assert all(p.grad is None for p in b)
    for p, q in zip(a, b):
        assert torch.equal(p.packed, q.packed) and torch.equal(p.scales.view(torch.uint8), q.scales.view(torch.uint8))
        assert torch.equal(o1.state[p]["phase"], o2.state[q]["phase"])


def test_overlapped_updates_match_step():
    """``overlap=True`` issues the updates on a side stream behind the gradient (the reference's worker thread and
    update stream, lattice.py:225-253); after ``step()`` has joined the streams the weights and the optimizer state
    are those of the plain optimizer, and forward passes in between read the updated weights."""
    a, b, c = _make_params(), _make_params(), _make_params()
    o1 = bl.Lattice(a, lr=5e-3, direction="colnorm", phase_bits=4, seed=3)
    o2 = bl.Lattice(b, lr=5e-3, direction="colnorm", phase_bits=4, seed=3, fused_backward=True, overlap=True)
    o3 = bl.Lattice(c, lr=5e-3, direction="colnorm", phase_bits=4, seed=3, overlap=True)
    _run(a, o1, 3)
    _run(b, o2, 3)
    _run(c, o3, 3)
    torch.cuda.synchronize()
    assert all(p.grad is None for p in b)
    for p, q, r in zip(a, b, c):
        for t in (q, r):
            assert torch.equal(p.packed, t.packed)
            assert torch.equal(p.scales.view(torch.uint8), t.scales.view(torch.uint8))
        assert torch.equal(o1.state[p]["phase"], o2.state[q]["phase"])
        assert torch.equal(o1.state[p]["phase"], o3.state[r]["phase"])


@pytest.mark.parametrize("M", [256, 40])
def test_shared_input_linears_sum_their_input_gradients_in_the_gemm(M):
    """parallel.shared_input_linears (q/k/v, gate/up in one process): outputs are those of F.linear per weight; the
    input gradient is the sum of the projections' input gradients in the order of the weights, formed in the GEMM
    epilogues (rows in multiples of 32) or by dense adds (padded rows) -- the same bits either way -- and the weight
    gradients are those of the separate layers under the same stochastic-rounding seeds."""
    from bitlattice_b200 import backend, parallel
    g = gen(61)
    ws = [torch.nn.Parameter(bl.LatticeTensor.from_float((torch.randn(n, 256, generator=g) * 0.05).to(DEV), "nvfp4",
                                                         method="rtn", dtype=torch.bfloat16)) for n in (128, 64, 96)]
    x = torch.randn(M, 256, generator=g).to(torch.bfloat16).to(DEV).requires_grad_(True)
    gys = [(torch.randn(M, w.shape[0], generator=g) * 0.1).to(torch.bfloat16).to(DEV) for w in ws]
    with bl.compute("fp4_all"):
        ys = parallel.shared_input_linears(x, ws)
        assert ys[0].grad_fn is ys[1].grad_fn                                # one function for all three
        for y, w in zip(ys, ws):
            assert torch.equal(y, torch.nn.functional.linear(x.detach(), w.detach()))
        backend.set_sr_seed(900)
        torch.autograd.backward(ys, gys)
        # the same by hand: three input-gradient GEMMs (seeds 900..902), dense adds, three weight-gradient GEMMs (903..905)
        backend.set_sr_seed(900)
        recipe = backend.FP4_RECIPES["nvidia"]
        parts = [backend.fp4_dgrad(gy, w, recipe) for gy, w in zip(gys, ws)]
        want_gx = (parts[0][0] + parts[1][0]) + parts[2][0]
        _, xt = backend._shared(x, recipe, "fwd+t", lambda: pytest.fail("the forward's operands should still be shared"))
        want_gw = [backend.fp4_wgrad(p[1], p[2], xt, w, recipe) for p, w in zip(parts, ws)]
    assert torch.equal(x.grad, want_gx)
    for w, gw in zip(ws, want_gw):
        assert torch.equal(w.grad, gw.to(w.dtype))
    assert bl._ops.gemm_status(0) == 0


def test_batched_step_reuses_its_plan_and_notices_new_storage():
    """step() marshals the static arguments of a batch of parameters once (an update plan) and reuses them; when a
    parameter's state or storage is replaced between steps the plan is rebuilt. Either way the result is that of the
    optimizer updating one tensor at a time."""
    a, b = _make_params(21), _make_params(21)
    o1 = bl.Lattice(a, lr=5e-3, direction="colnorm", phase_bits=4, seed=3)
    o2 = bl.Lattice(b, lr=5e-3, direction="colnorm", phase_bits=4, seed=3)
    o2._batchable = lambda *args: False                      # one library call per tensor
    _run(a, o1, 2)
    assert len(o1._plans) == 1
    plan = next(iter(o1._plans.values()))
    _run(a, o1, 1)
    assert next(iter(o1._plans.values())) is plan            # reused
    for p in a:                                              # new phase storage, as load_state_dict leaves it
        o1.state[p]["phase"] = o1.state[p]["phase"].clone()
    _run(a, o1, 2)
    assert next(iter(o1._plans.values())) is not plan        # rebuilt for the new addresses
    for n in (2, 1, 2):                                      # the same inputs as above, one tensor at a time
        _run(b, o2, n)
    assert not o2._plans
    torch.cuda.synchronize()
    for p, q in zip(a, b):
        assert torch.equal(p.packed, q.packed)
        assert torch.equal(p.scales.view(torch.uint8), q.scales.view(torch.uint8))
        assert torch.equal(o1.state[p]["phase"], o2.state[q]["phase"])


@pytest.mark.parametrize("flush", ["backward", "reader"])
@pytest.mark.parametrize("overlap", [False, True])
def test_hook_batches_match_immediate_updates(overlap, flush):
    """``hook_batch``: the backward hooks collect gradients and issue their updates several at a time (the rest when
    the backward pass ends, before anything reads the weights again); same weights and state as updating each
    parameter from its own hook, gradients freed either way."""
    def params():
        return [torch.nn.Parameter(bl.LatticeTensor.from_float((torch.randn(s, generator=gen(40 + i)) * 0.05).to(DEV),
                                                               "nvfp4", method="rtn", dtype=torch.bfloat16))
                for i, s in enumerate([(64, 128), (32, 256), (48, 128), (32, 128), (64, 256)])]
    a, b = params(), params()
    o1 = bl.Lattice(a, lr=5e-3, direction="colnorm", phase_bits=4, seed=3, fused_backward=True)
    o2 = bl.Lattice(b, lr=5e-3, direction="colnorm", phase_bits=4, seed=3, fused_backward=True, overlap=overlap,
                    hook_batch=2, hook_flush=flush)
    for ps, opt in ((a, o1), (b, o2)):
        for s in range(3):
            loss = 0
            for p in ps:       # (with 'reader', a weight whose update is still pending would be flushed here)
                x = torch.randn(16, p.shape[1], generator=gen(200 + s)).to(DEV, torch.bfloat16)
                loss = loss + torch.nn.functional.linear(x, p).float().square().mean()
            loss.backward()
            if opt is o1 or flush == "backward":      # 5 parameters: 2 + 2 + the last one at the end of backward
                assert all(p.grad is None for p in ps) and not opt._pending
            else:                                     # the last one waits for step() or for a reader
                assert len(opt._pending) == 1
                held = opt._pending[0]
                if s == 1:                            # a reader: the pending update goes out before the read
                    held.dequantize(torch.float32)
                    assert not opt._pending and held.grad is None
                if s == 2:                            # a cached GEMM operand is not handed out for the old version
                    version = held._bl_version
                    bl.backend.weight_operand(held)
                    assert not opt._pending and held._bl_version == version + 1
            opt.step()
            assert not opt._pending
    torch.cuda.synchronize()
    for p, q in zip(a, b):
        assert torch.equal(p.packed, q.packed)
        assert torch.equal(p.scales.view(torch.uint8), q.scales.view(torch.uint8))
        assert torch.equal(o1.state[p]["phase"], o2.state[q]["phase"])


def test_readers_wait_for_overlapped_updates():
    """With ``overlap=True`` an update may still be running on the update stream when the weight is read again;
    every reader (GEMM operands, dequantize) first waits for the update's event, so reading right after backward --
    without step() in between -- sees the updated weight, as with the in-line optimizer."""
    a, b = _make_params(40), _make_params(40)
    o1 = bl.Lattice(a, lr=5e-3, direction="colnorm", phase_bits=4, seed=9, fused_backward=True)
    o2 = bl.Lattice(b, lr=5e-3, direction="colnorm", phase_bits=4, seed=9, fused_backward=True, overlap=True)
    outs = []
    for ps in (a, b):
        loss = 0
        for p in ps:
            x = torch.randn(16, p.shape[1], generator=gen(77)).to(DEV, torch.bfloat16)
            loss = loss + torch.nn.functional.linear(x, p).float().square().mean()
        loss.backward()                                     # hooks issue the updates; no step() yet
        got = []
        for p in ps:
            x = torch.randn(32, p.shape[1], generator=gen(78)).to(DEV, torch.bfloat16)
            with bl.compute("fp4"):
                got.append(torch.nn.functional.linear(x, p))
            got.append(p.dequantize(torch.float32))
        outs.append(got)
    assert all(hasattr(p, "_bl_updated") for p in b)
    for u, v in zip(*outs):
        assert torch.equal(u, v)
    o1.step(), o2.step()


def test_accumulate_equals_summed_gradient():
    """Reference identity (tests/test_parallel.py:131-156): with fused_backward, micro-batches inside accumulate()
    are summed and applied once."""
    a, b = _make_params(20), _make_params(20)
    o1 = bl.Lattice(a, lr=5e-3, direction="sign", phase_bits=2, seed=5)
    o2 = bl.Lattice(b, lr=5e-3, direction="sign", phase_bits=2, seed=5, fused_backward=True)
    _run(a, o1, 2, micro=3)                         # plain: gradients sum in .grad, one step
    _run(b, o2, 2, micro=3, accumulate=True)
    for p, q in zip(a, b):
        assert torch.equal(p.packed, q.packed) and torch.equal(o1.state[p]["phase"], o2.state[q]["phase"])


def test_state_dict_round_trip():
    ps = _make_params(30)
    opt = bl.Lattice(ps, lr=5e-3, direction="sign", phase_bits=4)
    _run(ps, opt, 1)
    sd = opt.state_dict()
    opt2 = bl.Lattice(ps, lr=5e-3, direction="sign", phase_bits=4)
    opt2.load_state_dict(sd)
    k = next(iter(opt.state))
    assert torch.equal(opt2.state[k]["phase"], opt.state[k]["phase"]) and opt2.state[k]["step"] == 1
    assert opt.state_bytes() == sum(p.numel() // 2 for p in ps)


def test_row_shard_update_equals_whole_update():
    """N-sharding: shards carrying _bl_row_offset reproduce the unsharded update of the same rows."""
    from bitlattice_b200.parallel import shard_rows
    w = bl.LatticeTensor.from_float((torch.randn(128, 256, generator=gen(40)) * 0.05).to(DEV), "nvfp4", method="rtn",
                                    dtype=torch.bfloat16)
    G = (torch.randn(128, 256, generator=gen(41)) * 1e-2).to(DEV, torch.bfloat16)
    whole = torch.nn.Parameter(w.detach().clone())
    ow = bl.Lattice([whole], lr=3e-3, direction="sign", phase_bits=4, seed=9)
    whole.grad = G
    ow.step()
    for rank in range(2):
        sh = torch.nn.Parameter(shard_rows(w, rank, 2))
        assert sh._bl_row_offset == rank * 64              # Parameter(shard) keeps the shard's first global row
        os_ = bl.Lattice([sh], lr=3e-3, direction="sign", phase_bits=4, seed=9)
        sh.grad = G[rank * 64:(rank + 1) * 64].contiguous()
        os_.step()
        assert torch.equal(sh.packed, whole.packed[rank * 64:(rank + 1) * 64])
        assert torch.equal(os_.state[sh]["phase"], ow.state[whole]["phase"][rank * 64:(rank + 1) * 64])


@pytest.mark.parametrize("direction,clip,count", [("colnorm", 1.0, 2), ("colnorm", 0.25, 2), ("raw", 0.5, 2),
                                                  ("sign", 0.5, 2), ("colnorm", 1.0, 45)])
def test_row_shards_with_whole_weight_statistics_equal_the_whole_update(direction, clip, count):
    """``Lattice(shard_group=...)``: directions that normalise over the whole weight exchange their 128-row panel sums,
    and every shard then receives, bit for bit, the update of its rows in the unsharded weight. Four owners are played
    in turn on one GPU: a first pass collects each owner's panel sums, a second hands every owner the others' sums
    where the all-gather would have put them. 45 weights: more than one batch of kernels, still one exchange."""
    from bitlattice_b200.parallel import shard_rows
    world = 4
    shapes = [(512, 256), (1024, 384)] + [(512, 64)] * (count - 2)
    ws = [bl.LatticeTensor.from_float((torch.randn(*s, generator=gen(60 + i)) * 0.05).to(DEV), "nvfp4", method="rtn",
                                      dtype=torch.bfloat16) for i, s in enumerate(shapes)]
    Gs = [(torch.randn(*s, generator=gen(70 + i)) * (1e-2 * (1 + torch.arange(s[1]) % 7))).to(DEV, torch.bfloat16)
          for i, s in enumerate(shapes)]
    kw = dict(lr=3e-3, direction=direction, clip=clip, phase_bits=4, seed=11)
    whole = [torch.nn.Parameter(w.detach().clone()) for w in ws]
    ow = bl.Lattice(whole, **kw)
    for p, G in zip(whole, Gs):
        p.grad = G
    ow.step()

    class Stop(Exception):
        pass

    def owner(rank, exchange, **extra):
        ps = [torch.nn.Parameter(shard_rows(w, rank, world)) for w in ws]
        opt = bl.Lattice(ps, **kw, **extra)
        opt._exchange = exchange
        opt._shard_world = lambda: (world, rank, None)
        for p, G in zip(ps, Gs):
            n = p.shape[0]
            assert p._bl_rows_total == n * world
            p.grad = G[rank * n:(rank + 1) * n].contiguous()
        return ps, opt

    sums = {}
    for rank in range(world):
        def collect(blocks, rank=rank):
            assert blocks.shape[0] == world and rank not in sums          # one exchange per step
            sums[rank] = blocks[rank].clone()
            raise Stop
        _, opt = owner(rank, collect, shard_group=True)
        with pytest.raises(Stop):
            opt.step()
    for rank in range(world):
        def fill(blocks):
            for other in range(world):
                blocks[other] = sums[other]
        ps, opt = owner(rank, fill, shard_group=True)
        opt.step()
        for p, q in zip(ps, whole):
            n = p.shape[0]
            rows = slice(rank * n, (rank + 1) * n)
            assert torch.equal(p.packed, q.packed[rows]) and torch.equal(p.scales.view(torch.uint8), q.scales.view(torch.uint8)[rows])
            assert torch.equal(opt.state[p]["phase"], ow.state[q]["phase"][rows])
    # without the exchange a shard is a weight of its own: other statistics, another update
    if direction == "colnorm":
        ps, opt = owner(1, None)
        opt.step()
        assert not torch.equal(ps[0].packed, whole[0].packed[128:256])


def test_column_slice_draws_the_rounding_numbers_of_the_whole_gradient():
    """The column-parallel backward with ``parallel.MATCH_UNSHARDED``: a rank's gradient columns, quantized with the
    whole tensor's scale and with the index offset of its first column folded into the step counter, give exactly the
    rows of the whole gradient's transposed stochastic operand."""
    from bitlattice_b200 import _ops, backend, parallel
    M, N, p = 256, 384, 3
    gy = (torch.randn(M, N, generator=gen(81)) * 1e-2).to(DEV, torch.bfloat16)
    H = backend._hadamard16(gy.device, torch.float32)
    bound = _ops.amax_global(gy)[1:2] * 4.0
    whole = _ops.quantize_nvfp4_t(gy, H, 77, 0, bound, blocked=False)
    cols = N // p
    for rank in range(p):
        part = gy[:, rank * cols:(rank + 1) * cols].contiguous()
        step = (rank * cols * M * parallel._HASH_INDEX_MUL * parallel._HASH_STEP_INV) & 0xFFFFFFFF
        got = _ops.quantize_nvfp4_t(part, H, 77, step, bound, blocked=False)
        rows = slice(rank * cols, (rank + 1) * cols)
        assert torch.equal(got[0], whole[0][rows])
        assert torch.equal(got[1].view(torch.uint8), whole[1].view(torch.uint8)[rows])
        if rank:        # without the offset the slice draws other numbers
            other = _ops.quantize_nvfp4_t(part, H, 77, 0, bound, blocked=False)
            assert not torch.equal(other[0], whole[0][rows])


def test_converted_third_party_weights_dequantize_as_in_the_reference():
    """compressed-tensors / ModelOpt NVFP4 tensors converted to lattice weights decode to the reference's values
    (tests/golden/convert.npz, written by the reference's bitlattice.io.convert)."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "convert.npz"))
    t = lambda k: torch.from_numpy(g[k])
    ct = {"weight_packed": t("ct_weight_packed"), "weight_scale": t("ct_weight_scale").view(torch.float8_e4m3fn),
          "weight_global_scale": t("ct_weight_global_scale")}
    mo = {"weight": t("mo_weight"), "weight_scale": t("mo_weight_scale").view(torch.float8_e4m3fn),
          "weight_scale_2": t("mo_weight_scale_2")}
    for w, key in ((bl.io.from_ct_nvfp4(ct, torch.bfloat16, DEV), "ct_dequant"),
                   (bl.io.from_mo_nvfp4(mo, torch.bfloat16, DEV), "mo_dequant")):
        assert torch.equal(w.dequantize(torch.float32).cpu(), t(key))
        x = torch.randn(32, 128, generator=gen(4)).to(DEV, torch.bfloat16)
        with bl.compute("fp4"):
            y = torch.nn.functional.linear(x, w)
        ref = x.float() @ t(key).to(DEV).t()
        assert float((y.float() - ref).norm() / ref.norm()) < 0.1
