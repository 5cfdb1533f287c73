"""Worker of tests/test_parallel_gpu.py: one process per GPU under torch.distributed.run (NCCL).

Checks the column-parallel FP4 layer against the unsharded layer computed on the same rank:
  * the gathered operands Q(x), Q(rot(x^T)) equal the unsharded quantization bit for bit,
  * y_shard equals the matching columns of the unsharded y bit for bit,
  * gx (reduce-scattered) and gw_shard stay within the reference's FP4 bound of the exact route
    (their stochastic-rounding draws differ from the unsharded layer's by construction).
Prints "OK <rank>" on success.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bitlattice_b200 as bl                                    # noqa: E402
from bitlattice_b200 import backend                             # noqa: E402
from bitlattice_b200.parallel import (GatheredWeights, column_parallel_linear, column_parallel_linears,   # noqa: E402
                                      gathered_input_operands, shard_rows, token_parallel_linear,
                                      token_parallel_linears)


def rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm())


def token_parallel_checks(rank, world, dev, w, x, gy, w2, gy2):
    M, N = gy.shape
    rows = slice(rank * M // world, (rank + 1) * M // world)
    cols = slice(rank * N // world, (rank + 1) * N // world)
    xr, gr = x[rows].contiguous(), gy[rows].contiguous()
    gathered = GatheredWeights(None)
    p = torch.nn.Parameter(shard_rows(w, rank, world))
    assert p._bl_row_offset == rank * N // world          # the shard's first row travels into the Parameter
    for got, ref in ((gathered.operand(p), backend.weight_operand(w)), (gathered.t_operand(p), backend.weight_t_operand(w))):
        assert torch.equal(got.packed, ref.packed), "gathered weight codes differ from the unsharded operand"
        assert torch.equal(got.scales.view(torch.uint8).reshape(-1), ref.scales.view(torch.uint8).reshape(-1))
        assert torch.equal(got.global_scale, ref.global_scale)
    with bl.compute("fp4_all"):
        backend.set_sr_seed(500 + 64 * rank)
        pf = torch.nn.Parameter(w)
        xf = xr.detach().requires_grad_(True)
        yf = torch.nn.functional.linear(xf, pf)
        yf.backward(gr)
        backend.set_sr_seed(500 + 64 * rank)
        xs = xr.detach().requires_grad_(True)
        y = token_parallel_linear(xs, p, gathered)
        assert y.shape == (M // world, N) and torch.equal(y, yf), "token-parallel forward differs"
        y.backward(gr)
    assert torch.equal(xs.grad, xf.grad), "token-parallel input gradient differs from the single-GPU layer's"
    parts = [torch.empty_like(pf.grad) for _ in range(world)]
    dist.all_gather(parts, pf.grad.contiguous())
    assert p.grad.shape == (N // world, x.shape[1])
    if world == 2:
        assert torch.equal(p.grad, (parts[0] + parts[1])[cols]), "weight gradient is not the sum of the partials"
    total = sum(t.float() for t in parts)[cols]
    assert rel(p.grad, total) < 1e-2
    assert rel(p.grad, (gy.float().t() @ x.float())[cols]) < 0.25

    # the update changes the shard: the gathered operands must follow the new version
    opt = bl.Lattice([p], lr=3e-3, direction="sign", phase_bits=4, seed=77, fused_backward=False)
    opt.step()
    full = torch.empty(N, p.packed.shape[1], dtype=torch.uint8, device=dev)
    dist.all_gather_into_tensor(full, p.packed.contiguous())
    assert torch.equal(gathered.operand(p).packed, full) and not torch.equal(full, w.packed)
    assert gathered.t_operand(p).packed.shape == (x.shape[1], N // 2)

    # two layers on one input, gathers prefetched
    pa, pb = torch.nn.Parameter(shard_rows(w, rank, world)), torch.nn.Parameter(shard_rows(w2, rank, world))
    gathered.prefetch((pa, pb))
    with bl.compute("fp4_all"):
        xs2 = xr.detach().requires_grad_(True)
        ya, yb = token_parallel_linears(xs2, (pa, pb), gathered)
        assert torch.equal(ya, yf)
        torch.autograd.backward((ya, yb), (gr, gy2[rows].contiguous()))
    W, W2 = w.dequantize(torch.float32), w2.dequantize(torch.float32)
    assert rel(xs2.grad, gr.float() @ W + gy2[rows].float() @ W2) < 0.25
    cols2 = slice(rank * w2.shape[0] // world, (rank + 1) * w2.shape[0] // world)
    assert rel(pb.grad, (gy2.float().t() @ x.float())[cols2]) < 0.25
    assert rel(pa.grad, (gy.float().t() @ x.float())[cols]) < 0.25


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    M, N, K = 256 * world, 512, 1024
    gen = torch.Generator(device=dev).manual_seed(11)            # same stream on every rank
    wd = torch.randn(N, K, device=dev, generator=gen) * 0.02
    x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
    gy = (torch.randn(M, N, device=dev, generator=gen) * 1e-2).to(torch.bfloat16)
    w = bl.LatticeTensor.from_float(wd, "nvfp4", method="rtn", dtype=torch.bfloat16)
    ws = shard_rows(w, rank, world)
    rows = slice(rank * M // world, (rank + 1) * M // world)
    cols = slice(rank * N // world, (rank + 1) * N // world)

    # operands
    xq, xt = gathered_input_operands(x[rows].contiguous(), None, True)
    ref_q, ref_t = backend._input_operands(x, backend.Fp4Recipe())
    for got, ref in ((xq, ref_q), (xt.get(), ref_t)):
        assert torch.equal(got.packed, ref.packed), "codes differ from the unsharded quantization"
        assert torch.equal(got.scales.view(torch.uint8).reshape(-1), ref.scales.view(torch.uint8).reshape(-1))
        assert torch.equal(got.global_scale, ref.global_scale)

    with bl.compute("fp4_all"):
        p_full = torch.nn.Parameter(w)
        xf = x.detach().requires_grad_(True)
        y_full = torch.nn.functional.linear(xf, p_full)
        y_full.backward(gy)
        p = torch.nn.Parameter(ws)
        xs = x[rows].detach().contiguous().requires_grad_(True)
        y = column_parallel_linear(xs, p, None)
        assert torch.equal(y, y_full[:, cols]), "forward shard differs from the unsharded forward"
        y.backward(gy[:, cols].contiguous())
    W = w.dequantize(torch.float32)
    gx_exact = gy.float() @ W
    gw_exact = gy.float().t() @ x.float()
    assert xs.grad.shape == (M // world, K) and p.grad.shape == (N // world, K)
    # the reference's bound for FP4 gradients against the exact route (tests/test_backend.py:91-94)
    assert rel(xs.grad, gx_exact[rows]) < 0.25, rel(xs.grad, gx_exact[rows])
    assert rel(p.grad, gw_exact[cols]) < 0.25, rel(p.grad, gw_exact[cols])
    # and as close to it as the unsharded layer is (same estimator, different draws)
    assert rel(xs.grad, gx_exact[rows]) < 1.5 * rel(xf.grad, gx_exact) + 1e-3
    assert rel(p.grad, gw_exact[cols]) < 1.5 * rel(p_full.grad, gw_exact) + 1e-3

    # two layers on one input: one gather, one reduce-scatter of the summed input gradient
    wd2 = torch.randn(N // 2, K, device=dev, generator=gen) * 0.02
    gy2 = (torch.randn(M, N // 2, device=dev, generator=gen) * 1e-2).to(torch.bfloat16)
    w2 = bl.LatticeTensor.from_float(wd2, "nvfp4", method="rtn", dtype=torch.bfloat16)
    cols2 = slice(rank * N // 2 // world, (rank + 1) * N // 2 // world)
    with bl.compute("fp4_all"):
        pa, pb = torch.nn.Parameter(shard_rows(w, rank, world)), torch.nn.Parameter(shard_rows(w2, rank, world))
        xs2 = x[rows].detach().contiguous().requires_grad_(True)
        ya, yb = column_parallel_linears(xs2, (pa, pb), None)
        assert torch.equal(ya, y_full[:, cols])
        torch.autograd.backward((ya, yb), (gy[:, cols].contiguous(), gy2[:, cols2].contiguous()))
    gx2_exact = gx_exact + gy2.float() @ w2.dequantize(torch.float32)
    assert rel(xs2.grad, gx2_exact[rows]) < 0.25, rel(xs2.grad, gx2_exact[rows])
    assert rel(pb.grad, (gy2.float().t() @ x.float())[cols2]) < 0.25

    # a token shard that is not a multiple of 128 rows takes the generic route (bf16 all-gather, the layer's own
    # autograd function, reduce-scatter): same forward bits, gradients within the same bounds
    Mo = 96 * world
    xo, gyo = x[:Mo].contiguous(), gy[:Mo].contiguous()
    ro = slice(rank * 96, (rank + 1) * 96)
    with bl.compute("fp4_all"):
        pf = torch.nn.Parameter(w)
        xf2 = xo.detach().requires_grad_(True)
        yo_full = torch.nn.functional.linear(xf2, pf)
        po = torch.nn.Parameter(shard_rows(w, rank, world))
        xso = xo[ro].detach().contiguous().requires_grad_(True)
        yo = column_parallel_linear(xso, po, None)
        assert torch.equal(yo, yo_full[:, cols]), "generic route: forward shard differs from the unsharded forward"
        yo.backward(gyo[:, cols].contiguous())
    assert rel(xso.grad, (gyo.float() @ W)[ro]) < 0.25
    assert rel(po.grad, (gyo.float().t() @ xo.float())[cols]) < 0.25
    # large enough for the backward to split its input-gradient GEMMs into column blocks whose reduce-scatters run
    # under the following GEMMs: the same bits as the unsplit backward under the same stochastic-rounding seeds
    from bitlattice_b200 import parallel
    Mb, Kb, Nb = 4096 * world, 2048, (256, 128)
    xb = torch.randn(Mb, Kb, device=dev, generator=gen).to(torch.bfloat16)
    wbs = [bl.LatticeTensor.from_float(torch.randn(n, Kb, device=dev, generator=gen) * 0.02, "nvfp4", method="rtn",
                                       dtype=torch.bfloat16) for n in Nb]
    gbs = [(torch.randn(Mb, n, device=dev, generator=gen) * 1e-2).to(torch.bfloat16) for n in Nb]
    rb = slice(rank * Mb // world, (rank + 1) * Mb // world)
    got = {}
    for blocks in (4, 1):
        parallel.COLUMN_BLOCKS = blocks
        backend.set_sr_seed(4242)
        backend.clear_shared()
        with bl.compute("fp4_all"):
            ps = [torch.nn.Parameter(shard_rows(wb, rank, world)) for wb in wbs]
            xsb = xb[rb].detach().contiguous().requires_grad_(True)
            ys = column_parallel_linears(xsb, ps, None)
            torch.autograd.backward(ys, [g[:, rank * n // world:(rank + 1) * n // world].contiguous()
                                         for g, n in zip(gbs, Nb)])
        got[blocks] = (xsb.grad, [q.grad for q in ps])
    parallel.COLUMN_BLOCKS = 1
    assert torch.equal(got[4][0], got[1][0]), "column blocks change the input gradient"
    for a, b in zip(got[4][1], got[1][1]):
        assert torch.equal(a, b)
    exact = sum(g.float() @ wb.dequantize(torch.float32) for g, wb in zip(gbs, wbs))
    assert rel(got[4][0], exact[rb]) < 0.25
    token_parallel_checks(rank, world, dev, w, x, gy, w2, gy2)
    # a 128-rotation recipe does not exchange packed operands: both patterns take their generic routes (dense
    # all-gather / reduce-scatter around the local layer) and stay within the reference's bound of the exact gradients
    from bitlattice_b200.parallel import token_parallel_linear
    for fn, xin, rsel in ((column_parallel_linear, x[rows].detach().contiguous(), rows),
                          (token_parallel_linear, x[rows].detach().contiguous(), rows)):
        with bl.compute("quartet2_fast"):
            pq = torch.nn.Parameter(shard_rows(w, rank, world))
            xq_ = xin.clone().requires_grad_(True)
            if fn is column_parallel_linear:
                yq = fn(xq_, pq, None)
                yq.backward(gy[:, cols].contiguous())
            else:
                yq = fn(xq_, pq)
                yq.backward(gy[rows].contiguous())
        assert rel(xq_.grad, gx_exact[rsel]) < 0.25, (fn.__name__, rel(xq_.grad, gx_exact[rsel]))
        want_gw = gw_exact[cols]
        assert rel(pq.grad, want_gw) < 0.25, (fn.__name__, rel(pq.grad, want_gw))
    # colnorm over row shards with the panel sums exchanged (shard_group): every rank ends with exactly its rows of
    # the unsharded update, codes, scales and phase
    Nu = 256 * world
    wu = bl.LatticeTensor.from_float(torch.randn(Nu, K, device=dev, generator=gen) * 0.02, "nvfp4", method="rtn",
                                     dtype=torch.bfloat16)
    Gu = (torch.randn(Nu, K, device=dev, generator=gen) * 1e-2 * (1 + torch.arange(K, device=dev) % 5)).to(torch.bfloat16)
    ru = slice(rank * 256, (rank + 1) * 256)
    kw = dict(lr=3e-3, direction="colnorm", phase_bits=4, seed=21)
    pu = torch.nn.Parameter(wu.detach().clone())
    ou = bl.Lattice([pu], **kw)
    psh = torch.nn.Parameter(shard_rows(wu, rank, world))
    osh = bl.Lattice([psh], shard_group=True, **kw)
    for _ in range(2):
        pu.grad, psh.grad = Gu, Gu[ru].contiguous()
        ou.step()
        osh.step()
    assert torch.equal(psh.packed, pu.packed[ru]), "sharded colnorm update differs from the unsharded one"
    assert torch.equal(psh.scales.view(torch.uint8), pu.scales.view(torch.uint8)[ru])
    assert torch.equal(osh.state[psh]["phase"], ou.state[pu]["phase"][ru])
    # MATCH_UNSHARDED: the gradient columns are quantized with the unsharded tensor's scale and rounding draws, so the
    # weight-gradient shard equals the rows of the unsharded weight gradient bit for bit -- and with the panel sums
    # exchanged the colnorm update leaves exactly the weights the one-GPU step leaves
    Nm = 256 * world
    wm = bl.LatticeTensor.from_float(torch.randn(Nm, K, device=dev, generator=gen) * 0.02, "nvfp4", method="rtn",
                                     dtype=torch.bfloat16)
    gym = (torch.randn(M, Nm, device=dev, generator=gen) * 1e-2).to(torch.bfloat16)
    cm = slice(rank * 256, (rank + 1) * 256)
    parallel.MATCH_UNSHARDED = True
    try:
        with bl.compute("fp4_all"):
            backend.set_sr_seed(9000)
            backend.clear_shared()
            pf = torch.nn.Parameter(wm.detach().clone())
            xf3 = x.detach().requires_grad_(True)
            torch.nn.functional.linear(xf3, pf).backward(gym)
            backend.set_sr_seed(9000)
            backend.clear_shared()
            pm = torch.nn.Parameter(shard_rows(wm, rank, world))
            xs3 = x[rows].detach().contiguous().requires_grad_(True)
            column_parallel_linear(xs3, pm, None).backward(gym[:, cm].contiguous())
    finally:
        parallel.MATCH_UNSHARDED = False
    assert torch.equal(pm.grad, pf.grad[cm]), "weight-gradient shard differs from the unsharded weight gradient"
    assert rel(xs3.grad, xf3.grad[rows]) < 0.2
    kwm = dict(lr=3e-3, direction="colnorm", phase_bits=4, seed=33)
    of, om = bl.Lattice([pf], **kwm), bl.Lattice([pm], shard_group=True, **kwm)
    of.step()
    om.step()
    assert torch.equal(pm.packed, pf.packed[cm]) and torch.equal(om.state[pm]["phase"], of.state[pf]["phase"][cm])
    assert torch.equal(pm.scales.view(torch.uint8), pf.scales.view(torch.uint8)[cm])
    assert bl._ops.gemm_status(local) == 0
    dist.barrier()
    print(f"OK {rank}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
