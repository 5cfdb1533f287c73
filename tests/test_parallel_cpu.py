"""The N-sharded layer's bookkeeping on two gloo ranks (CPU): gathered input, feature-sharded output, reduce-scattered
input gradient and local weight-gradient shards agree with the unsharded layer; so do the token-parallel layer's
gathered weight, token-sharded output and reduce-scattered weight gradient."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from bitlattice_b200.parallel import column_parallel_linear, shard_bounds, token_parallel_linear, world


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, size, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=size)
    try:
        g = torch.Generator().manual_seed(0)
        M, K, N = 8 * size, 16, 64 * size
        x = torch.randn(M, K, generator=g)
        W = torch.randn(N, K, generator=g)
        gy = torch.randn(M, N, generator=g)
        # unsharded
        xr, Wr = x.clone().requires_grad_(True), W.clone().requires_grad_(True)
        torch.nn.functional.linear(xr, Wr).backward(gy)
        # sharded
        lo, hi = shard_bounds(N, rank, size)
        rows = M // size
        xs = x[rank * rows:(rank + 1) * rows].clone().requires_grad_(True)
        Ws = W[lo:hi].clone().requires_grad_(True)
        y = column_parallel_linear(xs, Ws)
        assert world() == (rank, size) and y.shape == (M, N // size)
        y.backward(gy[:, lo:hi].contiguous())
        ok = (torch.allclose(y, (x @ W.t())[:, lo:hi], atol=1e-5)
              and torch.allclose(xs.grad, xr.grad[rank * rows:(rank + 1) * rows], atol=1e-4)
              and torch.allclose(Ws.grad, Wr.grad[lo:hi], atol=1e-4))
        # the other exchange pattern over the same row shards: the rank keeps its tokens, the weight is gathered and
        # the weight-gradient partials are reduce-scattered to the shard owners
        xt = x[rank * rows:(rank + 1) * rows].clone().requires_grad_(True)
        Wt = W[lo:hi].clone().requires_grad_(True)
        yt = token_parallel_linear(xt, Wt)
        assert yt.shape == (rows, N)
        yt.backward(gy[rank * rows:(rank + 1) * rows].contiguous())
        ok = (ok and torch.allclose(yt, (x @ W.t())[rank * rows:(rank + 1) * rows], atol=1e-5)
              and torch.allclose(xt.grad, xr.grad[rank * rows:(rank + 1) * rows], atol=1e-4)
              and torch.allclose(Wt.grad, Wr.grad[lo:hi], atol=1e-4))
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("size", [2])
def test_column_parallel_linear_on_gloo(size):
    ctx = mp.get_context("spawn")
    out = ctx.Manager().dict()
    procs = [ctx.Process(target=_worker, args=(r, size, _free_port_once(), out)) for r in range(size)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert all(out.get(r) for r in range(size)), dict(out)


_PORT = []


def _free_port_once():
    if not _PORT:
        _PORT.append(_free_port())
    return _PORT[0]


def test_shard_bounds():
    assert shard_bounds(4096, 3, 8) == (1536, 2048)
    assert shard_bounds(1024, 0, 1) == (0, 1024)
    with pytest.raises(ValueError):
        shard_bounds(1024 + 32, 0, 8)


def test_single_process_degenerates_to_plain_linear():
    x, W = torch.randn(4, 8), torch.randn(6, 8)
    assert torch.equal(column_parallel_linear(x, W), torch.nn.functional.linear(x, W))
    assert torch.equal(token_parallel_linear(x, W), torch.nn.functional.linear(x, W))


def _io_worker(rank, size, port, out, ckpt, tmp):
    """Every rank holds its row shard of the lattice weight of a checkpoint; a sharded save must reproduce the
    unsharded checkpoint, and a sharded load must hand each rank exactly its rows."""
    import bitlattice_b200 as bl
    from bitlattice_b200.parallel import shard_rows
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=size)
    try:
        full = bl.io.load_state(ckpt)
        state = dict(full)
        state["up.weight"] = shard_rows(full["up.weight"], rank, size)
        bl.io.save(state, tmp)
        again = bl.io.load_state(tmp)
        ok = all(torch.equal(getattr(again["up.weight"], k).view(torch.uint8), getattr(full["up.weight"], k).view(torch.uint8))
                 for k in ("packed", "scales", "global_scale"))
        ok = ok and tuple(again["up.weight"].shape) == (64, 64) and torch.equal(again["down.weight"], full["down.weight"])

        class Tiny(torch.nn.Module):
            def __init__(self):
                super().__init__()
                self.up = torch.nn.Linear(64, 64 // size)
                self.down = torch.nn.Linear(64, 32)
                self.register_buffer("steps", torch.zeros(5, dtype=torch.int64))
        m = Tiny().to(torch.bfloat16)
        m.up.weight = torch.nn.Parameter(state["up.weight"])           # the row offset travels with the shard
        m.up.bias = torch.nn.Parameter(full["up.bias"].clone())
        m.up.weight.packed.zero_()
        bl.io.load_into(m, tmp)
        lo, hi = rank * 64 // size, (rank + 1) * 64 // size
        ok = ok and torch.equal(m.up.weight.packed, full["up.weight"].packed[lo:hi])
        ok = ok and m.up.weight._bl_row_offset == lo and tuple(m.up.weight.shape) == (64 // size, 64)
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_sharded_checkpoint_round_trip_on_gloo(tmp_path):
    size = 2
    ckpt = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ckpt")
    ctx = mp.get_context("spawn")
    out = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_io_worker, args=(r, size, port, out, ckpt, str(tmp_path / "sharded")))
             for r in range(size)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert all(out.get(r) for r in range(size)), dict(out)


def _exchange_worker(rank, size, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=size)
    try:
        from bitlattice_b200.optim.lattice import Lattice
        opt = object.__new__(Lattice)                 # the exchange reads nothing but the group
        opt.shard_group = True
        blocks = torch.full((size, 37), -1.0)
        blocks[rank] = torch.arange(37, dtype=torch.float32) + 100 * rank      # this owner's panel sums
        opt._exchange(blocks)
        want = torch.stack([torch.arange(37, dtype=torch.float32) + 100 * r for r in range(size)])
        out[rank] = bool(torch.equal(blocks, want)) and opt._shard_world()[:2] == (size, rank)
    finally:
        dist.destroy_process_group()


def test_panel_sum_exchange_is_an_in_place_all_gather_on_gloo():
    """``Lattice._exchange`` (whole-weight statistics over row shards): every rank has written its own row of the
    exchange area; afterwards every rank holds all rows."""
    size = 2
    ctx = mp.get_context("spawn")
    out = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_exchange_worker, args=(r, size, port, out)) for r in range(size)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert all(out.get(r) for r in range(size)), dict(out)
