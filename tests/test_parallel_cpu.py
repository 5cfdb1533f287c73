"""The N-sharded layer's bookkeeping on two gloo ranks (CPU): gathered input, feature-sharded output, reduce-scattered
input gradient and local weight-gradient shards agree with the unsharded layer."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from bitlattice_b200.parallel import column_parallel_linear, shard_bounds, world


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
