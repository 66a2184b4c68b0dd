"""Tensor-parallel layers on CPU: two `gloo` ranks, host matmul standing in for the CUDA GEMM."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from camblas_b200 import tp


def test_shard_bounds_and_qkv_heads():
    assert tp.shard_bounds(57344, 3, 8, 128) == (21504, 28672)
    with pytest.raises(ValueError):
        tp.shard_bounds(1536, 0, 8, 128)  # 192 per rank is not a whole FP8 scale block
    weight = torch.arange(10 * 4 * 3, dtype=torch.float32).reshape(40, 3)  # 6 q + 2 k + 2 v heads of 4
    shard, widths = tp.shard_qkv(weight, 6, 2, 4, 1, 2)
    assert widths == (12, 4, 4)
    expected = torch.cat([weight[12:24], weight[28:32], weight[36:40]])
    assert torch.equal(shard, expected)
    with pytest.raises(ValueError):
        tp.shard_qkv(weight, 6, 2, 4, 0, 4)


def _host_linear(x, weight, bias=None, residual=None):
    out = x.float() @ weight.float().t()
    if bias is not None:
        out = out + bias.float()
    return out.to(x.dtype)


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    generator = torch.Generator().manual_seed(7)
    x = torch.randn(6, 64, generator=generator)
    gate_up = torch.randn(256, 64, generator=generator)
    down = torch.randn(64, 128, generator=generator)
    bias = torch.randn(64, generator=generator)
    hidden = torch.randn(6, 128, generator=generator)
    column = tp.ColumnParallelLinear(gate_up, rank, world, linear=_host_linear, multiple=128)
    local = column(x)
    gathered = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(gathered, local)
    row = tp.RowParallelLinear(down, rank, world, bias=bias, linear=_host_linear)
    reduced = row(row.slice_input(hidden))
    if rank == 0:
        results["column"] = torch.allclose(torch.cat(gathered, dim=1), x @ gate_up.t(), atol=1e-4)
        results["row"] = torch.allclose(reduced, hidden @ down.t() + bias, atol=1e-4)
        results["bounds"] = (column.bounds, row.bounds)
    dist.barrier()
    dist.destroy_process_group()


def test_column_and_row_parallel_layers_with_two_gloo_ranks():
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    assert results["column"] and results["row"]
    assert results["bounds"] == ((0, 128), (0, 64))


def test_peer_region_capacity_counts_whole_tiles():
    """Staging holds whole 256 x 256 tiles: both extents round up to multiples of 256."""
    from camblas_b200.tp import PeerRegions

    assert PeerRegions.capacity_for(512, 8192) == 512 * 8192
    assert PeerRegions.capacity_for(300, 1000) == 512 * 1024
    assert PeerRegions.capacity_for(1, 8) == 256 * 256


def _failing_linear(x, weight, bias=None, residual=None):
    raise RuntimeError("injected: this rank's GEMM failed")


def _faulty_worker(rank, world, port, results):
    """Rank 1's product raises before the sum; rank 0 must get an error, not wait for ever."""
    import datetime
    import time

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=5))
    generator = torch.Generator().manual_seed(7)
    down = torch.randn(64, 128, generator=generator)
    hidden = torch.randn(6, 128, generator=generator)
    linear = _failing_linear if rank == 1 else _host_linear
    row = tp.RowParallelLinear(down, rank, world, linear=linear)
    dist.barrier()
    started = time.monotonic()
    try:
        row(row.slice_input(hidden))
        results[rank] = ("returned", time.monotonic() - started)
    except RuntimeError as error:
        results[rank] = ("raised", time.monotonic() - started, str(error)[:80])
    # no collective after a failure: the ranks leave on their own


def test_a_rank_that_fails_before_the_sum_gives_the_others_an_error_not_a_hang():
    """Failure injected on the host (an exception in one rank's GEMM): the rank that did
    compute its partial product finds out through the process group's timeout and gets a
    RuntimeError from the all-reduce within seconds; nothing waits indefinitely."""
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    import time

    context = mp.spawn(_faulty_worker, args=(2, port, results), nprocs=2, join=False)
    deadline = time.monotonic() + 90
    while not context.join(timeout=5):  # joins the ranks one at a time
        assert time.monotonic() < deadline, "the ranks did not finish: a hang"
    assert results[1][0] == "raised" and "injected" in results[1][2]
    assert results[0][0] == "raised", results[0]
    assert results[0][1] < 30
