"""One rank of the multi-GPU row-parallel test (run by test_row_parallel_multi_gpu.py).

Usage: python -m tests.row_parallel_worker (RANK, WORLD_SIZE, LOCAL_RANK, MASTER_ADDR,
MASTER_PORT in the environment). Prints one line "rank R OK" or raises.
"""

import os
import sys

import numpy as np
import torch
import torch.distributed as dist


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    device = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=torch.device("cuda", device))
    from camblas_b200 import _kernels, _native
    from camblas_b200.tp import PeerRegions, RowParallelLinear

    rows, inner, outputs = 512, 1024 * world, 2048
    generator = torch.Generator().manual_seed(705537)
    x = torch.randn((rows, inner), generator=generator).bfloat16().cuda()
    w = (torch.randn((outputs, inner), generator=generator) * 0.05).bfloat16().cuda()
    bias = torch.randn((outputs,), generator=generator).bfloat16().cuda()

    peers = PeerRegions.create(PeerRegions.capacity_for(rows, outputs), device)
    fused = RowParallelLinear(w, rank, world, bias=bias, peers=peers)
    plain = RowParallelLinear(w, rank, world, bias=bias)
    x_local = fused.slice_input(x)

    expected = plain(x_local).float()
    results = []
    for _ in range(3):
        results.append(fused(x_local).clone())
    torch.cuda.synchronize()
    status = _native.context(device).device_status()
    assert status == 0, f"device status {status:#x}"

    error = (results[0].float() - expected).norm() / expected.norm()
    assert error.item() <= 1e-2, f"rel-L2 against the NCCL path {error.item():.3e}"
    full = _kernels.linear(x, w, bias).float()
    error = (results[0].float() - full).norm() / full.norm()
    assert error.item() <= 1e-2, f"rel-L2 against the unsharded product {error.item():.3e}"
    for repeat in results[1:]:
        assert torch.equal(repeat, results[0]), "repeated calls differ"
    gathered = [torch.empty_like(results[0]) for _ in range(world)]
    dist.all_gather(gathered, results[0])
    for other in gathered:
        assert torch.equal(other, results[0]), "ranks hold different results"

    # decode-sized rows: product, then the one-shot peer all-reduce instead of NCCL's
    for tokens in (1, 16, 64):
        x_small = torch.randn((tokens, inner), generator=generator).bfloat16().cuda()
        local = fused.slice_input(x_small)
        summed = [fused(local).clone() for _ in range(3)]
        reference = plain(local)
        torch.cuda.synchronize()
        assert _native.context(device).device_status() == 0
        for repeat in summed[1:]:
            assert torch.equal(repeat, summed[0]), "repeated small all-reduces differ"
        error = (summed[0].float() - reference.float()).norm() / reference.float().norm()
        assert error.item() <= 1e-2, f"small all-reduce against NCCL {error.item():.3e}"
        whole = _kernels.linear(x_small, w, bias).float()
        error = (summed[0].float() - whole).norm() / whole.norm()
        assert error.item() <= 1e-2, f"small all-reduce against the unsharded product {error.item():.3e}"
        gathered = [torch.empty_like(summed[0]) for _ in range(world)]
        dist.all_gather(gathered, summed[0])
        for other in gathered:
            assert torch.equal(other, summed[0]), "ranks hold different sums"

    torch.cuda.synchronize()
    dist.barrier()
    peers.close(free=False)  # unmap the others' regions before anyone frees its own
    dist.barrier()
    peers.close(free=True)
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank} OK", flush=True)


if __name__ == "__main__":
    sys.exit(main())
