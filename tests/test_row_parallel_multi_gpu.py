"""The peer-memory row-parallel layer with one process per GPU (needs two GPUs).

Each rank runs `tests/row_parallel_worker.py`: regions exchanged as CUDA IPC
handles, the fused product compared with the NCCL all-reduce path and with the
unsharded product (rel-L2 <= 1e-2), repeated calls and all ranks bit-identical.
NVLS is switched off for NCCL so that no rank's memory is bound to an NVLink
group object while another rank exits. Skipped on a single-GPU machine, where
`tests/test_row_parallel_gpu.py` covers the kernels with emulated ranks.
"""

import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def free_port():
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        return probe.getsockname()[1]


@pytest.mark.parametrize("world", [2])
def test_ranks_in_processes(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = free_port()
    children = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world),
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        children.append(subprocess.Popen([sys.executable, "-m", "tests.row_parallel_worker"],
                                         cwd=ROOT, env=env, stdout=subprocess.PIPE,
                                         stderr=subprocess.STDOUT, text=True))
    outputs = []
    try:
        for child in children:
            text, _ = child.communicate(timeout=300)
            outputs.append(text)
    finally:
        for child in children:
            if child.poll() is None:
                child.kill()
    for rank, (child, text) in enumerate(zip(children, outputs)):
        assert child.returncode == 0, f"rank {rank} failed:\n{text[-3000:]}"
        assert f"rank {rank} OK" in text
