"""The allocation-free few-token linear entry point against the ordinary one.

`camblas_cuda_linear_bf16_static` serves callers that may not allocate device
memory at the moment they need a product - a process whose own memory pool owns
the device, a latency-bound path that cannot absorb an allocation - by
keeping the split-K partial sums in a fixed array inside the library instead of
a `cudaMalloc`-grown arena. It must give what `camblas_cuda_linear_bf16` gives.
The two are compared within the BF16 tolerance of the other GEMM tests (rel-L2
<= 1e-2; in fact the bits agree because both use the same kernel geometry), on
two calls in a row so that what the first call leaves in the shared array is
shown not to leak into the second. This file sorts last on purpose: a run that
stops at the first failure has then already run every other test.
"""

import ctypes as ct

import numpy as np
import pytest
import torch

from camblas_b200 import _kernels, _native
from oracle import oracle
from tests.helpers import BF16_TOLERANCE, bits_to_tensor, normal_bits, pointer

pytestmark = pytest.mark.gpu


def static_linear(x, w, out=None):
    rows, inner = x.shape
    outputs = w.shape[0]
    if out is None:
        out = torch.empty((rows, outputs), dtype=torch.bfloat16, device=x.device)
    stream = ct.c_void_p(torch.cuda.current_stream().cuda_stream)
    library = _native.library()
    status = library.camblas_cuda_linear_bf16_static(stream, rows, inner, outputs, pointer(x), inner,
                                                     pointer(w), inner, pointer(out), outputs)
    assert status == 0, library.camblas_cuda_error(None).decode()
    return out


def test_static_scratch_linear_matches_context_linear_twice():
    torch.cuda.set_device(0)
    rng = np.random.default_rng(20261125)
    # first call: four rows, a deep K (several splits); second call: one row, another shape
    for rows, outputs, inner in ((4, 1536, 16384), (1, 4096, 8192)):
        x = bits_to_tensor(normal_bits(rng, (rows, inner)))
        w = bits_to_tensor(normal_bits(rng, (outputs, inner), 0.02))
        with _native.kernel_family("skinny"):
            expected = _kernels.linear(x, w)
        actual = static_linear(x, w)
        torch.cuda.synchronize()
        error = oracle.rel_l2(actual.float().cpu().numpy(), expected.float().cpu().numpy())
        assert error <= BF16_TOLERANCE, (rows, outputs, inner, error)
        assert torch.equal(actual, expected)
        reference = oracle.bf16_values(oracle.linear_bf16(
            x[:1].cpu().view(torch.int16).numpy().view(np.uint16),
            w[:64].cpu().view(torch.int16).numpy().view(np.uint16)))
        assert oracle.rel_l2(actual[:1, :64].float().cpu().numpy(), reference) <= BF16_TOLERANCE


def test_static_scratch_linear_leaves_device_memory_alone():
    """Free device memory, as the driver reports it, is the same before and after.

    The buffers are made first and the entry point is called once beforehand,
    so the per-device look-up and the loading of the kernels are not counted.
    `cudaMemGetInfo` sees every allocation on the device whichever allocator
    made it; torch's own counters show that the caching allocator did not
    serve one either. Another process on the same GPU could move the driver's
    figure, so a mismatch is retried before it counts.
    """
    torch.cuda.set_device(0)
    rng = np.random.default_rng(20261126)
    x = bits_to_tensor(normal_bits(rng, (4, 16384)))
    w = bits_to_tensor(normal_bits(rng, (1536, 16384), 0.02))
    out = torch.empty((4, 1536), dtype=torch.bfloat16, device="cuda")
    static_linear(x, w, out)
    torch.cuda.synchronize()
    for attempt in range(3):
        free_before, _ = torch.cuda.mem_get_info()
        torch_before = torch.cuda.memory_stats().get("allocation.all.allocated", 0)
        for _ in range(8):
            static_linear(x, w, out)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        torch_after = torch.cuda.memory_stats().get("allocation.all.allocated", 0)
        assert torch_after == torch_before
        if free_after == free_before:
            break
    assert free_after == free_before, (free_before, free_after)


def test_static_scratch_linear_rejects_what_it_cannot_hold():
    torch.cuda.set_device(0)
    library = _native.library()
    stream = ct.c_void_p(torch.cuda.current_stream().cuda_stream)
    x = torch.zeros((4, 65536), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros((16, 65536), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros((4, 16), dtype=torch.bfloat16, device="cuda")
    # five rows are outside the entry point's range
    assert library.camblas_cuda_linear_bf16_static(stream, 5, 64, 16, pointer(x), 64, pointer(w), 64,
                                                   pointer(out), 16) == -1
    assert b"1 to 4 token rows" in library.camblas_cuda_error(None)
    # 4 rows x 40000 outputs x 16 splits x 4 bytes = 10 MiB of partial sums: more than the array
    # holds; the sizes are checked before anything is launched, so small buffers are enough here
    status = library.camblas_cuda_linear_bf16_static(stream, 4, 65536, 40000, pointer(x), 65536,
                                                     pointer(w), 65536, pointer(out), 40000)
    assert status == -1
    message = library.camblas_cuda_error(None).decode()
    assert "static scratch too small" in message and str(8 << 20) in message
    assert library.camblas_cuda_linear_bf16_static(stream, 0, 64, 16, None, 64, None, 64, None, 16) == 0
