"""Child process of test_alloc_faults_gpu.py: runs with the cudaMalloc shim preloaded."""

import ctypes as ct
import sys

import torch

from camblas_b200 import _kernels, _native


def main():
    shim = ct.CDLL(None)
    shim.alloc_shim_calls.restype = ct.c_long
    shim.alloc_shim_fail_after.argtypes = [ct.c_long]
    torch.cuda.set_device(0)
    library = _native.library()
    torch.manual_seed(7)

    # 1. scratch growth fails: negative status, message, clean CUDA state, context usable
    x = torch.randn(16, 8192, device="cuda").bfloat16()
    w = (torch.randn(1024, 8192, device="cuda") * 0.02).bfloat16()
    native = _native.context(0)
    torch.cuda.synchronize()
    shim.alloc_shim_reset()
    shim.alloc_shim_fail_after(0)
    out = torch.zeros(16, 1024, device="cuda", dtype=torch.bfloat16)  # torch's own pool: no cudaMalloc
    status = library.camblas_cuda_linear_bf16(native.handle, 16, 8192, 1024, x.data_ptr(), 8192,
                                              w.data_ptr(), 8192, None, None, 0, out.data_ptr(), 1024)
    if shim.alloc_shim_pending():  # torch allocated first after all: retry with everything resident
        raise SystemExit("the armed failure was not consumed by the library call")
    assert status == -2, status  # -cudaErrorMemoryAllocation
    assert b"scratch allocation failed (status 2)" in library.camblas_cuda_error(native.handle)
    good = _kernels.linear(x, w)  # same call, allocation allowed now: the context still works
    torch.cuda.synchronize()
    reference = torch.nn.functional.linear(x.float(), w.float())
    assert ((good.float() - reference).norm() / reference.norm()).item() <= 1e-2
    assert native.device_status() == 0

    # 2. a Strassen product that cannot get its planes falls back to the classical kernel
    #    and counts it, as the reference does (backend.cu:490-526)
    a = (torch.rand(2048, 2048, device="cuda") * 2 - 1).bfloat16()  # its planes need 59 MB, more than any arena so far
    b = (torch.rand(2048, 2048, device="cuda") * 2 - 1).bfloat16()
    classical = _kernels.matmul(a, b)
    fresh = torch.empty_like(classical)
    torch.cuda.synchronize()
    _native.stats(0, reset=True)
    shim.alloc_shim_fail_after(0)
    with _native.algorithm("strassen"), _native.options(bf16_strassen=1):
        _kernels.matmul(a, b, out=fresh)
    torch.cuda.synchronize()
    assert not shim.alloc_shim_pending()
    counts = _native.stats(0)
    assert counts["guard_fallback"] == 1 and counts["strassen"] == 0, counts
    assert torch.equal(fresh, classical)
    with _native.algorithm("strassen"), _native.options(bf16_strassen=1):
        _kernels.matmul(a, b, out=fresh)  # with memory available it does run Strassen
    assert _native.stats(0)["strassen"] == 1

    # 3. peer region allocation fails
    memory = ct.c_void_p()
    shim.alloc_shim_fail_after(0)
    status = library.camblas_cuda_peer_alloc(native.handle, 1 << 20, ct.byref(memory), None)
    assert status == -2 and not memory.value
    assert b"peer region allocation" in library.camblas_cuda_error(native.handle)
    assert library.camblas_cuda_peer_alloc(native.handle, 1 << 20, ct.byref(memory), None) == 0
    assert library.camblas_cuda_peer_free(native.handle, memory) == 0

    # 4. context creation fails on its first allocation and leaves nothing behind
    stream = torch.cuda.Stream()
    handle = ct.c_void_p()
    shim.alloc_shim_fail_after(0)
    status = library.camblas_cuda_create(0, ct.c_void_p(stream.cuda_stream), ct.byref(handle))
    assert status == -2 and not handle.value
    assert b"status word allocation failed" in library.camblas_cuda_error(None)
    assert library.camblas_cuda_create(0, ct.c_void_p(stream.cuda_stream), ct.byref(handle)) == 0
    assert library.camblas_cuda_destroy(handle) == 0

    # 5. the allocation-free entry point makes no cudaMalloc call at all, first call included
    xs = torch.randn(4, 16384, device="cuda").bfloat16()
    ws = (torch.randn(1536, 16384, device="cuda") * 0.02).bfloat16()
    outs = torch.empty(4, 1536, device="cuda", dtype=torch.bfloat16)
    torch.cuda.synchronize()
    shim.alloc_shim_reset()
    shim.alloc_shim_fail_after(0)  # any allocation would fail and be noticed
    for _ in range(3):
        status = library.camblas_cuda_linear_bf16_static(
            ct.c_void_p(torch.cuda.current_stream().cuda_stream), 4, 16384, 1536, xs.data_ptr(), 16384,
            ws.data_ptr(), 16384, outs.data_ptr(), 1536)
        assert status == 0, library.camblas_cuda_error(None)
    torch.cuda.synchronize()
    assert shim.alloc_shim_calls() == 0 and shim.alloc_shim_pending()
    shim.alloc_shim_reset()
    with _native.kernel_family("skinny"):
        assert torch.equal(outs, _kernels.linear(xs, ws))
    print("alloc faults OK", flush=True)


if __name__ == "__main__":
    sys.exit(main())
