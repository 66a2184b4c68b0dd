"""ATen overrides: route eligible CUDA ``mm``, ``mm.out`` and ``addmm`` through the C ABI.

The reference registers C++ kernels for ``DispatchKey::CUDA`` and falls back to
``at::cuda::mm`` for anything it does not take (``src/cuda/torch_backend.cuh:7-88``).
Here the registration is made from Python with ``torch.library``; the kernels
ATen had registered for the CUDA key are captured first with
``torch.library.get_kernel`` and are what ineligible calls fall back to, so a
fallback never re-enters these overrides. Only BF16 is intercepted: the FP32 and
FP64 GEMMs of the reference are not part of this build.
"""

import threading

import torch

from . import _kernels, _native

_INT_MAX = 2**31 - 1
_LOCK = threading.Lock()
_LIBRARY = None
_ORIGINAL = {}
_ALGORITHM = "lt"


def torch_matrix_supported(a, b):
    """Eligibility of ``a @ b`` (the predicate of ``torch_backend.cuh:7-28``, BF16 only)."""
    if not (a.is_cuda and b.is_cuda and a.layout == torch.strided and b.layout == torch.strided):
        return False
    if a.dim() != 2 or b.dim() != 2 or a.device != b.device or a.dtype != b.dtype:
        return False
    if a.dtype != torch.bfloat16 or a.shape[1] != b.shape[0]:
        return False
    if a.is_conj() or b.is_conj() or a.is_neg() or b.is_neg():
        return False
    for tensor in (a, b):
        if any(size == 0 or size > _INT_MAX for size in tensor.shape):
            return False
        if any(stride < 0 or stride > _INT_MAX for stride in tensor.stride()):
            return False
    return True


def _bias_supported(bias, a, b):
    if bias.device != a.device or bias.dtype != a.dtype or bias.layout != torch.strided:
        return False
    if bias.dim() > 2 or bias.is_conj() or bias.is_neg():
        return False
    if bias.dim() >= 1 and bias.shape[-1] not in (1, b.shape[1]):
        return False
    return bias.dim() < 2 or bias.shape[0] in (1, a.shape[0])


def _mm(keyset, a, b):
    if not torch_matrix_supported(a, b):
        return _ORIGINAL["mm"].call_boxed(keyset, a, b)
    with _native.algorithm(_ALGORITHM):
        return _kernels.matmul(a, b)


def _mm_out(keyset, a, b, out):
    eligible = (
        torch_matrix_supported(a, b)
        and out.device == a.device
        and out.dtype == a.dtype
        and out.layout == torch.strided
        and out.dim() == 2
        and out.shape[0] == a.shape[0]
        and out.shape[1] == b.shape[1]
        and out.is_contiguous()
        and not out.is_conj()
        and not out.is_neg()
        and out.untyped_storage().data_ptr() != a.untyped_storage().data_ptr()
        and out.untyped_storage().data_ptr() != b.untyped_storage().data_ptr()
    )
    if not eligible:
        return _ORIGINAL["mm.out"].call_boxed(keyset, a, b, out)
    with _native.algorithm(_ALGORITHM):
        _kernels.matmul(a, b, out=out)
    return out


def _addmm(keyset, bias, a, b, beta=1, alpha=1):
    if (not torch_matrix_supported(a, b) or not _bias_supported(bias, a, b)
            or isinstance(beta, complex) or isinstance(alpha, complex)):
        return _ORIGINAL["addmm"].call_boxed(keyset, bias, a, b, beta, alpha)
    beta, alpha = float(beta), float(alpha)
    with _native.algorithm(_ALGORITHM):
        # F.linear's shape: 1-D bias over the outputs, weight given as W.t():
        # the bias goes into the GEMM epilogue instead of being materialised.
        if (beta == 1.0 and alpha == 1.0 and bias.dim() == 1 and bias.shape[0] == b.shape[1]
                and bias.is_contiguous() and b.stride(0) == 1 and b.stride(1) >= b.shape[0]
                and a.stride(1) == 1 and a.stride(0) >= a.shape[1]):
            return _kernels.linear(a, b.t(), bias)
        if beta == 0.0:
            return _kernels.matmul(a, b, alpha=alpha)
        out = bias.expand(a.shape[0], b.shape[1]).clone(memory_format=torch.contiguous_format)
        return _kernels.matmul(a, b, out=out, alpha=alpha, beta=beta)


def install_torch_backend(algorithm="lt"):
    """Register the overrides once per process (``torch_backend.cuh:73-88``).

    Parameters
    ----------
    algorithm : str
        Policy name from the algorithm table; used for every intercepted call.
    """
    global _LIBRARY, _ALGORITHM
    with _LOCK:
        if _LIBRARY is not None:
            return
        if algorithm not in _native._ALGORITHMS:
            raise ValueError(f"Invalid CAMBLAS CUDA algorithm: {algorithm}")
        _native.library()  # fail now, loudly, if the kernels are not built
        _ALGORITHM = algorithm
        for name in ("mm", "mm.out", "addmm"):
            _ORIGINAL[name] = torch.library.get_kernel("aten::" + name, "CUDA")
        library = torch.library.Library("aten", "IMPL")
        library.impl("mm", _mm, "CUDA", with_keyset=True)
        library.impl("mm.out", _mm_out, "CUDA", with_keyset=True)
        library.impl("addmm", _addmm, "CUDA", with_keyset=True)
        _LIBRARY = library


def installed():
    """Return whether the overrides are active in this process."""
    return _LIBRARY is not None
