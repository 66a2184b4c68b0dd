"""B200-native CUDA GEMM path with the operator surface of camblas.

``_autoload`` is the ``torch.backends`` entry point of the reference
(``camblas/__init__.py:6-29``): when ``CAMBLAS_ENABLE=1`` it routes
``aten::mm``, ``mm.out`` and ``addmm`` for eligible CUDA tensors through
``libcamblas_cuda.so``. The algorithm comes from ``CAMBLAS_CUDA_ALGORITHM`` (or
``CAMBLAS_SGLANG_ALGORITHM``), default ``lt``.
"""

import os


def _autoload():
    """Install the ATen overrides when the process enables CAMBLAS."""
    if os.environ.get("CAMBLAS_ENABLE", "0") != "1":
        return
    from ._native import _ALGORITHMS
    from ._torch_backend import install_torch_backend

    name = os.environ.get(
        "CAMBLAS_CUDA_ALGORITHM", os.environ.get("CAMBLAS_SGLANG_ALGORITHM", "lt")
    )
    if name not in _ALGORITHMS:
        raise ValueError(f"Unknown CAMBLAS CUDA algorithm: {name}")
    install_torch_backend(name)
