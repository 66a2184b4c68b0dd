"""The C-ABI library loads without a GPU and exports what the header declares."""

import ctypes as ct
import re
from pathlib import Path

import pytest
import torch

from camblas_b200 import _kernels, _native

ROOT = Path(__file__).resolve().parents[1]

# the 28 entry points of the reference header (include/camblas_cuda.h:39-215)
REFERENCE_SYMBOLS = """create destroy error set_algorithm sgemm dgemm bgemm affine mlp attention
mlp_backward silu_multiply swiglu quantized_matmul fp8_decode_supported fp8_decode
fp8_workspace_size fp8_linear grouped_quantized_matmul route_groups reduce_groups rms_norm
rms_norm_decode add_rms_norm bfloat16_square rms_scale stats reset_stats""".split()


def declared_symbols():
    text = (ROOT / "include" / "camblas_cuda.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(camblas_cuda_\w+)\s*\(", text)))


def test_header_declares_every_reference_symbol():
    declared = declared_symbols()
    for name in REFERENCE_SYMBOLS:
        assert "camblas_cuda_" + name in declared


def test_library_exports_every_declared_symbol():
    library = ct.CDLL(str(_native.library_path()))
    for name in declared_symbols():
        assert hasattr(library, name), name
    assert sorted(_native.EXPORTED) == declared_symbols()


def test_host_only_entry_points_behave_without_a_device():
    library = _native.library()
    assert library.camblas_cuda_fp8_workspace_size(0, 4096, 1024) == 0
    assert library.camblas_cuda_destroy(None) == 0
    # a NULL context is a failure with a thread-local message, not a crash
    assert library.camblas_cuda_set_algorithm(None, 0) < 0
    assert b"invalid algorithm" in library.camblas_cuda_error(None)
    assert library.camblas_cuda_reset_stats(None) < 0
    assert b"missing context" in library.camblas_cuda_error(None)
    if not torch.cuda.is_available():
        handle = ct.c_void_p()
        assert library.camblas_cuda_create(0, None, ct.byref(handle)) < 0
        assert not handle.value
        assert library.camblas_cuda_error(None)


def test_python_validation_raises_before_any_launch():
    x = torch.zeros(2, 8, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        _kernels.matmul(x, x.t())  # CPU tensors
    with pytest.raises(ValueError):
        _kernels.linear(x, x)
    with pytest.raises(ValueError):
        _native.set_algorithm("fastest")
    with pytest.raises(ValueError):
        with _native.algorithm("nope"):
            pass
    with pytest.raises(ValueError):
        with _native.kernel_family("nope"):
            pass


def test_operand_mapping_matches_reference_rule():
    base = torch.zeros(6, 10, dtype=torch.bfloat16)
    tensor, flag, ld = _kernels._operand(base)
    assert (flag, ld) == (b"N", 10) and tensor is base
    tensor, flag, ld = _kernels._operand(base.t())
    assert (flag, ld) == (b"T", 10)
    tensor, flag, ld = _kernels._operand(base[:, :4])
    assert (flag, ld) == (b"N", 10)
    tensor, flag, ld = _kernels._operand(base[:, ::2])
    assert (flag, ld) == (b"N", 5) and tensor.is_contiguous()


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setenv("CAMBLAS_CUDA_LIBRARY", str(tmp_path / "absent.so"))
    _native.library.cache_clear()
    try:
        with pytest.raises(RuntimeError, match="missing"):
            _native.library()
    finally:
        monkeypatch.delenv("CAMBLAS_CUDA_LIBRARY")
        _native.library.cache_clear()


def test_peer_region_size_is_host_arithmetic():
    """camblas_cuda_peer_bytes: result + world staging slots (256-byte aligned) + 65536 flag
    words + two buffers of one 2 MiB slot of flagged lines per rank."""
    library = _native.library()
    slot = (1000 * 2 + 255) // 256 * 256
    lines = 2 * 64 * 8192 * 4  # per rank: two buffers, 16 bytes per 8 bytes of a 1 MiB tensor
    assert library.camblas_cuda_peer_bytes(2, 1000) == slot * 3 + 65536 * 4 + 2 * lines
    assert library.camblas_cuda_peer_bytes(8, 512 * 8192) == (512 * 8192 * 2 * 9 + 65536 * 4
                                                               + 8 * lines)
    assert library.camblas_cuda_peer_bytes(9, 1000) == 0
    assert library.camblas_cuda_peer_bytes(0, 1000) == 0
    assert library.camblas_cuda_peer_bytes(2, 0) == 0
