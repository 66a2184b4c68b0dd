"""Helpers shared by the GPU parity tests: tensors <-> numpy bit patterns, raw C-ABI calls."""

import ctypes as ct

import numpy as np
import torch

from camblas_b200 import _native
from oracle import oracle

BF16_TOLERANCE = 1e-2  # rel-L2 bound for BF16 outputs
FP8_TOLERANCE = 2e-2  # rel-L2 bound for FP8 outputs


def bits_to_tensor(bits, device="cuda"):
    """uint16 BF16 bit patterns (numpy) -> torch.bfloat16 tensor on the device."""
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16).to(device)


def tensor_to_bits(tensor):
    """torch.bfloat16 tensor -> uint16 bit patterns on the host."""
    return tensor.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def normal_bits(rng, shape, scale=1.0):
    return oracle.bf16_bits((rng.standard_normal(shape) * scale).astype(np.float32))


def pointer(tensor):
    return ct.c_void_p(tensor.data_ptr()) if tensor is not None else ct.c_void_p()


def native(device=0):
    return _native.context(device)


def raw(name, *arguments, device=0):
    """Call camblas_cuda_<name> on the current stream's context and return the raw status."""
    context = _native.context(device)
    return getattr(_native.library(), "camblas_cuda_" + name)(context.handle, *arguments), context


def error_text(context):
    return _native.library().camblas_cuda_error(context.handle).decode()


def ulp_distance_bf16(a_bits, b_bits):
    """Distance in BF16 units-in-the-last-place between two bit-pattern arrays (finite values)."""
    def ordered(bits):
        signed = bits.astype(np.int32)
        return np.where(signed & 0x8000, 0x8000 - signed, signed)
    return np.abs(ordered(a_bits) - ordered(b_bits))
