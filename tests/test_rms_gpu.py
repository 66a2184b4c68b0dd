"""Residual add + RMS norm and the elementwise kernels against the CPU oracle.

`added` is compared bit for bit. The normalised output is compared within one
BF16 unit in the last place, because the device's rsqrt is an approximation
(<= 2 ulp in FP32) while the oracle takes 1/sqrt in double; the reference's own
tests use rtol 0.02 / atol 0.002 for BF16 (tests/test_residual_rms.py:70-80).
"""

import numpy as np
import pytest
import torch

from camblas_b200 import _kernels, _native
from oracle import oracle
from tests.helpers import (bits_to_tensor, error_text, normal_bits, pointer, raw, tensor_to_bits,
                           ulp_distance_bf16)

pytestmark = pytest.mark.gpu


def gamma_bits(rng, width):
    return oracle.bf16_bits((1 + 0.1 * rng.standard_normal(width)).astype(np.float32))


@pytest.mark.parametrize("rows,width", [(1, 2048), (1, 8192), (3, 4096), (512, 8192), (2, 65536),
                                        (5, 4), (7, 1000)])
def test_add_rms_norm_rows_bf16(rng, rows, width):
    x, r, g = normal_bits(rng, (rows, width)), normal_bits(rng, (rows, width)), gamma_bits(rng, width)
    expected_added, expected = oracle.add_rms_norm_rows(x, r, g, 1e-5)
    added, out = _kernels.add_rms_norm(bits_to_tensor(x), bits_to_tensor(r), bits_to_tensor(g), 1e-5)
    assert np.array_equal(tensor_to_bits(added), expected_added)
    distance = ulp_distance_bf16(tensor_to_bits(out), expected)
    assert distance.max() <= 1, distance.max()
    assert (distance > 0).mean() < 0.02


def test_add_rms_norm_fp32(rng):
    rows, width = 4, 4096
    x = rng.standard_normal((rows, width)).astype(np.float32)
    r = rng.standard_normal((rows, width)).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(width)).astype(np.float32)
    expected_added, expected = oracle.add_rms_norm_rows(x, r, g, 1e-6)
    added, out = _kernels.add_rms_norm(torch.from_numpy(x).cuda(), torch.from_numpy(r).cuda(),
                                       torch.from_numpy(g).cuda(), 1e-6)
    assert np.array_equal(added.cpu().numpy(), expected_added)
    assert np.allclose(out.cpu().numpy(), expected, rtol=1e-6, atol=1e-7)


def test_single_row_entry_points_and_flags(rng):
    width = 4096
    x, r, g = normal_bits(rng, (1, width)), normal_bits(rng, (1, width)), gamma_bits(rng, width)
    dx, dr, dg = bits_to_tensor(x), bits_to_tensor(r), bits_to_tensor(g)
    added, out = torch.empty_like(dx), torch.empty_like(dx)
    status, context = raw("add_rms_norm", 2, width, 1e-5, pointer(dx), pointer(dr), pointer(dg),
                          pointer(added), pointer(out))
    assert status == 0, error_text(context)
    rows_added, rows_out = _kernels.add_rms_norm(dx, dr, dg, 1e-5)
    assert torch.equal(added, rows_added) and torch.equal(out, rows_out)
    g32 = torch.from_numpy(oracle.bf16_values(g)).cuda()
    for weight_dtype, weight, weight_host in ((2, dg, g), (0, g32, oracle.bf16_values(g))):
        for round_first in (0, 1):
            for descending in (0, 1):
                status, context = raw("rms_norm_decode", 2, weight_dtype, width, 1e-5, round_first,
                                      descending, pointer(dx), pointer(weight), pointer(out))
                assert status == 0, error_text(context)
                _, expected = oracle.rms_row(x[0], weight_host, 1e-5, None, bool(round_first),
                                             bool(descending))
                assert ulp_distance_bf16(tensor_to_bits(out)[0], expected).max() <= 1
    # rejected arguments (reference backend.cu:1371-1380, 1404-1408)
    bad = [
        ("add_rms_norm", (2, 2044, 1e-5, pointer(dx), pointer(dr), pointer(dg), pointer(added), pointer(out))),
        ("add_rms_norm", (2, width, -1.0, pointer(dx), pointer(dr), pointer(dg), pointer(added), pointer(out))),
        ("add_rms_norm", (2, width, 1e-5, pointer(dx), pointer(dr), pointer(dg), pointer(out), pointer(out))),
        ("add_rms_norm", (2, width, 1e-5, pointer(dx), pointer(dr), pointer(dg), pointer(dx), pointer(out))),
        ("add_rms_norm", (1, width, 1e-5, pointer(dx), pointer(dr), pointer(dg), pointer(added), pointer(out))),
        ("rms_norm_decode", (0, 2, width, 1e-5, 1, 0, pointer(dx), pointer(dg), pointer(out))),
        ("rms_norm_decode", (2, 2, width, 1e-5, 2, 0, pointer(dx), pointer(dg), pointer(out))),
        ("rms_norm_decode", (2, 2, width, 1e-5, 1, 0, pointer(dx), pointer(dg), pointer(dx))),
        ("add_rms_norm_rows", (2, 3, 6, 1e-5, pointer(dx), pointer(dr), pointer(dg), pointer(added), pointer(out))),
    ]
    for name, arguments in bad:
        status, context = raw(name, *arguments)
        assert status == -1 and "invalid" in error_text(context), (name, error_text(context))


@pytest.mark.parametrize("rows,width", [(1, 8192), (2, 3), (3, 127), (1, 4095), (64, 4096)])
def test_rms_norm_rows(rng, rows, width):
    x, g = normal_bits(rng, (rows, width)), gamma_bits(rng, width)
    out = _kernels.rms_norm(bits_to_tensor(x), bits_to_tensor(g), 1e-5)
    if rows == 1 and 2048 <= width <= 65536 and width % 4 == 0:
        _, expected = oracle.rms_row(x[0], g, 1e-5)
        expected = expected[None, :]
    else:
        expected = oracle.rms_norm_rows(x, g, 1e-5)
    assert ulp_distance_bf16(tensor_to_bits(out), expected).max() <= 1


def test_constant_row_known_answer():
    width = 4096
    x = bits_to_tensor(oracle.bf16_bits(np.full((2, width), 3.0, dtype=np.float32)))
    r = bits_to_tensor(oracle.bf16_bits(np.full((2, width), 1.0, dtype=np.float32)))
    g = bits_to_tensor(oracle.bf16_bits((np.arange(width) % 16).astype(np.float32)))
    added, out = _kernels.add_rms_norm(x, r, g, 0.0)
    assert torch.all(added == 4.0)
    assert torch.equal(out, g.expand(2, width))


def test_square_and_scale(rng):
    rows, width = 6, 1024
    x, g = normal_bits(rng, (rows, width)), gamma_bits(rng, width)
    dx, dg = bits_to_tensor(x), bits_to_tensor(g)
    squares = torch.empty((rows, width), dtype=torch.float32, device="cuda")
    status, context = raw("bfloat16_square", rows * width, pointer(dx), pointer(squares))
    assert status == 0, error_text(context)
    values = oracle.bf16_values(x)
    assert np.array_equal(squares.cpu().numpy(), values * values)
    means = squares.mean(dim=1)
    out = torch.empty_like(dx)
    status, context = raw("rms_scale", 2, rows * width, width, 1e-5, pointer(dx), pointer(dg),
                          pointer(means), pointer(out))
    assert status == 0, error_text(context)
    scale = 1.0 / np.sqrt(means.cpu().numpy().astype(np.float64) + 1e-5)
    normalised = oracle.bf16_values(oracle.bf16_bits((values * scale[:, None]).astype(np.float32)))
    expected = oracle.bf16_bits(normalised * oracle.bf16_values(g))
    assert ulp_distance_bf16(tensor_to_bits(out), expected).max() <= 1


def test_silu_multiply_and_swiglu(rng):
    gate = normal_bits(rng, (8, 512), 4.0)
    up = normal_bits(rng, (8, 512))
    out = _kernels.silu_multiply(bits_to_tensor(gate), bits_to_tensor(up))
    expected = oracle.silu_multiply_bf16(gate, up)
    assert ulp_distance_bf16(tensor_to_bits(out), expected).max() <= 1
    routing = rng.uniform(0.5, 1.5, 8).astype(np.float32)
    out = _kernels.swiglu(bits_to_tensor(gate), bits_to_tensor(up), 2.0,
                          torch.from_numpy(routing).cuda())
    expected = oracle.swiglu_bf16(gate, up, 2.0, routing)
    assert ulp_distance_bf16(tensor_to_bits(out), expected).max() <= 1
    nan = bits_to_tensor(np.full((1, 8), 0x7FC0, dtype=np.uint16))
    assert torch.isnan(_kernels.swiglu(nan, nan, 2.0)).all()


def test_add_rms_norm_on_spaced_rows(rng):
    """Rows that are contiguous but spaced apart (the two halves of an interleaved
    [rows, 2, width] buffer) are normalised where they lie and give the bits of the
    packed call."""
    rows, width = 37, 4096
    both = bits_to_tensor(normal_bits(rng, (rows, 2, width)))
    g = bits_to_tensor(gamma_bits(rng, width))
    x, r = both[:, 0], both[:, 1]
    assert not x.is_contiguous() and x.stride(0) == 2 * width
    added, out = _kernels.add_rms_norm(x, r, g, 1e-5)
    expected_added, expected_out = _kernels.add_rms_norm(x.contiguous(), r.contiguous(), g, 1e-5)
    assert torch.equal(added, expected_added) and torch.equal(out, expected_out)
    status, context = raw("add_rms_norm_strided", 2, rows, width, 1e-5, pointer(x), width - 4,
                          pointer(r), 2 * width, pointer(g), pointer(added), width, pointer(out), width)
    assert status == -1 and "invalid" in error_text(context)
