"""gate_up projection with SwiGLU applied in the GEMM epilogue.

`camblas_cuda_gate_up_swiglu_bf16` replaces the reference's two steps - a BF16
GEMM that writes `[rows, 2*intermediate]` and `camblas_cuda_silu_multiply`
(`inference_fusion.cuh:19-29`) that reads it back - and keeps their roundings.
Checkers: the oracle's BF16 linear layer followed by its `silu_multiply`
(rel-L2 <= 1e-2, the BF16 bound of the GEMM tests: a GEMM sum that lands one
BF16 ulp away moves the output by more than an ulp), the library's own two-step
path (bit-equal where both paths cut K the same way), and small integers whose
GEMM sums are exact, where only the device `expf` can differ (<= 1 ulp, as in
the silu_multiply test).
"""

import numpy as np
import pytest
import torch

from camblas_b200 import _kernels, _native
from oracle import oracle
from tests.helpers import (BF16_TOLERANCE, bits_to_tensor, normal_bits, tensor_to_bits,
                           ulp_distance_bf16)

pytestmark = pytest.mark.gpu


def two_step(x, w_packed):
    both = _kernels.linear(x, w_packed)
    gate, up = both.chunk(2, dim=-1)
    return _kernels.silu_multiply(gate.contiguous(), up.contiguous())


def oracle_two_step(x_bits, w_bits):
    both = oracle.linear_bf16(x_bits, w_bits)
    half = both.shape[1] // 2
    return oracle.silu_multiply_bf16(np.ascontiguousarray(both[:, :half]),
                                     np.ascontiguousarray(both[:, half:]))


def test_interleave_layout():
    weight = torch.arange(512 * 4, dtype=torch.float32).reshape(512, 4)
    mixed = _kernels.interleave_gate_up(weight)
    assert torch.equal(mixed[:128], weight[:128])          # gate block 0
    assert torch.equal(mixed[128:256], weight[256:384])    # up block 0
    assert torch.equal(mixed[256:384], weight[128:256])    # gate block 1
    assert torch.equal(mixed[384:], weight[384:])          # up block 1
    with pytest.raises(ValueError):
        _kernels.interleave_gate_up(weight[:300])


@pytest.mark.parametrize("rows,inner,intermediate", [
    (300, 512, 384),     # ragged rows, few tiles, short K: whole tiles only
    (512, 1024, 1280),
    (130, 200, 128),     # depth not a multiple of 64
    (64, 512, 256),      # fewer rows than a tile
    (1, 256, 128),
])
def test_matches_oracle_and_two_step(rows, inner, intermediate):
    rng = np.random.default_rng(705537 + rows + intermediate)
    x = normal_bits(rng, (rows, inner))
    w = normal_bits(rng, (2 * intermediate, inner), 0.06)
    w_device = bits_to_tensor(w)
    fused = _kernels.gate_up_swiglu(bits_to_tensor(x), _kernels.interleave_gate_up(w_device))
    assert _native.context(0).device_status() == 0
    assert fused.shape == (rows, intermediate)
    expected = oracle.bf16_values(oracle_two_step(x, w))
    assert oracle.rel_l2(oracle.bf16_values(tensor_to_bits(fused)), expected) <= BF16_TOLERANCE
    if rows > 128:
        # with the K split inside a cluster switched off the two-step path runs the same
        # two-SM kernel over the same K ranges, so the bits must agree
        with _native.options(cluster_split=0):
            assert torch.equal(fused, two_step(bits_to_tensor(x), w_device))
    else:
        reference = two_step(bits_to_tensor(x), w_device).float()
        assert ((fused.float() - reference).norm() / reference.norm()).item() <= BF16_TOLERANCE


def test_exact_integer_sums():
    rows, inner, intermediate = 260, 48, 256
    rng = np.random.default_rng(73013)
    x = oracle.bf16_bits(rng.integers(-1, 2, (rows, inner)).astype(np.float32))
    w = oracle.bf16_bits((rng.integers(-2, 3, (2 * intermediate, inner)) * 0.125).astype(np.float32))
    fused = _kernels.gate_up_swiglu(bits_to_tensor(x),
                                    _kernels.interleave_gate_up(bits_to_tensor(w)))
    expected = oracle_two_step(x, w)
    assert ulp_distance_bf16(tensor_to_bits(fused), expected).max() <= 1


def test_full_size_block_with_stream_k_tail():
    """M=512, hidden 8192, intermediate 28672: 448 tiles on 74 CTA pairs, stream-K tail."""
    torch.manual_seed(20261004)
    rows, inner, intermediate = 512, 8192, 28672
    x = torch.randn(rows, inner, device="cuda").bfloat16()
    w = (torch.randn(2 * intermediate, inner, device="cuda") * 0.02).bfloat16()
    fused = _kernels.gate_up_swiglu(x, _kernels.interleave_gate_up(w))
    again = _kernels.gate_up_swiglu(x, _kernels.interleave_gate_up(w))
    assert _native.context(0).device_status() == 0
    assert torch.equal(fused, again)  # fixed summation order
    reference = two_step(x, w).float()
    assert ((fused.float() - reference).norm() / reference.norm()).item() <= 2e-3
    # sampled entries against FP64 dot products with the two-step roundings
    generator = torch.Generator().manual_seed(5)
    picks_r = torch.randint(0, rows, (64,), generator=generator)
    picks_c = torch.randint(0, intermediate, (64,), generator=generator)
    xs = x[picks_r].double().cpu()
    gate = (xs * w[picks_c].double().cpu()).sum(1).float().bfloat16().float()
    up = (xs * w[intermediate + picks_c].double().cpu()).sum(1).float().bfloat16().float()
    activated = (gate / (1 + torch.exp(-gate))).bfloat16().float()
    expected = (activated * up).bfloat16().float()
    got = fused[picks_r, picks_c].float().cpu()
    assert ((got - expected).norm() / expected.norm()).item() <= BF16_TOLERANCE


def test_rejects_bad_shapes():
    x = torch.zeros((8, 64), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        _kernels.gate_up_swiglu(x, torch.zeros((200, 64), dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):
        _kernels.gate_up_swiglu(x, torch.zeros((256, 32), dtype=torch.bfloat16, device="cuda"))


@pytest.mark.parametrize("rows,inner,intermediate", [(300, 512, 384), (512, 1024, 1280), (64, 512, 256),
                                                     (512, 8192, 28672)])
def test_quantising_epilogue_equals_quantising_the_bf16_result(rows, inner, intermediate):
    """gate_up_swiglu_fp8 must give the bytes and scales that fp8_quantize gives on the
    BF16 result of gate_up_swiglu (the last shape has a stream-K tail, whose second
    pass quantises too), and an FP8 down projection on them the same product."""
    torch.manual_seed(20261127 + rows + intermediate)
    x = torch.randn(rows, inner, device="cuda").bfloat16()
    w = (torch.randn(2 * intermediate, inner, device="cuda") * (2.0 / inner ** 0.5)).bfloat16()
    mixed = _kernels.interleave_gate_up(w)
    q, scale = _kernels.gate_up_swiglu_fp8(x, mixed)
    assert _native.context(0).device_status() == 0
    expected_q, expected_scale = _kernels.fp8_quantize(_kernels.gate_up_swiglu(x, mixed))
    assert torch.equal(scale, expected_scale)
    assert torch.equal(q.view(torch.uint8), expected_q.view(torch.uint8))


@pytest.mark.parametrize("rows,inner,intermediate", [(1, 256, 128), (40, 384, 256), (300, 512, 384)])
def test_gated_mlp_function_and_prepared_module(rows, inner, intermediate):
    """`gated_mlp` (the reference's torch_bindings.cpp:703-723: gate and up projections,
    silu_multiply, down projection) against the oracle's BF16 linear layers and its
    silu_multiply; `GatedMLP` (weights interleaved once, SwiGLU in the GEMM epilogue) against
    the function - same roundings, so within the BF16 bound of one more GEMM."""
    rng = np.random.default_rng(705560 + rows)
    x = normal_bits(rng, (rows, inner))
    gate, up = normal_bits(rng, (intermediate, inner), 0.06), normal_bits(rng, (intermediate, inner), 0.06)
    down = normal_bits(rng, (inner, intermediate), 0.06)
    hidden = oracle.silu_multiply_bf16(oracle.linear_bf16(x, gate), oracle.linear_bf16(x, up))
    expected = oracle.bf16_values(oracle.linear_bf16(hidden, down))
    tensors = [bits_to_tensor(a) for a in (x, gate, up, down)]
    plain = _kernels.gated_mlp(*tensors)
    assert _native.context(0).device_status() == 0
    assert plain.shape == (rows, inner)
    assert oracle.rel_l2(oracle.bf16_values(tensor_to_bits(plain)), expected) <= 2 * BF16_TOLERANCE
    prepared = _kernels.GatedMLP(*tensors[1:])(tensors[0])
    assert oracle.rel_l2(oracle.bf16_values(tensor_to_bits(prepared)), expected) <= 2 * BF16_TOLERANCE
    difference = (prepared.float() - plain.float()).norm() / plain.float().norm()
    assert difference.item() <= BF16_TOLERANCE
    with pytest.raises(ValueError):
        _kernels.gated_mlp(tensors[0], tensors[1], tensors[2][:-1], tensors[3])


def test_python_wrappers_of_the_float_layers():
    """`affine`, `mlp` and `attention` of the host mirror (FP32 / FP64 tensors) against torch."""
    generator = torch.Generator(device="cuda").manual_seed(5)
    for dtype, tolerance in ((torch.float32, 1e-5), (torch.float64, 1e-13)):
        x = torch.randn(33, 20, device="cuda", dtype=dtype, generator=generator)
        w1 = torch.randn(20, 50, device="cuda", dtype=dtype, generator=generator)
        b1 = torch.randn(50, device="cuda", dtype=dtype, generator=generator)
        w2 = torch.randn(50, 7, device="cuda", dtype=dtype, generator=generator)
        b2 = torch.randn(7, device="cuda", dtype=dtype, generator=generator)
        hidden = torch.relu(x.double() @ w1.double() + b1.double())
        assert torch.allclose(_kernels.affine(x, w1, b1, relu=True).double(), hidden, rtol=0,
                              atol=tolerance * 50)
        out, kept = _kernels.mlp(x, w1, b1, w2, b2)
        assert torch.allclose(kept.double(), hidden, rtol=0, atol=tolerance * 50)
        assert torch.allclose(out.double(), kept.double() @ w2.double() + b2.double(), rtol=0,
                              atol=tolerance * 200)
        q, k = x, torch.randn(9, 20, device="cuda", dtype=dtype, generator=generator)
        v = torch.randn(9, 4, device="cuda", dtype=dtype, generator=generator)
        expected = torch.softmax(q.double() @ k.double().T / 20 ** 0.5, dim=1) @ v.double()
        assert torch.allclose(_kernels.attention(q, k, v).double(), expected, rtol=0, atol=tolerance * 50)
    with pytest.raises(ValueError):
        _kernels.affine(x.bfloat16(), w1, b1)
