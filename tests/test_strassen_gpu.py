"""One-level Strassen for BF16 squares against the oracle and the classical kernel.

Stated tolerance: rel-L2 <= 1e-2 against the exact product (BF16_TOLERANCE), and
at most five times the classical kernel's error, the factor the reference allows
its Strassen paths (tests/test_cuda.py:53-58). Elementwise, the cancellation
bound |err| <= 50 eps (|A||B|) of tests/test_cuda.py:916-930 with BF16 eps.
"""

import numpy as np
import pytest
import torch

from camblas_b200 import _kernels, _native
from oracle import oracle
from tests.helpers import BF16_TOLERANCE, bits_to_tensor, tensor_to_bits

pytestmark = pytest.mark.gpu


def uniform_square(rng, n):
    return oracle.bf16_bits(rng.uniform(-1, 1, (n, n)).astype(np.float32))


@pytest.mark.parametrize("n", [512, 1024])
def test_strassen_against_oracle_and_classical(rng, n):
    a, b = uniform_square(rng, n), uniform_square(rng, n)
    da, db = bits_to_tensor(a), bits_to_tensor(b)
    _native.stats(0, reset=True)
    with _native.algorithm("strassen"), _native.options(bf16_strassen=1):
        fast = _kernels.matmul(da, db)
    counts = _native.stats(0)
    assert counts["strassen"] == 1 and counts["guard_fallback"] == 0
    classical = _kernels.matmul(da, db)
    assert _native.context(0).device_status() == 0
    exact = oracle.bf16_values(a).astype(np.float64) @ oracle.bf16_values(b).astype(np.float64)
    error_fast = oracle.rel_l2(fast.float().cpu().numpy(), exact)
    error_classical = oracle.rel_l2(classical.float().cpu().numpy(), exact)
    assert error_fast <= BF16_TOLERANCE and error_fast <= 5 * error_classical, (error_fast, error_classical)
    bound = 50 * 2.0 ** -8 * (np.abs(oracle.bf16_values(a)).astype(np.float64)
                               @ np.abs(oracle.bf16_values(b)).astype(np.float64))
    assert np.all(np.abs(fast.float().cpu().numpy() - exact) <= bound)
    if n == 512:
        # row-major torch tensors are the transposed column-major matrices: C^T = B^T A^T
        expected = oracle.strassen_bf16(np.asfortranarray(b.T), np.asfortranarray(a.T))
        got = np.asfortranarray(tensor_to_bits(fast).T)
        assert oracle.rel_l2(oracle.bf16_values(got), oracle.bf16_values(expected)) < 2e-3


@pytest.mark.parametrize("n", [4096, 8192, 16384])
def test_benchmark_sizes_classical_and_strassen_by_sampled_dot_products(n):
    """The squares of the benchmark's large-GEMM configuration at their own sizes,
    uniform [-1, 1] BF16 inputs: classical and one-level Strassen, each checked on 256
    sampled entries against FP64 dot products of the same rows and columns (the way the
    reference samples large products, bench/cuda_workload.py:403-422). Bounds: rel-L2
    over the sample <= 1e-2 for both, Strassen at most five times the classical error
    (tests/test_cuda.py:53-58), and the elementwise cancellation bound
    50 eps (|A||B|) of tests/test_cuda.py:916-930 with the BF16 eps."""
    generator = torch.Generator(device="cuda").manual_seed(705537 + n)
    a = (torch.rand((n, n), device="cuda", generator=generator) * 2 - 1).bfloat16()
    b = (torch.rand((n, n), device="cuda", generator=generator) * 2 - 1).bfloat16()
    picks = torch.Generator().manual_seed(n)
    rows = torch.randint(0, n, (256,), generator=picks).cuda()
    cols = torch.randint(0, n, (256,), generator=picks).cuda()
    left, right = a[rows].double(), b[:, cols].t().double()
    exact = (left * right).sum(1)
    bound = 50 * 2.0 ** -8 * (left.abs() * right.abs()).sum(1)
    classical = _kernels.matmul(a, b)
    _native.stats(0, reset=True)
    with _native.algorithm("strassen"), _native.options(bf16_strassen=1):
        fast = _kernels.matmul(a, b)
    counts = _native.stats(0)
    assert counts["strassen"] == 1 and counts["guard_fallback"] == 0
    assert _native.context(0).device_status() == 0
    errors = {}
    for name, result in (("classical", classical), ("strassen", fast)):
        got = result[rows, cols].double()
        errors[name] = ((got - exact).norm() / exact.norm()).item()
        assert errors[name] <= BF16_TOLERANCE, (name, n, errors[name])
        assert bool(((got - exact).abs() <= bound).all()), (name, n)
    assert errors["strassen"] <= 5 * max(errors["classical"], 2.0 ** -9), errors
    # without the option the STRASSEN policy multiplies classically, as the reference does for BF16
    _native.stats(0, reset=True)
    with _native.algorithm("strassen"):
        plain = _kernels.matmul(a, b)
    assert _native.stats(0)["strassen"] == 0
    assert torch.equal(plain, classical)


def test_alpha_beta_and_ineligible_shapes(rng):
    n = 512
    a, b, c = uniform_square(rng, n), uniform_square(rng, n), uniform_square(rng, n)
    da, db = bits_to_tensor(a), bits_to_tensor(b)
    with _native.algorithm("strassen"), _native.options(bf16_strassen=1):
        out = _kernels.matmul(da, db, out=bits_to_tensor(c), alpha=0.5, beta=-2.0)
    exact = 0.5 * (oracle.bf16_values(a).astype(np.float64) @ oracle.bf16_values(b).astype(np.float64)) \
        - 2.0 * oracle.bf16_values(c)
    assert oracle.rel_l2(out.float().cpu().numpy(), exact) <= BF16_TOLERANCE
    # shapes Strassen does not take run the classical kernel and count as such
    _native.stats(0, reset=True)
    with _native.algorithm("strassen"), _native.options(bf16_strassen=1):
        _kernels.matmul(da[:384, :384].contiguous(), db[:384, :384].contiguous())
        _kernels.matmul(da, db.t())
    counts = _native.stats(0)
    assert counts["strassen"] == 0 and counts["classical"] == 2


def test_range_guard_falls_back_to_classical_without_a_host_sync():
    n = 512
    a = torch.full((n, n), 1.0, device="cuda", dtype=torch.bfloat16)
    b = torch.full((n, n), 2.0 ** -9, device="cuda", dtype=torch.bfloat16)
    a[3, 5] = 3.0e38  # above sqrt(FLT_MAX / (64 n)): the packed sums could overflow
    _native.stats(0, reset=True)
    with _native.algorithm("strassen"), _native.options(bf16_strassen=1):
        guarded = _kernels.matmul(a, b)
    classical = _kernels.matmul(a, b)
    torch.cuda.synchronize()
    assert torch.equal(guarded, classical)
    counts = _native.stats(0)
    assert counts["strassen"] == 1 and counts["guard_fallback"] == 1
    a[3, 5] = float("nan")
    with _native.algorithm("strassen"), _native.options(bf16_strassen=1):
        guarded = _kernels.matmul(a, b)
    torch.cuda.synchronize()
    assert torch.isnan(guarded[3]).all() and not torch.isnan(guarded[4]).any()
    assert _native.stats(0)["guard_fallback"] == 2
