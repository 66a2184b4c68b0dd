"""BF16 GEMM parity: the CUDA kernels, called through the C ABI, against the CPU oracle.

Tolerance: relative L2 error <= 1e-2 on BF16 outputs (BF16_TOLERANCE), the
bound the benchmark definition states; known-answer and exact-integer cases are
compared bit for bit. Shapes, padded leading dimensions with NaN canaries and
the alpha/beta cases follow the reference's tests/test_bfloat16.py:54-205.
"""

import ctypes as ct
from pathlib import Path

import numpy as np
import pytest
import torch

from camblas_b200 import _kernels, _native
from oracle import oracle
from tests.helpers import (BF16_TOLERANCE, bits_to_tensor, error_text, normal_bits, pointer, raw,
                           tensor_to_bits)

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
NAN = 0x7FC0


def padded(rng, rows, columns, ld):
    """Column-major rows x columns matrix inside an ld x columns buffer, NaN padding."""
    buffer = np.full((columns, ld), NAN, dtype=np.uint16)
    buffer[:, :rows] = normal_bits(rng, (columns, rows))
    return buffer  # buffer[j, i] is element (i, j)


def run_bgemm(ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc, family="auto"):
    da, db, dc = bits_to_tensor(a), bits_to_tensor(b), bits_to_tensor(c)
    with _native.kernel_family(family):
        status, context = raw("bgemm", ta.encode(), tb.encode(), m, n, k, alpha, pointer(da), lda,
                              pointer(db), ldb, beta, pointer(dc), ldc)
    assert status == 0, error_text(context)
    assert context.device_status() == 0
    return tensor_to_bits(dc)


@pytest.mark.parametrize("ta,tb", [("N", "N"), ("N", "T"), ("T", "N"), ("T", "T")])
@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (5, 3, 7), (64, 64, 64), (65, 129, 33), (130, 70, 257),
                                   (257, 5, 130)])
def test_transposes_padding_alpha_beta(rng, ta, tb, m, n, k):
    lda = (m if ta == "N" else k) + 3
    ldb = (k if tb == "N" else n) + 5
    ldc = m + 2
    a = padded(rng, m if ta == "N" else k, k if ta == "N" else m, lda)
    b = padded(rng, k if tb == "N" else n, n if tb == "N" else k, ldb)
    c = padded(rng, m, n, ldc)
    for alpha, beta in ((1.0, 0.0), (0.5, -1.25)):
        expected = c.copy()
        expected[:, m:] = 0  # keep the oracle away from NaN padding it never touches anyway
        oracle.bgemm(ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, expected, ldc)
        actual = run_bgemm(ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc)
        assert np.all(actual[:, m:] == NAN), "padding rows of C were written"
        error = oracle.rel_l2(oracle.bf16_values(actual[:, :m]), oracle.bf16_values(expected[:, :m]))
        assert error <= BF16_TOLERANCE, error


FAMILY_SHAPES = {
    "generic": [(40, 3, 72), (200, 130, 64)],
    "skinny": [(256, 1, 2048), (100, 2, 1000), (512, 3, 4104), (96, 4, 8200)],
    "tensor": [(256, 128, 64), (264, 130, 136), (520, 200, 264), (1024, 512, 1024), (72, 300, 128)],
    "tensor_pair": [(256, 256, 64), (264, 130, 136), (520, 300, 264), (1024, 512, 1024), (72, 300, 128),
                    (2304, 600, 520)],
    "tensor_swapped": [(128, 16, 64), (136, 5, 72), (1000, 40, 1032), (4096, 8, 2048),
                       (256, 64, 8192), (300, 70, 520)],
}


@pytest.mark.parametrize("family", list(FAMILY_SHAPES))
def test_each_kernel_family(rng, family):
    for m, n, k in FAMILY_SHAPES[family]:
        w = normal_bits(rng, (m, k))  # 'T' operand: outputs x inner, row-major
        x = normal_bits(rng, (n, k))  # 'N' operand: tokens x inner, row-major
        c = normal_bits(rng, (n, m))
        for alpha, beta in ((1.0, 0.0), (-0.5, 0.75)):
            expected = c.copy()
            oracle.bgemm("T", "N", m, n, k, alpha, w, k, x, k, beta, expected, m)
            actual = run_bgemm("T", "N", m, n, k, alpha, w, k, x, k, beta, c, m, family)
            error = oracle.rel_l2(oracle.bf16_values(actual), oracle.bf16_values(expected))
            assert error <= BF16_TOLERANCE, (family, m, n, k, error)


def test_forced_family_that_cannot_run_fails_loudly(rng):
    w = normal_bits(rng, (64, 63))  # inner width 63: rows are not 16-byte aligned
    x = normal_bits(rng, (16, 63))
    c = np.zeros((16, 64), dtype=np.uint16)
    dw, dx, dc = bits_to_tensor(w), bits_to_tensor(x), bits_to_tensor(c)
    for family in ("tensor", "tensor_swapped", "skinny"):
        with _native.kernel_family(family):
            status, context = raw("bgemm", b"T", b"N", 64, 16, 63, 1.0, pointer(dw), 63, pointer(dx),
                                  63, 0.0, pointer(dc), 64)
        assert status < 0 and "forced kernel family" in error_text(context)
    actual = run_bgemm("T", "N", 64, 16, 63, 1.0, w, 63, x, 63, 0.0, c, 64)  # automatic -> generic
    expected = oracle.linear_bf16(x, w)
    assert oracle.rel_l2(oracle.bf16_values(actual), oracle.bf16_values(expected)) <= BF16_TOLERANCE


@pytest.mark.parametrize("family,n", [("skinny", 1), ("skinny", 4), ("tensor_swapped", 8),
                                      ("tensor_swapped", 33), ("tensor", 128), ("tensor", 300),
                                      ("tensor_pair", 300), ("tensor_pair", 1000), ("generic", 9)])
def test_exact_integer_products(family, n):
    """Rank-2 integer operands make every output an exact small integer: any tile
    boundary or K-tail mistake shows as a wrong integer, not as rounding noise
    (the trick of the reference's tests/test_mlp_packing.py:120-224)."""
    m, k = 392, 1096
    i = np.arange(m)[:, None]
    j = np.arange(n)[:, None]
    l = np.arange(k)[None, :]
    w = ((i % 3) * (l % 2) + ((i + 1) % 2) * ((l + 1) % 2) * ((l % 5) == 0)).astype(np.float32)
    x = ((j % 2 + 1) * (l % 2) - ((j % 3) == 0) * ((l + 1) % 2) * ((l % 5) == 0)).astype(np.float32)
    expected = x.astype(np.int64) @ w.astype(np.int64).T
    assert 100 < np.abs(expected).max() < 2 ** 20  # every partial sum is an exact FP32 integer
    keep = np.abs(expected) <= 256  # integers up to 256 are exact in BF16
    actual = run_bgemm("T", "N", m, n, k, 1.0, oracle.bf16_bits(w), k, oracle.bf16_bits(x), k, 0.0,
                       np.zeros((n, m), dtype=np.uint16), m, family)
    values = oracle.bf16_values(actual)
    assert np.array_equal(values[keep], expected[keep].astype(np.float32))
    assert np.array_equal(actual, oracle.bf16_bits(expected.astype(np.float32)))


def test_identity_and_fp32_accumulation_probe():
    n = 192
    identity = np.zeros((n, n), dtype=np.uint16)
    identity[np.arange(n), np.arange(n)] = oracle.bf16_bits(np.float32(1.0))
    rng = np.random.default_rng(5)
    b = normal_bits(rng, (n, n))
    for ta in "NT":
        for family in ("auto", "generic"):
            actual = run_bgemm(ta, "N", n, n, n, 1.0, identity, n, b, n, 0.0,
                               np.zeros((n, n), dtype=np.uint16), n, family)
            assert np.array_equal(actual, b)
    k = 1024
    a = np.zeros((8, k), dtype=np.float32)
    a[:, [0, 500, 1023]] = [256.0, 1.0, -256.0]
    ones = np.ones((16, k), dtype=np.float32)
    for family, tokens in (("skinny", 1), ("tensor_swapped", 16), ("generic", 16)):
        actual = run_bgemm("T", "N", 8, tokens, k, 1.0, oracle.bf16_bits(a), k,
                           oracle.bf16_bits(ones[:tokens]), k, 0.0,
                           np.zeros((tokens, 8), dtype=np.uint16), 8, family)
        assert np.all(oracle.bf16_values(actual) == 1.0), family


def test_alpha_zero_ignores_operands_and_beta_zero_overwrites_nan():
    nan = bits_to_tensor(np.full((32, 32), NAN, dtype=np.uint16))
    c = bits_to_tensor(np.full((32, 32), NAN, dtype=np.uint16))
    status, context = raw("bgemm", b"N", b"N", 32, 32, 32, 0.0, pointer(nan), 32, pointer(nan), 32,
                          0.0, pointer(c), 32)
    assert status == 0, error_text(context)
    assert np.all(tensor_to_bits(c) == 0)
    c = bits_to_tensor(oracle.bf16_bits(np.full((32, 32), 2.0, dtype=np.float32)))
    status, context = raw("bgemm", b"N", b"N", 32, 32, 32, 0.0, None, 32, None, 32, -0.75,
                          pointer(c), 32)
    assert status == 0, error_text(context)
    assert np.all(oracle.bf16_values(tensor_to_bits(c)) == -1.5)
    # k == 0 behaves the same; beta == 1 is a no-op
    status, _ = raw("bgemm", b"T", b"N", 32, 32, 0, 1.0, None, 1, None, 1, 1.0, pointer(c), 32)
    assert status == 0 and np.all(oracle.bf16_values(tensor_to_bits(c)) == -1.5)
    # beta == 0 with a real product must not let NaNs in C through
    rng = np.random.default_rng(9)
    w, x = normal_bits(rng, (256, 128)), normal_bits(rng, (130, 128))
    actual = run_bgemm("T", "N", 256, 130, 128, 1.0, w, 128, x, 128, 0.0,
                       np.full((130, 256), NAN, dtype=np.uint16), 256)
    assert not np.isnan(oracle.bf16_values(actual)).any()


def test_argument_validation_and_error_text():
    buffer = bits_to_tensor(np.zeros((64, 64), dtype=np.uint16))
    other = bits_to_tensor(np.zeros((64, 64), dtype=np.uint16))
    out = bits_to_tensor(np.zeros((64, 64), dtype=np.uint16))
    p, q, c = pointer(buffer), pointer(other), pointer(out)
    cases = [
        ((b"X", b"N", 8, 8, 8, 1.0, p, 8, q, 8, 0.0, c, 8), "invalid BF16 GEMM arguments"),
        ((b"N", b"N", -1, 8, 8, 1.0, p, 8, q, 8, 0.0, c, 8), "invalid BF16 GEMM arguments"),
        ((b"N", b"N", 8, 8, 8, 1.0, p, 0, q, 8, 0.0, c, 8), "invalid BF16 GEMM arguments"),
        ((b"N", b"N", 8, 8, 8, 1.0, p, 7, q, 8, 0.0, c, 8), "invalid BF16 pointer or leading dimension"),
        ((b"T", b"T", 8, 8, 16, 1.0, p, 16, q, 7, 0.0, c, 8), "invalid BF16 pointer or leading dimension"),
        ((b"N", b"N", 8, 8, 8, 1.0, p, 8, q, 8, 0.0, c, 7), "invalid BF16 pointer or leading dimension"),
        ((b"N", b"N", 8, 8, 8, 1.0, p, 8, q, 8, 0.0, None, 8), "invalid BF16 pointer or leading dimension"),
        ((b"N", b"N", 8, 8, 8, 1.0, None, 8, q, 8, 0.0, c, 8), "missing or aliased BF16 GEMM operand"),
        ((b"N", b"N", 8, 8, 8, 1.0, c, 8, q, 8, 0.0, c, 8), "missing or aliased BF16 GEMM operand"),
        ((b"N", b"N", 8, 8, 8, 1.0, p, 8, c, 8, 0.0, c, 8), "missing or aliased BF16 GEMM operand"),
    ]
    for arguments, message in cases:
        status, context = raw("bgemm", *arguments)
        assert status == -1 and message in error_text(context), (arguments, error_text(context))
    # empty products succeed without looking at pointers; lower-case flags are accepted
    assert raw("bgemm", b"n", b"t", 0, 8, 8, 1.0, None, 1, None, 8, 0.0, None, 1)[0] == 0
    assert raw("bgemm", b"t", b"n", 8, 0, 8, 1.0, None, 8, None, 8, 0.0, None, 8)[0] == 0
    library = _native.library()
    context = _native.context(0)
    assert library.camblas_cuda_set_algorithm(context.handle, 8) == -1
    assert library.camblas_cuda_set_algorithm(context.handle, 3) == 0
    assert library.camblas_cuda_set_algorithm(context.handle, 0) == 0


def test_counters_count_launches(rng):
    context = _native.context(0)
    before = _native.stats(0, reset=True)
    assert set(before) == {"classical", "strassen", "gram", "affine", "lt", "guard_fallback",
                           "attention", "backward"}
    w, x = bits_to_tensor(normal_bits(rng, (64, 64))), bits_to_tensor(normal_bits(rng, (8, 64)))
    _kernels.linear(x, w)
    assert _native.stats(0)["classical"] == 1
    with _native.algorithm("lt"):
        _kernels.matmul(x, w.t())
        assert _native.stats(0)["lt"] == 1
    counts = (ct.c_uint64 * 6)()
    assert _native.library().camblas_cuda_stats(context.handle, counts, 6) == 0
    assert _native.library().camblas_cuda_stats(context.handle, counts, 7) == -1
    assert _native.stats(0, reset=True)["classical"] == 1
    assert _native.stats(0)["classical"] == 0


def test_golden_vectors_through_the_abi():
    data = np.load(GOLDEN / "gemm_small.npz")
    for index in range(3):
        x, w, y = data[f"x{index}"], data[f"w{index}"], data[f"y{index}"]
        out = _kernels.linear(bits_to_tensor(x), bits_to_tensor(w))
        assert oracle.rel_l2(out.float().cpu().numpy(), y) <= BF16_TOLERANCE
    from tests.golden.make_golden import config1_inputs

    data = np.load(GOLDEN / "c1_decode.npz")
    x, w = config1_inputs(int(data["seed"]))
    for family in ("auto", "skinny", "tensor_swapped", "generic"):
        with _native.kernel_family(family):
            out = _kernels.linear(bits_to_tensor(x), bits_to_tensor(w))
        assert oracle.rel_l2(out.float().cpu().numpy(), data["y"]) <= BF16_TOLERANCE, family


def test_fused_epilogue_and_packed_projection(rng):
    for rows in (1, 3, 20, 150):
        inner, outputs = 264, 392
        x, w = normal_bits(rng, (rows, inner)), normal_bits(rng, (outputs, inner))
        bias, residual = normal_bits(rng, (outputs,)), normal_bits(rng, (rows, outputs))
        expected = oracle.linear_bf16(x, w, bias, residual)
        out = _kernels.linear(bits_to_tensor(x), bits_to_tensor(w), bits_to_tensor(bias),
                              bits_to_tensor(residual))
        error = oracle.rel_l2(out.float().cpu().numpy(), oracle.bf16_values(expected))
        assert error <= BF16_TOLERANCE, (rows, error)
    for rows in (2, 24, 200):
        inner, widths = 256, (512, 128, 128)
        x, w = normal_bits(rng, (rows, inner)), normal_bits(rng, (sum(widths), inner))
        expected = oracle.bf16_values(oracle.linear_bf16(x, w))
        q, k, v = _kernels.qkv_linear(bits_to_tensor(x), bits_to_tensor(w), *widths)
        assert len({q.data_ptr(), k.data_ptr(), v.data_ptr()}) == 3
        packed = torch.cat([q, k, v], dim=1).float().cpu().numpy()
        assert oracle.rel_l2(packed, expected) <= BF16_TOLERANCE, rows


@pytest.mark.parametrize("tokens,outputs,inner", [(512, 10240, 8192), (512, 8192, 28672),
                                                  (64, 8192, 28672), (1, 57344, 8192)])
def test_full_size_properties(tokens, outputs, inner):
    """Benchmark-sized shapes: too large for the CPU oracle in full, so check
    (1) a sampled set of output features against the oracle, (2) exact scaling:
    doubling the activations doubles every output bit for bit, (3) splitting the
    weight by output rows gives the whole product again: bit for bit in all but
    the few tiles whose K range the scheduler cuts differently for the two
    shapes (tail wave, few-token K split), and there to BF16 rounding."""
    generator = torch.Generator(device="cuda").manual_seed(705539)
    x = torch.randn(tokens, inner, device="cuda", generator=generator).bfloat16()
    w = (torch.randn(outputs, inner, device="cuda", generator=generator) * 0.02).bfloat16()
    y = _kernels.linear(x, w)
    assert _native.context(0).device_status() == 0
    sample = torch.randperm(outputs, device="cuda", generator=generator)[:8].sort().values
    rows = min(tokens, 16)
    expected = oracle.linear_bf16(tensor_to_bits(x[:rows]), tensor_to_bits(w[sample]))
    actual = y[:rows][:, sample].float().cpu().numpy()
    assert oracle.rel_l2(actual, oracle.bf16_values(expected)) <= BF16_TOLERANCE
    assert torch.equal(_kernels.linear(x * 2, w), y * 2)
    half = outputs // 2
    for part, whole in ((_kernels.linear(x, w[:half]), y[:, :half]),
                        (_kernels.linear(x, w[half:]), y[:, half:])):
        assert oracle.rel_l2(part.float().cpu().numpy(), whole.float().cpu().numpy()) < 2e-3
        if tokens > 64:
            assert (part == whole).float().mean() > 0.5


@pytest.mark.parametrize("tokens", [9, 24, 64])
def test_leftover_tiles_of_the_few_token_kernel_are_a_product_of_their_own(tokens):
    """57 344 output features are 448 tiles of 128 on 148 SMs: three waves and four tiles. The
    four are multiplied as a separate product (bias, residual and output offset by the
    18 944 x 3 features before them): sampled features of both parts against the oracle, and
    the leftover part bit for bit against the product of its weight rows alone."""
    outputs, inner = 57344, 2048
    generator = torch.Generator(device="cuda").manual_seed(705571 + tokens)
    x = torch.randn(tokens, inner, device="cuda", generator=generator).bfloat16()
    w = (torch.randn(outputs, inner, device="cuda", generator=generator) * 0.05).bfloat16()
    bias = torch.randn(outputs, device="cuda", generator=generator).bfloat16()
    residual = torch.randn(tokens, outputs, device="cuda", generator=generator).bfloat16()
    y = _kernels.linear(x, w, bias, residual)
    assert _native.context(0).device_status() == 0
    whole = (outputs // 128 // 148) * 148 * 128
    sample = torch.cat([torch.arange(0, whole, 7001, device="cuda"), torch.tensor([whole - 1], device="cuda"),
                        torch.arange(whole, outputs, 37, device="cuda")])
    expected = oracle.linear_bf16(tensor_to_bits(x), tensor_to_bits(w[sample]), tensor_to_bits(bias[sample]),
                                  tensor_to_bits(residual[:, sample].contiguous()))
    actual = y[:, sample].float().cpu().numpy()
    assert oracle.rel_l2(actual, oracle.bf16_values(expected)) <= BF16_TOLERANCE
    alone = _kernels.linear(x, w[whole:], bias[whole:], residual[:, whole:])
    assert torch.equal(alone, y[:, whole:])


@pytest.mark.parametrize("ta,tb", [("N", "N"), ("N", "T"), ("T", "N"), ("T", "T")])
@pytest.mark.parametrize("m,n,k", [(256, 128, 64), (264, 136, 200), (520, 300, 72), (1024, 384, 1032)])
def test_tensor_family_takes_every_transpose_pair(rng, ta, tb, m, n, k):
    """Aligned operands of any transpose pair run on the tensor cores: 'N' for A
    and 'T' for B are read as MN-major tiles (64 x 64 TMA boxes)."""
    def pitch(rows, extra):
        return (rows + 7) // 8 * 8 + extra  # TMA needs 16-byte row pitches

    lda = pitch(m if ta == "N" else k, 8)
    ldb = pitch(k if tb == "N" else n, 16)
    ldc = pitch(m, 8)
    a = padded(rng, m if ta == "N" else k, k if ta == "N" else m, lda)
    b = padded(rng, k if tb == "N" else n, n if tb == "N" else k, ldb)
    c = padded(rng, m, n, ldc)
    for alpha, beta in ((1.0, 0.0), (-0.5, 2.0)):
        expected = c.copy()
        expected[:, m:] = 0
        oracle.bgemm(ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, expected, ldc)
        for family in ("tensor", "tensor_pair"):
            actual = run_bgemm(ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc, family)
            assert np.all(actual[:, m:] == NAN)
            error = oracle.rel_l2(oracle.bf16_values(actual[:, :m]), oracle.bf16_values(expected[:, :m]))
            assert error <= BF16_TOLERANCE, (family, error)


@pytest.mark.parametrize("width", [128, 144, 208, 240])
def test_two_sm_kernel_with_a_run_time_tile_width(rng, width):
    """The context option pair_width=<n> makes the two-SM kernel use tiles of n
    columns (any multiple of 16): ragged last tiles, slabs beyond the matrix and a
    packed projection whose outputs meet inside a tile all have to come out right."""
    with _native.options(pair_width=width):
        _run_time_width_cases(rng, width)


def _run_time_width_cases(rng, width):
    for m, n, k in [(264, 130, 136), (1000, 300, 520), (592, 512, 2048)]:
        w, x, c = normal_bits(rng, (m, k)), normal_bits(rng, (n, k)), normal_bits(rng, (n, m))
        expected = c.copy()
        oracle.bgemm("T", "N", m, n, k, 0.5, w, k, x, k, -1.0, expected, m)
        actual = run_bgemm("T", "N", m, n, k, 0.5, w, k, x, k, -1.0, c, m, "tensor_pair")
        error = oracle.rel_l2(oracle.bf16_values(actual), oracle.bf16_values(expected))
        assert error <= BF16_TOLERANCE, (width, m, n, k, error)
    rows, inner, widths = 200, 256, (400, 112, 112)
    x, w = normal_bits(rng, (rows, inner)), normal_bits(rng, (sum(widths), inner))
    expected = oracle.bf16_values(oracle.linear_bf16(x, w))
    with _native.kernel_family("tensor_pair"):
        q, k, v = _kernels.qkv_linear(bits_to_tensor(x), bits_to_tensor(w), *widths)
    packed = torch.cat([q, k, v], dim=1).float().cpu().numpy()
    assert oracle.rel_l2(packed, expected) <= BF16_TOLERANCE


@pytest.mark.parametrize("rows", [65, 200, 600])
@pytest.mark.parametrize("widths", [(400, 112, 112), (320, 64, 64), (256, 128, 72)])
def test_packed_projection_of_any_widths_in_automatic_mode(rng, rows, widths):
    """The reference's qkv_linear is three independent linears and takes any widths
    (torch_bindings.cpp:725-736). With more than 64 token rows the automatic choice
    is a tensor-core row kernel, which serves a packed projection in one launch only
    when the outputs start on 128-column boundaries; other widths must be split into
    three products, not refused. Compared bit for bit with three linear() calls."""
    inner = 512
    x = bits_to_tensor(normal_bits(rng, (rows, inner)))
    w = bits_to_tensor(normal_bits(rng, (sum(widths), inner), 0.05))
    q, k, v = _kernels.qkv_linear(x, w, *widths)
    assert _native.context(0).device_status() == 0
    parts = [_kernels.linear(x, part.contiguous()) for part in torch.split(w, list(widths))]
    for got, expected in zip((q, k, v), parts):
        assert got.shape == expected.shape and torch.equal(got, expected)
    reference = oracle.bf16_values(oracle.linear_bf16(tensor_to_bits(x[:8]), tensor_to_bits(w)))
    packed = torch.cat([q, k, v], dim=1)[:8].float().cpu().numpy()
    assert oracle.rel_l2(packed, reference) <= BF16_TOLERANCE


@pytest.mark.parametrize("widths", [(8192, 1024, 1024), (4096, 512, 512), (2048, 256, 256),
                                    (1024, 128, 128)])
def test_packed_projection_at_the_sharded_widths(widths):
    """QKV of the M=512 block on 1, 2, 4 and 8 ranks (whole heads per rank): one launch
    with three outputs must give what three separate linear layers give. The narrower
    shards have few tiles and take the one-SM route; K is split differently there, so the
    comparison is by tolerance, plus sampled FP64 dot products."""
    torch.manual_seed(705537 + widths[0])
    rows, inner = 512, 8192
    x = torch.randn(rows, inner, device="cuda").bfloat16()
    w = (torch.randn(sum(widths), inner, device="cuda") * 0.02).bfloat16()
    q, k, v = _kernels.qkv_linear(x, w, *widths)
    assert _native.context(0).device_status() == 0
    assert q.shape == (rows, widths[0]) and k.shape == (rows, widths[1]) and v.shape == (rows, widths[2])
    packed = torch.cat([q, k, v], dim=1).float()
    separate = torch.cat([_kernels.linear(x, part) for part in torch.split(w, list(widths))],
                         dim=1).float()
    assert ((packed - separate).norm() / separate.norm()).item() <= 2e-3
    generator = torch.Generator().manual_seed(11)
    picks_r = torch.randint(0, rows, (64,), generator=generator)
    picks_c = torch.randint(0, sum(widths), (64,), generator=generator)
    expected = (x[picks_r].double().cpu() * w[picks_c].double().cpu()).sum(1)
    got = packed[picks_r, picks_c].double().cpu()
    assert ((got - expected).norm() / expected.norm()).item() <= BF16_TOLERANCE


@pytest.mark.parametrize("rows,outputs,inner", [
    (512, 1280, 8192),    # the QKV shard of one rank at tensor-parallel 8: 20 tiles of 128 x 256
    (130, 1536, 2048),    # ragged rows: 12 tiles, large clusters
    (200, 2500, 1100),    # ragged columns and a K that is not a multiple of 64
    (16, 8192, 4096),     # few tokens: swapped kernel, 64 tiles, clusters of two
    (3, 4096, 8192),      # swapped, 16-column tiles
    (64, 5000, 2304),     # swapped, 64-column tiles, ragged weight rows
])
def test_k_split_inside_a_cluster(rng, rows, outputs, inner):
    """Products with few tiles and a long K split K over the CTAs of a cluster and add the
    partial accumulators through distributed shared memory. Checked against the oracle on a
    row sample, against the route through scratch and a second launch (context option
    cluster_split=0; different summation order, so by tolerance), with bias and residual,
    and for repeatability."""
    with _native.options(cluster_split=2):  # 2: the few-token tiles take it too
        _k_split_inside_a_cluster(rng, rows, outputs, inner)


def _k_split_inside_a_cluster(rng, rows, outputs, inner):
    x = bits_to_tensor(normal_bits(rng, (rows, inner)))
    w = bits_to_tensor(normal_bits(rng, (outputs, inner), 0.05))
    bias = bits_to_tensor(normal_bits(rng, (outputs,)))
    residual = bits_to_tensor(normal_bits(rng, (rows, outputs)))
    native = _native.context(0)
    before = native.kernel_launches()
    first = _kernels.linear(x, w, bias, residual)
    launches = native.kernel_launches() - before
    second = _kernels.linear(x, w, bias, residual)
    assert native.device_status() == 0
    assert launches == 1, "the cluster split is one launch"
    assert torch.equal(first, second)
    with _native.options(cluster_split=0):
        other = _kernels.linear(x, w, bias, residual)
    assert ((first.float() - other.float()).norm() / other.float().norm()).item() <= 2e-3
    sample = slice(0, min(rows, 6))
    expected = oracle.bf16_values(oracle.linear_bf16(tensor_to_bits(x[sample]), tensor_to_bits(w),
                                                     tensor_to_bits(bias), tensor_to_bits(residual[sample])))
    assert oracle.rel_l2(first[sample].float().cpu().numpy(), expected) <= BF16_TOLERANCE
    # exact small integers: a wrong row owner or slot shows as a wrong integer
    xi = bits_to_tensor(oracle.bf16_bits(rng.integers(-1, 2, (rows, inner)).astype(np.float32)))
    wi = bits_to_tensor(oracle.bf16_bits(rng.integers(-1, 2, (outputs, inner)).astype(np.float32)))
    exact = (xi.double() @ wi.double().t())
    keep = exact.abs() <= 256
    got = _kernels.linear(xi, wi).double()
    assert torch.equal(got[keep], exact[keep])


def test_packed_projection_through_the_cluster_split():
    """The QKV shard at tensor-parallel 8 (1024 + 128 + 128 outputs, K = 8192) is packed and
    has 20 tiles: one cluster launch must fill the three outputs like three linears."""
    torch.manual_seed(705537)
    rows, inner, widths = 512, 8192, (1024, 128, 128)
    x = torch.randn(rows, inner, device="cuda").bfloat16()
    w = (torch.randn(sum(widths), inner, device="cuda") * 0.02).bfloat16()
    native = _native.context(0)
    before = native.kernel_launches()
    q, k, v = _kernels.qkv_linear(x, w, *widths)
    assert native.kernel_launches() - before == 1
    assert native.device_status() == 0
    parts = [_kernels.linear(x, part.contiguous()) for part in torch.split(w, list(widths))]
    for got, expected in zip((q, k, v), parts):
        assert ((got.float() - expected.float()).norm() / expected.float().norm()).item() <= 2e-3
    generator = torch.Generator().manual_seed(3)
    picks_r = torch.randint(0, rows, (64,), generator=generator)
    picks_c = torch.randint(0, sum(widths), (64,), generator=generator)
    expected = (x[picks_r].double().cpu() * w[picks_c].double().cpu()).sum(1)
    got = torch.cat([q, k, v], dim=1)[picks_r, picks_c].double().cpu()
    assert ((got - expected).norm() / expected.norm()).item() <= BF16_TOLERANCE
