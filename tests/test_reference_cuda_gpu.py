"""This library against the reference's own CUDA library on the same device buffers.

`oracle/_ref/libcamblas_cuda_ref.so` is the reference's `src/cuda/backend.cu`
compiled unmodified for sm_100a by `oracle/Makefile` (its BF16 GEMM is cuBLAS /
cuBLASLt, `src/cuda/bfloat16.cuh:37-56`, `backend.cu:559-784`; its RMS and
elementwise kernels are its own, `src/cuda/inference_fusion.cuh`). Both
libraries export the same C ABI, so each test makes the same call on both with
the same inputs, one GPU, own memory only, and compares the outputs:

* BF16 GEMM (all transpose pairs, padded leading dimensions, alpha/beta,
  classical and `lt` policies): rel-L2 <= 1e-2 between the two, and each within
  1e-2 of the CPU oracle - the two sum in different orders, so not bitwise;
* residual add + RMS norm, single-row RMS norm with its flags, multi-row RMS
  norm, BF16 squares, RMS scaling, SiLU multiply, SwiGLU: **bit for bit**,
  because this library performs the reference's FP32 operations in the
  reference's order and both are compiled by the same compiler.

Test infrastructure only: the package never loads the reference library. The
tests are skipped when it has not been built (no reference sources at build
time).
"""

import ctypes as ct
from pathlib import Path

import numpy as np
import pytest
import torch

from camblas_b200 import _native
from oracle import oracle
from tests.helpers import BF16_TOLERANCE, bits_to_tensor, normal_bits, pointer, tensor_to_bits

pytestmark = pytest.mark.gpu
REFERENCE_LIBRARY = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "libcamblas_cuda_ref.so"
NAN = 0x7FC0


class Library:
    """One of the two libraries with a context of its own on the current stream."""

    def __init__(self, handle):
        self.lib = handle
        for name, (arguments, result) in _native._SIGNATURES.items():
            function = getattr(handle, "camblas_cuda_" + name, None)
            if function is not None:
                function.argtypes, function.restype = arguments, result
        self.context = ct.c_void_p()
        stream = ct.c_void_p(torch.cuda.current_stream().cuda_stream)
        status = handle.camblas_cuda_create(0, stream, ct.byref(self.context))
        assert status == 0, handle.camblas_cuda_error(None)

    def call(self, name, *arguments):
        status = getattr(self.lib, "camblas_cuda_" + name)(self.context, *arguments)
        assert status == 0, (name, self.lib.camblas_cuda_error(self.context))

    def close(self):
        self.lib.camblas_cuda_destroy(self.context)


@pytest.fixture(scope="module")
def both():
    if not REFERENCE_LIBRARY.is_file():
        pytest.skip("the reference's CUDA library was not built (no reference sources at build time)")
    torch.cuda.set_device(0)
    ours = Library(ct.CDLL(str(_native.library_path())))
    theirs = Library(ct.CDLL(str(REFERENCE_LIBRARY)))
    yield ours, theirs
    torch.cuda.synchronize()
    ours.close()
    theirs.close()


def padded(rng, rows, columns, ld, scale=1.0):
    buffer = np.full((columns, ld), NAN, dtype=np.uint16)
    buffer[:, :rows] = normal_bits(rng, (columns, rows), scale)
    return buffer


@pytest.mark.parametrize("policy", [1, 3])  # classical, lt
@pytest.mark.parametrize("ta,tb", [("N", "N"), ("N", "T"), ("T", "N"), ("T", "T")])
@pytest.mark.parametrize("m,n,k", [(5, 3, 7), (130, 70, 257), (520, 200, 264), (1024, 512, 1024),
                                   (4096, 1, 2048), (8192, 16, 1024)])
def test_bgemm_against_the_reference_library(both, rng, policy, ta, tb, m, n, k):
    ours, theirs = both
    pad = 8 if min(m, n, k) >= 64 else 3  # cuBLASLt and TMA paths want aligned pitches; small shapes go ragged
    lda = (m if ta == "N" else k) + pad
    ldb = (k if tb == "N" else n) + pad
    ldc = m + pad
    a = padded(rng, m if ta == "N" else k, k if ta == "N" else m, lda, 0.25)
    b = padded(rng, k if tb == "N" else n, n if tb == "N" else k, ldb)
    c = padded(rng, m, n, ldc)
    da, db = bits_to_tensor(a), bits_to_tensor(b)
    for alpha, beta in ((1.0, 0.0), (0.5, -1.25)):
        outputs = []
        for library in (ours, theirs):
            dc = bits_to_tensor(c)
            library.call("set_algorithm", policy)
            library.call("bgemm", ta.encode(), tb.encode(), m, n, k, alpha, pointer(da), lda,
                         pointer(db), ldb, beta, pointer(dc), ldc)
            torch.cuda.synchronize()
            outputs.append(tensor_to_bits(dc))
        mine, reference = outputs
        assert np.all(mine[:, m:] == NAN) and np.all(reference[:, m:] == NAN)
        values, expected = oracle.bf16_values(mine[:, :m]), oracle.bf16_values(reference[:, :m])
        assert oracle.rel_l2(values, expected) <= BF16_TOLERANCE
        if m * n * k <= 130 * 70 * 257:
            exact = c.copy()
            exact[:, m:] = 0
            oracle.bgemm(ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, exact, ldc)
            exact = oracle.bf16_values(exact[:, :m])
            assert oracle.rel_l2(values, exact) <= BF16_TOLERANCE
            assert oracle.rel_l2(expected, exact) <= BF16_TOLERANCE


def gamma_bits(rng, width):
    return oracle.bf16_bits((1 + 0.1 * rng.standard_normal(width)).astype(np.float32))


@pytest.mark.parametrize("width", [2048, 4096, 8192, 12288, 65536, 2052])
def test_add_rms_norm_bit_for_bit(both, rng, width):
    ours, theirs = both
    x = bits_to_tensor(normal_bits(rng, (1, width)))
    r = bits_to_tensor(normal_bits(rng, (1, width)))
    g = bits_to_tensor(gamma_bits(rng, width))
    results = []
    for library in (ours, theirs):
        added, out = torch.zeros_like(x), torch.zeros_like(x)
        library.call("add_rms_norm", 2, width, 1e-5, pointer(x), pointer(r), pointer(g),
                     pointer(added), pointer(out))
        torch.cuda.synchronize()
        results.append((added, out))
    assert torch.equal(results[0][0], results[1][0]), "added differs"
    assert torch.equal(results[0][1], results[1][1]), "normalised output differs"


def test_add_rms_norm_rows_equals_the_reference_row_by_row(both, rng):
    """The reference handles one row per call; this library's many-row entry point must
    give, row by row, exactly what the reference's single-row kernel gives."""
    ours, theirs = both
    rows, width = 24, 8192
    x = bits_to_tensor(normal_bits(rng, (rows, width)))
    r = bits_to_tensor(normal_bits(rng, (rows, width)))
    g = bits_to_tensor(gamma_bits(rng, width))
    added, out = torch.zeros_like(x), torch.zeros_like(x)
    ours.call("add_rms_norm_rows", 2, rows, width, 1e-5, pointer(x), pointer(r), pointer(g),
              pointer(added), pointer(out))
    expected_added, expected_out = torch.zeros_like(x), torch.zeros_like(x)
    for row in range(rows):
        theirs.call("add_rms_norm", 2, width, 1e-5, pointer(x[row]), pointer(r[row]), pointer(g),
                    pointer(expected_added[row]), pointer(expected_out[row]))
    torch.cuda.synchronize()
    assert torch.equal(added, expected_added) and torch.equal(out, expected_out)


def test_add_rms_norm_fp32_bit_for_bit(both, rng):
    ours, theirs = both
    width = 4096
    x = torch.from_numpy(rng.standard_normal((1, width)).astype(np.float32)).cuda()
    r = torch.from_numpy(rng.standard_normal((1, width)).astype(np.float32)).cuda()
    g = torch.from_numpy((1 + 0.1 * rng.standard_normal(width)).astype(np.float32)).cuda()
    results = []
    for library in (ours, theirs):
        added, out = torch.zeros_like(x), torch.zeros_like(x)
        library.call("add_rms_norm", 0, width, 1e-6, pointer(x), pointer(r), pointer(g),
                     pointer(added), pointer(out))
        torch.cuda.synchronize()
        results.append((added, out))
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])


@pytest.mark.parametrize("weight_fp32", [False, True])
@pytest.mark.parametrize("round_first", [0, 1])
@pytest.mark.parametrize("descending", [0, 1])
def test_rms_norm_decode_bit_for_bit(both, rng, weight_fp32, round_first, descending):
    ours, theirs = both
    width = 6144
    x = bits_to_tensor(normal_bits(rng, (1, width)))
    g_bits = gamma_bits(rng, width)
    g = torch.from_numpy(oracle.bf16_values(g_bits)).cuda() if weight_fp32 else bits_to_tensor(g_bits)
    results = []
    for library in (ours, theirs):
        out = torch.zeros_like(x)
        library.call("rms_norm_decode", 2, 0 if weight_fp32 else 2, width, 1e-5, round_first,
                     descending, pointer(x), pointer(g), pointer(out))
        torch.cuda.synchronize()
        results.append(out)
    assert torch.equal(results[0], results[1])


@pytest.mark.parametrize("rows,width", [(1, 8192), (64, 4096), (33, 1000), (5, 127), (3, 20480)])
@pytest.mark.parametrize("dtype", [2, 0])
def test_rms_norm_rows_bit_for_bit(both, rng, rows, width, dtype):
    ours, theirs = both
    if dtype == 2:
        x, g = bits_to_tensor(normal_bits(rng, (rows, width))), bits_to_tensor(gamma_bits(rng, width))
    else:
        x = torch.from_numpy(rng.standard_normal((rows, width)).astype(np.float32)).cuda()
        g = torch.from_numpy((1 + 0.1 * rng.standard_normal(width)).astype(np.float32)).cuda()
    results = []
    for library in (ours, theirs):
        out = torch.zeros_like(x)
        library.call("rms_norm", dtype, rows, width, 1e-5, pointer(x), pointer(g), pointer(out))
        torch.cuda.synchronize()
        results.append(out)
    assert torch.equal(results[0], results[1])


def test_square_and_scale_bit_for_bit(both, rng):
    ours, theirs = both
    for rows, width in ((6, 1024), (7, 1001)):
        x = bits_to_tensor(normal_bits(rng, (rows, width)))
        g = bits_to_tensor(gamma_bits(rng, width))
        results = []
        for library in (ours, theirs):
            squares = torch.zeros((rows, width), dtype=torch.float32, device="cuda")
            library.call("bfloat16_square", rows * width, pointer(x), pointer(squares))
            means = squares.mean(dim=1).contiguous()
            out = torch.zeros_like(x)
            library.call("rms_scale", 2, rows * width, width, 1e-5, pointer(x), pointer(g),
                         pointer(means), pointer(out))
            torch.cuda.synchronize()
            results.append((squares, out))
        assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])


@pytest.mark.parametrize("dtype", [2, 0])
def test_silu_multiply_and_swiglu_bit_for_bit(both, rng, dtype):
    ours, theirs = both
    for rows, width in ((8, 512), (3, 333)):
        if dtype == 2:
            gate = bits_to_tensor(normal_bits(rng, (rows, width), 4.0))
            up = bits_to_tensor(normal_bits(rng, (rows, width)))
        else:
            gate = torch.from_numpy((4 * rng.standard_normal((rows, width))).astype(np.float32)).cuda()
            up = torch.from_numpy(rng.standard_normal((rows, width)).astype(np.float32)).cuda()
        routing = torch.from_numpy(rng.uniform(0.5, 1.5, rows).astype(np.float32)).cuda()
        results = []
        for library in (ours, theirs):
            plain, clipped, routed = (torch.zeros_like(gate) for _ in range(3))
            library.call("silu_multiply", dtype, rows * width, pointer(gate), pointer(up), pointer(plain))
            library.call("swiglu", dtype, rows * width, width, 2.0, pointer(gate), pointer(up), None,
                         pointer(clipped))
            library.call("swiglu", dtype, rows * width, width, 0.0, pointer(gate), pointer(up),
                         pointer(routing), pointer(routed))
            torch.cuda.synchronize()
            results.append((plain, clipped, routed))
        for mine, reference in zip(*results):
            assert torch.equal(mine, reference)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("ta,tb", [("N", "N"), ("N", "T"), ("T", "N"), ("T", "T")])
@pytest.mark.parametrize("m,n,k", [(5, 3, 7), (130, 70, 257), (300, 129, 64), (512, 512, 512)])
def test_sgemm_dgemm_against_the_reference_library_and_float64(both, rng, dtype, ta, tb, m, n, k):
    """FP32/FP64 GEMM (off the BF16/FP8 path; a tiled CUDA-core kernel here, cuBLAS in the
    reference): same C-ABI call on both libraries, padded leading dimensions with NaN
    canaries, alpha/beta; each within a few units of the type's rounding of the float64
    product, scaled by sqrt(k) for the differing summation orders."""
    ours, theirs = both
    name = "sgemm" if dtype is np.float32 else "dgemm"
    lda, ldb, ldc = (m if ta == "N" else k) + 3, (k if tb == "N" else n) + 5, m + 2

    def padded_matrix(rows, columns, ld):
        buffer = np.full((columns, ld), np.nan, dtype=dtype)
        buffer[:, :rows] = rng.standard_normal((columns, rows)).astype(dtype)
        return buffer

    a = padded_matrix(m if ta == "N" else k, k if ta == "N" else m, lda)
    b = padded_matrix(k if tb == "N" else n, n if tb == "N" else k, ldb)
    c = padded_matrix(m, n, ldc)
    op_a = a[:, :m].T if ta == "N" else a[:, :k]       # m x k
    op_b = b[:, :k].T if tb == "N" else b[:, :n]       # k x n
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    eps = np.finfo(dtype).eps
    for alpha, beta in ((1.0, 0.0), (0.5, -1.25)):
        exact = alpha * (op_a.astype(np.float64) @ op_b.astype(np.float64)) + beta * c[:, :m].T.astype(np.float64)
        bound = 8 * eps * np.sqrt(k) * (np.abs(alpha) * (np.abs(op_a).astype(np.float64) @ np.abs(op_b))
                                         + np.abs(beta * c[:, :m].T))
        for library in (ours, theirs):
            dc = torch.from_numpy(c).cuda()
            library.call("set_algorithm", 1)
            library.call(name, ta.encode(), tb.encode(), m, n, k, alpha, pointer(da), lda, pointer(db),
                         ldb, beta, pointer(dc), ldc)
            torch.cuda.synchronize()
            result = dc.cpu().numpy()
            assert np.all(np.isnan(result[:, m:])), "padding rows of C were written"
            assert np.all(np.abs(result[:, :m].T - exact) <= bound + 1e-300)


def _device(array):
    return torch.from_numpy(np.ascontiguousarray(array)).cuda()


def _close(actual, exact, dtype, terms):
    """rel-L2 within a few roundings of `dtype` per summed term."""
    error = np.linalg.norm(actual.astype(np.float64) - exact) / max(np.linalg.norm(exact), 1e-300)
    return error <= 16 * np.finfo(dtype).eps * np.sqrt(max(terms, 1))


@pytest.mark.parametrize("dtype,code", [(np.float32, 0), (np.float64, 1)])
@pytest.mark.parametrize("rows,inputs,hidden,outputs", [(5, 7, 9, 3), (130, 96, 200, 64), (1, 300, 1, 17)])
def test_affine_and_two_layer_perceptron(both, rng, dtype, code, rows, inputs, hidden, outputs):
    """camblas_cuda_affine (with and without ReLU) and camblas_cuda_mlp on both libraries
    against float64: row-major x . w + bias, ReLU after the first layer, the hidden
    activations handed back to the caller."""
    ours, theirs = both
    x = rng.standard_normal((rows, inputs)).astype(dtype)
    w1, b1 = rng.standard_normal((inputs, hidden)).astype(dtype), rng.standard_normal(hidden).astype(dtype)
    w2, b2 = rng.standard_normal((hidden, outputs)).astype(dtype), rng.standard_normal(outputs).astype(dtype)
    hidden_exact = np.maximum(x.astype(np.float64) @ w1 + b1, 0)
    plain_exact = x.astype(np.float64) @ w1 + b1
    dx, dw1, db1, dw2, db2 = map(_device, (x, w1, b1, w2, b2))
    for library in (ours, theirs):
        out = torch.full((rows, hidden), float("nan"), dtype=dx.dtype, device="cuda")
        library.call("affine", code, rows, inputs, hidden, pointer(dx), pointer(dw1), pointer(db1), 0,
                     pointer(out))
        torch.cuda.synchronize()
        assert _close(out.cpu().numpy(), plain_exact, dtype, inputs)
        h = torch.full((rows, hidden), float("nan"), dtype=dx.dtype, device="cuda")
        y = torch.full((rows, outputs), float("nan"), dtype=dx.dtype, device="cuda")
        library.call("mlp", code, rows, inputs, hidden, outputs, pointer(dx), pointer(dw1), pointer(db1),
                     pointer(dw2), pointer(db2), pointer(h), pointer(y))
        torch.cuda.synchronize()
        assert _close(h.cpu().numpy(), hidden_exact, dtype, inputs)
        assert _close(y.cpu().numpy(), h.cpu().numpy().astype(np.float64) @ w2 + b2, dtype, hidden)
    counts = (ct.c_uint64 * 8)()
    assert ours.lib.camblas_cuda_stats(ours.context, counts, 8) == 0 and counts[3] >= 3


@pytest.mark.parametrize("dtype,code", [(np.float32, 0), (np.float64, 1)])
@pytest.mark.parametrize("queries,keys,depth,values", [(4, 6, 8, 5), (100, 300, 64, 48), (8, 32, 256, 256),
                                                       (3, 5000, 16, 7)])
def test_single_head_attention(both, rng, dtype, code, queries, keys, depth, values):
    """softmax(scale q k^T) v on both libraries against float64 (the third case is the one
    the reference serves with its fused FP64 kernel, fusion.cuh:110-127)."""
    ours, theirs = both
    q = rng.standard_normal((queries, depth)).astype(dtype)
    k = rng.standard_normal((keys, depth)).astype(dtype)
    v = rng.standard_normal((keys, values)).astype(dtype)
    scale = 1.0 / np.sqrt(depth)
    scores = scale * (q.astype(np.float64) @ k.astype(np.float64).T)
    weights = np.exp(scores - scores.max(axis=1, keepdims=True))
    exact = (weights / weights.sum(axis=1, keepdims=True)) @ v
    dq, dk, dv = map(_device, (q, k, v))
    for library in (ours, theirs):
        out = torch.full((queries, values), float("nan"), dtype=dq.dtype, device="cuda")
        library.call("attention", code, queries, keys, depth, values, scale, pointer(dq), pointer(dk),
                     pointer(dv), pointer(out))
        torch.cuda.synchronize()
        assert _close(out.cpu().numpy(), exact, dtype, depth + keys)


@pytest.mark.parametrize("dtype,code", [(np.float32, 0), (np.float64, 1)])
@pytest.mark.parametrize("rows,inputs,hidden,outputs", [(6, 5, 7, 4), (300, 64, 130, 33)])
def test_perceptron_backward(both, rng, dtype, code, rows, inputs, hidden, outputs):
    """All six gradients of the two-layer perceptron on both libraries against float64,
    then a call that asks for the second layer's gradients only (NULL elsewhere)."""
    ours, theirs = both
    x = rng.standard_normal((rows, inputs)).astype(dtype)
    w1 = rng.standard_normal((inputs, hidden)).astype(dtype)
    w2 = rng.standard_normal((hidden, outputs)).astype(dtype)
    h = np.maximum(x @ w1 + rng.standard_normal(hidden).astype(dtype), 0).astype(dtype)
    g = rng.standard_normal((rows, outputs)).astype(dtype)
    h64, g64 = h.astype(np.float64), g.astype(np.float64)
    dh_exact = (g64 @ w2.astype(np.float64).T) * (h64 > 0)
    exact = {"dh": dh_exact, "dx": dh_exact @ w1.astype(np.float64).T,
             "dw1": x.astype(np.float64).T @ dh_exact, "db1": dh_exact.sum(axis=0),
             "dw2": h64.T @ g64, "db2": g64.sum(axis=0)}
    terms = {"dh": outputs, "dx": hidden, "dw1": rows, "db1": rows, "dw2": rows, "db2": rows}
    dx_, dw1_, dw2_, dh_, dg_ = map(_device, (x, w1, w2, h, g))
    for library in (ours, theirs):
        outs = {name: torch.full(value.shape, float("nan"), dtype=dx_.dtype, device="cuda")
                for name, value in exact.items()}
        library.call("mlp_backward", code, rows, inputs, hidden, outputs, pointer(dx_), pointer(dw1_),
                     pointer(dw2_), pointer(dh_), pointer(dg_), pointer(outs["dh"]), pointer(outs["dx"]),
                     pointer(outs["dw1"]), pointer(outs["db1"]), pointer(outs["dw2"]), pointer(outs["db2"]))
        torch.cuda.synchronize()
        for name, value in exact.items():
            assert _close(outs[name].cpu().numpy(), value, dtype, terms[name]), name
        second = {name: torch.full(exact[name].shape, float("nan"), dtype=dx_.dtype, device="cuda")
                  for name in ("dw2", "db2")}
        library.call("mlp_backward", code, rows, inputs, hidden, outputs, pointer(dx_), pointer(dw1_),
                     pointer(dw2_), pointer(dh_), pointer(dg_), None, None, None, None,
                     pointer(second["dw2"]), pointer(second["db2"]))
        torch.cuda.synchronize()
        for name in second:
            assert _close(second[name].cpu().numpy(), exact[name], dtype, rows), name


def test_layer_compositions_reject_what_the_reference_rejects(both):
    ours, _ = both
    x = torch.zeros(4, 4, device="cuda")
    for name, arguments in (
            ("affine", (0, -1, 4, 4, pointer(x), pointer(x), pointer(x), 0, pointer(x))),
            ("affine", (0, 4, 4, 4, pointer(x), pointer(x), None, 0, pointer(x))),
            ("affine", (2, 4, 4, 4, pointer(x), pointer(x), pointer(x), 0, pointer(x))),
            ("attention", (0, 4, 4, 4, 4, 1.0, pointer(x), pointer(x), pointer(x), None)),
            ("attention", (3, 4, 4, 4, 4, 1.0, pointer(x), pointer(x), pointer(x), pointer(x))),
            ("mlp_backward", (0, 4, 4, 4, 4, pointer(x), pointer(x), pointer(x), pointer(x), None,
                              None, None, None, None, pointer(x), None))):
        status = getattr(ours.lib, "camblas_cuda_" + name)(ours.context, *arguments)
        assert status < 0, name
    # empty problems succeed without touching anything
    assert ours.lib.camblas_cuda_affine(ours.context, 0, 0, 4, 4, None, None, None, 0, None) == 0
    assert ours.lib.camblas_cuda_attention(ours.context, 0, 0, 4, 4, 4, 1.0, None, None, None, None) == 0
