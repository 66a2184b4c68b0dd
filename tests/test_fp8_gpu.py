"""FP8 E4M3 w8a8 parity through the C ABI.

The quantiser is byte-exact against the oracle. The block-scaled GEMM is checked
(1) against the oracle's per-block recurrence and (2) against the reference's
FP32 CPU GEMM on the dequantised operands, both within rel-L2 <= 2e-2
(FP8_TOLERANCE, the bound the benchmark definition states; in practice the
first is below 1e-3 because only the in-block summation order differs), and
bit for bit on known-answer inputs. The single-token block-32 entry points
follow the reference's tests/test_quantized.py:160-216.
"""

from pathlib import Path

import numpy as np
import pytest
import torch

from camblas_b200 import _kernels, _native
from oracle import oracle
from tests.helpers import (FP8_TOLERANCE, bits_to_tensor, error_text, normal_bits, pointer, raw,
                           tensor_to_bits)

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def fp8_tensor(array):
    return torch.from_numpy(np.ascontiguousarray(array)).cuda().view(torch.float8_e4m3fn)


def fp8_bytes(tensor):
    return tensor.view(torch.uint8).cpu().numpy()


@pytest.mark.parametrize("rows,inner", [(1, 128), (3, 256), (17, 1536), (130, 7168)])
def test_row_quantiser_is_byte_exact(rng, rows, inner):
    x = normal_bits(rng, (rows, inner), 3.0)
    x[0, :128] = 0  # an all-zero group takes the 1e-10 floor
    expected_q, expected_scale = oracle.fp8_quantize_rows(x)
    q, scale = _kernels.fp8_quantize(bits_to_tensor(x))
    assert np.array_equal(fp8_bytes(q), expected_q)
    assert np.array_equal(scale.cpu().numpy(), expected_scale)
    # strided input rows
    wide = bits_to_tensor(np.concatenate([x, x], axis=1))[:, :inner]
    q2, scale2 = _kernels.fp8_quantize(wide)
    assert torch.equal(q2.view(torch.uint8), q.view(torch.uint8)) and torch.equal(scale2, scale)


@pytest.mark.parametrize("swapped_rows", [16, 128, 0])
@pytest.mark.parametrize("rows", [1, 5, 16, 17, 33, 64, 65, 128, 300])
@pytest.mark.parametrize("outputs,inner", [(128, 128), (264, 256), (1000, 1536), (2112, 512)])
def test_block_gemm_against_oracle(rng, rows, outputs, inner, swapped_rows):
    """Every row count through the default choice of kernel, through the swapped
    (weights on the 128-row side) kernel wherever it is allowed, and through the row
    tiling alone."""
    x, w = normal_bits(rng, (rows, inner)), normal_bits(rng, (outputs, inner))
    q, q_scale = oracle.fp8_quantize_rows(x)
    wq, w_scale = oracle.fp8_quantize_weight(w)
    expected = oracle.bf16_values(oracle.fp8_block_gemm(q, q_scale, wq, w_scale))
    with _native.options(fp8_swapped_rows=swapped_rows):
        out = _kernels.fp8_block_gemm(fp8_tensor(q), torch.from_numpy(q_scale).cuda(),
                                      fp8_tensor(wq), torch.from_numpy(w_scale).cuda())
        torch.cuda.synchronize()
    assert _native.context(0).device_status() == 0
    error = oracle.rel_l2(out.float().cpu().numpy(), expected)
    assert error <= FP8_TOLERANCE and error < 4e-3, error


def test_block_gemm_known_answer():
    # q = 1.0 with scale 0.5, w = 2.0 with scale 2: every output is 2K, exactly;
    # the second weight band is scaled by 4 instead.
    for rows in (1, 24, 130):
        outputs, inner = 256, 512
        q = np.full((rows, inner), 0x38, dtype=np.uint8)
        w = np.full((outputs, inner), 0x40, dtype=np.uint8)
        q_scale = np.full((rows, inner // 128), 0.5, dtype=np.float32)
        w_scale = np.full((2, inner // 128), 2.0, dtype=np.float32)
        w_scale[1] = 4.0
        out = _kernels.fp8_block_gemm(fp8_tensor(q), torch.from_numpy(q_scale).cuda(),
                                      fp8_tensor(w), torch.from_numpy(w_scale).cuda())
        values = out.float().cpu().numpy()
        assert np.all(values[:, :128] == 2 * inner) and np.all(values[:, 128:] == 4 * inner)
        w[7, 3] = 0x7F  # a NaN weight poisons exactly its own output feature
        out = _kernels.fp8_block_gemm(fp8_tensor(q), torch.from_numpy(q_scale).cuda(),
                                      fp8_tensor(w), torch.from_numpy(w_scale).cuda())
        assert torch.isnan(out[:, 7]).all() and not torch.isnan(out[:, 8]).any()


def test_golden_slice_against_reference_gemm_on_dequantised_operands():
    data = np.load(GOLDEN / "fp8_slice.npz")
    q, scale = _kernels.fp8_quantize(bits_to_tensor(data["x"]))
    assert np.array_equal(fp8_bytes(q), data["q"]) and np.array_equal(scale.cpu().numpy(), data["q_scale"])
    out = _kernels.fp8_block_gemm(q, scale, fp8_tensor(data["wq"]),
                                  torch.from_numpy(data["w_scale"]).cuda())
    assert oracle.rel_l2(out.float().cpu().numpy(), data["y"]) <= FP8_TOLERANCE


def test_block_gemm_rejects_bad_arguments(rng):
    q = fp8_tensor(np.zeros((4, 256), dtype=np.uint8))
    scale = torch.ones((4, 2), device="cuda")
    w = fp8_tensor(np.zeros((128, 256), dtype=np.uint8))
    w_scale = torch.ones((1, 2), device="cuda")
    out = torch.empty((4, 128), dtype=torch.bfloat16, device="cuda")
    for arguments in [(4, 128, 200, pointer(q), pointer(scale), pointer(w), pointer(w_scale), pointer(out), 128),
                      (4, 128, 256, pointer(q), pointer(scale), pointer(w), pointer(w_scale), pointer(out), 100),
                      (4, 128, 256, None, pointer(scale), pointer(w), pointer(w_scale), pointer(out), 128),
                      (4, 128, 256, pointer(q), pointer(scale), pointer(w), pointer(w_scale), pointer(w), 128)]:
        status, context = raw("fp8_block_gemm", *arguments)
        assert status == -1, error_text(context)
    with pytest.raises(ValueError):
        _kernels.fp8_block_gemm(q, scale[:, :1], w, w_scale)
    with pytest.raises(ValueError):
        _kernels.fp8_quantize(torch.zeros((2, 100), dtype=torch.bfloat16, device="cuda"))


@pytest.mark.parametrize("outputs,inner", [(48, 96), (1152, 5120), (5120, 576), (64, 8192)])
def test_single_token_block32(rng, outputs, inner):
    assert _kernels.fp8_decode_supported(0)
    x = normal_bits(rng, (inner,), 2.0)
    w = normal_bits(rng, (outputs, inner))
    xq, sx = oracle.fp8_quantize_block32(x)
    wq = torch.from_numpy(oracle.bf16_values(w)).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    sw = rng.uniform(0.5, 2.0, ((outputs + 31) // 32, inner // 32)).astype(np.float32)
    expected = oracle.bf16_values(oracle.fp8_decode(xq, sx, wq, sw))
    out = _kernels.fp8_decode(fp8_tensor(xq), torch.from_numpy(sx).cuda(), fp8_tensor(wq),
                              torch.from_numpy(sw).cuda())
    assert oracle.rel_l2(out.float().cpu().numpy(), expected) < 4e-3
    fused = _kernels.fp8_linear(bits_to_tensor(x), fp8_tensor(wq), torch.from_numpy(sw).cuda())
    assert torch.equal(fused, out)  # the in-kernel quantiser reproduces the oracle's bytes and scales
    # strided scale views are honoured
    wide = torch.from_numpy(np.repeat(sw, 2, axis=1)).cuda()[:, ::2]
    assert torch.equal(_kernels.fp8_decode(fp8_tensor(xq), torch.from_numpy(sx).cuda(), fp8_tensor(wq), wide), out)


def test_single_token_known_answer_and_nan():
    for outputs, inner in ((48, 96), (1152, 5120)):
        x = np.full(inner, 0x38, dtype=np.uint8)
        w = np.full((outputs, inner), 0x40, dtype=np.uint8)
        sx = np.full(inner // 32, 0.5, dtype=np.float32)
        sw = np.full(((outputs + 31) // 32, inner // 32), 2.0, dtype=np.float32)
        sw[-1] *= 2
        out = _kernels.fp8_decode(fp8_tensor(x), torch.from_numpy(sx).cuda(), fp8_tensor(w),
                                  torch.from_numpy(sw).cuda()).float().cpu().numpy()
        expected = np.full(outputs, 2.0 * inner, dtype=np.float32)
        expected[((outputs + 31) // 32 - 1) * 32:] *= 2
        assert np.array_equal(out, oracle.bf16_values(oracle.bf16_bits(expected)))
        half = bits_to_tensor(oracle.bf16_bits(np.full(inner, 0.5, dtype=np.float32)))
        fused = _kernels.fp8_linear(half, fp8_tensor(w), torch.from_numpy(sw).cuda()).float().cpu().numpy()
        assert np.array_equal(fused, out)
        w[:] = 0x7F
        assert torch.isnan(_kernels.fp8_decode(fp8_tensor(x), torch.from_numpy(sx).cuda(), fp8_tensor(w),
                                               torch.from_numpy(sw).cuda())).all()
    with pytest.raises(ValueError):
        _kernels.fp8_decode(fp8_tensor(np.zeros(100, np.uint8)), torch.ones(3, device="cuda"),
                            fp8_tensor(np.zeros((16, 100), np.uint8)), torch.ones((1, 3), device="cuda"))


@pytest.mark.parametrize("outputs,inner", [(4096, 7168), (7168, 2048), (2112, 7168), (24576, 1536)])
@pytest.mark.parametrize("rows", [1, 16, 128, 4096])
def test_benchmark_shapes(outputs, inner, rows):
    """The FP8 benchmark grid: quantise on the GPU, multiply, and compare a sample of
    rows and output features with (1) the oracle's block recurrence on the same
    quantised bytes and (2) the FP32 GEMM of the reference's CPU library on the
    dequantised operands."""
    generator = torch.Generator(device="cuda").manual_seed(705540)
    x = torch.randn(rows, inner, device="cuda", generator=generator).bfloat16()
    w = torch.randn(outputs, inner, device="cuda", generator=generator).bfloat16()
    q, q_scale = _kernels.fp8_quantize(x)
    wq_host, w_scale_host = oracle.fp8_quantize_weight(tensor_to_bits(w))
    wq, w_scale = fp8_tensor(wq_host), torch.from_numpy(w_scale_host).cuda()
    out = _kernels.fp8_block_gemm(q, q_scale, wq, w_scale)
    assert _native.context(0).device_status() == 0
    row_sample = np.unique(np.linspace(0, rows - 1, 6).astype(int))
    features = np.unique(np.concatenate([np.arange(0, 128, 37), np.arange(outputs - 70, outputs, 9)]))
    q_host, qs_host = fp8_bytes(q)[row_sample], q_scale.cpu().numpy()[row_sample]
    # (1) block recurrence: evaluate whole 128-row bands so the band scales line up
    bands = np.unique(features // 128)
    for band in bands:
        lo, hi = band * 128, min(outputs, band * 128 + 128)
        expected = oracle.bf16_values(oracle.fp8_block_gemm(q_host, qs_host, wq_host[lo:hi],
                                                            w_scale_host[band:band + 1]))
        actual = out[row_sample][:, lo:hi].float().cpu().numpy()
        assert oracle.rel_l2(actual, expected) < 4e-3
        # (2) reference FP32 GEMM on the dequantised operands
        dequantised = oracle.reference_linear_f32(
            oracle.fp8_dequantize(q_host, qs_host, 1),
            oracle.fp8_dequantize(wq_host[lo:hi], w_scale_host[band:band + 1], 128))
        assert oracle.rel_l2(actual, dequantised) <= FP8_TOLERANCE


@pytest.mark.parametrize("rows,outputs,inner", [
    (129, 264, 128),      # one ragged tile, a second band of eight columns
    (300, 384, 256),      # ragged rows, a half-used column tile
    (1000, 2112, 512),    # the last column tile holds 64 columns
    (4096, 4096, 1536),   # the size at which the 256-column tiles are the default
    (2304, 7168, 2048),   # an odd number of 128-row blocks: the last pair holds one
])
def test_many_row_kernels_give_the_same_bits(rng, rows, outputs, inner):
    """The 128 x 128 row kernel (option fp8_rows = 5), the 128 x 256 form (3), the two-SM
    256 x 256 form (4) and the choice by size (0) promote the same block sums in the same
    order, so their outputs agree bit for bit; the first is checked against the oracle's
    recurrence on a sample of rows."""
    generator = torch.Generator(device="cuda").manual_seed(705541 + rows)
    x = torch.randn(rows, inner, device="cuda", generator=generator).bfloat16()
    w = torch.randn(outputs, inner, device="cuda", generator=generator).bfloat16()
    q, q_scale = _kernels.fp8_quantize(x)
    wq_host, w_scale_host = oracle.fp8_quantize_weight(tensor_to_bits(w))
    wq, w_scale = fp8_tensor(wq_host), torch.from_numpy(w_scale_host).cuda()
    results = {}
    for variant in (5, 3, 4, 0):
        with _native.options(fp8_rows=variant):
            results[variant] = _kernels.fp8_block_gemm(q, q_scale, wq, w_scale)
            torch.cuda.synchronize()
            assert _native.context(0).device_status() == 0
    for variant in (3, 4, 0):
        assert torch.equal(results[variant], results[5]), variant
    sample = np.unique(np.linspace(0, rows - 1, 5).astype(int))
    expected = oracle.bf16_values(oracle.fp8_block_gemm(fp8_bytes(q)[sample], q_scale.cpu().numpy()[sample],
                                                        wq_host[:256], w_scale_host[:2]))
    actual = results[5][sample][:, :256].float().cpu().numpy()
    assert oracle.rel_l2(actual, expected) < 4e-3


@pytest.mark.parametrize("rows,outputs,inner", [
    (128, 4096, 7168),   # 32 tiles, four K ranges each
    (100, 2112, 7168),   # 17 tiles (the last holds 64 columns), ragged rows
    (88, 1000, 4096),    # eight tiles, the last ragged, eight K ranges
    (81, 1032, 4096),    # nine tiles, the last eight columns wide
    (40, 1000, 4096),    # fewer than 80 rows: the two-launch form either way
    (256, 512, 8192),    # two row blocks
])
def test_k_ranges_in_a_cluster(rng, rows, outputs, inner):
    """Few tiles and a long K: the K ranges of a tile are the CTAs of a cluster and their
    FP32 sums meet in distributed shared memory. Against the two-launch form (ranges to
    scratch, then a reduction; option cluster_split = 0), which may cut K differently, and
    against the oracle's recurrence on a sample of rows."""
    generator = torch.Generator(device="cuda").manual_seed(88172 + rows)
    x = torch.randn(rows, inner, device="cuda", generator=generator).bfloat16()
    w = torch.randn(outputs, inner, device="cuda", generator=generator).bfloat16()
    q, q_scale = _kernels.fp8_quantize(x)
    wq_host, w_scale_host = oracle.fp8_quantize_weight(tensor_to_bits(w))
    wq, w_scale = fp8_tensor(wq_host), torch.from_numpy(w_scale_host).cuda()
    results = {}
    for cluster_split in (1, 0):
        with _native.options(cluster_split=cluster_split):
            first = _kernels.fp8_block_gemm(q, q_scale, wq, w_scale)
            again = _kernels.fp8_block_gemm(q, q_scale, wq, w_scale)
            torch.cuda.synchronize()
            assert _native.context(0).device_status() == 0
            assert torch.equal(first, again)
            results[cluster_split] = first
    assert oracle.rel_l2(results[1].float().cpu().numpy(), results[0].float().cpu().numpy()) < 3e-3
    sample = np.unique(np.linspace(0, rows - 1, 4).astype(int))
    columns = min(outputs, 256)
    bands = (columns + 127) // 128
    expected = oracle.bf16_values(oracle.fp8_block_gemm(fp8_bytes(q)[sample], q_scale.cpu().numpy()[sample],
                                                        wq_host[:columns], w_scale_host[:bands]))
    for result in results.values():
        actual = result[sample][:, :columns].float().cpu().numpy()
        assert oracle.rel_l2(actual, expected) < 4e-3
    bands_all = w_scale_host.shape[0]
    expected = oracle.bf16_values(oracle.fp8_block_gemm(
        fp8_bytes(q)[sample], q_scale.cpu().numpy()[sample], wq_host[(bands_all - 1) * 128:],
        w_scale_host[bands_all - 1:]))
    actual = results[1][sample][:, (bands_all - 1) * 128:].float().cpu().numpy()
    assert oracle.rel_l2(actual, expected) < 4e-3
