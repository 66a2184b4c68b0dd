"""The CPU restatement against the reference's golden vectors and its own CPU GEMM.

Known-answer cases are those of the reference's tests, re-derived here:
identity placement and the [256, 1, -256] FP32-accumulation probe
(tests/test_bfloat16.py:94-110), alpha == 0 fills (:112-121), the FP8 decode
answer x=0.5, W=2.0 -> 2K with the last scale block doubled
(tests/test_quantized.py:196-216, 0x38 = 1.0, 0x40 = 2.0, NaN byte 0x7F),
the constant-row RMS case (tests/test_inference_fusion.py:106-110) and the
sparse selector / cancellation GEMV cases (tests/test_float_gemv.py:69-90).
"""

import hashlib
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import oracle

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_storage_conversions_match_torch():
    patterns = np.arange(256, dtype=np.uint8)
    expected = torch.from_numpy(patterns).view(torch.float8_e4m3fn).float().numpy()
    actual = oracle.e4m3_values(patterns)
    assert np.array_equal(np.isnan(expected), np.isnan(actual))
    assert np.array_equal(expected[~np.isnan(expected)], actual[~np.isnan(actual)])
    rng = np.random.default_rng(1)
    values = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s
                             for s in (1e-3, 0.02, 1.0, 100.0, 600.0)])
    encoded = np.array([oracle.lib().oracle_float_to_e4m3(float(v)) for v in values], dtype=np.uint8)
    torch_encoded = torch.from_numpy(np.clip(values, -448, 448)).to(torch.float8_e4m3fn)
    assert np.array_equal(encoded, torch_encoded.view(torch.uint8).numpy())
    bits = oracle.bf16_bits(values)
    assert np.array_equal(bits, torch.from_numpy(values).bfloat16().view(torch.int16).numpy().view(np.uint16))


def test_sgemm_is_bit_identical_to_reference_library(rng):
    if oracle.reference_lib() is None:
        pytest.skip("reference library not built")
    for rows, outputs, inner in [(1, 33, 17), (5, 64, 129), (20, 7, 300)]:
        x = rng.standard_normal((rows, inner)).astype(np.float32)
        w = rng.standard_normal((outputs, inner)).astype(np.float32)
        expected = oracle.reference_linear_f32(x, w)
        actual = np.zeros((rows, outputs), dtype=np.float32)
        oracle.sgemm("T", "N", outputs, rows, inner, 1.0, w, inner, x, inner, 0.0, actual, outputs)
        assert np.array_equal(actual, expected)


def test_golden_small_products():
    data = np.load(GOLDEN / "gemm_small.npz")
    for index in range(3):
        x, w, y = data[f"x{index}"], data[f"w{index}"], data[f"y{index}"]
        out = oracle.linear_bf16(x, w)
        # the restatement rounds the same FP32 sums once to BF16
        assert np.array_equal(out, oracle.bf16_bits(y))
        column_major = np.zeros((x.shape[0], w.shape[0]), dtype=np.uint16)
        oracle.bgemm("T", "N", w.shape[0], x.shape[0], x.shape[1], 1.0, w, w.shape[1], x,
                     x.shape[1], 0.0, column_major, w.shape[0])
        assert np.array_equal(column_major, out)


def test_golden_config1_inputs_and_output():
    from tests.golden.make_golden import config1_inputs

    data = np.load(GOLDEN / "c1_decode.npz")
    x, w = config1_inputs(int(data["seed"]))
    sha = hashlib.sha256()
    sha.update(np.ascontiguousarray(x).tobytes())
    sha.update(np.ascontiguousarray(w).tobytes())
    assert sha.hexdigest() == str(data["sha256"]), "seeded generator no longer reproduces the fixture"
    out = oracle.linear_bf16(x, w)
    assert np.array_equal(out, oracle.bf16_bits(data["y"]))


def test_bgemm_identity_and_accumulation_probe():
    one = oracle.bf16_bits(np.float32(1.0))
    n = 16
    identity = np.zeros((n, n), dtype=np.uint16)
    identity[np.arange(n), np.arange(n)] = one
    rng = np.random.default_rng(3)
    b = oracle.bf16_bits(rng.standard_normal((n, n)).astype(np.float32))
    for ta in "NT":
        c = np.zeros((n, n), dtype=np.uint16)
        oracle.bgemm(ta, "N", n, n, n, 1.0, identity, n, b, n, 0.0, c, n)
        assert np.array_equal(c, b)
    # [256, 1, -256] . [1, 1, 1] = 1 only if the sum is kept in FP32
    a = oracle.bf16_bits(np.array([256.0, 1.0, -256.0], dtype=np.float32))
    ones = oracle.bf16_bits(np.ones(3, dtype=np.float32))
    c = np.zeros(1, dtype=np.uint16)
    oracle.bgemm("T", "N", 1, 1, 3, 1.0, a, 3, ones, 3, 0.0, c, 1)
    assert oracle.bf16_values(c)[0] == 1.0


def test_bgemm_alpha_zero_does_not_read_operands():
    nan = np.full((4, 4), 0x7FC0, dtype=np.uint16)
    c = np.full((4, 4), 0x7FC0, dtype=np.uint16)
    oracle.bgemm("N", "N", 4, 4, 4, 0.0, nan, 4, nan, 4, 0.0, c, 4)
    assert np.all(c == 0)
    c = oracle.bf16_bits(np.full((4, 4), 2.0, dtype=np.float32))
    oracle.bgemm("N", "N", 4, 4, 4, 0.0, nan, 4, nan, 4, -0.75, c, 4)
    assert np.all(oracle.bf16_values(c) == -1.5)


def test_gemv_selector_and_cancellation():
    inner = 4096
    w = np.zeros((8, inner), dtype=np.float32)
    w[np.arange(8), np.arange(8) * 511] = 1.0
    x = np.arange(inner, dtype=np.float32) % 251
    out = oracle.linear_bf16(oracle.bf16_bits(x)[None, :], oracle.bf16_bits(w))
    assert np.array_equal(oracle.bf16_values(out)[0], x[np.arange(8) * 511])
    w = np.zeros((1, inner), dtype=np.float32)
    w[0, [0, 1, 2]] = [256.0, 1.0, -256.0]
    out = oracle.linear_bf16(oracle.bf16_bits(np.ones((1, inner), dtype=np.float32)), oracle.bf16_bits(w))
    assert oracle.bf16_values(out)[0, 0] == 1.0


def test_rms_constant_row_gives_weight():
    width = 4096
    x = oracle.bf16_bits(np.full((1, width), 3.0, dtype=np.float32))
    r = oracle.bf16_bits(np.full((1, width), 1.0, dtype=np.float32))
    gamma = oracle.bf16_bits((np.arange(width) % 16).astype(np.float32))
    added, out = oracle.add_rms_norm_rows(x, r, gamma, 0.0)
    assert np.all(oracle.bf16_values(added) == 4.0)
    assert np.array_equal(out[0], gamma)


def test_rms_against_double_precision(rng):
    width = 8192
    x = oracle.bf16_bits(rng.standard_normal((3, width)).astype(np.float32))
    r = oracle.bf16_bits(rng.standard_normal((3, width)).astype(np.float32))
    gamma = oracle.bf16_bits((1 + 0.1 * rng.standard_normal(width)).astype(np.float32))
    added, out = oracle.add_rms_norm_rows(x, r, gamma, 1e-5)
    v = oracle.bf16_values(x).astype(np.float64) + oracle.bf16_values(r).astype(np.float64)
    assert np.array_equal(added, oracle.bf16_bits(v.astype(np.float32)))
    v = oracle.bf16_values(added).astype(np.float64)
    expected = v / np.sqrt((v * v).mean(axis=1, keepdims=True) + 1e-5) * oracle.bf16_values(gamma)
    assert oracle.rel_l2(oracle.bf16_values(out), expected) < 5e-3
    multi = oracle.rms_norm_rows(added, gamma, 1e-5)
    assert oracle.rel_l2(oracle.bf16_values(multi), expected) < 5e-3


def test_fp8_decode_known_answer():
    # x = 1.0 (0x38) with input scale 0.5, W = 2.0 (0x40) with weight scale 2:
    # every output is 2K; the last 32-row scale block is doubled again.
    inner, outputs = 256, 64
    x = np.full(inner, 0x38, dtype=np.uint8)
    w = np.full((outputs, inner), 0x40, dtype=np.uint8)
    sx = np.full(inner // 32, 0.5, dtype=np.float32)
    sw = np.full((outputs // 32, inner // 32), 2.0, dtype=np.float32)
    sw[-1, :] = 4.0
    out = oracle.bf16_values(oracle.fp8_decode(x, sx, w, sw))
    assert np.all(out[:32] == 2 * inner) and np.all(out[32:] == 4 * inner)
    # 0x33 is 0.6875: 256 * 1.0 * 0.6875 = 176 with unit scales
    ones = np.ones_like(sw)
    out = oracle.fp8_decode(x, np.ones_like(sx), np.full((outputs, inner), 0x33, dtype=np.uint8), ones)
    assert np.all(oracle.bf16_values(out) == 176.0)
    w[5, 7] = 0x7F
    out = oracle.bf16_values(oracle.fp8_decode(x, sx, w, sw))
    assert np.isnan(out[5]) and not np.isnan(out[4])


def test_fp8_power_of_two_quantiser(rng):
    x = oracle.bf16_bits(rng.standard_normal(256).astype(np.float32) * 3)
    q, scale = oracle.fp8_quantize_block32(x)
    exponents = np.log2(scale)
    assert np.array_equal(exponents, np.round(exponents))
    values = oracle.bf16_values(x).reshape(-1, 32)
    amax = np.abs(values).max(axis=1)
    assert np.all(scale * 448 >= amax) and np.all(scale * 224 < amax)
    restored = oracle.e4m3_values(q).reshape(-1, 32) * scale[:, None]
    assert oracle.rel_l2(restored, values) < 0.04


def test_fp8_block128_quantiser_and_product_against_reference_gemm():
    data = np.load(GOLDEN / "fp8_slice.npz")
    q, q_scale = oracle.fp8_quantize_rows(data["x"])
    wq, w_scale = oracle.fp8_quantize_weight(data["w"])
    assert np.array_equal(q, data["q"]) and np.array_equal(wq, data["wq"])
    assert np.array_equal(q_scale, data["q_scale"]) and np.array_equal(w_scale, data["w_scale"])
    amax = np.abs(oracle.bf16_values(data["x"])).reshape(3, -1, 128).max(axis=2)
    assert np.allclose(q_scale, np.maximum(amax, 1e-10) / 448, rtol=1e-6)
    out = oracle.bf16_values(oracle.fp8_block_gemm(q, q_scale, wq, w_scale))
    # reference FP32 GEMM on the dequantised operands
    assert oracle.rel_l2(out, data["y"]) < 5e-3
    # and the quantised product approximates the BF16 product within the FP8 bound
    exact = oracle.bf16_values(data["x"]).astype(np.float64) @ oracle.bf16_values(data["w"]).astype(np.float64).T
    assert oracle.rel_l2(out, exact) < 5e-2


def test_strassen_matches_classical_within_stated_bound(rng):
    n = 64
    a = np.asfortranarray(oracle.bf16_bits(rng.uniform(-1, 1, (n, n)).astype(np.float32)))
    b = np.asfortranarray(oracle.bf16_bits(rng.uniform(-1, 1, (n, n)).astype(np.float32)))
    fast = oracle.strassen_bf16(a, b)
    classical = np.zeros((n, n), dtype=np.uint16, order="F")
    oracle.bgemm("N", "N", n, n, n, 1.0, a, n, b, n, 0.0, classical, n)
    exact = oracle.bf16_values(a).astype(np.float64) @ oracle.bf16_values(b).astype(np.float64)
    error_classical = oracle.rel_l2(oracle.bf16_values(classical), exact)
    error_fast = oracle.rel_l2(oracle.bf16_values(fast), exact)
    assert error_classical < 5e-3
    assert error_fast < 1e-2


def test_silu_and_swiglu(rng):
    gate = oracle.bf16_bits(rng.standard_normal((4, 64)).astype(np.float32) * 4)
    up = oracle.bf16_bits(rng.standard_normal((4, 64)).astype(np.float32))
    g, u = oracle.bf16_values(gate).astype(np.float64), oracle.bf16_values(up).astype(np.float64)
    expected = g / (1 + np.exp(-g)) * u
    assert oracle.rel_l2(oracle.bf16_values(oracle.silu_multiply_bf16(gate, up)), expected) < 1e-2
    routing = rng.uniform(0.5, 1.5, 4).astype(np.float32)
    clipped = np.minimum(g, 2.0) / (1 + np.exp(-np.minimum(g, 2.0))) * np.clip(u, -2.0, 2.0)
    out = oracle.swiglu_bf16(gate, up, 2.0, routing)
    assert oracle.rel_l2(oracle.bf16_values(out), clipped * routing[:, None]) < 5e-3
