"""Block-scaled E8M0 products and expert routing against the reference's own CUDA kernels.

The reference's `quantized_matmul`, `grouped_quantized_matmul`, `route_groups`
and `reduce_groups` kernels (`src/cuda/quantized.cuh`, `src/cuda/routing.cuh`)
run on sm_100a (they use the legacy `mma.sync` FP8 path), so
`oracle/_ref/libcamblas_cuda_ref.so` serves as the checker on the same device
buffers, next to a float64 restatement in numpy:

* products: rel-L2 <= 2e-2 (the FP8 bound) against float64 and against the
  reference library; both form every term a*w exactly and differ only in the
  order of FP32 additions, so the measured differences are near 1e-3;
* `reduce_groups`: bit for bit (same values added in the same order);
* `route_groups`: the reference numbers the rows of a group with an atomic
  counter, in no fixed order, so the comparison is of what the contract fixes:
  counts, the set of slots of every group, `reverse` and `slots` being inverse
  to each other, and -1 everywhere else. This library's numbering is ascending
  by slot, which is also checked.
"""

import ctypes as ct
from pathlib import Path

import numpy as np
import pytest
import torch

from camblas_b200 import _kernels, _native
from oracle import oracle
from tests.helpers import FP8_TOLERANCE, pointer

pytestmark = pytest.mark.gpu
REFERENCE_LIBRARY = Path(__file__).resolve().parents[1] / "oracle" / "_ref" / "libcamblas_cuda_ref.so"
E2M1 = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6])


@pytest.fixture(scope="module")
def reference():
    if not REFERENCE_LIBRARY.is_file():
        pytest.skip("the reference's CUDA library was not built")
    torch.cuda.set_device(0)
    library = ct.CDLL(str(REFERENCE_LIBRARY))
    for name, (arguments, result) in _native._SIGNATURES.items():
        function = getattr(library, "camblas_cuda_" + name, None)
        if function is not None:
            function.argtypes, function.restype = arguments, result
    context = ct.c_void_p()
    stream = ct.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert library.camblas_cuda_create(0, stream, ct.byref(context)) == 0

    def call(name, *arguments):
        status = getattr(library, "camblas_cuda_" + name)(context, *arguments)
        assert status == 0, (name, library.camblas_cuda_error(context))

    yield call
    torch.cuda.synchronize()
    library.camblas_cuda_destroy(context)


def scale_values(codes):
    return np.where(codes == 0, 2.0 ** -127, 2.0 ** (codes.astype(np.float64) - 127))


def random_case(rng, rows, outputs, inner, packed, block):
    x = rng.integers(0, 256, (rows, inner), dtype=np.uint8)
    x[(x & 0x7F) == 0x7F] = 0x38  # no NaN bytes
    x_codes = rng.integers(120, 131, (rows, inner // block), dtype=np.uint8)
    if packed:
        w = rng.integers(0, 256, (outputs, inner // 2), dtype=np.uint8)
        w_codes = rng.integers(120, 131, (outputs, inner // 32), dtype=np.uint8)
        nibbles = np.stack([w & 15, w >> 4], axis=-1).reshape(outputs, inner)
        w_values = E2M1[nibbles] * np.repeat(scale_values(w_codes), 32, axis=1)
    else:
        w = rng.integers(0, 256, (outputs, inner), dtype=np.uint8)
        w[(w & 0x7F) == 0x7F] = 0x38
        w_codes = rng.integers(120, 131, ((outputs + 31) // 32, inner // 32), dtype=np.uint8)
        w_values = oracle.e4m3_values(w).astype(np.float64) * np.repeat(
            np.repeat(scale_values(w_codes), 32, axis=0)[:outputs], 32, axis=1)
    x_values = oracle.e4m3_values(x).astype(np.float64) * np.repeat(scale_values(x_codes), block, axis=1)
    return x, x_codes, w, w_codes, x_values @ w_values.T


def device_bytes(array, dtype):
    return torch.from_numpy(array).cuda().view(dtype)


@pytest.mark.parametrize("packed,block", [(False, 32), (True, 32), (True, 128)])
@pytest.mark.parametrize("rows,outputs,inner", [(1, 64, 256), (5, 136, 512), (16, 512, 1024),
                                                (200, 264, 384), (1024, 2048, 2048)])
def test_quantized_matmul(rng, reference, packed, block, rows, outputs, inner):
    x, x_codes, w, w_codes, exact = random_case(rng, rows, outputs, inner, packed, block)
    weight_dtype = torch.float4_e2m1fn_x2 if packed else torch.float8_e4m3fn
    dx, dxs = device_bytes(x, torch.float8_e4m3fn), device_bytes(x_codes, torch.float8_e8m0fnu)
    dw, dws = device_bytes(w, weight_dtype), device_bytes(w_codes, torch.float8_e8m0fnu)
    out = _kernels.quantized_matmul(dx, dxs, dw, dws, block)
    assert _native.context(0).device_status() == 0
    assert oracle.rel_l2(out.float().cpu().numpy(), exact) <= FP8_TOLERANCE
    theirs = torch.zeros_like(out)
    reference("quantized_matmul", int(packed), rows, outputs, inner, block, pointer(dx), pointer(dxs),
              pointer(dw), pointer(dws), pointer(theirs))
    torch.cuda.synchronize()
    assert oracle.rel_l2(theirs.float().cpu().numpy(), exact) <= FP8_TOLERANCE
    assert oracle.rel_l2(out.float().cpu().numpy(), theirs.float().cpu().numpy()) <= 5e-3


def test_quantized_matmul_special_scales_and_rejections(rng):
    rows, outputs, inner = 4, 64, 128
    x, x_codes, w, w_codes, _ = random_case(rng, rows, outputs, inner, False, 32)
    x_codes[1, 2] = 255  # NaN scale: that row is NaN everywhere
    dx, dxs = device_bytes(x, torch.float8_e4m3fn), device_bytes(x_codes, torch.float8_e8m0fnu)
    dw, dws = device_bytes(w, torch.float8_e4m3fn), device_bytes(w_codes, torch.float8_e8m0fnu)
    out = _kernels.quantized_matmul(dx, dxs, dw, dws)
    assert torch.isnan(out[1]).all() and not torch.isnan(out[0]).any()
    with pytest.raises(ValueError):
        _kernels.quantized_matmul(dx, dxs, dw, dws, 128)  # FP8 weights take block 32 only
    with pytest.raises(ValueError):
        _kernels.quantized_matmul(dx[:, :96].contiguous(), dxs[:, :3].contiguous(), dw, dws)
    library, native = _native.library(), _native.context(0)
    status = library.camblas_cuda_quantized_matmul(native.handle, 0, rows, 12, inner, 32, pointer(dx),
                                                   pointer(dxs), pointer(dw), pointer(dws), pointer(out))
    assert status == -1 and b"invalid quantized matrix dimensions" in library.camblas_cuda_error(native.handle)


@pytest.mark.parametrize("packed", [False, True])
def test_grouped_quantized_matmul(rng, reference, packed):
    groups, experts, rows, outputs, inner, block = 5, 3, 24, 136, 256, 32
    weight_dtype = torch.float4_e2m1fn_x2 if packed else torch.float8_e4m3fn
    weights, scales, exact_weights = [], [], []
    for _ in range(experts):
        _, _, w, w_codes, _ = random_case(rng, 1, outputs, inner, packed, block)
        weights.append(device_bytes(w, weight_dtype))
        scales.append(device_bytes(w_codes, torch.float8_e8m0fnu))
    x = rng.integers(0, 256, (groups, rows, inner), dtype=np.uint8)
    x[(x & 0x7F) == 0x7F] = 0x38
    x_codes = rng.integers(120, 131, (groups, rows, inner // block), dtype=np.uint8)
    active = torch.tensor([2, 0, -1, 1, 7], dtype=torch.int32, device="cuda")  # -1 and 7 are invalid
    counts = torch.tensor([24, 5, 9, 0, 3], dtype=torch.int32, device="cuda")
    dx, dxs = device_bytes(x, torch.float8_e4m3fn), device_bytes(x_codes, torch.float8_e8m0fnu)
    group = _kernels.QuantizedGroups(weights, scales)
    out = group.matmul(dx, dxs, active, counts, block)
    theirs = torch.full_like(out, float("nan"))
    reference("grouped_quantized_matmul", int(packed), groups, experts, rows, outputs, inner, block,
              pointer(dx), pointer(dxs), pointer(group.metadata), pointer(active), pointer(counts),
              pointer(theirs))
    torch.cuda.synchronize()
    assert not torch.isnan(theirs).any()
    for batch, (selected, count) in enumerate(zip(active.tolist(), counts.tolist())):
        live = count if 0 <= selected < experts else 0
        assert torch.all(out[batch, live:] == 0) and torch.all(theirs[batch, live:] == 0)
        if live:
            plain = _kernels.quantized_matmul(dx[batch, :live].contiguous(), dxs[batch, :live].contiguous(),
                                              weights[selected], scales[selected], block)
            assert torch.equal(out[batch, :live], plain) or oracle.rel_l2(
                out[batch, :live].float().cpu().numpy(), plain.float().cpu().numpy()) <= 2e-3
            assert oracle.rel_l2(out[batch, :live].float().cpu().numpy(),
                                 theirs[batch, :live].float().cpu().numpy()) <= 5e-3


def test_route_and_reduce_groups(rng, reference):
    tokens, choices, rows, width = 300, 4, 40, 264
    first_expert = 16
    experts_host = rng.integers(10, 40, (tokens, choices)).astype(np.int64)
    experts_host[3, 1] = -5
    experts_host[7, 2] = 2 ** 40  # ignored: not below INT_MAX
    experts = torch.from_numpy(experts_host).cuda()
    active = torch.tensor([3, 0, 11, 5, 3, 20], dtype=torch.int32, device="cuda")  # 3 twice: first wins
    slots, reverse, counts = _kernels.route_groups(experts, active, first_expert, rows)
    ref_counts, ref_slots, ref_reverse = torch.zeros_like(counts), torch.zeros_like(slots), torch.zeros_like(reverse)
    reference("route_groups", tokens, choices, first_expert, active.numel(), rows, pointer(experts),
              pointer(active), pointer(ref_counts), pointer(ref_slots), pointer(ref_reverse))
    torch.cuda.synchronize()
    assert torch.equal(counts, ref_counts)
    flat = experts_host.reshape(-1)
    local = flat - first_expert
    active_host = active.cpu().numpy()
    for g in range(active.numel()):
        wanted = np.nonzero(local == active_host[g])[0] if g == list(active_host).index(active_host[g]) else np.array([], dtype=np.int64)
        assert counts[g].item() == len(wanted)
        kept = slots[g].cpu().numpy()
        taken = min(rows, len(wanted))
        assert np.array_equal(kept[:taken], wanted[:taken])  # ascending slot order, deterministic
        assert np.all(kept[taken:] == -1)
        theirs = np.sort(ref_slots[g].cpu().numpy()[:taken])
        if len(wanted) <= rows:
            assert np.array_equal(theirs, wanted)  # the reference holds the same set
    reverse_host, slots_host = reverse.cpu().numpy().reshape(-1), slots.cpu().numpy().reshape(-1)
    assigned = reverse_host >= 0
    assert np.array_equal(slots_host[reverse_host[assigned]], np.nonzero(assigned)[0])
    assert (slots_host >= 0).sum() == assigned.sum()

    grouped = torch.randn((active.numel(), rows, width), device="cuda").bfloat16()
    mine = _kernels.reduce_groups(grouped, experts, reverse)
    theirs = torch.full_like(mine, float("nan"))
    reference("reduce_groups", tokens, choices, width, active.numel() * rows, pointer(experts),
              pointer(reverse), pointer(grouped), pointer(theirs))
    torch.cuda.synchronize()
    assert torch.equal(mine, theirs)
    narrow = grouped[:, :, :101].contiguous()  # width not a multiple of eight: scalar path
    mine = _kernels.reduce_groups(narrow, experts, reverse)
    theirs = torch.full_like(mine, float("nan"))
    reference("reduce_groups", tokens, choices, 101, active.numel() * rows, pointer(experts),
              pointer(reverse), pointer(narrow), pointer(theirs))
    torch.cuda.synchronize()
    assert torch.equal(mine, theirs)


@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("rows", [1, 8, 17])
def test_known_answers_and_scale_extremes(reference, packed, rows):
    """The reference's own known-answer cases (tests/test_quantized.py:238-262, 311-320):
    x = 1.0 everywhere (E4M3 0x38), weight 1.0 (E4M3 0x38, or E2M1 nibbles 0x22) with unit
    weight scales, and input scales at the ends of the E8M0 range: 2^-127 (code 0), 1, 2^127
    and NaN. Every output is inner * 2^(code-127), exactly, NaN for code 255; a NaN input
    byte (0x7F) makes everything NaN; weight nibbles 0x33 (1.5) with inner = 32 give 48."""
    outputs, inner = 40, 64
    weight_dtype = torch.float4_e2m1fn_x2 if packed else torch.float8_e4m3fn
    x = torch.full((rows, inner), 0x38, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    w = torch.full((outputs, inner // 2 if packed else inner), 0x22 if packed else 0x38,
                   dtype=torch.uint8, device="cuda").view(weight_dtype)
    sw = torch.full((outputs if packed else 2, inner // 32), 127, dtype=torch.uint8,
                    device="cuda").view(torch.float8_e8m0fnu)
    for code in (0, 127, 254, 255):
        sx = torch.full((rows, inner // 32), code, dtype=torch.uint8, device="cuda").view(torch.float8_e8m0fnu)
        out = _kernels.quantized_matmul(x, sx, w, sw)
        theirs = torch.zeros_like(out)
        reference("quantized_matmul", int(packed), rows, outputs, inner, 32, pointer(x), pointer(sx),
                  pointer(w), pointer(sw), pointer(theirs))
        torch.cuda.synchronize()
        if code == 255:
            assert torch.isnan(out).all() and torch.isnan(theirs).all()
            continue
        expected = torch.full_like(out, 0).double() + inner * 2.0 ** (code - 127)
        expected = expected.to(torch.bfloat16)  # 2^134 overflows to inf, 2^-121 is a normal BF16
        assert torch.equal(theirs, expected)
        assert torch.equal(out, expected), (code, out[0, :4])
    ones = torch.full((rows, inner // 32), 127, dtype=torch.uint8, device="cuda").view(torch.float8_e8m0fnu)
    nan_input = torch.full((rows, inner), 0x7F, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    assert torch.isnan(_kernels.quantized_matmul(nan_input, ones, w, sw)).all()
    if packed:
        x32 = torch.full((1, 32), 0x38, dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
        w32 = torch.full((8, 16), 0x33, dtype=torch.uint8, device="cuda").view(weight_dtype)
        unit = torch.full((1, 1), 127, dtype=torch.uint8, device="cuda").view(torch.float8_e8m0fnu)
        units = torch.full((8, 1), 127, dtype=torch.uint8, device="cuda").view(torch.float8_e8m0fnu)
        out = _kernels.quantized_matmul(x32, unit, w32, units)
        assert torch.equal(out, torch.full((1, 8), 48, dtype=torch.bfloat16, device="cuda"))
