"""Row-parallel linear layer whose sum over ranks goes through peer memory.

`camblas_cuda_linear_bf16_allreduce` is three launches per rank: the tcgen05
product that writes its tiles into the owner's staging slots, the owner's
reduction and broadcast, and the delivery wait. The reference has no such
operation (its tensor parallelism is SGLang's all-reduce after the hooked
`F.linear`, `camblas/sglang.py:250-285`), so the checker is the oracle's BF16
linear layer on the whole inner dimension (tolerance rel-L2 <= 1e-2, the BF16
bound of the other GEMM tests; the partial products are rounded to BF16 before
they are summed, as SGLang's BF16 all-reduce does) and, for small-integer
operands whose partial sums are exact, bit equality.

One GPU is enough: all ranks' regions live on it and the phases of the ranks
are issued in turn (all products, then all reductions, then all waits), so no
kernel ever waits for one that has not been launched. The same entry point with
one process per GPU is exercised by `tests/test_row_parallel_multi_gpu.py`.
"""

import numpy as np
import pytest
import torch

from camblas_b200 import _native
from camblas_b200.tp import PeerRegions
from oracle import oracle
from tests.helpers import BF16_TOLERANCE, bits_to_tensor, normal_bits, tensor_to_bits

pytestmark = pytest.mark.gpu


def run_emulated(views, xs, ws, bias=None, residual=None):
    """Issue one call on every emulated rank, phase by phase; return each rank's result bits."""
    for phase in (1, 2, 4):
        for view, x, w in zip(views, xs, ws):
            view.linear(x, w, bias, residual, phases=phase)
    torch.cuda.synchronize()
    assert _native.context(0).device_status() == 0
    rows, outputs = xs[0].shape[0], ws[0].shape[0]
    return [tensor_to_bits(view.result(rows, outputs)) for view in views]


def make_case(rng, world, rows, inner, outputs, scale=1.0):
    x = normal_bits(rng, (rows, world * inner), scale)
    w = normal_bits(rng, (outputs, world * inner), 0.05)
    xs = [bits_to_tensor(x[:, r * inner:(r + 1) * inner]) for r in range(world)]
    ws = [bits_to_tensor(w[:, r * inner:(r + 1) * inner]) for r in range(world)]
    return x, w, xs, ws


def close_all(views):
    for view in views:
        view.close(free=True)


@pytest.mark.parametrize("world,rows,inner,outputs", [
    (1, 512, 256, 1024),
    (2, 512, 512, 1024),
    (2, 300, 200, 1000),   # ragged rows, columns and depth
    (3, 257, 136, 520),    # owners get unequal numbers of column blocks
    (4, 64, 128, 256),     # fewer column blocks than ranks: some own nothing
    (8, 512, 192, 2048),
    (8, 33, 72, 136),
])
def test_matches_oracle_and_ranks_agree(world, rows, inner, outputs):
    rng = np.random.default_rng(20261004 + world * 1000 + rows)
    x, w, xs, ws = make_case(rng, world, rows, inner, outputs)
    views = PeerRegions.emulate(PeerRegions.capacity_for(rows, outputs), world, 0)
    try:
        first = run_emulated(views, xs, ws)
        second = run_emulated(views, xs, ws)
    finally:
        close_all(views)
    expected = oracle.bf16_values(oracle.linear_bf16(x, w))
    assert oracle.rel_l2(oracle.bf16_values(first[0]), expected) <= BF16_TOLERANCE
    for r in range(1, world):
        assert np.array_equal(first[r], first[0]), f"rank {r} differs from rank 0"
    # flag words were cleared by their consumers: the next call works and repeats the bits
    for r in range(world):
        assert np.array_equal(second[r], first[r])


def test_bias_and_residual_enter_once():
    world, rows, inner, outputs = 4, 384, 256, 768
    rng = np.random.default_rng(73013)
    x, w, xs, ws = make_case(rng, world, rows, inner, outputs)
    bias = normal_bits(rng, (outputs,))
    residual = normal_bits(rng, (rows, outputs))
    views = PeerRegions.emulate(PeerRegions.capacity_for(rows, outputs), world, 0)
    try:
        got = run_emulated(views, xs, ws, bits_to_tensor(bias), bits_to_tensor(residual))
    finally:
        close_all(views)
    expected = oracle.bf16_values(oracle.linear_bf16(x, w, bias, residual))
    assert oracle.rel_l2(oracle.bf16_values(got[0]), expected) <= BF16_TOLERANCE
    for r in range(1, world):
        assert np.array_equal(got[r], got[0])


def test_exact_integers_are_bit_exact():
    """Entries in {-1,0,1}: every partial and the sum are integers below 256, exact in BF16."""
    world, rows, inner, outputs = 8, 290, 24, 776
    rng = np.random.default_rng(705537)
    x = oracle.bf16_bits(rng.integers(-1, 2, (rows, world * inner)).astype(np.float32))
    w = oracle.bf16_bits(rng.integers(-1, 2, (outputs, world * inner)).astype(np.float32))
    bias = oracle.bf16_bits(rng.integers(-8, 9, (outputs,)).astype(np.float32))
    residual = oracle.bf16_bits(rng.integers(-8, 9, (rows, outputs)).astype(np.float32))
    xs = [bits_to_tensor(x[:, r * inner:(r + 1) * inner]) for r in range(world)]
    ws = [bits_to_tensor(w[:, r * inner:(r + 1) * inner]) for r in range(world)]
    views = PeerRegions.emulate(PeerRegions.capacity_for(rows, outputs), world, 0)
    try:
        got = run_emulated(views, xs, ws, bits_to_tensor(bias), bits_to_tensor(residual))
    finally:
        close_all(views)
    expected = oracle.linear_bf16(x, w, bias, residual)
    for r in range(world):
        assert np.array_equal(got[r], expected)


def test_narrow_tiles_give_the_same_sum():
    """The 128-column tile variant (tuning aid) is the same arithmetic."""
    world, rows, inner, outputs = 2, 512, 320, 1536
    rng = np.random.default_rng(99)
    x, w, xs, ws = make_case(rng, world, rows, inner, outputs)
    views = PeerRegions.emulate(PeerRegions.capacity_for(rows, outputs), world, 0)
    try:
        wide = run_emulated(views, xs, ws)
        with _native.options(push_width=128):
            narrow = run_emulated(views, xs, ws)
    finally:
        close_all(views)
    assert np.array_equal(wide[0], narrow[0])
    assert np.array_equal(narrow[1], narrow[0])


@pytest.mark.parametrize("world", [2, 8])
def test_benchmark_shape_against_partial_products(world):
    """The down projection of the benchmark (512 x 28672 -> 8192) split over `world` ranks:
    the exchanged result equals the sum of the ranks' BF16 partial products (each rounded
    once, summed in FP32 in rank order, rounded once) bit for bit - the partial products
    come from the same two-SM kernel without a stream-K split - and is within the BF16
    tolerance of the unsharded product."""
    from camblas_b200 import _kernels

    torch.manual_seed(705537 + world)
    rows, inner, outputs = 512, 28672, 8192
    x = torch.randn(rows, inner, device="cuda").bfloat16()
    w = (torch.randn(outputs, inner, device="cuda") * 0.02).bfloat16()
    step = inner // world
    xs = [x[:, r * step:(r + 1) * step].contiguous() for r in range(world)]
    ws = [w[:, r * step:(r + 1) * step].contiguous() for r in range(world)]
    views = PeerRegions.emulate(PeerRegions.capacity_for(rows, outputs), world, 0)
    try:
        got = run_emulated(views, xs, ws)
    finally:
        close_all(views)
    total = torch.zeros((rows, outputs), dtype=torch.float32, device="cuda")
    for x_r, w_r in zip(xs, ws):
        total += _kernels.linear(x_r, w_r).float()
    expected = tensor_to_bits(total.bfloat16())
    assert np.array_equal(got[0], expected)
    for r in range(1, world):
        assert np.array_equal(got[r], got[0])
    full = _kernels.linear(x, w).float().cpu().numpy()
    assert oracle.rel_l2(oracle.bf16_values(got[0]), full) <= BF16_TOLERANCE


def test_rejects_what_it_cannot_do():
    views = PeerRegions.emulate(64 * 64, 2, 0)
    try:
        x = torch.zeros((64, 64), dtype=torch.bfloat16, device="cuda")
        w = torch.zeros((128, 64), dtype=torch.bfloat16, device="cuda")
        with pytest.raises(RuntimeError, match="capacity"):
            views[0].linear(x, w)
        w_odd = torch.zeros((60, 64), dtype=torch.bfloat16, device="cuda")
        with pytest.raises(RuntimeError, match="multiples of 8"):
            views[0].linear(x, w_odd)
        with pytest.raises(RuntimeError, match="group description"):
            views[0].linear(x, w[:64], phases=8)
    finally:
        close_all(views)
    with pytest.raises(ValueError):
        PeerRegions.emulate(16, 9, 0)


def test_expired_wait_reports_and_reset_recovers():
    """A rank whose peer never sends: the bounded wait runs out, the kernel returns, the
    status word names the wait, and after camblas_cuda_peer_reset the regions work again.

    Rank 0 of two emulated ranks issues its product (one arrival per slab at the owner,
    which is rank 0 itself) and then its reduction, which needs two arrivals per slab and
    never gets the second because rank 1 launches nothing. The wait limit is lowered to
    50 ms through the context option so that the test is quick; nothing traps or faults,
    the kernel simply gives up. The stale arrival words (one instead of zero) would let
    the next call start on incomplete data, which is what the reset is for.
    """
    world, rows, inner, outputs = 2, 256, 128, 256
    rng = np.random.default_rng(20261127)
    x, w, xs, ws = make_case(rng, world, rows, inner, outputs)
    views = PeerRegions.emulate(PeerRegions.capacity_for(rows, outputs), world, 0)
    native = _native.context(0)
    try:
        good = run_emulated(views, xs, ws)
        with _native.options(peer_wait_ms=50):
            views[0].linear(xs[0], ws[0], phases=1)
            views[0].linear(xs[0], ws[0], phases=6)
            torch.cuda.synchronize()  # returns: the waits were bounded
            status = _native.context(0).device_status()
        assert status & 15 in (6, 7), hex(status)  # kRolePeerArrive / kRolePeerDelivered
        assert native.device_status() == 0  # reading cleared it
        for view in views:
            view.reset()
        torch.cuda.synchronize()
        again = run_emulated(views, xs, ws)
    finally:
        close_all(views)
    for r in range(world):
        assert np.array_equal(again[r], good[r])


@pytest.mark.parametrize("world,count", [(1, 8192), (2, 8), (2, 8192), (4, 64 * 8192), (8, 16 * 8192),
                                         (8, 3 * 2048 + 264), (2, 64 * 8192 + 8), (3, 80 * 8192),
                                         (4, 40 * 8192), (8, 64 * 8192), (5, 33 * 8192 + 8), (7, 24 * 8192)])
def test_small_all_reduce_sums_in_rank_order(world, count):
    """`camblas_cuda_peer_allreduce_bf16` with emulated ranks: every rank's result is the FP32
    sum of the ranks' tensors in rank order, rounded once - bit for bit - and stays so over
    repeated calls (both line buffers come round again; the counted flag words of the larger
    sizes hand themselves back), in place as well. Counts up to 64 x 8192 take the
    flagged-line exchange (in one step, or with four ranks and more and enough data in two
    steps over slices, which must give the same bits), the last two cases the counted one. The phases
    of the ranks are issued in turn so that no kernel waits for an unlaunched one."""
    torch.manual_seed(705537 + world + count)
    capacity = PeerRegions.capacity_for(80, 8192)
    views = PeerRegions.emulate(capacity, world, 0)
    try:
        for call in range(5):
            inputs = [torch.randn(count, device="cuda").bfloat16() for _ in range(world)]
            total = torch.zeros(count, device="cuda")
            for tensor in inputs:
                total = total + tensor.float()
            expected = total.bfloat16()
            outputs = [tensor.clone() if call == 2 else torch.empty_like(tensor) for tensor in inputs]
            sources = outputs if call == 2 else inputs  # third call: in place
            for phase in (1, 2, 4):  # the third phase exists in the sliced form only
                for view, source, output in zip(views, sources, outputs):
                    view.all_reduce(source, out=output, phases=phase)
            torch.cuda.synchronize()
            assert _native.context(0).device_status() == 0
            for output in outputs:
                assert torch.equal(output, expected)
    finally:
        close_all(views)


def test_small_all_reduce_of_changing_sizes_never_takes_an_old_line_for_a_new_one():
    """Calls of different sizes share the chunks' call counters and line buffers: a long
    tensor (two steps over slices at this size), then short ones and a medium one (one step),
    then the long one again. Lines that a call did not touch still carry older call numbers,
    of either form, and must not pass for current ones."""
    world = 4
    torch.manual_seed(20261201)
    views = PeerRegions.emulate(PeerRegions.capacity_for(64, 8192), world, 0)
    try:
        for count in (48 * 8192, 8, 2048 + 8, 8, 48 * 8192, 4096, 32 * 8192, 48 * 8192):
            inputs = [torch.randn(count, device="cuda").bfloat16() for _ in range(world)]
            total = torch.zeros(count, device="cuda")
            for tensor in inputs:
                total = total + tensor.float()
            outputs = [torch.empty_like(tensor) for tensor in inputs]
            for phase in (1, 2, 4):  # the third phase exists in the sliced form only
                for view, source, output in zip(views, inputs, outputs):
                    view.all_reduce(source, out=output, phases=phase)
            torch.cuda.synchronize()
            assert _native.context(0).device_status() == 0
            for output in outputs:
                assert torch.equal(output, total.bfloat16())
    finally:
        close_all(views)


def test_small_all_reduce_whose_peer_never_sends_gives_up_and_reset_recovers():
    """Rank 0 of two emulated ranks receives without rank 1 having sent: the polls of the
    lines run out after the lowered limit, the kernel returns and the status word names the
    wait. The ranks' call counters now disagree, which camblas_cuda_peer_reset puts right."""
    world, count = 2, 4096
    torch.manual_seed(5)
    views = PeerRegions.emulate(PeerRegions.capacity_for(1, 8192), world, 0)
    native = _native.context(0)
    try:
        inputs = [torch.randn(count, device="cuda").bfloat16() for _ in range(world)]
        output = torch.empty_like(inputs[0])
        with _native.options(peer_wait_ms=50):
            views[0].all_reduce(inputs[0], out=output, phases=3)
            torch.cuda.synchronize()  # returns: the wait was bounded
            status = native.device_status()
        assert status & 15 == 6, hex(status)  # kRolePeerArrive
        for view in views:
            view.reset()
        torch.cuda.synchronize()
        outputs = [torch.empty_like(tensor) for tensor in inputs]
        for phase in (1, 2, 4):  # the third phase exists in the sliced form only
            for view, source, result in zip(views, inputs, outputs):
                view.all_reduce(source, out=result, phases=phase)
        torch.cuda.synchronize()
        assert native.device_status() == 0
        expected = (inputs[0].float() + inputs[1].float()).bfloat16()
        assert torch.equal(outputs[0], expected) and torch.equal(outputs[1], expected)
    finally:
        close_all(views)


def test_small_all_reduce_rejects_what_it_cannot_take():
    views = PeerRegions.emulate(PeerRegions.capacity_for(1, 8), 2, 0)
    try:
        with pytest.raises(ValueError):
            views[0].all_reduce(torch.zeros(12, device="cuda", dtype=torch.bfloat16))
        with pytest.raises(ValueError):
            views[0].all_reduce(torch.zeros(16, device="cuda"))
        with pytest.raises(ValueError):
            views[0].all_reduce(torch.zeros(256 * 256 + 8, device="cuda", dtype=torch.bfloat16))
    finally:
        close_all(views)
