"""Benchmark of the BF16 GEMM hot path on the Llama-3.1-70B-shaped prefill block.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (one "step"): M = 512 tokens, hidden 8192, BF16 storage, FP32
accumulation: fused residual-add + RMSNorm (eps 1e-5) -> packed QKV projection
8192 -> 10240 (64 query + 8 key + 8 value heads of 128) -> gate_up projection
8192 -> 57344 -> down projection 28672 -> 8192. Attention and SwiGLU are not
part of the path: the gate_up and down projections read seeded stand-in
activations of the right shape. Weights are N(0, 0.02), activations N(0, 1),
gamma N(1, 0.1), all seeded and synthetic.

With N > 1 GPUs the block is tensor parallel, one process per GPU: QKV and
gate_up are column parallel (weight rows split, no communication), down is row
parallel (inner dimension split, NCCL all-reduce of the BF16 partial results).
The work per step is fixed, so the scaling is "strong".

The printed value is algorithmic TFLOP/s (2*M*N*K per projection, summed) of
the whole job with inputs resident in HBM. `e2e` is the same metric through the
package's public calls with every step's activations copied from pinned host
memory and its result copied back inside the timed region (copies on their own
streams, double buffered, so they overlap the previous step's kernels). `roofline` covers
the two-SM tcgen05 GEMM kernel (plus its stream-K fix-up pass where one
runs), timed with CUDA events around each projection in the timed region. `cpu_baseline` is the reference's own CPU GEMM on the box's
host cores, on a bounded row slab of the same projections.
"""

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

TOKENS, HIDDEN, INTERMEDIATE = 512, 8192, 28672
Q_HEADS, KV_HEADS, HEAD = 64, 8, 128
QKV_OUT = (Q_HEADS + 2 * KV_HEADS) * HEAD  # 10240
GATE_UP_OUT = 2 * INTERMEDIATE  # 57344
FLOPS_PER_TOKEN = 2 * HIDDEN * (QKV_OUT + GATE_UP_OUT) + 2 * INTERMEDIATE * HIDDEN
FLOPS_PER_STEP = TOKENS * FLOPS_PER_TOKEN
METRIC = "bf16_gemm_tflops_llama70b_prefill_block_m512"
UNIT = "TFLOP/s"
WORKLOAD = "llama70b_prefill_block_m512_hidden8192_qkv10240_gateup57344_down28672"
# DRAM bytes per launch of the dominant kernel relative to its algorithmic bytes:
# dram__bytes_read.sum + dram__bytes_write.sum = 147.4 MB against 155.2 MB for the
# ncu capture of the M=512, N=16384, K=4096 case summarised in
# profiles/gemm_bf16_pair_m512_n16384_k4096.md. Every operand byte is fetched from
# HBM once, so the traffic of a launch scales with its algorithmic bytes.
TRAFFIC_RATIO = 0.95


def parse():
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=1000)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    return parser.parse_args()


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            return json.loads(path.read_text()), "measured"
        except ValueError:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Sample SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.process = None

    def start(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.process = None

    def stop(self):
        result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.process is None:
            return result
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        self.file.flush()
        self.file.seek(0)
        clocks, reasons, maximum = [], set(), None
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.file.read().splitlines():
            fields = [field.strip() for field in line.split(",")]
            if len(fields) < 9:
                continue
            try:
                clocks.append(float(fields[1]))
                maximum = float(fields[2])
            except ValueError:
                continue
            for name, field in zip(names, fields[5:9]):
                if field.lower() == "active":
                    reasons.add(name)
        os.unlink(self.file.name)
        if clocks:
            clocks.sort()
            # the upper half of the samples is the part taken under load
            loaded = clocks[len(clocks) // 2:]
            result.update(sm_mhz=loaded[len(loaded) // 2], sm_max_mhz=maximum,
                          reasons=sorted(reasons), samples=len(clocks))
        return result


def host_cpus():
    return sorted(os.sched_getaffinity(0))


class CpuSample:
    """The reference's CPU GEMM on a bounded slab of the three projections.

    Uses the reference's own library (oracle/_ref, compiled from the reference
    sources) with its pinned pthread pool on every allowed core; falls back to
    the single-threaded C restatement when that library is absent. The slab is
    `rows` token rows by 1/16 of the output features of each projection with
    the full inner dimension; the portable kernel's cost is linear in both.
    """

    FRACTION = 16

    def __init__(self):
        import numpy as np
        from oracle import oracle

        self.np, self.oracle = np, oracle
        self.rng = np.random.default_rng(705540)
        shapes = [(QKV_OUT, HIDDEN), (GATE_UP_OUT, HIDDEN), (HIDDEN, INTERMEDIATE)]
        self.pool, self.kind, self.cores = None, "port", 1
        if oracle.reference_lib() is not None:
            self.kind = "reference"
            try:
                self.pool = oracle.ReferencePool(host_cpus())
                self.cores = len(self.pool.cpus)
            except RuntimeError:
                self.pool = None
        self.weights = [(self.rng.standard_normal((n // self.FRACTION, k)) * 0.02).astype(np.float32)
                        for n, k in shapes]
        self.flops_per_row = sum(2 * w.shape[0] * w.shape[1] for w in self.weights)
        self.inputs = {}
        self.rate = self.flops_per_row / self.run(1)  # calibration, FLOP/s

    def run(self, rows):
        """Multiply `rows` token rows through the three slabs; return seconds."""
        if rows not in self.inputs:
            self.inputs = {rows: [self.rng.standard_normal((rows, w.shape[1])).astype(self.np.float32)
                                  for w in self.weights]}
        start = time.perf_counter()
        for x, w in zip(self.inputs[rows], self.weights):
            if self.pool is not None:
                self.pool.linear_f32(x, w)
            else:
                self.oracle.reference_linear_f32(x, w)
        return time.perf_counter() - start

    def rows_for(self, seconds):
        return int(max(1, min(TOKENS, seconds * self.rate / self.flops_per_row)))

    def describe(self, rows, seconds):
        return (f"{rows} token rows x 1/{self.FRACTION} of the output features of the QKV, gate_up "
                f"and down projections (full K), FP32, {rows * self.flops_per_row / 1e9:.1f} GFLOP "
                f"in {seconds:.2f} s")

    def close(self):
        if self.pool is not None:
            self.pool.close()


def run_reference(args):
    """The reference arm: the reference's own CPU GEMM on bounded samples of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    sample = CpuSample()
    per_step = min(20.0, 150.0 / (steps + warmup))
    if "CAMBLAS_BENCH_STEP_SECONDS" in os.environ:  # tests shorten the sample
        per_step = float(os.environ["CAMBLAS_BENCH_STEP_SECONDS"])
    rows = sample.rows_for(per_step)
    passes = 1
    if rows == TOKENS:  # the whole slab is quicker than the step budget: repeat it
        passes = int(max(1, min(64, per_step / max(1e-3, sample.run(rows)))))

    def one_step():
        return sum(sample.run(rows) for _ in range(passes))

    for _ in range(warmup):
        one_step()
    seconds = [one_step() for _ in range(steps)]
    mean = sum(seconds) / len(seconds)
    value = passes * rows * sample.flops_per_row / mean / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": 1e3 * mean,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": WORKLOAD, "arm": "reference CPU GEMM"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": sample.cores, "kind": sample.kind,
                         "sample": f"{passes} passes per step of: " + sample.describe(rows, mean / passes)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    sample.close()
    print(json.dumps(line), flush=True)


class Block:
    """Weights and activations of one prefill block on one rank (tensor parallel)."""

    def __init__(self, torch, rank, world, device):
        from camblas_b200 import tp

        self.torch = torch
        self.world = world
        generator = torch.Generator(device="cpu").manual_seed(705537 + 2)

        def normal(shape, scale=1.0, mean=0.0):
            return (torch.randn(shape, generator=generator) * scale + mean).to(torch.bfloat16)

        # every rank draws the same full tensors and keeps its shard
        self.x = normal((TOKENS, HIDDEN)).to(device)
        self.residual = normal((TOKENS, HIDDEN)).to(device)
        self.gamma = normal((HIDDEN,), 0.1, 1.0).to(device)
        qkv = normal((QKV_OUT, HIDDEN), 0.02)
        self.qkv_weight, self.qkv_widths = tp.shard_qkv(qkv, Q_HEADS, KV_HEADS, HEAD, rank, world)
        self.qkv_weight = self.qkv_weight.to(device)
        del qkv
        gate_up = normal((GATE_UP_OUT, HIDDEN), 0.02)
        start, stop = tp.shard_bounds(GATE_UP_OUT, rank, world, 128)
        self.gate_up_weight = gate_up[start:stop].contiguous().to(device)
        del gate_up
        down = normal((HIDDEN, INTERMEDIATE), 0.02)
        start, stop = tp.shard_bounds(INTERMEDIATE, rank, world, 128)
        self.down_weight = down[:, start:stop].contiguous().to(device)
        del down
        self.mlp_input = normal((TOKENS, HIDDEN)).to(device)
        self.down_input = normal((TOKENS, INTERMEDIATE))[:, start:stop].contiguous().to(device)
        self.gemm_flops = [2 * TOKENS * HIDDEN * self.qkv_weight.shape[0],
                           2 * TOKENS * HIDDEN * self.gate_up_weight.shape[0],
                           2 * TOKENS * self.down_weight.shape[1] * HIDDEN]
        self.gemm_bytes = [2 * (w.numel() + TOKENS * w.shape[1] + TOKENS * w.shape[0])
                           for w in (self.qkv_weight, self.gate_up_weight, self.down_weight)]
        self.launches_per_step = 4
        self.peers, self.exchange = None, None
        if world > 1:
            self.exchange = self.choose_exchange(rank, world, device)

    def choose_exchange(self, rank, world, device):
        """Pick how the down projection's partial sums meet; returns its description.

        Default: the product kernel pushes its tiles through peer memory
        (`camblas_cuda_linear_bf16_allreduce`). All ranks check one step of it
        against the NCCL all-reduce of the same partial products and fall back to
        NCCL together if the regions cannot be set up or the check fails;
        CAMBLAS_B200_BENCH_EXCHANGE=nccl forces the NCCL path.
        """
        import torch.distributed as dist
        from camblas_b200 import _kernels, _native, tp

        torch = self.torch
        nccl = "NCCL sum of BF16 partials after the down projection"
        if os.environ.get("CAMBLAS_B200_BENCH_EXCHANGE", "peer") == "nccl":
            return nccl + " (forced)"
        try:
            peers = tp.PeerRegions.create(tp.PeerRegions.capacity_for(TOKENS, HIDDEN), device.index)
        except RuntimeError as error:
            return nccl + f" (peer regions unavailable: {error})"
        reason = None
        try:
            fused = peers.linear(self.down_input, self.down_weight).float()
            expected = _kernels.linear(self.down_input, self.down_weight)
            dist.all_reduce(expected, op=dist.ReduceOp.SUM)
            torch.cuda.synchronize()
            if _native.context(device.index).device_status() != 0:
                reason = "a bounded wait expired"
            else:
                error = ((fused - expected.float()).norm() / expected.float().norm()).item()
                if not error <= 2e-2:
                    reason = f"rel-L2 {error:.2e} against the NCCL path"
        except RuntimeError as error:
            reason = str(error)
        reasons = [None] * world
        dist.all_gather_object(reasons, reason)
        if any(reasons):
            peers.close()
            return nccl + " (peer path rejected: " + next(text for text in reasons if text) + ")"
        self.peers = peers
        return ("product epilogue writes BF16 partial tiles into the owner GPU's memory over NVLink; "
                "owner sums in rank order and writes the result to every GPU")

    def step(self, x, residual, events=None):
        """One pass of the block; returns the down-projection output."""
        from camblas_b200 import _kernels
        import torch.distributed as dist

        torch = self.torch
        _, normed = _kernels.add_rms_norm(x, residual, self.gamma, 1e-5)

        def timed(index, function):
            if events is None:
                return function()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            result = function()
            end.record()
            events.append((index, begin, end))
            return result

        timed(0, lambda: _kernels.qkv_linear(normed, self.qkv_weight, *self.qkv_widths))
        timed(1, lambda: _kernels.linear(self.mlp_input, self.gate_up_weight))
        if self.peers is not None:
            return timed(2, lambda: self.peers.linear(self.down_input, self.down_weight))
        out = timed(2, lambda: _kernels.linear(self.down_input, self.down_weight))
        if self.world > 1:
            dist.all_reduce(out, op=dist.ReduceOp.SUM)
        return out


def run_ours(args):
    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the kernels have no CPU route")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != max(1, args.gpus):
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    from camblas_b200 import _native

    block = Block(torch, rank, world, device)
    steps, warmup = max(1, args.steps), max(3, args.warmup)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        block.step(block.x, block.residual)
    barrier()

    # ---- device-resident timing ----
    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(local).uuid))
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    events = []
    barrier()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(steps):
        block.step(block.x, block.residual, events)
    end.record()
    barrier()
    elapsed_ms = begin.elapsed_time(end)
    clocks = sampler.stop() if rank == 0 else None
    status = _native.context(local).device_status()
    if status != 0:
        raise SystemExit(f"a pipelined kernel reported status {status:#x}")

    def capture(input_sets):
        """Capture one step per input set into CUDA graphs; None if that is not possible.

        The reference's surface supports capture after a warm-up on the stream. Replaying
        the block matters at eight ranks, where a step is 0.18 ms of GPU work and issuing
        its kernels from Python takes about as long. Not used with the NCCL exchange (a
        collective inside the captured region); any failure falls back, on all ranks
        together, to issuing the kernels one by one.
        """
        graphs = None
        if world == 1 or block.peers is not None:
            try:
                capture_stream = torch.cuda.Stream()
                capture_stream.wait_stream(torch.cuda.current_stream())
                graphs = []
                with torch.cuda.stream(capture_stream):
                    for inputs in input_sets:
                        block.step(*inputs)  # creates this stream's native context and scratch
                    capture_stream.synchronize()
                    if world > 1:
                        dist.barrier()
                    for inputs in input_sets:
                        graph = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(graph, stream=capture_stream):
                            result = block.step(*inputs)
                            if block.peers is not None:
                                result = result.clone()  # the peer region is reused by the next step
                        graphs.append((graph, result))
                capture_stream.synchronize()
            except Exception as error:  # noqa: BLE001 - any capture problem means: no graphs
                if rank == 0:
                    print(f"bench: CUDA-graph capture of the step failed ({error}); "
                          "issuing kernels directly", file=sys.stderr, flush=True)
                graphs = None
                torch.cuda.synchronize()
        if world > 1:
            flags = [None] * world
            dist.all_gather_object(flags, graphs is not None)
            if not all(flags):
                graphs = None
        return graphs

    # ---- the same steps without per-launch events (the headline device number) ----
    resident = capture([(block.x, block.residual)])
    barrier()
    begin.record()
    for _ in range(steps):
        if resident is not None:
            resident[0][0].replay()
        else:
            block.step(block.x, block.residual)
    end.record()
    barrier()
    plain_ms = begin.elapsed_time(end)

    # ---- end to end: pinned host activations in, result out, every step ----
    # Every step copies its own x and residual from pinned host memory and copies its
    # result back; the copies run on their own streams with two buffer sets, so the
    # transfer of step i+1 overlaps the kernels of step i (a serving loop would do
    # the same). The timed region ends when the last result has reached the host.
    # With N ranks every rank needs the whole activations, but only 1/N of them crosses
    # its own host link: rank r uploads its block of token rows and the ranks exchange the
    # blocks over NVLink (NCCL all-gather on the upload stream); likewise rank r downloads
    # only its block of the (replicated) result. Whole-job bytes per step stay the same.
    host_x = block.x.cpu().pin_memory()
    host_residual = block.residual.cpu().pin_memory()
    host_out = [torch.empty((TOKENS, HIDDEN), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    device_in = [(torch.empty_like(block.x), torch.empty_like(block.residual)) for _ in range(2)]
    # its own communicator, so that the all-gather does not queue behind the step's collectives
    transfer_group = dist.new_group() if world > 1 else None
    share = TOKENS // world if TOKENS % world == 0 else TOKENS
    mine = slice(rank * share, (rank + 1) * share) if share != TOKENS else slice(0, TOKENS)
    compute = torch.cuda.current_stream()
    upload, download = torch.cuda.Stream(), torch.cuda.Stream()
    e2e_steps = min(steps, 200)

    replay = capture(device_in)

    def pipeline(count):
        loaded = [torch.cuda.Event() for _ in range(2)]
        consumed = [torch.cuda.Event() for _ in range(2)]
        stored = [torch.cuda.Event() for _ in range(2)]
        upload.wait_stream(compute)
        download.wait_stream(compute)
        for index in range(count):
            slot = index & 1
            with torch.cuda.stream(upload):
                if index >= 2:
                    upload.wait_event(consumed[slot])
                for target, source in zip(device_in[slot], (host_x, host_residual)):
                    target[mine].copy_(source[mine], non_blocking=True)
                    if share != TOKENS:
                        dist.all_gather_into_tensor(target, target[mine], group=transfer_group)
                loaded[slot].record(upload)
            compute.wait_event(loaded[slot])
            if replay is not None:
                if index >= 2:
                    compute.wait_event(stored[slot])  # the graph writes the result it read from
                replay[slot][0].replay()
                out = replay[slot][1]
            else:
                out = block.step(*device_in[slot])
                if block.peers is not None:
                    out = out.clone()  # the peer region is overwritten by the next step
            consumed[slot].record(compute)
            with torch.cuda.stream(download):
                download.wait_event(consumed[slot])
                if index >= 2:
                    download.wait_event(stored[slot])
                host_out[slot][mine].copy_(out[mine], non_blocking=True)
                if replay is None:
                    out.record_stream(download)
                stored[slot].record(download)
        compute.wait_stream(download)

    pipeline(4)
    barrier()
    begin.record()
    pipeline(e2e_steps)
    end.record()
    barrier()
    e2e_ms = begin.elapsed_time(end)

    def across_ranks(value):
        if world == 1:
            return value
        tensor = torch.tensor([value], dtype=torch.float64, device=device)
        dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
        return float(tensor.item())

    launches_before = _native.context(local).kernel_launches()
    block.step(block.x, block.residual)
    launches_per_step = _native.context(local).kernel_launches() - launches_before
    torch.cuda.synchronize()
    plain_ms = across_ranks(plain_ms)
    e2e_ms = across_ranks(e2e_ms)

    gemm_ms = [0.0, 0.0, 0.0]
    for index, first, second in events:
        gemm_ms[index] += first.elapsed_time(second)
    if rank == 0:
        peaks, peak_source = measured_peaks()
        sustained = plain_ms >= 1000.0
        peak = peaks["bf16_tflops_sustained" if sustained else "bf16_tflops"]
        flops = sum(block.gemm_flops) * steps
        achieved = flops / (sum(gemm_ms) * 1e-3) / 1e12
        launch_bytes = sum(block.gemm_bytes) / 3
        line = {
            "metric": METRIC,
            "value": FLOPS_PER_STEP * steps / (plain_ms * 1e-3) / 1e12,
            "unit": UNIT,
            "n_gpus": world,
            "steps": steps,
            "warmup": warmup,
            "ms_per_step": plain_ms / steps,
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic",
            "config": {
                "workload": WORKLOAD,
                "tokens": TOKENS,
                "parallelism": f"tp{world}" if world > 1 else "single",
                "l2": "weights of one step (1.58 GB per GPU at tp1) exceed the 126 MB L2; no flush",
                "all_reduce": block.exchange,
                "issue": ("step replayed from a CUDA graph" if resident is not None
                          else "kernels issued one by one"),
            },
            "roofline": {
                "bound": "tensor",
                "kernel": "sm100::gemm_bf16_pair (two-SM tcgen05 tiles)",
                "achieved": achieved,
                "peak": peak,
                "unit": "TFLOP/s",
                "frac": achieved / peak,
                "peak_source": f"{peak_source} cuBLAS bf16, {'sustained' if sustained else 'burst'}",
                "traffic": launch_bytes * TRAFFIC_RATIO if TRAFFIC_RATIO else None,
                "algorithmic_bytes_per_launch": launch_bytes,
                "per_projection_tflops": [f / (m * 1e-3 / steps) / 1e12 if m else None
                                          for f, m in zip(block.gemm_flops, gemm_ms)],
            },
            "e2e": {
                "value": FLOPS_PER_STEP * e2e_steps / (e2e_ms * 1e-3) / 1e12,
                "unit": UNIT,
                "h2d_bytes_per_step": 2 * TOKENS * HIDDEN * 2,
                "d2h_bytes_per_step": TOKENS * HIDDEN * 2,
                "steps": e2e_steps,
            },
            "gpu_launches": launches_per_step * steps,
            "clocks": clocks,
        }
        if world == 1:
            sample = CpuSample()
            rows = sample.rows_for(12.0)
            seconds, passes = sample.run(rows), 1
            while seconds < 10.0 and passes < 64:  # repeat the slab up to about 10 s of CPU work
                seconds += sample.run(rows)
                passes += 1
            line["cpu_baseline"] = {"value": passes * rows * sample.flops_per_row / seconds / 1e12,
                                    "unit": UNIT, "cores": sample.cores, "kind": sample.kind,
                                    "sample": f"{passes} passes of: " + sample.describe(rows, seconds / passes)}
            sample.close()
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        if block.peers is not None:
            block.peers.close(free=False)  # unmap the others' regions before anyone frees
            dist.barrier()
            block.peers.close(free=True)
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
