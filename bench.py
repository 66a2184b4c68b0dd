"""Benchmark of the BF16 GEMM hot path on the Llama-3.1-70B-shaped prefill block.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Other measurements of the same library, each printing JSON rows (not the
headline line) and taking `--json FILE` to keep them:

    python bench.py --table 1,2,3,4,5,6,7   one kernel at a time over the benchmark's
                                            configurations on one GPU (7 = the RMS and
                                            elementwise kernels), with torch/cuBLAS and,
                                            when oracle/_ref holds it, the reference's
                                            own CUDA library as comparator rows
    python bench.py --workload decode_tp    the decode sweep M = 1..64 on the down and
                                            gate_up projections, sharded over the ranks
                                            it is launched with (row / column parallel)
    python bench.py --workload square_tp    the large squares, column-sharded likewise
    python bench.py --single bf16,M,N,K     one product a few times, for a profiler

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
    parser.add_argument("--workload", choices=("block", "decode_tp", "square_tp"), default="block")
    parser.add_argument("--table", default=None, metavar="LIST",
                        help="kernel-level table over configurations, e.g. 1,2,3,4,5,6,7")
    parser.add_argument("--single", default=None, metavar="KIND,M,N,K",
                        help="run one product a few times eagerly (for a profiler): bf16, fp8 or rms")
    parser.add_argument("--json", default=None, help="also write the rows of a table or sweep here")
    parser.add_argument("--sustain", type=float, default=3.0,
                        help="seconds of the sustained-clock loop after the timed steps (0 = skip)")
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


def distributed_setup(args):
    """Join the process group the launcher describes; returns (torch, dist, rank, world, device)."""
    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the kernels have no CPU route")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    return torch, dist, rank, world, device


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
        self.peers, self.exchange = None, None
        if world > 1:
            self.exchange = self.choose_exchange(rank, world, device)

    def choose_exchange(self, rank, world, device):
        """Pick how the down projection's partial sums meet; returns its description.

        Default: the product kernel pushes its tiles through peer memory
        (`camblas_cuda_linear_bf16_allreduce`). All ranks check one step of it
        against the NCCL all-reduce of the same partial products (rel-L2 <= 1e-2,
        the BF16 bound) and fall back to NCCL together if the regions cannot be
        set up or the check fails; CAMBLAS_B200_BENCH_EXCHANGE=nccl forces NCCL.
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
                if not error <= 1e-2:
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

    def projection(self, index, normed=None):
        """Launch projection `index` (0 QKV, 1 gate_up, 2 down with its exchange)."""
        from camblas_b200 import _kernels
        import torch.distributed as dist

        if index == 0:
            return _kernels.qkv_linear(self.x if normed is None else normed, self.qkv_weight,
                                       *self.qkv_widths)
        if index == 1:
            return _kernels.linear(self.mlp_input, self.gate_up_weight)
        if self.peers is not None:
            return self.peers.linear(self.down_input, self.down_weight)
        out = _kernels.linear(self.down_input, self.down_weight)
        if self.world > 1:
            dist.all_reduce(out, op=dist.ReduceOp.SUM)
        return out

    def step(self, x, residual):
        """One pass of the block; returns the down-projection output."""
        from camblas_b200 import _kernels

        _, normed = _kernels.add_rms_norm(x, residual, self.gamma, 1e-5)
        self.projection(0, normed)
        self.projection(1)
        return self.projection(2)


def across_ranks(torch, dist, world, device, value):
    """Maximum of a host number over the ranks."""
    if world == 1:
        return value
    tensor = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
    return float(tensor.item())


def run_ours(args):
    torch, dist, rank, world, device = distributed_setup(args)
    local = device.index
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
    status = _native.context(local).device_status()
    if status != 0:
        raise SystemExit(f"a pipelined kernel reported status {status:#x}")

    def capture(bodies):
        """Capture each callable of `bodies` into a CUDA graph; None if that is not possible.

        The reference's surface supports capture after a warm-up on the stream. Replaying
        the block matters at eight ranks, where a step is 0.17 ms of GPU work and issuing
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
                    for body in bodies:
                        body()  # creates this stream's native context and scratch
                    capture_stream.synchronize()
                    if world > 1:
                        dist.barrier()
                    for body in bodies:
                        graph = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(graph, stream=capture_stream):
                            result = body()
                        graphs.append((graph, result))
                capture_stream.synchronize()
            except Exception as error:  # noqa: BLE001 - any capture problem means: no graphs
                if rank == 0:
                    print(f"bench: CUDA-graph capture failed ({error}); issuing kernels directly",
                          file=sys.stderr, flush=True)
                graphs = None
                torch.cuda.synchronize()
        if world > 1:
            flags = [None] * world
            dist.all_gather_object(flags, graphs is not None)
            if not all(flags):
                graphs = None
        return graphs

    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    # ---- the dominant kernel on its own: each projection ten times per graph ----
    # These durations give roofline.achieved; they contain no launch gaps because the
    # launches of a graph follow one another on the device.
    per_graph = 10
    projections = capture([(lambda index=index: [block.projection(index) for _ in range(per_graph)][-1])
                           for index in range(3)])
    gemm_ms = [0.0, 0.0, 0.0]
    gemm_launches = per_graph * max(1, -(-steps // per_graph))
    for index in range(3):
        barrier()
        begin.record()
        for _ in range(gemm_launches // per_graph):
            if projections is not None:
                projections[index][0].replay()
            else:
                for _ in range(per_graph):
                    block.projection(index)
        end.record()
        barrier()
        gemm_ms[index] = across_ranks(torch, dist, world, device, begin.elapsed_time(end))
    del projections

    # ---- device-resident timing of the whole step (the headline value) ----
    def resident_step():
        result = block.step(block.x, block.residual)
        return result.clone() if block.peers is not None else result

    resident = capture([resident_step])
    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(local).uuid))
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    begin.record()
    for _ in range(steps):
        if resident is not None:
            resident[0][0].replay()
        else:
            block.step(block.x, block.residual)
    end.record()
    barrier()
    plain_ms = across_ranks(torch, dist, world, device, begin.elapsed_time(end))
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end: pinned host activations in, result out, every step ----
    # Every step copies its own x and residual from pinned host memory and copies its
    # result back; the copies run on their own streams with two buffer sets, so the
    # transfer of step i+1 overlaps the kernels of step i (a serving loop would do the
    # same). The timed region ends when the last result has reached the host. x and
    # residual travel as ONE buffer [tokens, 2, hidden] (row t holds x[t] then
    # residual[t]) and are normalised where they lie. With N ranks every rank needs the
    # whole activations, but only 1/N of them crosses its own host link: rank r uploads
    # its block of token rows in one copy and the ranks exchange the blocks over NVLink
    # in one NCCL all-gather on the upload stream; likewise rank r downloads only its
    # block of the (replicated) result. Whole-job bytes per step stay the same.
    host_in = torch.empty((TOKENS, 2, HIDDEN), dtype=torch.bfloat16).pin_memory()
    host_in[:, 0].copy_(block.x)
    host_in[:, 1].copy_(block.residual)
    host_out = [torch.empty((TOKENS, HIDDEN), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    device_in = [torch.empty((TOKENS, 2, HIDDEN), dtype=torch.bfloat16, device=device) for _ in range(2)]
    # its own communicator, so that the all-gather does not queue behind the step's collectives
    transfer_group = dist.new_group() if world > 1 else None
    share = TOKENS // world if TOKENS % world == 0 else TOKENS
    mine = slice(rank * share, (rank + 1) * share) if share != TOKENS else slice(0, TOKENS)
    compute = torch.cuda.current_stream()
    upload, download = torch.cuda.Stream(), torch.cuda.Stream()
    e2e_steps = min(steps, 200)

    def e2e_step(slot):
        result = block.step(device_in[slot][:, 0], device_in[slot][:, 1])
        return result.clone() if block.peers is not None else result

    replay = capture([lambda: e2e_step(0), lambda: e2e_step(1)])

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
                device_in[slot][mine].copy_(host_in[mine], non_blocking=True)
                if share != TOKENS:
                    dist.all_gather_into_tensor(device_in[slot], device_in[slot][mine],
                                                group=transfer_group)
                loaded[slot].record(upload)
            compute.wait_event(loaded[slot])
            if replay is not None:
                if index >= 2:
                    compute.wait_event(stored[slot])  # the graph writes the result it read from
                replay[slot][0].replay()
                out = replay[slot][1]
            else:
                out = e2e_step(slot)
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
    e2e_ms = across_ranks(torch, dist, world, device, begin.elapsed_time(end))
    expected_out = block.step(block.x, block.residual)
    torch.cuda.synchronize()
    e2e_matches = bool(torch.equal(host_out[(e2e_steps - 1) & 1][mine], expected_out[mine].cpu()))

    # ---- the same step for at least `--sustain` seconds: the clock under sustained load ----
    # (last of the measurements, so that the end-to-end leg above is not taken on a GPU
    # that three seconds of full load have just driven into its power cap)
    sustained = None
    if args.sustain > 0:
        count = int(max(steps, min(200000, args.sustain * 1e3 / max(1e-3, plain_ms / steps))))
        sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(local).uuid))
        if rank == 0:
            sampler.start()
        barrier()
        begin.record()
        for _ in range(count):
            if resident is not None:
                resident[0][0].replay()
            else:
                block.step(block.x, block.residual)
        end.record()
        barrier()
        sustained_ms = across_ranks(torch, dist, world, device, begin.elapsed_time(end))
        sustained = {"steps": count, "seconds": sustained_ms * 1e-3,
                     "value": FLOPS_PER_STEP * count / (sustained_ms * 1e-3) / 1e12,
                     "clocks": sampler.stop() if rank == 0 else None}


    launches_before = _native.context(local).kernel_launches()
    block.step(block.x, block.residual)
    launches_per_step = _native.context(local).kernel_launches() - launches_before
    torch.cuda.synchronize()
    status = _native.context(local).device_status()
    if status != 0:
        raise SystemExit(f"a pipelined kernel reported status {status:#x}")

    if rank == 0:
        peaks, peak_source = measured_peaks()
        long_region = plain_ms >= 1000.0
        peak = peaks["bf16_tflops_sustained" if long_region else "bf16_tflops"]
        achieved = sum(block.gemm_flops) * gemm_launches / (sum(gemm_ms) * 1e-3) / 1e12
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
                "peak_source": f"{peak_source} cuBLAS bf16, {'sustained' if long_region else 'burst'}",
                "traffic": launch_bytes * TRAFFIC_RATIO if TRAFFIC_RATIO else None,
                "algorithmic_bytes_per_launch": launch_bytes,
                "timing": (f"{gemm_launches} launches per projection, {per_graph} per replayed graph, "
                           "CUDA events on the launching stream"),
                "per_projection_tflops": [f / (m * 1e-3 / gemm_launches) / 1e12 if m else None
                                          for f, m in zip(block.gemm_flops, gemm_ms)],
            },
            "e2e": {
                "value": FLOPS_PER_STEP * e2e_steps / (e2e_ms * 1e-3) / 1e12,
                "unit": UNIT,
                "h2d_bytes_per_step": 2 * TOKENS * HIDDEN * 2,
                "d2h_bytes_per_step": TOKENS * HIDDEN * 2,
                "steps": e2e_steps,
                "result_equals_resident_step": e2e_matches,
            },
            "gpu_launches": launches_per_step * steps,
            "clocks": clocks,
        }
        if sustained is not None:
            sustained["frac_of_sustained_peak"] = sustained["value"] / (
                world * peaks["bf16_tflops_sustained"])
            line["sustained"] = sustained
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
    shutdown(torch, dist, world, block.peers)


def shutdown(torch, dist, world, peers=None):
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        if peers is not None:
            peers.close(free=False)  # unmap the others' regions before anyone frees
            dist.barrier()
            peers.close(free=True)
        dist.barrier()
        dist.destroy_process_group()


# ---- kernel-level measurements ------------------------------------------------------
#
# One kernel at a time, the way the reference's bench/cuda_workload.py times single
# operations (warm-ups, repeated timed runs, CUDA events, :352-399). Timing is taken
# inside a replayed CUDA graph of many launches so that microsecond kernels are not
# hidden behind host launch cost; HBM-bound cases rotate through enough distinct
# copies of the weight to exceed the 126 MB L2 ("cold") and are also reported
# re-reading one copy ("warm"). The FP8 tensor peak is taken as twice the BF16 figure.

L2_BYTES = 126 * 2**20


class Rows:
    """Collects and prints the rows of a table or sweep (rank 0 prints)."""

    def __init__(self, rank=0):
        peaks, source = measured_peaks()
        self.peaks = {"hbm": peaks["hbm_gbs"], "bf16": peaks["bf16_tflops"], "source": source}
        self.rank, self.rows = rank, []

    def add(self, name, microseconds, flops=None, nbytes=None, bound="hbm", note="", **extra):
        entry = {"case": name, "us": round(microseconds, 2), "bound": bound, "note": note}
        if flops is not None:
            entry["tflops"] = round(flops / microseconds / 1e6, 1)
        if nbytes is not None:
            entry["gbs"] = round(nbytes / microseconds / 1e3, 1)
        if bound == "hbm":
            entry["frac"] = round(entry["gbs"] / self.peaks["hbm"], 3)
        elif bound == "tensor_bf16":
            entry["frac"] = round(entry["tflops"] / self.peaks["bf16"], 3)
        elif bound == "tensor_fp8":
            entry["frac"] = round(entry["tflops"] / (2 * self.peaks["bf16"]), 3)
        entry.update(extra)
        self.rows.append(entry)
        if self.rank == 0:
            print(json.dumps(entry), flush=True)
        return entry

    def save(self, path):
        if path and self.rank == 0:
            Path(path).write_text(json.dumps({"peaks": self.peaks, "rows": self.rows}, indent=1))


def graph_time_us(call, variants, launches=20, replays=7, collective=None):
    """Median microseconds per launch of ``call(i)`` inside a replayed CUDA graph.

    ``call(i)`` must launch the operation on variant ``i % variants``. The
    warm-up runs on the capture stream first, because a native context belongs
    to one stream and cannot be created during capture. ``collective`` is
    ``(dist, world, device)`` when the ranks of a group time the same thing: they
    meet at a barrier before every replay and the maximum over ranks is returned.
    """
    import statistics
    import torch
    from camblas_b200 import _native

    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.inference_mode(), torch.cuda.stream(stream):
        for i in range(max(variants, 2)):
            call(i)
        stream.synchronize()
        if collective is not None:
            collective[0].barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(launches):
                call(i)
        for _ in range(2):
            graph.replay()
        stream.synchronize()
        times = []
        for _ in range(replays):
            if collective is not None:
                collective[0].barrier()
                torch.cuda.synchronize()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record(stream)
            graph.replay()
            end.record(stream)
            stream.synchronize()
            times.append(begin.elapsed_time(end) * 1e3 / launches)
    status = _native.context(torch.cuda.current_device()).device_status()
    if status:
        raise RuntimeError(f"kernel reported status {status:#x}")
    graph.reset()
    value = statistics.median(times)
    if collective is not None:
        dist, world, device = collective
        value = across_ranks(torch, dist, world, device, value)
    return value


def copies_for_cold(nbytes):
    return max(1, min(64, -(-2 * L2_BYTES // nbytes)))


class ReferenceCuda:
    """The reference's own CUDA library (oracle/_ref, built by oracle/Makefile) as a
    comparator for the BF16 GEMM rows: its classical route (cublasGemmEx,
    src/cuda/bfloat16.cuh:37-56) and its `lt` route (cublasLtMatmul plan cache,
    backend.cu:559-784). Measurement only; None when the library is absent."""

    PATH = ROOT / "oracle" / "_ref" / "libcamblas_cuda_ref.so"

    @classmethod
    def load(cls):
        import ctypes as ct

        if not cls.PATH.is_file():
            return None
        try:
            return cls(ct.CDLL(str(cls.PATH)))
        except OSError:
            return None

    def __init__(self, library):
        import ctypes as ct

        self.ct, self.lib, self.contexts = ct, library, {}
        p, i, f = ct.c_void_p, ct.c_int, ct.c_float
        library.camblas_cuda_create.argtypes = [i, p, ct.POINTER(p)]
        library.camblas_cuda_set_algorithm.argtypes = [p, i]
        library.camblas_cuda_bgemm.argtypes = [p, ct.c_char, ct.c_char, i, i, i, f, p, i, p, i, f, p, i]
        library.camblas_cuda_error.restype = ct.c_char_p
        library.camblas_cuda_error.argtypes = [p]

    def linear(self, x, weight, out, policy):
        """out[rows, outputs] = x @ weight.T through the reference's camblas_cuda_bgemm."""
        import torch

        ct = self.ct
        stream = torch.cuda.current_stream().cuda_stream
        context = self.contexts.get(stream)
        if context is None:
            context = ct.c_void_p()
            if self.lib.camblas_cuda_create(torch.cuda.current_device(), ct.c_void_p(stream),
                                            ct.byref(context)) != 0:
                raise RuntimeError(self.lib.camblas_cuda_error(None).decode())
            self.contexts[stream] = context
        self.lib.camblas_cuda_set_algorithm(context, policy)
        rows, inner = x.shape
        outputs = weight.shape[0]
        status = self.lib.camblas_cuda_bgemm(context, b"T", b"N", outputs, rows, inner, 1.0,
                                             ct.c_void_p(weight.data_ptr()), inner,
                                             ct.c_void_p(x.data_ptr()), inner, 0.0,
                                             ct.c_void_p(out.data_ptr()), outputs)
        if status != 0:
            raise RuntimeError(self.lib.camblas_cuda_error(context).decode())
        return out


def bf16_weight(outputs, inner, scale, copies):
    import torch

    return [(torch.randn(outputs, inner, device="cuda") * scale).bfloat16() for _ in range(copies)]


def linear_case(rows_out, name, tokens, outputs, inner, scale=0.02, bound=None, comparators=True):
    import torch
    from camblas_b200 import _kernels

    nbytes = 2 * (outputs * inner + tokens * inner + tokens * outputs)
    flops = 2 * tokens * outputs * inner
    if bound is None:
        bound = "hbm" if tokens <= 64 else "tensor_bf16"
    x = torch.randn(tokens, inner, device="cuda").bfloat16()
    reference = ReferenceCuda.load() if comparators else None
    for label, copies in (("cold", copies_for_cold(nbytes)), ("warm", 1)):
        if label == "warm" and (bound != "hbm" or nbytes > L2_BYTES):
            continue
        weights = bf16_weight(outputs, inner, scale, copies)
        mine = graph_time_us(lambda i: _kernels.linear(x, weights[i % copies]), copies)
        rows_out.add(f"{name} [{label}]", mine, flops, nbytes, bound)
        if comparators:
            theirs = graph_time_us(lambda i: torch.nn.functional.linear(x, weights[i % copies]), copies)
            rows_out.add(f"{name} [{label}] torch/cuBLAS", theirs, flops, nbytes, bound, "comparator")
        if reference is not None:
            out = torch.empty((tokens, outputs), dtype=torch.bfloat16, device="cuda")
            for policy, route in ((1, "cublasGemmEx"), (3, "cublasLt")):
                try:
                    theirs = graph_time_us(
                        lambda i: reference.linear(x, weights[i % copies], out, policy), copies)
                    rows_out.add(f"{name} [{label}] reference library, {route}", theirs, flops,
                                 nbytes, bound, "comparator")
                except RuntimeError as error:
                    rows_out.add(f"{name} [{label}] reference library, {route}", float("nan"),
                                 note=f"failed: {error}", bound="none")
        del weights


def table_config1(rows_out):
    linear_case(rows_out, "C1 decode 1x2048 -> 4096", 1, 4096, 2048, scale=1.0)


def table_config2(rows_out):
    import torch
    from camblas_b200 import _kernels

    tokens, hidden = 512, 8192
    x = torch.randn(tokens, hidden, device="cuda").bfloat16()
    residual = torch.randn(tokens, hidden, device="cuda").bfloat16()
    gamma = (1 + 0.1 * torch.randn(hidden, device="cuda")).bfloat16()
    microseconds = graph_time_us(lambda i: _kernels.add_rms_norm(x, residual, gamma, 1e-5), 1)
    rows_out.add("C2 add+RMSNorm 512x8192 [warm L2]", microseconds, None,
                 4 * tokens * hidden * 2 + 2 * hidden, "hbm", "33.5 MB fits in L2")
    big = [(torch.randn(4096, hidden, device="cuda").bfloat16(),
            torch.randn(4096, hidden, device="cuda").bfloat16()) for _ in range(2)]
    microseconds = graph_time_us(lambda i: _kernels.add_rms_norm(*big[i % 2], gamma, 1e-5), 2)
    rows_out.add("C2 add+RMSNorm 4096x8192 [cold]", microseconds, None,
                 4 * 4096 * hidden * 2 + 2 * hidden, "hbm", "same kernel, rows beyond L2")
    del big
    weight = bf16_weight(10240, hidden, 0.02, 1)[0]
    microseconds = graph_time_us(lambda i: _kernels.qkv_linear(x, weight, 8192, 1024, 1024), 1)
    rows_out.add("C2 QKV packed 512x8192 -> 10240", microseconds, 2 * tokens * 10240 * hidden,
                 2 * (10240 * hidden + tokens * hidden + tokens * 10240), "tensor_bf16")
    del weight
    linear_case(rows_out, "C2 QKV as one linear 512x8192 -> 10240", tokens, 10240, hidden)
    linear_case(rows_out, "C2 gate_up 512x8192 -> 57344", tokens, 57344, hidden)
    # the same projection with SwiGLU in the epilogue, against GEMM + silu_multiply
    weights = bf16_weight(57344, hidden, 0.02, 2)
    mixed = [_kernels.interleave_gate_up(w) for w in weights]
    flops = 2 * tokens * 57344 * hidden
    fused_bytes = 2 * (57344 * hidden + tokens * hidden + tokens * 28672)
    microseconds = graph_time_us(lambda i: _kernels.gate_up_swiglu(x, mixed[i % 2]), 2)
    rows_out.add("C2 gate_up + SwiGLU in the epilogue -> 28672", microseconds, flops, fused_bytes,
                 "tensor_bf16")
    del mixed

    def two_step(i):
        both = _kernels.linear(x, weights[i % 2]).view(tokens, 2, 28672)
        return _kernels.silu_multiply(both[:, 0], both[:, 1])

    microseconds = graph_time_us(two_step, 2)
    rows_out.add("C2 gate_up GEMM, then silu_multiply (two kernels + copies)", microseconds, flops,
                 fused_bytes + 3 * tokens * 57344 * 2, "tensor_bf16", "comparator")
    del weights
    linear_case(rows_out, "C2 down 512x28672 -> 8192", tokens, 8192, 28672)


def quantise_weight_blocks(weight):
    """128x128 block quantisation of a BF16 weight with torch ops (set-up only, not timed)."""
    import torch

    outputs, inner = weight.shape
    bands = (outputs + 127) // 128
    padded = torch.zeros(bands * 128, inner, device=weight.device, dtype=torch.float32)
    padded[:outputs] = weight.float()
    blocks = padded.view(bands, 128, inner // 128, 128)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-10)
    scale = amax * (1.0 / 448.0)
    q = (blocks * (448.0 / amax)[:, None, :, None]).clamp(-448, 448).view(bands * 128, inner)
    return q[:outputs].to(torch.float8_e4m3fn).contiguous(), scale.contiguous()


def table_config3(rows_out):
    import torch
    from camblas_b200 import _kernels

    for outputs, inner in ((4096, 7168), (7168, 2048), (2112, 7168), (24576, 1536)):
        for tokens in (1, 16, 128, 4096):
            nbytes = (outputs * inner + tokens * inner + 4 * tokens * inner // 128
                      + 4 * ((outputs + 127) // 128) * inner // 128 + 2 * tokens * outputs)
            flops = 2 * tokens * outputs * inner
            bound = "hbm" if tokens <= 128 else "tensor_fp8"
            copies = copies_for_cold(nbytes) if bound == "hbm" else 1
            weights = [quantise_weight_blocks(torch.randn(outputs, inner, device="cuda").bfloat16())
                       for _ in range(copies)]
            x = torch.randn(tokens, inner, device="cuda").bfloat16()
            q, q_scale = _kernels.fp8_quantize(x)
            microseconds = graph_time_us(
                lambda i: _kernels.fp8_block_gemm(q, q_scale, *weights[i % copies]), copies)
            rows_out.add(f"C3 FP8 GEMM M={tokens} N={outputs} K={inner}"
                         + (" [cold]" if bound == "hbm" else ""), microseconds, flops, nbytes, bound)
            if outputs == 4096:
                microseconds = graph_time_us(lambda i: _kernels.fp8_quantize(x), 1)
                rows_out.add(f"C3 quantise prologue M={tokens} K={inner}", microseconds, None,
                             2 * tokens * inner + tokens * inner + 4 * tokens * inner // 128, "hbm",
                             "warm L2 below 42 MB")
            del weights


def table_config4(rows_out):
    for name, outputs, inner in (("down", 8192, 28672), ("gate_up", 57344, 8192)):
        for tokens in (1, 2, 4, 8, 16, 32, 64):
            linear_case(rows_out, f"C4 {name} M={tokens}", tokens, outputs, inner,
                        comparators=tokens in (1, 16, 64))


def table_config5(rows_out):
    import torch
    from camblas_b200 import _kernels, _native

    reference = ReferenceCuda.load()
    for n in (4096, 8192, 16384):
        a = (torch.rand(n, n, device="cuda") * 2 - 1).bfloat16()
        b = (torch.rand(n, n, device="cuda") * 2 - 1).bfloat16()
        flops, nbytes = 2 * n**3, 6 * n * n
        launches = 4 if n == 16384 else 10
        microseconds = graph_time_us(lambda i: _kernels.matmul(a, b), 1, launches=launches, replays=5)
        rows_out.add(f"C5 classical n={n}", microseconds, flops, nbytes, "tensor_bf16")
        microseconds = graph_time_us(lambda i: torch.matmul(a, b), 1, launches=launches, replays=5)
        rows_out.add(f"C5 classical n={n} torch/cuBLAS", microseconds, flops, nbytes, "tensor_bf16",
                     "comparator")
        if reference is not None:
            out = torch.empty((n, n), dtype=torch.bfloat16, device="cuda")
            for policy, route in ((1, "cublasGemmEx"), (3, "cublasLt")):
                microseconds = graph_time_us(lambda i: reference.linear(a, b, out, policy), 1,
                                             launches=launches, replays=5)
                rows_out.add(f"C5 classical n={n} reference library, {route} (A.B^T)", microseconds,
                             flops, nbytes, "tensor_bf16", "comparator")

        def strassen(i):
            with _native.algorithm("strassen"), _native.options(bf16_strassen=1):
                return _kernels.matmul(a, b)

        microseconds = graph_time_us(strassen, 1, launches=launches, replays=5)
        rows_out.add(f"C5 one-level Strassen n={n} (effective 2n^3)", microseconds, flops, nbytes,
                     "tensor_bf16")
        del a, b


def table_config6(rows_out):
    """What one rank multiplies when the M=512 block is sharded over 2, 4 and 8 GPUs:
    column-parallel QKV and gate_up (outputs / tp), row-parallel down (inner / tp)."""
    tokens = 512
    for tp in (2, 4, 8):
        linear_case(rows_out, f"C2/tp{tp} QKV shard 512x8192 -> {10240 // tp}", tokens, 10240 // tp, 8192)
        linear_case(rows_out, f"C2/tp{tp} gate_up shard 512x8192 -> {57344 // tp}", tokens,
                    57344 // tp, 8192)
        linear_case(rows_out, f"C2/tp{tp} down shard 512x{28672 // tp} -> 8192", tokens, 8192,
                    28672 // tp)


def table_config7(rows_out):
    """The RMS and elementwise kernels beside the GEMMs, cold (operands beyond L2)."""
    import torch
    from camblas_b200 import _kernels

    rows, width = 8192, 8192
    count = rows * width
    x = [torch.randn(rows, width, device="cuda").bfloat16() for _ in range(2)]
    y = [torch.randn(rows, width, device="cuda").bfloat16() for _ in range(2)]
    gamma = (1 + 0.1 * torch.randn(width, device="cuda")).bfloat16()
    routing = torch.rand(rows, device="cuda") + 0.5
    cases = (
        ("add+RMSNorm 8192x8192", lambda i: _kernels.add_rms_norm(x[i % 2], y[i % 2], gamma, 1e-5), 8),
        ("rms_norm 8192x8192 (multi-row order)", lambda i: _kernels.rms_norm(x[i % 2], gamma, 1e-5), 4),
        ("silu_multiply 8192x8192", lambda i: _kernels.silu_multiply(x[i % 2], y[i % 2]), 6),
        ("swiglu 8192x8192, limit and routing", lambda i: _kernels.swiglu(x[i % 2], y[i % 2], 7.0, routing), 6),
    )
    for name, call, bytes_per_element in cases:
        microseconds = graph_time_us(call, 2)
        rows_out.add(f"C7 {name} [cold]", microseconds, None, bytes_per_element * count, "hbm")
    one = torch.randn(1, 8192, device="cuda").bfloat16()
    microseconds = graph_time_us(lambda i: _kernels.rms_norm(one, gamma, 1e-5), 1)
    rows_out.add("C7 rms_norm 1x8192 (single-row order, latency)", microseconds, None, 6 * 8192, "hbm")
    microseconds = graph_time_us(lambda i: _kernels.add_rms_norm(one, one.clone(), gamma, 1e-5), 1)
    rows_out.add("C7 add+RMSNorm 1x8192 (latency)", microseconds, None, 10 * 8192, "hbm")


TABLES = {1: table_config1, 2: table_config2, 3: table_config3, 4: table_config4, 5: table_config5,
          6: table_config6, 7: table_config7}


def run_table(args):
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("the kernels need a CUDA device; there is no CPU route")
    torch.manual_seed(705537)
    rows_out = Rows()
    print(json.dumps({"peaks": rows_out.peaks, "device": torch.cuda.get_device_name(0)}), flush=True)
    for index in (int(part) for part in args.table.split(",")):
        TABLES[index](rows_out)
        torch.cuda.empty_cache()
    rows_out.save(args.json)


def run_single(args):
    """Run one operation a few times without a graph (for a profiler); print mean times."""
    import torch
    from camblas_b200 import _kernels, _native

    kind, tokens, outputs, inner = args.single.split(",")
    tokens, outputs, inner = int(tokens), int(outputs), int(inner)
    torch.manual_seed(705537)
    x = torch.randn(tokens, inner, device="cuda").bfloat16()
    if kind == "rms":
        residual = torch.randn(tokens, inner, device="cuda").bfloat16()
        gamma = (1 + 0.1 * torch.randn(inner, device="cuda")).bfloat16()
        calls = {"ours": lambda: _kernels.add_rms_norm(x, residual, gamma, 1e-5)}
        work = 0
    else:
        weight = (torch.randn(outputs, inner, device="cuda") * 0.02).bfloat16()
        work = 2 * tokens * outputs * inner
        if kind == "fp8":
            q, q_scale = _kernels.fp8_quantize(x)
            w8, w_scale = quantise_weight_blocks(weight)
            calls = {"ours": lambda: _kernels.fp8_block_gemm(q, q_scale, w8, w_scale)}
        else:
            calls = {"ours": lambda: _kernels.linear(x, weight),
                     "cublas": lambda: torch.nn.functional.linear(x, weight)}
    result = {"single": [kind, tokens, outputs, inner]}
    for name, call in calls.items():
        call()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(20):
            call()
        end.record()
        torch.cuda.synchronize()
        microseconds = begin.elapsed_time(end) * 1e3 / 20
        result[name + "_us"] = round(microseconds, 1)
        if work:
            result[name + "_tflops"] = round(work / microseconds / 1e6, 1)
    result["status"] = _native.context(0).device_status()
    print(json.dumps(result), flush=True)


# ---- tensor-parallel sweeps ------------------------------------------------------------


def sampled_dots(torch, x, weight, out, samples=64, seed=11):
    """rel-L2 of `samples` entries of out = x @ weight.T against FP64 dot products
    (the way the reference samples large products, bench/cuda_workload.py:403-422)."""
    generator = torch.Generator().manual_seed(seed)
    picks_r = torch.randint(0, x.shape[0], (samples,), generator=generator).to(x.device)
    picks_c = torch.randint(0, weight.shape[0], (samples,), generator=generator).to(x.device)
    expected = (x[picks_r].double() * weight[picks_c].double()).sum(1)
    got = out[picks_r, picks_c].double()
    return ((got - expected).norm() / expected.norm().clamp_min(1e-30)).item()


def run_decode_tp(args):
    """Decode sweep M = 1..64 on the Llama-70B down (row parallel: inner dimension split,
    NCCL all-reduce of the BF16 partial results) and gate_up (column parallel: outputs
    split, no communication) projections over the ranks this was launched with.

    Per case: the shard's product alone (cold: rotating weight copies beyond L2), for the
    row-parallel layer the all-reduce alone and product + all-reduce together, each as
    the maximum over ranks inside replayed CUDA graphs; per-GPU GB/s of the product
    against the HBM roofline. Parity on every rank: 64 sampled entries of its own shard
    against FP64 dot products, and the assembled result against the unsharded product
    computed by the same library on that GPU (rel-L2 <= 1e-2).
    """
    torch, dist, rank, world, device = distributed_setup(args)
    from camblas_b200 import _kernels, tp

    rows_out = Rows(rank)
    collective = (dist, world, device) if world > 1 else None
    failures = []
    peers = None
    if world > 1:
        try:
            peers = tp.PeerRegions.create(tp.PeerRegions.capacity_for(64, 8192), device.index)
        except RuntimeError as error:
            if rank == 0:
                print(f"bench: peer regions unavailable ({error}); NCCL only", file=sys.stderr)
    for name, outputs, inner, mode in (("down", 8192, 28672, "row"), ("gate_up", 57344, 8192, "column")):
        generator = torch.Generator(device=device).manual_seed(705537 + 4)
        weight = (torch.randn((outputs, inner), device=device, generator=generator) * 0.02).bfloat16()
        if mode == "row":
            layer = tp.RowParallelLinear(weight, rank, world, multiple=128)
        else:
            layer = tp.ColumnParallelLinear(weight, rank, world, multiple=128)
        shard = layer.weight
        shard_bytes = 2 * shard.numel()
        copies = copies_for_cold(shard_bytes)
        shards = [shard] + [shard.clone() for _ in range(copies - 1)]
        for tokens in (1, 2, 4, 8, 16, 32, 64):
            x = torch.randn((tokens, inner), device=device, generator=generator).bfloat16()
            x_local = layer.slice_input(x) if mode == "row" else x
            nbytes = shard_bytes + 2 * x_local.numel() + 2 * tokens * shard.shape[0]
            product = graph_time_us(lambda i: _kernels.linear(x_local, shards[i % copies]), copies,
                                    collective=collective)
            entry = {"tp": world, "tokens": tokens, "mode": mode}
            if mode == "row" and world > 1:
                payload = torch.zeros((tokens, outputs), dtype=torch.bfloat16, device=device)
                try:
                    reduce_us = graph_time_us(lambda i: dist.all_reduce(payload), 1, collective=collective)
                    entry["all_reduce_us"] = round(reduce_us, 2)

                    def both(i):
                        partial = _kernels.linear(x_local, shards[i % copies])
                        dist.all_reduce(partial)
                        return partial

                    entry["product_plus_all_reduce_us"] = round(
                        graph_time_us(both, copies, collective=collective), 2)
                except Exception as error:  # noqa: BLE001 - a collective that cannot be captured
                    entry["all_reduce_us"] = None
                    entry["note_all_reduce"] = f"not captured in a graph: {error}"
                entry["all_reduce_bytes"] = 2 * tokens * outputs
                if peers is not None:
                    # the library's own one-shot exchange over peer memory
                    entry["peer_all_reduce_us"] = round(graph_time_us(
                        lambda i: peers.all_reduce(payload, out=payload), 1, collective=collective), 2)

                    def fused(i):
                        partial = _kernels.linear(x_local, shards[i % copies])
                        return peers.all_reduce(partial, out=partial)

                    entry["product_plus_peer_all_reduce_us"] = round(
                        graph_time_us(fused, copies, collective=collective), 2)
                    summed = peers.all_reduce(_kernels.linear(x_local, shard))
                    whole_sum = _kernels.linear(x, weight).float()
                    entry["peer_sum_rel_l2_vs_unsharded"] = (
                        (summed.float() - whole_sum).norm() / whole_sum.norm()).item()
                    if not entry["peer_sum_rel_l2_vs_unsharded"] <= 1e-2:
                        failures.append((name, tokens, "peer sum"))
            # parity: own shard by sampled FP64 dots, assembled result against the unsharded product
            local = layer.linear(x_local, shard)
            entry["shard_rel_l2_fp64_samples"] = sampled_dots(torch, x_local, shard, local)
            assembled = layer(x_local)
            if mode == "column" and world > 1:
                pieces = [torch.empty_like(assembled) for _ in range(world)]
                dist.all_gather(pieces, assembled)
                assembled = torch.cat(pieces, dim=1)
            whole = _kernels.linear(x, weight).float()
            entry["assembled_rel_l2_vs_unsharded"] = (
                (assembled.float() - whole).norm() / whole.norm()).item()
            entry["assembled_rel_l2_fp64_samples"] = sampled_dots(torch, x, weight, assembled)
            bad = max(entry["shard_rel_l2_fp64_samples"], entry["assembled_rel_l2_vs_unsharded"],
                      entry["assembled_rel_l2_fp64_samples"])
            if not bad <= 1e-2:
                failures.append((name, tokens, bad))
            rows_out.add(f"C4 {name} M={tokens} tp{world} per-GPU shard [cold]", product, None, nbytes,
                         "hbm", **entry)
        del shards, layer, weight
        torch.cuda.empty_cache()
    rows_out.save(args.json)
    shutdown(torch, dist, world, peers)
    if failures:
        raise SystemExit(f"parity failures: {failures}")


def run_square_tp(args):
    """Large squares C = A.B, n in {4096, 8192, 16384}, uniform [-1, 1] BF16, B and C split
    by columns over the ranks (no communication). Per rank: the shard product timed in a
    replayed graph (max over ranks), TFLOP/s per GPU and aggregate, 64 sampled entries
    against FP64 dot products, and the gathered C against the unsharded product on the
    same GPU. One Strassen level applies to squares only, so it is timed at one rank."""
    torch, dist, rank, world, device = distributed_setup(args)
    from camblas_b200 import _kernels, _native

    rows_out = Rows(rank)
    collective = (dist, world, device) if world > 1 else None
    failures = []
    for n in (4096, 8192, 16384):
        generator = torch.Generator(device=device).manual_seed(705537 + 5 + n)
        a = (torch.rand((n, n), device=device, generator=generator) * 2 - 1).bfloat16()
        b = (torch.rand((n, n), device=device, generator=generator) * 2 - 1).bfloat16()
        width = n // world
        b_shard = b[:, rank * width:(rank + 1) * width]  # a view: row pitch n, no copy
        launches = 4 if n == 16384 else 10
        microseconds = graph_time_us(lambda i: _kernels.matmul(a, b_shard), 1, launches=launches,
                                     replays=5, collective=collective)
        shard = _kernels.matmul(a, b_shard)
        entry = {"tp": world, "n": n, "aggregate_tflops": round(2 * n**3 / microseconds / 1e6, 1)}
        entry["shard_rel_l2_fp64_samples"] = sampled_dots(torch, a, b_shard.t(), shard)
        if world > 1:
            pieces = [torch.empty_like(shard) for _ in range(world)]
            dist.all_gather(pieces, shard)
            gathered = torch.cat(pieces, dim=1)
        else:
            gathered = shard
        whole = _kernels.matmul(a, b)
        entry["gathered_rel_l2_vs_unsharded"] = (
            (gathered.float() - whole.float()).norm() / whole.float().norm()).item()
        del gathered, whole
        bad = max(entry["shard_rel_l2_fp64_samples"], entry["gathered_rel_l2_vs_unsharded"])
        if not bad <= 1e-2:
            failures.append((n, bad))
        rows_out.add(f"C5 classical n={n} tp{world} per-GPU column shard", microseconds,
                     2 * n**3 / world, 2 * (n * n + 2 * n * width), "tensor_bf16", **entry)
        if world == 1:
            def strassen(i):
                with _native.algorithm("strassen"), _native.options(bf16_strassen=1):
                    return _kernels.matmul(a, b)

            microseconds = graph_time_us(strassen, 1, launches=launches, replays=5)
            fast = strassen(0)
            rows_out.add(f"C5 one-level Strassen n={n} (effective 2n^3)", microseconds, 2 * n**3,
                         6 * n * n, "tensor_bf16",
                         rel_l2_fp64_samples=sampled_dots(torch, a, b.t(), fast))
        del a, b, shard
        torch.cuda.empty_cache()
    rows_out.save(args.json)
    shutdown(torch, dist, world)
    if failures:
        raise SystemExit(f"parity failures: {failures}")


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    elif args.table:
        run_table(args)
    elif args.single:
        run_single(args)
    elif args.workload == "decode_tp":
        run_decode_tp(args)
    elif args.workload == "square_tp":
        run_square_tp(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
