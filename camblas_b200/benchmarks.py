"""Kernel-level measurements over the five benchmark configurations.

    python -m camblas_b200.benchmarks [--configs 1,2,3,4,5] [--json out.json]

``bench.py`` at the repository root measures the headline workload; this module
measures every configuration of the benchmark definition one kernel at a time,
the way the reference's ``bench/cuda_workload.py`` times single operations
(warm-ups, repeated timed runs, CUDA events, ``:352-399``), and prints one row
per case with absolute throughput and the fraction of the roofline that bounds
it. Timing is taken inside a replayed CUDA graph of many launches so that
microsecond kernels are not hidden behind host launch cost; HBM-bound cases
rotate through enough distinct copies of the weight to exceed the 126 MB L2
("cold"), and are also reported re-reading one copy ("warm").

Peaks are the driver-measured figures in ``MEASURED_PEAKS.json`` when that file
exists (copy bandwidth and cuBLAS BF16 throughput of this machine), otherwise
6650 GB/s and 1590 TFLOP/s. The FP8 tensor peak is taken as twice the BF16
figure.
"""

import argparse
import json
import statistics
from pathlib import Path

import torch

from . import _kernels, _native

ROOT = Path(__file__).resolve().parents[1]
L2_BYTES = 126 * 2**20


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        data = json.loads(path.read_text())
        return {"hbm": data["hbm_gbs"], "bf16": data["bf16_tflops"], "source": "measured"}
    return {"hbm": 6650.0, "bf16": 1590.0, "source": "fallback"}


def graph_time_us(call, variants, launches=20, replays=7):
    """Median microseconds per launch of ``call(i)`` inside a replayed CUDA graph.

    ``call(i)`` must launch the operation on variant ``i % variants``. The
    warm-up runs on the capture stream first, because a native context belongs
    to one stream and cannot be created during capture.
    """
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.inference_mode(), torch.cuda.stream(stream):
        for i in range(max(variants, 2)):
            call(i)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(launches):
                call(i)
        for _ in range(2):
            graph.replay()
        stream.synchronize()
        times = []
        for _ in range(replays):
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
    return statistics.median(times)


def copies_for_cold(nbytes):
    return max(1, min(64, -(-2 * L2_BYTES // nbytes)))


def bf16_weight(outputs, inner, scale, copies):
    return [(torch.randn(outputs, inner, device="cuda") * scale).bfloat16() for _ in range(copies)]


def row(results, name, microseconds, flops=None, nbytes=None, bound="hbm", note=""):
    peak = peaks()
    entry = {"case": name, "us": round(microseconds, 2), "bound": bound, "note": note}
    if flops is not None:
        entry["tflops"] = round(flops / microseconds / 1e6, 1)
    if nbytes is not None:
        entry["gbs"] = round(nbytes / microseconds / 1e3, 1)
    if bound == "hbm":
        entry["frac"] = round(entry["gbs"] / peak["hbm"], 3)
    elif bound == "tensor_bf16":
        entry["frac"] = round(entry["tflops"] / peak["bf16"], 3)
    else:
        entry["frac"] = round(entry["tflops"] / (2 * peak["bf16"]), 3)
    results.append(entry)
    print(json.dumps(entry), flush=True)


def linear_case(results, name, tokens, outputs, inner, scale=0.02, bound=None, reference=True):
    nbytes = 2 * (outputs * inner + tokens * inner + tokens * outputs)
    flops = 2 * tokens * outputs * inner
    if bound is None:
        bound = "hbm" if tokens <= 64 else "tensor_bf16"
    x = torch.randn(tokens, inner, device="cuda").bfloat16()
    for label, copies in (("cold", copies_for_cold(nbytes)), ("warm", 1)):
        if label == "warm" and (bound != "hbm" or nbytes > L2_BYTES):
            continue
        weights = bf16_weight(outputs, inner, scale, copies)
        mine = graph_time_us(lambda i: _kernels.linear(x, weights[i % copies]), copies)
        row(results, f"{name} [{label}]", mine, flops, nbytes, bound)
        if reference:
            theirs = graph_time_us(lambda i: torch.nn.functional.linear(x, weights[i % copies]), copies)
            row(results, f"{name} [{label}] torch/cuBLAS", theirs, flops, nbytes, bound, "comparator")
        del weights


def config1(results):
    linear_case(results, "C1 decode 1x2048 -> 4096", 1, 4096, 2048, scale=1.0)


def config2(results):
    tokens, hidden = 512, 8192
    x = torch.randn(tokens, hidden, device="cuda").bfloat16()
    residual = torch.randn(tokens, hidden, device="cuda").bfloat16()
    gamma = (1 + 0.1 * torch.randn(hidden, device="cuda")).bfloat16()
    microseconds = graph_time_us(lambda i: _kernels.add_rms_norm(x, residual, gamma, 1e-5), 1)
    row(results, "C2 add+RMSNorm 512x8192 [warm L2]", microseconds, None,
        4 * tokens * hidden * 2 + 2 * hidden, "hbm", "33.5 MB fits in L2")
    big = [(torch.randn(4096, hidden, device="cuda").bfloat16(),
            torch.randn(4096, hidden, device="cuda").bfloat16()) for _ in range(2)]
    microseconds = graph_time_us(lambda i: _kernels.add_rms_norm(*big[i % 2], gamma, 1e-5), 2)
    row(results, "C2 add+RMSNorm 4096x8192 [cold]", microseconds, None,
        4 * 4096 * hidden * 2 + 2 * hidden, "hbm", "same kernel, rows beyond L2")
    weight = bf16_weight(10240, hidden, 0.02, 1)[0]
    microseconds = graph_time_us(lambda i: _kernels.qkv_linear(x, weight, 8192, 1024, 1024), 1)
    row(results, "C2 QKV packed 512x8192 -> 10240", microseconds, 2 * tokens * 10240 * hidden,
        2 * (10240 * hidden + tokens * hidden + tokens * 10240), "tensor_bf16")
    del weight
    linear_case(results, "C2 gate_up 512x8192 -> 57344", tokens, 57344, hidden)
    # the same projection with SwiGLU in the epilogue, against GEMM + silu_multiply
    weights = bf16_weight(57344, hidden, 0.02, 2)
    mixed = [_kernels.interleave_gate_up(w) for w in weights]
    flops = 2 * tokens * 57344 * hidden
    fused_bytes = 2 * (57344 * hidden + tokens * hidden + tokens * 28672)
    microseconds = graph_time_us(lambda i: _kernels.gate_up_swiglu(x, mixed[i % 2]), 2)
    row(results, "C2 gate_up + SwiGLU in the epilogue -> 28672", microseconds, flops, fused_bytes,
        "tensor_bf16")
    del mixed

    def two_step(i):
        both = _kernels.linear(x, weights[i % 2]).view(tokens, 2, 28672)
        return _kernels.silu_multiply(both[:, 0], both[:, 1])

    microseconds = graph_time_us(two_step, 2)
    row(results, "C2 gate_up GEMM, then silu_multiply (two kernels + copies)", microseconds, flops,
        fused_bytes + 3 * tokens * 57344 * 2, "tensor_bf16", "comparator")
    del weights
    linear_case(results, "C2 down 512x28672 -> 8192", tokens, 8192, 28672)


def quantise_weight_blocks(weight):
    """128x128 block quantisation of a BF16 weight with torch ops (set-up only, not timed)."""
    outputs, inner = weight.shape
    bands = (outputs + 127) // 128
    padded = torch.zeros(bands * 128, inner, device=weight.device, dtype=torch.float32)
    padded[:outputs] = weight.float()
    blocks = padded.view(bands, 128, inner // 128, 128)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-10)
    scale = amax * (1.0 / 448.0)
    q = (blocks * (448.0 / amax)[:, None, :, None]).clamp(-448, 448).view(bands * 128, inner)
    return q[:outputs].to(torch.float8_e4m3fn).contiguous(), scale.contiguous()


def config3(results):
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
            row(results, f"C3 FP8 GEMM M={tokens} N={outputs} K={inner}"
                + (" [cold]" if bound == "hbm" else ""), microseconds, flops, nbytes, bound)
            if outputs == 4096:
                microseconds = graph_time_us(lambda i: _kernels.fp8_quantize(x), 1)
                row(results, f"C3 quantise prologue M={tokens} K={inner}", microseconds, None,
                    2 * tokens * inner + tokens * inner + 4 * tokens * inner // 128, "hbm",
                    "warm L2 below 42 MB")
            del weights


def config4(results):
    for name, outputs, inner in (("down", 8192, 28672), ("gate_up", 57344, 8192)):
        for tokens in (1, 2, 4, 8, 16, 32, 64):
            linear_case(results, f"C4 {name} M={tokens}", tokens, outputs, inner,
                        reference=tokens in (1, 16, 64))


def config5(results):
    for n in (4096, 8192, 16384):
        a = (torch.rand(n, n, device="cuda") * 2 - 1).bfloat16()
        b = (torch.rand(n, n, device="cuda") * 2 - 1).bfloat16()
        flops, nbytes = 2 * n**3, 6 * n * n
        launches = 4 if n == 16384 else 10
        microseconds = graph_time_us(lambda i: _kernels.matmul(a, b), 1, launches=launches, replays=5)
        row(results, f"C5 classical n={n}", microseconds, flops, nbytes, "tensor_bf16")
        microseconds = graph_time_us(lambda i: torch.matmul(a, b), 1, launches=launches, replays=5)
        row(results, f"C5 classical n={n} torch/cuBLAS", microseconds, flops, nbytes, "tensor_bf16",
            "comparator")

        def strassen(i):
            with _native.algorithm("strassen"):
                return _kernels.matmul(a, b)

        microseconds = graph_time_us(strassen, 1, launches=launches, replays=5)
        row(results, f"C5 one-level Strassen n={n} (effective 2n^3)", microseconds, flops, nbytes,
            "tensor_bf16")
        del a, b


def single(kind, tokens, outputs, inner, launches=20):
    """Run one product `launches` times without a graph; print its mean time and, for
    BF16, the time of torch's own (cuBLAS) linear on the same tensors in the same process."""
    x = torch.randn(tokens, inner, device="cuda").bfloat16()
    weight = (torch.randn(outputs, inner, device="cuda") * 0.02).bfloat16()
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
        for _ in range(launches):
            call()
        end.record()
        torch.cuda.synchronize()
        microseconds = begin.elapsed_time(end) * 1e3 / launches
        result[name + "_us"] = round(microseconds, 1)
        result[name + "_tflops"] = round(2 * tokens * outputs * inner / microseconds / 1e6, 1)
    result["status"] = _native.context(0).device_status()
    print(json.dumps(result), flush=True)


def config6(results):
    """What one rank multiplies when the M=512 block is sharded over 2, 4 and 8 GPUs:
    column-parallel QKV and gate_up (outputs / tp), row-parallel down (inner / tp)."""
    tokens = 512
    for tp in (2, 4, 8):
        linear_case(results, f"C2/tp{tp} QKV shard 512x8192 -> {10240 // tp}", tokens, 10240 // tp, 8192)
        linear_case(results, f"C2/tp{tp} gate_up shard 512x8192 -> {57344 // tp}", tokens,
                    57344 // tp, 8192)
        linear_case(results, f"C2/tp{tp} down shard 512x{28672 // tp} -> 8192", tokens, 8192,
                    28672 // tp)


CONFIGS = {1: config1, 2: config2, 3: config3, 4: config4, 5: config5, 6: config6}


def main():
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--configs", default="1,2,3,4,5")
    parser.add_argument("--json", default=None)
    parser.add_argument("--single", default=None, metavar="KIND,M,N,K",
                        help="run one product a few times eagerly (for a profiler): KIND is bf16 or fp8")
    args = parser.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("the kernels need a CUDA device; there is no CPU route")
    torch.manual_seed(705537)
    if args.single:
        kind, tokens, outputs, inner = args.single.split(",")
        single(kind, int(tokens), int(outputs), int(inner))
        return
    results = []
    print(json.dumps({"peaks": peaks(), "device": torch.cuda.get_device_name(0)}), flush=True)
    for index in (int(part) for part in args.configs.split(",")):
        CONFIGS[index](results)
        torch.cuda.empty_cache()
    if args.json:
        Path(args.json).write_text(json.dumps({"peaks": peaks(), "rows": results}, indent=1))


if __name__ == "__main__":
    main()
