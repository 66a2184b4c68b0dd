"""Generate the committed golden vectors from the reference's own CPU GEMM.

Run in a container that has the reference tree: ``make -C oracle`` compiles the
reference's portable library from its sources into ``oracle/_ref`` and this
script calls its ``cblas_sgemm`` (reference ``src/cblas_shim.c:162-205``) on
seeded inputs. The outputs are what the reference itself computes; the tests
compare the C restatement and the CUDA kernels against them.

    python tests/golden/make_golden.py

Files written beside this script:
  gemm_small.npz   small BF16 products, inputs stored as BF16 bit patterns
  c1_decode.npz    benchmark configuration 1 (x [1,2048], W [4096,2048], N(0,1)):
                   seed, SHA-256 of the regenerated inputs, reference output
  fp8_slice.npz    a slice of the FP8 configuration: BF16 sources, and the
                   reference FP32 GEMM on the dequantised E4M3 operands
"""

import hashlib
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import oracle  # noqa: E402

HERE = Path(__file__).resolve().parent


def digest(*arrays):
    sha = hashlib.sha256()
    for array in arrays:
        sha.update(np.ascontiguousarray(array).tobytes())
    return sha.hexdigest()


def config1_inputs(seed=705538):
    """x [1,2048] and W [4096,2048] drawn N(0,1) from the seed, rounded to BF16."""
    rng = np.random.default_rng(seed)
    x = oracle.bf16_bits(rng.standard_normal((1, 2048)).astype(np.float32))
    w = oracle.bf16_bits(rng.standard_normal((4096, 2048)).astype(np.float32))
    return x, w


def main():
    if oracle.reference_lib() is None:
        raise SystemExit("oracle/_ref/libcamblas_ref.so is missing: run make -C oracle first")
    rng = np.random.default_rng(20261004)
    cases = {}
    for index, (rows, outputs, inner) in enumerate([(7, 40, 72), (66, 130, 136), (1, 96, 520)]):
        x = oracle.bf16_bits(rng.standard_normal((rows, inner)).astype(np.float32))
        w = oracle.bf16_bits(rng.standard_normal((outputs, inner)).astype(np.float32))
        y = oracle.reference_linear_f32(oracle.bf16_values(x), oracle.bf16_values(w))
        cases[f"x{index}"], cases[f"w{index}"], cases[f"y{index}"] = x, w, y
    np.savez_compressed(HERE / "gemm_small.npz", **cases)

    x, w = config1_inputs()
    y = oracle.reference_linear_f32(oracle.bf16_values(x), oracle.bf16_values(w))
    np.savez_compressed(HERE / "c1_decode.npz", seed=np.int64(705538),
                        sha256=np.array(digest(x, w)), y=y)

    rows, outputs, inner = 3, 136, 256
    x = oracle.bf16_bits(rng.standard_normal((rows, inner)).astype(np.float32))
    w = oracle.bf16_bits(rng.standard_normal((outputs, inner)).astype(np.float32))
    q, qs = oracle.fp8_quantize_rows(x)
    wq, ws = oracle.fp8_quantize_weight(w)
    y = oracle.reference_linear_f32(oracle.fp8_dequantize(q, qs, 1), oracle.fp8_dequantize(wq, ws, 128))
    np.savez_compressed(HERE / "fp8_slice.npz", x=x, w=w, q=q, q_scale=qs, wq=wq, w_scale=ws, y=y)
    for name in ("gemm_small.npz", "c1_decode.npz", "fp8_slice.npz"):
        print(name, (HERE / name).stat().st_size, "bytes")


if __name__ == "__main__":
    main()
