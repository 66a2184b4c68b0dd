"""ctypes access to the CPU checkers in this directory.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
CPU leg of ``bench.py``. The package ``camblas_b200`` never imports it.

``liboracle.so`` is the C restatement (``camblas_oracle.c``);
``_ref/libcamblas_ref.so`` is the reference's own portable CPU GEMM compiled
from its sources by ``oracle/Makefile`` and called through its ``cblas_sgemm``
(reference ``src/cblas_shim.c:162-205``) - single threaded, FP32 accumulation
in ascending k.
"""

import ctypes as ct
import os
import subprocess
from functools import lru_cache
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_P = ct.c_void_p
_I = ct.c_int
_F = ct.c_float


def reference_tree():
    """Where the reference's sources are, or None.

    ``CAMBLAS_REFERENCE`` names the tree; without it a checkout called
    ``reference`` beside this repository is used when it exists. On a machine
    with neither, only the prebuilt files under ``_ref/`` are available.
    """
    named = os.environ.get("CAMBLAS_REFERENCE")
    candidates = [Path(named)] if named else [HERE.parents[1] / "reference"]
    for candidate in candidates:
        if (candidate / "src" / "scalar.c").is_file():
            return candidate
    return None


def build():
    """Compile ``liboracle.so`` and, when the reference's sources are at hand, the
    reference's own CPU and CUDA libraries into ``_ref/`` (see the Makefile)."""
    command = ["make", "-C", str(HERE)]
    tree = reference_tree()
    if tree is not None:
        command.append(f"REFERENCE={tree}")
    subprocess.run(command, check=True, capture_output=True)


@lru_cache(maxsize=1)
def lib():
    """Load the C restatement, building it first if necessary."""
    path = HERE / "liboracle.so"
    if not path.is_file():
        build()
    library = ct.CDLL(str(path))
    library.oracle_bf16_to_float.restype = _F
    library.oracle_bf16_to_float.argtypes = [ct.c_uint16]
    library.oracle_float_to_bf16.restype = ct.c_uint16
    library.oracle_float_to_bf16.argtypes = [_F]
    library.oracle_e4m3_to_float.restype = _F
    library.oracle_e4m3_to_float.argtypes = [ct.c_uint8]
    library.oracle_float_to_e4m3.restype = ct.c_uint8
    library.oracle_float_to_e4m3.argtypes = [_F]
    library.oracle_sgemm.argtypes = [ct.c_char, ct.c_char, _I, _I, _I, _F, _P, _I, _P, _I, _F, _P, _I]
    library.oracle_bgemm.argtypes = [ct.c_char, ct.c_char, _I, _I, _I, _F, _P, _I, _P, _I, _F, _P, _I]
    library.oracle_linear_bf16.argtypes = [_I, _I, _I, _P, _I, _P, _I, _P, _P, _I, _P, _I]
    library.oracle_rms_row.argtypes = [_I, _I, _I, _F, _I, _I, _P, _P, _P, _P, _P]
    library.oracle_add_rms_norm_rows.argtypes = [_I, _I, _I, _F, _P, _P, _P, _P, _P]
    library.oracle_rms_norm_rows.argtypes = [_I, _I, _I, _F, _P, _P, _P]
    library.oracle_silu_multiply_bf16.argtypes = [ct.c_size_t, _P, _P, _P]
    library.oracle_swiglu_bf16.argtypes = [ct.c_size_t, _I, _F, _P, _P, _P, _P]
    library.oracle_fp8_quantize_rows.argtypes = [_I, _I, _P, _I, _P, _P]
    library.oracle_fp8_quantize_weight.argtypes = [_I, _I, _P, _P, _P]
    library.oracle_fp8_block_gemm.argtypes = [_I, _I, _I, _P, _P, _P, _P, _P, _I]
    library.oracle_fp8_dequantize.argtypes = [_I, _I, _I, _P, _P, _P]
    library.oracle_fp8_quantize_block32.argtypes = [_I, _P, _P, _P]
    library.oracle_fp8_decode.argtypes = [_I, _I, _P, _P, _I, _P, _P, _I, _I, _P]
    library.oracle_strassen_bf16.argtypes = [_I, _F, _P, _I, _P, _I, _F, _P, _I, _P]
    return library


@lru_cache(maxsize=1)
def reference_lib():
    """Load the reference's own CPU library, or return None when it is absent."""
    path = HERE / "_ref" / "libcamblas_ref.so"
    if not path.is_file():
        try:
            build()
        except (subprocess.CalledProcessError, OSError):
            return None
    if not path.is_file():
        return None
    library = ct.CDLL(str(path))
    library.cblas_sgemm.argtypes = [_I, _I, _I, _I, _I, _I, _F, _P, _I, _P, _I, _F, _P, _I]
    library.cblas_sgemm.restype = None
    return library


def _ptr(array):
    return array.ctypes.data_as(_P) if array is not None else _P()


# ---- storage conversions on numpy arrays -------------------------------------

def bf16_bits(values):
    """Round an FP32 array to BF16 (nearest even) and return the uint16 bit patterns."""
    words = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    nan = (words & 0x7FFFFFFF) > 0x7F800000
    rounded = ((words + 0x7FFF + ((words >> 16) & 1)) >> 16).astype(np.uint16)
    rounded[nan] = 0x7FFF
    return rounded


def bf16_values(bits):
    """Expand uint16 BF16 bit patterns to FP32 values."""
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def e4m3_values(bits):
    """Decode uint8 E4M3 bit patterns to FP32 values."""
    table = np.array([lib().oracle_e4m3_to_float(i) for i in range(256)], dtype=np.float32)
    return table[np.ascontiguousarray(bits, dtype=np.uint8)]


# ---- GEMM ---------------------------------------------------------------------

def sgemm(trans_a, trans_b, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc):
    """Column-major FP32 GEMM restating the reference's scalar kernel; c is updated in place."""
    lib().oracle_sgemm(trans_a.encode(), trans_b.encode(), m, n, k, alpha, _ptr(a), lda, _ptr(b),
                       ldb, beta, _ptr(c), ldc)
    return c


def bgemm(trans_a, trans_b, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc):
    """Column-major BF16 GEMM on uint16 bit patterns; c is updated in place."""
    lib().oracle_bgemm(trans_a.encode(), trans_b.encode(), m, n, k, alpha, _ptr(a), lda, _ptr(b),
                       ldb, beta, _ptr(c), ldc)
    return c


def linear_bf16(x, w, bias=None, residual=None):
    """Row-major ``x @ w.T + bias + residual`` on uint16 BF16 arrays, one rounding."""
    rows, inner = x.shape
    outputs = w.shape[0]
    out = np.empty((rows, outputs), dtype=np.uint16)
    lib().oracle_linear_bf16(rows, inner, outputs, _ptr(x), x.strides[0] // 2, _ptr(w),
                             w.strides[0] // 2, _ptr(bias), _ptr(residual),
                             residual.strides[0] // 2 if residual is not None else 0, _ptr(out),
                             outputs)
    return out


def reference_linear_f32(x, w):
    """``x @ w.T`` in FP32 through the reference's own ``cblas_sgemm``.

    Row-major call ``cblas_sgemm(RowMajor, NoTrans, Trans, M, N, K, 1, x, K, w, K, 0, y, N)``.
    Falls back to the C restatement (bit-identical arithmetic) when the
    reference library is not present.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, inner = x.shape
    outputs = w.shape[0]
    y = np.zeros((rows, outputs), dtype=np.float32)
    reference = reference_lib()
    if reference is not None:
        reference.cblas_sgemm(101, 111, 112, rows, outputs, inner, 1.0, _ptr(x), inner, _ptr(w),
                              inner, 0.0, _ptr(y), outputs)
    else:
        # column-major view: y^T[outputs, rows] = w[outputs, inner] x^T -> 'T','N'
        sgemm("T", "N", outputs, rows, inner, 1.0, w, inner, x, inner, 0.0, y, outputs)
    return y


class _ReferenceContext(ct.Structure):
    """``camblas_ctx_t`` of the reference (``include/camblas.h:63-69``)."""

    _fields_ = [("num_threads", _I), ("reproducibility", _I), ("planner_mode", ct.c_char_p),
                ("topo", _P), ("executor", _P)]


class ReferencePool:
    """The reference's pinned pthread pool driving its own ``camblas_sgemm``.

    ``cblas_sgemm`` uses the default single-thread context; the native entry
    point takes a context whose executor may be the reference's pool
    (``include/camblas_pthread.h``, ``src/pthread_pool.c``), which the portable
    kernel feeds with up to 256 row tiles of C (``src/scalar.c:456-461``).
    """

    def __init__(self, cpus=None):
        import os

        self.library = reference_lib()
        if self.library is None:
            raise RuntimeError("reference library not built")
        cpus = sorted(os.sched_getaffinity(0)) if cpus is None else list(cpus)
        self.cpus = cpus
        self.library.camblas_pthread_pool_create.restype = _P
        self.library.camblas_pthread_pool_create.argtypes = [_I, ct.POINTER(_I)]
        self.library.camblas_pthread_pool_executor.restype = _P
        self.library.camblas_pthread_pool_executor.argtypes = [_P]
        self.library.camblas_pthread_pool_destroy.argtypes = [_P]
        self.library.camblas_sgemm.argtypes = [ct.POINTER(_ReferenceContext), ct.c_char, ct.c_char,
                                               _I, _I, _I, _F, _P, _I, _P, _I, _F, _P, _I]
        self.pool = self.library.camblas_pthread_pool_create(len(cpus), (_I * len(cpus))(*cpus))
        if not self.pool:
            raise RuntimeError("reference pthread pool could not be created")
        self.context = _ReferenceContext(len(cpus), 0, b"none", None,
                                         self.library.camblas_pthread_pool_executor(self.pool))

    def linear_f32(self, x, w):
        """``x @ w.T`` in FP32: column-major C[outputs, rows] = w^T-view x, 'T','N'."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.float32)
        rows, inner = x.shape
        outputs = w.shape[0]
        y = np.zeros((rows, outputs), dtype=np.float32)
        status = self.library.camblas_sgemm(ct.byref(self.context), b"T", b"N", outputs, rows, inner,
                                            1.0, _ptr(w), inner, _ptr(x), inner, 0.0, _ptr(y), outputs)
        if status != 0:
            raise RuntimeError("reference camblas_sgemm failed")
        return y

    def close(self):
        if self.pool:
            self.library.camblas_pthread_pool_destroy(self.pool)
            self.pool = None


# ---- RMS ------------------------------------------------------------------------

def add_rms_norm_rows(x, residual, weight, epsilon):
    """Residual add + RMS norm per row on uint16 BF16 (or FP32) arrays -> (added, out)."""
    bf16 = int(x.dtype == np.uint16)
    rows, width = x.shape
    added, out = np.empty_like(x), np.empty_like(x)
    lib().oracle_add_rms_norm_rows(bf16, rows, width, epsilon, _ptr(x), _ptr(residual),
                                   _ptr(weight), _ptr(added), _ptr(out))
    return added, out


def rms_row(x, weight, epsilon, residual=None, round_before_weight=True, descending=False):
    """One row with the reference's selectable rounding and shuffle direction."""
    bf16 = int(x.dtype == np.uint16)
    weight_fp32 = int(bf16 and weight.dtype == np.float32)
    width = x.shape[-1]
    added = np.empty_like(x) if residual is not None else None
    out = np.empty_like(x)
    lib().oracle_rms_row(bf16, weight_fp32, width, epsilon, int(round_before_weight),
                         int(descending), _ptr(x), _ptr(residual), _ptr(weight), _ptr(added),
                         _ptr(out))
    return added, out


def rms_norm_rows(x, weight, epsilon):
    """Multi-row RMS norm in the order of the reference's 256-thread kernel."""
    bf16 = int(x.dtype == np.uint16)
    rows, width = x.shape
    out = np.empty_like(x)
    lib().oracle_rms_norm_rows(bf16, rows, width, epsilon, _ptr(x), _ptr(weight), _ptr(out))
    return out


def silu_multiply_bf16(gate, up):
    out = np.empty_like(gate)
    lib().oracle_silu_multiply_bf16(gate.size, _ptr(gate), _ptr(up), _ptr(out))
    return out


def swiglu_bf16(gate, up, limit=0.0, routing=None):
    out = np.empty_like(gate)
    lib().oracle_swiglu_bf16(gate.size, gate.shape[-1], limit, _ptr(gate), _ptr(up), _ptr(routing),
                             _ptr(out))
    return out


# ---- FP8 -------------------------------------------------------------------------

def fp8_quantize_rows(x):
    """Block-128 activation quantiser on uint16 BF16 [rows, inner] -> (uint8 q, fp32 scale)."""
    rows, inner = x.shape
    q = np.empty((rows, inner), dtype=np.uint8)
    scale = np.empty((rows, inner // 128), dtype=np.float32)
    lib().oracle_fp8_quantize_rows(rows, inner, _ptr(x), x.strides[0] // 2, _ptr(q), _ptr(scale))
    return q, scale


def fp8_quantize_weight(w):
    """128x128 block weight quantiser on uint16 BF16 [outputs, inner]."""
    outputs, inner = w.shape
    q = np.empty((outputs, inner), dtype=np.uint8)
    scale = np.empty(((outputs + 127) // 128, inner // 128), dtype=np.float32)
    lib().oracle_fp8_quantize_weight(outputs, inner, _ptr(np.ascontiguousarray(w)), _ptr(q),
                                     _ptr(scale))
    return q, scale


def fp8_block_gemm(q, q_scale, w, w_scale):
    """Block-128 product with per-block promotion -> uint16 BF16 [rows, outputs]."""
    rows, inner = q.shape
    outputs = w.shape[0]
    out = np.empty((rows, outputs), dtype=np.uint16)
    lib().oracle_fp8_block_gemm(rows, outputs, inner, _ptr(q), _ptr(q_scale), _ptr(w),
                                _ptr(w_scale), _ptr(out), outputs)
    return out


def fp8_dequantize(q, scale, block_rows):
    """E4M3 * block scale -> FP32; block_rows is 1 for activations, 128 for weights."""
    rows, inner = q.shape
    out = np.empty((rows, inner), dtype=np.float32)
    lib().oracle_fp8_dequantize(rows, inner, block_rows, _ptr(q), _ptr(scale), _ptr(out))
    return out


def fp8_quantize_block32(x):
    """Power-of-two block-32 quantiser on a uint16 BF16 vector."""
    inner = x.size
    q = np.empty(inner, dtype=np.uint8)
    scale = np.empty(inner // 32, dtype=np.float32)
    lib().oracle_fp8_quantize_block32(inner, _ptr(x), _ptr(q), _ptr(scale))
    return q, scale


def fp8_decode(x, sx, w, sw):
    """Single-token block-32 product with ordered FP32 accumulation."""
    outputs, inner = w.shape
    out = np.empty(outputs, dtype=np.uint16)
    lib().oracle_fp8_decode(outputs, inner, _ptr(x), _ptr(sx), sx.strides[-1] // 4, _ptr(w),
                            _ptr(sw), sw.strides[0] // 4, sw.strides[1] // 4, _ptr(out))
    return out


def strassen_bf16(a, b, alpha=1.0, beta=0.0, c=None):
    """One-level Strassen on column-major uint16 BF16 squares (Fortran-ordered arrays)."""
    n = a.shape[0]
    if c is None:
        c = np.zeros((n, n), dtype=np.uint16, order="F")
    work = np.empty(21 * (n // 2) ** 2, dtype=np.float32)
    lib().oracle_strassen_bf16(n, alpha, _ptr(a), a.strides[1] // 2, _ptr(b), b.strides[1] // 2,
                               beta, _ptr(c), c.strides[1] // 2, _ptr(work))
    return c


def rel_l2(actual, expected):
    """Relative L2 error of two real arrays, in double."""
    actual = np.asarray(actual, dtype=np.float64)
    expected = np.asarray(expected, dtype=np.float64)
    denominator = np.linalg.norm(expected)
    return float(np.linalg.norm(actual - expected) / (denominator if denominator else 1.0))
