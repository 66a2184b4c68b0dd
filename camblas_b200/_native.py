"""Load libcamblas_cuda.so, declare its C ABI and keep one context per stream.

Mirrors ``camblas/_native.py`` of the reference: the same algorithm table and
counter names (``_native.py:17-37``), the ``CAMBLAS_CUDA_LIBRARY`` override
(``:48, 84-88``), one native context per host thread, device and stream
(``:247-275``), a thread-local algorithm (``:299-357``) and ``stats``
(``:360-414``). There is no separate compiled tensor binding: tensors reach
the library as raw device pointers through ctypes.
"""

import atexit
import ctypes as ct
import os
import threading
from contextlib import contextmanager
from functools import lru_cache
from pathlib import Path

import torch

_LOCAL = threading.local()
_CONTEXTS = []
_LOCK = threading.Lock()
_ALGORITHMS = {
    "auto": 0,
    "classical": 1,
    "strassen": 2,
    "lt": 3,
    "symmetric": 4,
    "strassen2": 5,
    "strassen3": 6,
    "strassen4": 7,
}
_COUNTERS = (
    "classical",
    "strassen",
    "gram",
    "affine",
    "lt",
    "guard_fallback",
    "attention",
    "backward",
)
_FAMILIES = {"auto": 0, "generic": 1, "skinny": 2, "tensor": 3, "tensor_swapped": 4,
             "tensor_pair": 5}

_P = ct.c_void_p
_I = ct.c_int
_F = ct.c_float
_U64 = ct.c_uint64
_FP = ct.POINTER(ct.c_float)

# name -> (argument types after the context, result type); the context pointer
# is always the first argument except where noted.
_SIGNATURES = {
    "create": ([_I, _P, ct.POINTER(_P)], _I),
    "destroy": ([_P], _I),
    "error": ([_P], ct.c_char_p),
    "set_algorithm": ([_P, _I], _I),
    "stats": ([_P, ct.POINTER(_U64), _I], _I),
    "reset_stats": ([_P], _I),
    "device_status": ([_P, ct.POINTER(ct.c_uint)], _I),
    "force_kernel": ([_P, _I], _I),
    "kernel_launches": ([_P, ct.POINTER(_U64)], _I),
    "bgemm": ([_P, ct.c_char, ct.c_char, _I, _I, _I, _F, _P, _I, _P, _I, _F, _P, _I], _I),
    "sgemm": ([_P, ct.c_char, ct.c_char, _I, _I, _I, _F, _P, _I, _P, _I, _F, _P, _I], _I),
    "dgemm": (
        [_P, ct.c_char, ct.c_char, _I, _I, _I, ct.c_double, _P, _I, _P, _I, ct.c_double, _P, _I],
        _I,
    ),
    "linear_bf16": ([_P, _I, _I, _I, _P, _I, _P, _I, _P, _P, _I, _P, _I], _I),
    "linear_bf16_static": ([_P, _I, _I, _I, _P, _I, _P, _I, _P, _I], _I),
    "gate_up_swiglu_bf16": ([_P, _I, _I, _I, _P, _I, _P, _I, _P, _I], _I),
    "peer_bytes": ([_I, ct.c_size_t], ct.c_size_t),
    "peer_alloc": ([_P, ct.c_size_t, ct.POINTER(_P), _P], _I),
    "peer_open": ([_P, _P, ct.POINTER(_P)], _I),
    "peer_close": ([_P, _P], _I),
    "peer_free": ([_P, _P], _I),
    "peer_reset": ([_P, _P, _I, ct.c_size_t], _I),
    "linear_bf16_allreduce": (
        [_P, _I, _I, ct.c_size_t, ct.POINTER(_P), _I, _I, _I, _I, _P, _I, _P, _I, _P, _P, _I],
        _I,
    ),
    "qkv_linear_bf16": ([_P, _I, _I, _I, _I, _I, _P, _I, _P, _I, _P, _I, _P, _I, _P, _I], _I),
    "rms_norm": ([_P, _I, _I, _I, _F, _P, _P, _P], _I),
    "rms_norm_decode": ([_P, _I, _I, _I, _F, _I, _I, _P, _P, _P], _I),
    "add_rms_norm": ([_P, _I, _I, _F, _P, _P, _P, _P, _P], _I),
    "add_rms_norm_rows": ([_P, _I, _I, _I, _F, _P, _P, _P, _P, _P], _I),
    "bfloat16_square": ([_P, _U64, _P, _P], _I),
    "rms_scale": ([_P, _I, _U64, _I, _F, _P, _P, _P, _P], _I),
    "silu_multiply": ([_P, _I, _U64, _P, _P, _P], _I),
    "swiglu": ([_P, _I, _U64, _I, _F, _P, _P, _P, _P], _I),
    "fp8_quantize_rows": ([_P, _I, _I, _P, _I, _P, _P], _I),
    "fp8_block_gemm": ([_P, _I, _I, _I, _P, _P, _P, _P, _P, _I], _I),
    "fp8_decode_supported": ([_P], _I),
    "fp8_decode": ([_P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _P, ct.c_size_t, _P], _I),
    "fp8_workspace_size": ([_I, _I, _I], ct.c_size_t),
    "fp8_linear": ([_P, _I, _I, _P, _P, _P, _I, _I, _P, ct.c_size_t, _P], _I),
    "affine": ([_P, _I, _I, _I, _I, _P, _P, _P, _I, _P], _I),
    "mlp": ([_P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P], _I),
    "attention": ([_P, _I, _I, _I, _I, _I, ct.c_double, _P, _P, _P, _P], _I),
    "mlp_backward": ([_P, _I, _I, _I, _I, _I] + [_P] * 11, _I),
    "quantized_matmul": ([_P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P], _I),
    "grouped_quantized_matmul": ([_P, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P], _I),
    "route_groups": ([_P, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P], _I),
    "reduce_groups": ([_P, _I, _I, _I, _I, _P, _P, _P, _P], _I),
}

EXPORTED = tuple("camblas_cuda_" + name for name in _SIGNATURES)


def library_path():
    """Return the path the C ABI is loaded from.

    ``CAMBLAS_CUDA_LIBRARY`` overrides the in-tree ``libcamblas_cuda.so``.
    """
    return Path(
        os.environ.get("CAMBLAS_CUDA_LIBRARY", Path(__file__).resolve().parent / "libcamblas_cuda.so")
    )


@lru_cache(maxsize=1)
def library():
    """Load the CUDA C ABI once per process and declare every entry point.

    Raises
    ------
    RuntimeError
        If the library has not been built. There is no fallback path: without
        the compiled kernels no operation of this package works.
    """
    path = library_path()
    if not path.is_file():
        raise RuntimeError(
            f"libcamblas_cuda.so is missing ({path}); run `python -m camblas_b200.build`"
        )
    lib = ct.CDLL(str(path))
    for name, (arguments, result) in _SIGNATURES.items():
        function = getattr(lib, "camblas_cuda_" + name)
        function.argtypes = arguments
        function.restype = result
    return lib


def _check(status, handle):
    """Raise ``RuntimeError`` with the native message when status is non-zero."""
    if status:
        raise RuntimeError(library().camblas_cuda_error(handle).decode())


class Context:
    """Own one native context: one device, one stream, one host thread."""

    def __init__(self, device, stream):
        self.pid = os.getpid()
        self.device = device
        self.stream = stream
        self.handle = _P()
        _check(library().camblas_cuda_create(device, stream, ct.byref(self.handle)), None)
        self.algorithm = "auto"
        self.family = "auto"
        with _LOCK:
            _CONTEXTS.append(self)

    def set_algorithm(self, name):
        """Select the multiplication policy of this context by name."""
        if name != self.algorithm:
            _check(
                library().camblas_cuda_set_algorithm(self.handle, _ALGORITHMS[name]), self.handle
            )
            self.algorithm = name

    def force_kernel(self, family):
        """Pin the BF16 kernel family (see ``camblas_cuda_force_kernel``)."""
        if family != self.family:
            _check(library().camblas_cuda_force_kernel(self.handle, _FAMILIES[family]), self.handle)
            self.family = family

    def call(self, name, *arguments):
        """Call ``camblas_cuda_<name>(handle, *arguments)`` and check its status."""
        _check(getattr(library(), "camblas_cuda_" + name)(self.handle, *arguments), self.handle)

    def kernel_launches(self):
        """Return how many CUDA kernels this context has enqueued so far."""
        count = _U64(0)
        _check(library().camblas_cuda_kernel_launches(self.handle, ct.byref(count)), self.handle)
        return count.value

    def device_status(self):
        """Wait for the stream and return (then clear) the device status word."""
        word = ct.c_uint(0)
        _check(library().camblas_cuda_device_status(self.handle, ct.byref(word)), self.handle)
        return word.value


def context(device):
    """Return this thread's context for ``device`` and its current stream.

    A context is created on first use; creation is refused while the stream is
    being captured (``camblas/_native.py:262-266`` in the reference).
    """
    if not hasattr(_LOCAL, "contexts"):
        _LOCAL.contexts = {}
    stream = torch.cuda.current_stream(device)
    key = (device, stream.cuda_stream)
    native = _LOCAL.contexts.get(key)
    if native is None or not native.handle:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("Warm up CAMBLAS on this stream before CUDA graph capture")
        native = Context(device, stream.cuda_stream)
        _LOCAL.contexts[key] = native
    if native.pid != os.getpid():
        raise RuntimeError("CUDA contexts cannot be reused after fork; use spawn")
    native.set_algorithm(getattr(_LOCAL, "algorithm", "auto"))
    native.force_kernel(getattr(_LOCAL, "family", "auto"))
    return native


def close():
    """Destroy every native context of this process after its stream drains."""
    if not library.cache_info().currsize:
        return
    with _LOCK:
        for native in _CONTEXTS:
            if native.handle and native.pid == os.getpid():
                library().camblas_cuda_destroy(native.handle)
                native.handle = _P()
        _CONTEXTS.clear()
    if hasattr(_LOCAL, "contexts"):
        _LOCAL.contexts.clear()


atexit.register(close)


@contextmanager
def algorithm(name):
    """Select a multiplication policy for the calling thread within a block."""
    if name not in _ALGORITHMS:
        raise ValueError(f"Unknown algorithm {name!r}; choose {tuple(_ALGORITHMS)}")
    previous = getattr(_LOCAL, "algorithm", "auto")
    _LOCAL.algorithm = name
    try:
        yield
    finally:
        _LOCAL.algorithm = previous


def set_algorithm(name):
    """Select the multiplication policy for the calling thread."""
    if name not in _ALGORITHMS:
        raise ValueError(f"Unknown algorithm {name!r}; choose {tuple(_ALGORITHMS)}")
    _LOCAL.algorithm = name


@contextmanager
def kernel_family(name):
    """Pin the BF16 kernel family for the calling thread within a block."""
    if name not in _FAMILIES:
        raise ValueError(f"Unknown kernel family {name!r}; choose {tuple(_FAMILIES)}")
    previous = getattr(_LOCAL, "family", "auto")
    _LOCAL.family = name
    try:
        yield
    finally:
        _LOCAL.family = previous


def stats(device=None, reset=False, all_threads=False):
    """Read the eight launch counters for a device.

    Returns a dict keyed by the reference's counter names. Graph replays do not
    move the counters; they count launches issued by the host.
    """
    if device is None:
        device = torch.cuda.current_device()
    elif not isinstance(device, int):
        device = torch.device(device).index
        if device is None:
            device = torch.cuda.current_device()
    lib = library()
    if all_threads:
        totals = dict.fromkeys(_COUNTERS, 0)
        with _LOCK:
            for native in _CONTEXTS:
                if native.device != device or native.pid != os.getpid() or not native.handle:
                    continue
                counts = (_U64 * 8)()
                _check(lib.camblas_cuda_stats(native.handle, counts, 8), native.handle)
                for name, count in zip(_COUNTERS, counts):
                    totals[name] += count
                if reset:
                    _check(lib.camblas_cuda_reset_stats(native.handle), native.handle)
        return totals
    native = context(device)
    counts = (_U64 * 8)()
    _check(lib.camblas_cuda_stats(native.handle, counts, 8), native.handle)
    if reset:
        _check(lib.camblas_cuda_reset_stats(native.handle), native.handle)
    return dict(zip(_COUNTERS, counts))
