"""Load libcamblas_cuda.so, declare its C ABI and keep one context per stream.

The public behaviour is that of ``camblas/_native.py`` in the reference: the
same algorithm table and counter names (``_native.py:17-37``), the
``CAMBLAS_CUDA_LIBRARY`` override (``:48, 84-88``), one native context per host
thread, device and stream (``:247-275``), a per-thread multiplication policy
(``:299-357``) and ``stats`` (``:360-414``). There is no separate compiled
tensor binding: tensors reach the library as raw device pointers through
ctypes.

Organisation. What a host thread has chosen (policy, kernel family, option
values) lives in one ``_Selection`` per thread; a ``Context`` remembers which
of those it has already passed to the native side and forwards only the
differences; every live context of the process is listed in ``_REGISTRY`` so
that ``close`` and ``stats(all_threads=True)`` can reach contexts of other
threads.
"""

import atexit
import ctypes as ct
import os
import threading
from contextlib import contextmanager
from functools import lru_cache
from pathlib import Path

import torch

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
    "set_option": ([_P, ct.c_char_p, _I], _I),
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
    "gate_up_swiglu_fp8": ([_P, _I, _I, _I, _P, _I, _P, _I, _P, _P], _I),
    "peer_bytes": ([_I, ct.c_size_t], ct.c_size_t),
    "peer_alloc": ([_P, ct.c_size_t, ct.POINTER(_P), _P], _I),
    "peer_open": ([_P, _P, ct.POINTER(_P)], _I),
    "peer_close": ([_P, _P], _I),
    "peer_free": ([_P, _P], _I),
    "peer_reset": ([_P, _P, _I, ct.c_size_t], _I),
    "peer_allreduce_bf16": ([_P, _I, _I, ct.c_size_t, ct.POINTER(_P), _I, ct.c_size_t, _P, _P], _I),
    "linear_bf16_allreduce": (
        [_P, _I, _I, ct.c_size_t, ct.POINTER(_P), _I, _I, _I, _I, _P, _I, _P, _I, _P, _P, _I],
        _I,
    ),
    "qkv_linear_bf16": ([_P, _I, _I, _I, _I, _I, _P, _I, _P, _I, _P, _I, _P, _I, _P, _I], _I),
    "rms_norm": ([_P, _I, _I, _I, _F, _P, _P, _P], _I),
    "rms_norm_decode": ([_P, _I, _I, _I, _F, _I, _I, _P, _P, _P], _I),
    "add_rms_norm": ([_P, _I, _I, _F, _P, _P, _P, _P, _P], _I),
    "add_rms_norm_rows": ([_P, _I, _I, _I, _F, _P, _P, _P, _P, _P], _I),
    "add_rms_norm_strided": ([_P, _I, _I, _I, _F, _P, ct.c_longlong, _P, ct.c_longlong, _P, _P,
                              ct.c_longlong, _P, ct.c_longlong], _I),
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


class _Selection(threading.local):
    """What the calling host thread has asked for; every thread starts from the defaults."""

    def __init__(self):
        self.policy = "auto"
        self.family = "auto"
        self.options = {}
        self.contexts = {}


_SELECTION = _Selection()


class _Registry:
    """Every live native context of this process, whichever thread made it."""

    def __init__(self):
        self._guard = threading.Lock()
        self._members = []

    def add(self, native):
        with self._guard:
            self._members.append(native)

    def live(self, device=None):
        """Snapshot of the open contexts of this process (optionally of one device)."""
        me = os.getpid()
        with self._guard:
            return [native for native in self._members
                    if native.handle and native.pid == me
                    and (device is None or native.device == device)]

    def drain(self):
        """Remove and return every member."""
        with self._guard:
            members, self._members = self._members, []
        return members


_REGISTRY = _Registry()


class Context:
    """Own one native context: one device, one stream, one host thread."""

    def __init__(self, device, stream):
        self.pid = os.getpid()
        self.device = device
        self.stream = stream
        self.handle = _P()
        _check(library().camblas_cuda_create(device, stream, ct.byref(self.handle)), None)
        # what the native side currently holds, so that unchanged settings cost nothing
        self._sent = {"policy": "auto", "family": "auto"}
        _REGISTRY.add(self)

    def _forward(self, key, value, entry, argument):
        if self._sent.get(key) != value:
            _check(getattr(library(), "camblas_cuda_" + entry)(self.handle, *argument), self.handle)
            self._sent[key] = value

    def set_algorithm(self, name):
        """Select the multiplication policy of this context by name."""
        self._forward("policy", name, "set_algorithm", (_ALGORITHMS[name],))

    def force_kernel(self, family):
        """Pin the BF16 kernel family (see ``camblas_cuda_force_kernel``)."""
        self._forward("family", family, "force_kernel", (_FAMILIES[family],))

    def set_option(self, name, value):
        """Set one named switch of the context (see ``camblas_cuda_set_option``)."""
        self._forward("option:" + name, int(value), "set_option", (name.encode(), int(value)))

    def adopt(self, selection):
        """Bring the native side in line with the calling thread's selection."""
        self.set_algorithm(selection.policy)
        self.force_kernel(selection.family)
        for name, value in selection.options.items():
            self.set_option(name, value)

    def call(self, name, *arguments):
        """Call ``camblas_cuda_<name>(handle, *arguments)`` and check its status."""
        _check(getattr(library(), "camblas_cuda_" + name)(self.handle, *arguments), self.handle)

    def counters(self, reset=False):
        """Return the eight launch counters as a tuple (optionally clearing them)."""
        counts = (_U64 * len(_COUNTERS))()
        _check(library().camblas_cuda_stats(self.handle, counts, len(_COUNTERS)), self.handle)
        if reset:
            _check(library().camblas_cuda_reset_stats(self.handle), self.handle)
        return tuple(counts)

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

    def release(self):
        """Destroy the native context (waits for its stream)."""
        if self.handle and self.pid == os.getpid():
            library().camblas_cuda_destroy(self.handle)
        self.handle = _P()


def context(device):
    """Return this thread's context for ``device`` and its current stream.

    A context is created on first use; creation is refused while the stream is
    being captured (``camblas/_native.py:262-266`` in the reference), and a
    context made before a ``fork`` is refused in the child (``:270-271``).
    """
    stream = torch.cuda.current_stream(device).cuda_stream
    native = _SELECTION.contexts.get((device, stream))
    if native is not None and native.pid != os.getpid():
        raise RuntimeError("CUDA contexts cannot be reused after fork; use spawn")
    if native is None or not native.handle:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("Warm up CAMBLAS on this stream before CUDA graph capture")
        native = _SELECTION.contexts[(device, stream)] = Context(device, stream)
    native.adopt(_SELECTION)
    return native


def close():
    """Destroy every native context of this process after its stream drains."""
    if not library.cache_info().currsize:
        return
    for native in _REGISTRY.drain():
        native.release()
    _SELECTION.contexts.clear()


atexit.register(close)


def _known(table, kind, name):
    if name not in table:
        raise ValueError(f"Unknown {kind} {name!r}; choose {tuple(table)}")
    return name


@contextmanager
def algorithm(name):
    """Select a multiplication policy for the calling thread within a block."""
    previous, _SELECTION.policy = _SELECTION.policy, _known(_ALGORITHMS, "algorithm", name)
    try:
        yield
    finally:
        _SELECTION.policy = previous


def set_algorithm(name):
    """Select the multiplication policy for the calling thread."""
    _SELECTION.policy = _known(_ALGORITHMS, "algorithm", name)


@contextmanager
def kernel_family(name):
    """Pin the BF16 kernel family for the calling thread within a block."""
    previous, _SELECTION.family = _SELECTION.family, _known(_FAMILIES, "kernel family", name)
    try:
        yield
    finally:
        _SELECTION.family = previous


_OPTION_DEFAULTS = {"pair_tail": 0, "pair_width": 0, "push_width": 0, "fp8_rows": 0,
                    "fp8_swapped_rows": 16, "cluster_split": 1,
                    "bf16_strassen": 0, "peer_wait_ms": 5000}


@contextmanager
def options(**values):
    """Set named context switches for the calling thread within a block.

    The names are those of ``camblas_cuda_set_option`` (``pair_tail``,
    ``pair_width``, ``push_width``, ``fp8_rows``, ``bf16_strassen``,
    ``peer_wait_ms``). On leaving the block a switch returns to the value it
    had before, or to its library default if the thread had not set it.
    """
    for name in values:
        _known(_OPTION_DEFAULTS, "option", name)
    before = dict(_SELECTION.options)
    _SELECTION.options.update({name: int(value) for name, value in values.items()})
    try:
        yield
    finally:
        restored = {name: before.get(name, _OPTION_DEFAULTS[name]) for name in values}
        _SELECTION.options = {**before, **restored}


def stats(device=None, reset=False, all_threads=False):
    """Read the eight launch counters for a device.

    Returns a dict keyed by the reference's counter names. Graph replays do not
    move the counters; they count launches issued by the host. With
    ``all_threads`` the counters of every context of the process on that device
    are added up, otherwise only those of the calling thread's current stream.
    """
    if device is None:
        index = torch.cuda.current_device()
    elif isinstance(device, int):
        index = device
    else:
        index = torch.device(device).index
        if index is None:
            index = torch.cuda.current_device()
    sources = _REGISTRY.live(index) if all_threads else [context(index)]
    totals = [0] * len(_COUNTERS)
    for native in sources:
        totals = [a + b for a, b in zip(totals, native.counters(reset))]
    return dict(zip(_COUNTERS, totals))
