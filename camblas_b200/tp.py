"""Tensor-parallel linear layers over ``torch.distributed``.

The reference has no distributed code: in its published runs the tensor
parallelism comes from SGLang (``configs/sglang.json:8`` ``tp_size``), whose
Column/RowParallel linear layers call the hooked ``F.linear`` on each rank's
shard (``camblas/sglang.py:250-285``). These classes are that arrangement for
one process per GPU:

* column parallel (QKV, gate_up): the weight is split by output rows, every
  rank holds ``[outputs/tp, inner]`` and the activations are replicated; there
  is no communication and each rank returns its slice of the outputs;
* row parallel (down projection): the weight is split along the inner
  dimension, rank ``r`` multiplies its ``[rows, inner/tp]`` slice of the
  activations and the BF16 partial results are summed with one all-reduce on
  the stream the GEMM ran on.

``linear`` is the GEMM each rank runs; it defaults to the CUDA kernels of this
package. The CPU tests drive the same classes over the ``gloo`` backend with a
host matmul passed in, which exercises the sharding arithmetic and the
collective without a GPU.

``PeerRegions`` is the alternative to the all-reduce for the row-parallel
layer on GPUs of one machine: the product's epilogue writes its partial tiles
straight into the memory of the GPU that sums them, and that GPU writes the
finished tiles into every GPU's result buffer
(``camblas_cuda_linear_bf16_allreduce``). Pass one to ``RowParallelLinear``.
"""

import ctypes as ct

import torch
import torch.distributed as dist


def _default_linear(x, weight, bias=None, residual=None):
    from . import _kernels

    return _kernels.linear(x, weight, bias, residual)


def shard_bounds(extent, rank, world, multiple=1):
    """Return ``(start, stop)`` of rank's contiguous share of ``extent``.

    ``extent`` must divide into ``world`` shares that are multiples of
    ``multiple`` (for example 128 so FP8 scale blocks never straddle ranks).
    """
    if extent % (world * multiple) != 0:
        raise ValueError(f"{extent} does not split into {world} shares of multiples of {multiple}")
    share = extent // world
    return rank * share, (rank + 1) * share


def shard_qkv(weight, q_heads, kv_heads, head_dim, rank, world):
    """Rows of a packed ``[q|k|v]`` projection that belong to ``rank``.

    Whole heads stay together: every rank gets ``q_heads/world`` query heads
    and ``kv_heads/world`` key and value heads, packed again as ``[q|k|v]``.
    Returns ``(weight_shard, (q_out, k_out, v_out))``.
    """
    if q_heads % world or kv_heads % world:
        raise ValueError("head counts must be divisible by the tensor-parallel size")
    q_rows, kv_rows = q_heads * head_dim, kv_heads * head_dim
    if weight.shape[0] != q_rows + 2 * kv_rows:
        raise ValueError("weight rows do not match the head layout")
    q0, q1 = shard_bounds(q_rows, rank, world, head_dim)
    k0, k1 = shard_bounds(kv_rows, rank, world, head_dim)
    parts = [weight[q0:q1], weight[q_rows + k0:q_rows + k1],
             weight[q_rows + kv_rows + k0:q_rows + kv_rows + k1]]
    return torch.cat(parts, dim=0).contiguous(), (q1 - q0, k1 - k0, k1 - k0)


class _DeviceWords:
    """Expose raw device memory to ``torch.as_tensor`` as 16-bit words."""

    def __init__(self, pointer, count):
        self.__cuda_array_interface__ = {
            "shape": (count,), "typestr": "<i2", "data": (pointer, False), "version": 2,
        }


class PeerRegions:
    """The peer regions of one tensor-parallel group, seen from one rank.

    Every rank owns a region that holds the result, one staging slot per rank
    and flag words (``include/camblas_cuda.h``); ``memory[r]`` is rank ``r``'s
    region as mapped here. ``capacity`` bounds ``rows * outputs`` of a call, both
    rounded up to multiples of 256 (``capacity_for``).

    Use ``PeerRegions.create`` with one process per GPU (regions are exchanged
    as CUDA IPC handles through ``all_gather_object``), or
    ``PeerRegions.emulate`` to get all ranks' views in one process on one GPU,
    which is how the single-GPU tests drive the kernels.
    """

    @staticmethod
    def capacity_for(rows, outputs):
        """Capacity that fits calls of up to ``rows`` x ``outputs``: staging holds whole
        256 x 256 tiles, so both extents count rounded up to multiples of 256."""
        return (-(-rows // 256) * 256) * (-(-outputs // 256) * 256)

    def __init__(self, device, rank, world, capacity, memory, owned, opened):
        self.device, self.rank, self.world, self.capacity = device, rank, world, capacity
        self.memory = list(memory)
        self._owned, self._opened = owned, list(opened)
        self._array = (ct.c_void_p * world)(*self.memory)

    @staticmethod
    def _native(device):
        from . import _native

        with torch.cuda.device(device):
            return _native.context(device)

    @classmethod
    def create(cls, capacity, device, group=None):
        """Allocate this rank's region and map every other rank's (collective)."""
        from . import _native

        rank, world = dist.get_rank(group), dist.get_world_size(group)
        native = cls._native(device)
        size = _native.library().camblas_cuda_peer_bytes(world, capacity)
        if size == 0:
            raise ValueError("peer regions support 1 to 8 ranks and a non-zero capacity")
        # Failures are collected and agreed on by all ranks, so that no rank is
        # left alone in a collective when another could not map a region.
        own, handle, failure = ct.c_void_p(), ct.create_string_buffer(64), None
        try:
            native.call("peer_alloc", size, ct.byref(own), handle)
        except RuntimeError as error:
            failure = str(error)
        handles = [None] * world
        dist.all_gather_object(handles, None if failure else handle.raw, group=group)
        memory, opened = [], []
        for r in range(world):
            if r == rank:
                memory.append(own.value)
                continue
            mapped = ct.c_void_p()
            if failure is None and handles[r] is not None:
                try:
                    native.call("peer_open", ct.create_string_buffer(handles[r], 64),
                                ct.byref(mapped))
                    opened.append(mapped.value)
                except RuntimeError as error:
                    failure = str(error)
            memory.append(mapped.value)
        failures = [None] * world
        dist.all_gather_object(failures, failure, group=group)
        regions = cls(device, rank, world, capacity, memory, own.value, opened)
        if any(handle_bytes is None for handle_bytes in handles) or any(failures):
            regions.close()
            reasons = [text for text in failures if text] or ["a rank could not allocate its region"]
            raise RuntimeError("peer regions could not be set up: " + reasons[0])
        return regions

    @classmethod
    def emulate(cls, capacity, world, device):
        """Return the views of all ``world`` ranks with every region on ``device``."""
        from . import _native

        native = cls._native(device)
        size = _native.library().camblas_cuda_peer_bytes(world, capacity)
        if size == 0:
            raise ValueError("peer regions support 1 to 8 ranks and a non-zero capacity")
        memory = []
        for _ in range(world):
            own = ct.c_void_p()
            native.call("peer_alloc", size, ct.byref(own), None)
            memory.append(own.value)
        return [cls(device, r, world, capacity, memory, memory[r], []) for r in range(world)]

    def result(self, rows, outputs):
        """View the first ``rows * outputs`` elements of this rank's result buffer."""
        words = torch.as_tensor(_DeviceWords(self._owned, rows * outputs),
                                device=torch.device("cuda", self.device))
        return words.view(torch.bfloat16).view(rows, outputs)

    def linear(self, x, weight, bias=None, residual=None, phases=7):
        """Enqueue ``sum_r x_r @ weight_r.T (+ bias + residual)``; return the result view.

        ``x`` ``[rows, inner/world]`` and ``weight`` ``[outputs, inner/world]``
        are this rank's slices. The returned tensor aliases the region: use it
        (on the same stream) before the next call overwrites it.
        """
        if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
            raise ValueError("the peer row-parallel product takes BF16 operands")
        if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1]:
            raise ValueError("expected x [rows, inner] and weight [outputs, inner]")
        rows, inner, outputs = x.shape[0], x.shape[1], weight.shape[0]
        x2 = x if x.stride(1) == 1 else x.contiguous()
        w2 = weight if weight.stride(1) == 1 else weight.contiguous()
        r2 = None
        if residual is not None:
            r2 = residual if residual.stride(-1) == 1 else residual.contiguous()
        native = self._native(self.device)
        native.call("linear_bf16_allreduce", self.rank, self.world, self.capacity, self._array,
                    phases, rows, inner, outputs, x2.data_ptr(),
                    x2.stride(0) if rows > 1 else inner, w2.data_ptr(), w2.stride(0),
                    bias.data_ptr() if bias is not None else None,
                    r2.data_ptr() if r2 is not None else None,
                    (r2.stride(0) if rows > 1 else outputs) if r2 is not None else 0)
        return self.result(rows, outputs)

    def all_reduce(self, tensor, out=None, phases=3):
        """Sum a small contiguous BF16 tensor over the ranks; returns the sum (``out`` or new).

        One kernel per rank over peer memory (``camblas_cuda_peer_allreduce_bf16``):
        FP32 sum in rank order, one rounding, identical bits on every rank. The
        element count must be a multiple of 8 and fit the regions' capacity.
        """
        if tensor.dtype != torch.bfloat16 or not tensor.is_contiguous():
            raise ValueError("the peer all-reduce takes a contiguous BF16 tensor")
        if tensor.numel() % 8 or tensor.numel() > self.capacity:
            raise ValueError("element count must be a multiple of 8 within the region capacity")
        if out is None:
            out = torch.empty_like(tensor)
        native = self._native(self.device)
        native.call("peer_allreduce_bf16", self.rank, self.world, self.capacity, self._array, phases,
                    tensor.numel(), tensor.data_ptr(), out.data_ptr())
        return out

    def reset(self):
        """Clear this rank's flag words (after a failed call; all ranks idle)."""
        self._native(self.device).call("peer_reset", self._owned, self.world, self.capacity)

    def close(self, free=True):
        """Unmap the other ranks' regions and, with ``free``, release this rank's."""
        native = self._native(self.device)
        for mapped in self._opened:
            native.call("peer_close", mapped)
        self._opened = []
        if free and self._owned:
            native.call("peer_free", self._owned)
            self._owned = None


class ColumnParallelLinear:
    """``y_r = x @ W_r^T`` with ``W_r`` the rank's block of output rows; no communication."""

    def __init__(self, weight, rank, world, bias=None, linear=None, multiple=1):
        start, stop = shard_bounds(weight.shape[0], rank, world, multiple)
        self.weight = weight[start:stop].contiguous()
        self.bias = bias[start:stop].contiguous() if bias is not None else None
        self.bounds = (start, stop)
        self.linear = linear or _default_linear

    def __call__(self, x):
        return self.linear(x, self.weight, self.bias)


class RowParallelLinear:
    """``y = sum_r x[:, K_r] @ W[:, K_r]^T`` with one all-reduce of the BF16 partials.

    The bias, if any, is added by rank 0 only so that it enters the sum once.
    ``group`` is the process group of the tensor-parallel ranks. With ``peers``
    (a ``PeerRegions``) the all-reduce is replaced by the product kernel
    writing its tiles into peer memory; the result then aliases the peer region.
    """

    def __init__(self, weight, rank, world, bias=None, linear=None, group=None, multiple=8,
                 peers=None):
        start, stop = shard_bounds(weight.shape[1], rank, world, multiple)
        self.weight = weight[:, start:stop].contiguous()
        self.full_bias = bias
        self.bias = bias if (bias is not None and rank == 0) else None
        self.bounds = (start, stop)
        self.world = world
        self.group = group
        self.linear = linear or _default_linear
        self.peers = peers

    def slice_input(self, x):
        """Return the rank's columns of a replicated activation tensor."""
        return x[..., self.bounds[0]:self.bounds[1]].contiguous()

    # Below this many token rows the product is a weight-streaming kernel (GEMV or
    # swapped tcgen05) and the payload of the sum is at most 1 MB: the partial results
    # meet in the one-shot peer all-reduce. From here on the peer-memory path multiplies
    # with 256-row tiles and exchanges them from the GEMM epilogue, which is what
    # prefill needs.
    PEER_ROWS = 65

    def __call__(self, x_local):
        rows = x_local.numel() // x_local.shape[-1]
        if self.peers is not None and rows >= self.PEER_ROWS:
            # product and sum in one sequence of kernels over peer memory; the
            # bias enters once, on the rank that sums each tile
            return self.peers.linear(x_local.reshape(-1, x_local.shape[-1]), self.weight,
                                     self.full_bias)
        partial = self.linear(x_local, self.weight, self.bias)
        if self.world > 1:
            if (self.peers is not None and partial.dtype == torch.bfloat16 and partial.is_cuda
                    and partial.numel() % 8 == 0 and partial.numel() <= self.peers.capacity):
                return self.peers.all_reduce(partial, out=partial)
            dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.group)
        return partial
