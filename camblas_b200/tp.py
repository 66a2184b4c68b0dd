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
"""

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
    ``group`` is the process group of the tensor-parallel ranks.
    """

    def __init__(self, weight, rank, world, bias=None, linear=None, group=None, multiple=8):
        start, stop = shard_bounds(weight.shape[1], rank, world, multiple)
        self.weight = weight[:, start:stop].contiguous()
        self.bias = bias if (bias is not None and rank == 0) else None
        self.bounds = (start, stop)
        self.world = world
        self.group = group
        self.linear = linear or _default_linear

    def slice_input(self, x):
        """Return the rank's columns of a replicated activation tensor."""
        return x[..., self.bounds[0]:self.bounds[1]].contiguous()

    def __call__(self, x_local):
        partial = self.linear(x_local, self.weight, self.bias)
        if self.world > 1:
            dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.group)
        return partial
