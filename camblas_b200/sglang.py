"""SGLang plugin: the ``linear`` and ``fp8`` operations behind SGLang's hook registry.

Mirrors ``camblas/sglang.py:199-747`` of the reference for the dense path:

* ``install()`` is the ``sglang.srt.plugins`` entry point. ``CAMBLAS_SGLANG_OPS``
  selects a subset of ``linear,fp8`` (anything else raises ``ValueError``);
  ``CAMBLAS_SGLANG_ALGORITHM`` (default ``lt``) names the GEMM policy.
* ``linear``: an AROUND hook on ``UnquantizedLinearMethod.apply``; eligible calls
  (CUDA, BF16, contiguous, same device and dtype, no gradient) go through
  ``F.linear`` under the ATen overrides, everything else through the original.
* ``linear`` also hooks ``ColumnParallelBatchedLinear.forward`` (``sglang.py:294-336``):
  a batched BF16 projection ``[batch, rows, inner] x [batch, outputs, inner]`` runs
  as one GEMM per batch entry. The reference takes exactly the shape
  ``(2, 1, 128) x (2, 2048, 128)`` on Hopper with its Gluon kernel; here any
  contiguous BF16 shape of that form is taken.
* ``fp8``: AROUND hooks on the block-128 dense entry point, the block-32
  pre-quantised product and the block-32 BF16-input linear. The block-128 hook
  takes any number of token rows (the reference takes one row and a fixed list
  of eleven shapes, ``sglang.py:458-470``).

The expert-parallel hooks of the reference (``fused_experts``, the stable MoE
ordering) are not part of the dense GEMM path and are not installed. Every hook returns ``original(...)`` for inputs it does not
take, and counts what it does take in ``dispatch_counts()``.
"""

import os

_calls = {}


def dispatch_counts():
    """Return a copy of the per-operation host dispatch counts of this process."""
    return dict(_calls)


def _count(name):
    _calls[name] = _calls.get(name, 0) + 1


def install():
    """Register the selected operations with SGLang's ``HookRegistry``."""
    selected = set(filter(None, os.environ.get("CAMBLAS_SGLANG_OPS", "").split(",")))
    if not selected:
        return
    if selected - {"linear", "fp8"}:
        raise ValueError(f"Unknown CAMBLAS SGLang operations: {sorted(selected)}")

    import torch
    from sglang.srt.plugins.hook_registry import HookRegistry, HookType

    from . import _kernels as cb
    from ._torch_backend import install_torch_backend

    algorithm = os.environ.get("CAMBLAS_SGLANG_ALGORITHM", "lt")
    cb.set_algorithm(algorithm)
    if "linear" in selected:
        install_torch_backend(algorithm)

    def no_gradient(*tensors):
        return not (torch.is_grad_enabled() and any(t.requires_grad for t in tensors))

    def linear(original, method, layer, x, bias=None):
        """Unquantised linear: eligible BF16 calls run ``F.linear`` under the overrides."""
        weight = layer.weight
        operands = (x, weight) if bias is None else (x, weight, bias)
        if (x.is_cuda and x.ndim >= 2 and weight.ndim == 2 and x.dtype == torch.bfloat16
                and all(t.is_contiguous() and t.device == x.device for t in operands)
                and all(t.dtype == x.dtype for t in operands) and no_gradient(*operands)):
            _count("linear")
            output = torch.nn.functional.linear(x.view(-1, x.shape[-1]), weight, bias)
            return output.view(*x.shape[:-1], weight.shape[0])
        return original(method, layer, x, bias)

    def batched(original, layer, input):
        """Batched BF16 projection: ``output[b] = input[b] @ weight[b].T`` for every entry."""
        weight = layer.weight
        if (input.is_cuda and input.ndim == 3 and weight.ndim == 3
                and input.shape[0] == weight.shape[0] and input.shape[2] == weight.shape[2]
                and input.dtype == weight.dtype == torch.bfloat16 and input.is_contiguous()
                and weight.is_contiguous() and weight.device == input.device
                and not torch.is_grad_enabled() and not torch._dynamo.is_compiling()):
            _count("bmm")
            return torch.stack([cb.linear(input[entry], weight[entry])
                                for entry in range(input.shape[0])])
        return original(layer, input)

    def dense(original, input, weight, block_size, weight_scale, input_scale=None, bias=None):
        """Block-128 w8a8 linear: quantise the BF16 rows, then the block-scaled GEMM."""
        if (input.is_cuda and input.ndim >= 2 and weight.ndim == 2
                and input.dtype == torch.bfloat16 and weight.dtype == torch.float8_e4m3fn
                and input.shape[-1] == weight.shape[1] and weight.shape[1] % 128 == 0
                and weight.shape[0] % 8 == 0 and list(block_size) == [128, 128]
                and weight_scale.dtype == torch.float32
                and tuple(weight_scale.shape) == ((weight.shape[0] + 127) // 128, weight.shape[1] // 128)
                and input_scale is None and bias is None
                and all(t.is_contiguous() and t.device == input.device
                        for t in (input, weight, weight_scale))
                and not torch.is_grad_enabled() and not torch._dynamo.is_compiling()):
            rows = input.numel() // weight.shape[1]
            q, q_scale = cb.fp8_quantize(input.view(rows, weight.shape[1]))
            output = cb.fp8_block_gemm(q, q_scale, weight, weight_scale)
            _count("fp8")
            _count("fp8_dense_block128")
            return output.view(*input.shape[:-1], weight.shape[0])
        return original(input, weight, block_size, weight_scale, input_scale, bias)

    def block32_shape_ok(weight):
        outputs, inner = weight.shape
        return inner % 32 == 0 and 32 <= inner <= 8192 and outputs % 16 == 0 and outputs > 0

    def fp8_product(original, A, B, As, Bs, block_size, output_dtype=torch.float16):
        """Block-32 pre-quantised single-token product (``camblas_cuda_fp8_decode``)."""
        operands = (A, B, As, Bs)
        if (not torch._dynamo.is_compiling() and A.is_cuda and A.ndim >= 2 and B.ndim == 2
                and As.ndim == A.ndim and Bs.ndim == 2 and A.numel() == A.shape[-1]
                and A.shape[-1] == B.shape[1] and block32_shape_ok(B)
                and list(block_size) == [32, 32] and output_dtype == torch.bfloat16
                and A.dtype == B.dtype == torch.float8_e4m3fn
                and As.dtype == Bs.dtype == torch.float32 and A.is_contiguous() and B.is_contiguous()
                and A.data_ptr() % 4 == B.data_ptr() % 4 == 0
                and As.numel() == B.shape[1] // 32
                and tuple(Bs.shape) == ((B.shape[0] + 31) // 32, B.shape[1] // 32)
                and all(t.device == A.device for t in operands)
                and all(0 < stride <= 2147483647 for stride in (As.stride(-1), *Bs.stride()))
                and no_gradient(*operands)):
            _count("fp8")
            _count(f"fp8_decode:{B.shape[0]},{B.shape[1]}")
            scales = As[(0,) * (As.ndim - 1)]  # [inner/32], keeps a strided last dimension
            return cb.fp8_decode(A.view(-1), scales, B, Bs).view(*A.shape[:-1], B.shape[0])
        return original(A, B, As, Bs, block_size, output_dtype)

    def fp8_linear(original, input, weight, block_size, weight_scale, input_scale=None, bias=None,
                   act_scale_ue8m0=False, weight_bf16=None):
        """Block-32 BF16-input single-token linear (``camblas_cuda_fp8_linear``)."""
        if (not torch._dynamo.is_compiling() and input.is_cuda and input.ndim >= 2
                and weight.ndim == 2 and input.numel() == weight.shape[1]
                and input.dtype == torch.bfloat16 and weight.dtype == torch.float8_e4m3fn
                and block32_shape_ok(weight) and list(block_size) == [32, 32]
                and weight_scale.dtype == torch.float32 and weight_scale.ndim == 2
                and tuple(weight_scale.shape) == ((weight.shape[0] + 31) // 32, weight.shape[1] // 32)
                and input_scale is None and bias is None and act_scale_ue8m0
                and input.is_contiguous() and weight.is_contiguous()
                and weight.device == input.device and weight_scale.device == input.device
                and all(0 < stride <= 2147483647 for stride in weight_scale.stride())
                and not torch.is_grad_enabled()):
            _count("fp8")
            _count(f"fp8_linear:{weight.shape[0]},{weight.shape[1]}")
            return cb.fp8_linear(input.view(-1), weight, weight_scale).view(*input.shape[:-1],
                                                                            weight.shape[0])
        return original(input, weight, block_size, weight_scale, input_scale, bias,
                        act_scale_ue8m0, weight_bf16)

    if "linear" in selected:
        HookRegistry.register(
            "sglang.srt.layers.quantization.unquant.UnquantizedLinearMethod.apply", linear,
            HookType.AROUND)
        HookRegistry.register("sglang.srt.layers.linear.ColumnParallelBatchedLinear.forward", batched,
                              HookType.AROUND)
    if "fp8" in selected:
        HookRegistry.register(
            "sglang.srt.layers.quantization.fp8_utils.deepgemm_w8a8_block_fp8_linear_with_fallback",
            dense, HookType.AROUND)
        HookRegistry.register(
            "sglang.kernels.ops.quantization.fp8_kernel.w8a8_block_fp8_matmul_triton",
            fp8_product, HookType.AROUND)
        HookRegistry.register(
            "sglang.srt.layers.quantization.fp8_utils.triton_w8a8_block_fp8_linear", fp8_linear,
            HookType.AROUND)
