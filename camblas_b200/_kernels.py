"""Tensor-level operations over the C ABI.

The names and argument meaning follow ``camblas/_kernels.py:34-59`` and the
functions of ``src/cuda/torch_bindings.cpp`` they resolve to in the reference:
``matmul`` (:155-199), ``linear`` (:244-270), ``qkv_linear`` (:725-736),
``add_rms_norm`` (:675-701), ``rms_norm`` (:602-673), ``silu_multiply``,
``swiglu``, ``fp8_decode`` / ``fp8_linear`` (:389-452). Tensors are validated in
Python, then passed to ``libcamblas_cuda.so`` as device pointers; every
operation runs on the current CUDA stream of the tensor's device. Bad metadata
raises ``ValueError`` before anything is launched; a native failure raises
``RuntimeError`` with the library's message.
"""

import ctypes as ct

import torch

from . import _native
from ._native import algorithm, kernel_family, set_algorithm, stats  # noqa: F401

_INT_MAX = 2**31 - 1


def _require(condition, message):
    if not condition:
        raise ValueError(message)


def _pointer(tensor):
    return ct.c_void_p(tensor.data_ptr()) if tensor is not None else ct.c_void_p()


def _check_tensor(tensor, reference, what="operand"):
    _require(tensor.is_cuda and tensor.dtype == torch.bfloat16, f"{what} must be a CUDA BF16 tensor")
    _require(
        tensor.device == reference.device and tensor.dtype == reference.dtype,
        "All operands must have the same device and dtype",
    )
    _require(all(size <= _INT_MAX for size in tensor.shape), "LP64 dimension overflow")
    _require(all(stride <= _INT_MAX for stride in tensor.stride()), "LP64 stride overflow")


def _operand(tensor):
    """Map a 2-D tensor to (tensor, transpose flag, leading dimension).

    A row-major [r, c] tensor is the column-major c x r matrix, flag 'N'; a
    tensor with unit row stride is flagged 'T'; anything else is copied
    (``torch_bindings.cpp:146-153``).
    """
    rows, columns = tensor.shape
    stride0, stride1 = tensor.stride()
    if stride1 == 1 and stride0 >= max(1, columns):
        return tensor, b"N", stride0
    if stride0 == 1 and stride1 >= max(1, rows):
        return tensor, b"T", stride1
    return tensor.contiguous(), b"N", max(1, columns)


def matmul(a, b, out=None, alpha=1.0, beta=0.0):
    """Return ``alpha * a @ b + beta * out`` for 2-D BF16 CUDA tensors.

    The row-major product is issued as the transposed column-major product
    ``bgemm(op(b), op(a))`` with ``m = b.shape[1]``, ``n = a.shape[0]``, exactly
    as the reference binding does (``torch_bindings.cpp:189-194``).
    """
    _check_tensor(a, a)
    _check_tensor(b, a)
    _require(a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[0],
             "matmul requires compatible rank-two operands")
    m, k, n = a.shape[0], a.shape[1], b.shape[1]
    if out is not None:
        _check_tensor(out, a, "output")
        _require(out.dim() == 2 and tuple(out.shape) == (m, n) and out.is_contiguous(),
                 "Output must have the product shape and contiguous row storage")
        _require(out.untyped_storage().data_ptr() != a.untyped_storage().data_ptr()
                 and out.untyped_storage().data_ptr() != b.untyped_storage().data_ptr(),
                 "GEMM output cannot alias an input")
        c = out
    else:
        _require(beta == 0, "beta requires an existing output tensor")
        c = torch.empty((m, n), dtype=a.dtype, device=a.device)
    if m == 0 or n == 0:
        return c
    left, left_flag, left_ld = _operand(b)
    right, right_flag, right_ld = _operand(a)
    with torch.cuda.device(a.device):
        native = _native.context(a.device.index)
        native.call("bgemm", left_flag, right_flag, n, m, k, float(alpha), _pointer(left), left_ld,
                    _pointer(right), right_ld, float(beta), _pointer(c), max(1, n))
    return c


def linear(x, weight, bias=None, residual=None):
    """Return ``x @ weight.T (+ bias) (+ residual)`` with the epilogue fused.

    ``x`` is ``[..., inner]``, ``weight`` ``[outputs, inner]``; leading
    dimensions are flattened (``torch_bindings.cpp:244-270``). Unlike the
    reference, which adds the bias with a second kernel, bias and residual are
    applied in the GEMM epilogue before the single rounding to BF16.
    """
    _check_tensor(x, x)
    _check_tensor(weight, x, "weight")
    _require(x.dim() >= 1 and weight.dim() == 2 and x.shape[-1] == weight.shape[1],
             "linear requires matching input and [outputs, inputs] weight dimensions")
    inner, outputs = weight.shape[1], weight.shape[0]
    rows = 1
    for size in x.shape[:-1]:
        rows *= size
    _require(rows <= _INT_MAX, "LP64 flattened row overflow")
    x2 = x.reshape(rows, inner)
    if x2.stride(-1) != 1 or (rows > 1 and x2.stride(0) < inner):
        x2 = x2.contiguous()
    w2 = weight if weight.stride(1) == 1 and weight.stride(0) >= inner else weight.contiguous()
    if bias is not None:
        _check_tensor(bias, x, "bias")
        _require(bias.dim() == 1 and bias.shape[0] == outputs and bias.is_contiguous(),
                 "linear bias must have the output width")
    r2 = None
    if residual is not None:
        _check_tensor(residual, x, "residual")
        _require(tuple(residual.shape) == tuple(x.shape[:-1]) + (outputs,),
                 "residual must have the output shape")
        r2 = residual.reshape(rows, outputs)
        if r2.stride(-1) != 1:
            r2 = r2.contiguous()
    out = torch.empty((rows, outputs), dtype=x.dtype, device=x.device)
    if rows and outputs:
        with torch.cuda.device(x.device):
            native = _native.context(x.device.index)
            native.call("linear_bf16", rows, inner, outputs, _pointer(x2),
                        x2.stride(0) if rows > 1 else inner, _pointer(w2), w2.stride(0),
                        _pointer(bias), _pointer(r2),
                        (r2.stride(0) if rows > 1 else outputs) if r2 is not None else 0,
                        _pointer(out), outputs)
    return out.reshape(tuple(x.shape[:-1]) + (outputs,))


def qkv_linear(x, weight, q_out, k_out, v_out):
    """Project ``x`` with a packed ``[q_out+k_out+v_out, inner]`` weight.

    Returns three separately allocated tensors, like the reference's
    ``qkv_linear`` (``torch_bindings.cpp:725-736``, ``tests/test_qkv.py:37``),
    but from one kernel launch over the packed weight.
    """
    _check_tensor(x, x)
    _check_tensor(weight, x, "weight")
    _require(x.dim() >= 1 and weight.dim() == 2 and x.shape[-1] == weight.shape[1]
             and weight.shape[0] == q_out + k_out + v_out and min(q_out, k_out, v_out) > 0,
             "qkv_linear requires a [q+k+v, inner] weight")
    inner = weight.shape[1]
    rows = 1
    for size in x.shape[:-1]:
        rows *= size
    x2 = x.reshape(rows, inner).contiguous()
    w2 = weight.contiguous()
    outs = [torch.empty((rows, width), dtype=x.dtype, device=x.device)
            for width in (q_out, k_out, v_out)]
    if rows:
        with torch.cuda.device(x.device):
            native = _native.context(x.device.index)
            native.call("qkv_linear_bf16", rows, inner, q_out, k_out, v_out, _pointer(x2), inner,
                        _pointer(w2), inner, _pointer(outs[0]), q_out, _pointer(outs[1]), k_out,
                        _pointer(outs[2]), v_out)
    lead = tuple(x.shape[:-1])
    return tuple(o.reshape(lead + (o.shape[1],)) for o in outs)


def _dtype_code(tensor):
    if tensor.dtype == torch.float32:
        return 0
    if tensor.dtype == torch.bfloat16:
        return 2
    raise ValueError("RMS operations take FP32 or BF16 tensors")


def add_rms_norm(x, residual, weight, epsilon):
    """Return ``(added, normalised)`` for ``added = x + residual``.

    ``added`` is rounded to the storage type before the mean of squares;
    ``normalised = rnd(rnd(added * rsqrt(mean(added^2)+eps)) * weight)``
    (``inference_fusion.cuh:136-191``). Any number of rows is handled by one
    launch with one CTA per row. Two-dimensional ``x`` and ``residual`` may be
    views whose rows are contiguous but spaced apart (a column slice, one half
    of an interleaved buffer): they are read where they lie.
    """
    _require(x.is_cuda and residual.is_cuda and weight.is_cuda, "operands must be CUDA tensors")
    _require(x.dtype == residual.dtype == weight.dtype and x.device == residual.device == weight.device,
             "All operands must have the same device and dtype")
    _require(x.shape == residual.shape and weight.dim() == 1 and weight.shape[0] == x.shape[-1],
             "residual must match x and weight the last dimension")
    code = _dtype_code(x)
    width = x.shape[-1]
    _require(4 <= width <= 65536 and width % 4 == 0, "width must be a multiple of four up to 65536")
    w2 = weight.contiguous()

    def rows_in_place(tensor):
        return (tensor.dim() == 2 and tensor.stride(1) == 1 and tensor.stride(0) >= width
                and tensor.stride(0) % 4 == 0 and tensor.stride(0) <= _INT_MAX)

    if rows_in_place(x) and rows_in_place(residual) and not (x.is_contiguous()
                                                              and residual.is_contiguous()):
        added = torch.empty((x.shape[0], width), dtype=x.dtype, device=x.device)
        out = torch.empty_like(added)
        if x.shape[0]:
            with torch.cuda.device(x.device):
                native = _native.context(x.device.index)
                native.call("add_rms_norm_strided", code, x.shape[0], width, float(epsilon),
                            _pointer(x), x.stride(0), _pointer(residual), residual.stride(0),
                            _pointer(w2), _pointer(added), width, _pointer(out), width)
        return added, out
    x2, r2 = x.contiguous(), residual.contiguous()
    added, out = torch.empty_like(x2), torch.empty_like(x2)
    rows = x2.numel() // width
    if rows:
        with torch.cuda.device(x.device):
            native = _native.context(x.device.index)
            native.call("add_rms_norm_rows", code, rows, width, float(epsilon), _pointer(x2),
                        _pointer(r2), _pointer(w2), _pointer(added), _pointer(out))
    return added, out


def rms_norm(x, weight, epsilon):
    """Return ``rnd(rnd(x * rsqrt(mean(x^2)+eps)) * weight)`` over the last dimension."""
    _require(x.is_cuda and weight.is_cuda and x.dtype == weight.dtype and x.device == weight.device,
             "All operands must have the same device and dtype")
    _require(weight.dim() == 1 and weight.shape[0] == x.shape[-1], "weight must match the last dimension")
    code = _dtype_code(x)
    width = x.shape[-1]
    x2, w2 = x.contiguous(), weight.contiguous()
    out = torch.empty_like(x2)
    rows = x2.numel() // width if width else 0
    if rows:
        with torch.cuda.device(x.device):
            native = _native.context(x.device.index)
            native.call("rms_norm", code, rows, width, float(epsilon), _pointer(x2), _pointer(w2),
                        _pointer(out))
    return out


def silu_multiply(gate, up):
    """Return ``rnd(rnd(silu(gate)) * up)`` (``inference_fusion.cuh:19-29``)."""
    _require(gate.is_cuda and gate.shape == up.shape and gate.dtype == up.dtype
             and gate.device == up.device, "gate and up must match")
    code = _dtype_code(gate)
    g, u = gate.contiguous(), up.contiguous()
    out = torch.empty_like(g)
    if g.numel():
        with torch.cuda.device(gate.device):
            native = _native.context(gate.device.index)
            native.call("silu_multiply", code, g.numel(), _pointer(g), _pointer(u), _pointer(out))
    return out


def interleave_gate_up(weight, block=128):
    """Permute a packed ``[gate; up]`` weight for ``gate_up_swiglu`` (done once, at load time).

    ``weight`` is ``[2 * intermediate, inner]`` with the gate rows first. The
    result holds, for every block ``j`` of 128 features, the gate rows of the
    block followed by its up rows, so that one 256-column tile of the GEMM
    carries both halves of 128 outputs.
    """
    _require(weight.dim() == 2 and weight.shape[0] % (2 * block) == 0,
             "gate_up weight rows must be a multiple of 256")
    intermediate = weight.shape[0] // 2
    gate = weight[:intermediate].reshape(intermediate // block, block, weight.shape[1])
    up = weight[intermediate:].reshape(intermediate // block, block, weight.shape[1])
    return torch.stack((gate, up), dim=1).reshape(2 * intermediate, weight.shape[1]).contiguous()


def gate_up_swiglu(x, weight_interleaved):
    """Return ``silu_multiply(x @ Wg.T, x @ Wu.T)`` from one GEMM pass.

    ``weight_interleaved`` comes from ``interleave_gate_up``. The roundings are
    those of the two-step path (BF16 GEMM outputs, then
    ``inference_fusion.cuh:19-29``), so the result equals
    ``silu_multiply(*linear(x, W).chunk(2, -1))`` whenever the GEMM sums agree.
    """
    _check_tensor(x, x)
    _check_tensor(weight_interleaved, x, "weight")
    _require(x.dtype == torch.bfloat16, "gate_up_swiglu takes BF16 operands")
    _require(x.dim() >= 1 and weight_interleaved.dim() == 2
             and x.shape[-1] == weight_interleaved.shape[1]
             and weight_interleaved.shape[0] % 256 == 0,
             "gate_up_swiglu requires x [..., inner] and an interleaved [2*intermediate, inner] weight")
    inner, intermediate = weight_interleaved.shape[1], weight_interleaved.shape[0] // 2
    rows = 1
    for size in x.shape[:-1]:
        rows *= size
    _require(rows <= _INT_MAX, "LP64 flattened row overflow")
    x2 = x.reshape(rows, inner)
    if x2.stride(-1) != 1 or (rows > 1 and x2.stride(0) < inner) or x2.stride(0) % 8:
        x2 = x2.contiguous()
    w2 = weight_interleaved
    if w2.stride(1) != 1 or w2.stride(0) < inner or w2.stride(0) % 8:
        w2 = w2.contiguous()
    out = torch.empty((rows, intermediate), dtype=x.dtype, device=x.device)
    if rows:
        with torch.cuda.device(x.device):
            native = _native.context(x.device.index)
            native.call("gate_up_swiglu_bf16", rows, inner, intermediate, _pointer(x2),
                        x2.stride(0) if rows > 1 else inner, _pointer(w2), w2.stride(0),
                        _pointer(out), intermediate)
    return out.reshape(tuple(x.shape[:-1]) + (intermediate,))


def gate_up_swiglu_fp8(x, weight_interleaved):
    """``fp8_quantize(gate_up_swiglu(x, weight))`` from one GEMM pass.

    Returns ``(q, scale)``: E4M3 ``[rows, intermediate]`` and FP32
    ``[rows, intermediate/128]``, bit-equal to quantising the BF16 result of
    ``gate_up_swiglu`` with ``fp8_quantize``; the BF16 tensor is never stored.
    """
    _check_tensor(x, x)
    _check_tensor(weight_interleaved, x, "weight")
    _require(x.dim() == 2 and weight_interleaved.dim() == 2
             and x.shape[1] == weight_interleaved.shape[1]
             and weight_interleaved.shape[0] % 256 == 0,
             "gate_up_swiglu_fp8 requires x [rows, inner] and an interleaved [2*intermediate, inner] weight")
    rows, inner = x.shape
    intermediate = weight_interleaved.shape[0] // 2
    x2 = x if x.stride(1) == 1 and x.stride(0) >= inner and x.stride(0) % 8 == 0 else x.contiguous()
    w2 = weight_interleaved
    if w2.stride(1) != 1 or w2.stride(0) < inner or w2.stride(0) % 8:
        w2 = w2.contiguous()
    q = torch.empty((rows, intermediate), dtype=torch.float8_e4m3fn, device=x.device)
    scale = torch.empty((rows, intermediate // 128), dtype=torch.float32, device=x.device)
    if rows:
        with torch.cuda.device(x.device):
            native = _native.context(x.device.index)
            native.call("gate_up_swiglu_fp8", rows, inner, intermediate, _pointer(x2),
                        x2.stride(0) if rows > 1 else inner, _pointer(w2), w2.stride(0),
                        _pointer(q), _pointer(scale))
    return q, scale


def gated_mlp(x, gate_weight, up_weight, down_weight):
    """Bias-free SiLU-gated MLP for inference: ``linear(silu_multiply(linear(x, Wg), linear(x, Wu)), Wd)``.

    The reference's ``gated_mlp`` (``torch_bindings.cpp:703-723``): two projections, the
    elementwise product written over the gate, the down projection. ``GatedMLP`` does the
    same with the first two projections and the product in one GEMM pass.
    """
    _require(x.dim() >= 1 and gate_weight.dim() == 2 and up_weight.dim() == 2 and down_weight.dim() == 2
             and gate_weight.shape == up_weight.shape and x.shape[-1] == gate_weight.shape[1]
             and down_weight.shape[1] == gate_weight.shape[0], "Invalid gated MLP dimensions")
    return linear(silu_multiply(linear(x, gate_weight), linear(x, up_weight)), down_weight)


class GatedMLP:
    """The gated MLP with its weights prepared once: gate and up rows interleaved in blocks
    of 128 so that ``gate_up_swiglu`` produces ``silu(gate) * up`` from one GEMM pass
    (no ``[rows, 2 * intermediate]`` round trip through HBM), then the down projection.
    Same roundings as ``gated_mlp``; the bits agree whenever the GEMM sums do. The
    intermediate width must be a multiple of 128.
    """

    def __init__(self, gate_weight, up_weight, down_weight):
        _require(gate_weight.dim() == 2 and gate_weight.shape == up_weight.shape
                 and down_weight.dim() == 2 and down_weight.shape[1] == gate_weight.shape[0]
                 and gate_weight.shape[0] % 128 == 0, "Invalid gated MLP dimensions")
        self.gate_up = interleave_gate_up(torch.cat((gate_weight, up_weight)))
        self.down = down_weight

    def __call__(self, x):
        return linear(gate_up_swiglu(x, self.gate_up), self.down)


def _float_code(tensor):
    _require(tensor.is_cuda and tensor.dtype in (torch.float32, torch.float64),
             "operand must be a CUDA FP32 or FP64 tensor")
    return 0 if tensor.dtype == torch.float32 else 1


def affine(x, weight, bias, relu=False):
    """``x @ weight + bias`` with optional ReLU in FP32 / FP64 (``camblas_cuda_affine``; the
    reference's ``affine``, ``torch_bindings.cpp:738-770``, forward only). ``x`` is
    ``[rows, inner]``, ``weight`` ``[inner, columns]``."""
    code = _float_code(x)
    _require(x.dim() == 2 and weight.dim() == 2 and bias.dim() == 1 and x.shape[1] == weight.shape[0]
             and bias.shape[0] == weight.shape[1] and weight.dtype == x.dtype == bias.dtype
             and weight.device == x.device == bias.device, "Invalid affine operands")
    x2, w2, b2 = x.contiguous(), weight.contiguous(), bias.contiguous()
    out = torch.empty((x.shape[0], weight.shape[1]), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        _native.context(x.device.index).call("affine", code, x.shape[0], x.shape[1], weight.shape[1],
                                             _pointer(x2), _pointer(w2), _pointer(b2), int(bool(relu)),
                                             _pointer(out))
    return out


def mlp(x, w1, b1, w2, b2):
    """``relu(x @ w1 + b1) @ w2 + b2`` in FP32 / FP64 (``camblas_cuda_mlp``); returns
    ``(output, hidden)`` - the hidden activations are what the backward pass needs."""
    code = _float_code(x)
    _require(x.dim() == 2 and w1.dim() == 2 and w2.dim() == 2 and x.shape[1] == w1.shape[0]
             and w1.shape[1] == w2.shape[0] and b1.shape == (w1.shape[1],) and b2.shape == (w2.shape[1],)
             and all(t.dtype == x.dtype and t.device == x.device for t in (w1, b1, w2, b2)),
             "Invalid MLP operands")
    operands = [t.contiguous() for t in (x, w1, b1, w2, b2)]
    hidden = torch.empty((x.shape[0], w1.shape[1]), dtype=x.dtype, device=x.device)
    out = torch.empty((x.shape[0], w2.shape[1]), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        _native.context(x.device.index).call("mlp", code, x.shape[0], x.shape[1], w1.shape[1], w2.shape[1],
                                             *(_pointer(t) for t in operands), _pointer(hidden),
                                             _pointer(out))
    return out, hidden


def attention(q, k, v, scale=None):
    """Dense single-head ``softmax(scale * q @ k.T) @ v`` in FP32 / FP64, no mask
    (``camblas_cuda_attention``); the default scale is ``1 / sqrt(depth)``."""
    code = _float_code(q)
    _require(q.dim() == 2 and k.dim() == 2 and v.dim() == 2 and q.shape[1] == k.shape[1]
             and k.shape[0] == v.shape[0] and all(t.dtype == q.dtype and t.device == q.device for t in (k, v)),
             "Invalid attention operands")
    if scale is None:
        scale = q.shape[1] ** -0.5 if q.shape[1] else 1.0
    q2, k2, v2 = q.contiguous(), k.contiguous(), v.contiguous()
    out = torch.empty((q.shape[0], v.shape[1]), dtype=q.dtype, device=q.device)
    with torch.cuda.device(q.device):
        _native.context(q.device.index).call("attention", code, q.shape[0], k.shape[0], q.shape[1],
                                             v.shape[1], float(scale), _pointer(q2), _pointer(k2),
                                             _pointer(v2), _pointer(out))
    return out


def swiglu(gate, up, limit=0.0, routing=None):
    """Return ``rnd(silu(gate) * up [* routing[row]])`` with optional clipping."""
    _require(gate.is_cuda and gate.shape == up.shape and gate.dtype == up.dtype
             and gate.device == up.device and gate.dim() >= 1, "gate and up must match")
    code = _dtype_code(gate)
    g, u = gate.contiguous(), up.contiguous()
    out = torch.empty_like(g)
    width = g.shape[-1]
    if routing is not None:
        _require(routing.dtype == torch.float32 and routing.is_cuda and routing.is_contiguous()
                 and routing.numel() == g.numel() // max(1, width), "routing is one FP32 per row")
    if g.numel():
        with torch.cuda.device(gate.device):
            native = _native.context(gate.device.index)
            native.call("swiglu", code, g.numel(), width, float(limit), _pointer(g), _pointer(u),
                        _pointer(routing), _pointer(out))
    return out


def fp8_quantize(x):
    """Quantise BF16 rows to E4M3 with one FP32 scale per 128 elements.

    Returns ``(q, scale)`` with ``q`` ``float8_e4m3fn [rows, inner]`` and
    ``scale`` ``float32 [rows, inner/128]``; ``scale = max(amax,1e-10)/448``
    (``camblas/_hopper.py:82-98``).
    """
    _check_tensor(x, x)
    _require(x.dim() == 2 and x.shape[1] % 128 == 0 and x.shape[1] > 0,
             "fp8_quantize takes [rows, inner] with inner a multiple of 128")
    x2 = x if x.stride(1) == 1 and x.stride(0) >= x.shape[1] else x.contiguous()
    rows, inner = x2.shape
    q = torch.empty((rows, inner), dtype=torch.float8_e4m3fn, device=x.device)
    scale = torch.empty((rows, inner // 128), dtype=torch.float32, device=x.device)
    if rows:
        with torch.cuda.device(x.device):
            native = _native.context(x.device.index)
            native.call("fp8_quantize_rows", rows, inner, _pointer(x2),
                        x2.stride(0) if rows > 1 else inner, _pointer(q), _pointer(scale))
    return q, scale


def fp8_block_gemm(q, q_scale, weight, weight_scale):
    """Block-scaled w8a8 product, BF16 ``[rows, outputs]``.

    ``q`` E4M3 ``[rows, inner]`` with ``q_scale`` FP32 ``[rows, inner/128]``;
    ``weight`` E4M3 ``[outputs, inner]`` with ``weight_scale`` FP32
    ``[ceil(outputs/128), inner/128]``. Each 128-deep block is accumulated on
    its own and promoted as ``fma(dot, q_scale*w_scale, acc)`` in ascending
    block order (``camblas/_hopper.py:118-126, 168-182``).
    """
    _require(q.is_cuda and weight.is_cuda and q.dtype == torch.float8_e4m3fn
             and weight.dtype == torch.float8_e4m3fn, "operands must be CUDA float8_e4m3fn")
    _require(q.dim() == 2 and weight.dim() == 2 and q.shape[1] == weight.shape[1]
             and q.shape[1] % 128 == 0, "inner dimensions must match and divide by 128")
    rows, inner = q.shape
    outputs = weight.shape[0]
    groups = inner // 128
    _require(q_scale.dtype == torch.float32 and tuple(q_scale.shape) == (rows, groups)
             and q_scale.is_contiguous(), "q_scale must be contiguous FP32 [rows, inner/128]")
    _require(weight_scale.dtype == torch.float32
             and tuple(weight_scale.shape) == ((outputs + 127) // 128, groups)
             and weight_scale.is_contiguous(),
             "weight_scale must be contiguous FP32 [ceil(outputs/128), inner/128]")
    _require(q.is_contiguous() and weight.is_contiguous(), "operands must be contiguous")
    out = torch.empty((rows, outputs), dtype=torch.bfloat16, device=q.device)
    if rows and outputs:
        with torch.cuda.device(q.device):
            native = _native.context(q.device.index)
            native.call("fp8_block_gemm", rows, outputs, inner, _pointer(q), _pointer(q_scale),
                        _pointer(weight), _pointer(weight_scale), _pointer(out), outputs)
    return out


def fp8_decode_supported(device=None):
    """Return whether the single-token block-32 FP8 product is available."""
    if device is None:
        device = torch.cuda.current_device()
    native = _native.context(torch.device("cuda", device).index if not isinstance(device, int) else device)
    return bool(_native.library().camblas_cuda_fp8_decode_supported(native.handle))


def _fp8_scales(weight_scale):
    _require(weight_scale.dtype == torch.float32 and weight_scale.dim() == 2
             and all(stride > 0 for stride in weight_scale.stride()),
             "weight scales must be FP32 [ceil(outputs/32), inner/32] with positive strides")
    return weight_scale.stride(0), weight_scale.stride(1)


def fp8_decode(x, x_scale, weight, weight_scale):
    """Single-token block-32 E4M3 product with FP32 scales, BF16 ``[outputs]``."""
    _require(x.is_cuda and x.dtype == torch.float8_e4m3fn and weight.dtype == torch.float8_e4m3fn,
             "input and weight must be CUDA float8_e4m3fn")
    outputs, inner = weight.shape
    _require(x.numel() == inner and weight.is_contiguous() and x.is_contiguous(),
             "input must hold one token of the weight's inner width")
    _require(inner % 32 == 0 and 32 <= inner <= 8192 and outputs % 16 == 0 and outputs > 0,
             "inner must be a multiple of 32 in [32, 8192] and outputs a positive multiple of 16")
    _require(x_scale.dtype == torch.float32 and x_scale.numel() == inner // 32
             and x_scale.dim() >= 1 and x_scale.stride(-1) > 0, "input scales must be FP32 [inner/32]")
    _require(tuple(weight_scale.shape) == ((outputs + 31) // 32, inner // 32),
             "weight scales must be [ceil(outputs/32), inner/32]")
    row_stride, column_stride = _fp8_scales(weight_scale)
    out = torch.empty((outputs,), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        native = _native.context(x.device.index)
        native.call("fp8_decode", outputs, inner, _pointer(x), _pointer(x_scale), _pointer(weight),
                    _pointer(weight_scale), x_scale.stride(-1), row_stride, column_stride,
                    ct.c_void_p(), 0, _pointer(out))
    return out


def fp8_linear(x, weight, weight_scale):
    """Single BF16 token quantised to block-32 power-of-two scales, then ``fp8_decode``."""
    _require(x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.float8_e4m3fn,
             "input must be CUDA BF16 and weight float8_e4m3fn")
    outputs, inner = weight.shape
    _require(x.numel() == inner and weight.is_contiguous() and x.is_contiguous(),
             "input must hold one token of the weight's inner width")
    _require(inner % 32 == 0 and 32 <= inner <= 8192 and outputs % 16 == 0 and outputs > 0,
             "inner must be a multiple of 32 in [32, 8192] and outputs a positive multiple of 16")
    _require(tuple(weight_scale.shape) == ((outputs + 31) // 32, inner // 32),
             "weight scales must be [ceil(outputs/32), inner/32]")
    row_stride, column_stride = _fp8_scales(weight_scale)
    out = torch.empty((outputs,), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        native = _native.context(x.device.index)
        native.call("fp8_linear", outputs, inner, _pointer(x), _pointer(weight),
                    _pointer(weight_scale), row_stride, column_stride, ct.c_void_p(), 0,
                    _pointer(out))
    return out


def _is_e8m0(tensor):
    return tensor.dtype in (torch.float8_e8m0fnu, torch.uint8)


def _packed_weight(weight):
    packed_dtype = getattr(torch, "float4_e2m1fn_x2", None)
    if packed_dtype is not None and weight.dtype == packed_dtype:
        return True
    _require(weight.dtype == torch.float8_e4m3fn,
             "Quantized weight must be FP8 E4M3 or packed FP4 E2M1")
    return False


def quantized_matmul(x, x_scale, weight, weight_scale, activation_block=32):
    """Block-scaled product with power-of-two (E8M0) scales, BF16 ``[..., outputs]``.

    ``x`` is E4M3 ``[..., inner]`` with scales ``[..., inner/activation_block]``;
    ``weight`` is E4M3 ``[outputs, inner]`` with scales ``[ceil(outputs/32),
    inner/32]``, or packed E2M1 ``[outputs, inner/2]`` with scales ``[outputs,
    inner/32]``. Argument meaning and checks follow ``quantized_matmul_public``
    (``torch_bindings.cpp:328-377``).
    """
    _require(x.is_cuda and x.dtype == torch.float8_e4m3fn, "Quantized input must be CUDA FP8 E4M3")
    packed = _packed_weight(weight)
    _require(_is_e8m0(x_scale) and _is_e8m0(weight_scale), "Quantized scales must be E8M0")
    for tensor in (x, x_scale, weight, weight_scale):
        _require(tensor.device == x.device and tensor.is_contiguous(),
                 "Quantized operands must be contiguous and on the same CUDA device")
    _require(x.dim() >= 1 and weight.dim() == 2 and x_scale.dim() == x.dim()
             and weight_scale.dim() == 2, "Quantized matrix and scale ranks do not match")
    inner, outputs = x.shape[-1], weight.shape[0]
    _require(inner >= 32 and inner % 32 == 0 and outputs >= 8 and outputs % 8 == 0
             and weight.shape[1] == inner // (2 if packed else 1)
             and (activation_block == 32 or (packed and activation_block == 128))
             and inner % activation_block == 0,
             "Invalid quantized matrix dimensions or activation block")
    rows = 1
    for index in range(x.dim() - 1):
        _require(x_scale.shape[index] == x.shape[index], "Input scale shape mismatch")
        rows *= x.shape[index]
    _require(rows <= 65535, "Quantized multiplication supports at most 65535 rows")
    _require(x_scale.shape[-1] == inner // activation_block
             and weight_scale.shape[0] == (outputs if packed else (outputs + 31) // 32)
             and weight_scale.shape[1] == inner // 32,
             "Quantized scale shapes do not match their blocks")
    out = torch.empty(tuple(x.shape[:-1]) + (outputs,), dtype=torch.bfloat16, device=x.device)
    if rows:
        with torch.cuda.device(x.device):
            native = _native.context(x.device.index)
            native.call("quantized_matmul", int(packed), rows, outputs, inner, activation_block,
                        _pointer(x), _pointer(x_scale), _pointer(weight), _pointer(weight_scale),
                        _pointer(out))
    return out


class QuantizedGroups:
    """Weights and scales of a set of experts for ``matmul`` over routed rows.

    Mirrors the reference's ``QuantizedGroups`` (``torch_bindings.cpp:466-550``):
    the constructor records the device addresses of every expert's weight and
    scale tensor in a device table, ``matmul`` multiplies batch ``b`` of ``x``
    ``[groups, rows, inner]`` with expert ``active[b]`` for its first
    ``counts[b]`` rows and returns BF16 ``[groups, rows, outputs]`` with every
    other row zero.
    """

    def __init__(self, weights, scales):
        _require(len(weights) >= 1 and len(weights) <= 65535 and len(weights) == len(scales),
                 "Supply matching non-empty weight and scale groups")
        first = weights[0]
        _require(first.is_cuda and first.dim() == 2, "Grouped weights must be CUDA matrices")
        self.packed = _packed_weight(first)
        self.outputs = first.shape[0]
        self.inner = first.shape[1] * (2 if self.packed else 1)
        _require(self.outputs >= 8 and self.outputs % 8 == 0 and self.inner % 32 == 0,
                 "Invalid grouped weight dimensions")
        scale_rows = self.outputs if self.packed else (self.outputs + 31) // 32
        addresses = []
        for weight, scale in zip(weights, scales):
            _require(weight.device == first.device and weight.dtype == first.dtype
                     and weight.shape == first.shape and weight.is_contiguous()
                     and scale.device == first.device and _is_e8m0(scale) and scale.dim() == 2
                     and tuple(scale.shape) == (scale_rows, self.inner // 32)
                     and scale.is_contiguous(),
                     "Grouped weight shapes, dtypes, devices or scales differ")
            addresses.append([weight.data_ptr(), scale.data_ptr()])
        self.weights, self.scales = list(weights), list(scales)
        self.metadata = torch.tensor(addresses, dtype=torch.int64).to(first.device)

    def matmul(self, x, x_scale, active, counts, activation_block=32):
        """Multiply each batch of ``x`` with its expert; see the class docstring."""
        _require(x.device == self.metadata.device and x.dtype == torch.float8_e4m3fn
                 and x.dim() == 3 and x.shape[0] <= 65535 and x.shape[1] <= 65535
                 and x.shape[2] == self.inner
                 and (activation_block == 32 or (self.packed and activation_block == 128))
                 and self.inner % activation_block == 0,
                 "Invalid grouped input dimensions or activation block")
        _require(x_scale.device == x.device and _is_e8m0(x_scale)
                 and tuple(x_scale.shape) == (x.shape[0], x.shape[1], self.inner // activation_block),
                 "Grouped input scale shape or dtype mismatch")
        for index in (active, counts):
            _require(index.device == x.device and index.dtype == torch.int32 and index.dim() == 1
                     and index.numel() == x.shape[0],
                     "Grouped indices/counts require one CUDA int32 value per group")
        for value in (x, x_scale, active, counts):
            _require(value.is_contiguous(), "Grouped operands must be contiguous")
        for weight, scale, (w_address, s_address) in zip(self.weights, self.scales,
                                                         self.metadata.tolist()):
            _require(weight.data_ptr() == w_address and scale.data_ptr() == s_address,
                     "Captured weight storage changed; recreate the group")
        out = torch.empty((x.shape[0], x.shape[1], self.outputs), dtype=torch.bfloat16,
                          device=x.device)
        if x.shape[0] and x.shape[1]:
            with torch.cuda.device(x.device):
                native = _native.context(x.device.index)
                native.call("grouped_quantized_matmul", int(self.packed), x.shape[0],
                            len(self.weights), x.shape[1], self.outputs, self.inner,
                            activation_block, _pointer(x), _pointer(x_scale),
                            _pointer(self.metadata), _pointer(active), _pointer(counts),
                            _pointer(out))
        return out


def route_groups(experts, active, first_expert, rows):
    """Route ``experts`` ``[tokens, choices]`` (int64 ids) to the local groups ``active``.

    Returns ``(slots [groups, rows], reverse [tokens, choices], counts [groups])``
    as ``route_groups_public`` does (``torch_bindings.cpp:552-576``). Row ``r`` of
    group ``g`` is the ``r``-th routed slot in ascending slot order.
    """
    _require(experts.is_cuda and experts.dtype == torch.int64 and experts.dim() == 2
             and experts.is_contiguous() and 1 <= experts.shape[1] <= 64
             and experts.numel() <= _INT_MAX and active.device == experts.device
             and active.dtype == torch.int32 and active.dim() == 1 and active.is_contiguous()
             and 1 <= active.numel() <= 65535 and 1 <= rows <= 65535
             and active.numel() * rows <= _INT_MAX and first_expert >= 0,
             "Invalid expert routing dimensions, indices or devices")
    groups = active.numel()
    counts = torch.empty((groups,), dtype=torch.int32, device=experts.device)
    slots = torch.empty((groups, rows), dtype=torch.int32, device=experts.device)
    reverse = torch.empty(experts.shape, dtype=torch.int32, device=experts.device)
    with torch.cuda.device(experts.device):
        native = _native.context(experts.device.index)
        native.call("route_groups", experts.shape[0], experts.shape[1], int(first_expert), groups,
                    int(rows), _pointer(experts), _pointer(active), _pointer(counts),
                    _pointer(slots), _pointer(reverse))
    return slots, reverse, counts


def reduce_groups(grouped, experts, reverse):
    """Sum the routed BF16 rows of every token in ascending (expert, choice) order.

    ``grouped`` is ``[groups, rows, width]``; returns FP32 ``[tokens, width]``
    (``reduce_groups_public``, ``torch_bindings.cpp:578-600``).
    """
    _require(grouped.is_cuda and grouped.dtype == torch.bfloat16 and grouped.dim() == 3
             and grouped.is_contiguous() and grouped.shape[0] * grouped.shape[1] <= _INT_MAX
             and grouped.shape[2] >= 1 and experts.device == grouped.device
             and experts.dtype == torch.int64 and experts.dim() == 2 and experts.is_contiguous()
             and 1 <= experts.shape[1] <= 64 and experts.numel() <= _INT_MAX
             and reverse.device == grouped.device and reverse.dtype == torch.int32
             and reverse.shape == experts.shape and reverse.is_contiguous(),
             "Invalid grouped reduction shapes, types or devices")
    out = torch.empty((experts.shape[0], grouped.shape[2]), dtype=torch.float32,
                      device=grouped.device)
    if experts.shape[0]:
        with torch.cuda.device(grouped.device):
            native = _native.context(grouped.device.index)
            native.call("reduce_groups", experts.shape[0], experts.shape[1], grouped.shape[2],
                        grouped.shape[0] * grouped.shape[1], _pointer(experts), _pointer(reverse),
                        _pointer(grouped), _pointer(out))
    return out
