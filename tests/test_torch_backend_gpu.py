"""The ATen overrides and the SGLang hooks on a GPU, each in a fresh process.

The overrides are process-wide once installed, so every scenario runs in its own
interpreter with ``CAMBLAS_ENABLE=1``, as the reference's tests require
(tests/test_linear.py:12-15). Checks follow tests/test_linear.py: results
against CPU FP64 with the BF16 tolerance rtol 2**-6 / atol 0.002 (:40-46), a
launch counter must move when a call is intercepted (:63-65), strided and empty
shapes (:72-84), one version bump for ``out=`` (:105-108), and CUDA-graph
capture on a side stream with inputs mutated before replay (:148-169).
"""

import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]

PRELUDE = """
import sys
sys.path.insert(0, %r)
import torch
import torch.nn.functional as F
import camblas_b200
from camblas_b200 import _native, _kernels
camblas_b200._autoload()
from camblas_b200 import _torch_backend
assert _torch_backend.installed()

def close(actual, expected):
    torch.testing.assert_close(actual.double().cpu(), expected, rtol=2 ** -6, atol=0.002)

def launches():
    counts = _native.stats(0, all_threads=True)
    return counts["classical"] + counts["lt"]
""" % str(ROOT)


def run(body, **environment):
    env = dict(os.environ, CAMBLAS_ENABLE="1", **environment)
    script = PRELUDE + textwrap.dedent(body) + "\nprint('SCENARIO-OK')\n"
    result = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, env=env,
                            timeout=600)
    assert result.returncode == 0 and "SCENARIO-OK" in result.stdout, result.stdout + result.stderr


def test_linear_mm_addmm_matmul_are_intercepted_and_correct():
    run("""
    torch.manual_seed(705537)
    x = torch.randn(48, 256, device="cuda").bfloat16()
    w = torch.randn(384, 256, device="cuda").bfloat16()
    b = torch.randn(384, device="cuda").bfloat16()
    xd, wd, bd = x.double().cpu(), w.double().cpu(), b.double().cpu()
    before = launches()
    close(F.linear(x, w), xd @ wd.t())
    close(F.linear(x, w, b), xd @ wd.t() + bd)
    close(torch.mm(x, w.t()), xd @ wd.t())
    close(torch.matmul(x, w.t()), xd @ wd.t())
    close(x @ w.t().contiguous(), xd @ wd.t())
    c = torch.randn(48, 384, device="cuda").bfloat16()
    close(torch.addmm(c, x, w.t(), beta=0.5, alpha=-1.25), 0.5 * c.double().cpu() - 1.25 * (xd @ wd.t()))
    close(torch.addmm(b, x, w.t(), beta=0), xd @ wd.t())
    assert launches() - before == 7, launches() - before
    # three-dimensional input flattens to one GEMM
    close(F.linear(x.view(4, 12, 256), w, b), (xd @ wd.t() + bd).view(4, 12, 384))
    # FP32 is not intercepted and still works
    before = launches()
    y = torch.mm(x.float(), w.float().t())
    assert launches() == before
    torch.testing.assert_close(y.double().cpu(), xd @ wd.t(), rtol=1e-2, atol=1e-2)
    assert _native.context(0).device_status() == 0
    """, CAMBLAS_CUDA_ALGORITHM="lt")


def test_strided_empty_out_and_autograd():
    run("""
    torch.manual_seed(73013)
    base = torch.randn(64, 520, device="cuda").bfloat16()
    x = base[:, 4:260]   # row stride 520 and a start that is not 16-byte aligned
    wt = torch.randn(256, 136, device="cuda").bfloat16()
    close(torch.mm(x, wt), x.double().cpu() @ wt.double().cpu())
    a = torch.randn(40, 72, device="cuda").bfloat16()
    b = torch.randn(72, 56, device="cuda").bfloat16()
    for left in (a, a.t().contiguous().t()):
        for right in (b, b.t().contiguous().t()):
            close(torch.mm(left, right), a.double().cpu() @ b.double().cpu())
    odd = torch.randn(40, 144, device="cuda").bfloat16()[:, ::2]     # inner stride 2 -> copied
    close(torch.mm(odd, b), odd.double().cpu() @ b.double().cpu())
    assert torch.mm(a[:0], b).shape == (0, 56)
    assert torch.mm(a[:, :0], b[:0]).abs().sum() == 0
    out = torch.empty(40, 56, device="cuda", dtype=torch.bfloat16)
    version = out._version
    result = torch.mm(a, b, out=out)
    assert result is out and out._version == version + 1
    close(out, a.double().cpu() @ b.double().cpu())
    # gradients flow through the overridden kernels (mm backward is two more mm calls)
    p = a.clone().requires_grad_(True)
    q = b.clone().requires_grad_(True)
    before = launches()
    torch.mm(p, q).float().sum().backward()
    assert launches() - before == 3
    ones = torch.ones(40, 56, dtype=torch.double)
    close(p.grad, ones @ b.double().cpu().t())
    close(q.grad, a.double().cpu().t() @ ones)
    """)


def test_cuda_graph_capture_and_replay_on_a_side_stream():
    run("""
    torch.manual_seed(20261004)
    for rows in (1, 24, 200):
        x = torch.randn(rows, 4096, device="cuda").bfloat16()
        w = torch.randn(512, 4096, device="cuda").bfloat16()
        b = torch.randn(512, device="cuda").bfloat16()
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.inference_mode(), torch.cuda.stream(stream):
            F.linear(x, w, b)                      # warm up: context and scratch on this stream
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                y = F.linear(x, w, b)
            x.copy_(torch.randn(rows, 4096, device="cuda").bfloat16())
            w.mul_(0.5)
            graph.replay()
        stream.synchronize()
        close(y, x.double().cpu() @ w.double().cpu().t() + b.double().cpu())
        graph.reset()
    # a context cannot be created while its stream is being captured
    fresh = torch.cuda.Stream()
    with torch.cuda.stream(fresh):
        graph = torch.cuda.CUDAGraph()
        try:
            with torch.cuda.graph(graph, stream=fresh):
                F.linear(x, w)
        except RuntimeError as error:
            assert "Warm up CAMBLAS" in str(error), error
        else:
            raise AssertionError("capture without a warm-up must be refused")
    """)


def test_unknown_algorithm_is_rejected():
    env = dict(os.environ, CAMBLAS_ENABLE="1", CAMBLAS_CUDA_ALGORITHM="fastest")
    script = ("import sys; sys.path.insert(0, %r); import camblas_b200\n"
              "try:\n    camblas_b200._autoload()\nexcept ValueError as error:\n"
              "    print('REJECTED', error)\n") % str(ROOT)
    result = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, env=env)
    assert "REJECTED Unknown CAMBLAS CUDA algorithm" in result.stdout, result.stdout + result.stderr


def test_sglang_hooks_on_cuda_tensors():
    run("""
    import types
    from tests.sglang_stub import install_stub
    from camblas_b200 import sglang as plugin
    from oracle import oracle
    import numpy as np
    registry = install_stub()
    plugin.install()
    hooks = {name.rsplit(".", 1)[-1]: function for name, (function, _) in registry.hooks.items()}
    assert len(hooks) == 5

    def original(*arguments):
        raise AssertionError("an eligible call fell back to the original function")

    torch.manual_seed(5)
    x = torch.randn(2, 3, 256, device="cuda").bfloat16()
    layer = types.SimpleNamespace(weight=torch.randn(128, 256, device="cuda").bfloat16())
    bias = torch.randn(128, device="cuda").bfloat16()
    y = hooks["apply"](original, None, layer, x, bias)
    assert y.shape == (2, 3, 128)
    close(y, x.double().cpu() @ layer.weight.double().cpu().t() + bias.double().cpu())
    # batched projection, the reference's shape (2, 1, 128) x (2, 2048, 128) and a larger one
    torch.set_grad_enabled(False)
    for batch, rows, outputs, inner in ((2, 1, 2048, 128), (3, 70, 136, 256)):
        entries = torch.randn(batch, rows, inner, device="cuda").bfloat16()
        stacked = types.SimpleNamespace(weight=torch.randn(batch, outputs, inner, device="cuda").bfloat16())
        y = hooks["forward"](original, stacked, entries)
        assert y.shape == (batch, rows, outputs)
        close(y, torch.bmm(entries.double().cpu(), stacked.weight.double().cpu().transpose(1, 2)))
    torch.set_grad_enabled(True)
    # block-128 dense hook, several token rows
    rows, outputs, inner = 5, 384, 512
    x = torch.randn(rows, inner, device="cuda").bfloat16()
    w = torch.randn(outputs, inner).bfloat16()
    wq, ws = oracle.fp8_quantize_weight(w.view(torch.int16).numpy().view(np.uint16))
    weight = torch.from_numpy(wq).cuda().view(torch.float8_e4m3fn)
    scale = torch.from_numpy(ws).cuda()
    torch.set_grad_enabled(False)  # SGLang serves under inference mode; the FP8 hooks require it
    y = hooks["deepgemm_w8a8_block_fp8_linear_with_fallback"](original, x, weight, [128, 128], scale)
    exact = x.double().cpu() @ w.double().t()
    assert ((y.double().cpu() - exact).norm() / exact.norm()) < 0.05
    # block-32 hooks, one token
    outputs, inner = 64, 256
    token = torch.randn(1, inner, device="cuda").bfloat16()
    w8 = torch.randn(outputs, inner, device="cuda").to(torch.float8_e4m3fn)
    sw = torch.rand(outputs // 32, inner // 32, device="cuda") + 0.5
    fused = hooks["triton_w8a8_block_fp8_linear"](original, token, w8, [32, 32], sw, None, None, True)
    host = token.cpu().view(torch.int16).numpy().view(np.uint16).ravel()
    q, sx = oracle.fp8_quantize_block32(host)
    a = torch.from_numpy(q).cuda().view(torch.float8_e4m3fn).view(1, inner)
    split = hooks["w8a8_block_fp8_matmul_triton"](original, a, w8, torch.from_numpy(sx).cuda().view(1, -1),
                                                  sw, [32, 32], torch.bfloat16)
    assert fused.shape == split.shape == (1, outputs) and torch.equal(fused, split)
    counts = plugin.dispatch_counts()
    assert counts["linear"] == 1 and counts["fp8"] == 3 and counts["fp8_dense_block128"] == 1
    assert counts["bmm"] == 2
    # ineligible inputs reach the original
    marker = object()
    assert hooks["apply"](lambda *a: marker, None, layer, x.float()[:, :256], None) is marker
    """, CAMBLAS_SGLANG_OPS="linear,fp8", PYTHONPATH=str(ROOT))
