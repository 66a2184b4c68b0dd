"""The SGLang plugin against a stub hook registry, on CPU: selection, registration, fallbacks."""

import types

import pytest
import torch

from camblas_b200 import sglang as plugin
from tests.sglang_stub import HookType, install_stub

TARGETS = {
    "linear": ["sglang.srt.layers.quantization.unquant.UnquantizedLinearMethod.apply",
               "sglang.srt.layers.linear.ColumnParallelBatchedLinear.forward"],
    "fp8": ["sglang.srt.layers.quantization.fp8_utils.deepgemm_w8a8_block_fp8_linear_with_fallback",
            "sglang.kernels.ops.quantization.fp8_kernel.w8a8_block_fp8_matmul_triton",
            "sglang.srt.layers.quantization.fp8_utils.triton_w8a8_block_fp8_linear"],
}


def test_nothing_selected_registers_nothing(monkeypatch):
    registry = install_stub()
    monkeypatch.delenv("CAMBLAS_SGLANG_OPS", raising=False)
    plugin.install()
    assert registry.hooks == {}


def test_unknown_operation_is_rejected(monkeypatch):
    install_stub()
    monkeypatch.setenv("CAMBLAS_SGLANG_OPS", "linear,attention")
    with pytest.raises(ValueError, match="Unknown CAMBLAS SGLang operations"):
        plugin.install()


def test_fp8_hooks_register_and_fall_back_on_cpu(monkeypatch):
    registry = install_stub()
    monkeypatch.setenv("CAMBLAS_SGLANG_OPS", "fp8")
    plugin.install()
    assert sorted(registry.hooks) == sorted(TARGETS["fp8"])
    assert all(kind is HookType.AROUND for _, kind in registry.hooks.values())
    before = plugin.dispatch_counts()
    seen = []

    def original(*arguments):
        seen.append(arguments)
        return "original"

    x = torch.zeros(1, 256, dtype=torch.bfloat16)
    weight = torch.zeros(128, 256).to(torch.float8_e4m3fn)
    scale = torch.ones(1, 2)
    dense = registry.hooks[TARGETS["fp8"][0]][0]
    assert dense(original, x, weight, [128, 128], scale) == "original"  # CPU tensors are not taken
    assert seen[-1] == (x, weight, [128, 128], scale, None, None)
    product = registry.hooks[TARGETS["fp8"][1]][0]
    a = torch.zeros(1, 256).to(torch.float8_e4m3fn)
    assert product(original, a, weight, torch.ones(1, 8), torch.ones(4, 8), [32, 32], torch.bfloat16) == "original"
    linear32 = registry.hooks[TARGETS["fp8"][2]][0]
    assert linear32(original, x, weight, [32, 32], torch.ones(4, 8), None, None, True) == "original"
    assert len(seen[-1]) == 8
    assert plugin.dispatch_counts() == before


def test_linear_hook_falls_back_for_ineligible_inputs(monkeypatch):
    registry = install_stub()
    monkeypatch.setenv("CAMBLAS_SGLANG_OPS", "linear")
    installed = []
    monkeypatch.setattr("camblas_b200._torch_backend.install_torch_backend", installed.append)
    monkeypatch.setenv("CAMBLAS_SGLANG_ALGORITHM", "classical")
    plugin.install()
    assert installed == ["classical"]
    assert list(registry.hooks) == TARGETS["linear"]
    hook = registry.hooks[TARGETS["linear"][0]][0]
    layer = types.SimpleNamespace(weight=torch.zeros(8, 16, dtype=torch.bfloat16))
    x = torch.zeros(2, 3, 16, dtype=torch.bfloat16)
    calls = []
    result = hook(lambda *arguments: calls.append(arguments) or "original", "method", layer, x, None)
    assert result == "original" and calls == [("method", layer, x, None)]
    batched = registry.hooks[TARGETS["linear"][1]][0]
    stacked = types.SimpleNamespace(weight=torch.zeros(2, 8, 16, dtype=torch.bfloat16))
    entries = torch.zeros(2, 1, 16, dtype=torch.bfloat16)
    assert batched(lambda *arguments: "original", stacked, entries) == "original"  # CPU tensors
