"""A stand-in for ``sglang.srt.plugins.hook_registry`` (SGLang is not installable offline).

Records what the plugin registers, the way the reference's own test mocks
``HookRegistry.register`` (tests/test_sglang.py:62-72).
"""

import enum
import sys
import types


class HookType(enum.Enum):
    BEFORE = "before"
    AFTER = "after"
    AROUND = "around"


class HookRegistry:
    hooks = {}

    @classmethod
    def register(cls, target, function, hook_type):
        cls.hooks[target] = (function, hook_type)


def install_stub():
    """Put the stub into ``sys.modules`` under SGLang's module path and reset it."""
    HookRegistry.hooks = {}
    names = ["sglang", "sglang.srt", "sglang.srt.plugins", "sglang.srt.plugins.hook_registry"]
    for name in names:
        sys.modules.setdefault(name, types.ModuleType(name))
    module = sys.modules["sglang.srt.plugins.hook_registry"]
    module.HookRegistry = HookRegistry
    module.HookType = HookType
    return HookRegistry
