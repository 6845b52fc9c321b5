"""``sglang_b200.plugin.register()`` executed on the CPU against a hook registry.

The plugin's job is to hand SGLang's ``HookRegistry`` one (target path, callable, hook type) triple per
operator of the path. It is run here against a minimal registry with the reference's interface
(``HookRegistry.register(target, hook, hook_type)``, ``HookType.{BEFORE,AFTER,AROUND,REPLACE}``;
python/sglang/srt/plugins/hook_registry.py:60-143) and, when the environment variable
``SGLANG_REFERENCE_ROOT`` names a checkout of the reference, against the reference's own
``hook_registry.py`` loaded from that tree, where every target path is also resolved to a ``def`` in the
reference's source files."""
import ast
import enum
import importlib.util
import os
import sys
import types

import pytest


def _fake_registry_module():
    mod = types.ModuleType("sglang.srt.plugins.hook_registry")

    class HookType(enum.Enum):
        BEFORE = "before"
        AFTER = "after"
        AROUND = "around"
        REPLACE = "replace"

    class HookRegistry:
        _hooks = {}

        @classmethod
        def register(cls, target, hook, hook_type=HookType.AFTER, *, source=None):
            if isinstance(hook, type) and hook_type != HookType.REPLACE:
                raise TypeError("classes can only REPLACE")
            cls._hooks.setdefault(target, []).append((hook_type, hook, source))

    mod.HookType, mod.HookRegistry = HookType, HookRegistry
    return mod


def _real_registry_module(root):
    path = os.path.join(root, "python", "sglang", "srt", "plugins", "hook_registry.py")
    spec = importlib.util.spec_from_file_location("sglang.srt.plugins.hook_registry", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _run_register(monkeypatch, registry_mod):
    # only the leaf module is needed: the parents are empty packages so that importing the plugin does not
    # pull in the whole serving stack
    for name in ("sglang", "sglang.srt", "sglang.srt.plugins"):
        pkg = types.ModuleType(name)
        pkg.__path__ = []
        monkeypatch.setitem(sys.modules, name, pkg)
    monkeypatch.setitem(sys.modules, "sglang.srt.plugins.hook_registry", registry_mod)
    from sglang_b200 import plugin

    plugin.register()
    return plugin, registry_mod.HookRegistry._hooks, registry_mod.HookType


def _check(plugin, hooks, HookType):
    import sglang_b200 as S

    assert set(hooks) >= set(plugin.HOOKS)
    kinds = {t: hooks[t][-1][0] for t in plugin.HOOKS}
    fns = {t: hooks[t][-1][1] for t in plugin.HOOKS}
    around = {t for t, n in plugin.HOOKS.items() if n.endswith("_around")}
    for t in plugin.HOOKS:
        assert kinds[t] == (HookType.AROUND if t in around else HookType.REPLACE), t
        assert callable(fns[t])
    assert fns["sglang.srt.layers.quantization.fp8_kernel.w8a8_block_fp8_matmul"] is S.w8a8_block_fp8_matmul
    assert fns["sglang.srt.layers.quantization.fp8_kernel.per_token_group_quant_fp8"] is S.per_token_group_quant_fp8
    assert fns["sglang.srt.layers.moe.moe_runner.triton_utils.fused_moe.fused_experts"] is plugin.fused_experts_around


def test_register_against_a_minimal_registry(monkeypatch):
    plugin, hooks, HookType = _run_register(monkeypatch, _fake_registry_module())
    _check(plugin, hooks, HookType)


def test_around_hooks_fall_through_for_other_configurations():
    """The AROUND hooks must hand anything outside the block-FP8 path to the wrapped function."""
    from sglang_b200 import plugin

    seen = []

    def original(*a, **k):
        seen.append((a, k))
        return "original"

    assert plugin.fused_experts_around(original, 1, 2, 3, 4, 5, use_fp8_w8a8=False) == "original"
    assert plugin.fused_experts_around(original, 1, 2, 3, 4, 5, use_fp8_w8a8=True, block_shape=[64, 64]) == "original"
    assert len(seen) == 2 and seen[0][0] == (1, 2, 3, 4, 5)

    class Cpu:
        is_cuda = False

    assert plugin.biased_grouped_topk_around(original, None, Cpu(), None, 8, True, 8, 4) == "original"


@pytest.mark.skipif(not os.environ.get("SGLANG_REFERENCE_ROOT"), reason="SGLANG_REFERENCE_ROOT is not set")
def test_register_against_the_reference_registry(monkeypatch):
    root = os.environ["SGLANG_REFERENCE_ROOT"]
    real = _real_registry_module(root)
    real.HookRegistry._hooks.clear()
    plugin, hooks, HookType = _run_register(monkeypatch, real)
    _check(plugin, hooks, HookType)
    # every target names a function the reference really defines
    for target in plugin.HOOKS:
        module, func = target.rsplit(".", 1)
        path = os.path.join(root, "python", *module.split(".")) + ".py"
        assert os.path.exists(path), path
        tree = ast.parse(open(path).read())
        names = {n.name for n in ast.walk(tree) if isinstance(n, (ast.FunctionDef, ast.AsyncFunctionDef))}
        names |= {t.id for n in ast.walk(tree) if isinstance(n, ast.Assign) for t in n.targets if isinstance(t, ast.Name)}
        assert func in names, target
