"""SGLang plugin entry point: REPLACE-hooks the four operators of the block-FP8 path.

Register it under the setuptools entry-point group ``sglang.srt.plugins``
(python/sglang/srt/plugins/__init__.py:29,103-141):

    [project.entry-points."sglang.srt.plugins"]
    b200_blockfp8 = "sglang_b200.plugin:register"
"""
from __future__ import annotations

HOOKS = {
    "sglang.srt.layers.quantization.fp8_kernel.per_token_group_quant_fp8": "per_token_group_quant_fp8",
    "sglang.srt.layers.quantization.fp8_kernel.sglang_per_token_group_quant_fp8": "per_token_group_quant_fp8",
    "sglang.srt.layers.quantization.fp8_kernel.w8a8_block_fp8_matmul": "w8a8_block_fp8_matmul",
    "sglang.srt.layers.moe.moe_runner.triton_utils.moe_align_block_size.moe_align_block_size": "moe_align_block_size",
    "sglang.srt.layers.moe.moe_runner.triton_utils.fused_moe.fused_experts": "fused_experts_around",
}



def fused_experts_around(original_fn, hidden_states, w1, w2, topk_output, moe_runner_config, *args, **kwargs):
    """AROUND hook: the B200 kernels for ``use_fp8_w8a8=True, block_shape=[128, 128]``; every
    other configuration goes to the function being wrapped."""
    from . import fused_moe

    block_shape = kwargs.get("block_shape")
    if kwargs.get("use_fp8_w8a8") and block_shape is not None and list(block_shape) == [128, 128]:
        return fused_moe.fused_experts(hidden_states, w1, w2, topk_output, moe_runner_config, *args, **kwargs)
    return original_fn(hidden_states, w1, w2, topk_output, moe_runner_config, *args, **kwargs)


def register() -> None:
    """Called by SGLang's ``load_plugins()`` in every process."""
    from sglang.srt.plugins.hook_registry import HookRegistry, HookType  # hook_registry.py:84-143

    import sglang_b200 as S

    impl = {
        "per_token_group_quant_fp8": (S.per_token_group_quant_fp8, HookType.REPLACE),
        "w8a8_block_fp8_matmul": (S.w8a8_block_fp8_matmul, HookType.REPLACE),
        "moe_align_block_size": (S.moe_align_block_size, HookType.REPLACE),
        "fused_experts_around": (fused_experts_around, HookType.AROUND),
    }
    for target, name in HOOKS.items():
        fn, kind = impl[name]
        HookRegistry.register(target, fn, kind)
