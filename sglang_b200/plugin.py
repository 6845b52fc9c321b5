"""SGLang plugin entry point: hooks the operators of the block-FP8 path and the routing step
before it.

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
    "sglang.srt.layers.moe.topk.fused_topk": "fused_topk",
    "sglang.srt.layers.moe.topk.biased_grouped_topk_gpu": "biased_grouped_topk_around",
}



def fused_experts_around(original_fn, hidden_states, w1, w2, topk_output, moe_runner_config, *args, **kwargs):
    """AROUND hook: the B200 kernels for ``use_fp8_w8a8=True, block_shape=[128, 128]``; every
    other configuration goes to the function being wrapped."""
    from . import fused_moe

    block_shape = kwargs.get("block_shape")
    if kwargs.get("use_fp8_w8a8") and block_shape is not None and list(block_shape) == [128, 128]:
        return fused_moe.fused_experts(hidden_states, w1, w2, topk_output, moe_runner_config, *args, **kwargs)
    return original_fn(hidden_states, w1, w2, topk_output, moe_runner_config, *args, **kwargs)


def biased_grouped_topk_around(original_fn, hidden_states, gating_output, correction_bias, topk, renormalize,
                               num_expert_group=None, topk_group=None, num_fused_shared_experts=0,
                               routed_scaling_factor=None, apply_routed_scaling_factor_on_output=False):
    """AROUND hook for ``biased_grouped_topk_gpu`` (python/sglang/srt/layers/moe/topk.py:1022-1033):
    the B200 routing kernel for CUDA tensors (fused shared experts included)."""
    from . import topk as routing

    if not gating_output.is_cuda:
        return original_fn(hidden_states, gating_output, correction_bias, topk, renormalize, num_expert_group,
                           topk_group, num_fused_shared_experts, routed_scaling_factor,
                           apply_routed_scaling_factor_on_output)
    return routing.biased_grouped_topk(hidden_states, gating_output, correction_bias, topk, renormalize,
                                       num_expert_group, topk_group, num_fused_shared_experts, routed_scaling_factor,
                                       apply_routed_scaling_factor_on_output)


def register() -> None:
    """Called by SGLang's ``load_plugins()`` in every process."""
    from sglang.srt.plugins.hook_registry import HookRegistry, HookType  # hook_registry.py:84-143

    import sglang_b200 as S

    impl = {
        "per_token_group_quant_fp8": (S.per_token_group_quant_fp8, HookType.REPLACE),
        "w8a8_block_fp8_matmul": (S.w8a8_block_fp8_matmul, HookType.REPLACE),
        "moe_align_block_size": (S.moe_align_block_size, HookType.REPLACE),
        "fused_experts_around": (fused_experts_around, HookType.AROUND),
        "fused_topk": (S.fused_topk, HookType.REPLACE),
        "biased_grouped_topk_around": (biased_grouped_topk_around, HookType.AROUND),
    }
    for target, name in HOOKS.items():
        fn, kind = impl[name]
        HookRegistry.register(target, fn, kind)
