"""sglang_b200: the block-FP8 W8A8 linear + fused-MoE hot path of SGLang on B200 (sm_100a).

Operators keep the reference's names and signatures; all compute is hand-written CUDA
behind the C ABI of ``include/b200_blockfp8.h``."""
from .fp8_kernel import (  # noqa: F401
    create_per_token_group_quant_fp8_output_scale,
    per_token_group_quant_fp8,
    set_quant_formula,
    w8a8_block_fp8_linear,
    w8a8_block_fp8_matmul,
)
from .moe_align_block_size import moe_align_block_size, sgl_moe_align_block_size  # noqa: F401

__version__ = "0.1.0"
from .fused_moe import (  # noqa: F401,E402
    MoeRunnerConfig,
    StandardTopKOutput,
    fused_experts,
    fused_moe,
    masked_fused_experts,
)
from .topk import (  # noqa: F401,E402
    TopKConfig,
    biased_grouped_topk,
    fused_topk,
    grouped_topk,
    moe_fused_gate,
    select_experts,
    topk_sigmoid,
    topk_softmax,
)
from . import fp8  # noqa: F401,E402
from . import custom_ops  # noqa: F401,E402  (registers torch.ops.sglang_b200.*)
