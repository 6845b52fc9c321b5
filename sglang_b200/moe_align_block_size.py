"""``moe_align_block_size`` with the reference's signature
(python/sglang/srt/layers/moe/moe_runner/triton_utils/moe_align_block_size.py:19-87) and
the raw out-parameter form of ``sgl_kernel.moe_align_block_size``
(sgl-kernel/python/sgl_kernel/moe.py:6-25), on the sm_100a kernels. The order of the flat
indices inside one expert is ascending (the reference leaves it unspecified)."""
from __future__ import annotations

from typing import Tuple

import torch

from . import _native as N
from .fp8_kernel import _workspace


def cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b


def sgl_moe_align_block_size(
    topk_ids: torch.Tensor,
    num_experts: int,
    block_size: int,
    sorted_token_ids: torch.Tensor,
    experts_ids: torch.Tensor,
    num_tokens_post_pad: torch.Tensor,
    cumsum_buffer: torch.Tensor,
    pad_sorted_token_ids: bool = False,
) -> None:
    """Out-parameter form. ``num_experts`` here counts BUCKETS (real experts + 1 for the
    "-1" ids), exactly as the reference passes it. ``cumsum_buffer`` needs num_experts + 1
    int32 entries."""
    N.require_cuda(topk_ids, sorted_token_ids, experts_ids, num_tokens_post_pad, cumsum_buffer)
    assert topk_ids.dtype in (torch.int32, torch.int64), "topk_ids must be int32 or int64"
    assert topk_ids.is_contiguous()
    for t in (sorted_token_ids, experts_ids, num_tokens_post_pad, cumsum_buffer):
        assert t.dtype == torch.int32 and t.is_contiguous()
    assert cumsum_buffer.numel() >= num_experts + 1
    assert num_tokens_post_pad.numel() >= 1
    lib = N.load()
    numel = topk_ids.numel()
    ws_bytes = lib.b200_moe_align_workspace_bytes(numel, num_experts)
    with N.on_device(topk_ids):
        ws = _workspace(topk_ids.device, ws_bytes)
        st = lib.b200_moe_align_block_size(
            N.ptr(topk_ids), N.DTYPE_CODE[topk_ids.dtype], numel, num_experts, block_size,
            N.ptr(sorted_token_ids), sorted_token_ids.numel(), N.ptr(experts_ids), experts_ids.numel(),
            N.ptr(num_tokens_post_pad), N.ptr(cumsum_buffer), int(pad_sorted_token_ids), N.ptr(ws), ws_bytes,
            N.current_stream(),
        )
    N.check(st, "moe_align_block_size")


def moe_align_block_size(
    topk_ids: torch.Tensor, block_size: int, num_experts: int
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns ``(sorted_token_ids, expert_ids, num_tokens_post_padded)`` sized as the
    reference sizes them; ids equal to -1 (expert on another rank) land in a leading bucket
    whose blocks carry expert id -1."""
    numel = topk_ids.numel()
    if numel < num_experts + 1:
        max_num_tokens_padded = numel * block_size
    else:
        max_num_tokens_padded = numel + (num_experts + 1) * (block_size - 1)
    dev = topk_ids.device
    sorted_ids = torch.empty((max_num_tokens_padded,), dtype=torch.int32, device=dev)
    expert_ids = torch.empty((cdiv(max_num_tokens_padded, block_size),), dtype=torch.int32, device=dev)
    num_tokens_post_pad = torch.empty((1,), dtype=torch.int32, device=dev)
    cumsum_buffer = torch.empty((num_experts + 2,), dtype=torch.int32, device=dev)
    sgl_moe_align_block_size(
        topk_ids, num_experts + 1, block_size, sorted_ids, expert_ids, num_tokens_post_pad, cumsum_buffer, True
    )
    return sorted_ids, expert_ids, num_tokens_post_pad
