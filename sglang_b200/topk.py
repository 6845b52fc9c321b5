"""Routing that feeds ``fused_experts``: softmax / sigmoid top-k and DeepSeek-style biased
grouped top-k, with the reference's function names and argument order
(python/sglang/srt/layers/moe/topk.py: ``fused_topk_torch_native`` :550-588,
``biased_grouped_topk_impl`` :923-992). This is the step BEFORE the hot path; it is stated
here in torch ops on the tensors' own device so that benchmarks and callers can produce
``(topk_weights fp32, topk_ids int32)`` without the reference installed."""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def fused_topk(
    hidden_states: torch.Tensor,
    gating_output: torch.Tensor,
    topk: int,
    renormalize: bool,
    correction_bias: Optional[torch.Tensor] = None,
    scoring_func: str = "softmax",
) -> Tuple[torch.Tensor, torch.Tensor]:
    assert hidden_states.shape[0] == gating_output.shape[0], "Number of tokens mismatch"
    if scoring_func == "softmax":
        scores = gating_output.float().softmax(dim=-1)
    elif scoring_func == "sigmoid":
        scores = gating_output.float().sigmoid()
    else:
        raise ValueError(f"Invalid scoring function: {scoring_func}")
    if correction_bias is not None:
        ids = torch.topk(scores + correction_bias.unsqueeze(0), k=topk, dim=-1, sorted=False)[1]
        w = scores.gather(1, ids)
    else:
        w, ids = torch.topk(scores, topk, dim=-1)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return w.to(torch.float32), ids.to(torch.int32)


def biased_grouped_topk(
    hidden_states: torch.Tensor,
    gating_output: torch.Tensor,
    correction_bias: torch.Tensor,
    topk: int,
    renormalize: bool,
    num_expert_group: int,
    topk_group: int,
    routed_scaling_factor: Optional[float] = None,
    apply_routed_scaling_factor_on_output: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sigmoid scores; a group's score is the sum of its two best biased scores; keep
    ``topk_group`` groups; take the top-k biased scores among them; weights are the unbiased
    scores, renormalised."""
    assert hidden_states.shape[0] == gating_output.shape[0], "Number of tokens mismatch"
    scores = gating_output.float().sigmoid()
    T, E = scores.shape
    sfc = scores + correction_bias.float().unsqueeze(0)
    group_scores = sfc.view(T, num_expert_group, -1).topk(2, dim=-1)[0].sum(dim=-1)
    group_idx = torch.topk(group_scores, k=topk_group, dim=-1, sorted=False)[1]
    group_mask = torch.zeros_like(group_scores)
    group_mask.scatter_(1, group_idx, 1)
    score_mask = group_mask.unsqueeze(-1).expand(T, num_expert_group, E // num_expert_group).reshape(T, -1)
    tmp = sfc.masked_fill(~score_mask.bool(), float("-inf"))
    ids = torch.topk(tmp, k=topk, dim=-1, sorted=False)[1]
    w = scores.gather(1, ids)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
        if apply_routed_scaling_factor_on_output and routed_scaling_factor is not None:
            w = w * routed_scaling_factor
    return w.to(torch.float32), ids.to(torch.int32)
