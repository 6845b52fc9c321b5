"""Expert routing that feeds ``fused_experts``: softmax / sigmoid top-k, grouped top-k and the
DeepSeek-style biased grouped top-k, with the reference's function names and argument order
(python/sglang/srt/layers/moe/topk.py: ``fused_topk`` :640-700, ``grouped_topk_gpu`` :703-764,
``biased_grouped_topk_impl`` :923-992, ``select_experts`` :1355-1500; sgl-kernel's in-place
``topk_softmax`` / ``topk_sigmoid`` / ``moe_fused_gate``). One hand-written warp-per-token CUDA
kernel behind ``b200_route_topk`` computes all of them; CUDA tensors only, no fallback.

Ties go to the lower expert index and results come in descending order of the selection value
(the reference's ``sorted=False`` calls leave the order unspecified)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _native as N

SOFTMAX, SIGMOID = 0, 1
GROUP_MAX, GROUP_TOP2_SUM = 0, 1


def _route(
    gating_output: torch.Tensor,
    topk: int,
    renormalize: bool,
    scoring: int,
    correction_bias: Optional[torch.Tensor] = None,
    num_expert_group: int = 0,
    topk_group: int = 0,
    group_score: int = GROUP_MAX,
    output_scale: float = 1.0,
    num_token_non_padded: Optional[torch.Tensor] = None,
    topk_weights: Optional[torch.Tensor] = None,
    topk_ids: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    assert gating_output.dim() == 2, "gating_output must be [num_tokens, num_experts]"
    N.require_cuda(gating_output)
    assert gating_output.dtype in (torch.float32, torch.bfloat16, torch.float16), "unsupported logits dtype"
    logits = gating_output if gating_output.is_contiguous() else gating_output.contiguous()
    T, E = logits.shape
    dev = logits.device
    if topk_weights is None:
        topk_weights = torch.empty(T, topk, dtype=torch.float32, device=dev)
    if topk_ids is None:
        topk_ids = torch.empty(T, topk, dtype=torch.int32, device=dev)
    assert topk_weights.dtype == torch.float32 and topk_ids.dtype == torch.int32
    assert topk_weights.is_contiguous() and topk_ids.is_contiguous()
    assert tuple(topk_weights.shape) == (T, topk) and tuple(topk_ids.shape) == (T, topk)
    bias = None
    if correction_bias is not None:
        assert correction_bias.numel() == E, "correction_bias must have one entry per expert"
        bias = correction_bias.to(device=dev, dtype=torch.float32).contiguous()
    nvalid = None
    if num_token_non_padded is not None:
        nvalid = num_token_non_padded.to(device=dev, dtype=torch.int32).reshape(1)
    if T == 0:
        return topk_weights, topk_ids
    with N.on_device(logits):
        st = N.load().b200_route_topk(
            N.ptr(logits), N.DTYPE_CODE[logits.dtype], N.ptr(bias), T, E, topk, scoring, num_expert_group or 0,
            topk_group or 0, group_score, int(bool(renormalize)), float(output_scale), N.ptr(nvalid),
            N.ptr(topk_weights), N.ptr(topk_ids), N.current_stream(),
        )
    N.check(st, "route_topk")
    return topk_weights, topk_ids


def _scoring_code(scoring_func: str) -> int:
    if scoring_func == "softmax":
        return SOFTMAX
    if scoring_func == "sigmoid":
        return SIGMOID
    raise ValueError(f"Invalid scoring function: {scoring_func}")


# ------------------------------------------------------------- sgl-kernel style (in place)
def topk_softmax(
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    gating_output: torch.Tensor,
    renormalize: bool = False,
    moe_softcapping: float = 0.0,
    correction_bias: Optional[torch.Tensor] = None,
) -> None:
    """sgl-kernel ``topk_softmax`` (sgl-kernel/python/sgl_kernel/moe.py:28-54): fills the two outputs.
    ``moe_softcapping != 0`` turns the logits into ``tanh(x / cap) * cap`` and ``correction_bias`` (fp32
    ``[num_experts]``) is added to them, both BEFORE the softmax, as the reference kernel does
    (moe_topk_softmax_kernels.cu:107-115)."""
    if moe_softcapping == 0.0 and correction_bias is None:
        _route(gating_output, topk_ids.shape[1], renormalize, SOFTMAX, topk_weights=topk_weights, topk_ids=topk_ids)
        return
    assert gating_output.dim() == 2, "gating_output must be [num_tokens, num_experts]"
    N.require_cuda(gating_output, topk_weights, topk_ids)
    assert gating_output.dtype in (torch.float32, torch.bfloat16, torch.float16), "unsupported logits dtype"
    logits = gating_output if gating_output.is_contiguous() else gating_output.contiguous()
    T, E = logits.shape
    topk = topk_ids.shape[1]
    assert topk_weights.dtype == torch.float32 and topk_ids.dtype == torch.int32
    assert topk_weights.is_contiguous() and topk_ids.is_contiguous()
    assert tuple(topk_weights.shape) == (T, topk) and tuple(topk_ids.shape) == (T, topk)
    if correction_bias is not None:
        assert correction_bias.dim() == 1 and correction_bias.shape[0] == E, "correction_bias size must match num_experts"
        assert correction_bias.dtype == torch.float32, "correction_bias must be float32"
        N.require_cuda(correction_bias)
        correction_bias = correction_bias.contiguous()
    if T == 0:
        return
    with N.on_device(logits):
        st = N.load().b200_route_topk_softmax_capped(
            N.ptr(logits), N.DTYPE_CODE[logits.dtype], float(moe_softcapping), N.ptr(correction_bias), T, E, topk,
            int(bool(renormalize)), N.ptr(topk_weights), N.ptr(topk_ids), N.current_stream(),
        )
    N.check(st, "route_topk_softmax_capped")


def topk_sigmoid(
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    gating_output: torch.Tensor,
    renormalize: bool = False,
    correction_bias: Optional[torch.Tensor] = None,
) -> None:
    """sgl-kernel ``topk_sigmoid``: sigmoid scores, selection on ``scores + correction_bias``."""
    _route(gating_output, topk_ids.shape[1], renormalize, SIGMOID, correction_bias,
           topk_weights=topk_weights, topk_ids=topk_ids)


def moe_fused_gate(
    input_tensor: torch.Tensor,
    bias: torch.Tensor,
    num_expert_group: int,
    topk_group: int,
    topk: int,
    num_fused_shared_experts: int = 0,
    routed_scaling_factor: float = 0.0,
    apply_routed_scaling_factor_on_output: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """sgl-kernel ``moe_fused_gate``: sigmoid + bias, top-2-sum group selection, top-k, renormalised."""
    if num_fused_shared_experts:
        raise NotImplementedError("fused shared experts are not part of this path")
    scale = routed_scaling_factor if apply_routed_scaling_factor_on_output else 1.0
    return _route(input_tensor, topk, True, SIGMOID, bias, num_expert_group, topk_group, GROUP_TOP2_SUM, scale)


def _with_fused_shared_experts(raw_weights: torch.Tensor, topk_ids: torch.Tensor, num_experts: int,
                               num_fused_shared_experts: int, renormalize: bool, routed_scaling_factor: Optional[float],
                               apply_routed_scaling_factor_on_output: bool,
                               num_token_non_padded: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """The tail of the reference's grouped routing functions when shared experts are fused into the routed ones
    (topk.py:735-764, 968-992): ``raw_weights`` / ``topk_ids`` are the un-normalised top-k in descending order;
    the LAST slot is handed to a shared-expert replica drawn uniformly from ``[num_experts, num_experts +
    num_fused_shared_experts)`` with weight ``sum(routed weights) / routed_scaling_factor`` (left as it is when
    no factor is given), and renormalisation divides by the sum of the routed slots only. A handful of
    elementwise torch ops on ``[T, k]`` tensors; the selection itself is the CUDA kernel's."""
    T, k = topk_ids.shape
    assert k >= 2, "fused shared experts need at least one routed slot"
    weights, ids = raw_weights.clone(), topk_ids.clone()
    ids[:, -1] = torch.randint(num_experts, num_experts + num_fused_shared_experts, (T,), dtype=ids.dtype, device=ids.device)
    routed_sum = weights[:, :-1].sum(dim=-1)
    if routed_scaling_factor is not None:
        weights[:, -1] = routed_sum / routed_scaling_factor
    if renormalize:
        weights = weights / routed_sum.unsqueeze(-1)
        if apply_routed_scaling_factor_on_output:
            weights = weights * routed_scaling_factor
    if num_token_non_padded is not None:  # rows past the real tokens carry id -1, as without shared experts
        pad = torch.arange(T, device=ids.device) >= num_token_non_padded.to(ids.device)
        ids[pad] = -1
    return weights.to(torch.float32), ids.to(torch.int32)


# --------------------------------------------------------------------- topk.py functions
def fused_topk(
    hidden_states: torch.Tensor,
    gating_output: torch.Tensor,
    topk: int,
    renormalize: bool,
    correction_bias: Optional[torch.Tensor] = None,
    scoring_func: str = "softmax",
    num_token_non_padded: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Softmax or sigmoid top-k (python/sglang/srt/layers/moe/topk.py:640-700). As in the reference's GPU
    path, ``correction_bias`` takes part in the selection only for ``scoring_func="sigmoid"``
    (``topk_sigmoid``); the softmax branch calls ``topk_softmax`` without it."""
    assert hidden_states.shape[0] == gating_output.shape[0], "Number of tokens mismatch"
    code = _scoring_code(scoring_func)
    return _route(gating_output, topk, renormalize, code, correction_bias if code == SIGMOID else None,
                  num_token_non_padded=num_token_non_padded)


def grouped_topk(
    hidden_states: torch.Tensor,
    gating_output: torch.Tensor,
    topk: int,
    renormalize: bool,
    num_expert_group: Optional[int] = None,
    topk_group: Optional[int] = None,
    num_fused_shared_experts: int = 0,
    routed_scaling_factor: Optional[float] = None,
    apply_routed_scaling_factor_on_output: bool = False,
    num_token_non_padded: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Softmax scores, a group's score is its maximum (DeepSeek-V2 routing)."""
    assert hidden_states.shape[0] == gating_output.shape[0], "Number of tokens mismatch"
    if num_fused_shared_experts:
        raw, ids = _route(gating_output, topk, False, SOFTMAX, None, num_expert_group, topk_group, GROUP_MAX, 1.0)
        return _with_fused_shared_experts(raw, ids, gating_output.shape[1], num_fused_shared_experts, renormalize,
                                          routed_scaling_factor, apply_routed_scaling_factor_on_output,
                                          num_token_non_padded)
    scale = 1.0
    if renormalize and apply_routed_scaling_factor_on_output and routed_scaling_factor is not None:
        scale = routed_scaling_factor
    return _route(gating_output, topk, renormalize, SOFTMAX, None, num_expert_group, topk_group, GROUP_MAX, scale,
                  num_token_non_padded)


def biased_grouped_topk(
    hidden_states: torch.Tensor,
    gating_output: torch.Tensor,
    correction_bias: torch.Tensor,
    topk: int,
    renormalize: bool,
    num_expert_group: Optional[int] = None,
    topk_group: Optional[int] = None,
    num_fused_shared_experts: int = 0,
    routed_scaling_factor: Optional[float] = None,
    apply_routed_scaling_factor_on_output: bool = False,
    num_token_non_padded: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sigmoid scores; a group's score is the sum of its two best biased scores; keep
    ``topk_group`` groups; take the top-k biased scores among them; weights are the unbiased
    scores, renormalised (DeepSeek-V3 routing)."""
    assert hidden_states.shape[0] == gating_output.shape[0], "Number of tokens mismatch"
    if num_fused_shared_experts:
        raw, ids = _route(gating_output, topk, False, SIGMOID, correction_bias, num_expert_group, topk_group,
                          GROUP_TOP2_SUM, 1.0)
        return _with_fused_shared_experts(raw, ids, gating_output.shape[1], num_fused_shared_experts, renormalize,
                                          routed_scaling_factor, apply_routed_scaling_factor_on_output,
                                          num_token_non_padded)
    scale = 1.0
    if renormalize and apply_routed_scaling_factor_on_output and routed_scaling_factor is not None:
        scale = routed_scaling_factor
    return _route(gating_output, topk, renormalize, SIGMOID, correction_bias, num_expert_group, topk_group,
                  GROUP_TOP2_SUM, scale, num_token_non_padded)


@dataclass
class TopKConfig:
    """The routing knobs of the reference's ``TopKConfig`` (topk.py:199-214) this path reads."""

    top_k: int
    use_grouped_topk: bool = False
    topk_group: Optional[int] = None
    num_expert_group: Optional[int] = None
    renormalize: bool = True
    num_fused_shared_experts: int = 0
    correction_bias: Optional[torch.Tensor] = None
    routed_scaling_factor: Optional[float] = None
    apply_routed_scaling_factor_on_output: bool = False
    scoring_func: str = "softmax"


def select_experts(
    hidden_states: torch.Tensor,
    router_logits: torch.Tensor,
    topk_config: TopKConfig,
    num_token_non_padded: Optional[torch.Tensor] = None,
):
    """Dispatch of the reference's ``select_experts`` (topk.py:1355-1500): grouped (with or
    without correction bias) or plain top-k; returns ``StandardTopKOutput``."""
    from .fused_moe import StandardTopKOutput

    c = topk_config
    if c.use_grouped_topk:
        assert c.topk_group is not None and c.num_expert_group is not None
        if c.correction_bias is None:
            w, ids = grouped_topk(hidden_states, router_logits, c.top_k, c.renormalize, c.num_expert_group,
                                  c.topk_group, c.num_fused_shared_experts, c.routed_scaling_factor,
                                  c.apply_routed_scaling_factor_on_output, num_token_non_padded)
        else:
            w, ids = biased_grouped_topk(hidden_states, router_logits, c.correction_bias, c.top_k, c.renormalize,
                                         c.num_expert_group, c.topk_group, c.num_fused_shared_experts,
                                         c.routed_scaling_factor, c.apply_routed_scaling_factor_on_output,
                                         num_token_non_padded)
    else:
        w, ids = fused_topk(hidden_states, router_logits, c.top_k, c.renormalize, c.correction_bias, c.scoring_func,
                            num_token_non_padded)
    return StandardTopKOutput(w, ids, router_logits)
