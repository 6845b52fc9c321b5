"""``fused_experts`` / ``fused_moe`` for block-FP8 W8A8 experts with the reference's
signature (python/sglang/srt/layers/moe/moe_runner/triton_utils/fused_moe.py:218-306,
:896-998), executed by the sm_100a grouped tcgen05 GEMMs behind the C ABI.

Only the configuration this path is about is built: ``use_fp8_w8a8=True``,
``block_shape=[128, 128]``, SiLU-gated experts, dynamic activation scales. Every other
argument combination raises instead of silently computing something else."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, NamedTuple, Optional

import torch

from . import _native as N
from .fp8_kernel import _workspace, fp8_dtype


class StandardTopKOutput(NamedTuple):
    """Routing result (python/sglang/srt/layers/moe/topk.py:252-261)."""

    topk_weights: torch.Tensor
    topk_ids: torch.Tensor
    router_logits: Optional[torch.Tensor] = None


@dataclass
class MoeRunnerConfig:
    """The fields of the reference's MoeRunnerConfig
    (python/sglang/srt/layers/moe/moe_runner/base.py:45-67) this path reads."""

    num_experts: Optional[int] = None
    num_local_experts: Optional[int] = None
    hidden_size: Optional[int] = None
    intermediate_size_per_partition: Optional[int] = None
    layer_id: Optional[int] = None
    top_k: Optional[int] = None
    num_fused_shared_experts: Optional[int] = None
    params_dtype: Optional[torch.dtype] = None
    routing_method_type: Optional[object] = None
    activation: str = "silu"
    is_gated: bool = True
    apply_router_weight_on_input: bool = False
    inplace: bool = True
    no_combine: bool = False
    routed_scaling_factor: Optional[float] = None
    gemm1_alpha: Optional[float] = None
    gemm1_clamp_limit: Optional[float] = None
    swiglu_limit: Optional[float] = None


def fused_experts_impl(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    w1_scale: torch.Tensor,
    w2_scale: torch.Tensor,
    inplace: bool = False,
    no_combine: bool = False,
    apply_router_weight_on_input: bool = False,
    routed_scaling_factor: Optional[float] = None,
    hidden_states_scale: Optional[torch.Tensor] = None,
    output_dtype: Optional[torch.dtype] = None,
    out: Optional[torch.Tensor] = None,
    skip_unrouted_rows: bool = False,
) -> torch.Tensor:
    """Checks of the reference's ``fused_experts_impl`` (fused_moe.py:824-834) + the launch.

    ``out`` (extension): a preallocated contiguous result tensor, e.g. a region of peer-mapped
    memory that other ranks read. ``skip_unrouted_rows`` (extension): rows none of whose ids is valid
    are left unwritten instead of being zeroed.

    ``hidden_states_scale`` (extension used by the expert-parallel all-to-all path): when given,
    ``hidden_states`` is already FP8 E4M3 ``[T, H]`` with row-major fp32 1x128 scales
    ``[T, H/128]`` and ``output_dtype`` names the result dtype."""
    assert hidden_states.shape[1] == w1.shape[2], "Hidden size mismatch"
    assert topk_weights.shape == topk_ids.shape, "topk shape mismatch"
    assert hidden_states.is_contiguous(), "Hidden_states must be contiguous"
    assert w1.is_contiguous(), "Expert weights1 must be contiguous"
    assert w2.is_contiguous(), "Expert weights2 must be contiguous"
    if hidden_states_scale is None:
        assert hidden_states.dtype in [torch.float16, torch.bfloat16]
        out_dtype = hidden_states.dtype
    else:
        assert hidden_states.dtype == fp8_dtype and not inplace, "pre-quantised input is FP8 and out of place"
        assert output_dtype in (torch.float16, torch.bfloat16), "output_dtype must be given for FP8 input"
        assert tuple(hidden_states_scale.shape) == (hidden_states.shape[0], hidden_states.shape[1] // 128)
        hidden_states_scale = hidden_states_scale.to(torch.float32).contiguous()
        N.require_cuda(hidden_states_scale)
        out_dtype = output_dtype
    assert w1.dtype == fp8_dtype and w2.dtype == fp8_dtype, "expert weights must be float8_e4m3fn"
    assert not (inplace and no_combine), "no combine + inplace makes no sense"
    N.require_cuda(hidden_states, w1, w2, topk_weights, topk_ids, w1_scale, w2_scale)
    T, H = hidden_states.shape
    E, two_i, _ = w1.shape
    I = two_i // 2
    topk = topk_ids.shape[1]
    assert w2.shape == (E, H, I), f"w2 shape {tuple(w2.shape)} != {(E, H, I)}"
    assert tuple(w1_scale.shape) == (E, (two_i + 127) // 128, (H + 127) // 128), "w1_scale shape"
    assert tuple(w2_scale.shape) == (E, (H + 127) // 128, (I + 127) // 128), "w2_scale shape"
    if apply_router_weight_on_input:
        assert topk == 1, "Only support topk=1 when `apply_router_weight_on_input` is True"
    topk_weights = topk_weights.to(torch.float32).contiguous()
    topk_ids = topk_ids.to(torch.int32).contiguous()
    w1_scale = w1_scale.to(torch.float32).contiguous()
    w2_scale = w2_scale.to(torch.float32).contiguous()
    if out is not None:
        assert not inplace and out.is_contiguous() and out.dtype == out_dtype
        assert tuple(out.shape) == ((T, topk, H) if no_combine else (T, H)), "preallocated output shape"
        N.require_cuda(out)
    elif inplace:
        out = hidden_states
    elif no_combine:
        out = torch.empty((T, topk, H), dtype=out_dtype, device=hidden_states.device)
    else:
        out = torch.empty((T, H), dtype=out_dtype, device=hidden_states.device)
    if T == 0:
        return out
    lib = N.load()
    ws_bytes = lib.b200_fused_experts_fp8_workspace_bytes(T, topk, E, H, I)
    with N.on_device(hidden_states):
        ws = _workspace(hidden_states.device, ws_bytes)
        st = lib.b200_fused_experts_fp8(
            N.ptr(hidden_states), N.ptr(hidden_states_scale), N.DTYPE_CODE[out_dtype], N.ptr(w1), N.ptr(w2), N.ptr(w1_scale),
            N.ptr(w2_scale), N.ptr(topk_weights), N.ptr(topk_ids), N.ptr(out), T, topk, E, H, I,
            1 if no_combine else (2 if skip_unrouted_rows else 0),
            int(apply_router_weight_on_input),
            1.0 if routed_scaling_factor is None else float(routed_scaling_factor), N.ptr(ws), ws_bytes,
            N.current_stream(),
        )
    N.check(st, "fused_experts")
    return out


def fused_experts_scatter(
    rows_q: torch.Tensor, rows_scale: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk_weights: torch.Tensor,
    topk_ids: torch.Tensor, w1_scale: torch.Tensor, w2_scale: torch.Tensor, dest_ptrs, rows_per_dest: int,
    output_dtype: torch.dtype = torch.bfloat16,
) -> None:
    """Experts of this rank over ``T`` positions of already quantised rows (``rows_q [T, H]`` e4m3,
    ``rows_scale [T, H/128]``, ``topk_ids`` local to this rank with -1 for "not mine"), router weight applied
    and NO slot sum: the down GEMM sends the row of pair ``t * topk + j`` into buffer
    ``dest_ptrs[(t * topk + j) // rows_per_dest]`` (a ``ctypes`` array of device pointers, peer memory allowed)
    at row ``(t * topk + j) % rows_per_dest``. The combine half of an expert-parallel layer
    (python/sglang/srt/layers/moe/token_dispatcher/deepep.py:560-602) done by the GEMM's own epilogue."""
    N.require_cuda(rows_q, rows_scale, w1, w2, topk_weights, topk_ids, w1_scale, w2_scale)
    T, H = rows_q.shape
    E, two_i, _ = w1.shape
    I = two_i // 2
    topk = topk_ids.shape[1]
    assert rows_q.dtype == fp8_dtype and rows_q.is_contiguous() and rows_scale.dtype == torch.float32
    assert rows_scale.is_contiguous() and tuple(rows_scale.shape) == (T, H // 128)
    assert topk_weights.dtype == torch.float32 and topk_ids.dtype == torch.int32
    assert topk_weights.is_contiguous() and topk_ids.is_contiguous() and tuple(topk_weights.shape) == (T, topk)
    assert w1.dtype == fp8_dtype and w2.dtype == fp8_dtype and w1.is_contiguous() and w2.is_contiguous()
    assert w2.shape == (E, H, I)
    w1_scale = w1_scale.to(torch.float32).contiguous()
    w2_scale = w2_scale.to(torch.float32).contiguous()
    if T == 0:
        return
    lib = N.load()
    ws_bytes = lib.b200_fused_experts_fp8_workspace_bytes(T, topk, E, H, I)
    with N.on_device(rows_q):
        ws = _workspace(rows_q.device, ws_bytes)
        st = lib.b200_fused_experts_fp8_scatter(
            N.ptr(rows_q), N.ptr(rows_scale), N.DTYPE_CODE[output_dtype], N.ptr(w1), N.ptr(w2), N.ptr(w1_scale),
            N.ptr(w2_scale), N.ptr(topk_weights), N.ptr(topk_ids), dest_ptrs, len(dest_ptrs), rows_per_dest, T, topk, E, H, I,
            N.ptr(ws), ws_bytes, N.current_stream(),
        )
    N.check(st, "fused_experts_scatter")


def moe_sum_reduce(rows: torch.Tensor, topk_ids: torch.Tensor, out: torch.Tensor, num_experts: int,
                   routed_scaling_factor: float = 1.0, skip_unrouted_rows: bool = False,
                   poison_on_status: bool = False) -> torch.Tensor:
    """``out[t] = routed_scaling_factor * sum_j rows[t, j]`` over the slots whose id is in ``[0, num_experts)``
    (fp32 sum in slot order; the last step of ``fused_experts``, fused_moe.py:726-745). ``rows [T, topk, H]``.
    ``poison_on_status``: fill ``out`` with NaN when the device status word reports an expired wait."""
    N.require_cuda(rows, topk_ids, out)
    T, topk, H = rows.shape
    assert rows.is_contiguous() and out.is_contiguous() and tuple(out.shape) == (T, H) and out.dtype == rows.dtype
    assert topk_ids.dtype == torch.int32 and topk_ids.is_contiguous() and tuple(topk_ids.shape) == (T, topk)
    with N.on_device(rows):
        st = N.load().b200_moe_sum_reduce(N.ptr(rows), N.ptr(topk_ids), N.ptr(out), N.DTYPE_CODE[rows.dtype], T, topk,
                                          num_experts, H, float(routed_scaling_factor), int(skip_unrouted_rows),
                                          int(poison_on_status), N.current_stream())
    N.check(st, "moe_sum_reduce")
    return out


def fused_experts(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    topk_output: StandardTopKOutput,
    moe_runner_config: MoeRunnerConfig,
    b1: Optional[torch.Tensor] = None,
    b2: Optional[torch.Tensor] = None,
    use_fp8_w8a8: bool = False,
    use_int8_w8a8: bool = False,
    use_int8_w8a16: bool = False,
    use_int4_w4a16: bool = False,
    per_channel_quant: bool = False,
    w1_scale: Optional[torch.Tensor] = None,
    w2_scale: Optional[torch.Tensor] = None,
    w1_zp: Optional[torch.Tensor] = None,
    w2_zp: Optional[torch.Tensor] = None,
    a1_scale: Optional[torch.Tensor] = None,
    a2_scale: Optional[torch.Tensor] = None,
    block_shape: Optional[List[int]] = None,
) -> torch.Tensor:
    """Same arguments as the reference. ``w1 [E, 2I, H]`` (gate rows then up rows) and
    ``w2 [E, H, I]`` FP8 E4M3 with fp32 128x128 block scales; ids equal to -1 (expert on
    another rank) contribute zero. With ``moe_runner_config.inplace`` the result overwrites
    and is returned as ``hidden_states``."""
    if not use_fp8_w8a8 or block_shape is None or list(block_shape) != [128, 128]:
        raise NotImplementedError("this path is fused_experts(use_fp8_w8a8=True, block_shape=[128, 128]) only")
    if use_int8_w8a8 or use_int8_w8a16 or use_int4_w4a16 or per_channel_quant:
        raise NotImplementedError("integer / per-channel quantisation is not part of this path")
    if b1 is not None or b2 is not None or w1_zp is not None or w2_zp is not None:
        raise NotImplementedError("expert biases / zero points are not part of this path")
    if a1_scale is not None or a2_scale is not None:
        raise NotImplementedError("static activation scales are not used with block quantisation")
    c = moe_runner_config
    if c.activation != "silu" or not c.is_gated:
        raise NotImplementedError("only the SiLU-gated expert MLP is built")
    if c.gemm1_alpha is not None or c.gemm1_clamp_limit is not None or c.swiglu_limit is not None:
        raise NotImplementedError("gemm1_alpha / clamp limits are not part of this path")
    assert w1_scale is not None and w2_scale is not None, "block-FP8 experts need w1_scale and w2_scale"
    topk_weights, topk_ids = topk_output[0], topk_output[1]
    if c.inplace:
        assert not c.no_combine, "no combine + inplace makes no sense"
    return fused_experts_impl(
        hidden_states, w1, w2, topk_weights, topk_ids, w1_scale, w2_scale, inplace=c.inplace,
        no_combine=c.no_combine, apply_router_weight_on_input=c.apply_router_weight_on_input,
        routed_scaling_factor=c.routed_scaling_factor,
    )


def masked_fused_experts(
    hidden_states: torch.Tensor,
    hidden_states_scale: torch.Tensor,
    w13_weight: torch.Tensor,
    w13_scale: torch.Tensor,
    w2_weight: torch.Tensor,
    w2_scale: torch.Tensor,
    masked_m: torch.Tensor,
    expected_m: Optional[int] = None,
    output_dtype: torch.dtype = torch.bfloat16,
) -> torch.Tensor:
    """Experts over the masked (low-latency expert-parallel) layout, the job of the reference's
    ``DeepGemmRunnerCore._run_masked_gemm`` (moe_runner/deep_gemm.py:362-494): ``hidden_states
    [E, T_pad, H]`` FP8 with ``hidden_states_scale [E, T_pad, H/128]`` fp32, the first
    ``masked_m[e]`` rows of expert ``e`` valid; returns ``[E, T_pad, H]`` whose valid rows hold
    ``down(silu(gate) * up)`` (rows past ``masked_m[e]`` are not written). ``expected_m`` is the
    reference's scheduling hint and is not needed here."""
    assert hidden_states.dim() == 3 and hidden_states.dtype == fp8_dtype and hidden_states.is_contiguous()
    E, T_pad, H = hidden_states.shape
    assert tuple(hidden_states_scale.shape) == (E, T_pad, H // 128), "hidden_states_scale shape"
    two_i = w13_weight.shape[1]
    I = two_i // 2
    assert w13_weight.shape == (E, two_i, H) and w2_weight.shape == (E, H, I), "expert weight shapes"
    assert w13_weight.dtype == fp8_dtype and w2_weight.dtype == fp8_dtype
    assert w13_weight.is_contiguous() and w2_weight.is_contiguous()
    assert tuple(w13_scale.shape) == (E, (two_i + 127) // 128, (H + 127) // 128), "w13_scale shape"
    assert tuple(w2_scale.shape) == (E, (H + 127) // 128, (I + 127) // 128), "w2_scale shape"
    assert masked_m.shape == (E,), "masked_m holds one count per local expert"
    assert output_dtype in (torch.bfloat16, torch.float16)
    N.require_cuda(hidden_states, hidden_states_scale, w13_weight, w2_weight, w13_scale, w2_scale, masked_m)
    hs = hidden_states_scale.to(torch.float32).contiguous()
    w13_scale = w13_scale.to(torch.float32).contiguous()
    w2_scale = w2_scale.to(torch.float32).contiguous()
    mm = masked_m.to(torch.int32).contiguous()
    out = torch.empty((E, T_pad, H), dtype=output_dtype, device=hidden_states.device)
    lib = N.load()
    ws_bytes = lib.b200_masked_experts_fp8_workspace_bytes(E, T_pad, H, I)
    with N.on_device(hidden_states):
        ws = _workspace(hidden_states.device, ws_bytes)
        st = lib.b200_masked_experts_fp8(
            N.ptr(hidden_states), N.ptr(hs), N.ptr(w13_weight), N.ptr(w2_weight), N.ptr(w13_scale), N.ptr(w2_scale),
            N.ptr(mm), N.ptr(out), N.DTYPE_CODE[output_dtype], E, T_pad, H, I, N.ptr(ws), ws_bytes, N.current_stream(),
        )
    N.check(st, "masked_fused_experts")
    return out


def fused_moe(
    hidden_states: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    topk_output: StandardTopKOutput,
    moe_runner_config: Optional[MoeRunnerConfig] = None,
    **kwargs,
) -> torch.Tensor:
    """The reference's ``fused_moe`` (fused_moe.py:896-998) forwards to ``fused_experts``;
    like there, the default runner config is ``MoeRunnerConfig()``, i.e. in place."""
    if moe_runner_config is None:
        moe_runner_config = MoeRunnerConfig()
    return fused_experts(hidden_states, w1, w2, topk_output, moe_runner_config, **kwargs)
