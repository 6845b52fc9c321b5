"""``torch.library`` registration of the path's operators, namespace ``sglang_b200``.

The reference exposes its kernels as dispatcher ops (sgl-kernel/csrc/common_extension.cc:127-139,
165-190) and wraps its Python-level MoE entry points the same way
(python/sglang/srt/layers/moe/fused_moe_triton/fused_moe.py:91-215 through
python/sglang/srt/utils/custom_op.py:56-118), so that graph capture and tracing see one opaque node
with known aliasing. The schemas below repeat the reference's, argument for argument; each has a
CUDA implementation (this package's C ABI) and a fake implementation that only describes shapes,
which is all a tracer needs. There is no CPU implementation: on a CPU tensor the dispatcher raises.

    import sglang_b200.custom_ops          # registers the ops
    torch.ops.sglang_b200.fp8_blockwise_scaled_mm(a_q, w.T, a_s, w_s.T, torch.bfloat16)
"""
from __future__ import annotations

from typing import List, Optional

import torch

from . import _native as N
from . import fp8_kernel as _q
from . import topk as _topk
from .fused_moe import fused_experts_impl as _experts
from .moe_align_block_size import sgl_moe_align_block_size as _align_into

NAMESPACE = "sglang_b200"
_lib = torch.library.Library(NAMESPACE, "DEF")

SCHEMAS = {
    "sgl_per_token_group_quant_8bit": "(Tensor input, Tensor(a!) output_q, Tensor(b!) output_s, int group_size, "
    "float eps, float fp8_min, float fp8_max, bool scale_ue8m0) -> ()",
    "sgl_per_token_group_quant_8bit_v2": "(Tensor input, Tensor(a!) output_q, Tensor(b!) output_s, int group_size, "
    "float eps, float fp8_min, float fp8_max, bool scale_ue8m0, bool fuse_silu_and_mul, Tensor? masked_m) -> ()",
    "fp8_blockwise_scaled_mm": "(Tensor mat_a, Tensor mat_b, Tensor scales_a, Tensor scales_b, ScalarType out_dtype) "
    "-> Tensor",
    "moe_align_block_size": "(Tensor topk_ids, int num_experts, int block_size, Tensor(a!) sorted_token_ids, "
    "Tensor(b!) experts_ids, Tensor(c!) num_tokens_post_pad, Tensor(d!) cumsum_buffer, bool pad_sorted_token_ids) "
    "-> ()",
    "topk_softmax": "(Tensor(a!) topk_weights, Tensor(b!) topk_indices, Tensor gating_output, bool renormalize, "
    "float moe_softcapping, Tensor? correction_bias) -> ()",
    "topk_sigmoid": "(Tensor(a!) topk_weights, Tensor(b!) topk_indices, Tensor gating_output, bool renormalize, "
    "Tensor? correction_bias) -> ()",
    "moe_fused_gate": "(Tensor input, Tensor bias, int num_expert_group, int topk_group, int topk, "
    "int num_fused_shared_experts, float routed_scaling_factor, bool apply_routed_scaling_factor_on_output) "
    "-> Tensor[]",
    "inplace_fused_experts": "(Tensor(a!) hidden_states, Tensor w1, Tensor w2, Tensor topk_weights, Tensor topk_ids, "
    "Tensor w1_scale, Tensor w2_scale, int[] block_shape, bool apply_router_weight_on_input, "
    "float? routed_scaling_factor) -> ()",
    "outplace_fused_experts": "(Tensor hidden_states, Tensor w1, Tensor w2, Tensor topk_weights, Tensor topk_ids, "
    "Tensor w1_scale, Tensor w2_scale, int[] block_shape, bool apply_router_weight_on_input, bool no_combine, "
    "float? routed_scaling_factor) -> Tensor",
}
for _name, _schema in SCHEMAS.items():
    _lib.define(_name + _schema)


def _impl(name):
    def deco(fn):
        _lib.impl(name, fn, "CUDA")
        return fn

    return deco


def _fake(name):
    def deco(fn):
        torch.library.register_fake(f"{NAMESPACE}::{name}", fn, lib=_lib)
        return fn

    return deco


# ------------------------------------------------------------------------------------------ quant

def _quant_into(x, output_q, output_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0, fuse_silu_and_mul, masked_m):
    """Out-parameter quantisation with the checks of the reference's launcher
    (sgl-kernel/csrc/gemm/per_token_group_quant_8bit_v2.cu:269-330): contiguous input and FP8
    output; the layout of ``output_s`` is read from its strides."""
    N.require_cuda(x, output_q, output_s)
    assert x.is_contiguous() and output_q.is_contiguous(), "input and output_q must be contiguous"
    assert output_q.dtype == _q.fp8_dtype, "only the FP8 E4M3 output of the block-FP8 path is built"
    assert abs(fp8_max - 448.0) < 1e-6 and abs(fp8_min + 448.0) < 1e-6, "E4M3 range expected"
    k = output_q.shape[-1]
    assert x.shape[-1] == (2 * k if fuse_silu_and_mul else k) and k % group_size == 0
    rows = output_q.numel() // k if k else 0
    if rows == 0:
        return
    lib = N.load()
    if scale_ue8m0:
        assert output_s.dtype == torch.int32 and output_s.stride(-2) == 1, "packed scales are MN-major int32"
        experts = output_q.shape[0] if masked_m is not None else 1
        mm = None
        if masked_m is not None:
            assert fuse_silu_and_mul and output_q.dim() == 3 and masked_m.shape == (experts,)
            mm = masked_m.to(torch.int32).contiguous()
        aligned_mn = output_s.stride(-1)
        assert aligned_mn % 4 == 0 and aligned_mn >= output_q.shape[-2], "row extent of the scale storage is padded to 4"
        with N.on_device(x):
            st = lib.b200_per_token_group_quant_fp8_ue8m0(
                N.ptr(x), N.DTYPE_CODE[x.dtype], N.ptr(output_q), output_s.data_ptr(), rows, k, group_size,
                aligned_mn, int(fuse_silu_and_mul), N.ptr(mm), experts, N.current_stream())
        N.check(st, "sgl_per_token_group_quant_8bit (UE8M0)")
        return
    if fuse_silu_and_mul or masked_m is not None:
        raise NotImplementedError("fuse_silu_and_mul / masked_m are built for scale_ue8m0=True only")
    assert output_s.dtype == torch.float32 and output_s.dim() == 2 and output_q.dim() == 2
    assert output_s.shape == (rows, k // group_size)
    with N.on_device(x):
        st = lib.b200_per_token_group_quant_fp8(
            N.ptr(x), N.DTYPE_CODE[x.dtype], N.ptr(output_q), N.ptr(output_s), rows, k, group_size,
            output_s.stride(0), output_s.stride(1), eps, _q.quant_formula_for(x.dtype, eps), N.current_stream())
    N.check(st, "sgl_per_token_group_quant_8bit")


@_impl("sgl_per_token_group_quant_8bit")
def _quant_v1(input, output_q, output_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0):
    _quant_into(input, output_q, output_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0, False, None)


@_impl("sgl_per_token_group_quant_8bit_v2")
def _quant_v2(input, output_q, output_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0, fuse_silu_and_mul,
              masked_m):
    _quant_into(input, output_q, output_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0, fuse_silu_and_mul,
                masked_m)


@_fake("sgl_per_token_group_quant_8bit")
def _quant_v1_fake(input, output_q, output_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0):
    return None


@_fake("sgl_per_token_group_quant_8bit_v2")
def _quant_v2_fake(input, output_q, output_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0, fuse_silu_and_mul,
                   masked_m):
    return None


# ------------------------------------------------------------------------------------------- GEMM

def _mm_checks(mat_a, mat_b, scales_a, scales_b, out_dtype):
    """The reference's preconditions (sgl-kernel/csrc/gemm/fp8_blockwise_gemm_kernel.cu:431-463):
    ``mat_a [M, K]`` row-major, ``mat_b [K, N]`` column-major (a transposed ``[N, K]`` weight),
    ``scales_a [M, K/128]`` M-major, ``scales_b [K/128, N/128]`` K-major."""
    assert mat_a.dim() == 2 and mat_b.dim() == 2, "mat_a and mat_b must be 2D tensors"
    assert mat_a.stride(1) == 1, "mat_a must be a row major tensor"
    assert mat_b.stride(0) == 1, "mat_b must be a column major tensor"
    assert mat_a.shape[1] == mat_b.shape[0], "mat_a and mat_b shapes cannot be multiplied"
    assert out_dtype in (torch.float16, torch.bfloat16), "out_dtype must be Half or BFloat16"
    assert scales_a.shape[0] == mat_a.shape[0] and scales_a.shape[1] == mat_a.shape[1] // 128, \
        "size of scales_a is not matched"
    assert scales_b.shape[0] == mat_b.shape[0] // 128 and scales_b.shape[1] == mat_b.shape[1] // 128, \
        "size of scales_b is not matched"
    assert (mat_b.shape[1] * 2) % 16 == 0, "out must be multiple of 16 bytes for memory alignment"


@_impl("fp8_blockwise_scaled_mm")
def _mm(mat_a, mat_b, scales_a, scales_b, out_dtype):
    _mm_checks(mat_a, mat_b, scales_a, scales_b, out_dtype)
    assert mat_a.dtype == _q.fp8_dtype and mat_b.dtype == _q.fp8_dtype, "mat_a and mat_b must be Float8_e4m3fn"
    assert scales_a.dtype == torch.float32 and scales_b.dtype == torch.float32, "scales must be Float32"
    return _q.w8a8_block_fp8_matmul(mat_a.contiguous(), mat_b.t(), scales_a, scales_b.t(), [128, 128], out_dtype)


@_fake("fp8_blockwise_scaled_mm")
def _mm_fake(mat_a, mat_b, scales_a, scales_b, out_dtype):
    _mm_checks(mat_a, mat_b, scales_a, scales_b, out_dtype)
    return mat_a.new_empty((mat_a.shape[0], mat_b.shape[1]), dtype=out_dtype)


# ------------------------------------------------------------------------------------------ align

@_impl("moe_align_block_size")
def _align_impl(topk_ids, num_experts, block_size, sorted_token_ids, experts_ids, num_tokens_post_pad,
                cumsum_buffer, pad_sorted_token_ids):
    _align_into(topk_ids, num_experts, block_size, sorted_token_ids, experts_ids, num_tokens_post_pad, cumsum_buffer,
                pad_sorted_token_ids)


@_fake("moe_align_block_size")
def _align_fake(topk_ids, num_experts, block_size, sorted_token_ids, experts_ids, num_tokens_post_pad,
                cumsum_buffer, pad_sorted_token_ids):
    return None


# ---------------------------------------------------------------------------------------- routing

@_impl("topk_softmax")
def _topk_softmax(topk_weights, topk_indices, gating_output, renormalize, moe_softcapping, correction_bias):
    _topk.topk_softmax(topk_weights, topk_indices, gating_output, renormalize, moe_softcapping, correction_bias)


@_fake("topk_softmax")
def _topk_softmax_fake(topk_weights, topk_indices, gating_output, renormalize, moe_softcapping, correction_bias):
    return None


@_impl("topk_sigmoid")
def _topk_sigmoid(topk_weights, topk_indices, gating_output, renormalize, correction_bias):
    _topk.topk_sigmoid(topk_weights, topk_indices, gating_output, renormalize, correction_bias)


@_fake("topk_sigmoid")
def _topk_sigmoid_fake(topk_weights, topk_indices, gating_output, renormalize, correction_bias):
    return None


@_impl("moe_fused_gate")
def _fused_gate(input, bias, num_expert_group, topk_group, topk, num_fused_shared_experts, routed_scaling_factor,
                apply_routed_scaling_factor_on_output) -> List[torch.Tensor]:
    w, i = _topk.moe_fused_gate(input, bias, num_expert_group, topk_group, topk, num_fused_shared_experts,
                                routed_scaling_factor, apply_routed_scaling_factor_on_output)
    return [w, i]


@_fake("moe_fused_gate")
def _fused_gate_fake(input, bias, num_expert_group, topk_group, topk, num_fused_shared_experts,
                     routed_scaling_factor, apply_routed_scaling_factor_on_output):
    t = input.shape[0]
    return [input.new_empty((t, topk), dtype=torch.float32), input.new_empty((t, topk), dtype=torch.int32)]


# ------------------------------------------------------------------------------------------- MoE

def _moe_checks(hidden_states, w1, w2, topk_weights, topk_ids, block_shape):
    assert list(block_shape) == [128, 128], "only block_shape=[128, 128] is built"
    assert hidden_states.dim() == 2 and w1.dim() == 3 and w2.dim() == 3
    assert hidden_states.shape[1] == w1.shape[2], "Hidden size mismatch"
    assert topk_weights.shape == topk_ids.shape, "topk shape mismatch"


@_impl("inplace_fused_experts")
def _moe_inplace(hidden_states, w1, w2, topk_weights, topk_ids, w1_scale, w2_scale, block_shape,
                 apply_router_weight_on_input, routed_scaling_factor):
    _moe_checks(hidden_states, w1, w2, topk_weights, topk_ids, block_shape)
    _experts(hidden_states, w1, w2, topk_weights, topk_ids, w1_scale, w2_scale, inplace=True,
             apply_router_weight_on_input=apply_router_weight_on_input, routed_scaling_factor=routed_scaling_factor)


@_fake("inplace_fused_experts")
def _moe_inplace_fake(hidden_states, w1, w2, topk_weights, topk_ids, w1_scale, w2_scale, block_shape,
                      apply_router_weight_on_input, routed_scaling_factor):
    _moe_checks(hidden_states, w1, w2, topk_weights, topk_ids, block_shape)
    return None


@_impl("outplace_fused_experts")
def _moe_outplace(hidden_states, w1, w2, topk_weights, topk_ids, w1_scale, w2_scale, block_shape,
                  apply_router_weight_on_input, no_combine, routed_scaling_factor):
    _moe_checks(hidden_states, w1, w2, topk_weights, topk_ids, block_shape)
    return _experts(hidden_states, w1, w2, topk_weights, topk_ids, w1_scale, w2_scale, inplace=False,
                    no_combine=no_combine, apply_router_weight_on_input=apply_router_weight_on_input,
                    routed_scaling_factor=routed_scaling_factor)


@_fake("outplace_fused_experts")
def _moe_outplace_fake(hidden_states, w1, w2, topk_weights, topk_ids, w1_scale, w2_scale, block_shape,
                       apply_router_weight_on_input, no_combine, routed_scaling_factor):
    _moe_checks(hidden_states, w1, w2, topk_weights, topk_ids, block_shape)
    if no_combine:
        return hidden_states.new_empty((hidden_states.shape[0], topk_ids.shape[1], w2.shape[1]))
    return torch.empty_like(hidden_states)


def op_names() -> List[str]:
    return sorted(SCHEMAS)
