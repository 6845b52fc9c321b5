"""Dispatcher ops of namespace ``sglang_b200``: schemas equal the reference's
(sgl-kernel/csrc/common_extension.cc:127-139,165-190), fake implementations give the right shapes
without a device, CPU tensors are refused (no CPU fallback), and on the GPU every op returns the
bits of the direct Python entry point."""
import pytest
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

import sglang_b200 as S
import sglang_b200.custom_ops as C

ops = torch.ops.sglang_b200
fp8 = torch.float8_e4m3fn


def test_schemas_match_reference_text():
    # the reference's argument lists, as written in its registration file
    want = {
        "fp8_blockwise_scaled_mm": "Tensor mat_a, Tensor mat_b, Tensor scales_a, Tensor scales_b, ScalarType out_dtype",
        "sgl_per_token_group_quant_8bit": "Tensor input, Tensor! output_q, Tensor! output_s, int group_size, float eps, "
        "float fp8_min, float fp8_max, bool scale_ue8m0",
        "sgl_per_token_group_quant_8bit_v2": "Tensor input, Tensor! output_q, Tensor! output_s, int group_size, float eps, "
        "float fp8_min, float fp8_max, bool scale_ue8m0, bool fuse_silu_and_mul, Tensor? masked_m",
        "moe_align_block_size": "Tensor topk_ids, int num_experts, int block_size, Tensor! sorted_token_ids, Tensor! "
        "experts_ids, Tensor! num_tokens_post_pad, Tensor! cumsum_buffer, bool pad_sorted_token_ids",
        "topk_softmax": "Tensor! topk_weights, Tensor! topk_indices, Tensor gating_output, bool renormalize, float "
        "moe_softcapping, Tensor? correction_bias",
        "topk_sigmoid": "Tensor! topk_weights, Tensor! topk_indices, Tensor gating_output, bool renormalize, Tensor? "
        "correction_bias",
        "moe_fused_gate": "Tensor input, Tensor bias, int num_expert_group, int topk_group, int topk, int "
        "num_fused_shared_experts, float routed_scaling_factor, bool apply_routed_scaling_factor_on_output",
    }
    for name, args in want.items():
        schema = getattr(ops, name).default._schema
        got = [(a.name, str(a.type), a.alias_info is not None and a.alias_info.is_write) for a in schema.arguments]
        parsed = torch._C.parse_schema(f"{name}({args}) -> ()")  # same parser as the registration macro
        exp = [(a.name, str(a.type), a.alias_info is not None and a.alias_info.is_write) for a in parsed.arguments]
        assert got == exp, name
    assert set(C.op_names()) >= set(want)


def test_fake_shapes_and_cpu_refusal():
    with FakeTensorMode():
        a = torch.empty(64, 2048, dtype=fp8, device="cuda")
        w = torch.empty(4096, 2048, dtype=fp8, device="cuda")
        sa = torch.empty(16, 64, device="cuda").t()
        sw = torch.empty(32, 16, device="cuda")
        out = ops.fp8_blockwise_scaled_mm(a, w.t(), sa, sw.t(), torch.bfloat16)
        assert out.shape == (64, 4096) and out.dtype == torch.bfloat16 and out.device.type == "cuda"
        with pytest.raises(AssertionError, match="column major"):
            ops.fp8_blockwise_scaled_mm(a, w.t().contiguous(), sa, sw.t(), torch.bfloat16)
        wts, ids = ops.moe_fused_gate(torch.empty(7, 256, device="cuda"), torch.empty(256, device="cuda"), 8, 4, 8, 0,
                                      1.0, False)
        assert wts.shape == (7, 8) and wts.dtype == torch.float32 and ids.dtype == torch.int32
        x = torch.empty(5, 7168, dtype=torch.bfloat16, device="cuda")
        w1 = torch.empty(4, 512, 7168, dtype=fp8, device="cuda")
        w2 = torch.empty(4, 7168, 256, dtype=fp8, device="cuda")
        tw = torch.empty(5, 2, device="cuda")
        ti = torch.empty(5, 2, dtype=torch.int32, device="cuda")
        s1 = torch.empty(4, 4, 56, device="cuda")
        s2 = torch.empty(4, 56, 2, device="cuda")
        assert ops.outplace_fused_experts(x, w1, w2, tw, ti, s1, s2, [128, 128], False, False, None).shape == (5, 7168)
        assert ops.outplace_fused_experts(x, w1, w2, tw, ti, s1, s2, [128, 128], False, True, None).shape == (5, 2, 7168)
        assert ops.inplace_fused_experts(x, w1, w2, tw, ti, s1, s2, [128, 128], False, 2.5) is None
    with pytest.raises(NotImplementedError):  # no CPU kernel is registered
        ops.fp8_blockwise_scaled_mm(torch.zeros(4, 128).to(fp8), torch.zeros(128, 128).to(fp8).t(), torch.ones(4, 1),
                                    torch.ones(1, 1), torch.bfloat16)


@pytest.mark.gpu
def test_ops_equal_direct_calls():
    g = torch.Generator(device="cuda").manual_seed(7)
    M, K, Nn = 96, 1024, 1536
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    # quant, column-major scales, out-parameter form
    q_ref, s_ref = S.per_token_group_quant_fp8(x, 128, column_major_scales=True)
    q = torch.empty_like(q_ref)
    s = torch.empty(K // 128, M, device="cuda").t()
    ops.sgl_per_token_group_quant_8bit(x, q, s, 128, 1e-10, -448.0, 448.0, False)
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8)) and torch.equal(s, s_ref)
    q2 = torch.empty_like(q_ref)
    s2 = torch.empty(M, K // 128, device="cuda")
    ops.sgl_per_token_group_quant_8bit_v2(x, q2, s2, 128, 1e-10, -448.0, 448.0, False, False, None)
    assert torch.equal(q2.view(torch.uint8), q_ref.view(torch.uint8)) and torch.equal(s2, s_ref)
    # power-of-two packed scales with fused silu*mul
    xg = torch.randn(M, 2 * K, device="cuda", generator=g).bfloat16()
    qu_ref, su_ref = S.per_token_group_quant_fp8(xg, 128, column_major_scales=True, scale_tma_aligned=True,
                                                 scale_ue8m0=True, fuse_silu_and_mul=True)
    qu = torch.empty_like(qu_ref)
    su = S.create_per_token_group_quant_fp8_output_scale((M, K), x.device, 128, True, True, True)
    ops.sgl_per_token_group_quant_8bit_v2(xg, qu, su, 128, 1e-10, -448.0, 448.0, True, True, None)
    assert torch.equal(qu.view(torch.uint8), qu_ref.view(torch.uint8)) and torch.equal(su, su_ref)
    # GEMM with the transposed-weight convention
    w = (torch.randn(Nn, K, device="cuda", generator=g) * 0.5).to(fp8)
    ws = torch.rand(Nn // 128, K // 128, device="cuda", generator=g)
    c_ref = S.w8a8_block_fp8_matmul(q_ref, w, s_ref, ws, [128, 128], torch.bfloat16)
    c = ops.fp8_blockwise_scaled_mm(q_ref, w.t(), s_ref, ws.t(), torch.bfloat16)
    assert torch.equal(c, c_ref)
    # routing
    logits = torch.randn(33, 256, device="cuda", generator=g)
    bias = torch.randn(256, device="cuda", generator=g) * 0.1
    tw = torch.empty(33, 8, device="cuda")
    ti = torch.empty(33, 8, dtype=torch.int32, device="cuda")
    ops.topk_softmax(tw, ti, logits, True, 0.0, None)
    tw_ref, ti_ref = S.fused_topk(logits, logits, 8, True)
    assert torch.equal(ti, ti_ref) and torch.equal(tw, tw_ref)
    ops.topk_sigmoid(tw, ti, logits, True, bias)
    tw_ref, ti_ref = S.fused_topk(logits, logits, 8, True, bias, "sigmoid")
    assert torch.equal(ti, ti_ref) and torch.equal(tw, tw_ref)
    gw, gi = ops.moe_fused_gate(logits, bias, 8, 4, 8, 0, 2.5, True)
    gw_ref, gi_ref = S.moe_fused_gate(logits, bias, 8, 4, 8, 0, 2.5, True)
    assert torch.equal(gi, gi_ref) and torch.equal(gw, gw_ref)
    # align, out-parameter form
    E, block = 256, 128
    sorted_ref, experts_ref, post_ref = S.moe_align_block_size(gi, block, E)
    sorted_ids = torch.empty_like(sorted_ref)
    expert_ids = torch.empty_like(experts_ref)
    post = torch.empty_like(post_ref)
    cumsum = torch.empty(E + 2, dtype=torch.int32, device="cuda")
    ops.moe_align_block_size(gi, E + 1, block, sorted_ids, expert_ids, post, cumsum, True)
    n = int(post.item())
    assert n == int(post_ref.item())
    assert torch.equal(sorted_ids[:n], sorted_ref[:n]) and torch.equal(expert_ids[: n // block], experts_ref[: n // block])


@pytest.mark.gpu
def test_moe_ops_equal_direct_calls():
    g = torch.Generator(device="cuda").manual_seed(11)
    T, H, I, E, topk = 40, 512, 256, 8, 2
    x = torch.randn(T, H, device="cuda", generator=g).bfloat16()
    w1 = (torch.randn(E, 2 * I, H, device="cuda", generator=g) * 0.5).to(fp8)
    w2 = (torch.randn(E, H, I, device="cuda", generator=g) * 0.5).to(fp8)
    s1 = torch.rand(E, 2 * I // 128, H // 128, device="cuda", generator=g) * 0.02
    s2 = torch.rand(E, H // 128, I // 128, device="cuda", generator=g) * 0.02
    logits = torch.randn(T, E, device="cuda", generator=g)
    tw, ti = S.fused_topk(x, logits, topk, True)
    ref = S.fused_experts(x, w1, w2, S.StandardTopKOutput(tw, ti, None), S.MoeRunnerConfig(inplace=False),
                          use_fp8_w8a8=True, w1_scale=s1, w2_scale=s2, block_shape=[128, 128])
    out = ops.outplace_fused_experts(x, w1, w2, tw, ti, s1, s2, [128, 128], False, False, None)
    assert torch.equal(out, ref)
    parts = ops.outplace_fused_experts(x, w1, w2, tw, ti, s1, s2, [128, 128], False, True, None)
    assert parts.shape == (T, topk, H)
    xin = x.clone()
    ops.inplace_fused_experts(xin, w1, w2, tw, ti, s1, s2, [128, 128], False, None)
    assert torch.equal(xin, ref)


@pytest.mark.gpu
def test_ops_trace_and_capture():
    """A quantised linear written with the dispatcher ops traces as one graph (no graph break: the fake
    implementations supply the shapes) and captures into a CUDA graph; both replay the eager bits."""
    g = torch.Generator(device="cuda").manual_seed(3)
    M, K, Nn = 48, 1024, 768
    x = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    w = (torch.randn(Nn, K, device="cuda", generator=g) * 0.5).to(fp8)
    ws = torch.rand(Nn // 128, K // 128, device="cuda", generator=g)

    def linear(x):
        q = torch.empty_like(x, dtype=fp8)
        s = torch.empty(K // 128, x.shape[0], device=x.device).t()
        ops.sgl_per_token_group_quant_8bit(x, q, s, 128, 1e-10, -448.0, 448.0, False)
        return ops.fp8_blockwise_scaled_mm(q, w.t(), s, ws.t(), torch.bfloat16)

    eager = linear(x)
    traced = torch.compile(linear, backend="eager", fullgraph=True)
    assert torch.equal(traced(x), eager)
    linear(x)  # workspaces exist before capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = linear(x)
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
