"""Generate the golden fixtures in this directory from the REFERENCE's own code.

Run where the reference tree is importable:

    python tests/golden/make_golden.py --reference <path-to-reference-checkout>

It imports the reference's torch-native functions
(test/manual/quant/test_block_fp8.py: ``native_per_token_group_quant_fp8`` :41-66,
``native_w8a8_block_fp8_matmul`` :291-340, ``torch_w8a8_block_fp8_moe`` :518-547;
python/sglang/srt/layers/moe/topk.py: ``fused_topk_torch_native`` :550-588,
``grouped_topk_gpu`` :703-764, ``biased_grouped_topk_impl`` :923-992; test/registered/cpu/utils.py
``convert_weight`` :53-101), runs them on small seeded inputs built the way the
reference's tests build theirs, asserts that ``oracle/`` reproduces every output
exactly, and stores inputs + outputs as ``.npz`` (FP8 and bf16 tensors are stored as
their raw bytes). The CPU test-suite re-checks the oracle against these files; the GPU
tests check the CUDA path against them. The fixtures travel; the reference does not.

The only literal known-answer the reference holds for this path, the worked example
in the docstring of moe_align_block_size.py:44-57, is stored too.
"""
import argparse
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def _stub_modules():
    """Two import-time dependencies of the reference that are not needed for its
    torch-native functions and are absent from this image."""
    import json

    oj = types.ModuleType("orjson")
    oj.dumps = lambda o, **k: json.dumps(o).encode()
    oj.loads = json.loads
    oj.OPT_NON_STR_KEYS = 0
    oj.OPT_SERIALIZE_NUMPY = 0
    oj.JSONDecodeError = ValueError
    sys.modules.setdefault("orjson", oj)
    ip = types.ModuleType("IPython")
    ipd = types.ModuleType("IPython.display")
    ipd.display = lambda *a, **k: None
    ipd.HTML = type("HTML", (), {"__init__": lambda self, *a, **k: None})
    ip.display = ipd
    sys.modules.setdefault("IPython", ip)
    sys.modules.setdefault("IPython.display", ipd)


def raw(t):
    """Tensor -> numpy array of its raw storage (fp8 -> uint8, bf16 -> uint16)."""
    import torch

    t = t.detach().contiguous()
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy()
    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).numpy()
    return t.numpy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of a checkout of the reference project")
    args = ap.parse_args()
    os.environ["CUDA_VISIBLE_DEVICES"] = "0"  # parsed at import by the reference test utilities
    _stub_modules()
    sys.path.insert(0, os.path.join(args.reference, "python"))
    sys.path.insert(0, os.path.join(args.reference, "test/manual/quant"))
    sys.path.insert(0, os.path.join(args.reference, "test/registered/cpu"))
    sys.path.insert(0, ROOT)
    import torch

    from sglang.srt.server_args import ServerArgs, set_global_server_args_for_scheduler

    set_global_server_args_for_scheduler(ServerArgs(model_path="dummy"))
    import test_block_fp8 as R  # the reference's test module
    from sglang.srt.layers.moe import topk as RT

    import oracle as O

    fp8 = torch.float8_e4m3fn
    out = {}

    # ---- quant: inputs as in TestPerTokenGroupQuantFP8 (torch.rand, seed 0) plus N(0,1)
    # with outliers; bf16 / fp16 / fp32; groups 64 and 128.
    cases = [
        ("q_rand_bf16_7x512_g128", 7, 512, torch.bfloat16, 128, "rand"),
        ("q_rand_f16_7x512_g64", 7, 512, torch.float16, 64, "rand"),
        ("q_rand_f32_5x256_g128", 5, 256, torch.float32, 128, "rand"),
        ("q_randn_bf16_83x1024_g128", 83, 1024, torch.bfloat16, 128, "randn"),
        ("q_randn_f32_9x512_g256", 9, 512, torch.float32, 256, "randn"),
    ]
    for name, m, d, dt, g, kind in cases:
        torch.manual_seed(0)
        x = torch.rand(m, d, dtype=dt) if kind == "rand" else torch.randn(m, d, dtype=dt)
        if kind == "randn":
            x[:, 3] *= 20
        rq, rs = R.native_per_token_group_quant_fp8(x, g)
        oq, os_ = O.per_token_group_quant_fp8(x, g)
        assert torch.equal(rq.view(torch.uint8), oq.view(torch.uint8)), name
        assert torch.equal(rs, os_), name
        out[name + "/x"] = raw(x)
        out[name + "/q"] = raw(rq)
        out[name + "/s"] = raw(rs)
        out[name + "/meta"] = np.array([m, d, g, {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[dt]])
    np.savez_compressed(os.path.join(HERE, "quant.npz"), **out)
    print("quant ok", len(cases))

    # ---- GEMM: inputs as in TestW8A8BlockFP8Matmul._w8a8_block_fp8_matmul (seed 0)
    out = {}
    for name, M, N, K in [("g_33x256x512", 33, 256, 512), ("g_7x320x384", 7, 320, 384), ("g_130x128x256", 130, 128, 256)]:
        torch.manual_seed(0)
        A = ((torch.rand(M, K) - 0.5) * 2 * 448).clamp(-448, 448).to(fp8)
        B = ((torch.rand(N, K) - 0.5) * 2 * 448).clamp(-448, 448).to(fp8)
        nt, kt = (N + 127) // 128, (K + 127) // 128
        As = torch.rand(M, kt) * 1e-2
        Bs = torch.rand(nt, kt) * 1e-2
        ref = R.native_w8a8_block_fp8_matmul(A, B, As, Bs, [128, 128], torch.float32)
        mine = O.w8a8_block_fp8_matmul(A, B, As, Bs, [128, 128], torch.float32)
        assert torch.equal(ref, mine), name
        for k, v in dict(A=A, B=B, As=As, Bs=Bs, C=ref).items():
            out[f"{name}/{k}"] = raw(v)
    np.savez_compressed(os.path.join(HERE, "gemm.npz"), **out)
    print("gemm ok")

    # ---- weight quantiser
    from utils import convert_weight

    out = {}
    torch.manual_seed(1)
    w = (torch.randn(256, 384) * 0.02).bfloat16()
    w[128:, 128:256] = 0  # an all-zero block
    rq, rs, _ = convert_weight(w.float(), [128, 128], torch.bfloat16)
    oq, os_ = O.block_quant_weight_fp8(w, (128, 128))
    assert torch.equal(rq.view(torch.uint8), oq.view(torch.uint8)) and torch.equal(rs, os_)
    out["w/w"] = raw(w)
    out["w/q"] = raw(rq)
    out["w/s"] = raw(rs)
    np.savez_compressed(os.path.join(HERE, "weight_quant.npz"), **out)
    print("weight quant ok")

    # ---- UE8M0 (power-of-two scales): the reference's torch functions of fp8_utils.py:1186-1410.
    # Its layout helper imports two one-line functions from DeepGEMM, which is not installed here.
    dg = types.ModuleType("deep_gemm")
    dgu = types.ModuleType("deep_gemm.utils")
    dgu.align = lambda x, a: (x + a - 1) // a * a
    dgu.get_tma_aligned_size = lambda mn, elem: (mn + 16 // elem - 1) // (16 // elem) * (16 // elem)
    dg.utils = dgu
    sys.modules.setdefault("deep_gemm", dg)
    sys.modules.setdefault("deep_gemm.utils", dgu)
    from sglang.srt.layers.quantization import fp8_utils as FU

    out = {}
    torch.manual_seed(2)
    w = (torch.randn(300, 520) * 0.02).bfloat16()
    w[:128, 128:256] = 0  # an all-zero block: amax clamps at 1e-4
    rq, rs = FU.quant_weight_ue8m0(w, [128, 128])
    oq, os_ = O.quant_weight_ue8m0(w)
    assert torch.equal(rq.view(torch.uint8), oq.view(torch.uint8)) and torch.equal(rs, os_)
    x = torch.rand(1000) * 10 + 1e-6
    assert torch.equal(FU.ceil_to_ue8m0(x), O.ceil_pow2(x))
    sf_rows = rs.index_select(-2, torch.arange(300) // 128)
    rp = FU._get_mn_major_tma_aligned_packed_ue8m0_tensor_torch_impl(sf_rows)
    op = O.pack_ue8m0_mn_major(sf_rows)
    assert rp.shape == op.shape and rp.stride() == op.stride() and torch.equal(rp, op)
    ru = FU._unpack_ue8m0_scale_for_triton(rp.contiguous(), (300, 520), [128, 128])
    assert torch.equal(ru, rs)
    q0, s0 = O.block_quant_weight_fp8(w, (128, 128))
    rrq, rrs = FU.quant_weight_ue8m0(FU.block_quant_dequant(q0, s0, [128, 128], torch.bfloat16), [128, 128])
    for k, v in dict(w=w, q=rq, s=rs, packed=rp.contiguous(), q0=q0, s0=s0, requant_q=rrq, requant_s=rrs).items():
        out[f"w/{k}"] = raw(v)
    np.savez_compressed(os.path.join(HERE, "ue8m0.npz"), **out)
    print("ue8m0 ok")

    # ---- MoE: inputs as in TestW8A8BlockFP8FusedMoE (seed 0), fp32 and bf16 activations
    out = {}
    for name, M, N, K, E, topk, dt in [
        ("m_33x128x256_e8k2_f32", 33, 128, 256, 8, 2, torch.float32),
        ("m_5x256x256_e8k6_bf16", 5, 256, 256, 8, 6, torch.bfloat16),
    ]:
        torch.manual_seed(0)
        a = torch.randn(M, K, dtype=dt) / 10
        w1 = ((torch.rand(E, 2 * N, K) - 0.5) * 2 * 448).clamp(-448, 448).to(fp8)
        w2 = ((torch.rand(E, K, N) - 0.5) * 2 * 448).clamp(-448, 448).to(fp8)
        w1_s = torch.rand(E, (2 * N + 127) // 128, (K + 127) // 128) * 1e-2
        w2_s = torch.rand(E, (K + 127) // 128, (N + 127) // 128) * 1e-2
        score = torch.randn(M, E, dtype=dt)
        ref = R.torch_w8a8_block_fp8_moe(a, w1, w2, w1_s, w2_s, score, topk, [128, 128])
        sm = torch.softmax(score, dim=-1, dtype=torch.float32)
        tw, ti = torch.topk(sm, topk)
        mine = O.fused_experts_fp8(a, w1, w2, w1_s, w2_s, tw, ti.to(torch.int32), [128, 128], compute_dtype=dt)
        # the reference multiplies by the weights cast to the activation dtype and sums in it
        assert torch.allclose(ref.float(), mine.float(), rtol=2e-2 if dt == torch.bfloat16 else 1e-5, atol=1e-4), name
        if dt == torch.float32:
            assert O.rel_frobenius(mine, ref) < 1e-6
        for k, v in dict(a=a, w1=w1, w2=w2, w1_s=w1_s, w2_s=w2_s, tw=tw, ti=ti.to(torch.int32), out=ref.float()).items():
            out[f"{name}/{k}"] = raw(v)
        out[f"{name}/meta"] = np.array([M, N, K, E, topk, 0 if dt == torch.bfloat16 else 2])
    np.savez_compressed(os.path.join(HERE, "moe.npz"), **out)
    print("moe ok")

    # ---- routing
    def same_routing(rw, ri, ow, oi):
        # the reference's sorted=False calls leave the order of the k results unspecified; the
        # oracle pins it (descending, lower index first on ties): compare by expert id
        rw, ri = O.canonical_routing(rw, ri)
        ow, oi = O.canonical_routing(ow, oi)
        assert torch.equal(ri, oi)
        torch.testing.assert_close(rw, ow, rtol=1e-6, atol=0)

    out = {}
    torch.manual_seed(0)
    logits = torch.randn(17, 8)
    rw, ri = RT.fused_topk_torch_native(torch.zeros(17, 4), logits, 2, True)
    ow, oi = O.softmax_topk(logits, 2, True)
    assert torch.equal(rw, ow) and torch.equal(ri.to(torch.int32), oi)
    out["softmax/logits"], out["softmax/w"], out["softmax/ids"] = raw(logits), raw(rw), raw(ri.to(torch.int32))
    impl = RT.biased_grouped_topk_impl
    impl = getattr(impl, "_torchdynamo_orig_callable", None) or getattr(impl, "__wrapped__", impl)
    logits = torch.randn(19, 256)
    bias = torch.randn(256) * 0.01
    rw, ri = impl(torch.zeros(19, 4), logits, bias, 8, True, 8, 4)
    ow, oi = O.biased_grouped_topk(logits, bias, 8, 8, 4, True)
    same_routing(rw, ri, ow, oi)
    out["grouped/logits"], out["grouped/bias"], out["grouped/w"], out["grouped/ids"] = raw(logits), raw(bias), raw(rw), raw(ri)
    # sigmoid scores with a correction bias, no groups (fused_topk_torch_native :550-588)
    logits = torch.randn(23, 64)
    bias = torch.randn(64) * 0.05
    rw, ri = RT.fused_topk_torch_native(torch.zeros(23, 4), logits, 6, True, correction_bias=bias, scoring_func="sigmoid")
    ow, oi = O.sigmoid_topk(logits, 6, True, bias)
    same_routing(rw, ri.to(torch.int32), ow, oi)
    out["sigmoid/logits"], out["sigmoid/bias"], out["sigmoid/w"], out["sigmoid/ids"] = raw(logits), raw(bias), raw(rw), raw(ri.to(torch.int32))
    # softmax scores, group score = maximum (grouped_topk_gpu :703-764; DeepSeek-V2 shape: 160 experts, 8 groups)
    impl = RT.grouped_topk_gpu
    impl = getattr(impl, "_torchdynamo_orig_callable", None) or getattr(impl, "__wrapped__", impl)
    logits = torch.randn(21, 160)
    rw, ri = impl(torch.zeros(21, 4), logits, 6, True, 8, 3)
    ow, oi = O.grouped_topk(logits, 6, 8, 3, True)
    same_routing(rw, ri, ow, oi)
    out["grouped_softmax/logits"], out["grouped_softmax/w"], out["grouped_softmax/ids"] = raw(logits), raw(rw), raw(ri)
    # shared experts fused into the routed ones: the reference replaces the last (smallest) slot of the sorted
    # top-k by a shared-expert replica drawn at random, so the weights and the routed ids are what is pinned
    impl = RT.biased_grouped_topk_impl
    impl = getattr(impl, "_torchdynamo_orig_callable", None) or getattr(impl, "__wrapped__", impl)
    logits = torch.randn(13, 256)
    bias = torch.randn(256) * 0.01
    rw, ri = impl(torch.zeros(13, 4), logits, bias, 9, True, 8, 4, 2, 2.5, False)
    raw_w, raw_i = O.biased_grouped_topk(logits, bias, 9, 8, 4, False)
    ow, oi = O.fused_shared_experts_tail(raw_w, raw_i, True, 2.5, False)
    assert torch.equal(ri[:, :-1], oi) and bool(((ri[:, -1] >= 256) & (ri[:, -1] < 258)).all())
    torch.testing.assert_close(rw, ow, rtol=1e-6, atol=0)
    out["grouped_shared/logits"], out["grouped_shared/bias"] = raw(logits), raw(bias)
    out["grouped_shared/w"], out["grouped_shared/routed_ids"] = raw(rw), raw(ri[:, :-1].contiguous())
    impl = RT.grouped_topk_gpu
    impl = getattr(impl, "_torchdynamo_orig_callable", None) or getattr(impl, "__wrapped__", impl)
    logits = torch.randn(11, 160)
    rw, ri = impl(torch.zeros(11, 4), logits, 7, True, 8, 3, 1, 16.0, True)
    raw_w, raw_i = O.grouped_topk(logits, 7, 8, 3, False)
    ow, oi = O.fused_shared_experts_tail(raw_w, raw_i, True, 16.0, True)
    assert torch.equal(ri[:, :-1], oi) and bool((ri[:, -1] == 160).all())
    torch.testing.assert_close(rw, ow, rtol=1e-6, atol=0)
    out["grouped_softmax_shared/logits"], out["grouped_softmax_shared/w"] = raw(logits), raw(rw)
    out["grouped_softmax_shared/routed_ids"] = raw(ri[:, :-1].contiguous())
    np.savez_compressed(os.path.join(HERE, "routing.npz"), **out)
    print("routing ok")

    # ---- align: the docstring example of moe_align_block_size.py:44-57 (literal known answer)
    out = {
        "doc/topk_ids": np.array([[2, 3, 4], [1, 2, 4], [1, 3, 4], [1, 2, 3]], dtype=np.int32) - 1,
        "doc/block_size": np.array(4),
        "doc/num_experts": np.array(4),
        "doc/sorted_ids": np.array([3, 6, 9, 12, 0, 4, 10, 12, 1, 7, 11, 12, 2, 5, 8, 12], dtype=np.int32),
    }
    # NOTE: the docstring numbers experts 1..4; the kernel's ids are 0-based, hence the -1.
    s, e, n, c = O.moe_align_block_size(torch.from_numpy(out["doc/topk_ids"]), 4, 4)
    assert n.item() == 16 and s[:16].tolist() == out["doc/sorted_ids"].tolist(), s
    assert e[:4].tolist() == [0, 1, 2, 3]
    np.savez_compressed(os.path.join(HERE, "align.npz"), **out)
    print("align ok")


if __name__ == "__main__":
    main()
