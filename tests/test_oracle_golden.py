"""The oracle against the vectors produced by the reference's own functions
(tests/golden/make_golden.py) -- runs on CPU."""
import torch

import oracle as O
from conftest import DT, as_fp8, golden_tensor, load_golden


def test_quant_matches_reference_vectors():
    for name, c in load_golden("quant.npz").items():
        m, d, g, code = c["meta"].tolist()
        x = golden_tensor(c["x"], code)
        q, s = O.per_token_group_quant_fp8(x, g)
        assert torch.equal(q.view(torch.uint8), torch.from_numpy(c["q"])), name
        assert torch.equal(s, torch.from_numpy(c["s"])), name


def test_quant_all_zero_group_uses_fp32_eps():
    x = torch.zeros(2, 256, dtype=torch.bfloat16)
    x[1, 130] = 1.0
    q, s = O.per_token_group_quant_fp8(x, 128)
    assert s[0, 0].item() == torch.tensor(1e-10, dtype=torch.float32).div(448.0).item()
    assert q.view(torch.uint8)[0].eq(0).all()
    assert q[1, 130].float().item() == 448.0


def test_quant_formula_variants_close():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(16, 512, generator=g).bfloat16()
    q0, s0 = O.per_token_group_quant_fp8(x, 128, formula=0)
    for f in (1, 2):
        q, s = O.per_token_group_quant_fp8(x, 128, formula=f)
        assert torch.allclose(s, s0, rtol=1e-6)
        assert (q.view(torch.uint8) != q0.view(torch.uint8)).float().mean() < 0.01


def test_gemm_matches_reference_vectors():
    for name, c in load_golden("gemm.npz").items():
        C = O.w8a8_block_fp8_matmul(
            as_fp8(c["A"]), as_fp8(c["B"]), torch.from_numpy(c["As"]), torch.from_numpy(c["Bs"]), [128, 128],
            torch.float32,
        )
        assert torch.equal(C, torch.from_numpy(c["C"])), name


def test_weight_quant_matches_reference_vectors():
    c = load_golden("weight_quant.npz")["w"]
    q, s = O.block_quant_weight_fp8(golden_tensor(c["w"], 0), (128, 128))
    assert torch.equal(q.view(torch.uint8), torch.from_numpy(c["q"]))
    assert torch.equal(s, torch.from_numpy(c["s"]))


def test_moe_matches_reference_vectors():
    for name, c in load_golden("moe.npz").items():
        M, Nn, K, E, topk, code = c["meta"].tolist()
        a = golden_tensor(c["a"], code)
        out = O.fused_experts_fp8(
            a, as_fp8(c["w1"]), as_fp8(c["w2"]), torch.from_numpy(c["w1_s"]), torch.from_numpy(c["w2_s"]),
            torch.from_numpy(c["tw"]), torch.from_numpy(c["ti"]), [128, 128], compute_dtype=DT[code],
        )
        ref = torch.from_numpy(c["out"])
        tol = 2e-2 if code == 0 else 1e-6
        assert O.rel_frobenius(out.float(), ref) < tol, name


def _same_routing(w, ids, ref_w, ref_ids):
    """The reference's ``sorted=False`` calls leave the order of the k results (and with it the
    last bit of the renormalising sum) unspecified: compare by expert id, weights to 1e-6."""
    w, ids = O.canonical_routing(w, ids)
    ref_w, ref_ids = O.canonical_routing(ref_w, ref_ids)
    assert torch.equal(ids, ref_ids)
    torch.testing.assert_close(w, ref_w, rtol=1e-6, atol=0)


def test_routing_matches_reference_vectors():
    c = load_golden("routing.npz")
    w, ids = O.softmax_topk(torch.from_numpy(c["softmax"]["logits"]), 2, True)
    assert torch.equal(w, torch.from_numpy(c["softmax"]["w"])) and torch.equal(ids, torch.from_numpy(c["softmax"]["ids"]))
    g = c["grouped"]
    w, ids = O.biased_grouped_topk(torch.from_numpy(g["logits"]), torch.from_numpy(g["bias"]), 8, 8, 4, True)
    _same_routing(w, ids, torch.from_numpy(g["w"]), torch.from_numpy(g["ids"]))
    g = c["sigmoid"]
    w, ids = O.sigmoid_topk(torch.from_numpy(g["logits"]), 6, True, torch.from_numpy(g["bias"]))
    _same_routing(w, ids, torch.from_numpy(g["w"]), torch.from_numpy(g["ids"]))
    g = c["grouped_softmax"]
    w, ids = O.grouped_topk(torch.from_numpy(g["logits"]), 6, 8, 3, True)
    _same_routing(w, ids, torch.from_numpy(g["w"]), torch.from_numpy(g["ids"]))


def test_fused_shared_experts_tail_matches_reference_vectors():
    """Shared experts fused into the routed ones (topk.py:735-764, 968-992): the weights of all k slots and
    the routed ids (the shared slot's id is drawn at random by the reference)."""
    c = load_golden("routing.npz")
    g = c["grouped_shared"]
    raw_w, raw_i = O.biased_grouped_topk(torch.from_numpy(g["logits"]), torch.from_numpy(g["bias"]), 9, 8, 4, False)
    w, routed = O.fused_shared_experts_tail(raw_w, raw_i, True, 2.5, False)
    assert torch.equal(routed, torch.from_numpy(g["routed_ids"]))
    torch.testing.assert_close(w, torch.from_numpy(g["w"]), rtol=1e-6, atol=0)
    g = c["grouped_softmax_shared"]
    raw_w, raw_i = O.grouped_topk(torch.from_numpy(g["logits"]), 7, 8, 3, False)
    w, routed = O.fused_shared_experts_tail(raw_w, raw_i, True, 16.0, True)
    assert torch.equal(routed, torch.from_numpy(g["routed_ids"]))
    torch.testing.assert_close(w, torch.from_numpy(g["w"]), rtol=1e-6, atol=0)


def test_align_docstring_example():
    c = load_golden("align.npz")["doc"]
    s, e, n, cum = O.moe_align_block_size(torch.from_numpy(c["topk_ids"]), int(c["block_size"]), int(c["num_experts"]))
    assert n.item() == 16
    assert s[:16].tolist() == c["sorted_ids"].tolist()
    assert e[:4].tolist() == [0, 1, 2, 3]


def test_align_properties_and_minus_one_bucket():
    g = torch.Generator().manual_seed(0)
    for numel, E, bs in [(1, 8, 16), (37, 8, 4), (5000, 256, 128), (300, 32, 64)]:
        ids = torch.randint(-1, E, (numel,), generator=g, dtype=torch.int32)
        s, e, n, cum = O.moe_align_block_size(ids.view(-1, 1), bs, E)
        total = n.item()
        assert total % bs == 0 and total <= s.numel()
        real = s[:total][s[:total] < numel]
        assert sorted(real.tolist()) == list(range(numel))  # a permutation of every flat index
        for blk in range(total // bs):
            seg = s[blk * bs : (blk + 1) * bs]
            seg = seg[seg < numel]
            assert (ids[seg.long()] == e[blk]).all()
            assert (seg[1:] > seg[:-1]).all()  # ascending inside a block
        assert (e[total // bs :] == -1).all()
        assert cum[E + 1].item() == total


def test_ep_local_expert_ids():
    ids = torch.tensor([[0, 5], [7, 3]], dtype=torch.int32)
    assert O.ep_local_expert_ids(ids, 8, 2, 1).tolist() == [[-1, 1], [3, -1]]


def test_ue8m0_weight_side_matches_reference_vectors():
    c = load_golden("ue8m0.npz")["w"]
    w = torch.from_numpy(c["w"]).view(torch.bfloat16)
    q, s = O.quant_weight_ue8m0(w)
    assert torch.equal(q.view(torch.uint8), torch.from_numpy(c["q"])) and torch.equal(s, torch.from_numpy(c["s"]))
    rows = s.index_select(-2, torch.arange(w.shape[0]) // 128)
    packed = O.pack_ue8m0_mn_major(rows)
    assert torch.equal(packed.contiguous(), torch.from_numpy(c["packed"])) and packed.stride() == (1, w.shape[0])
    x = torch.tensor([1.0, 1.5, 2.0, 3e-5, 448.0, 0.75])
    assert O.ceil_pow2(x).tolist() == [1.0, 2.0, 2.0, 2.0**-15, 512.0, 1.0]
