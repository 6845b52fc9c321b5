"""Routing kernel (softmax / sigmoid top-k, grouped and biased grouped top-k) vs the oracle and
the reference's vectors. Expert ids must match exactly; weights are compared with rtol 1e-5
(fp32 exp and summation order differ from the CPU library in the last bits). The reference
leaves the order of the k results unspecified, so rows are compared sorted by expert id; the
kernel's own order (descending selection value) is checked separately."""
import pytest
import torch

import oracle as O
from conftest import load_golden

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-5, 1e-8


def _same(w, ids, ref_w, ref_ids):
    w, ids = O.canonical_routing(w.cpu(), ids.cpu())
    ref_w, ref_ids = O.canonical_routing(ref_w, ref_ids)
    assert torch.equal(ids, ref_ids)
    torch.testing.assert_close(w, ref_w, rtol=RTOL, atol=ATOL)


def test_reference_vectors():
    from sglang_b200 import topk as R

    c = load_golden("routing.npz")
    g = c["softmax"]
    x = torch.from_numpy(g["logits"]).cuda()
    w, ids = R.fused_topk(x, x, 2, True)
    _same(w, ids, torch.from_numpy(g["w"]), torch.from_numpy(g["ids"]))
    assert torch.equal(ids.cpu(), torch.from_numpy(g["ids"]))  # sorted=True in the reference: same order
    g = c["grouped"]
    x = torch.from_numpy(g["logits"]).cuda()
    w, ids = R.biased_grouped_topk(x, x, torch.from_numpy(g["bias"]).cuda(), 8, True, 8, 4)
    _same(w, ids, torch.from_numpy(g["w"]), torch.from_numpy(g["ids"]))
    w2, ids2 = R.moe_fused_gate(x, torch.from_numpy(g["bias"]).cuda(), 8, 4, 8)
    assert torch.equal(ids2, ids) and torch.equal(w2, w)
    g = c["sigmoid"]
    x = torch.from_numpy(g["logits"]).cuda()
    w, ids = R.fused_topk(x, x, 6, True, torch.from_numpy(g["bias"]).cuda(), "sigmoid")
    _same(w, ids, torch.from_numpy(g["w"]), torch.from_numpy(g["ids"]))
    g = c["grouped_softmax"]
    x = torch.from_numpy(g["logits"]).cuda()
    w, ids = R.grouped_topk(x, x, 6, True, 8, 3)
    _same(w, ids, torch.from_numpy(g["w"]), torch.from_numpy(g["ids"]))


def test_fused_shared_experts_reference_vectors():
    """``num_fused_shared_experts > 0``: routed slots and all weights against the reference's vectors; the shared
    slot's id is random in the reference, so it is checked for its range."""
    from sglang_b200 import topk as R

    c = load_golden("routing.npz")
    g = c["grouped_shared"]
    x = torch.from_numpy(g["logits"]).cuda()
    w, ids = R.biased_grouped_topk(x, x, torch.from_numpy(g["bias"]).cuda(), 9, True, 8, 4, 2, 2.5, False)
    assert w.dtype == torch.float32 and ids.dtype == torch.int32 and tuple(ids.shape) == (13, 9)
    assert torch.equal(ids[:, :-1].cpu(), torch.from_numpy(g["routed_ids"]))
    assert bool(((ids[:, -1] >= 256) & (ids[:, -1] < 258)).all())
    torch.testing.assert_close(w.cpu(), torch.from_numpy(g["w"]), rtol=RTOL, atol=ATOL)
    g = c["grouped_softmax_shared"]
    x = torch.from_numpy(g["logits"]).cuda()
    w, ids = R.grouped_topk(x, x, 7, True, 8, 3, 1, 16.0, True)
    assert torch.equal(ids[:, :-1].cpu(), torch.from_numpy(g["routed_ids"])) and bool((ids[:, -1] == 160).all())
    torch.testing.assert_close(w.cpu(), torch.from_numpy(g["w"]), rtol=RTOL, atol=ATOL)
    # through the config dispatch, with padded rows masked
    cfg = R.TopKConfig(top_k=7, use_grouped_topk=True, topk_group=3, num_expert_group=8, renormalize=True,
                       num_fused_shared_experts=1, routed_scaling_factor=16.0, apply_routed_scaling_factor_on_output=True)
    out = R.select_experts(x, x, cfg, num_token_non_padded=torch.tensor(5, device="cuda"))
    assert torch.equal(out.topk_ids[:5], ids[:5]) and bool((out.topk_ids[5:] == -1).all())


@pytest.mark.parametrize("T,E,topk", [(1, 8, 2), (17, 8, 2), (64, 60, 4), (333, 128, 8), (16, 256, 8), (5, 1024, 32),
                                      (7, 48, 3), (4097, 64, 6), (3, 2, 1), (9, 33, 33 - 1)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_softmax_and_sigmoid_topk(T, E, topk, dtype):
    from sglang_b200 import topk as R

    g = torch.Generator().manual_seed(T * 7 + E)
    logits = (torch.randn(T, E, generator=g) * 2).to(dtype)
    bias = torch.randn(E, generator=g) * 0.1
    x = logits.cuda()
    for renorm in (True, False):
        w, ids = R.fused_topk(x, x, topk, renorm)
        _same(w, ids, *O.softmax_topk(logits, topk, renorm))
        assert w.dtype == torch.float32 and ids.dtype == torch.int32 and tuple(ids.shape) == (T, topk)
        w, ids = R.fused_topk(x, x, topk, renorm, bias.cuda(), "sigmoid")
        _same(w, ids, *O.sigmoid_topk(logits, topk, renorm, bias))
        w, ids = R.fused_topk(x, x, topk, renorm, None, "sigmoid")
        _same(w, ids, *O.sigmoid_topk(logits, topk, renorm, None))
    # in place, sgl-kernel style
    w = torch.empty(T, topk, device="cuda")
    ids = torch.empty(T, topk, dtype=torch.int32, device="cuda")
    R.topk_softmax(w, ids, x, True)
    _same(w, ids, *O.softmax_topk(logits, topk, True))
    R.topk_sigmoid(w, ids, x, False, bias.cuda())
    _same(w, ids, *O.sigmoid_topk(logits, topk, False, bias))


@pytest.mark.parametrize("T,E,n_group,topk_group,topk", [(19, 256, 8, 4, 8), (300, 256, 8, 4, 8), (21, 160, 8, 3, 6),
                                                        (33, 64, 4, 2, 6), (8, 1024, 16, 4, 16), (5, 96, 3, 2, 4),
                                                        (11, 64, 32, 8, 8), (2048, 256, 8, 4, 8)])
def test_grouped_topk(T, E, n_group, topk_group, topk):
    from sglang_b200 import topk as R

    g = torch.Generator().manual_seed(T + E + n_group)
    logits = torch.randn(T, E, generator=g)
    bias = torch.randn(E, generator=g) * 0.05
    x = logits.cuda()
    w, ids = R.biased_grouped_topk(x, x, bias.cuda(), topk, True, n_group, topk_group)
    _same(w, ids, *O.biased_grouped_topk(logits, bias, topk, n_group, topk_group, True))
    w, ids = R.biased_grouped_topk(x, x, bias.cuda(), topk, True, n_group, topk_group, routed_scaling_factor=2.5,
                                   apply_routed_scaling_factor_on_output=True)
    _same(w, ids, *O.biased_grouped_topk(logits, bias, topk, n_group, topk_group, True, routed_scaling_factor=2.5))
    w, ids = R.biased_grouped_topk(x, x, bias.cuda(), topk, False, n_group, topk_group)
    _same(w, ids, *O.biased_grouped_topk(logits, bias, topk, n_group, topk_group, False))
    if E // n_group >= 2:  # the softmax variant's group score is a maximum: any group size
        w, ids = R.grouped_topk(x, x, topk, True, n_group, topk_group)
        _same(w, ids, *O.grouped_topk(logits, topk, n_group, topk_group, True))


def test_order_ties_padding_and_config_dispatch():
    from sglang_b200 import topk as R

    # descending selection value; ties -> lower expert index first
    logits = torch.tensor([[0.5, 2.0, 2.0, -1.0, 2.0, 0.5, 0.0, 0.5]], device="cuda")
    w, ids = R.fused_topk(logits, logits, 5, False)
    assert ids.tolist() == [[1, 2, 4, 0, 5]]
    assert torch.all(w[:, :-1] >= w[:, 1:])
    # equal group scores: lower group index is kept
    x = torch.zeros(1, 16, device="cuda")
    w, ids = R.biased_grouped_topk(x, x, torch.zeros(16, device="cuda"), 4, True, 4, 2)
    assert ids.tolist() == [[0, 1, 2, 3]] and torch.allclose(w, torch.full_like(w, 0.25))
    # rows past num_token_non_padded get id -1
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(10, 256, generator=g)
    x = logits.cuda()
    nvalid = torch.tensor(6, device="cuda")
    w, ids = R.biased_grouped_topk(x, x, torch.zeros(256, device="cuda"), 8, True, 8, 4, num_token_non_padded=nvalid)
    rw, ri = O.biased_grouped_topk(logits, torch.zeros(256), 8, 8, 4, True)
    _same(w[:6], ids[:6], rw[:6], ri[:6])
    assert torch.all(ids[6:] == -1)
    # select_experts dispatches on the config like the reference
    out = R.select_experts(x, x, R.TopKConfig(top_k=8, use_grouped_topk=True, topk_group=4, num_expert_group=8,
                                              correction_bias=torch.zeros(256, device="cuda")))
    _same(out.topk_weights, out.topk_ids, rw, ri)
    out = R.select_experts(x, x, R.TopKConfig(top_k=4))
    _same(out.topk_weights, out.topk_ids, *O.softmax_topk(logits, 4, True))
    # empty batch, and preconditions
    e = torch.empty(0, 8, device="cuda")
    w, ids = R.fused_topk(e, e, 2, True)
    assert tuple(w.shape) == (0, 2)
    with pytest.raises(AssertionError):
        R.fused_topk(x, x, 300, True)
    with pytest.raises(NotImplementedError):  # the sgl-kernel style fused gate does not take shared experts here
        R.moe_fused_gate(x, torch.zeros(256, device="cuda"), 8, 4, 8, num_fused_shared_experts=1)


def test_routing_feeds_fused_experts_under_graph_capture():
    """The kernel allocates nothing and takes its stream from torch: usable inside a CUDA graph."""
    from sglang_b200 import topk as R

    g = torch.Generator().manual_seed(9)
    logits = torch.randn(64, 256, generator=g)
    x = logits.cuda()
    w = torch.empty(64, 8, device="cuda")
    ids = torch.empty(64, 8, dtype=torch.int32, device="cuda")
    bias = torch.zeros(256, device="cuda")
    s = torch.cuda.Stream()
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        R._route(x, 8, True, R.SIGMOID, bias, 8, 4, R.GROUP_TOP2_SUM, topk_weights=w, topk_ids=ids)
        torch.cuda.synchronize()
        w.zero_()
        with torch.cuda.graph(gr, stream=s):
            R._route(x, 8, True, R.SIGMOID, bias, 8, 4, R.GROUP_TOP2_SUM, topk_weights=w, topk_ids=ids)
    gr.replay()
    torch.cuda.synchronize()
    _same(w, ids, *O.biased_grouped_topk(logits, torch.zeros(256), 8, 8, 4, True))


@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (37, 64, 6), (256, 128, 8), (19, 200, 4)])
@pytest.mark.parametrize("cap,with_bias", [(30.0, False), (0.0, True), (5.0, True)])
def test_softmax_with_softcapping_and_bias(T, E, k, cap, with_bias):
    """``topk_softmax(..., moe_softcapping, correction_bias)``: both act on the logits before the softmax.
    Weights to rtol 1e-5 (tanh and exp of the device library against the host's); ids exact except where two
    scores are closer than that tolerance, which the comparison of weight-sorted values covers."""
    from sglang_b200 import topk as R

    g = torch.Generator().manual_seed(100 * T + E + k)
    x = torch.randn(T, E, generator=g) * 4
    bias = torch.randn(E, generator=g) * 0.5 if with_bias else None
    w = torch.empty(T, k, device="cuda")
    ids = torch.empty(T, k, dtype=torch.int32, device="cuda")
    for renorm in (False, True):
        R.topk_softmax(w, ids, x.cuda(), renorm, cap, bias.cuda() if with_bias else None)
        ref_w, ref_ids = O.softmax_topk_capped(x, k, renorm, cap, bias)
        torch.testing.assert_close(w.cpu(), ref_w, rtol=1e-5, atol=1e-8)
        same = ids.cpu() == ref_ids
        if not bool(same.all()):  # a swap is only acceptable between scores equal within the tolerance
            torch.testing.assert_close(w.cpu()[~same], ref_w[~same], rtol=1e-5, atol=1e-8)
            assert torch.equal(torch.sort(ids.cpu(), dim=1).values, torch.sort(ref_ids, dim=1).values)
    # the dispatcher op takes the same arguments
    w2 = torch.empty_like(w)
    ids2 = torch.empty_like(ids)
    torch.ops.sglang_b200.topk_softmax(w2, ids2, x.cuda(), True, cap, bias.cuda() if with_bias else None)
    assert torch.equal(w2, w) and torch.equal(ids2, ids)
    # off switches fall back to the plain kernel's result
    R.topk_softmax(w, ids, x.cuda(), True, 0.0, None)
    pw, pids = R.fused_topk(x.cuda(), x.cuda(), k, True)
    assert torch.equal(w, pw) and torch.equal(ids, pids)
