"""Host-side pieces that need no GPU: weight quantiser, routing, synthetic inputs."""
import pytest
import torch

import oracle as O
from conftest import golden_tensor, load_golden


def test_package_weight_quantiser_is_bit_identical_to_oracle_and_reference():
    from sglang_b200.weight_quant import block_dequant_weight, block_quant_weight_fp8

    c = load_golden("weight_quant.npz")["w"]
    w = golden_tensor(c["w"], 0)
    q, s = block_quant_weight_fp8(w)
    assert torch.equal(q.view(torch.uint8), torch.from_numpy(c["q"])) and torch.equal(s, torch.from_numpy(c["s"]))
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(200, 300, generator=g) * 0.02).bfloat16()  # ragged: pads to 256 x 384
    q, s = block_quant_weight_fp8(w)
    oq, os_ = O.block_quant_weight_fp8(w)
    assert torch.equal(q.view(torch.uint8), oq.view(torch.uint8)) and torch.equal(s, os_)
    assert (block_dequant_weight(q, s) - w.float()).abs().max() < 0.02 * 4 / 8


def test_routing_refuses_cpu_tensors():
    """The routing kernels are CUDA only: a CPU tensor is an error, never a silent torch path."""
    from sglang_b200.topk import biased_grouped_topk, fused_topk

    logits = torch.randn(4, 8)
    with pytest.raises((AssertionError, RuntimeError)):
        fused_topk(torch.zeros(4, 4), logits, 2, True)
    with pytest.raises((AssertionError, RuntimeError)):
        biased_grouped_topk(torch.zeros(4, 4), logits, torch.zeros(8), 2, True, 2, 1)


def test_synthetic_inputs_are_seeded_and_shaped():
    from sglang_b200 import synthetic

    a = synthetic.activation(16, 4096, 7)
    b = synthetic.activation(16, 4096, 7)
    assert torch.equal(a, b) and a.dtype == torch.bfloat16
    col_amax = a.float().abs().amax(dim=0)
    assert (col_amax > 10).sum() >= 30  # ~1% of 4096 channels carry x20 outliers
    wq, ws = synthetic.weight(256, 384, 3)
    assert wq.dtype == torch.float8_e4m3fn and tuple(ws.shape) == (2, 3)
    lg = synthetic.zipf_router_logits(4096, 8, 1)
    _, ids = O.softmax_topk(lg, 2, True)
    counts = torch.bincount(ids.flatten().long(), minlength=8).float()
    assert counts.max() / counts.min().clamp(min=1) > 3  # skewed load


def test_ue8m0_weight_requant_and_scale_layout_on_cpu():
    """Load-time helpers are plain torch: check them against the reference's vectors without a GPU."""
    from sglang_b200 import weight_quant as W

    c = load_golden("ue8m0.npz")["w"]
    w = torch.from_numpy(c["w"]).view(torch.bfloat16)
    q, s = W.quant_weight_ue8m0(w)
    assert torch.equal(q.view(torch.uint8), torch.from_numpy(c["q"])) and torch.equal(s, torch.from_numpy(c["s"]))
    packed = W.transform_scale_ue8m0(s, mn=w.shape[0])
    assert packed.dtype == torch.int32 and packed.stride() == (1, 300)
    assert torch.equal(packed.contiguous(), torch.from_numpy(c["packed"]))
    assert torch.equal(W.unpack_ue8m0_scale(packed, tuple(w.shape)), s)
    rq, rs = W.requant_weight_ue8m0(torch.from_numpy(c["q0"]).view(torch.float8_e4m3fn), torch.from_numpy(c["s0"]))
    assert torch.equal(rq.view(torch.uint8), torch.from_numpy(c["requant_q"]))
    assert torch.equal(W.unpack_ue8m0_scale(rs, tuple(w.shape)), torch.from_numpy(c["requant_s"]))
    # every scale is a power of two and the re-quantised weight stays within FP8 resolution of the original
    assert torch.all(torch.frexp(s)[0] == 0.5)
    err = (W.block_dequant_weight(q, s) - w.float()).abs().max()
    assert err < 0.02 * 4 / 8
