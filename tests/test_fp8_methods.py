"""Weight-side objects: config parsing, parameter creation, checkpoint loading with tensor-parallel
sharding (CPU), and ``apply`` through the kernels (GPU)."""
import os

import pytest
import torch

import oracle as O
from conftest import make_activation, make_weight


def _checkpoint(tmp_path):
    """A tiny block-FP8 checkpoint: one attention block, one dense MLP, two experts."""
    from safetensors.torch import save_file

    H, I, E = 256, 512, 2
    t = {}
    for i, (name, n, k) in enumerate([("self_attn.q_proj", 512, H), ("self_attn.k_proj", 256, H), ("self_attn.v_proj", 256, H),
                                      ("self_attn.o_proj", H, 512), ("mlp.gate_proj", I, H), ("mlp.up_proj", I, H),
                                      ("mlp.down_proj", H, I)]):
        q, s = make_weight(n, k, 100 + i)
        t[f"model.layers.0.{name}.weight"], t[f"model.layers.0.{name}.weight_scale_inv"] = q, s
    for e in range(E):
        for j, (proj, n, k) in enumerate([("gate_proj", I, H), ("down_proj", H, I), ("up_proj", I, H)]):
            q, s = make_weight(n, k, 200 + 10 * e + j)
            t[f"model.layers.0.moe.experts.{e}.{proj}.weight"] = q
            t[f"model.layers.0.moe.experts.{e}.{proj}.weight_scale_inv"] = s
    t["model.layers.0.input_layernorm.weight"] = torch.ones(H, dtype=torch.bfloat16)
    path = os.path.join(tmp_path, "model.safetensors")
    save_file({k: v.contiguous() for k, v in t.items()}, path)
    return path, t, (H, I, E)


def _load(path, tp_rank, tp_size, device=None):
    from sglang_b200 import fp8 as F

    cfg = F.Fp8Config.from_config({"quant_method": "fp8", "activation_scheme": "dynamic", "weight_block_size": [128, 128],
                                   "modules_to_not_convert": ["model.lm_head"]})
    assert cfg.is_checkpoint_fp8_serialized and cfg.weight_block_size == [128, 128] and cfg.is_layer_skipped("lm_head.x")
    lin = F.Fp8LinearMethod(cfg, tp_size)
    H, I, E = 256, 512, 2
    layers = {n: torch.nn.Module() for n in ("qkv_proj", "o_proj", "gate_up_proj", "down_proj", "experts")}
    lin.create_weights(layers["qkv_proj"], H, [512 // tp_size, 256 // tp_size, 256 // tp_size], H, 1024, torch.bfloat16, device=device)
    lin.create_weights(layers["o_proj"], 512 // tp_size, [H], 512, H, torch.bfloat16, device=device)
    lin.create_weights(layers["gate_up_proj"], H, [I // tp_size] * 2, H, 2 * I, torch.bfloat16, device=device)
    lin.create_weights(layers["down_proj"], I // tp_size, [H], I, H, torch.bfloat16, device=device)
    moe = F.Fp8MoEMethod(cfg)
    moe.create_weights(layers["experts"], E, H, I // tp_size, torch.bfloat16, device=device)
    offsets = {"q": 0, "k": 512 // tp_size, "v": (512 + 256) // tp_size, 0: 0, 1: I // tp_size}
    others = []
    for name, w, s in F.iter_block_fp8_pairs(F.load_safetensors(path)):
        if s is None:
            others.append(name)
            continue
        leaf = name.split(".")[-1]
        if ".experts." in name:
            e = int(name.split(".experts.")[1].split(".")[0])
            F.load_expert_shard(layers["experts"], e, {"gate_proj": "w1", "down_proj": "w2", "up_proj": "w3"}[leaf], w, s,
                                tp_rank, tp_size)
        elif leaf in F.STACKED_PARAMS:
            target, shard_id = F.STACKED_PARAMS[leaf]
            F.load_linear_shard(layers[target], w, s, "column", tp_rank, tp_size, offsets[shard_id])
        else:
            F.load_linear_shard(layers[leaf], w, s, "row", tp_rank, tp_size)
    assert others == ["model.layers.0.input_layernorm.weight"]
    for n in ("qkv_proj", "o_proj", "gate_up_proj", "down_proj"):
        lin.process_weights_after_loading(layers[n])
    moe.process_weights_after_loading(layers["experts"])
    return cfg, lin, moe, layers


@pytest.mark.parametrize("tp_size", [1, 2])
def test_checkpoint_loads_into_sharded_parameters(tmp_path, tp_size):
    path, t, (H, I, E) = _checkpoint(str(tmp_path))
    P = "model.layers.0."
    for rank in range(tp_size):
        _, _, _, L = _load(path, rank, tp_size)
        rows = lambda x, r=rank: x.chunk(tp_size, 0)[r]
        cols = lambda x, r=rank: x.chunk(tp_size, 1)[r]
        qkv = torch.cat([rows(t[P + f"self_attn.{p}_proj.weight"]).view(torch.uint8) for p in "qkv"])
        assert torch.equal(L["qkv_proj"].weight.data.view(torch.uint8), qkv)
        qkv_s = torch.cat([rows(t[P + f"self_attn.{p}_proj.weight_scale_inv"]) for p in "qkv"])
        assert torch.equal(L["qkv_proj"].weight_scale_inv.data, qkv_s)
        assert torch.equal(L["o_proj"].weight.data.view(torch.uint8), cols(t[P + "self_attn.o_proj.weight"]).contiguous().view(torch.uint8))
        assert torch.equal(L["o_proj"].weight_scale_inv.data, cols(t[P + "self_attn.o_proj.weight_scale_inv"]))
        gu_s = torch.cat([rows(t[P + f"mlp.{p}_proj.weight_scale_inv"]) for p in ("gate", "up")])
        assert torch.equal(L["gate_up_proj"].weight_scale_inv.data, gu_s)
        assert torch.equal(L["down_proj"].weight_scale_inv.data, cols(t[P + "mlp.down_proj.weight_scale_inv"]))
        for e in range(E):
            w13 = torch.cat([rows(t[P + f"moe.experts.{e}.{p}_proj.weight"]).view(torch.uint8) for p in ("gate", "up")])
            assert torch.equal(L["experts"].w13_weight.data[e].view(torch.uint8), w13)
            assert torch.equal(L["experts"].w2_weight.data[e].view(torch.uint8),
                               cols(t[P + f"moe.experts.{e}.down_proj.weight"]).contiguous().view(torch.uint8))


def test_shape_rules_and_unsupported_configs():
    from sglang_b200 import fp8 as F

    with pytest.raises(NotImplementedError):
        F.Fp8Config(True, "static")
    with pytest.raises(NotImplementedError):
        F.Fp8Config(True, "dynamic", weight_block_size=[64, 64])
    with pytest.raises(ValueError):
        F.Fp8Config(False, "dynamic", weight_block_size=[128, 128])
    with pytest.raises(ValueError):  # a row-parallel shard of 192 columns does not hold whole K blocks
        F.validate_block_quant_shapes(384, 192, 256, 256, [256], 2)
    with pytest.raises(ValueError):  # merged partitions must hold whole N blocks
        F.validate_block_quant_shapes(256, 256, 320, 320, [192, 128], 1)
    F.validate_block_quant_shapes(256, 256, 512, 512, [256, 128, 128], 1)
    with pytest.raises(ValueError):
        list(F.iter_block_fp8_pairs([("a.weight", torch.zeros(2, 2).to(torch.float8_e4m3fn))]))


@pytest.mark.gpu
def test_apply_through_the_kernels(tmp_path):
    import sglang_b200 as S

    path, t, (H, I, E) = _checkpoint(str(tmp_path))
    cfg, lin, moe, L = _load(path, 0, 1, device="cuda")
    P = "model.layers.0."
    x = make_activation(40, H, 9)
    y = lin.apply(L["gate_up_proj"], x.cuda())
    wq = torch.cat([t[P + "mlp.gate_proj.weight"].view(torch.uint8), t[P + "mlp.up_proj.weight"].view(torch.uint8)]).view(torch.float8_e4m3fn)
    ws = torch.cat([t[P + "mlp.gate_proj.weight_scale_inv"], t[P + "mlp.up_proj.weight_scale_inv"]])
    ref = O.w8a8_block_fp8_linear(x, wq, ws, output_dtype=torch.float32)
    assert O.rel_frobenius(y.float().cpu(), ref) < 1e-2
    # a 16-bit checkpoint is quantised after loading
    cfg16 = S.fp8.Fp8Config(False, "dynamic")
    lin16 = S.fp8.Fp8LinearMethod(cfg16)
    layer = torch.nn.Module()
    lin16.create_weights(layer, H, [384], H, 384, torch.bfloat16, device="cuda")
    w = (torch.randn(384, H, generator=torch.Generator().manual_seed(1)) * 0.02).bfloat16()
    layer.weight.data.copy_(w)
    lin16.process_weights_after_loading(layer)
    oq, os_ = O.block_quant_weight_fp8(w, (128, 128))
    assert torch.equal(layer.weight.data.cpu().view(torch.uint8), oq.view(torch.uint8))
    assert O.rel_frobenius(lin16.apply(layer, x.cuda()).float().cpu(), O.w8a8_block_fp8_linear(x, oq, os_, output_dtype=torch.float32)) < 1e-2
    # power-of-two scales: re-quantised weights + packed scales, same operator
    lin.process_weights_after_loading(L["down_proj"], requant_ue8m0=True)
    assert L["down_proj"].weight_scale_inv.dtype == torch.int32
    xi = make_activation(40, I, 10)
    yd = lin.apply(L["down_proj"], xi.cuda())
    # oracle of the same pipeline: re-quantised weights (pinned to the reference's torch functions),
    # power-of-two activation scales, block GEMM
    from sglang_b200 import weight_quant as W

    rq, rs = W.requant_weight_ue8m0(t[P + "mlp.down_proj.weight"], t[P + "mlp.down_proj.weight_scale_inv"])
    assert torch.equal(L["down_proj"].weight.data.cpu().view(torch.uint8), rq.view(torch.uint8))
    aq, asf = O.per_token_group_quant_fp8_ue8m0(xi, 128)
    refd = O.w8a8_block_fp8_matmul(aq, rq, asf, W.unpack_ue8m0_scale(rs, (H, I)), [128, 128], output_dtype=torch.float32)
    assert O.rel_frobenius(yd.float().cpu(), refd) < 1e-2
    # and it stays within FP8 resolution of the unquantised product
    exact = xi.float() @ W.block_dequant_weight(t[P + "mlp.down_proj.weight"], t[P + "mlp.down_proj.weight_scale_inv"]).t()
    assert O.rel_frobenius(yd.float().cpu(), exact) < 8e-2
    # experts
    g = torch.Generator().manual_seed(2)
    xm = torch.randn(33, H, generator=g).bfloat16()
    tw, ti = O.softmax_topk(torch.randn(33, E, generator=g), 1, True)
    out = moe.apply(L["experts"], xm.cuda(), S.StandardTopKOutput(tw.cuda(), ti.cuda(), None))
    w1 = torch.stack([torch.cat([t[P + f"moe.experts.{e}.gate_proj.weight"].view(torch.uint8), t[P + f"moe.experts.{e}.up_proj.weight"].view(torch.uint8)]).view(torch.float8_e4m3fn) for e in range(E)])
    w1s = torch.stack([torch.cat([t[P + f"moe.experts.{e}.gate_proj.weight_scale_inv"], t[P + f"moe.experts.{e}.up_proj.weight_scale_inv"]]) for e in range(E)])
    w2 = torch.stack([t[P + f"moe.experts.{e}.down_proj.weight"] for e in range(E)])
    w2s = torch.stack([t[P + f"moe.experts.{e}.down_proj.weight_scale_inv"] for e in range(E)])
    refm = O.fused_experts_fp8(xm, w1, w2, w1s, w2s, tw, ti, [128, 128])
    assert O.rel_frobenius(out.float().cpu(), refm) < 1e-2
