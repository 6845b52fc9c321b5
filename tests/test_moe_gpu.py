"""fused_experts(use_fp8_w8a8=True, block_shape=[128,128]) vs the fp32 oracle and the
reference's vectors. Tolerance: relative Frobenius error <= 1e-2."""
import pytest
import torch

import oracle as O
from conftest import DT, as_fp8, golden_tensor, load_golden

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _status_ok():
    from sglang_b200 import _native

    assert _native.read_device_status() == 0, "a bounded device-side wait timed out"


def _weights(E, I, H, seed):
    g = torch.Generator().manual_seed(seed)
    w1 = torch.stack([O.block_quant_weight_fp8((torch.randn(2 * I, H, generator=g) * 0.02).bfloat16())[0] for _ in range(E)])
    w2 = torch.stack([O.block_quant_weight_fp8((torch.randn(H, I, generator=g) * 0.02).bfloat16())[0] for _ in range(E)])
    w1_s = torch.rand(E, 2 * I // 128, H // 128, generator=g) * 2e-4 + 1e-4
    w2_s = torch.rand(E, H // 128, I // 128, generator=g) * 2e-4 + 1e-4
    return w1, w2, w1_s, w2_s


def _run(x, w1, w2, w1_s, w2_s, tw, ti, **cfg):
    import sglang_b200 as S

    config = S.MoeRunnerConfig(**{"inplace": False, **cfg})
    out = S.fused_experts(
        x.cuda(), w1.cuda(), w2.cuda(), S.StandardTopKOutput(tw.cuda(), ti.cuda(), None), config,
        use_fp8_w8a8=True, w1_scale=w1_s.cuda(), w2_scale=w2_s.cuda(), block_shape=[128, 128],
    )
    _status_ok()
    return out


def test_reference_vectors():
    for name, c in load_golden("moe.npz").items():
        M, Nn, K, E, topk, code = c["meta"].tolist()
        a = golden_tensor(c["a"], code)
        args = (as_fp8(c["w1"]), as_fp8(c["w2"]), torch.from_numpy(c["w1_s"]), torch.from_numpy(c["w2_s"]),
                torch.from_numpy(c["tw"]), torch.from_numpy(c["ti"]))
        out = _run(a.bfloat16(), *args)
        # The kernel takes 16-bit activations, so the tight comparison is the fp32 oracle on the
        # bf16-rounded input. The stored vector was computed by the reference from the unrounded
        # (fp32) input or entirely in bf16: rounding the input alone flips ~3% of the FP8 codes,
        # hence the loose bound there.
        ref32 = O.fused_experts_fp8(a.bfloat16(), *args, [128, 128], compute_dtype=torch.float32)
        assert O.rel_frobenius(out.float().cpu(), ref32) < TOL, name
        assert O.rel_frobenius(out.float().cpu(), torch.from_numpy(c["out"])) < 5e-2, name


@pytest.mark.parametrize(
    "T,E,topk,H,I", [(1, 8, 2, 256, 128), (33, 8, 2, 512, 256), (64, 8, 2, 1024, 512), (200, 32, 8, 512, 256),
                     (1024, 8, 2, 512, 384), (129, 64, 6, 256, 128)]
)
def test_shapes_vs_fp32_oracle(T, E, topk, H, I):
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, H, generator=g).bfloat16()
    w1, w2, w1_s, w2_s = _weights(E, I, H, 7 + T)
    tw, ti = O.softmax_topk(torch.randn(T, E, generator=g), topk, True)
    ref = O.fused_experts_fp8(x, w1, w2, w1_s, w2_s, tw, ti, [128, 128])
    out = _run(x, w1, w2, w1_s, w2_s, tw, ti)
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (T, H)
    assert O.rel_frobenius(out.float().cpu(), ref) < TOL


@pytest.mark.parametrize("T,E,topk", [(300, 48, 11), (260, 64, 40)])
def test_many_experts_per_token_slot_sum(T, E, topk):
    """More slots per token than one round of the slot sum takes (four loads per thread, 32 ids per ballot), with a
    third of the ids belonging to another rank (-1): the sum visits exactly the valid slots, in order."""
    H, I = 256, 128
    g = torch.Generator().manual_seed(3 * T + topk)
    x = torch.randn(T, H, generator=g).bfloat16()
    w1, w2, w1_s, w2_s = _weights(E, I, H, 11 + topk)
    tw, ti = O.softmax_topk(torch.randn(T, E, generator=g), topk, True)
    ti = torch.where(torch.rand(T, topk, generator=g) < 0.33, torch.full_like(ti, -1), ti)
    ti[0] = -1  # a token none of whose experts is local
    ref = O.fused_experts_fp8(x, w1, w2, w1_s, w2_s, tw, ti, [128, 128])
    out = _run(x, w1, w2, w1_s, w2_s, tw, ti)
    assert O.rel_frobenius(out.float().cpu(), ref) < TOL
    assert float(out[0].float().abs().max()) == 0.0


@pytest.mark.parametrize("T,E,topk,H,I", [(1, 8, 2, 256, 2048), (3, 8, 2, 512, 1024), (5, 16, 4, 256, 1536)])
def test_few_tokens_split_k_down_gemm(T, E, topk, H, I):
    """A handful of tokens: the down GEMM splits K = I over the SMs and the slot reduction sums
    the fp32 partials; with and without the slot reduction, and with ids of other ranks (-1)."""
    g = torch.Generator().manual_seed(100 + T)
    x = torch.randn(T, H, generator=g).bfloat16()
    w1, w2, w1_s, w2_s = _weights(E, I, H, 40 + T)
    tw, ti = O.softmax_topk(torch.randn(T, E, generator=g), topk, True)
    ref = O.fused_experts_fp8(x, w1, w2, w1_s, w2_s, tw, ti, [128, 128])
    out = _run(x, w1, w2, w1_s, w2_s, tw, ti, routed_scaling_factor=1.5)
    assert O.rel_frobenius(out.float().cpu(), ref * 1.5) < TOL
    nc = _run(x, w1, w2, w1_s, w2_s, tw, ti, no_combine=True)
    ref_nc = O.fused_experts_fp8(x, w1, w2, w1_s, w2_s, tw, ti, [128, 128], no_combine=True)
    assert O.rel_frobenius(nc.float().cpu(), ref_nc) < TOL
    local = ti.clone()
    local[:, 0] = -1  # first slot of every token lives on another rank
    part = _run(x, w1, w2, w1_s, w2_s, tw, local)
    ref_part = O.fused_experts_fp8(x, w1, w2, w1_s, w2_s, tw, local, [128, 128])
    assert O.rel_frobenius(part.float().cpu(), ref_part) < TOL
    nc_part = _run(x, w1, w2, w1_s, w2_s, tw, local, no_combine=True)
    assert nc_part[:, 0].abs().max().item() == 0


@pytest.mark.parametrize("T,E,topk,H,I", [(1, 8, 2, 512, 256), (7, 64, 8, 1024, 256), (16, 16, 4, 256, 384), (17, 8, 2, 512, 256),
                                          (32, 256, 8, 512, 128), (40, 8, 2, 256, 1152), (64, 8, 2, 512, 256)])
def test_few_token_path_vs_oracle_and_tile_path(T, E, topk, H, I):
    """The swapped-operand kernels for T <= 64 (token tiles of 16 / 32 / 64, no align or gather pass; opt-in
    with the knob ``moe_decode=1``). Against the oracle, and against the default 128 x 256 tile path on the
    same inputs: both quantise the token rows identically, so they differ only by the intermediate's
    quantisation arithmetic and the summation order."""
    from sglang_b200._native import tuning

    with tuning(moe_decode=1):
        _few_token_case(T, E, topk, H, I, tuning)


def _few_token_case(T, E, topk, H, I, tuning):
    g = torch.Generator().manual_seed(900 + T + E)
    x = torch.randn(T, H, generator=g).bfloat16()
    w1, w2, w1_s, w2_s = _weights(E, I, H, 60 + T)
    tw, ti = O.softmax_topk(torch.randn(T, E, generator=g), topk, True)
    ref = O.fused_experts_fp8(x, w1, w2, w1_s, w2_s, tw, ti, [128, 128])
    out = _run(x, w1, w2, w1_s, w2_s, tw, ti)
    assert O.rel_frobenius(out.float().cpu(), ref) < TOL
    with tuning(moe_decode=0):
        tile = _run(x, w1, w2, w1_s, w2_s, tw, ti)  # the default path
    assert O.rel_frobenius(out.float().cpu(), tile.float().cpu()) < TOL
    # called again: same bits (no state is carried between calls)
    assert torch.equal(_run(x, w1, w2, w1_s, w2_s, tw, ti), out)
    # ids of other ranks, and the un-combined form
    local = ti.clone()
    local[::2, 0] = -1
    part = _run(x, w1, w2, w1_s, w2_s, tw, local)
    assert O.rel_frobenius(part.float().cpu(), O.fused_experts_fp8(x, w1, w2, w1_s, w2_s, tw, local, [128, 128])) < TOL
    nc = _run(x, w1, w2, w1_s, w2_s, tw, ti, no_combine=True)
    assert O.rel_frobenius(nc.float().cpu(), O.fused_experts_fp8(x, w1, w2, w1_s, w2_s, tw, ti, [128, 128], no_combine=True)) < TOL


def test_few_token_path_router_weight_on_input_and_prequantised_rows():
    from sglang_b200._native import tuning

    with tuning(moe_decode=1):
        _few_token_other_inputs()


def _few_token_other_inputs():
    import sglang_b200 as S
    from sglang_b200.fused_moe import fused_experts_impl

    T, E, H, I = 9, 8, 512, 256
    g = torch.Generator().manual_seed(77)
    x = torch.randn(T, H, generator=g).bfloat16()
    w1, w2, w1_s, w2_s = _weights(E, I, H, 78)
    tw, ti = O.softmax_topk(torch.randn(T, E, generator=g), 1, False)
    ref = O.fused_experts_fp8(x, w1, w2, w1_s, w2_s, tw, ti, [128, 128], apply_router_weight_on_input=True)
    out = _run(x, w1, w2, w1_s, w2_s, tw, ti, apply_router_weight_on_input=True)
    assert O.rel_frobenius(out.float().cpu(), ref) < TOL
    # rows that arrive quantised (what an expert-parallel dispatch delivers)
    tw2, ti2 = O.softmax_topk(torch.randn(T, E, generator=g), 2, True)
    q, s = S.per_token_group_quant_fp8(x.cuda(), 128)
    got = fused_experts_impl(q, w1.cuda(), w2.cuda(), tw2.cuda(), ti2.cuda().int(), w1_s.cuda(), w2_s.cuda(), inplace=False,
                             hidden_states_scale=s, output_dtype=torch.bfloat16)
    _status_ok()
    assert O.rel_frobenius(got.float().cpu(), O.fused_experts_fp8(x, w1, w2, w1_s, w2_s, tw2, ti2, [128, 128])) < TOL


def test_expert_parallel_minus_one_ids_sum_to_full_result():
    T, E, topk, H, I = 96, 16, 4, 512, 256
    g = torch.Generator().manual_seed(11)
    x = torch.randn(T, H, generator=g).bfloat16()
    w1, w2, w1_s, w2_s = _weights(E, I, H, 12)
    tw, ti = O.softmax_topk(torch.randn(T, E, generator=g), topk, True)
    ref = O.fused_experts_fp8(x, w1, w2, w1_s, w2_s, tw, ti, [128, 128])
    total = torch.zeros(T, H)
    for r in range(4):
        lo, hi = r * 4, r * 4 + 4
        local = O.ep_local_expert_ids(ti, E, 4, r)
        part = _run(x, w1[lo:hi], w2[lo:hi], w1_s[lo:hi], w2_s[lo:hi], tw, local, num_experts=E, num_local_experts=4)
        ref_part = O.fused_experts_fp8(x, w1[lo:hi], w2[lo:hi], w1_s[lo:hi], w2_s[lo:hi], tw, local, [128, 128])
        assert O.rel_frobenius(part.float().cpu(), ref_part) < TOL
        total += part.float().cpu()
    assert O.rel_frobenius(total, ref) < TOL
    # a rank that owns none of the selected experts returns exact zeros
    none = _run(x, w1[:4], w2[:4], w1_s[:4], w2_s[:4], tw, torch.full_like(ti, -1))
    assert none.abs().max().item() == 0


def test_flags_inplace_no_combine_scaling_weight_on_input():
    import sglang_b200 as S

    T, E, topk, H, I = 50, 8, 2, 256, 128
    g = torch.Generator().manual_seed(21)
    x = torch.randn(T, H, generator=g).bfloat16()
    w1, w2, w1_s, w2_s = _weights(E, I, H, 22)
    tw, ti = O.softmax_topk(torch.randn(T, E, generator=g), topk, True)
    ref = O.fused_experts_fp8(x, w1, w2, w1_s, w2_s, tw, ti, [128, 128])
    out = _run(x, w1, w2, w1_s, w2_s, tw, ti, routed_scaling_factor=2.5)
    assert O.rel_frobenius(out.float().cpu(), ref * 2.5) < TOL
    nc = _run(x, w1, w2, w1_s, w2_s, tw, ti, no_combine=True)
    ref_nc = O.fused_experts_fp8(x, w1, w2, w1_s, w2_s, tw, ti, [128, 128], no_combine=True)
    assert tuple(nc.shape) == (T, topk, H) and O.rel_frobenius(nc.float().cpu(), ref_nc) < TOL
    xd = x.cuda()
    res = S.fused_experts(
        xd, w1.cuda(), w2.cuda(), S.StandardTopKOutput(tw.cuda(), ti.cuda(), None), S.MoeRunnerConfig(),
        use_fp8_w8a8=True, w1_scale=w1_s.cuda(), w2_scale=w2_s.cuda(), block_shape=[128, 128],
    )
    assert res.data_ptr() == xd.data_ptr() and O.rel_frobenius(xd.float().cpu(), ref) < TOL
    tw1, ti1 = O.softmax_topk(torch.randn(T, E, generator=g), 1, False)
    ref1 = O.fused_experts_fp8(x, w1, w2, w1_s, w2_s, tw1, ti1, [128, 128], apply_router_weight_on_input=True)
    out1 = _run(x, w1, w2, w1_s, w2_s, tw1, ti1, apply_router_weight_on_input=True)
    assert O.rel_frobenius(out1.float().cpu(), ref1) < TOL
    with pytest.raises(NotImplementedError):
        S.fused_experts(xd, w1.cuda(), w2.cuda(), S.StandardTopKOutput(tw.cuda(), ti.cuda(), None),
                        S.MoeRunnerConfig(), use_fp8_w8a8=False)


def test_deepseek_routing_skewed_load():
    """256 experts, top-8 grouped sigmoid routing (reduced hidden sizes so the oracle is quick)."""
    T, E, topk, H, I = 300, 256, 8, 512, 256
    g = torch.Generator().manual_seed(31)
    x = torch.randn(T, H, generator=g).bfloat16()
    w1, w2, w1_s, w2_s = _weights(E, I, H, 32)
    tw, ti = O.biased_grouped_topk(torch.randn(T, E, generator=g), torch.zeros(E), topk, 8, 4, True)
    ref = O.fused_experts_fp8(x, w1, w2, w1_s, w2_s, tw, ti, [128, 128])
    out = _run(x, w1, w2, w1_s, w2_s, tw, ti)
    assert O.rel_frobenius(out.float().cpu(), ref) < TOL


@pytest.mark.parametrize("E,T_pad,H,I,counts", [(4, 128, 256, 128, [5, 0, 128, 77]), (8, 256, 512, 256, [0, 1, 129, 256, 17, 0, 200, 64]),
                                               (2, 384, 256, 384, [300, 130])])
def test_masked_layout_experts(E, T_pad, H, I, counts):
    """Low-latency layout [E, T_pad, H] with masked_m valid rows per expert: valid rows vs the fp32
    oracle; rows past masked_m[e] are never written."""
    import sglang_b200 as S

    g = torch.Generator().manual_seed(E * 1000 + T_pad)
    w1, w2, w1_s, w2_s = _weights(E, I, H, 50 + E)
    x = torch.randn(E, T_pad, H, generator=g).bfloat16()
    xq, xs = O.per_token_group_quant_fp8(x.view(-1, H).contiguous(), 128)
    xq, xs = xq.view(E, T_pad, H), xs.view(E, T_pad, H // 128)
    masked_m = torch.tensor(counts, dtype=torch.int32)
    ref = O.masked_experts_fp8(xq, xs, w1, w2, w1_s, w2_s, masked_m)
    out = S.masked_fused_experts(xq.cuda(), xs.cuda(), w1.cuda(), w1_s.cuda(), w2.cuda(), w2_s.cuda(), masked_m.cuda())
    _status_ok()
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (E, T_pad, H)
    for e in range(E):
        m = counts[e]
        if m:
            assert O.rel_frobenius(out[e, :m].float().cpu(), ref[e, :m]) < TOL, e
    # untouched rows: run again into a poisoned buffer through the C ABI's view of `out`
    from sglang_b200 import _native as N
    from sglang_b200.fp8_kernel import _workspace

    lib = N.load()
    poison = torch.full((E, T_pad, H), 7.0, dtype=torch.bfloat16, device="cuda")
    nbytes = lib.b200_masked_experts_fp8_workspace_bytes(E, T_pad, H, I)
    ws = _workspace(poison.device, nbytes)
    args = [t.cuda() for t in (xq, xs, w1, w2, w1_s, w2_s, masked_m)]
    st = lib.b200_masked_experts_fp8(*[N.ptr(t) for t in args], N.ptr(poison), N.BF16, E, T_pad, H, I, N.ptr(ws), nbytes,
                                     N.current_stream())
    N.check(st, "masked_experts")
    torch.cuda.synchronize()
    for e in range(E):
        assert torch.all(poison[e, counts[e]:] == 7.0), e
        assert torch.equal(poison[e, : counts[e]], out[e, : counts[e]])


@pytest.mark.parametrize("name,T,E,topk,H,I", [("mixtral", 8192, 8, 2, 4096, 14336), ("deepseek_v3", 16384, 256, 8, 7168, 2048)])
def test_full_size_layer_properties(name, T, E, topk, H, I):
    """The layers at the sizes the benchmark runs. The whole layer is too big for the CPU oracle,
    so: (a) a token's result does not depend on the other tokens, hence a few sampled rows of the
    full run are compared with the oracle evaluated on those tokens alone; (b) doubling the router weights doubles the output exactly;
    (c) permuting the tokens permutes the output rows."""
    import sglang_b200 as S

    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(77)
    fp8 = torch.float8_e4m3fn
    w1 = torch.empty(E, 2 * I, H, dtype=fp8, device=dev)
    w2 = torch.empty(E, H, I, dtype=fp8, device=dev)
    for e in range(E):  # per expert: bounded temporary memory
        w1[e] = (torch.randn(2 * I, H, device=dev, generator=g) * 60).clamp(-448, 448).to(fp8)
        w2[e] = (torch.randn(H, I, device=dev, generator=g) * 60).clamp(-448, 448).to(fp8)
    w1_s = torch.rand(E, 2 * I // 128, H // 128, device=dev, generator=g) * 2e-4 + 1e-4
    w2_s = torch.rand(E, H // 128, I // 128, device=dev, generator=g) * 2e-4 + 1e-4
    x = torch.randn(T, H, device=dev, generator=g).bfloat16()
    logits = torch.randn(T, E, device=dev, generator=g)
    if name == "deepseek_v3":
        tw, ti = S.biased_grouped_topk(x, logits, torch.zeros(E, device=dev), topk, True, 8, 4)
    else:
        tw, ti = S.fused_topk(x, logits, topk, True)
    cfg = S.MoeRunnerConfig(inplace=False)

    def run(x_, tw_, ti_):
        return S.fused_experts(x_, w1, w2, S.StandardTopKOutput(tw_, ti_, None), cfg, use_fp8_w8a8=True,
                               w1_scale=w1_s, w2_scale=w2_s, block_shape=[128, 128])

    out = run(x, tw, ti)
    _status_ok()
    # the oracle runs on the CPU (on a CUDA tensor torch divides by a Python scalar through its
    # reciprocal, which is not the arithmetic being restated): a few rows, only the experts they use
    rows = torch.randperm(T, device=dev, generator=g)[: (16 if E <= 8 else 6)]
    used = torch.unique(ti[rows].flatten()).long()
    local = torch.searchsorted(used, ti[rows].long()).to(torch.int32)
    ref = O.fused_experts_fp8(x[rows].cpu(), w1[used].cpu(), w2[used].cpu(), w1_s[used].cpu(), w2_s[used].cpu(),
                              tw[rows].cpu(), local.cpu(), [128, 128])
    assert O.rel_frobenius(out[rows].float().cpu(), ref) < TOL
    assert torch.equal(run(x, tw * 2, ti), out * 2)
    perm = torch.randperm(T, device=dev, generator=g)
    assert torch.equal(run(x[perm].contiguous(), tw[perm].contiguous(), ti[perm].contiguous()), out[perm])
