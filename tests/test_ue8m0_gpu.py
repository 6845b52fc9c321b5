"""Power-of-two (UE8M0) scales: activation quantiser with packed MN-major scales (plain, fused
SiLU*mul, masked layout) vs the oracle's restatement of the reference kernel's arithmetic, the
packing vs the reference's torch layout function (golden), and the GEMM on packed scales."""
import pytest
import torch

import oracle as O
from conftest import load_golden, make_activation

pytestmark = pytest.mark.gpu


def _status_ok():
    from sglang_b200 import _native

    assert _native.read_device_status() == 0, "a bounded device-side wait timed out"


def _exp_bytes(packed, k_groups):
    """int32 [.., mn, ceil(k/4)] (any strides) -> uint8 exponent bytes [.., mn, k_groups]."""
    p = torch.empty(packed.shape, dtype=packed.dtype).copy_(packed)  # dense row-major copy whatever the strides
    return p.view(torch.uint8).view(*p.shape[:-1], p.shape[-1] * 4)[..., :k_groups]


@pytest.mark.parametrize("M,K,g", [(1, 128, 128), (7, 512, 128), (83, 1024, 128), (130, 640, 128), (33, 384, 64), (5, 7168, 128)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_quant_ue8m0_bytes_scales_and_packing(M, K, g, dtype):
    import sglang_b200 as S

    x = make_activation(M, K, M + K, dtype=dtype)
    x[0, :g] = 0  # an all-zero group: amax floors at 1e-10
    if M > 2:
        x[2, :g] = torch.tensor(448.0 * 4).to(dtype)  # amax/448 an exact power of two: no round-up
    q, s = S.per_token_group_quant_fp8(x.cuda(), g, column_major_scales=True, scale_tma_aligned=True, scale_ue8m0=True)
    oq, osf = O.per_token_group_quant_fp8_ue8m0(x, g)
    assert s.dtype == torch.int32 and tuple(s.shape) == (M, (K // g + 3) // 4)
    assert s.stride() == (1, (M + 3) // 4 * 4)
    assert torch.equal(q.cpu().view(torch.uint8), oq.view(torch.uint8))
    ref_packed = O.pack_ue8m0_mn_major(osf)
    assert torch.equal(s.cpu(), ref_packed) and s.stride() == ref_packed.stride()
    q2, s2 = S.fp8_kernel.sglang_per_token_group_quant_fp8_ue8m0(x.cuda(), g)
    assert torch.equal(q2.view(torch.uint8), q.view(torch.uint8)) and torch.equal(s2, s)


def test_packing_matches_reference_layout_vectors():
    from sglang_b200 import weight_quant as W

    c = load_golden("ue8m0.npz")["w"]
    w = torch.from_numpy(c["w"]).view(torch.bfloat16)
    q, s = W.quant_weight_ue8m0(w)
    assert torch.equal(q.view(torch.uint8), torch.from_numpy(c["q"])) and torch.equal(s, torch.from_numpy(c["s"]))
    packed = W.transform_scale_ue8m0(s, mn=w.shape[0])
    assert torch.equal(packed.contiguous(), torch.from_numpy(c["packed"]))
    assert torch.equal(W.unpack_ue8m0_scale(packed.contiguous(), tuple(w.shape)), s)
    q0 = torch.from_numpy(c["q0"]).view(torch.float8_e4m3fn)
    rq, rs = W.requant_weight_ue8m0(q0, torch.from_numpy(c["s0"]))
    assert torch.equal(rq.view(torch.uint8), torch.from_numpy(c["requant_q"]))
    assert torch.equal(W.unpack_ue8m0_scale(rs.contiguous(), tuple(w.shape)), torch.from_numpy(c["requant_s"]))


@pytest.mark.parametrize("M,K", [(9, 256), (64, 2048), (130, 384)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fused_silu_and_mul_ue8m0(M, K, dtype):
    import sglang_b200 as S

    g = torch.Generator().manual_seed(M + K)
    x = (torch.randn(M, 2 * K, generator=g) * 2).to(dtype)
    q, s = S.per_token_group_quant_fp8(x.cuda(), 128, column_major_scales=True, scale_tma_aligned=True,
                                       scale_ue8m0=True, fuse_silu_and_mul=True)
    oq, osf = O.per_token_group_quant_fp8_ue8m0(x, 128, fuse_silu_and_mul=True)
    assert tuple(q.shape) == (M, K)
    # silu is evaluated with different exp implementations: after rounding to 16 bits a handful of
    # values differ by one step; scales (group maxima) and nearly all codes are identical
    assert torch.equal(_exp_bytes(s.cpu(), K // 128), _exp_bytes(O.pack_ue8m0_mn_major(osf), K // 128))
    mismatch = (q.cpu().view(torch.uint8) != oq.view(torch.uint8)).float().mean().item()
    assert mismatch < 2e-3, mismatch
    deq = q.cpu().float() * osf.repeat_interleave(128, dim=-1)
    ref = (torch.nn.functional.silu(x[:, :K].float()) * x[:, K:].float())
    assert O.rel_frobenius(deq, ref) < 4e-2  # FP8 quantisation noise


def test_masked_layout_fused_silu_ue8m0():
    import sglang_b200 as S

    E, T_pad, K = 4, 24, 256
    counts = torch.tensor([5, 0, 24, 13], dtype=torch.int32)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(E, T_pad, 2 * K, generator=g).bfloat16()
    q, s = S.per_token_group_quant_fp8(x.cuda(), 128, column_major_scales=True, scale_tma_aligned=True,
                                       scale_ue8m0=True, fuse_silu_and_mul=True, masked_m=counts.cuda())
    assert tuple(q.shape) == (E, T_pad, K) and tuple(s.shape) == (E, T_pad, 1) and s.stride() == (T_pad, 1, T_pad)
    for e in range(E):
        m = int(counts[e])
        if m == 0:
            continue
        oq, osf = O.per_token_group_quant_fp8_ue8m0(x[e, :m].contiguous(), 128, fuse_silu_and_mul=True)
        mismatch = (q[e, :m].cpu().view(torch.uint8) != oq.view(torch.uint8)).float().mean().item()
        assert mismatch < 2e-3
        assert torch.equal(_exp_bytes(s[e, :m].cpu(), 2), (osf.view(torch.int32) >> 23).to(torch.uint8))


def _ue8m0_case(M, N, K, seed):
    import sglang_b200 as S
    from sglang_b200 import weight_quant as W

    x = make_activation(M, K, seed)
    g = torch.Generator().manual_seed(seed + 1)
    w = (torch.randn(N, K, generator=g) * 0.02).bfloat16()
    wq, ws = W.quant_weight_ue8m0(w)
    xq, xs_packed = S.per_token_group_quant_fp8(x.cuda(), 128, column_major_scales=True, scale_tma_aligned=True,
                                                scale_ue8m0=True)
    oq, osf = O.per_token_group_quant_fp8_ue8m0(x, 128)
    ref = O.w8a8_block_fp8_matmul(oq, wq, osf, ws, [128, 128], output_dtype=torch.float32)
    return xq, xs_packed, wq, ws, osf, ref


def test_gemm_on_packed_power_of_two_scales():
    """Weights re-quantised to power-of-two scales + UE8M0 activation quant, packed scales handed to the GEMM:
    the block-scaled tensor-core kernel (scales applied inside the MMA, accumulator in tensor memory for the
    whole K loop). Close to the fp32 oracle, and equal up to the fp32 summation order to the promotion kernel on
    the unpacked scales, which is also what the knob ``gemm_ue8m0=0`` selects for packed scales."""
    import sglang_b200 as S
    from sglang_b200 import weight_quant as W
    from sglang_b200._native import tuning

    M, N, K = 200, 384, 640
    xq, xs_packed, wq, ws, osf, ref = _ue8m0_case(M, N, K, 5)
    ws_packed = W.transform_scale_ue8m0(ws, mn=N)
    out = S.w8a8_block_fp8_matmul(xq, wq.cuda(), xs_packed, ws_packed.cuda(), [128, 128], torch.bfloat16)
    _status_ok()
    assert O.rel_frobenius(out.float().cpu(), ref) < 5e-3
    plain = S.w8a8_block_fp8_matmul(xq, wq.cuda(), osf.cuda(), ws.cuda(), [128, 128], torch.bfloat16)
    assert float((out.float() - plain.float()).norm() / plain.float().norm()) < 2e-3
    with tuning(gemm_ue8m0=0):
        unpacked = S.w8a8_block_fp8_matmul(xq, wq.cuda(), xs_packed, ws_packed.cuda(), [128, 128], torch.bfloat16)
    assert torch.equal(unpacked, plain)


@pytest.mark.parametrize("M,N,K", [(128, 224, 128), (130, 448, 512), (300, 1024, 640), (1024, 4096, 2048),
                                   (257, 232, 4096 + 128), (4096, 7168, 2048), (65, 8, 128)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_block_scaled_kernel_shapes(M, N, K, out_dtype):
    """The block-scaled kernel on ragged and multi-tile shapes (tiles are 128 x 224; scales refresh every four
    K blocks; two accumulator stages), fp32 output held to 1e-4 of the oracle: every product and scale is exact
    and only the summation order differs."""
    import sglang_b200 as S
    from sglang_b200 import weight_quant as W

    xq, xs_packed, wq, ws, osf, ref = _ue8m0_case(M, N, K, 11 + M + N)
    per_row = W.transform_scale_ue8m0(ws, mn=N).cuda()
    out = S.w8a8_block_fp8_matmul(xq, wq.cuda(), xs_packed, per_row, [128, 128], out_dtype)
    _status_ok()
    assert out.dtype == out_dtype and tuple(out.shape) == (M, N)
    assert O.rel_frobenius(out.float().cpu(), ref) < (1e-4 if out_dtype == torch.float32 else 5e-3)
    # one scale word per 128-row block of the weight instead of one per row: same result
    per_block = W.pack_ue8m0_mn_major(ws).cuda()
    out2 = S.w8a8_block_fp8_matmul(xq, wq.cuda(), xs_packed, per_block, [128, 128], out_dtype)
    _status_ok()
    assert torch.equal(out2, out)
