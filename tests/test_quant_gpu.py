"""per_token_group_quant_fp8 on the GPU vs the oracle and the reference's vectors: bit-exact."""
import pytest
import torch

import oracle as O
from conftest import golden_tensor, load_golden, make_activation

pytestmark = pytest.mark.gpu


def _check(x_cpu, group, **kw):
    import sglang_b200 as S

    q, s = S.per_token_group_quant_fp8(x_cpu.cuda(), group, **kw)
    rq, rs = O.per_token_group_quant_fp8(x_cpu, group)
    assert q.dtype == torch.float8_e4m3fn and s.dtype == torch.float32
    assert tuple(s.shape) == tuple(rs.shape)
    assert torch.equal(q.cpu().view(torch.uint8), rq.view(torch.uint8))
    assert torch.equal(s.cpu(), rs)
    return q, s


def test_reference_vectors_bit_exact():
    import sglang_b200 as S

    for name, c in load_golden("quant.npz").items():
        m, d, g, code = c["meta"].tolist()
        x = golden_tensor(c["x"], code)
        q, s = S.per_token_group_quant_fp8(x.cuda(), g)
        assert torch.equal(q.cpu().view(torch.uint8), torch.from_numpy(c["q"])), name
        assert torch.equal(s.cpu(), torch.from_numpy(c["s"])), name


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("group", [16, 32, 64, 128, 256, 512])
@pytest.mark.parametrize("M,K", [(1, 512), (7, 1024), (83, 4096), (333, 1536)])
def test_shapes_groups_dtypes(M, K, group, dtype):
    _check(make_activation(M, K, 1000 * M + K, dtype), group)


@pytest.mark.parametrize("M", [1, 3, 64, 130])
def test_scale_layouts(M):
    x = make_activation(M, 2048, 7 + M)
    q, s = _check(x, 128, column_major_scales=True)
    assert s.stride() == (1, M)
    q, s = _check(x, 128, column_major_scales=True, scale_tma_aligned=True)
    assert s.stride() == (1, (M + 3) // 4 * 4)


def test_all_zero_group_and_extremes():
    x = torch.zeros(4, 256, dtype=torch.bfloat16)
    x[1, 5] = -3.0
    x[2, 128:] = 1e-20
    x[3, :] = 6e4
    q, s = _check(x, 128)
    assert s[0, 0].item() == (torch.tensor(1e-10) / 448).item()


def test_config1_and_large_row_count():
    _check(make_activation(64, 2048, 1000), 128)
    _check(make_activation(8192, 4096, 2000), 128)


def test_formula_variants():
    import sglang_b200 as S

    x = make_activation(33, 1024, 5)
    try:
        for f in (1, 2):
            S.set_quant_formula(f)
            q, s = S.per_token_group_quant_fp8(x.cuda(), 128)
            rq, rs = O.per_token_group_quant_fp8(x, 128, formula=f)
            assert torch.equal(q.cpu().view(torch.uint8), rq.view(torch.uint8))
            assert torch.equal(s.cpu(), rs)
    finally:
        S.set_quant_formula(0)


def test_empty_and_errors():
    import sglang_b200 as S

    q, s = S.per_token_group_quant_fp8(torch.empty(0, 256, dtype=torch.bfloat16, device="cuda"), 128)
    assert q.shape == (0, 256) and s.shape == (0, 2)
    with pytest.raises(AssertionError):
        S.per_token_group_quant_fp8(torch.zeros(2, 200, dtype=torch.bfloat16, device="cuda"), 128)
    with pytest.raises(AssertionError):
        S.per_token_group_quant_fp8(torch.zeros(4, 256, dtype=torch.bfloat16, device="cuda").t(), 128)
    with pytest.raises(AssertionError):  # power-of-two scales need the column-major TMA-aligned layout, as in the reference
        S.per_token_group_quant_fp8(torch.zeros(2, 256, dtype=torch.bfloat16, device="cuda"), 128, scale_ue8m0=True)
    with pytest.raises(NotImplementedError):  # fused SiLU is built for power-of-two scales only
        S.per_token_group_quant_fp8(torch.zeros(2, 256, dtype=torch.bfloat16, device="cuda"), 128, fuse_silu_and_mul=True)
    with pytest.raises(RuntimeError):
        S.per_token_group_quant_fp8(torch.zeros(2, 256, dtype=torch.bfloat16), 128)


@pytest.mark.parametrize("dtype,max_pattern", [(torch.bfloat16, 0x7F7F), (torch.float16, 0x7BFF)])
def test_corrected_reciprocal_equals_division_for_every_16bit_pair(dtype, max_pattern):
    """Arithmetic variant 3 (reciprocal + one residual step) against variant 0 (IEEE division) on EVERY
    pair (x, amax) a 16-bit input can produce: for each positive finite bit pattern ``a`` taken as the group's
    amax, every value of magnitude <= a with either sign appears in some group whose first element is ``a``.
    Bytes and scales must be identical; this is what allows the wrapper to use variant 3 for 16-bit inputs."""
    from sglang_b200 import _native as N

    lib = N.load()
    code = N.DTYPE_CODE[dtype]
    dev = torch.device("cuda")
    slots = torch.arange(127, device=dev, dtype=torch.int64)[None, :]
    pairs = 0
    step = 2048
    for i0 in range(0, max_pattern + 1, step):
        i_vals = torch.arange(i0, min(i0 + step, max_pattern + 1), device=dev, dtype=torch.int64)
        n_groups = (2 * (i_vals + 1) + 126) // 127
        amax_of_group = torch.repeat_interleave(i_vals, n_groups)
        first = torch.cumsum(n_groups, 0) - n_groups
        local = torch.arange(amax_of_group.numel(), device=dev, dtype=torch.int64) - torch.repeat_interleave(first, n_groups)
        e = local[:, None] * 127 + slots
        cnt = (amax_of_group + 1)[:, None]
        pattern = torch.where(e < cnt, e, torch.where(e < 2 * cnt, 0x8000 | (e - cnt), torch.zeros_like(e)))
        rows = torch.cat([amax_of_group[:, None], pattern], 1)
        del e, pattern
        x = torch.where(rows >= 0x8000, rows - 0x10000, rows).to(torch.int16).view(dtype).contiguous()
        del rows
        M = x.shape[0]
        pairs += int((2 * (i_vals + 1)).sum())
        outs = []
        for formula in (0, 3):
            q = torch.empty(M, 128, dtype=torch.uint8, device=dev)
            s = torch.empty(M, dtype=torch.float32, device=dev)
            st = lib.b200_per_token_group_quant_fp8(N.ptr(x), code, N.ptr(q), N.ptr(s), M, 128, 128, 1, 1, 1e-10, formula,
                                                    N.current_stream())
            N.check(st, "per_token_group_quant_fp8")
            outs.append((q, s))
        assert torch.equal(outs[0][1], outs[1][1])
        same = outs[0][0] == outs[1][0]
        if not bool(same.all()):
            bad = (~same).nonzero()[:5]
            raise AssertionError(f"bytes differ, first (row, col): {bad.tolist()}, amax patterns from {i0}")
        del x, outs
    assert pairs == (max_pattern + 1) * (max_pattern + 2)  # 2 * sum_{i=0..max} (i + 1)
