"""Weight-side data format of the path: FP8 E4M3 weights with one fp32 scale per 128x128
block (``weight`` + ``weight_scale_inv`` of a block-FP8 checkpoint,
python/sglang/srt/layers/quantization/fp8.py:445-494). Offline preparation, not a hot
kernel: plain torch ops on whatever device the weight lives on."""
from __future__ import annotations

from typing import Sequence, Tuple

import torch
import torch.nn.functional as F

FP8_MAX = 448.0


def block_quant_weight_fp8(w: torch.Tensor, block: Sequence[int] = (128, 128)) -> Tuple[torch.Tensor, torch.Tensor]:
    """``[N, K]`` (or ``[E, N, K]``) weight -> (FP8 weight, fp32 scales ``[.., ceil(N/bn), ceil(K/bk)]``)
    with ``scale = amax / 448`` per block (1.0 for an all-zero block) and ``q = w / scale``:
    the arithmetic of the reference's ``convert_weight`` (test/registered/cpu/utils.py:53-101)."""
    if w.dim() == 3:
        qs = [block_quant_weight_fp8(w[e], block) for e in range(w.shape[0])]
        return torch.stack([q for q, _ in qs]), torch.stack([s for _, s in qs])
    N, K = w.shape
    bn, bk = block
    pn, pk = (-N) % bn, (-K) % bk
    wf = w.to(torch.float32)
    if pn or pk:
        wf = F.pad(wf, (0, pk, 0, pn))
    nb, kb = wf.shape[0] // bn, wf.shape[1] // bk
    blocks = wf.view(nb, bn, kb, bk).permute(0, 2, 1, 3)
    amax = blocks.abs().amax(dim=(-2, -1), keepdim=True)
    # tensor / tensor: on a CUDA device torch turns division by a Python scalar into a multiplication by
    # its reciprocal, which rounds differently from the division the reference performs on the CPU
    scales = amax / torch.full_like(amax, FP8_MAX)
    scales = torch.where(scales == 0, torch.ones_like(scales), scales)
    q = (blocks / scales).to(torch.float8_e4m3fn).permute(0, 2, 1, 3).reshape(nb * bn, kb * bk)
    return q[:N, :K].contiguous(), scales.view(nb, kb).contiguous()


def block_dequant_weight(q: torch.Tensor, s: torch.Tensor, block: Sequence[int] = (128, 128)) -> torch.Tensor:
    """Inverse of ``block_quant_weight_fp8`` (fp32 result)."""
    N, K = q.shape[-2:]
    full = s.repeat_interleave(block[0], dim=-2).repeat_interleave(block[1], dim=-1)[..., :N, :K]
    return q.to(torch.float32) * full


# ------------------------------------------------------------------ UE8M0 (power-of-two) scales
# The format DeepGEMM-style consumers on Blackwell take: every scale is 2^e, stored as the biased
# exponent byte, four bytes packed per int32, "MN-major" (the row index is the contiguous one) with
# the row extent padded to a multiple of 4 for TMA. Restated from the reference's torch functions
# (python/sglang/srt/layers/quantization/fp8_utils.py:1186-1410). Load-time work: plain torch ops.


def ceil_align(x: int, a: int) -> int:
    return (x + a - 1) // a * a


def ceil_to_ue8m0(x: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= |x| (fp8_utils.py:1404-1405)."""
    return torch.pow(2.0, torch.ceil(torch.log2(x.abs())))


def per_block_cast_to_fp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``[m, n]`` -> FP8 with one power-of-two scale per 128x128 block: ``amax`` clamped at 1e-4,
    ``sf = ceil_to_ue8m0(amax / 448)``, ``q = x * (1 / sf)`` (fp8_utils.py:1385-1401)."""
    assert x.dim() == 2
    m, n = x.shape
    x_padded = torch.zeros((ceil_align(m, 128), ceil_align(n, 128)), dtype=x.dtype, device=x.device)
    x_padded[:m, :n] = x
    x_view = x_padded.view(-1, 128, x_padded.size(1) // 128, 128)
    x_amax = x_view.abs().float().amax(dim=(1, 3), keepdim=True).clamp(1e-4)
    sf = ceil_to_ue8m0(x_amax / torch.full_like(x_amax, 448.0))  # tensor / tensor: a true division on every device
    x_scaled = (x_view * (1.0 / sf)).to(torch.float8_e4m3fn)
    return x_scaled.view_as(x_padded)[:m, :n].contiguous(), sf.view(x_view.size(0), x_view.size(2))


def quant_weight_ue8m0(weight_dequant: torch.Tensor, weight_block_size=(128, 128)) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 ``[.., n, k]`` -> (FP8 weight, fp32 power-of-two scales ``[.., ceil(n/128), ceil(k/128)]``)
    (fp8_utils.py:1247-1270)."""
    assert list(weight_block_size) == [128, 128] and weight_dequant.dtype == torch.bfloat16
    *batch, n, k = weight_dequant.shape
    w, s = per_block_cast_to_fp8(weight_dequant.view(-1, k))
    return w.view(*batch, n, k), s.view(*batch, ceil_align(n, 128) // 128, ceil_align(k, 128) // 128)


def pack_ue8m0_mn_major(sf: torch.Tensor) -> torch.Tensor:
    """fp32 power-of-two scales ``[.., mn, k]`` -> int32 ``[.., mn, ceil(k/4)]`` with strides
    ``(.., 1, align(mn, 4))``: exponent bytes, four consecutive k per int32, zero padded
    (the torch statement of DeepGEMM's layout helper, fp8_utils.py:1306-1334)."""
    assert sf.dtype == torch.float32 and sf.dim() in (2, 3)
    squeeze = sf.dim() == 2
    if squeeze:
        sf = sf.unsqueeze(0)
    b, mn, k = sf.shape
    ue8m0 = (sf.contiguous().view(torch.int32) >> 23).to(torch.uint8)
    aligned_mn, aligned_k = ceil_align(mn, 4), ceil_align(k, 4)
    padded = torch.zeros((b, aligned_mn, aligned_k), device=sf.device, dtype=torch.uint8)
    padded[:, :mn, :k] = ue8m0
    packed = padded.view(-1).view(torch.int32).view(b, aligned_mn, aligned_k // 4)
    transposed = torch.zeros((b, aligned_k // 4, aligned_mn), device=sf.device, dtype=torch.int32).mT
    transposed[:, :, :] = packed
    out = transposed[:, :mn, :]
    return out.squeeze(0) if squeeze else out


def transform_scale_ue8m0(sf: torch.Tensor, mn: int) -> torch.Tensor:
    """Per-block weight scales ``[.., ceil(mn/128), k]`` -> one row per weight row (each block row
    repeated 128 times), packed as ``pack_ue8m0_mn_major`` (fp8_utils.py:1278-1303)."""
    sf = sf.index_select(-2, torch.arange(mn, device=sf.device) // 128)
    return pack_ue8m0_mn_major(sf)


def unpack_ue8m0_scale(sf_packed: torch.Tensor, weight_shape, block_size=(128, 128)) -> torch.Tensor:
    """Packed int32 scales ``[N or ceil(N/128), ceil(k/4)]`` -> fp32 ``[ceil(N/128), ceil(K/128)]``,
    what the fp32-scale GEMM takes (fp8_utils.py:699-756)."""
    assert sf_packed.dtype == torch.int32 and sf_packed.dim() == 2
    N, K = weight_shape
    bn, bk = block_size
    n_groups, k_groups = (N + bn - 1) // bn, (K + bk - 1) // bk
    rows, k_div_4 = sf_packed.shape
    dense = torch.empty((rows, k_div_4), dtype=torch.int32, device=sf_packed.device).copy_(sf_packed)
    u8 = dense.view(torch.uint8).view(rows, k_div_4 * 4)
    f = (u8.to(torch.int32) << 23).view(torch.float32)
    if rows == N and N != n_groups:
        f = f.index_select(0, torch.arange(0, N, bn, device=sf_packed.device))
    elif rows != n_groups:
        raise ValueError(f"unexpected packed scale shape {tuple(sf_packed.shape)} for weight {tuple(weight_shape)}")
    return f[:, :k_groups].contiguous()


def unpack_ue8m0_rows(sf_packed: torch.Tensor, k_groups: int) -> torch.Tensor:
    """Packed int32 activation scales ``[M, ceil(k/4)]`` (any strides) -> fp32 ``[M, k_groups]``."""
    assert sf_packed.dtype == torch.int32 and sf_packed.dim() == 2
    rows, k_div_4 = sf_packed.shape
    dense = torch.empty((rows, k_div_4), dtype=torch.int32, device=sf_packed.device).copy_(sf_packed)
    u8 = dense.view(torch.uint8).view(rows, k_div_4 * 4)
    return (u8.to(torch.int32) << 23).view(torch.float32)[:, :k_groups].contiguous()


def requant_weight_ue8m0(weight: torch.Tensor, weight_scale_inv: torch.Tensor, weight_block_size=(128, 128)):
    """A block-FP8 weight with fp32 scales -> the same weight re-quantised with power-of-two
    scales, scales packed for MN-major consumers (fp8_utils.py:1221-1244): dequantise to bf16,
    ``quant_weight_ue8m0``, ``transform_scale_ue8m0``."""
    assert list(weight_block_size) == [128, 128]
    dequant = block_dequant_weight(weight, weight_scale_inv, weight_block_size).to(torch.bfloat16)
    out_w, out_s = quant_weight_ue8m0(dequant, weight_block_size)
    return out_w, transform_scale_ue8m0(out_s, mn=out_w.shape[-2])
