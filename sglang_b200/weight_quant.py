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
    scales = amax / FP8_MAX
    scales = torch.where(scales == 0, torch.ones_like(scales), scales)
    q = (blocks / scales).to(torch.float8_e4m3fn).permute(0, 2, 1, 3).reshape(nb * bn, kb * bk)
    return q[:N, :K].contiguous(), scales.view(nb, kb).contiguous()


def block_dequant_weight(q: torch.Tensor, s: torch.Tensor, block: Sequence[int] = (128, 128)) -> torch.Tensor:
    """Inverse of ``block_quant_weight_fp8`` (fp32 result)."""
    N, K = q.shape[-2:]
    full = s.repeat_interleave(block[0], dim=-2).repeat_interleave(block[1], dim=-1)[..., :N, :K]
    return q.to(torch.float32) * full
