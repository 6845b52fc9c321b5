"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (model SHAPES only; no dataset is involved). Everything random is drawn on
the CPU from ``torch.Generator().manual_seed(seed)`` so that a CPU baseline and the GPU see
identical bits; seed = 1000 * config + index (+ the row / token count)."""
from __future__ import annotations

import math
from typing import Dict, Tuple

import torch

from .weight_quant import block_quant_weight_fp8

LLAMA3_8B_LINEARS: Dict[str, Tuple[int, int]] = {
    "qkv": (6144, 4096),
    "o_proj": (4096, 4096),
    "gate_up": (28672, 4096),
    "down": (4096, 14336),
}
LLAMA3_70B_TP_LINEARS = {
    # name: (N, K, how it is sharded)
    "qkv": (10240, 8192, "column"),
    "gate_up": (57344, 8192, "column"),
    "o_proj": (8192, 8192, "row"),
    "down": (8192, 28672, "row"),
}
MIXTRAL = dict(E=8, topk=2, H=4096, I=14336)
DEEPSEEK_V3 = dict(E=256, topk=8, H=7168, I=2048, n_group=8, topk_group=4)


def activation(M: int, K: int, seed: int, outlier_frac: float = 0.01, dtype=torch.bfloat16) -> torch.Tensor:
    """N(0,1) with a fraction of channels scaled x20."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    if outlier_frac > 0:
        idx = torch.randperm(K, generator=g)[: math.ceil(outlier_frac * K)]
        x[:, idx] *= 20
    return x.to(dtype)


def weight(N: int, K: int, seed: int, device="cpu"):
    """N(0, 0.02^2) bf16 weight drawn on the CPU, block-quantised on ``device``."""
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(N, K, generator=g) * 0.02).bfloat16().to(device)
    return block_quant_weight_fp8(w)


def expert_weights(E: int, I: int, H: int, seed: int, device="cuda", first_expert: int = 0):
    """Per-expert N(0, 0.02^2) weights for experts ``[first_expert, first_expert + E)``.
    Generated on ``device`` from a per-expert seed (the DeepSeek-V3 layer is 11.3 GB of FP8: too
    slow to draw on the host; an expert-parallel rank draws only its own experts), then
    block-quantised."""
    w1 = torch.empty(E, 2 * I, H, dtype=torch.float8_e4m3fn, device=device)
    w2 = torch.empty(E, H, I, dtype=torch.float8_e4m3fn, device=device)
    w1_s = torch.empty(E, 2 * I // 128, H // 128, dtype=torch.float32, device=device)
    w2_s = torch.empty(E, H // 128, I // 128, dtype=torch.float32, device=device)
    g = torch.Generator(device=device)
    for e in range(E):
        g.manual_seed(seed * 100003 + first_expert + e)
        a = (torch.randn(2 * I, H, generator=g, device=device) * 0.02).bfloat16()
        w1[e], w1_s[e] = block_quant_weight_fp8(a)
        b = (torch.randn(H, I, generator=g, device=device) * 0.02).bfloat16()
        w2[e], w2_s[e] = block_quant_weight_fp8(b)
    return w1, w2, w1_s, w2_s


def zipf_router_logits(T: int, E: int, seed: int, exponent: float = 1.2) -> torch.Tensor:
    """N(0,1) logits plus a per-expert bias -exponent*ln(rank): softmax of the bias alone is
    Zipf(exponent) over a seeded permutation of the experts."""
    g = torch.Generator().manual_seed(seed)
    rank = torch.randperm(E, generator=g).float() + 1
    return torch.randn(T, E, generator=g) - exponent * rank.log()
