"""Torch-native (CPU) restatement of the reference's block-FP8 algorithms.

TEST INFRASTRUCTURE ONLY -- see ``oracle/__init__.py``.

Each function names the reference source it restates (paths are relative to
the reference project root):

* ``per_token_group_quant_fp8``  <- ``native_per_token_group_quant_fp8``
  (test/manual/quant/test_block_fp8.py:41-66) with the CUDA kernels' fp32
  ``eps`` (sgl-kernel/csrc/gemm/per_token_group_quant_8bit.cu:45,79-86,110).
* ``block_quant_weight_fp8``     <- ``convert_weight``
  (test/registered/cpu/utils.py:53-101).
* ``w8a8_block_fp8_matmul``      <- ``native_w8a8_block_fp8_matmul``
  (test/manual/quant/test_block_fp8.py:291-340).
* ``moe_align_block_size``       <- ``moe_align_block_size_kernel`` +
  ``count_and_sort_expert_tokens_kernel``
  (sgl-kernel/csrc/moe/moe_align_kernel.cu:27-41,55-233) and the output sizing
  of python/sglang/srt/layers/moe/moe_runner/triton_utils/moe_align_block_size.py:58-87,
  with the stable (ascending flat index) order of the small-batch kernel
  (moe_align_kernel.cu:309-314).
* ``silu_and_mul``               <- ``SiluAndMul.forward_native``
  (python/sglang/srt/layers/activation.py:86-88).
* ``fused_experts_fp8``          <- ``torch_w8a8_block_fp8_moe``
  (test/manual/quant/test_block_fp8.py:518-547), taking ``topk_weights`` /
  ``topk_ids`` as inputs instead of its internal softmax-top-k, skipping ids
  outside ``[0, E)`` (the expert-parallel "-1" convention of
  python/sglang/srt/layers/moe/token_dispatcher/standard.py:172-210).
* ``softmax_topk``               <- ``fused_topk_torch_native``
  (python/sglang/srt/layers/moe/topk.py:550-588).
* ``biased_grouped_topk``        <- ``biased_grouped_topk_impl``
  (python/sglang/srt/layers/moe/topk.py:923-992).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

FP8 = torch.float8_e4m3fn
FP8_MAX = 448.0
FP8_MIN = -448.0

__all__ = [
    "FP8",
    "FP8_MAX",
    "per_token_group_quant_fp8",
    "block_quant_weight_fp8",
    "w8a8_block_fp8_matmul",
    "w8a8_block_fp8_linear",
    "moe_align_sizes",
    "moe_align_block_size",
    "silu_and_mul",
    "fused_experts_fp8",
    "masked_experts_fp8",
    "ceil_pow2",
    "quant_weight_ue8m0",
    "pack_ue8m0_mn_major",
    "per_token_group_quant_fp8_ue8m0",
    "softmax_topk",
    "softmax_topk_capped",
    "biased_grouped_topk",
    "sigmoid_topk",
    "grouped_topk",
    "fused_shared_experts_tail",
    "canonical_routing",
    "ep_local_expert_ids",
    "rel_frobenius",
]


# --------------------------------------------------------------------------- quant
def per_token_group_quant_fp8(
    x: torch.Tensor, group_size: int, eps: float = 1e-10, formula: int = 0
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row, per-``group_size`` FP8 E4M3 quantisation with fp32 scales.

    ``formula`` selects which of the reference's three arithmetic variants is
    reproduced (all share ``amax = max(|x|, eps)`` over the group, in fp32):

    * 0: ``s = amax / 448``; ``q = x / s``        (torch-native oracle, CUDA v1)
    * 1: ``s = amax / 448``; ``q = x * (1 / s)``  (Triton row-major kernel,
         python/sglang/srt/layers/quantization/fp8_kernel.py:180-183)
    * 2: ``s = amax * (1/448)``; ``q = x * (448 / amax)`` (CUDA v2,
         sgl-kernel/csrc/gemm/per_token_group_quant_8bit_v2.cu:69-80)

    Differences from ``native_per_token_group_quant_fp8``: ``eps`` is applied
    after the upcast to fp32 (as every CUDA kernel of the reference does), which
    only matters for an all-zero group.
    """
    assert x.shape[-1] % group_size == 0
    assert x.is_contiguous()
    xf = x.reshape(-1, group_size).to(torch.float32)
    amax = xf.abs().amax(dim=-1, keepdim=True).clamp(min=eps)
    if formula == 0:
        s = amax / FP8_MAX
        q = xf / s
    elif formula == 1:
        s = amax / FP8_MAX
        q = xf * (torch.ones_like(s) / s)
    elif formula == 2:
        s = amax * torch.tensor(1.0 / 448.0, dtype=torch.float32, device=amax.device)
        # tensor / tensor: one IEEE division, as `MAX / amax` in the kernel (a Python scalar
        # divided by a tensor would be reciprocal-then-multiply, i.e. rounded twice)
        q = xf * (torch.full_like(amax, FP8_MAX) / amax)
    else:
        raise ValueError(f"unknown formula {formula}")
    q = q.clamp(min=FP8_MIN, max=FP8_MAX).to(FP8).reshape(x.shape)
    s = s.reshape(x.shape[:-1] + (x.shape[-1] // group_size,))
    return q, s


def block_quant_weight_fp8(
    w: torch.Tensor, block: Sequence[int] = (128, 128)
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantise a ``[N, K]`` weight to FP8 with one fp32 scale per ``block``.

    ``scale = amax / 448`` (1.0 where a block is all zero), ``q = w / scale``.
    """
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
    q = (blocks / scales).to(FP8).permute(0, 2, 1, 3).reshape(nb * bn, kb * bk)
    return q[:N, :K].contiguous(), scales.view(nb, kb).contiguous()


# ---------------------------------------------------------------------------- GEMM
def w8a8_block_fp8_matmul(
    A: torch.Tensor,
    B: torch.Tensor,
    As: torch.Tensor,
    Bs: torch.Tensor,
    block_size: Sequence[int],
    output_dtype: torch.dtype = torch.float16,
) -> torch.Tensor:
    """``C = sum_kb (A_kb @ B_kb^T) * As[:, kb] * Bs[n // bn, kb]``, fp32 accumulate."""
    A = A.to(torch.float32)
    B = B.to(torch.float32)
    bn, bk = block_size
    assert A.shape[-1] == B.shape[-1] and B.ndim == 2 and Bs.ndim == 2
    K = A.shape[-1]
    M = A.numel() // K
    N = B.shape[0]
    nt, kt = (N + bn - 1) // bn, (K + bk - 1) // bk
    assert As.shape[-1] == kt and tuple(Bs.shape) == (nt, kt)
    out_shape = A.shape[:-1] + (N,)
    A = A.reshape(M, K)
    As = As.reshape(M, kt).to(torch.float32)
    C = torch.zeros(M, N, dtype=torch.float32, device=A.device)
    for i in range(kt):
        a = A[:, i * bk : min((i + 1) * bk, K)]
        for j in range(nt):
            b = B[j * bn : min((j + 1) * bn, N), i * bk : min((i + 1) * bk, K)]
            s = As[:, i : i + 1] * Bs[j, i]
            C[:, j * bn : min((j + 1) * bn, N)] += torch.matmul(a, b.t()) * s
    return C.reshape(out_shape).to(output_dtype)


def w8a8_block_fp8_linear(x, wq, ws, block_size=(128, 128), bias=None, output_dtype=None):
    """quant(1 x block_k) -> block GEMM -> optional bias; the composition of
    ``triton_w8a8_block_fp8_linear`` (python/sglang/srt/layers/quantization/fp8_utils.py:814-834)."""
    output_dtype = output_dtype or x.dtype
    x2 = x.reshape(-1, x.shape[-1]).contiguous()
    q, s = per_token_group_quant_fp8(x2, block_size[1])
    out = w8a8_block_fp8_matmul(q, wq, s, ws, block_size, output_dtype=torch.float32)
    if bias is not None:
        out = out + bias.to(torch.float32)
    return out.to(output_dtype).reshape(x.shape[:-1] + (wq.shape[0],))


# --------------------------------------------------------------------------- align
def moe_align_sizes(numel: int, block_size: int, num_experts: int) -> Tuple[int, int]:
    """(max_num_tokens_padded, max_num_m_blocks) exactly as the reference sizes its outputs."""
    if numel < num_experts + 1:
        max_pad = numel * block_size
    else:
        max_pad = numel + (num_experts + 1) * (block_size - 1)
    return max_pad, (max_pad + block_size - 1) // block_size


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int):
    """Bucket flat ``topk_ids`` by expert (ids in ``[-1, E)``; bucket 0 is "-1"),
    pad every bucket to a multiple of ``block_size`` and emit, in bucket order, the
    flat indices (ascending inside a bucket, ``numel`` in pad slots).

    Returns ``(sorted_ids[max_pad], expert_ids[max_blocks], num_post_pad[1], cumsum[E+2])``.
    ``expert_ids`` past the last real block is -1; ``cumsum[b]`` is the END of
    bucket ``b``'s real (unpadded) entries, which is the state the reference's
    scatter kernel leaves behind; ``cumsum[E+1]`` is the padded total.
    """
    flat = topk_ids.reshape(-1).to(torch.int64)
    numel = flat.numel()
    nb = num_experts + 1
    max_pad, max_blocks = moe_align_sizes(numel, block_size, num_experts)
    sorted_ids = torch.full((max_pad,), numel, dtype=torch.int32)
    expert_ids = torch.full((max_blocks,), -1, dtype=torch.int32)
    cumsum = torch.zeros(nb + 1, dtype=torch.int32)
    bucket = flat + 1
    valid = (bucket >= 0) & (bucket < nb)
    counts = torch.bincount(bucket[valid], minlength=nb)
    padded = (counts + block_size - 1) // block_size * block_size
    starts = torch.cumsum(padded, 0) - padded
    total = int(padded.sum())
    order = torch.argsort(bucket, stable=True)
    order = order[valid[order]]
    pos_in_bucket = torch.arange(order.numel()) - (torch.cumsum(counts, 0) - counts)[bucket[order]]
    sorted_ids[(starts[bucket[order]] + pos_in_bucket)] = order.to(torch.int32)
    for b in range(nb):
        lo, hi = int(starts[b]) // block_size, int(starts[b] + padded[b]) // block_size
        expert_ids[lo:hi] = b - 1
    cumsum[:nb] = (starts + counts).to(torch.int32)
    cumsum[nb] = total
    return sorted_ids, expert_ids, torch.tensor([total], dtype=torch.int32), cumsum


# ----------------------------------------------------------------------------- MoE
def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1] // 2
    return F.silu(x[..., :d]) * x[..., d:]


def fused_experts_fp8(
    a: torch.Tensor,
    w1: torch.Tensor,
    w2: torch.Tensor,
    w1_s: torch.Tensor,
    w2_s: torch.Tensor,
    topk_weights: torch.Tensor,
    topk_ids: torch.Tensor,
    block_shape: Sequence[int] = (128, 128),
    compute_dtype: torch.dtype = torch.float32,
    routed_scaling_factor: Optional[float] = None,
    no_combine: bool = False,
    apply_router_weight_on_input: bool = False,
) -> torch.Tensor:
    """Block-FP8 W8A8 MoE: for every (token, slot) pair run expert ``ids[t, j]``'s
    gate_up GEMM -> SiLU*mul -> re-quant -> down GEMM, weight and sum over slots.

    ``compute_dtype`` is the dtype activations are carried in between the
    kernels (fp32 = the "computed in fp32" oracle)."""
    T, D = a.shape
    topk = topk_ids.shape[1]
    E = w1.shape[0]
    bk = block_shape[1]
    a = a.to(compute_dtype)
    if apply_router_weight_on_input:
        assert topk == 1
    a_rep = a.view(T, 1, D).repeat(1, topk, 1).reshape(-1, D)
    out = torch.zeros(T * topk, w2.shape[1], dtype=compute_dtype, device=a.device)
    ids = topk_ids.reshape(-1)
    a_q, a_s = per_token_group_quant_fp8(a_rep.contiguous(), bk)
    a_q = a_q.to(torch.float32)
    for e in range(E):
        mask = ids == e
        if mask.sum():
            inter = w8a8_block_fp8_matmul(a_q[mask], w1[e], a_s[mask], w1_s[e], block_shape, output_dtype=compute_dtype)
            if apply_router_weight_on_input:
                # the reference's first grouped GEMM multiplies its fp32 accumulator by the router
                # weight (fused_moe_triton_kernels.py:602-604 with mul_routed_weight set for GEMM 1)
                inter = inter * topk_weights.reshape(-1)[mask].view(-1, 1).to(inter.dtype)
            act = silu_and_mul(inter)
            act_q, act_s = per_token_group_quant_fp8(act.contiguous(), bk)
            out[mask] = w8a8_block_fp8_matmul(act_q, w2[e], act_s, w2_s[e], block_shape, output_dtype=compute_dtype)
    out = out.view(T, topk, -1)
    if not apply_router_weight_on_input:
        out = out * topk_weights.view(T, topk, 1).to(out.dtype)
    if no_combine:
        return out
    out = out.sum(dim=1)
    if routed_scaling_factor is not None:
        out = out * routed_scaling_factor
    return out


# ------------------------------------------------------------------------------ UE8M0
def ceil_pow2(x: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= x for positive fp32 x, computed on the bits (no log2 rounding):
    what ``ceil_to_ue8m0`` = ``2 ** ceil(log2(x))`` means
    (python/sglang/srt/layers/quantization/fp8_utils.py:1404-1405)."""
    bits = x.to(torch.float32).contiguous().view(torch.int32)
    exp = (bits >> 23) & 0xFF
    exp = exp + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    return (exp << 23).view(torch.float32)


def quant_weight_ue8m0(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 ``[n, k]`` -> FP8 + one power-of-two fp32 scale per 128x128 block: amax clamped at
    1e-4, ``sf = ceil_pow2(amax / 448)``, ``q = w * (1 / sf)`` with the multiply in bf16
    (fp8_utils.py:1247-1270, 1385-1401)."""
    assert w.dim() == 2 and w.dtype == torch.bfloat16
    n, k = w.shape
    nb, kb = (n + 127) // 128, (k + 127) // 128
    q = torch.zeros(nb * 128, kb * 128, dtype=FP8)
    sf = torch.empty(nb, kb, dtype=torch.float32)
    wp = torch.zeros(nb * 128, kb * 128, dtype=torch.bfloat16)
    wp[:n, :k] = w
    for i in range(nb):
        for j in range(kb):
            blk = wp[i * 128 : i * 128 + 128, j * 128 : j * 128 + 128]
            amax = blk.abs().float().amax().clamp(min=1e-4)
            s = ceil_pow2((amax / FP8_MAX).reshape(1))[0]
            sf[i, j] = s
            # bf16 tensor times fp32 0-dim tensor stays bf16 in torch: one rounding to bf16, then FP8
            q[i * 128 : i * 128 + 128, j * 128 : j * 128 + 128] = (blk * (1.0 / s)).to(FP8)
    return q[:n, :k].contiguous(), sf


def pack_ue8m0_mn_major(sf: torch.Tensor) -> torch.Tensor:
    """fp32 power-of-two scales ``[mn, k]`` -> int32 ``[mn, ceil(k/4)]`` with strides
    ``(1, align(mn, 4))``: byte ``j`` of word ``[r, c]`` is the exponent byte of ``sf[r, 4c + j]``
    (zero past k) (fp8_utils.py:1306-1334)."""
    mn, k = sf.shape
    amn, kw = (mn + 3) // 4 * 4, (k + 3) // 4
    exp = ((sf.contiguous().view(torch.int32) >> 23) & 0xFF).to(torch.int64)
    words = torch.zeros(kw, amn, dtype=torch.int64)
    for c in range(k):
        words[c // 4, :mn] |= exp[:, c] << (8 * (c % 4))
    words = torch.where(words >= 2**31, words - 2**32, words).to(torch.int32)
    return words.t()[:mn, :]


def per_token_group_quant_fp8_ue8m0(x: torch.Tensor, group_size: int = 128, fuse_silu_and_mul: bool = False):
    """Activation quantisation with power-of-two scales as the reference's CUDA kernel computes it
    (sgl-kernel/csrc/gemm/per_token_group_quant_8bit_v2.cu:56-80, 343-395): ``amax`` floored at
    1e-10, ``e = ceil(log2(amax * (1/448)))`` on the bits, ``q = x * 2**-e``; returns the FP8
    tensor and the fp32 scales ``2**e`` ``[.., K/g]`` (pack with ``pack_ue8m0_mn_major``).
    ``fuse_silu_and_mul``: ``x`` is ``[.., 2K]`` = gate | up and the quantised value is
    ``T(silu(gate)) * up`` in the input dtype ``T``. PARITY UNPINNED for this flag: on sm_100 the
    reference evaluates silu with the hardware ``tanh.approx``; here it is the exact fp32 silu."""
    if fuse_silu_and_mul:
        k = x.shape[-1] // 2
        gate, up = x[..., :k], x[..., k:]
        act = (gate.float() * torch.sigmoid(gate.float())).to(x.dtype)
        x = (act.float() * up.float()).to(x.dtype)  # the product of two 16-bit values is exact in fp32
    xf = x.reshape(-1, group_size).to(torch.float32)
    amax = xf.abs().amax(dim=-1, keepdim=True).clamp(min=1e-10)
    sf = ceil_pow2(amax * torch.tensor(1.0 / 448.0, dtype=torch.float32))
    q = (xf * (torch.ones_like(sf) / sf)).clamp(min=FP8_MIN, max=FP8_MAX).to(FP8).reshape(x.shape)
    return q, sf.reshape(x.shape[:-1] + (x.shape[-1] // group_size,))


def masked_experts_fp8(hidden_q, hidden_s, w1, w2, w1_s, w2_s, masked_m, block_shape=(128, 128)):
    """Experts over the masked layout (python/sglang/srt/layers/moe/moe_runner/deep_gemm.py:362-494):
    for every expert ``e`` and row ``t < masked_m[e]``: gate_up GEMM -> SiLU*mul -> 1x128 re-quant
    -> down GEMM, in fp32. Rows past ``masked_m[e]`` are returned as NaN (unspecified)."""
    E, T_pad, H = hidden_q.shape
    out = torch.full((E, T_pad, w2.shape[1]), float("nan"), dtype=torch.float32)
    for e in range(E):
        m = int(masked_m[e])
        if m == 0:
            continue
        inter = w8a8_block_fp8_matmul(hidden_q[e, :m].to(torch.float32), w1[e], hidden_s[e, :m], w1_s[e], block_shape,
                                      output_dtype=torch.float32)
        act_q, act_s = per_token_group_quant_fp8(silu_and_mul(inter).contiguous(), block_shape[1])
        out[e, :m] = w8a8_block_fp8_matmul(act_q, w2[e], act_s, w2_s[e], block_shape, output_dtype=torch.float32)
    return out


# ------------------------------------------------------------------------- routing
def _topk(x: torch.Tensor, k: int):
    """``torch.topk`` with the tie rule pinned: equal values go to the lower index (what the
    reference's CUDA kernels do, sgl-kernel/csrc/moe/moe_topk_softmax_kernels.cu:545-546;
    ``torch.topk`` itself leaves ties unspecified). Results in descending order."""
    v, i = torch.sort(x, dim=-1, descending=True, stable=True)
    return v[..., :k], i[..., :k]


def softmax_topk(logits: torch.Tensor, topk: int, renormalize: bool = True):
    w = logits.float().softmax(dim=-1)
    w, ids = _topk(w, topk)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return w, ids.to(torch.int32)


def biased_grouped_topk(
    logits: torch.Tensor,
    correction_bias: torch.Tensor,
    topk: int,
    num_expert_group: int,
    topk_group: int,
    renormalize: bool = True,
    routed_scaling_factor: Optional[float] = None,
):
    """Sigmoid scores; group score = sum of the top-2 biased scores of the group;
    keep ``topk_group`` groups; top-k experts among them; weights are the unbiased
    scores, renormalised."""
    scores = logits.float().sigmoid()
    T, E = scores.shape
    sfc = scores + correction_bias.float().unsqueeze(0)
    group_scores = sfc.view(T, num_expert_group, -1).topk(2, dim=-1)[0].sum(dim=-1)
    group_idx = _topk(group_scores, topk_group)[1]
    group_mask = torch.zeros_like(group_scores)
    group_mask.scatter_(1, group_idx, 1)
    score_mask = group_mask.unsqueeze(-1).expand(T, num_expert_group, E // num_expert_group).reshape(T, -1)
    tmp = sfc.masked_fill(~score_mask.bool(), float("-inf"))
    ids = _topk(tmp, topk)[1]
    w = scores.gather(1, ids)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    if routed_scaling_factor is not None:
        w = w * routed_scaling_factor
    return w.to(torch.float32), ids.to(torch.int32)


def sigmoid_topk(logits: torch.Tensor, topk: int, renormalize: bool = True,
                 correction_bias: Optional[torch.Tensor] = None):
    """Sigmoid scores, selection on ``scores + correction_bias``, weights are the unbiased
    scores (python/sglang/srt/layers/moe/topk.py:550-588 with scoring_func="sigmoid")."""
    scores = logits.float().sigmoid()
    if correction_bias is not None:
        ids = _topk(scores + correction_bias.float().unsqueeze(0), topk)[1]
        w = scores.gather(1, ids)
    else:
        w, ids = _topk(scores, topk)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return w.to(torch.float32), ids.to(torch.int32)


def grouped_topk(logits: torch.Tensor, topk: int, num_expert_group: int, topk_group: int,
                 renormalize: bool = True):
    """Softmax scores; a group's score is its maximum; experts outside the ``topk_group`` best
    groups are zeroed; top-k of what is left (python/sglang/srt/layers/moe/topk.py:703-764)."""
    scores = torch.softmax(logits.float(), dim=-1)
    T, E = scores.shape
    group_scores = scores.view(T, num_expert_group, -1).max(dim=-1).values
    group_idx = _topk(group_scores, topk_group)[1]
    group_mask = torch.zeros_like(group_scores)
    group_mask.scatter_(1, group_idx, 1)
    score_mask = group_mask.unsqueeze(-1).expand(T, num_expert_group, E // num_expert_group).reshape(T, -1)
    tmp = scores.masked_fill(~score_mask.bool(), 0.0)
    w, ids = _topk(tmp, topk)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return w.to(torch.float32), ids.to(torch.int32)


def fused_shared_experts_tail(raw_w: torch.Tensor, ids: torch.Tensor, renormalize: bool,
                              routed_scaling_factor: Optional[float], apply_routed_scaling_factor_on_output: bool):
    """Weights of the grouped routing functions when shared experts are fused into the routed ones
    (python/sglang/srt/layers/moe/topk.py:735-764 and :968-992): ``raw_w`` / ``ids`` are the un-normalised top-k
    in descending order. The last slot goes to a shared-expert replica (its id is drawn at random by the
    reference, so only the routed ids ``ids[:, :-1]`` are comparable) with weight ``sum(routed) /
    routed_scaling_factor``; renormalisation divides by the sum of the routed slots."""
    w = raw_w.clone().float()
    if routed_scaling_factor is not None:
        w[:, -1] = w[:, :-1].sum(dim=-1) / routed_scaling_factor
    if renormalize:
        w = w / w[:, :-1].sum(dim=-1, keepdim=True)
        if apply_routed_scaling_factor_on_output:
            w = w * routed_scaling_factor
    return w.to(torch.float32), ids[:, :-1].to(torch.int32)


def canonical_routing(w: torch.Tensor, ids: torch.Tensor):
    """Rows reordered by expert id: the reference leaves the order of the k results unspecified
    (``sorted=False``), so two correct routings are compared in this form."""
    order = torch.argsort(ids.long(), dim=-1, stable=True)
    return w.gather(1, order), ids.gather(1, order)


def ep_local_expert_ids(topk_ids: torch.Tensor, num_experts: int, ep_size: int, ep_rank: int):
    """Expert-parallel id remap: rank ``r`` owns experts ``[r*E/p, (r+1)*E/p)``; local ids are
    rebased to 0, everything else becomes -1
    (python/sglang/srt/layers/moe/token_dispatcher/standard.py:172-210)."""
    per = num_experts // ep_size
    lo = ep_rank * per
    local = topk_ids - lo
    return torch.where((topk_ids >= lo) & (topk_ids < lo + per), local, torch.full_like(topk_ids, -1))


def rel_frobenius(x: torch.Tensor, ref: torch.Tensor) -> float:
    x = x.to(torch.float64)
    ref = ref.to(torch.float64)
    return float((x - ref).norm() / ref.norm().clamp(min=1e-30))


def softmax_topk_capped(logits: torch.Tensor, topk: int, renormalize: bool, softcap: float = 0.0,
                        logit_bias: torch.Tensor = None):
    """Softmax top-k over transformed logits, the arithmetic of the reference's ``topk_softmax`` kernel with
    ``moe_softcapping`` / ``correction_bias`` (sgl-kernel/csrc/moe/moe_topk_softmax_kernels.cu:101-130):
    ``v = tanh(x / cap) * cap`` when ``cap != 0``, ``v += bias``, ``scores = softmax(v)``, top-k of the scores
    (lower index wins ties), weights optionally divided by their sum. fp32 throughout. Parity unpinned: the
    reference's tests (sgl-kernel/tests/test_moe_topk_softmax.py) never pass these two arguments, so this follows
    the kernel text only; with both arguments off it equals ``softmax_topk``, which is pinned."""
    v = logits.float()
    if softcap != 0.0:
        v = torch.tanh(v / torch.tensor(softcap, dtype=torch.float32)) * torch.tensor(softcap, dtype=torch.float32)
    if logit_bias is not None:
        v = v + logit_bias.float().unsqueeze(0)
    scores = torch.softmax(v, dim=-1)
    w, ids = _topk(scores, topk)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return w, ids.to(torch.int32)
