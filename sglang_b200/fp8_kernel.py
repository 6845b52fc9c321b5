"""Block-FP8 operators with the reference's names, arguments and error behaviour
(python/sglang/srt/layers/quantization/fp8_kernel.py and fp8_utils.py), executed by the
hand-written sm_100a kernels behind the C ABI. CUDA tensors only; no fallback.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from . import _native as N

fp8_dtype = torch.float8_e4m3fn
fp8_max = 448.0
fp8_min = -448.0

# Which of the reference's three quant arithmetic variants is computed (see the C header):
# 0 = torch-native / CUDA-v1 formula (default, the parity oracle), 1 = Triton row-major, 2 = CUDA v2.
_QUANT_FORMULA = 0


def set_quant_formula(mode: int) -> None:
    global _QUANT_FORMULA
    assert mode in (0, 1, 2), "formula mode must be 0, 1 or 2"
    _QUANT_FORMULA = mode


def quant_formula_for(dtype: torch.dtype, eps: float) -> int:
    """Arithmetic variant handed to the C ABI. Variant 0 (``x / (amax / 448)``) is computed for 16-bit
    inputs with the default ``eps`` by variant 3 (rounded reciprocal + one residual step, no per-element
    division): the two give identical bytes and scales on every (x, amax) pair those types can produce,
    which the GPU tests enumerate in full. fp32 inputs and other ``eps`` values keep the division."""
    if _QUANT_FORMULA == 0 and dtype in (torch.bfloat16, torch.float16) and abs(eps - 1e-10) < 1e-16:
        return 3
    return _QUANT_FORMULA


def ceil_align(x: int, a: int) -> int:
    return (x + a - 1) // a * a


def create_per_token_group_quant_fp8_output_scale(
    x_shape,
    device,
    group_size: int,
    column_major_scales: bool,
    scale_tma_aligned: bool,
    scale_ue8m0: bool,
) -> torch.Tensor:
    """Scale buffer in one of the reference's layouts (fp8_kernel.py:454-495): row-major
    ``[..., M, K/g]``; column-major (same shape, strides ``(1, M)``); column-major with the
    M extent of the storage padded to a multiple of 4 ("TMA aligned")."""
    x_shape = tuple(x_shape)
    if scale_ue8m0:
        # packed exponent bytes, four groups per int32, MN-major with the row extent padded to 4
        assert column_major_scales and scale_tma_aligned
        *x_batch, x_q_mn, x_q_k = x_shape
        aligned_mn = ceil_align(x_q_mn, 4)
        aligned_k = ceil_align(x_q_k // group_size, 4)
        return torch.empty(
            (*x_batch, aligned_k // 4, aligned_mn), device=device, dtype=torch.int32
        ).transpose(-1, -2)[..., :x_q_mn, :]
    if column_major_scales:
        if scale_tma_aligned:
            aligned = ceil_align(x_shape[-2], 4)
            return torch.empty(
                x_shape[:-2] + (x_shape[-1] // group_size, aligned), device=device, dtype=torch.float32
            ).transpose(-1, -2)[..., : x_shape[-2], :]
        return torch.empty(
            (x_shape[-1] // group_size,) + x_shape[:-1], device=device, dtype=torch.float32
        ).permute(-1, -2)
    return torch.empty(x_shape[:-1] + (x_shape[-1] // group_size,), device=device, dtype=torch.float32)


def per_token_group_quant_fp8(
    x: torch.Tensor,
    group_size: int,
    eps: float = 1e-10,
    column_major_scales: bool = False,
    scale_tma_aligned: bool = False,
    scale_ue8m0: bool = False,
    fuse_silu_and_mul: bool = False,
    masked_m: Optional[torch.Tensor] = None,
    enable_v2: Optional[bool] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row, per-``group_size`` FP8 E4M3 quantisation; returns ``(x_q, x_s)``.

    Same contract as the reference's ``per_token_group_quant_fp8``
    (fp8_kernel.py:498-565): ``x`` contiguous with last dim divisible by ``group_size``.
    ``enable_v2`` is accepted and ignored (one kernel per scale format here).

    ``scale_ue8m0`` (with ``column_major_scales`` and ``scale_tma_aligned``, as the reference
    requires): power-of-two scales packed as exponent bytes, four groups per int32, MN-major.
    ``fuse_silu_and_mul`` (UE8M0 only, like the reference's kernel): ``x`` is ``[.., 2K]`` =
    gate | up and ``silu(gate) * up`` is quantised. ``masked_m`` (with ``fuse_silu_and_mul``):
    ``x`` is ``[E, T_pad, 2K]`` and only the first ``masked_m[e]`` rows of expert ``e`` are
    processed.
    """
    assert x.shape[-1] % group_size == 0, "the last dimension of `x` cannot be divisible by `group_size`"
    assert x.is_contiguous(), "`x` is not contiguous"
    N.require_cuda(x)
    assert x.dtype in (torch.bfloat16, torch.float16, torch.float32), f"unsupported input dtype {x.dtype}"
    if scale_ue8m0 or fuse_silu_and_mul or masked_m is not None:
        if not scale_ue8m0:
            raise NotImplementedError("fuse_silu_and_mul / masked_m are built for scale_ue8m0=True only")
        if masked_m is not None and not fuse_silu_and_mul:
            raise NotImplementedError("masked_m is built together with fuse_silu_and_mul only")
        return _per_token_group_quant_fp8_ue8m0(x, group_size, eps, column_major_scales, scale_tma_aligned,
                                                fuse_silu_and_mul, masked_m)
    if column_major_scales:
        assert x.dim() == 2, "column-major scales need a 2-D input"
    x_q = torch.empty_like(x, dtype=fp8_dtype)
    x_s = create_per_token_group_quant_fp8_output_scale(
        x.shape, x.device, group_size, column_major_scales, scale_tma_aligned, scale_ue8m0
    )
    K = x.shape[-1]
    M = x.numel() // K if K else 0
    if M > 0:
        if column_major_scales:
            sm, sg = x_s.stride(0), x_s.stride(1)
        else:
            sm, sg = K // group_size, 1
        with N.on_device(x):
            st = N.load().b200_per_token_group_quant_fp8(
                N.ptr(x), N.DTYPE_CODE[x.dtype], N.ptr(x_q), N.ptr(x_s), M, K, group_size, sm, sg, eps,
                quant_formula_for(x.dtype, eps), N.current_stream(),
            )
        N.check(st, "per_token_group_quant_fp8")
    return x_q, x_s


def _per_token_group_quant_fp8_ue8m0(x, group_size, eps, column_major_scales, scale_tma_aligned, fuse_silu_and_mul,
                                     masked_m):
    assert abs(eps - 1e-10) < 1e-13, "the power-of-two kernel floors amax at 1e-10 like the reference's"
    assert (x.shape[-1] // (2 if fuse_silu_and_mul else 1)) % group_size == 0
    out_shape = (*x.shape[:-1], x.shape[-1] // (2 if fuse_silu_and_mul else 1))
    assert len(out_shape) == (3 if masked_m is not None else 2), "2-D input, or [E, T_pad, 2K] with masked_m"
    x_q = torch.empty(out_shape, device=x.device, dtype=fp8_dtype)
    x_s = create_per_token_group_quant_fp8_output_scale(out_shape, x.device, group_size, column_major_scales,
                                                        scale_tma_aligned, True)
    K = out_shape[-1]
    rows = x_q.numel() // K if K else 0
    if rows == 0:
        return x_q, x_s
    experts = out_shape[0] if masked_m is not None else 1
    mm = None
    if masked_m is not None:
        assert masked_m.shape == (experts,)
        mm = masked_m.to(device=x.device, dtype=torch.int32).contiguous()
    with N.on_device(x):
        st = N.load().b200_per_token_group_quant_fp8_ue8m0(
            N.ptr(x), N.DTYPE_CODE[x.dtype], N.ptr(x_q), x_s.data_ptr(), rows, K, group_size, ceil_align(out_shape[-2], 4),
            int(fuse_silu_and_mul), N.ptr(mm), experts, N.current_stream(),
        )
    N.check(st, "per_token_group_quant_fp8 (UE8M0)")
    return x_q, x_s


def sglang_per_token_group_quant_fp8_ue8m0(x: torch.Tensor, group_size: int, eps: float = 1e-10):
    """The reference's shorthand (fp8_kernel.py:568-610): FP8 + packed power-of-two scales."""
    return per_token_group_quant_fp8(x, group_size, eps, column_major_scales=True, scale_tma_aligned=True,
                                     scale_ue8m0=True)


sglang_per_token_group_quant_fp8 = per_token_group_quant_fp8


def prepare_block_fp8_matmul_inputs(
    A: torch.Tensor, B: torch.Tensor, As: torch.Tensor, Bs: torch.Tensor, block_size: List[int],
    output_dtype: torch.dtype,
):
    """Shape / layout checks of the reference (fp8_kernel.py:1135-1180)."""
    assert len(block_size) == 2
    block_n, block_k = block_size
    assert A.shape[-1] == B.shape[-1]
    assert A.shape[:-1] == As.shape[:-1]
    assert A.is_contiguous()
    assert (A.shape[-1] + block_k - 1) // block_k == As.shape[-1]
    M = A.numel() // A.shape[-1]
    assert B.ndim == 2 and B.is_contiguous() and Bs.ndim == 2
    Nn, K = B.shape
    assert (Nn + block_n - 1) // block_n == Bs.shape[0]
    assert (K + block_k - 1) // block_k == Bs.shape[1]
    C = A.new_empty(A.shape[:-1] + (Nn,), dtype=output_dtype)
    return M, Nn, K, C


_workspaces = {}
_retired = []  # superseded buffers that a captured CUDA graph may still address
_capture_seen = False


def _workspace(device, nbytes: int) -> Optional[torch.Tensor]:
    """Grow-only per-(device, stream) scratch buffer for the kernels that need one.

    A CUDA graph bakes the buffer's address into its kernel nodes. Once any call has been made during a
    stream capture, a buffer that has to grow is therefore kept alive (never returned to the allocator)
    instead of being dropped, so replays of an earlier capture keep writing into memory nobody else owns.
    ``reserve_workspace`` sizes the buffer up front."""
    global _capture_seen
    if nbytes == 0:
        return None
    key = (device.index, N.current_stream(device))
    buf = _workspaces.get(key)
    capturing = torch.cuda.is_current_stream_capturing()
    _capture_seen = _capture_seen or capturing
    if buf is None or buf.numel() < nbytes:
        if buf is not None and _capture_seen:
            _retired.append(buf)
        buf = torch.empty(max(nbytes, 0 if buf is None else buf.numel() * 3 // 2), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def reserve_workspace(max_bytes: int, device=None) -> None:
    """Size the scratch buffer of the current stream on ``device`` once, before CUDA graphs are captured on
    it, so that no later call has to grow it (see ``_workspace``)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    _workspace(device, int(max_bytes))


UE8M0_MIN_M = 65  # fewer rows: the decode kernel (weights streamed once) on the unpacked scales


def _matmul_ue8m0(A, B, As, Bs, block_size, output_dtype) -> Optional[torch.Tensor]:
    """Both scale tensors packed power-of-two exponents (``[rows, ceil(K/512)]`` int32, the row index
    contiguous: what ``per_token_group_quant_fp8(scale_ue8m0=True)`` and ``transform_scale_ue8m0`` produce):
    the block-scaled tensor-core kernel, which applies the scales inside the MMA and keeps the accumulator in
    tensor memory for the whole K loop. Returns None when the layout or size is outside that kernel and the
    caller unpacks to fp32 instead (same result up to the fp32 summation order)."""
    if list(block_size) != [128, 128] or A.dim() != 2 or not A.is_cuda or N.get_tuning("gemm_ue8m0") == 0:
        return None
    M, K = A.shape
    Nn = B.shape[0]
    groups = (K + 511) // 512
    if M < UE8M0_MIN_M or K % 16 or Nn % 8 or not (A.is_contiguous() and B.is_contiguous()) or B.shape[1] != K:
        return None
    if A.dtype != fp8_dtype or B.dtype != fp8_dtype or output_dtype not in (torch.bfloat16, torch.float16, torch.float32):
        return None

    def mn_major(s, rows):
        return (s.dim() == 2 and s.shape[0] == rows and s.shape[1] >= groups
                and (s.stride(0) == 1 or rows == 1) and (s.shape[1] == 1 or s.stride(1) >= rows))

    if not mn_major(As, M):
        return None
    if mn_major(Bs, Nn):
        rows_per_word = 1
    elif mn_major(Bs, (Nn + 127) // 128):
        rows_per_word = 128
    else:
        return None
    sfa_ld = As.stride(1) if As.shape[1] > 1 else max(As.shape[0], 1)
    sfb_ld = Bs.stride(1) if Bs.shape[1] > 1 else max(Bs.shape[0], 1)
    C = torch.empty(M, Nn, dtype=output_dtype, device=A.device)
    with N.on_device(A):
        st = N.load().b200_w8a8_block_fp8_gemm_ue8m0(
            N.ptr(A), N.ptr(As), sfa_ld, N.ptr(B), N.ptr(Bs), sfb_ld, rows_per_word, N.ptr(C),
            N.DTYPE_CODE[output_dtype], M, Nn, K, N.current_stream(),
        )
    N.check(st, "w8a8_block_fp8_matmul (UE8M0)")
    return C


def w8a8_block_fp8_matmul(
    A: torch.Tensor,
    B: torch.Tensor,
    As: torch.Tensor,
    Bs: torch.Tensor,
    block_size: List[int],
    output_dtype: torch.dtype = torch.float16,
) -> torch.Tensor:
    """``C = sum_kb (A_kb @ B_kb^T) * As[:, kb] * Bs[n//128, kb]`` on the tcgen05 tensor cores.

    Same contract as the reference (fp8_kernel.py:1285-1300): ``A [.., K]`` and ``B [N, K]``
    FP8 E4M3, contiguous; ``As [.., ceil(K/128)]`` fp32 with any strides (row- or
    column-major); ``Bs [ceil(N/128), ceil(K/128)]`` fp32. Only ``block_size == [128, 128]``.
    """
    if As.dtype == torch.int32 and Bs.dtype == torch.int32:
        C = _matmul_ue8m0(A, B, As, Bs, block_size, output_dtype)
        if C is not None:
            return C
    if As.dtype == torch.int32 or Bs.dtype == torch.int32:
        # power-of-two scales packed as exponent bytes: unpack to fp32 (exact) as the reference does
        # for its Triton path (fp8_utils.py:699-756)
        from .weight_quant import unpack_ue8m0_rows, unpack_ue8m0_scale

        if As.dtype == torch.int32:
            As = unpack_ue8m0_rows(As.reshape(-1, As.shape[-1]), (A.shape[-1] + 127) // 128).reshape(
                *A.shape[:-1], (A.shape[-1] + 127) // 128)
        if Bs.dtype == torch.int32:
            Bs = unpack_ue8m0_scale(Bs, tuple(B.shape), block_size)
    M, Nn, K, C = prepare_block_fp8_matmul_inputs(A, B, As, Bs, block_size, output_dtype)
    if list(block_size) != [128, 128]:
        raise NotImplementedError("only block_size=[128, 128] is built")
    N.require_cuda(A, B, As, Bs)
    assert A.dtype == fp8_dtype and B.dtype == fp8_dtype, "A and B must be float8_e4m3fn"
    assert output_dtype in (torch.bfloat16, torch.float16, torch.float32)
    if M == 0 or Nn == 0:
        return C
    As2 = As.reshape(M, As.shape[-1]) if As.dim() != 2 else As
    if As2.dtype != torch.float32:
        As2 = As2.float()
    Bs = Bs.float().contiguous() if (Bs.dtype != torch.float32 or not Bs.is_contiguous()) else Bs
    lib = N.load()
    ws_bytes = lib.b200_w8a8_block_fp8_gemm_workspace_bytes(M, Nn, K)
    with N.on_device(A):
        ws = _workspace(A.device, ws_bytes)
        st = lib.b200_w8a8_block_fp8_gemm(
            N.ptr(A), N.ptr(As2), As2.stride(0), As2.stride(1), N.ptr(B), N.ptr(Bs), N.ptr(C),
            N.DTYPE_CODE[output_dtype], M, Nn, K, N.ptr(ws), ws_bytes, N.current_stream(),
        )
    N.check(st, "w8a8_block_fp8_matmul")
    return C


def w8a8_block_fp8_linear(
    input: torch.Tensor,
    weight: torch.Tensor,
    block_size: List[int],
    weight_scale: torch.Tensor,
    input_scale: Optional[torch.Tensor] = None,
    bias: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Quantise the activation per 1x128 group, run the block GEMM, add the bias: the
    composition the reference's ``*_w8a8_block_fp8_linear`` wrappers perform
    (fp8_utils.py:814-834). Scales are produced column-major so the GEMM reads one
    contiguous run of 128 row-scales per K block."""
    assert input_scale is None
    input_2d = input.view(-1, input.shape[-1])
    output_shape = [*input.shape[:-1], weight.shape[0]]
    output = _linear_decode_fused(input_2d, weight, block_size, weight_scale)
    if output is None:
        q_input, x_scale = per_token_group_quant_fp8(input_2d, block_size[1], column_major_scales=True)
        output = w8a8_block_fp8_matmul(q_input, weight, x_scale, weight_scale, block_size, output_dtype=input_2d.dtype)
    if bias is not None:
        output += bias
    return output.to(dtype=input_2d.dtype).view(*output_shape)


_tickets = {}
# Rows up to which the one-launch kernel is taken. Measured on B200 (us, one launch / quantiser + GEMM + split-K sum,
# weights rotated so that they come from HBM): 6144x4096 8.8/11.4 at M=1, 12.7/12.1 at M=4, 26.8/12.9 at M=16;
# 4096x4096 6.7/10.8, 9.0/11.0, 16.9/11.6: the in-kernel quantisers pace the weight stream once many rows are live.
DECODE_FUSED_MAX_M = 4


def _linear_decode_fused(x: torch.Tensor, weight: torch.Tensor, block_size, weight_scale: torch.Tensor,
                         max_rows: int = DECODE_FUSED_MAX_M):
    """A few rows (the kernel takes up to 16, this wrapper sends it up to ``DECODE_FUSED_MAX_M``) of 16-bit
    activations: quantiser, GEMM and split-K sum as ONE launch (every CTA
    quantises the slice of ``x`` it needs; same bytes and scales as ``per_token_group_quant_fp8``). Returns
    None when the shapes or dtypes are outside that kernel, and the caller takes the two-step path."""
    M, K = x.shape
    if not (0 < M <= max_rows and x.is_cuda and x.dtype in (torch.bfloat16, torch.float16)
            and list(block_size) == [128, 128] and weight.dtype == fp8_dtype and weight.dim() == 2
            and weight_scale.dtype == torch.float32 and weight_scale.is_contiguous() and x.is_contiguous()
            and weight.is_contiguous() and K % 16 == 0 and weight.shape[0] % 8 == 0 and weight.shape[1] == K):
        return None
    if N.get_tuning("linear_decode_fused") == 0:
        return None
    Nn = weight.shape[0]
    assert tuple(weight_scale.shape) == ((Nn + 127) // 128, (K + 127) // 128)
    lib = N.load()
    out = torch.empty(M, Nn, dtype=x.dtype, device=x.device)
    with N.on_device(x):
        stream = N.current_stream()
        key = (x.device.index, stream)
        tickets = _tickets.get(key)
        if tickets is None:  # zero once; every call leaves them zero
            tickets = _tickets[key] = torch.zeros(4096, dtype=torch.int32, device=x.device)
        ws_bytes = lib.b200_w8a8_block_fp8_linear_decode_workspace_bytes(M, Nn, K)
        ws = _workspace(x.device, ws_bytes)
        st = lib.b200_w8a8_block_fp8_linear_decode(
            N.ptr(x), N.DTYPE_CODE[x.dtype], N.ptr(weight), N.ptr(weight_scale), N.ptr(out), M, Nn, K, 1e-10,
            N.ptr(ws), ws_bytes, N.ptr(tickets), stream,
        )
    N.check(st, "w8a8_block_fp8_linear (decode)")
    return out
