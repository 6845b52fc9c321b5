"""Small fixed workloads for profiling one kernel at a time (the commands quoted in ``profiles/``).

    python -m sglang_b200.profile_cases gemm M N K [calls]
    python -m sglang_b200.profile_cases gemm_ue8m0 M N K [calls]          (packed power-of-two scales: block-scaled kernel)
    python -m sglang_b200.profile_cases linear_decode M N K [calls]       (one-launch quantise + GEMM + split-K sum)
    python -m sglang_b200.profile_cases quant M K [calls]
    python -m sglang_b200.profile_cases align T topk E [calls]
    python -m sglang_b200.profile_cases route T E topk grouped|softmax [calls]
    python -m sglang_b200.profile_cases moe deepseek|mixtral T [calls]
    python -m sglang_b200.profile_cases allreduce_finish M N [calls]      (single rank: handshake with itself)

Inputs are seeded synthetic tensors created on the device; every case prints one checksum so the
run has an observable result. Meant to be run as is, and again under ``ncu`` with a kernel filter.
"""
from __future__ import annotations

import ctypes
import sys

import torch


def main(argv) -> int:
    import sglang_b200 as S
    from sglang_b200 import _native as N
    from sglang_b200 import synthetic

    case, args = argv[0], argv[1:]
    dev = "cuda"
    fp8 = torch.float8_e4m3fn
    g = torch.Generator(device=dev).manual_seed(1234)

    def calls(i, default=3):
        return int(args[i]) if len(args) > i else default

    if case == "gemm":
        M, Nn, K = (int(a) for a in args[:3])
        A = torch.randn(M, K, device=dev, generator=g).to(fp8)
        B = torch.randn(Nn, K, device=dev, generator=g).to(fp8)
        As = torch.rand((K + 127) // 128, M, device=dev, generator=g).t()
        Bs = torch.rand((Nn + 127) // 128, (K + 127) // 128, device=dev, generator=g)
        for _ in range(calls(3)):
            out = S.w8a8_block_fp8_matmul(A, B, As, Bs, [128, 128], torch.bfloat16)
    elif case == "gemm_ue8m0":
        from sglang_b200 import weight_quant

        M, Nn, K = (int(a) for a in args[:3])
        x = torch.randn(M, K, device=dev, generator=g).bfloat16()
        w = (torch.randn(Nn, K, device=dev, generator=g) * 0.05).bfloat16()
        A, As = S.per_token_group_quant_fp8(x, 128, column_major_scales=True, scale_tma_aligned=True, scale_ue8m0=True)
        B, Bs_f = weight_quant.quant_weight_ue8m0(w)
        Bs = weight_quant.transform_scale_ue8m0(Bs_f, mn=Nn)
        del x, w
        for _ in range(calls(3)):
            out = S.w8a8_block_fp8_matmul(A, B, As, Bs, [128, 128], torch.bfloat16)
    elif case == "linear_decode":
        from sglang_b200 import fp8_kernel

        M, Nn, K = (int(a) for a in args[:3])
        x = torch.randn(M, K, device=dev, generator=g).bfloat16()
        B = torch.randn(Nn, K, device=dev, generator=g).to(fp8)
        Bs = torch.rand((Nn + 127) // 128, (K + 127) // 128, device=dev, generator=g) * 1e-2
        for _ in range(calls(3)):
            out = fp8_kernel._linear_decode_fused(x, B, [128, 128], Bs, max_rows=16)
            assert out is not None, "shape outside the one-launch kernel"
    elif case == "quant":
        M, K = (int(a) for a in args[:2])
        x = torch.randn(M, K, device=dev, generator=g).bfloat16()
        for _ in range(calls(2)):
            out, _ = S.per_token_group_quant_fp8(x, 128, column_major_scales=True)
        out = out.view(torch.uint8)
    elif case == "align":
        T, topk, E = (int(a) for a in args[:3])
        ids = torch.randint(0, E, (T, topk), device=dev, generator=g, dtype=torch.int32)
        for _ in range(calls(3)):
            out = S.moe_align_block_size(ids, 128, E)[0]
    elif case == "route":
        T, E, topk = (int(a) for a in args[:3])
        grouped = args[3] == "grouped"
        x = torch.randn(T, E, device=dev, generator=g)
        bias = torch.zeros(E, device=dev)
        for _ in range(calls(4)):
            if grouped:
                out, _ = S.biased_grouped_topk(x, x, bias, topk, True, 8, 4)
            else:
                out, _ = S.fused_topk(x, x, topk, True)
    elif case == "moe":
        cfg = synthetic.DEEPSEEK_V3 if args[0] == "deepseek" else synthetic.MIXTRAL
        T = int(args[1])
        E, topk, H, I = cfg["E"], cfg["topk"], cfg["H"], cfg["I"]
        w1 = torch.randn(E, 2 * I, H, device=dev, dtype=torch.bfloat16).to(fp8)
        w2 = torch.randn(E, H, I, device=dev, dtype=torch.bfloat16).to(fp8)
        w1s = torch.rand(E, 2 * I // 128, H // 128, device=dev, generator=g) * 1e-3
        w2s = torch.rand(E, H // 128, I // 128, device=dev, generator=g) * 1e-3
        x = torch.randn(T, H, device=dev, generator=g).bfloat16()
        logits = torch.randn(T, E, device=dev, generator=g)
        if args[0] == "deepseek":
            tw, ti = S.biased_grouped_topk(x, logits, torch.zeros(E, device=dev), topk, True, 8, 4)
        else:
            tw, ti = S.fused_topk(x, logits, topk, True)
        conf = S.MoeRunnerConfig(inplace=False)
        for _ in range(calls(2, 2)):
            out = S.fused_experts(x, w1, w2, S.StandardTopKOutput(tw, ti, None), conf, use_fp8_w8a8=True,
                                  w1_scale=w1s, w2_scale=w2s, block_shape=[128, 128])
    elif case == "allreduce_finish":
        M, Nn = (int(a) for a in args[:2])
        lib = N.load()
        slot = torch.randn(M, Nn, device=dev, generator=g).bfloat16()
        resid = torch.randn(M, Nn, device=dev, generator=g).bfloat16()
        gamma = torch.ones(Nn, device=dev).bfloat16()
        out = torch.empty_like(slot)
        res_out = torch.empty_like(slot)
        flags = torch.zeros(64, dtype=torch.int32, device=dev)
        outs = (ctypes.c_void_p * 1)(out.data_ptr())
        res_outs = (ctypes.c_void_p * 1)(res_out.data_ptr())
        peers = (ctypes.c_void_p * 1)(flags.data_ptr())
        for i in range(calls(2)):
            N.check(lib.b200_allreduce_finish(slot.data_ptr(), M * Nn, outs, N.BF16, M, Nn, 1, 0, 0, resid.data_ptr(),
                                              res_outs, gamma.data_ptr(), 1e-6, flags.data_ptr(), peers, i + 1, None,
                                              None, N.current_stream()), "allreduce_finish")
    else:
        print(__doc__)
        return 2
    torch.cuda.synchronize()
    print(case, *args, "checksum", float(out.float().abs().mean()), "device status", N.read_device_status())
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
