#!/usr/bin/env python
"""Benchmark of the block-FP8 W8A8 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N = 1 and every N): the four Llama-3-8B-shaped block-FP8 linears -- qkv
(6144x4096), o_proj (4096x4096), gate_up (28672x4096), down (4096x14336) -- at M = 8192
rows. One step = per-token-group quantisation + block-FP8 GEMM for each of the four, i.e.
one pass of the quantised-linear hot path over one batch. Inputs are seeded synthetic
tensors (N(0,1) activations with 1% outlier channels x20, N(0, 0.02^2) weights
block-quantised 128x128); there is no dataset. With N > 1 every rank processes its own
batch (no data-path collective: weak scaling); the tensor-/expert-parallel variants are
reported as extra keys.

`value`    TFLOP/s (2*M*N*K summed over the four GEMMs, all ranks) with inputs resident in HBM.
`e2e`      the same metric through the public operators with HOST buffers: pinned host ->
           device copy of the activations and device -> host copy of the outputs inside
           the timed region, every step.
`roofline` the GEMM kernel's achieved TFLOP/s (CUDA events around its launches in the timed
           steps) against 2 x the measured dense bf16 rate (FP8 issues at twice the bf16 rate;
           MEASURED_PEAKS.json holds no FP8 entry).
`cpu_baseline` the oracle's torch-native restatement of the reference path on the host cores,
           on a bounded sample (fewer rows) of the same workload.
`--impl reference` times that CPU path alone.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
if "reference" in sys.argv and os.environ.get("OMP_NUM_THREADS") == "1":
    # torchrun pins OMP_NUM_THREADS=1 for its ranks; the CPU arm is meant to use every host thread
    del os.environ["OMP_NUM_THREADS"]

import torch  # noqa: E402

M_ROWS = 8192
GEMM_TRAFFIC_RATIO = 1.10  # measured DRAM bytes / algorithmic bytes of the GEMM kernel (ncu, see profiles/)
LINEARS = [("qkv", 6144, 4096), ("o_proj", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)]
FLOPS_PER_ROW = sum(2 * n * k for _, n, k in LINEARS)
WORKLOAD = "llama3-8b block-fp8 linears (qkv,o_proj,gate_up,down), M=8192: quant + GEMM each"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """SM clock and throttle reasons sampled every ~5 ms (NVML) while a timed region runs."""

    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index: int):
        self.index, self.sm, self.mask, self.max_sm, self.power = index, [], 0, None, []
        self._stop = threading.Event()
        self.thread = None

    def __enter__(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(vis.split(",")[self.index]) if vis and vis.split(",")[self.index].isdigit() else self.index
            h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)

            def loop():
                while not self._stop.is_set():
                    try:
                        self.sm.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                        self.mask |= pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                        self.power.append(pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0)
                    except Exception:
                        pass
                    time.sleep(0.005)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
        except Exception:
            self.thread = None
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self):
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max_sm,
                "reasons": sorted(n for n, bit in self.REASONS.items() if self.mask & bit), "samples": len(self.sm),
                "power_w_max": max(self.power) if self.power else None, "source": "nvml"}


def build_workload(device, rank: int):
    """Seeded CPU tensors -> pinned host copies + device copies. Seeds: 2000 + index (+ rank)."""
    from sglang_b200 import synthetic

    acts_host, acts_dev, weights = {}, {}, {}
    for i, (name, n, k) in enumerate(LINEARS):
        x = synthetic.activation(M_ROWS, k, 2000 + 10 * i + 100 * rank).pin_memory()
        acts_host[name] = x
        acts_dev[name] = x.to(device, non_blocking=True)
        weights[name] = synthetic.weight(n, k, 2001 + 10 * i, device=device)
    torch.cuda.synchronize()
    return acts_host, acts_dev, weights


def run_step(S, acts, weights, gemm_events=None):
    outs = {}
    for name, n, k in LINEARS:
        wq, ws = weights[name]
        q, s = S.per_token_group_quant_fp8(acts[name], 128, column_major_scales=True)
        if gemm_events is not None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        outs[name] = S.w8a8_block_fp8_matmul(q, wq, s, ws, [128, 128], torch.bfloat16)
        if gemm_events is not None:
            e1.record()
            gemm_events.append((name, e0, e1))
    return outs


def dist_max(value: float, world: int, device) -> float:
    if world == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())


def barrier(world: int):
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()


def cpu_linears(rows: int, threads: int, weights_cpu, acts_cpu):
    """One pass of the four linears through the oracle (torch-native reference restatement)."""
    import oracle as O

    torch.set_num_threads(threads)
    for name, n, k in LINEARS:
        wq, ws = weights_cpu[name]
        O.w8a8_block_fp8_linear(acts_cpu[name][:rows], wq, ws, output_dtype=torch.bfloat16)


def cpu_inputs(rows: int):
    """Same seeds as the GPU workload; weights quantised by the package's quantiser (bit-identical
    to the oracle's, see tests)."""
    from sglang_b200 import synthetic

    acts, weights = {}, {}
    for i, (name, n, k) in enumerate(LINEARS):
        acts[name] = synthetic.activation(rows, k, 2000 + 10 * i)
        weights[name] = synthetic.weight(n, k, 2001 + 10 * i)
    return acts, weights


def time_cpu_baseline(budget_s: float = 15.0):
    """Oracle on the host cores on a bounded row sample sized to ~budget_s of CPU work."""
    threads = os.cpu_count() or 1
    rows = 64
    acts, weights = cpu_inputs(4096)
    t0 = time.perf_counter()
    cpu_linears(rows, threads, weights, acts)
    dt = time.perf_counter() - t0
    # scale the sample towards the budget (the first pass doubles as warm-up)
    rows = int(max(64, min(4096, rows * budget_s / max(dt, 1e-3) / 2)))
    rows = rows // 32 * 32
    t0 = time.perf_counter()
    cpu_linears(rows, threads, weights, acts)
    dt = time.perf_counter() - t0
    return {"value": rows * FLOPS_PER_ROW / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"the four linears on the first {rows} of {M_ROWS} rows, one pass, {dt:.1f} s (torch fp32, oracle/)"}


def run_reference(args, rank: int):
    """The reference's CPU implementation of the path (its torch-native functions, restated in
    oracle/ and pinned to them by the golden vectors) on all host threads."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    acts, weights = cpu_inputs(2048)
    # Size the step from one probe pass: about 1.5 s of host work per step (less when many steps are asked
    # for, so that the whole run stays near two minutes), at least 64 rows. Larger samples amortise the
    # per-call weight dequantisation the way the full 8192-row workload does.
    cpu_linears(64, threads, weights, acts)
    cpu_linears(256, threads, weights, acts)
    t1 = time.perf_counter()
    cpu_linears(256, threads, weights, acts)
    per_256 = time.perf_counter() - t1
    target = min(1.5, 120.0 / max(1, args.steps + args.warmup))
    rows = int(max(64, min(2048, 256 * target / max(per_256, 1e-3)))) // 32 * 32
    for _ in range(args.warmup):
        cpu_linears(rows, threads, weights, acts)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_linears(rows, threads, weights, acts)
    dt = (time.perf_counter() - t0) / args.steps
    v = rows * FLOPS_PER_ROW / dt / 1e12
    sample = f"each step = the four linears on {rows} of {M_ROWS} rows (torch fp32 on {threads} threads)"
    print(json.dumps({
        "impl": "reference", "metric": "block-FP8 GEMM TFLOPS", "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 weights+activations, fp32 accumulate (emulated in fp32 on CPU)",
        "data": "synthetic", "config": {"workload": WORKLOAD, "rows_per_step": rows},
        "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


NVLINK_GBS = 770.0  # measured peer copy per direction per GPU on this pool (nominal 900)


def roofline_frac(ms: float, flops: float, hbm_bytes: float = 0.0, link_bytes: float = 0.0) -> dict:
    """Measured time against max(flops / FP8 peak, HBM bytes / copy rate, NVLink bytes / link rate), per GPU;
    FP8 peak = 2 x the measured sustained dense bf16 rate."""
    peaks = load_peaks()
    terms = {"tensor": flops / (2 * peaks["bf16_sustained"] * 1e12), "hbm": hbm_bytes / (peaks["hbm_gbs"] * 1e9),
             "nvlink": link_bytes / (NVLINK_GBS * 1e9)}
    bound = max(terms, key=terms.get)
    return {"roofline_frac": terms[bound] / (ms * 1e-3), "roofline_bound": bound}


def graph_time_us(fns, rounds: int = 5) -> float:
    """Device time per call, in microseconds: the calls of ``fns`` captured once into a CUDA graph (no host
    launch gaps), median of ``rounds`` replays timed with events on the replaying stream."""
    for fn in fns[:3]:
        fn()
    torch.cuda.synchronize()
    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(side):
        fns[0]()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for fn in fns:
                fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(rounds):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3 / len(fns))
    return sorted(times)[len(times) // 2]


def bench_kernels(S, device):
    """Extra line items for the HBM-bound kernels of the path: achieved GB/s on algorithmic bytes and the fraction
    of the measured copy rate. Inputs exceed L2, or (decode linears) every call of a replay reads another copy of
    the weight so that weights come from HBM as they do in a model with many layers."""
    from sglang_b200.topk import biased_grouped_topk

    hbm = load_peaks()["hbm_gbs"]
    g = torch.Generator(device=device).manual_seed(77)
    fp8 = torch.float8_e4m3fn
    out = {}

    def item(us, nbytes, **extra):
        gbs = nbytes / us / 1e3
        return {"us": us, "GB/s": gbs, "frac_of_measured_hbm": gbs / hbm, **extra}

    M, K = 8192, 14336
    x = torch.randn(M, K, device=device, generator=g).bfloat16()
    us = graph_time_us([lambda: S.per_token_group_quant_fp8(x, 128, column_major_scales=True)] * 4)
    out["per_token_group_quant_fp8_8192x14336_bf16"] = item(us, M * K * 3 + M * (K // 128) * 4)
    del x
    T, E, topk = 16384, 256, 8
    logits = torch.randn(T, E, device=device, generator=g)
    bias = torch.zeros(E, device=device)
    us = graph_time_us([lambda: biased_grouped_topk(logits, logits, bias, topk, True, 8, 4)] * 4)
    out["biased_grouped_topk_16384x256_top8"] = item(us, T * E * 4 + T * topk * 8)
    _, ids = biased_grouped_topk(logits, logits, bias, topk, True, 8, 4)
    us = graph_time_us([lambda: S.moe_align_block_size(ids, 128, E)] * 4)
    max_pad = T * topk + (E + 1) * 127
    out["moe_align_block_size_16384x8_E256"] = item(us, T * topk * 4 + 4 * (max_pad + max_pad // 128 + E + 3))
    for name, n, k in LINEARS:
        copies = max(3, -(-400_000_000 // (n * k)))
        ws = [torch.randn(n, k, device=device, generator=g).to(fp8) for _ in range(copies)]
        wscale = torch.rand(n // 128, k // 128, device=device, generator=g)
        for m in (1, 16):
            xm = torch.randn(m, k, device=device, generator=g).bfloat16()
            fns = [(lambda w=w: S.w8a8_block_fp8_linear(xm, w, [128, 128], wscale)) for w in ws]
            us = graph_time_us(fns)
            out[f"linear_{name}_M{m}"] = item(us, n * k + n * k // 16384 * 4 + m * k * 2 + m * n * 2, N=n, K=k,
                                              weight_copies_rotated=copies)
        del ws
    torch.cuda.empty_cache()
    return out


def bench_moe(S, device, steps: int):
    """Extra line items: fused-MoE tokens/s for the DeepSeek-V3 and Mixtral shaped layers (1 GPU)."""
    from sglang_b200 import synthetic
    from sglang_b200.topk import biased_grouped_topk, fused_topk

    out = {}
    for label, cfg, T in (("deepseek_v3_T16384", synthetic.DEEPSEEK_V3, 16384), ("mixtral_8x7b_T8192", synthetic.MIXTRAL, 8192)):
        E, topk, H, I = cfg["E"], cfg["topk"], cfg["H"], cfg["I"]
        w1, w2, w1_s, w2_s = synthetic.expert_weights(E, I, H, 4000 + E, device=device)
        g = torch.Generator().manual_seed(5000 + T)
        x = torch.randn(T, H, generator=g).bfloat16().to(device)
        if E == 256:
            logits = torch.randn(T, E, generator=g).to(device)
            tw, ti = biased_grouped_topk(x, logits, torch.zeros(E, device=device), topk, True, cfg["n_group"], cfg["topk_group"])
        else:
            logits = synthetic.zipf_router_logits(T, E, 5001).to(device)
            tw, ti = fused_topk(x, logits, topk, True)
        conf = S.MoeRunnerConfig(inplace=False)
        topk_out = S.StandardTopKOutput(tw, ti, None)

        def call():
            return S.fused_experts(x, w1, w2, topk_out, conf, use_fp8_w8a8=True, w1_scale=w1_s, w2_scale=w2_s, block_shape=[128, 128])

        for _ in range(3):
            call()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            call()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        active = int(torch.unique(ti).numel())
        moe_bytes = 4 * T * H + 3 * H * I * active * (1 + 4 / 16384) + 8 * T * topk
        out[label] = {"tokens_per_s": T / ms * 1e3, "ms": ms, "tflops": 6 * T * topk * H * I / ms / 1e9,
                      **roofline_frac(ms, 6 * T * topk * H * I, moe_bytes),
                      "config": {"E": E, "topk": topk, "H": H, "I": I, "T": T, "weights_mb": (w1.numel() + w2.numel()) / 1e6}}
        del w1, w2, w1_s, w2_s
        torch.cuda.empty_cache()
    return out


def bench_parallel(S, device, rank: int, world: int, steps: int):
    """Extra line items at N > 1: Llama-3-70B-shaped tensor-parallel linears (M = 4096; column-parallel
    qkv + gate_up, row-parallel o_proj + down with the bf16 all-reduce) and the DeepSeek-V3-shaped MoE
    layer expert-parallel over the N ranks (T = 16384 tokens in total; "standard" = replicated tokens +
    all-reduce, "a2a" = tokens partitioned + all-to-all dispatch / combine). Device time, max over ranks."""
    from sglang_b200 import parallel as P
    from sglang_b200 import synthetic
    from sglang_b200.topk import biased_grouped_topk

    def timed(fn, n):
        for _ in range(2):
            fn()
        barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier(world)
        return dist_max(e0.elapsed_time(e1) / n, world, device)

    out = {}
    M = 4096
    layers, flops = [], 0
    for i, (name, (n, k, kind)) in enumerate(synthetic.LLAMA3_70B_TP_LINEARS.items()):
        g = torch.Generator(device=device).manual_seed(3000 + i)
        # each rank draws only its own shard (same values as slicing a full tensor would need 0.5 GB per layer on every rank)
        if kind == "column":
            w = (torch.randn(n // world, k, generator=g, device=device) * 0.02).bfloat16()
            x = torch.randn(M, k, generator=g, device=device).bfloat16()
        else:
            w = (torch.randn(n, k // world, generator=g, device=device) * 0.02).bfloat16()
            x = torch.randn(M, k // world, generator=g, device=device).bfloat16()
        wq, ws = synthetic.block_quant_weight_fp8(w)
        layers.append((kind, x, wq, ws))
        flops += 2 * M * n * k
    del w

    from sglang_b200.peer_allreduce import PeerAllReduce

    # row-parallel layers share one set of peer buffers per output width (N = 8192 for both)
    peer = {}
    for kind, x, wq, ws in layers:
        if kind == "row" and wq.shape[0] not in peer:
            peer[wq.shape[0]] = PeerAllReduce(M, wq.shape[0], torch.bfloat16)

    def tp_step(rows: int, fused: bool):
        for kind, x, wq, ws in layers:
            if kind == "row" and fused:
                peer[wq.shape[0]].linear_bf16_input(x[:rows], wq, ws)
                continue
            y = S.w8a8_block_fp8_linear(x[:rows], wq, [128, 128], ws)
            if kind == "row":
                P.tensor_model_parallel_all_reduce(y)

    # prefill-sized (M = 4096) and decode-sized (M = 16) steps, all-reduce by NCCL or fused with the
    # GEMM over peer memory (fan-out epilogue + finishing kernel)
    for rows in (M, 16):
        for fused in (False, True):
            ms = timed(lambda: tp_step(rows, fused), steps)
            key = f"tp_llama70b_M{rows}" + ("_peer_fused" if fused else "")
            # per GPU: 1/world of the flops, its weight shard streamed once, 2 all-reduces of [rows, 8192] bf16
            w_bytes = sum(wq.numel() for _, _, wq, _ in layers)
            out[key] = {"tflops": flops * rows / M / ms / 1e9, "ms": ms, "tp": world,
                        "allreduce": "peer memory, fused with the GEMM" if fused else "nccl",
                        "allreduce_bytes_per_step": 2 * rows * 8192 * 2,
                        **roofline_frac(ms, flops * rows / M / world, w_bytes,
                                        2 * (world - 1) / world * 2 * rows * 8192 * 2)}
    del peer
    # the decode-sized step again, replayed from a CUDA graph (how a server runs decode): the peer
    # path uses device-side epochs and a single slot buffer so that the capture can be replayed
    peer = {n_: PeerAllReduce(16, n_, torch.bfloat16, graph_safe=True)
            for n_ in {wq.shape[0] for kind, _, wq, _ in layers if kind == "row"}}
    for fused in (False, True):
        key = "tp_llama70b_M16_graph" + ("_peer_fused" if fused else "")
        try:
            stream = torch.cuda.Stream()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(stream):
                tp_step(16, fused)
                torch.cuda.synchronize()
                barrier(world)
                with torch.cuda.graph(graph, stream=stream):
                    tp_step(16, fused)
            ms = timed(graph.replay, steps)
            out[key] = {"ms": ms, "tp": world, "allreduce": "peer memory, fused with the GEMM" if fused else "nccl"}
        except Exception as e:  # a capture that fails must not take the other line items with it
            out[key] = {"error": repr(e)}
            torch.cuda.synchronize()
            barrier(world)
    del peer
    del layers
    torch.cuda.empty_cache()

    cfg = synthetic.DEEPSEEK_V3
    E, topk, H, I, T = cfg["E"], cfg["topk"], cfg["H"], cfg["I"], 16384
    el = E // world
    w1, w2, w1_s, w2_s = synthetic.expert_weights(el, I, H, 4000 + E, device=device, first_expert=rank * el)
    g = torch.Generator().manual_seed(5000 + T)
    x = torch.randn(T, H, generator=g).bfloat16().to(device)
    logits = torch.randn(T, E, generator=g).to(device)
    tw, ti = biased_grouped_topk(x, logits, torch.zeros(E, device=device), topk, True, cfg["n_group"], cfg["topk_group"])
    for mode, label in (("ep", "standard"), ("ep_a2a", "a2a"), ("ep_peer", "a2a_peer_memory")):
        layer = P.FusedMoE(w1, w2, w1_s, w2_s, rank, world, mode=mode, presharded=True, num_experts=E,
                           max_tokens=T // world)
        if mode == "ep":
            xs, ws_, is_ = x, tw, ti
        else:
            per = T // world
            sl = slice(rank * per, (rank + 1) * per)
            xs, ws_, is_ = x[sl].contiguous(), tw[sl].contiguous(), ti[sl].contiguous()
        ms = timed(lambda: layer(xs, ws_, is_), max(2, steps // 2))
        # per GPU: 1/world of the flops, its experts' weights once; all-to-all modes move every local token's
        # FP8 row + scales to the other owning ranks and bf16 partial rows back (at most topk_group ranks per token)
        per = T // world
        link = 0.0 if mode == "ep" else per * min(cfg["topk_group"], world) * (world - 1) / world * (H + H // 32 + 2 * H)
        if mode == "ep":
            link = 2 * (world - 1) / world * T * H * 2
        out[f"ep_deepseek_v3_T16384_{label}"] = {"tokens_per_s": T / ms * 1e3, "ms": ms, "ep": world,
                                                 "tflops": 6 * T * topk * H * I / ms / 1e9,
                                                 **roofline_frac(ms, 6 * T * topk * H * I / world,
                                                                 3 * H * I * el * (1 + 4 / 16384), link)}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the MoE / cpu-baseline line items")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (sm_100a); there is no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")  # keep stdout to the one JSON line
        torch.distributed.init_process_group("nccl", device_id=device)
    import sglang_b200 as S
    from sglang_b200 import _native

    peaks = load_peaks()
    acts_host, acts_dev, weights = build_workload(device, rank)

    # ---------------------------------------------------------------- device-resident timing
    for _ in range(args.warmup):
        run_step(S, acts_dev, weights)
    gemm_events = []
    barrier(world)
    with ClockSampler(local_rank) as clocks:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            run_step(S, acts_dev, weights, gemm_events)
        e1.record()
        barrier(world)
    ms_step = dist_max(e0.elapsed_time(e1) / args.steps, world, device)
    status = _native.read_device_status()
    if status != 0:
        raise SystemExit(f"device status word = {status}: a bounded wait timed out; the numbers are void")
    value = world * M_ROWS * FLOPS_PER_ROW / ms_step / 1e9

    per_shape = {}
    for name, a, b in gemm_events:
        per_shape.setdefault(name, []).append(a.elapsed_time(b))
    gemm_ms = sum(statistics.mean(v) for v in per_shape.values())
    gemm_tflops = M_ROWS * FLOPS_PER_ROW / gemm_ms / 1e9
    fp8_peak = 2 * peaks["bf16_sustained"]
    alg_bytes = {n: M_ROWS * kk + nn * kk + 2 * M_ROWS * nn + 4 * (M_ROWS * kk // 128 + nn * kk // 16384) for n, nn, kk in LINEARS}
    roofline = {"bound": "tensor", "achieved": gemm_tflops, "peak": fp8_peak, "unit": "TFLOP/s", "frac": gemm_tflops / fp8_peak,
                "traffic": GEMM_TRAFFIC_RATIO * sum(alg_bytes.values()) / len(alg_bytes), "kernel": "block_fp8_gemm_kernel<256,dense,bf16>",
                "traffic_note": "dram read+write of one ncu capture at 8192x8192x4096 was 1.10 x its algorithmic bytes "
                                "(profiles/block_fp8_gemm_kernel_dense_8192x8192x4096.md); scaled to the mean algorithmic "
                                "bytes of the four launches of a step",
                "algorithmic_bytes_per_launch": sum(alg_bytes.values()) / len(alg_bytes),
                "peak_note": f"2 x {peaks['source']} sustained dense bf16 ({peaks['bf16_sustained']} TF/s); nominal dense FP8 is 4500",
                "frac_of_nominal_fp8": gemm_tflops / 4500.0,
                "per_shape_tflops": {n: 2 * M_ROWS * nn * kk / statistics.mean(per_shape[n]) / 1e9 for n, nn, kk in LINEARS}}

    # ------------------------------------------------------------------ end-to-end (host buffers)
    outs_host = {name: torch.empty(M_ROWS, n, dtype=torch.bfloat16).pin_memory() for name, n, k in LINEARS}
    h2d = sum(x.numel() * x.element_size() for x in acts_host.values())
    d2h = sum(x.numel() * x.element_size() for x in outs_host.values())

    # The copies run on their own streams so that the H2D copy of one linear, the kernels of the
    # previous one and the D2H copy of the one before overlap (both PCIe directions busy at once);
    # every byte still crosses inside the timed region. Device input buffers are double-buffered
    # per linear; an event per buffer says when the kernels have finished reading it.
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    dev_in = {name: [torch.empty_like(acts_dev[name]) for _ in range(2)] for name, _, _ in LINEARS}
    consumed = {name: [None, None] for name, _, _ in LINEARS}
    step_no = [0]

    def e2e_step():
        b = step_no[0] & 1
        step_no[0] += 1
        last = None
        for name, n, k in LINEARS:
            wq, ws = weights[name]
            buf = dev_in[name][b]
            with torch.cuda.stream(s_in):
                if consumed[name][b] is not None:
                    s_in.wait_event(consumed[name][b])
                buf.copy_(acts_host[name], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(s_in)
            main.wait_event(arrived)
            q, sc = S.per_token_group_quant_fp8(buf, 128, column_major_scales=True)
            out = S.w8a8_block_fp8_matmul(q, wq, sc, ws, [128, 128], torch.bfloat16)
            done = torch.cuda.Event()
            done.record(main)
            consumed[name][b] = done
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                outs_host[name].copy_(out, non_blocking=True)
                out.record_stream(s_out)
                last = torch.cuda.Event()
                last.record(s_out)
        return last

    for _ in range(2):
        e2e_step()
    torch.cuda.synchronize()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(3, min(args.steps, 10))
    e0.record()
    for _ in range(e2e_steps):
        last = e2e_step()
    main.wait_event(last)  # the timed region ends when the last result is in host memory
    e1.record()
    barrier(world)
    e2e_ms = dist_max(e0.elapsed_time(e1) / e2e_steps, world, device)
    e2e = {"value": world * M_ROWS * FLOPS_PER_ROW / e2e_ms / 1e9, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps,
           "overlap": "H2D, kernels and D2H of consecutive linears run on three streams; every copy is inside the timed region"}

    line = {
        "metric": "block-FP8 GEMM TFLOPS", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp8_e4m3 x fp8_e4m3 -> fp32 accumulate, bf16 out", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows_per_gpu": M_ROWS, "block_shape": [128, 128],
                   "l2": "per-step working set 1.4 GB (weights 218 MB + activations 436 MB + outputs 705 MB) > 126 MB L2",
                   "parallelism": f"{world} independent replicas" if world > 1 else "single GPU"},
        "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": args.steps * 2 * len(LINEARS), "roofline": roofline,
    }
    del acts_dev, outs_host
    torch.cuda.empty_cache()
    if world > 1 and not args.no_extras:
        try:
            line["parallel"] = bench_parallel(S, device, rank, world, steps=6)
        except Exception as e:  # the headline number stands without the extra line items
            line["parallel"] = {"error": repr(e)}
            barrier(world)
    if rank == 0 and not args.no_extras:
        if world == 1:
            try:
                line["moe"] = bench_moe(S, device, steps=5)
            except Exception as e:  # the headline number stands without the extra line items
                line["moe"] = {"error": repr(e)}
        if world == 1:
            try:
                line["kernels"] = bench_kernels(S, device)
            except Exception as e:  # the headline number stands without the extra line items
                line["kernels"] = {"error": repr(e)}
            line["cpu_baseline"] = time_cpu_baseline()
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
