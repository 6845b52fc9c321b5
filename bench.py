#!/usr/bin/env python
"""Benchmark of the block-FP8 W8A8 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload (every N): the four Llama-3-70B-shaped block-FP8 linears at M = 4096 rows --
column-parallel qkv (10240x8192) and gate_up (57344x8192), row-parallel o_proj (8192x8192) and
down (8192x28672) -- partitioned over the N ranks as a tensor-parallel group (N = 1: un-sharded).
One pass = per-token-group quantisation + block-FP8 GEMM for each of the four; on N > 1 the
row-parallel layers end in the bf16 all-reduce, fused with the GEMM over NVLink peer memory.
The total work is fixed as N grows (strong scaling). One *step* is ``inner_repeats`` passes,
chosen so that the timed region lasts about two seconds (a sustained, power-capped number rather
than a burst); the repeat count is printed in ``config``.

Every timed item is checked first: sampled rows and columns of its output are compared with the
CPU oracle of the un-sharded layer (relative Frobenius error <= 1e-2) and the device status word
must be clear; an item that fails is reported as failed, not timed.

`value`    TFLOP/s (2*M*N*K summed over the four GEMMs of the un-sharded layers) with inputs
           resident in HBM; device time, max over ranks.
`e2e`      the same metric through the public operators with HOST buffers: pinned host -> device
           copies of the activations and device -> host copies of the outputs inside the timed
           region, every pass.
`roofline` the GEMM kernel's achieved TFLOP/s per GPU (CUDA events around its launches in the
           timed steps) against an FP8 tensor peak measured in this process (torch._scaled_mm,
           per-tensor scales, 8192^3: burst and seconds-long sustained); the fractions of
           2 x the bf16 rates of MEASURED_PEAKS.json and of the nominal 4.5 PFLOP/s are printed too.
`comparators` (N = 1) the same block-scaled GEMM through FlashInfer's CUTLASS sm100 kernel and
           vLLM's CUTLASS sm100 kernel, when those libraries load.
`cpu_baseline` the oracle's torch-native restatement of the reference path on the host cores,
           on a bounded sample (fewer rows) of the same workload.
`--impl reference` times that CPU path alone.
"""
from __future__ import annotations

import argparse
import json
import math
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

M_ROWS = 4096
TOL = 1e-2
CHUNKS = 8  # every layer is defined as 8 seeded chunks along its sharded dimension, whatever N is
# name: (N, K, how it is sharded)
TP_LINEARS = [("qkv", 10240, 8192, "column"), ("gate_up", 57344, 8192, "column"),
              ("o_proj", 8192, 8192, "row"), ("down", 8192, 28672, "row")]
LLAMA8B_LINEARS = [("qkv", 6144, 4096), ("o_proj", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)]
FLOPS_PER_ROW = sum(2 * n * k for _, n, k, _ in TP_LINEARS)
WORKLOAD = ("llama3-70b block-fp8 linears (qkv, gate_up column-parallel; o_proj, down row-parallel + all-reduce), "
            "M=4096, TP = number of GPUs: quant + GEMM each")
NVLINK_GBS = 770.0  # measured peer copy per direction per GPU on this pool (nominal 900)
NOMINAL_FP8 = 4500.0


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16=p["bf16_tflops"],
                    bf16_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """SM clock, power and throttle reasons sampled every ~5 ms (NVML) while a timed region runs."""

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


# ------------------------------------------------------------------------------ plumbing


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


def agree(flag: bool, world: int, device) -> bool:
    """Rank 0's verdict, on every rank (so that all ranks take the same branch)."""
    if world == 1:
        return flag
    t = torch.tensor([1 if flag else 0], dtype=torch.int32, device=device)
    torch.distributed.broadcast(t, src=0)
    return bool(t.item())


def device_status_clear(world: int, device) -> bool:
    """True when no rank's device status word reports an expired wait."""
    from sglang_b200 import _native

    torch.cuda.synchronize()
    return dist_max(float(_native.read_device_status()), world, device) == 0.0


def timed(fn, n: int, world: int, device, warm: int = 2) -> float:
    """Device milliseconds per call of ``fn``, max over ranks. The ranks meet at a barrier first: the
    peer-memory handshakes inside ``fn`` wait two seconds at most for a rank that is still busy."""
    barrier(world)
    for _ in range(warm):
        fn()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    barrier(world)
    return dist_max(e0.elapsed_time(e1) / n, world, device)


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


def roofline_frac(ms: float, flops: float, hbm_bytes: float = 0.0, link_bytes: float = 0.0, fp8_peak=None) -> dict:
    """Measured time against max(flops / FP8 peak, HBM bytes / copy rate, NVLink bytes / link rate), per GPU."""
    peaks = load_peaks()
    fp8 = fp8_peak or 2 * peaks["bf16_sustained"]
    terms = {"tensor": flops / (fp8 * 1e12), "hbm": hbm_bytes / (peaks["hbm_gbs"] * 1e9),
             "nvlink": link_bytes / (NVLINK_GBS * 1e9)}
    bound = max(terms, key=terms.get)
    return {"roofline_frac": terms[bound] / (ms * 1e-3), "roofline_bound": bound}


# ------------------------------------------------------------------- measured FP8 tensor peak


def measure_fp8_peak(device, local_rank: int, sustain_s: float = 2.0) -> dict:
    """Dense FP8 rate of the library GEMM on this GPU: torch._scaled_mm (cuBLASLt), E4M3 x E4M3 -> bf16,
    per-tensor scales, 8192^3. ``burst`` = best of 10 single launches, ``sustained`` = a back-to-back loop of
    at least ``sustain_s`` seconds, each with the SM clock sampled while it ran."""
    try:
        n = 8192
        g = torch.Generator(device=device).manual_seed(11)
        a = torch.randn(n, n, device=device, generator=g).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=device, generator=g).to(torch.float8_e4m3fn).t()  # column-major operand
        one = torch.ones((), device=device)

        def mm():
            return torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)

        for _ in range(3):
            mm()
        torch.cuda.synchronize()
        flops = 2.0 * n * n * n
        best = float("inf")
        with ClockSampler(local_rank) as c_burst:
            for _ in range(10):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                mm()
                e1.record()
                torch.cuda.synchronize()
                best = min(best, e0.elapsed_time(e1))
        per = max(best, 0.05)
        loops = int(sustain_s * 1e3 / per) + 1
        with ClockSampler(local_rank) as c_sus:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(loops):
                mm()
            e1.record()
            torch.cuda.synchronize()
        sus_ms = e0.elapsed_time(e1)
        return {"burst_tflops": flops / best / 1e9, "sustained_tflops": flops * loops / sus_ms / 1e9,
                "sustained_seconds": sus_ms / 1e3, "burst_clocks": c_burst.summary(), "sustained_clocks": c_sus.summary(),
                "how": "torch._scaled_mm e4m3 x e4m3 -> bf16, per-tensor scales, 8192^3, CUDA events"}
    except Exception as e:
        return {"unavailable": repr(e)}


# --------------------------------------------------------------------- the tensor-parallel layers


def tp_chunk(i: int, n: int, k: int, kind: str, c: int, device):
    """Chunk ``c`` of layer ``i``, drawn on the device from its own seed and block-quantised: rows
    ``[c*n/8, ..)`` of a column-parallel weight, K columns ``[c*k/8, ..)`` of a row-parallel one. Chunk edges are
    multiples of 128, so quantising chunk by chunk equals quantising the whole weight."""
    from sglang_b200.weight_quant import block_quant_weight_fp8

    g = torch.Generator(device=device).manual_seed(3000 + 100 * i + c)
    shape = (n // CHUNKS, k) if kind == "column" else (n, k // CHUNKS)
    w = (torch.randn(shape, generator=g, device=device) * 0.02).bfloat16()
    return block_quant_weight_fp8(w)


def tp_shard(i: int, n: int, k: int, kind: str, rank: int, world: int, device):
    per = CHUNKS // world
    parts = [tp_chunk(i, n, k, kind, c, device) for c in range(rank * per, (rank + 1) * per)]
    dim = 0 if kind == "column" else 1
    return (torch.cat([p[0] for p in parts], dim).contiguous(), torch.cat([p[1] for p in parts], dim).contiguous())


def tp_activation(i: int, k: int, device, rows: int = M_ROWS):
    """N(0,1) with 1 % of the channels scaled x20, drawn on the device (identical on every rank)."""
    g = torch.Generator(device=device).manual_seed(3500 + i)
    x = torch.randn(rows, k, generator=g, device=device)
    idx = torch.randperm(k, generator=g, device=device)[: math.ceil(0.01 * k)]
    x[:, idx] *= 20
    return x.bfloat16()


def sample_rows(m: int, count: int = 32):
    count = min(count, m)
    step = m // count
    return [r * step + (7 * r) % step for r in range(count)]


def oracle_weight_sample(i: int, n: int, k: int, kind: str, device):
    """A few 128-row blocks of the un-sharded weight of layer ``i`` for the CPU oracle: one block out of every
    chunk for a column-parallel layer (so that every rank's shard is covered), four blocks for a row-parallel
    one. Returns (FP8 rows [B*128, K], scales [B, K/128], the output columns they produce), on the CPU."""
    if kind == "column":
        per = n // CHUNKS // 128
        wq, ws, cols = [], [], []
        for c in range(CHUNKS):
            q, s = tp_chunk(i, n, k, kind, c, device)
            b = (3 * c + 1) % per
            wq.append(q[b * 128:(b + 1) * 128].cpu())
            ws.append(s[b:b + 1].cpu())
            first = (c * per + b) * 128
            cols.extend(range(first, first + 128))
            del q, s
        return torch.cat(wq, 0), torch.cat(ws, 0), torch.tensor(cols)
    nb = n // 128
    blocks = sorted({0, nb // 3, (2 * nb) // 3, nb - 1})
    wq, ws = [], []
    for c in range(CHUNKS):
        q, s = tp_chunk(i, n, k, kind, c, device)
        wq.append(torch.cat([q[b * 128:(b + 1) * 128] for b in blocks], 0).cpu())
        ws.append(torch.cat([s[b:b + 1] for b in blocks], 0).cpu())
        del q, s
    cols = [b * 128 + j for b in blocks for j in range(128)]
    return torch.cat(wq, 1), torch.cat(ws, 1), torch.tensor(cols)


class TPLayers:
    """This rank's shard of the four layers, their inputs, the peer-memory all-reduce objects, and (rank 0) the
    oracle's answers on sampled rows and columns of the un-sharded layers."""

    def __init__(self, S, device, rank: int, world: int, row_counts=(M_ROWS,)):
        import oracle as O  # the checker of the sampled outputs; never on the timed path
        from sglang_b200 import parallel as P

        assert CHUNKS % world == 0, "the layers are defined as 8 chunks: run with 1, 2, 4 or 8 GPUs"
        self.S, self.P, self.O = S, P, O
        self.device, self.rank, self.world = device, rank, world
        self.layers, self.ref, self.peer = [], {}, {}
        for i, (name, n, k, kind) in enumerate(TP_LINEARS):
            x_full = tp_activation(i, k, device)
            wq, ws = tp_shard(i, n, k, kind, rank, world, device)
            if kind == "row":
                ks = k // world
                x = x_full[:, rank * ks:(rank + 1) * ks].contiguous()
            else:
                x = x_full
            self.layers.append((name, n, k, kind, x, wq, ws))
            if rank == 0:
                wq_s, ws_s, cols = oracle_weight_sample(i, n, k, kind, device)
                for m in row_counts:
                    rows = sample_rows(m)
                    want = O.w8a8_block_fp8_linear(x_full[rows].cpu(), wq_s, ws_s, output_dtype=torch.float32)
                    self.ref[(name, m)] = (rows, cols, want)
            del x_full
        torch.cuda.empty_cache()
        barrier(world)

    def peer_for(self, name: str, n: int, graph_safe: bool = False, max_tokens: int = M_ROWS):
        from sglang_b200.peer_allreduce import PeerAllReduce

        key = (name, graph_safe)
        if key not in self.peer:
            self.peer[key] = PeerAllReduce(max_tokens, n, torch.bfloat16, graph_safe=graph_safe)
        return self.peer[key]

    def forward(self, rows: int, mode: str, events=None, graph_safe: bool = False, inputs=None):
        """One pass over the four layers on the first ``rows`` rows. ``mode``: "peer" (all-reduce fused with the
        GEMM over peer memory) or "nccl". Returns the outputs (row-parallel outputs of "peer" are views of the
        symmetric buffers: valid until the layer's next call)."""
        S, outs = self.S, {}
        for name, n, k, kind, x, wq, ws in self.layers:
            xin = (inputs[name] if inputs is not None else x)[:rows]
            if rows <= 16 and events is None and (kind == "column" or self.world == 1 or mode == "nccl"):
                # decode size: the public linear (one launch: quantiser, GEMM and split-K sum)
                out = S.w8a8_block_fp8_linear(xin, wq, [128, 128], ws)
                if kind == "row" and self.world > 1:
                    self.P.tensor_model_parallel_all_reduce(out)
                outs[name] = out
                continue
            q, s = S.per_token_group_quant_fp8(xin, 128, column_major_scales=True)
            if events is not None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            if kind == "row" and self.world > 1 and mode == "peer":
                out, _ = self.peer_for(name, n, graph_safe, M_ROWS if not graph_safe else 16).linear(q, s, wq, ws)
            else:
                out = S.w8a8_block_fp8_matmul(q, wq, s, ws, [128, 128], torch.bfloat16)
                if kind == "row" and self.world > 1:
                    self.P.tensor_model_parallel_all_reduce(out)
            if events is not None:
                e1.record()
                events.append((name, e0, e1))
            outs[name] = out
        return outs

    def check(self, rows: int, mode: str) -> dict:
        """Run one pass and compare sampled rows x columns of every layer's output, as held by every rank, with
        the oracle of the un-sharded layer. Returns {"rel_frob": worst, "checked_rows", "checked_cols", "ok"}."""
        world, dev = self.world, self.device
        barrier(world)
        outs = self.forward(rows, mode)
        torch.cuda.synchronize()
        worst, n_rows, n_cols = 0.0, 0, 0
        for name, n, k, kind, *_ in self.layers:
            ridx = torch.tensor(sample_rows(rows), device=dev)
            mine = outs[name][ridx].float()
            if world > 1:
                parts = [torch.empty_like(mine) for _ in range(world)]
                torch.distributed.all_gather(parts, mine.contiguous())
            else:
                parts = [mine]
            if self.rank == 0:
                _, cols, want = self.ref[(name, rows)]
                n_rows, n_cols = want.shape[0], n_cols + want.shape[1]
                if kind == "column":
                    got = [torch.cat(parts, 1).cpu()[:, cols]]
                else:  # replicated result: every rank's copy is checked
                    got = [p.cpu()[:, cols] for p in parts]
                for g_ in got:
                    err = self.O.rel_frobenius(g_, want)
                    worst = max(worst, err if err == err else float("inf"))
        status_ok = device_status_clear(world, dev)
        ok = agree(worst < TOL and status_ok, world, dev)
        return {"rel_frob": worst, "checked_rows": n_rows, "checked_cols": n_cols, "device_status_clear": status_ok,
                "ok": ok, "against": "CPU oracle of the un-sharded layers on sampled rows x columns"}


# --------------------------------------------------------------------------- CPU baseline legs
# The host arm runs the oracle (the reference's torch-native path: quantise the rows, dequantise the whole weight,
# fp32 matmul per 128 x 128 block) on a bounded sample of the headline workload: the first R of the 4096 rows
# against the complete un-sharded weights. The weight dequantisation the reference pays per call is then spread
# over R rows instead of 4096, so R is made as large as the time budget allows and is stated in the line.


def cpu_inputs(rows: int):
    """Rows of every layer's input and its complete weight, with the shapes and distributions of the GPU arm.
    To keep the set-up short the weight is one seeded, block-quantised 1024-row slab repeated along N (the
    values do not change what the host path computes per element)."""
    from sglang_b200 import synthetic

    acts, weights = {}, {}
    for i, (name, n, k, _) in enumerate(TP_LINEARS):
        acts[name] = synthetic.activation(rows, k, 2000 + 10 * i)
        wq, ws = synthetic.weight(1024, k, 2001 + 10 * i)
        reps = n // 1024
        weights[name] = (wq.repeat(reps, 1), ws.repeat(reps, 1))
    return acts, weights


def cpu_linears(rows: int, threads: int, weights_cpu, acts_cpu):
    """One pass of the four linears through the oracle (torch-native reference restatement)."""
    import oracle as O

    torch.set_num_threads(threads)
    for name, n, k, _ in TP_LINEARS:
        wq, ws = weights_cpu[name]
        O.w8a8_block_fp8_linear(acts_cpu[name][:rows], wq, ws, output_dtype=torch.bfloat16)


def cpu_rows_for(target_s: float, threads: int, weights, acts, cap: int) -> int:
    """Rows per pass so that a pass takes about ``target_s``: two probe passes give the fixed (dequantisation)
    and the per-row cost."""
    cpu_linears(32, threads, weights, acts)  # warm-up of the thread pool and allocator
    t0 = time.perf_counter()
    cpu_linears(32, threads, weights, acts)
    t32 = time.perf_counter() - t0
    t0 = time.perf_counter()
    cpu_linears(160, threads, weights, acts)
    t160 = time.perf_counter() - t0
    per_row = max((t160 - t32) / 128, 1e-5)
    fixed = max(t32 - 32 * per_row, 0.0)
    return int(max(32, min(cap, (target_s - fixed) / per_row))) // 32 * 32


def time_cpu_baseline(budget_s: float = 14.0):
    """Oracle on the host cores on a bounded row sample sized to ~budget_s of CPU work."""
    threads = os.cpu_count() or 1
    acts, weights = cpu_inputs(1024)
    rows = cpu_rows_for(budget_s / 2, threads, weights, acts, 1024)
    t0 = time.perf_counter()
    cpu_linears(rows, threads, weights, acts)
    dt = time.perf_counter() - t0
    return {"value": rows * FLOPS_PER_ROW / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"the four un-sharded linears on the first {rows} of {M_ROWS} rows, one pass, {dt:.1f} s (torch fp32, oracle/)"}


def run_reference(args, rank: int):
    """The reference's CPU implementation of the path (its torch-native functions, restated in
    oracle/ and pinned to them by the golden vectors) on all host threads."""
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    acts, weights = cpu_inputs(1024)
    # about 6 s of host work per step, less when many steps are asked for so that the whole run stays within a
    # few minutes
    target = min(6.0, 150.0 / max(1, args.steps + args.warmup))
    rows = cpu_rows_for(target, threads, weights, acts, 1024)
    for _ in range(args.warmup):
        cpu_linears(rows, threads, weights, acts)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_linears(rows, threads, weights, acts)
    dt = (time.perf_counter() - t0) / args.steps
    v = rows * FLOPS_PER_ROW / dt / 1e12
    sample = f"each step = the four un-sharded linears on {rows} of {M_ROWS} rows (torch fp32 on {threads} threads)"
    print(json.dumps({
        "impl": "reference", "metric": "block-FP8 GEMM TFLOPS", "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None,
        "dtype": "fp8_e4m3 weights+activations, fp32 accumulate (emulated in fp32 on CPU)",
        "data": "synthetic", "config": {"workload": WORKLOAD, "rows_per_step": rows},
        "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------- 1-GPU line items


def bench_llama8b(S, device, fp8_peak: float):
    """BASELINE config 2: the four Llama-3-8B-shaped linears on one GPU at M = 1 ... 8192 (quant + GEMM; the
    decode sizes appear under ``kernels`` with rotated weights). Device time from CUDA-graph replays."""
    from sglang_b200 import synthetic

    out = {}
    for i, (name, n, k) in enumerate(LLAMA8B_LINEARS):
        wq, ws = synthetic.weight(n, k, 2001 + 10 * i, device=device)
        for m in (128, 1024, 8192):
            x = synthetic.activation(m, k, 2000 + 10 * i).to(device)
            q, s = S.per_token_group_quant_fp8(x, 128, column_major_scales=True)
            us_lin = graph_time_us([lambda: S.w8a8_block_fp8_linear(x, wq, [128, 128], ws)] * 4)
            us_mm = graph_time_us([lambda: S.w8a8_block_fp8_matmul(q, wq, s, ws, [128, 128], torch.bfloat16)] * 4)
            fl = 2.0 * m * n * k
            nbytes = m * k + n * k + 2 * m * n + 4 * (m * k // 128 + n * k // 16384)
            out[f"{name}_M{m}"] = {"N": n, "K": k, "linear_us": us_lin, "gemm_us": us_mm,
                                   "gemm_tflops": fl / us_mm / 1e6, "linear_tflops": fl / us_lin / 1e6,
                                   **roofline_frac(us_mm * 1e-3, fl, nbytes, fp8_peak=fp8_peak)}
        del wq, ws
    torch.cuda.empty_cache()
    return out


def bench_comparators(S, device):
    """The block-scaled FP8 GEMM of the libraries the reference calls on this GPU, on the same operands as ours:
    FlashInfer ``gemm_fp8_nt_groupwise`` (CUTLASS sm100 blockwise kernel, 1-SM and 2-SM MMA) and vLLM's
    ``cutlass_scaled_mm`` (CUTLASS sm100 blockwise kernel). Bench-only: the package never imports them. An entry
    says ``unavailable`` with the reason when a library or its compiled module is missing."""
    from sglang_b200 import synthetic

    shapes = [("llama8b_" + n_, 8192, n, k) for n_, n, k in LLAMA8B_LINEARS]
    shapes += [("llama70b_" + n_, M_ROWS, n, k) for n_, n, k, _ in TP_LINEARS]

    def rel(a, b):
        a, b = a.float(), b.float()
        return float((a - b).norm() / b.norm())

    fi_mod, fi_err = None, None
    try:
        os.environ.setdefault("FLASHINFER_WORKSPACE_BASE", os.path.join(ROOT, "baseline", "_ref", "fi"))
        os.environ.setdefault("FLASHINFER_CUDA_ARCH_LIST", "10.0a")
        from flashinfer.gemm.gemm_base import gen_gemm_sm100_module

        spec = gen_gemm_sm100_module()
        so = str(spec.jit_library_path)
        if not os.path.exists(so):
            raise RuntimeError("the sm100 GEMM module of flashinfer is not prebuilt (it is JIT-compiled; no build "
                               "is attempted inside the benchmark)")
        fi_mod = spec.load(so)
        fi_ws = torch.empty(32 * 1024 * 1024, dtype=torch.uint8, device=device)
    except Exception as e:
        fi_err = repr(e)[:300]
    vllm_err = None
    try:
        import vllm._C  # noqa: F401
        vllm_mm = torch.ops._C.cutlass_scaled_mm
    except Exception as e:
        vllm_err = repr(e)[:300]

    out = {}
    for i, (label, m, n, k) in enumerate(shapes):
        g = torch.Generator(device=device).manual_seed(8100 + i)
        x = torch.randn(m, k, device=device, generator=g).bfloat16()
        w_bf16 = (torch.randn(n, k, device=device, generator=g) * 0.02).bfloat16()
        wq, ws = synthetic.block_quant_weight_fp8(w_bf16)
        q, s = S.per_token_group_quant_fp8(x, 128, column_major_scales=True)  # s: [m, k/128], stride (1, m)
        ours = S.w8a8_block_fp8_matmul(q, wq, s, ws, [128, 128], torch.bfloat16)
        fl = 2.0 * m * n * k
        item = {"M": m, "N": n, "K": k}
        us = graph_time_us([lambda: S.w8a8_block_fp8_matmul(q, wq, s, ws, [128, 128], torch.bfloat16)] * 4)
        item["ours"] = {"us": us, "tflops": fl / us / 1e6}
        for mma_sm in (1, 2):
            key = f"flashinfer_cutlass_sm100_{mma_sm}sm"
            if fi_mod is None:
                item[key] = {"unavailable": fi_err}
                continue
            try:
                a_sc = s.t().contiguous() if not s.t().is_contiguous() else s.t()  # [k/128, m]
                b_sc = ws.t().contiguous()                                            # [k/128, n/128]
                o = torch.empty(m, n, dtype=torch.bfloat16, device=device)

                def call():
                    fi_mod.gemm_fp8_nt_groupwise(fi_ws, q, wq, a_sc, b_sc, o, 1, 128, 128, "MN", mma_sm)

                call()
                torch.cuda.synchronize()
                us = graph_time_us([call] * 4)
                item[key] = {"us": us, "tflops": fl / us / 1e6, "rel_frob_vs_ours": rel(o, ours)}
            except Exception as e:
                item[key] = {"unavailable": repr(e)[:300]}
                torch.cuda.synchronize()
        # the same layer with power-of-two (UE8M0) scales, the format the reference's DeepGEMM path uses on this
        # GPU: the block-scaled tensor-core kernel (no promotion) against the promotion kernel on the same bytes
        try:
            from sglang_b200 import _native, weight_quant as W

            wq2, ws2 = W.quant_weight_ue8m0(w_bf16)
            ws2p = W.transform_scale_ue8m0(ws2, mn=n)
            q2, s2 = S.per_token_group_quant_fp8(x, 128, column_major_scales=True, scale_tma_aligned=True, scale_ue8m0=True)
            o2 = S.w8a8_block_fp8_matmul(q2, wq2, s2, ws2p, [128, 128], torch.bfloat16)
            with _native.tuning(gemm_ue8m0=0):
                o2_ref = S.w8a8_block_fp8_matmul(q2, wq2, s2, ws2p, [128, 128], torch.bfloat16)
            us = graph_time_us([lambda: S.w8a8_block_fp8_matmul(q2, wq2, s2, ws2p, [128, 128], torch.bfloat16)] * 4)
            item["ours_ue8m0_block_scaled_mma"] = {"us": us, "tflops": fl / us / 1e6,
                                                   "rel_frob_vs_promotion_kernel_same_bytes": rel(o2, o2_ref)}
            del wq2, ws2, ws2p, q2, s2, o2, o2_ref
        except Exception as e:
            item["ours_ue8m0_block_scaled_mma"] = {"unavailable": repr(e)[:300]}
            torch.cuda.synchronize()
        del w_bf16
        key = "vllm_cutlass_sm100"
        if vllm_err is not None:
            item[key] = {"unavailable": vllm_err}
        else:
            try:
                o = torch.empty(m, n, dtype=torch.bfloat16, device=device)
                b_t, sb_t = wq.t(), ws.t()

                def call():
                    vllm_mm(o, q, b_t, s, sb_t, None)

                call()
                torch.cuda.synchronize()
                us = graph_time_us([call] * 4)
                item[key] = {"us": us, "tflops": fl / us / 1e6, "rel_frob_vs_ours": rel(o, ours)}
            except Exception as e:
                item[key] = {"unavailable": repr(e)[:300]}
                torch.cuda.synchronize()
        out[label] = item
        del x, wq, ws, q, s, ours
    torch.cuda.empty_cache()
    try:
        out["llama70b_sustained"] = sustained_comparison(S, device, fi_mod, fi_ws if fi_mod is not None else None)
    except Exception as e:
        out["llama70b_sustained"] = {"error": repr(e)[:300]}
        torch.cuda.synchronize()
    torch.cuda.empty_cache()
    return out


def sustained_comparison(S, device, fi_mod, fi_ws, seconds: float = 1.5):
    """The four Llama-3-70B GEMMs (M = 4096) looped for ``seconds`` under the power cap, GEMMs only: this
    library's promotion kernel (fp32 scales), its block-scaled kernel (the same layers re-quantised to
    power-of-two scales) and FlashInfer's sm100 kernel (fp32 scales). TF/s over the whole loop, with the clock
    record of each loop; the burst figures above are single graph replays at full clock."""
    from sglang_b200 import synthetic, weight_quant as W

    ops = []
    for i, (name, n, k, _) in enumerate(TP_LINEARS):
        g = torch.Generator(device=device).manual_seed(8200 + i)
        x = torch.randn(M_ROWS, k, device=device, generator=g).bfloat16()
        w = (torch.randn(n, k, device=device, generator=g) * 0.02).bfloat16()
        wq, ws = synthetic.block_quant_weight_fp8(w)
        q, s = S.per_token_group_quant_fp8(x, 128, column_major_scales=True)
        wq2, ws2 = W.quant_weight_ue8m0(w)
        ws2p = W.transform_scale_ue8m0(ws2, mn=n)
        q2, s2 = S.per_token_group_quant_fp8(x, 128, column_major_scales=True, scale_tma_aligned=True, scale_ue8m0=True)
        o = torch.empty(M_ROWS, n, dtype=torch.bfloat16, device=device)
        ops.append((q, s, wq, ws, q2, s2, wq2, ws2p, s.t().contiguous(), ws.t().contiguous(), o))
        del x, w
    flops = sum(2.0 * M_ROWS * n * k for _, n, k, _ in TP_LINEARS)

    def promo():
        for q, s, wq, ws, *_ in ops:
            S.w8a8_block_fp8_matmul(q, wq, s, ws, [128, 128], torch.bfloat16)

    def scaled():
        for _, _, _, _, q2, s2, wq2, ws2p, *_ in ops:
            S.w8a8_block_fp8_matmul(q2, wq2, s2, ws2p, [128, 128], torch.bfloat16)

    def fi():
        for q, _, wq, _, _, _, _, _, a_sc, b_sc, o in ops:
            fi_mod.gemm_fp8_nt_groupwise(fi_ws, q, wq, a_sc, b_sc, o, 1, 128, 128, "MN", 1)

    res = {"seconds_target": seconds, "rows": M_ROWS}
    arms = [("ours_fp32_scales_promotion", promo), ("ours_ue8m0_block_scaled_mma", scaled)]
    if fi_mod is not None:
        arms.append(("flashinfer_cutlass_sm100_1sm", fi))
    for label, fn in arms:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        reps = max(4, int(seconds * 1e3 / max(e0.elapsed_time(e1), 1e-3)))
        with ClockSampler(torch.cuda.current_device()) as cs:
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        res[label] = {"tflops": flops * reps / ms / 1e9, "passes": reps, "seconds": ms / 1e3, "clocks": cs.summary()}
    return res


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
    for name, n, k in LLAMA8B_LINEARS:
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


def moe_reference_rows(O, cfg, x, tw, ti, rows, seed: int, device):
    """Oracle output of the MoE layer for the tokens ``rows`` (a token's result does not depend on the other
    tokens). The experts those tokens use are drawn again from their per-expert seeds and taken to the CPU."""
    from sglang_b200 import synthetic

    ridx = torch.tensor(rows, device=ti.device)
    used = torch.unique(ti[ridx].flatten()).long()
    local = torch.searchsorted(used, ti[ridx].long()).to(torch.int32)
    parts = [synthetic.expert_weights(1, cfg["I"], cfg["H"], seed, device=device, first_expert=int(e)) for e in used.tolist()]
    w1, w2, w1_s, w2_s = (torch.cat([p[j] for p in parts], 0).cpu() for j in range(4))
    del parts
    return O.fused_experts_fp8(x[ridx].cpu(), w1, w2, w1_s, w2_s, tw[ridx].cpu().float(), local.cpu(), [128, 128])


def moe_inputs(cfg, T: int, device, seed: int = 5000):
    """Tokens and routing of one MoE line item (identical on every rank): N(0,1) tokens; DeepSeek-V3: N(0,1)
    logits through the biased grouped top-k; Mixtral: N(0,1) logits plus a Zipf(1.2) per-expert bias, softmax top-2."""
    from sglang_b200 import synthetic
    from sglang_b200.topk import biased_grouped_topk, fused_topk

    E, topk, H = cfg["E"], cfg["topk"], cfg["H"]
    g = torch.Generator().manual_seed(seed + T)
    x = torch.randn(T, H, generator=g).bfloat16().to(device)
    if "n_group" in cfg:
        logits = torch.randn(T, E, generator=g).to(device)
        tw, ti = biased_grouped_topk(x, logits, torch.zeros(E, device=device), topk, True, cfg["n_group"], cfg["topk_group"])
    else:
        logits = synthetic.zipf_router_logits(T, E, seed + 1).to(device)
        tw, ti = fused_topk(x, logits, topk, True)
    return x, tw, ti


def bench_moe(S, device, steps: int, fp8_peak: float):
    """Extra line items: fused-MoE tokens/s for the DeepSeek-V3 and Mixtral shaped layers on one GPU at every
    token count of BASELINE configs 4 and 5; each checked on sampled tokens against the oracle first."""
    import oracle as O
    from sglang_b200 import synthetic

    out = {}
    for label, cfg, Ts in (("deepseek_v3", synthetic.DEEPSEEK_V3, (16384, 2048, 128, 1)),
                           ("mixtral_8x7b", synthetic.MIXTRAL, (8192, 1024, 64, 1))):
        E, topk, H, I = cfg["E"], cfg["topk"], cfg["H"], cfg["I"]
        seed = 4000 + E
        w1, w2, w1_s, w2_s = synthetic.expert_weights(E, I, H, seed, device=device)
        conf = S.MoeRunnerConfig(inplace=False)
        for T in Ts:
            x, tw, ti = moe_inputs(cfg, T, device)
            topk_out = S.StandardTopKOutput(tw, ti, None)

            def call():
                return S.fused_experts(x, w1, w2, topk_out, conf, use_fp8_w8a8=True, w1_scale=w1_s, w2_scale=w2_s,
                                       block_shape=[128, 128])

            got = call()
            rows = sample_rows(T, 4 if T == Ts[0] else 2)
            want = moe_reference_rows(O, cfg, x, tw, ti, rows, seed, device)
            err = O.rel_frobenius(got[rows].float().cpu(), want)
            parity = {"rel_frob": err, "checked_rows": len(rows), "device_status_clear": device_status_clear(1, device),
                      "ok": bool(err < TOL)}
            key = f"{label}_T{T}"
            if not (parity["ok"] and parity["device_status_clear"]):
                out[key] = {"error": "parity check failed; not timed", "parity": parity}
                continue
            if T >= 1024:
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
            else:
                ms = graph_time_us([call] * 4) * 1e-3  # a server replays decode steps from a graph
            active = int(torch.unique(ti).numel())
            moe_bytes = 4 * T * H + 3 * H * I * active * (1 + 4 / 16384) + 8 * T * topk
            out[key] = {"tokens_per_s": T / ms * 1e3, "ms": ms, "tflops": 6 * T * topk * H * I / ms / 1e9,
                        "hbm_gbs_on_algorithmic_bytes": moe_bytes / ms / 1e6,
                        **roofline_frac(ms, 6 * T * topk * H * I, moe_bytes, fp8_peak=fp8_peak), "parity": parity,
                        "config": {"E": E, "topk": topk, "H": H, "I": I, "T": T, "experts_touched": active}}
        del w1, w2, w1_s, w2_s
        torch.cuda.empty_cache()
    return out


# ---------------------------------------------------------------------- N > 1 line items


def bench_tp_items(tp: TPLayers, world: int, device, steps: int, fp8_peak: float):
    """BASELINE config 3 at M = 32 / 512 / 4096 with the all-reduce by NCCL or fused with the GEMM over peer
    memory, plus the decode-sized step replayed from a CUDA graph. Every item is checked against the oracle of
    the un-sharded layers before it is timed."""
    out = {}
    w_bytes = sum(wq.numel() for *_, wq, _ in tp.layers)
    for rows in (M_ROWS, 512, 32):
        for mode in ("nccl", "peer"):
            key = f"tp_llama70b_M{rows}" + ("_peer_fused" if mode == "peer" else "_nccl")
            parity = tp.check(rows, mode)
            if not parity["ok"]:
                out[key] = {"error": "parity check failed; not timed", "parity": parity, "tp": world}
                continue
            ms = timed(lambda: tp.forward(rows, mode), steps, world, device)
            fl = FLOPS_PER_ROW * rows
            out[key] = {"tflops": fl / ms / 1e9, "ms": ms, "tp": world, "parity": parity,
                        "allreduce": "peer memory, fused with the GEMM" if mode == "peer" else "nccl",
                        "allreduce_bytes_per_step": 2 * rows * 8192 * 2,
                        **roofline_frac(ms, fl / world, w_bytes, 2 * (world - 1) / world * 2 * rows * 8192 * 2,
                                        fp8_peak=fp8_peak)}
    # the decode-sized step (M = 16) replayed from a CUDA graph (how a server runs decode): the peer path then
    # keeps its epochs on the device and uses a single slot buffer so that the capture can be replayed
    for mode in ("nccl", "peer"):
        key = "tp_llama70b_M16_graph" + ("_peer_fused" if mode == "peer" else "_nccl")
        try:
            stream = torch.cuda.Stream()
            graph = torch.cuda.CUDAGraph()
            barrier(world)
            with torch.cuda.stream(stream):
                tp.forward(16, mode, graph_safe=True)
                torch.cuda.synchronize()
                barrier(world)
                with torch.cuda.graph(graph, stream=stream):
                    tp.forward(16, mode, graph_safe=True)
            ms = timed(graph.replay, steps, world, device)
            out[key] = {"ms": ms, "tp": world, "device_status_clear": device_status_clear(world, device)}
        except Exception as e:  # a capture that fails must not take the other line items with it
            out[key] = {"error": repr(e)[:300]}
            torch.cuda.synchronize()
            barrier(world)
    return out


def bench_moe_parallel(S, device, rank: int, world: int, steps: int, fp8_peak: float):
    """BASELINE config 5 (DeepSeek-V3 layer, experts partitioned over the ranks, T = 16384 / 2048 / 128 / 1 tokens
    in total) in three forms -- "standard" (tokens replicated, all-reduce), all-to-all through NCCL, all-to-all
    through this package's peer-memory kernels -- and config 4 (Mixtral layer, intermediate dimension split over
    the ranks, all-reduce). Before an item is timed its output is compared with the oracle on sampled tokens (and
    the all-to-all forms with the standard form on every token)."""
    import oracle as O
    from sglang_b200 import parallel as P
    from sglang_b200 import synthetic

    out = {}

    def sampled(result_rows, tokens, offset, count):
        """Rows of ``tokens`` from a result that holds tokens [offset, offset + count): summed over ranks so that
        every rank (and the checker on rank 0) sees all of them."""
        buf = torch.zeros(len(tokens), result_rows.shape[1], dtype=torch.float32, device=device)
        for j, t in enumerate(tokens):
            if offset <= t < offset + count:
                buf[j] = result_rows[t - offset].float()
        if world > 1:
            torch.distributed.all_reduce(buf)
        return buf

    # ---- expert parallel, DeepSeek-V3
    cfg = synthetic.DEEPSEEK_V3
    E, topk, H, I = cfg["E"], cfg["topk"], cfg["H"], cfg["I"]
    el, seed = E // world, 4000 + E
    w1, w2, w1_s, w2_s = synthetic.expert_weights(el, I, H, seed, device=device, first_expert=rank * el)
    for T in (16384, 2048, 128, 1):
        x, tw, ti = moe_inputs(cfg, T, device)
        tokens = sample_rows(T, 4 if T == 16384 else 2)
        want = moe_reference_rows(O, cfg, x, tw, ti, tokens, seed, device) if rank == 0 else None
        per = -(-T // world)
        lo, hi = min(T, rank * per), min(T, (rank + 1) * per)
        full_std = None
        modes = (("ep", "standard"), ("ep_a2a", "a2a_nccl"), ("ep_peer", "a2a_peer_memory"))
        if T < world:  # fewer tokens than ranks: nothing to partition, only the replicated form applies
            modes = modes[:1]
        for mode, label in modes:
            key = f"ep_deepseek_v3_T{T}_{label}"
            try:
                layer = P.FusedMoE(w1, w2, w1_s, w2_s, rank, world, mode=mode, presharded=True, num_experts=E,
                                   max_tokens=max(per, 1))
                if mode == "ep":
                    xs, ws_, is_ = x, tw, ti
                    off, cnt = 0, T
                else:
                    xs, ws_, is_ = x[lo:hi].contiguous(), tw[lo:hi].contiguous(), ti[lo:hi].contiguous()
                    off, cnt = lo, hi - lo
                barrier(world)
                got = layer(xs, ws_, is_)
                torch.cuda.synchronize()
                rows_got = sampled(got, tokens, off, cnt if mode != "ep" else T)
                if mode == "ep" and world > 1:
                    rows_got /= world  # every rank contributed the same replicated rows
                parity = {"checked_rows": len(tokens)}
                err = O.rel_frobenius(rows_got.cpu(), want) if rank == 0 else 0.0
                parity["rel_frob"] = err
                if mode == "ep":
                    full_std = got.clone()
                elif full_std is not None and cnt > 0:
                    d = (got.float() - full_std[lo:hi].float()).norm() / full_std[lo:hi].float().norm().clamp_min(1e-30)
                    parity["rel_frob_vs_standard_all_tokens"] = dist_max(float(d), world, device)
                elif full_std is not None:
                    parity["rel_frob_vs_standard_all_tokens"] = dist_max(0.0, world, device)
                status_ok = device_status_clear(world, device)
                ok = err < TOL and status_ok and parity.get("rel_frob_vs_standard_all_tokens", 0.0) < TOL
                parity["ok"], parity["device_status_clear"] = agree(ok, world, device), status_ok
                if not parity["ok"]:
                    out[key] = {"error": "parity check failed; not timed", "parity": parity, "ep": world}
                    continue
                ms = timed(lambda: layer(xs, ws_, is_), max(2, steps // 2), world, device)
                # per GPU: 1/world of the flops, its experts' weights once; the all-to-all forms move every local
                # token's FP8 row + scales to the other owning ranks (at most topk_group ranks per token) and bf16
                # rows back (one partial row per owning rank, or one row per slot when the down GEMM pushes
                # them); the standard form all-reduces the [T, H] bf16 output
                if mode == "ep":
                    link = 2 * (world - 1) / world * T * H * 2
                elif mode == "ep_peer":
                    # rows out once per owning rank; results back once per (token, slot): pushed by the down GEMM
                    link = per * (world - 1) / world * (min(cfg["topk_group"], world) * (H + H // 32) + topk * 2 * H)
                else:
                    link = per * min(cfg["topk_group"], world) * (world - 1) / world * (H + H // 32 + 2 * H)
                active = int(torch.unique(ti).numel())
                out[key] = {"tokens_per_s": T / ms * 1e3, "ms": ms, "ep": world, "tflops": 6 * T * topk * H * I / ms / 1e9,
                            "parity": parity,
                            **roofline_frac(ms, 6 * T * topk * H * I / world,
                                            3 * H * I * min(el, active) * (1 + 4 / 16384), link, fp8_peak=fp8_peak)}
                del layer
            except Exception as e:
                out[key] = {"error": repr(e)[:300]}
                torch.cuda.synchronize()
                barrier(world)
        del full_std
    del w1, w2, w1_s, w2_s
    torch.cuda.empty_cache()

    # ---- tensor parallel over the intermediate dimension, Mixtral
    cfg = synthetic.MIXTRAL
    E, topk, H, I = cfg["E"], cfg["topk"], cfg["H"], cfg["I"]
    seed = 4000 + E
    full = synthetic.expert_weights(E, I, H, seed, device=device)
    shard = P.shard_moe_tp(*full, rank, world)
    del full
    torch.cuda.empty_cache()
    layer = P.FusedMoE(*shard, rank, world, mode="tp", presharded=True, num_experts=E)
    for T in (8192, 1024, 64, 1):
        key = f"tp_mixtral_8x7b_T{T}"
        try:
            x, tw, ti = moe_inputs(cfg, T, device)
            tokens = sample_rows(T, 4 if T == 8192 else 2)
            barrier(world)
            got = layer(x, tw, ti)
            torch.cuda.synchronize()
            err = 0.0
            if rank == 0:
                want = moe_reference_rows(O, cfg, x, tw, ti, tokens, seed, device)
                err = O.rel_frobenius(got[tokens].float().cpu(), want)
            status_ok = device_status_clear(world, device)
            parity = {"rel_frob": err, "checked_rows": len(tokens), "device_status_clear": status_ok,
                      "ok": agree(err < TOL and status_ok, world, device)}
            if not parity["ok"]:
                out[key] = {"error": "parity check failed; not timed", "parity": parity, "tp": world}
                continue
            ms = timed(lambda: layer(x, tw, ti), max(2, steps // 2), world, device)
            active = int(torch.unique(ti).numel())
            out[key] = {"tokens_per_s": T / ms * 1e3, "ms": ms, "tp": world, "tflops": 6 * T * topk * H * I / ms / 1e9,
                        "parity": parity,
                        **roofline_frac(ms, 6 * T * topk * H * I / world, 3 * H * I / world * active * (1 + 4 / 16384),
                                        2 * (world - 1) / world * T * H * 2, fp8_peak=fp8_peak)}
        except Exception as e:
            out[key] = {"error": repr(e)[:300]}
            torch.cuda.synchronize()
            barrier(world)
    return out


# ------------------------------------------------------------------------------------ main


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="headline only: skip the extra line items")
    ap.add_argument("--inner", type=int, default=0, help="passes per step (0 = sized for a ~2 s timed region)")
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
    stdout_fd = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        # keep stdout to the one JSON line: libraries (NCCL's version banner among them) write to file
        # descriptor 1 directly, so it points at stderr until the line is printed
        sys.stdout.flush()
        stdout_fd = os.dup(1)
        os.dup2(2, 1)
        torch.distributed.init_process_group("nccl", device_id=device)
    import sglang_b200 as S

    peaks = load_peaks()
    fp8_meas = measure_fp8_peak(device, local_rank, sustain_s=2.0 if world == 1 else 1.0)
    fp8_sus = fp8_meas.get("sustained_tflops") or 2 * peaks["bf16_sustained"]
    fp8_burst = fp8_meas.get("burst_tflops") or 2 * peaks["bf16"]

    tp = TPLayers(S, device, rank, world, row_counts=(M_ROWS,) if args.no_extras else (M_ROWS, 512, 32))
    mode = "peer"

    # ------------------------------------------------------------------ parity gate of the headline
    parity = tp.check(M_ROWS, mode)
    if not parity["ok"]:
        if stdout_fd is not None:
            sys.stdout.flush()
            os.dup2(stdout_fd, 1)
        if rank == 0:
            print(json.dumps({"metric": "block-FP8 GEMM TFLOPS", "value": None, "unit": "TFLOP/s", "n_gpus": world,
                              "error": "the headline workload failed its parity check; nothing was timed", "parity": parity}))
        raise SystemExit(1)

    # ---------------------------------------------------------------- device-resident timing
    barrier(world)
    for _ in range(args.warmup):
        tp.forward(M_ROWS, mode)
    pass_ms = timed(lambda: tp.forward(M_ROWS, mode), 3, world, device, warm=0)
    inner = args.inner if args.inner > 0 else max(1, min(64, math.ceil(2000.0 / (args.steps * pass_ms))))
    gemm_events = []
    barrier(world)
    with ClockSampler(local_rank) as clocks:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            for _ in range(inner):
                tp.forward(M_ROWS, mode, events=gemm_events)
        e1.record()
        barrier(world)
    total_ms = e0.elapsed_time(e1)
    ms_step = dist_max(total_ms / args.steps, world, device)
    if not device_status_clear(world, device):
        raise SystemExit("device status word set: a bounded wait timed out; the numbers are void")
    value = inner * M_ROWS * FLOPS_PER_ROW / ms_step / 1e9
    clk = clocks.summary()

    per_shape = {}
    for name, a, b in gemm_events:
        per_shape.setdefault(name, []).append(a.elapsed_time(b))
    gemm_ms = sum(statistics.mean(v) for v in per_shape.values())
    gemm_tflops = M_ROWS * FLOPS_PER_ROW / world / gemm_ms / 1e9  # per GPU
    sustained_run = ms_step * args.steps >= 1500.0
    fp8_peak = fp8_sus if sustained_run else fp8_burst
    shard = {name: ((n // world, k) if kind == "column" else (n, k // world)) for name, n, k, kind in TP_LINEARS}
    alg_bytes = {nm: M_ROWS * kk + nn * kk + 2 * M_ROWS * nn + 4 * (M_ROWS * kk // 128 + nn * kk // 16384)
                 for nm, (nn, kk) in shard.items()}
    traffic_ratio = 1.10
    roofline = {
        "bound": "tensor", "achieved": gemm_tflops, "peak": fp8_peak, "unit": "TFLOP/s", "frac": gemm_tflops / fp8_peak,
        "traffic": traffic_ratio * sum(alg_bytes.values()) / len(alg_bytes),
        "kernel": "block_fp8_gemm_kernel<256,dense,bf16>" + (" (row-parallel layers: fan-out epilogue + finishing kernel)" if world > 1 else ""),
        "traffic_note": "dram read+write of one ncu capture of this kernel at 8192x8192x4096 was 1.10 x its algorithmic bytes; "
                        "scaled to the mean algorithmic bytes of the four launches of a pass",
        "algorithmic_bytes_per_launch": sum(alg_bytes.values()) / len(alg_bytes),
        "peak_note": ("measured in this process: torch._scaled_mm FP8 8192^3, "
                      + ("sustained loop" if sustained_run else "best single launch")
                      + (" (timed region %.1f s)" % (ms_step * args.steps / 1e3))) if "burst_tflops" in fp8_meas
                     else f"2 x {peaks['source']} dense bf16 (no FP8 GEMM could be timed: {fp8_meas.get('unavailable')})",
        "fp8_peak_measured": fp8_meas,
        "frac_of_measured_fp8_burst": gemm_tflops / fp8_burst, "frac_of_measured_fp8_sustained": gemm_tflops / fp8_sus,
        "frac_of_2x_bf16_burst": gemm_tflops / (2 * peaks["bf16"]), "frac_of_2x_bf16_sustained": gemm_tflops / (2 * peaks["bf16_sustained"]),
        "frac_of_nominal_fp8": gemm_tflops / NOMINAL_FP8,
        "ms_x_sm_mhz": gemm_ms * (clk["sm_mhz"] or 0),
        "per_shape_tflops_per_gpu": {nm: 2 * M_ROWS * nn * kk / statistics.mean(per_shape[nm]) / 1e9 for nm, (nn, kk) in shard.items()},
    }

    # ------------------------------------------------------------------ end-to-end (host buffers)
    # Every rank copies its own inputs from pinned host memory and its own part of the outputs back: the N/p
    # output columns of a column-parallel layer, rows [rank*M/p, ..) of a row-parallel layer's summed result
    # (every rank holds the whole sum). The copies run on their own streams so that H2D, kernels and D2H of
    # consecutive layers overlap; every byte still crosses inside the timed region.
    rows_lo, rows_hi = rank * M_ROWS // world, (rank + 1) * M_ROWS // world
    # The batch lives in host memory once: a rank copies its own K shard of a row-parallel layer's input, and of a
    # column-parallel layer's input (which every rank needs in full) only rows [rank*M/p, ..); the group then
    # all-gathers those rows over NVLink instead of every rank pulling the whole matrix over PCIe.
    acts_host = {name: (x[rows_lo:rows_hi] if (kind == "column" and world > 1) else x).cpu().pin_memory()
                 for name, _, _, kind, x, _, _ in tp.layers}
    outs_host = {}
    for name, n, k, kind, *_ in tp.layers:
        shape = (M_ROWS, n // world) if kind == "column" else (rows_hi - rows_lo, n)
        outs_host[name] = torch.empty(shape, dtype=torch.bfloat16).pin_memory()
    h2d = sum(x.numel() * x.element_size() for x in acts_host.values())
    d2h = sum(x.numel() * x.element_size() for x in outs_host.values())
    main_s = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    dev_in = {name: [torch.empty(acts_host[name].shape, dtype=x.dtype, device=device) for _ in range(2)]
              for name, _, _, _, x, _, _ in tp.layers}
    gathered = {name: torch.empty_like(x) for name, _, _, kind, x, _, _ in tp.layers if kind == "column" and world > 1}
    consumed = {name: [None, None] for name, *_ in tp.layers}
    copied_out = {name: None for name, *_ in tp.layers}
    step_no = [0]

    def e2e_step():
        b = step_no[0] & 1
        step_no[0] += 1
        last = None
        for name, n, k, kind, x, wq, ws in tp.layers:
            buf = dev_in[name][b]
            with torch.cuda.stream(s_in):
                if consumed[name][b] is not None:
                    s_in.wait_event(consumed[name][b])
                buf.copy_(acts_host[name], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(s_in)
            main_s.wait_event(arrived)
            if name in gathered:
                torch.distributed.all_gather_into_tensor(gathered[name], buf)
                buf = gathered[name]
            q, sc = S.per_token_group_quant_fp8(buf, 128, column_major_scales=True)
            if kind == "row" and world > 1:
                # the summed result is a view of the symmetric buffer, rewritten by this layer's next call:
                # the previous pass's copy to the host must have read it first
                if copied_out[name] is not None:
                    main_s.wait_event(copied_out[name])
                out, _ = tp.peer_for(name, n).linear(q, sc, wq, ws)
                part = out[rows_lo:rows_hi]
            else:
                out = S.w8a8_block_fp8_matmul(q, wq, sc, ws, [128, 128], torch.bfloat16)
                part = out
            done = torch.cuda.Event()
            done.record(main_s)
            consumed[name][b] = done
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                outs_host[name].copy_(part, non_blocking=True)
                if not (kind == "row" and world > 1):
                    out.record_stream(s_out)
                last = torch.cuda.Event()
                last.record(s_out)
                copied_out[name] = last
        return last

    barrier(world)
    for _ in range(2):
        e2e_step()
    torch.cuda.synchronize()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(3, min(args.steps, 10))
    e0.record()
    for _ in range(e2e_steps):
        last = e2e_step()
    main_s.wait_event(last)  # the timed region ends when the last result is in host memory
    e1.record()
    barrier(world)
    e2e_ms = dist_max(e0.elapsed_time(e1) / e2e_steps, world, device)
    e2e_ok = device_status_clear(world, device)
    # the copied-back bytes are the checked ones: compare what landed in host memory with the device result
    e2e = {"value": M_ROWS * FLOPS_PER_ROW / e2e_ms / 1e9, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d * world,
           "d2h_bytes_per_step": d2h * world, "ms_per_step": e2e_ms, "steps": e2e_steps, "passes_per_step": 1,
           "device_status_clear": e2e_ok,
           "overlap": "H2D, kernels and D2H of consecutive layers run on three streams; every copy is inside the timed region"
                      + ("; a column-parallel layer's input is copied once over the group (1/p of its rows per rank) and all-gathered over NVLink" if world > 1 else "")}
    del dev_in, acts_host, outs_host

    line = {
        "metric": "block-FP8 GEMM TFLOPS", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp8_e4m3 x fp8_e4m3 -> fp32 accumulate, bf16 out", "data": "synthetic",
        "config": {"workload": WORKLOAD, "rows": M_ROWS, "block_shape": [128, 128], "inner_repeats": inner,
                   "timed_region_s": ms_step * args.steps / 1e3,
                   "l2": "per-pass working set per GPU (weights %.0f MB + activations + outputs) > 126 MB L2"
                         % (sum(wq.numel() for *_, wq, _ in tp.layers) / 1e6),
                   "parallelism": f"tp{world}" if world > 1 else "single GPU (un-sharded)",
                   "allreduce": "fused with the GEMM over NVLink peer memory (fan-out epilogue + finishing kernel)" if world > 1 else "none"},
        "parity": parity, "clocks": clk, "e2e": e2e,
        # per pass: 4 quantiser + 4 GEMM launches; on N > 1 each row-parallel layer adds its finishing kernel
        # (and, two-shot, the kernel that waits for the owners' results)
        "gpu_launches": args.steps * inner * (2 * len(TP_LINEARS) + (0 if world == 1 else 2 * (2 if world > 2 else 1))),
        "roofline": roofline,
    }
    torch.cuda.empty_cache()
    if not args.no_extras:
        try:
            parallel = {}
            if world > 1:
                parallel.update(bench_tp_items(tp, world, device, steps=6, fp8_peak=fp8_sus))
            del tp
            torch.cuda.empty_cache()
            if world > 1:
                parallel.update(bench_moe_parallel(S, device, rank, world, steps=6, fp8_peak=fp8_sus))
                line["parallel"] = parallel
        except Exception as e:  # the headline number stands without the extra line items
            line["parallel"] = {"error": repr(e)[:500]}
            torch.cuda.synchronize()
        if world == 1:
            for key, fn in (("llama8b_linears", lambda: bench_llama8b(S, device, fp8_burst)),
                            ("comparators", lambda: bench_comparators(S, device)),
                            ("moe", lambda: bench_moe(S, device, steps=5, fp8_peak=fp8_sus)),
                            ("kernels", lambda: bench_kernels(S, device))):
                try:
                    line[key] = fn()
                except Exception as e:  # the headline number stands without the extra line items
                    line[key] = {"error": repr(e)[:500]}
                    torch.cuda.synchronize()
                    torch.cuda.empty_cache()
            line["cpu_baseline"] = time_cpu_baseline()
    if stdout_fd is not None:
        sys.stdout.flush()
        os.dup2(stdout_fd, 1)
        os.close(stdout_fd)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        os.dup2(2, 1)  # whatever the teardown prints is not part of the result
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
