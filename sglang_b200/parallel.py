"""Tensor- and expert-parallel partitioning of the block-FP8 path on one NVLink box: one
process per GPU, ``torch.distributed`` (NCCL) for the exchange steps.

Semantics follow the reference's callers:
* column-parallel linear: weight rows ``[r*N/p, (r+1)*N/p)``, no exchange
  (python/sglang/srt/layers/linear.py:292, forward :467-488);
* row-parallel linear: K split, each rank quantises its own K slice, bf16 partial outputs are
  summed by an all-reduce, bias on rank 0 only (linear.py:1340, forward :1520-1563);
* MoE tensor parallel: the intermediate dimension is split (gate rows and up rows of ``w1``,
  columns of ``w2``; python/sglang/srt/layers/moe/fused_moe_triton/layer.py:202-223);
* MoE expert parallel, "standard": tokens replicated, rank r owns experts
  ``[r*E/p, (r+1)*E/p)``, other ids become -1, partial outputs all-reduced
  (python/sglang/srt/layers/moe/token_dispatcher/standard.py:115-218, layer.py:1075-1100);
* MoE expert parallel, all-to-all: tokens partitioned over ranks; each token is sent ONCE to
  every rank that owns one of its experts as FP8 bytes + 1x128 scales + its ids / weights,
  the owner runs the grouped GEMMs, bf16 partial rows travel back and are summed at the source
  (the exchange DeepEP performs for the reference, token_dispatcher/deepep.py:507-602; here a
  variable-count ``all_to_all_single`` each way, counts exchanged first).

The dispatch / combine index arithmetic is plain torch on whatever device the tensors are
on, so the world_size-2 ``gloo`` tests exercise it on CPU with a stand-in expert function.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

# ------------------------------------------------------------------------- sharding


def shard_column(wq: torch.Tensor, ws: torch.Tensor, rank: int, size: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rows ``[rank*N/p, ...)`` of ``wq [N, K]`` and the matching rows of ``ws [N/128, K/128]``."""
    N = wq.shape[0]
    assert N % (128 * size) == 0, "column shards must be whole 128-row scale blocks"
    n = N // size
    return wq[rank * n : (rank + 1) * n].contiguous(), ws[rank * n // 128 : (rank + 1) * n // 128].contiguous()


def shard_row(wq: torch.Tensor, ws: torch.Tensor, rank: int, size: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Columns ``[rank*K/p, ...)`` of ``wq [N, K]`` and the matching columns of ``ws``."""
    K = wq.shape[1]
    assert K % (128 * size) == 0, "row shards must be whole 128-column scale blocks"
    k = K // size
    return wq[:, rank * k : (rank + 1) * k].contiguous(), ws[:, rank * k // 128 : (rank + 1) * k // 128].contiguous()


def shard_moe_tp(w1, w2, w1_s, w2_s, rank: int, size: int):
    """Split the intermediate size I: gate rows ``[r*I/p..)`` + up rows ``[I + r*I/p..)`` of
    ``w1 [E, 2I, H]`` and columns of ``w2 [E, H, I]``."""
    I = w2.shape[2]
    assert I % (128 * size) == 0
    i = I // size
    lo, hi = rank * i, (rank + 1) * i
    w1l = torch.cat([w1[:, lo:hi], w1[:, I + lo : I + hi]], dim=1).contiguous()
    w1sl = torch.cat([w1_s[:, lo // 128 : hi // 128], w1_s[:, (I + lo) // 128 : (I + hi) // 128]], dim=1).contiguous()
    return w1l, w2[:, :, lo:hi].contiguous(), w1sl, w2_s[:, :, lo // 128 : hi // 128].contiguous()


def shard_moe_ep(w1, w2, w1_s, w2_s, rank: int, size: int):
    """Experts ``[r*E/p, (r+1)*E/p)``."""
    E = w1.shape[0]
    assert E % size == 0
    e = E // size
    sl = slice(rank * e, (rank + 1) * e)
    return w1[sl].contiguous(), w2[sl].contiguous(), w1_s[sl].contiguous(), w2_s[sl].contiguous()


def local_expert_ids(topk_ids: torch.Tensor, num_experts: int, ep_size: int, ep_rank: int) -> torch.Tensor:
    """Global expert ids -> ids local to ``ep_rank`` (0-based), -1 for experts of other ranks."""
    per = num_experts // ep_size
    lo = ep_rank * per
    keep = (topk_ids >= lo) & (topk_ids < lo + per)
    return torch.where(keep, topk_ids - lo, torch.full_like(topk_ids, -1))


def tensor_model_parallel_all_reduce(x: torch.Tensor, group=None) -> torch.Tensor:
    """Sum over the group (python/sglang/srt/distributed/communication_op.py:18-20)."""
    if group is not None or (dist.is_initialized() and dist.get_world_size() > 1):
        dist.all_reduce(x, group=group)
    return x


# -------------------------------------------------------------------------- linears


class ColumnParallelLinear:
    """Block-FP8 linear whose output columns are split over the group."""

    def __init__(self, wq, ws, tp_rank: int, tp_size: int, bias=None, gather_output: bool = False, group=None):
        self.weight, self.weight_scale = shard_column(wq, ws, tp_rank, tp_size)
        n = wq.shape[0] // tp_size
        self.bias = None if bias is None else bias[tp_rank * n : (tp_rank + 1) * n].contiguous()
        self.gather_output, self.group, self.tp_size = gather_output, group, tp_size

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from .fp8_kernel import w8a8_block_fp8_linear

        out = w8a8_block_fp8_linear(x, self.weight, [128, 128], self.weight_scale, bias=self.bias)
        if self.gather_output and self.tp_size > 1:
            parts = [torch.empty_like(out) for _ in range(self.tp_size)]
            dist.all_gather(parts, out, group=self.group)
            out = torch.cat(parts, dim=-1)
        return out

    __call__ = forward


class RowParallelLinear:
    """Block-FP8 linear whose reduction dimension is split; partial outputs are all-reduced."""

    def __init__(self, wq, ws, tp_rank: int, tp_size: int, bias=None, reduce_results: bool = True,
                 input_is_parallel: bool = True, group=None, reduce_mode: str = "nccl", max_tokens: int = 8192):
        """``reduce_mode="peer"``: the all-reduce is fused with the GEMM over NVLink peer memory
        (see ``peer_allreduce.PeerAllReduce``; buffers sized for ``max_tokens`` rows) instead of a
        separate NCCL collective."""
        assert reduce_mode in ("nccl", "peer")
        self.weight, self.weight_scale = shard_row(wq, ws, tp_rank, tp_size)
        self.bias = bias if tp_rank == 0 else None  # added once, before the sum
        self.tp_rank, self.tp_size = tp_rank, tp_size
        self.reduce_results, self.input_is_parallel, self.group = reduce_results, input_is_parallel, group
        self.reduce_mode, self.max_tokens, self._peer = reduce_mode, max_tokens, None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from .fp8_kernel import w8a8_block_fp8_linear

        if not self.input_is_parallel:
            k = x.shape[-1] // self.tp_size
            x = x[..., self.tp_rank * k : (self.tp_rank + 1) * k].contiguous()
        if self.reduce_mode == "peer" and self.reduce_results and self.tp_size > 1 and self.bias is None:
            from .peer_allreduce import PeerAllReduce

            if self._peer is None:
                self._peer = PeerAllReduce(self.max_tokens, self.weight.shape[0], x.dtype, self.group)
            x2 = x.reshape(-1, x.shape[-1])
            out, _ = self._peer.linear_bf16_input(x2, self.weight, self.weight_scale)
            return out.view(*x.shape[:-1], self.weight.shape[0])
        out = w8a8_block_fp8_linear(x, self.weight, [128, 128], self.weight_scale, bias=self.bias)
        if self.reduce_results and self.tp_size > 1:
            out = tensor_model_parallel_all_reduce(out, self.group)
        return out

    __call__ = forward


# ----------------------------------------------------------------- all-to-all dispatch


@dataclass
class DispatchHandle:
    """What combine() needs to route partial rows back."""

    send_counts: List[int]
    recv_counts: List[int]
    send_token: torch.Tensor  # [S] local token index of every sent row (grouped by destination rank)
    num_tokens: int


def dispatch_layout(topk_ids: torch.Tensor, num_experts: int, ep_size: int):
    """For local tokens with global ``topk_ids [T, k]``: the (token, rank) pairs to send, grouped
    by destination rank, ascending token inside a rank. Returns (send_token [S], send_counts [p])."""
    per = num_experts // ep_size
    dest = torch.div(topk_ids.clamp(min=0), per, rounding_mode="floor")  # [T, k]
    valid = topk_ids >= 0
    ranks = torch.arange(ep_size, device=topk_ids.device).view(1, ep_size, 1)
    needs = ((dest.unsqueeze(1) == ranks) & valid.unsqueeze(1)).any(dim=-1)  # [T, p]
    send_counts = needs.sum(dim=0)
    # rank-major order: nonzero of the transposed mask is sorted by (rank, token)
    send_token = needs.t().nonzero(as_tuple=False)[:, 1]
    return send_token, send_counts


class AllToAllDispatcher:
    """Expert-parallel token exchange with ``dist.all_to_all_single`` and per-rank counts."""

    def __init__(self, num_experts: int, ep_rank: int, ep_size: int, group=None):
        self.num_experts, self.ep_rank, self.ep_size, self.group = num_experts, ep_rank, ep_size, group

    def _a2a(self, out: torch.Tensor, inp: torch.Tensor, out_splits, in_splits):
        dist.all_to_all_single(out, inp, output_split_sizes=out_splits, input_split_sizes=in_splits, group=self.group)

    def dispatch(self, x_q: torch.Tensor, x_s: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor):
        """``x_q [T, H]`` FP8 (or any 1-byte dtype) rows, ``x_s [T, H/128]`` fp32 scales, routing
        ``[T, k]``. Returns the rows this rank must process -- (q [R, H], s [R, H/128],
        weights [R, k], LOCAL ids [R, k] with -1 for experts of other ranks) -- and the handle."""
        T, H = x_q.shape
        k = topk_ids.shape[1]
        dev = x_q.device
        send_token, send_counts_t = dispatch_layout(topk_ids, self.num_experts, self.ep_size)
        recv_counts_t = torch.empty_like(send_counts_t)
        dist.all_to_all_single(recv_counts_t, send_counts_t, group=self.group)
        send_counts, recv_counts = send_counts_t.tolist(), recv_counts_t.tolist()  # host sync: sizes of the exchange
        # one packed row per (token, rank): FP8 bytes | scales | weights | ids
        row_bytes = H + 4 * (H // 128) + 8 * k
        row_bytes_pad = (row_bytes + 15) // 16 * 16
        S, R = int(send_token.numel()), int(sum(recv_counts))
        send = torch.empty(S, row_bytes_pad, dtype=torch.uint8, device=dev)
        send[:, :H] = x_q.view(torch.uint8)[send_token]
        send[:, H : H + 4 * (H // 128)] = x_s.contiguous().view(torch.uint8).view(T, -1)[send_token]
        o = H + 4 * (H // 128)
        send[:, o : o + 4 * k] = topk_weights.to(torch.float32).contiguous().view(torch.uint8).view(T, -1)[send_token]
        send[:, o + 4 * k : o + 8 * k] = topk_ids.to(torch.int32).contiguous().view(torch.uint8).view(T, -1)[send_token]
        recv = torch.empty(R, row_bytes_pad, dtype=torch.uint8, device=dev)
        self._a2a(recv, send, recv_counts, send_counts)
        q = recv[:, :H].contiguous().view(x_q.dtype)
        s = recv[:, H:o].contiguous().view(torch.float32)
        w = recv[:, o : o + 4 * k].contiguous().view(torch.float32)
        ids = recv[:, o + 4 * k : o + 8 * k].contiguous().view(torch.int32)
        ids = local_expert_ids(ids, self.num_experts, self.ep_size, self.ep_rank)
        return (q, s, w, ids), DispatchHandle(send_counts, recv_counts, send_token, T)

    def combine(self, partial: torch.Tensor, handle: DispatchHandle) -> torch.Tensor:
        """``partial [R, H]``: this rank's weighted expert outputs for the rows it received.
        Returns ``[T, H]``: for every local token the fp32 sum of the partial rows that came back."""
        H = partial.shape[1]
        back = torch.empty(int(sum(handle.send_counts)), H, dtype=partial.dtype, device=partial.device)
        self._a2a(back, partial.contiguous(), handle.send_counts, handle.recv_counts)
        out = torch.zeros(handle.num_tokens, H, dtype=torch.float32, device=partial.device)
        out.index_add_(0, handle.send_token, back.to(torch.float32))
        return out.to(partial.dtype)


# ------------------------------------------------------------------------------ MoE


class FusedMoE:
    """Block-FP8 MoE layer partitioned over a group.

    ``mode``: "tp" (split I, all-reduce), "ep" (standard: replicated tokens, local experts,
    all-reduce), "ep_a2a" (tokens partitioned, all-to-all dispatch / combine through
    ``all_to_all_single``), "ep_peer" (tokens partitioned, dispatch / combine by this package's
    kernels over NVLink peer memory, ``peer_ep.PeerExpertParallel``; ``max_tokens`` local tokens
    at most). ``forward`` takes the tokens this rank holds (all tokens for "tp"/"ep", its
    partition otherwise) and GLOBAL expert ids."""

    def __init__(self, w1, w2, w1_s, w2_s, rank: int, size: int, mode: str = "ep", group=None,
                 expert_fn: Optional[Callable] = None, presharded: bool = False, num_experts: Optional[int] = None,
                 max_tokens: int = 8192, peer_combine: str = "push"):
        """``presharded``: the four tensors are already this rank's shard (a loader that never
        materialises the full layer); ``num_experts`` then gives the global expert count."""
        assert mode in ("tp", "ep", "ep_a2a", "ep_peer")
        self.mode, self.rank, self.size, self.group = mode, rank, size, group
        assert peer_combine in ("push", "pull")
        self.max_tokens, self._peer, self.peer_combine = max_tokens, None, peer_combine
        if presharded:
            self.num_experts = num_experts if num_experts is not None else w1.shape[0] * (1 if mode == "tp" else size)
            self.w1, self.w2, self.w1_s, self.w2_s = w1, w2, w1_s, w2_s
        else:
            self.num_experts = w1.shape[0]
            shard = shard_moe_tp if mode == "tp" else shard_moe_ep
            self.w1, self.w2, self.w1_s, self.w2_s = shard(w1, w2, w1_s, w2_s, rank, size)
        self.dispatcher = AllToAllDispatcher(self.num_experts, rank, size, group) if mode == "ep_a2a" else None
        self._expert_fn = expert_fn  # tests on CPU inject a stand-in for the CUDA kernels

    def _experts(self, x, x_s, w, ids, out_dtype):
        if self._expert_fn is not None:
            return self._expert_fn(x, x_s, self.w1, self.w2, self.w1_s, self.w2_s, w, ids, out_dtype)
        from .fused_moe import fused_experts_impl

        return fused_experts_impl(x, self.w1, self.w2, w, ids, self.w1_s, self.w2_s, inplace=False,
                                  hidden_states_scale=x_s, output_dtype=out_dtype)

    def forward(self, hidden_states: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        if self.mode == "tp":
            out = self._experts(hidden_states, None, topk_weights, topk_ids, hidden_states.dtype)
            return tensor_model_parallel_all_reduce(out, self.group) if self.size > 1 else out
        if self.mode == "ep":
            ids = local_expert_ids(topk_ids, self.num_experts, self.size, self.rank)
            out = self._experts(hidden_states, None, topk_weights, ids, hidden_states.dtype)
            return tensor_model_parallel_all_reduce(out, self.group) if self.size > 1 else out
        if self.mode == "ep_peer":
            from .fused_moe import fused_experts_impl
            from .peer_ep import PeerExpertParallel

            if self._peer is None:
                self._peer = PeerExpertParallel(self.max_tokens, hidden_states.shape[1], topk_ids.shape[1],
                                                self.num_experts, hidden_states.dtype, self.group)

            def experts(q, s, w, ids, out):
                fused_experts_impl(q, self.w1, self.w2, w, ids, self.w1_s, self.w2_s, inplace=False,
                                   hidden_states_scale=s, output_dtype=out.dtype, out=out, skip_unrouted_rows=True)

            def experts_scatter(q, s, w, ids, dest_ptrs, rows_per_dest):
                from .fused_moe import fused_experts_scatter

                fused_experts_scatter(q, s, self.w1, self.w2, w, ids, self.w1_s, self.w2_s, dest_ptrs, rows_per_dest,
                                      hidden_states.dtype)

            return self._peer.forward(hidden_states, topk_weights, topk_ids, experts,
                                      experts_scatter if self.peer_combine == "push" else None)
        from .fp8_kernel import per_token_group_quant_fp8

        quant = getattr(self, "_quant_fn", None) or (lambda t: per_token_group_quant_fp8(t, 128))
        x_q, x_s = quant(hidden_states)
        (q, s, w, ids), handle = self.dispatcher.dispatch(x_q, x_s, topk_weights, topk_ids)
        partial = self._experts(q, s, w, ids, hidden_states.dtype)
        return self.dispatcher.combine(partial, handle)

    __call__ = forward
