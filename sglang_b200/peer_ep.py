"""Expert-parallel MoE whose token exchange runs over NVLink peer memory with this package's own
kernels: no library collective, no counts to exchange, no host synchronisation.

Every rank holds a receive area indexed by (source rank, source token position) in
``torch.distributed._symmetric_memory`` (PyTorch only hands out the peer pointers). A call is

  quantise local tokens -> ``b200_ep_dispatch`` (peer stores of FP8 rows + scales + weights +
  rebased ids into the owners' areas) -> handshake -> ``fused_experts`` over all p*T_max
  positions (unfilled positions carry ids -1 and cost nothing past the alignment step), writing
  into this rank's output area -> handshake -> ``b200_ep_combine`` (peer loads of the partial
  rows from the owners' output areas, fp32 sum at the source).

With ``experts_scatter`` (what ``parallel.FusedMoE`` passes) the combine is a push fused into the owners'
down GEMM: its epilogue sends every finished (token, slot) row straight into the SOURCE rank's inbox
``[T_max * topk, H]`` while the remaining tiles are still being multiplied, and after the second handshake the
source sums its slots locally -- the combine traffic overlaps the GEMM instead of following it (at 8 ranks the
pull cost 0.15 ms after a 0.06 ms pre-reduction on the owner).

It replaces the DeepEP normal-mode dispatch / combine the reference uses for this exchange
(python/sglang/srt/layers/moe/token_dispatcher/deepep.py:507-602).

Buffer reuse needs no double buffering: a rank starts the dispatch of call n+1 only after its
combine of call n, i.e. after the second handshake of call n, which every owner enters after its
experts of call n have finished reading the receive area; and an owner starts writing outputs of
call n+1 only after the first handshake of call n+1, which every source enters after its combine
of call n. The same holds for the inbox of the push form: owners write it in their down GEMM of call
n+1, i.e. after the first handshake of call n+1, which the source enters after its slot sum of call n."""
from __future__ import annotations

import ctypes
from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import _native as N
from .fp8_kernel import fp8_dtype, per_token_group_quant_fp8


class PeerExpertParallel:
    def __init__(self, max_tokens: int, hidden: int, topk: int, num_experts: int,
                 dtype: torch.dtype = torch.bfloat16, group=None, graph_safe: bool = False):
        """``graph_safe``: epochs live on the device (advanced by the handshake kernels), so a
        captured ``forward`` can be replayed from a CUDA graph."""
        import torch.distributed._symmetric_memory as symm

        assert dist.is_initialized(), "torch.distributed must be initialised (one process per GPU, NCCL)"
        assert dtype in (torch.bfloat16, torch.float16) and hidden % 128 == 0
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        assert self.world <= 8 and num_experts % self.world == 0
        self.T_max, self.H, self.k, self.E, self.dtype = max_tokens, hidden, topk, num_experts, dtype
        pos = self.world * max_tokens  # positions of a receive area
        self.positions = pos

        def up(x):
            return (x + 255) // 256 * 256

        self.off_q = 0
        self.off_s = up(self.off_q + pos * hidden)
        self.off_w = up(self.off_s + pos * (hidden // 128) * 4)
        self.off_ids = up(self.off_w + pos * topk * 4)
        self.off_out = up(self.off_ids + pos * topk * 4)
        self.off_inbox = up(self.off_out + pos * hidden * 2)  # [T_max * topk, H]: rows pushed by the owners
        self.off_flags = up(self.off_inbox + max_tokens * topk * hidden * 2)
        total = self.off_flags + 256
        dev = torch.device("cuda", torch.cuda.current_device())
        self.buf = symm.empty(total, dtype=torch.uint8, device=dev)
        self.handle = symm.rendezvous(self.buf, self.group)
        self.base = [int(p) for p in self.handle.buffer_ptrs]
        self.buf[self.off_flags:].zero_()
        self.buf[self.off_ids : self.off_ids + pos * topk * 4].view(torch.int32).fill_(-1)
        torch.cuda.synchronize(dev)
        dist.barrier(self.group)
        self.epoch = 0
        self.graph_safe = graph_safe
        arr = ctypes.c_void_p * self.world
        self._recv_q = arr(*[b + self.off_q for b in self.base])
        self._recv_s = arr(*[b + self.off_s for b in self.base])
        self._recv_w = arr(*[b + self.off_w for b in self.base])
        self._recv_ids = arr(*[b + self.off_ids for b in self.base])
        self._peer_out = arr(*[b + self.off_out for b in self.base])
        self._peer_flags = arr(*[b + self.off_flags for b in self.base])
        self._peer_inbox = arr(*[b + self.off_inbox for b in self.base])
        # this rank's areas as tensors
        b = self.buf
        self.q = b[self.off_q : self.off_q + pos * hidden].view(fp8_dtype).view(pos, hidden)
        self.s = b[self.off_s : self.off_s + pos * (hidden // 128) * 4].view(torch.float32).view(pos, hidden // 128)
        self.w = b[self.off_w : self.off_w + pos * topk * 4].view(torch.float32).view(pos, topk)
        self.ids = b[self.off_ids : self.off_ids + pos * topk * 4].view(torch.int32).view(pos, topk)
        self.out = b[self.off_out : self.off_out + pos * hidden * 2].view(dtype).view(pos, hidden)
        self.inbox = b[self.off_inbox : self.off_inbox + max_tokens * topk * hidden * 2].view(dtype).view(max_tokens, topk, hidden)

    def _handshake(self, phase: int, stream: int) -> None:
        st = N.load().b200_peer_handshake(self.base[self.rank] + self.off_flags, self._peer_flags, self.world, self.rank,
                                          phase, 0 if self.graph_safe else self.epoch & 0xFFFFFFFF, stream)
        N.check(st, "peer_handshake")

    def check_status(self) -> None:
        """Synchronise the current stream and raise if a handshake of an earlier ``forward`` gave up. The
        kernels never hang: on expiry they set the device status word and the combine step fills its result
        with NaNs, so the failure is visible in the outputs even without this call; poll it at a cadence of
        your choice (once per model step, say) to turn it into an exception."""
        status = N.read_device_status()
        if status != 0:
            raise RuntimeError(f"peer expert-parallel exchange: device status {status}: a bounded device-side wait for "
                               "another GPU ran out; results since the last check are invalid (filled with NaN)")

    def forward(self, hidden_states: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                experts: Optional[Callable[[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor], None]],
                experts_scatter: Optional[Callable] = None):
        """``hidden_states [T, H]`` (T <= max_tokens) local tokens with GLOBAL ``topk_ids``;
        ``experts(q, s, w, local_ids, out)`` runs this rank's experts over the receive area and
        writes ``out`` (combine by pull), or ``experts_scatter(q, s, w, local_ids, dest_ptrs, rows_per_dest)``
        runs them and sends every (token, slot) row to its source rank's inbox (combine by push, taken when
        given). Returns ``[T, H]``."""
        N.require_cuda(hidden_states, topk_weights, topk_ids)
        T, H = hidden_states.shape
        assert H == self.H and T <= self.T_max and topk_ids.shape == (T, self.k), "sized for other shapes"
        lib = N.load()
        x_q, x_s = per_token_group_quant_fp8(hidden_states, 128)
        tw = topk_weights.to(torch.float32).contiguous()
        ti = topk_ids.to(torch.int32).contiguous()
        result = torch.empty(T, H, dtype=self.dtype, device=hidden_states.device)
        self.epoch += 1
        with N.on_device(hidden_states):
            stream = N.current_stream()
            st = lib.b200_ep_dispatch(N.ptr(x_q), N.ptr(x_s), N.ptr(tw), N.ptr(ti), T, self.T_max, self.k, H, self.E,
                                      self.world, self.rank, self._recv_q, self._recv_s, self._recv_w, self._recv_ids,
                                      stream)
            N.check(st, "ep_dispatch")
            self._handshake(0, stream)
            if experts_scatter is not None:
                # position s * T_max + t, slot j -> pair (s * T_max + t) * k + j: inbox of rank s, row t * k + j
                experts_scatter(self.q, self.s, self.w, self.ids, self._peer_inbox, self.T_max * self.k)
                self._handshake(1, stream)
                from .fused_moe import moe_sum_reduce

                moe_sum_reduce(self.inbox[:T], ti, result, self.E, poison_on_status=True)
                return result
            experts(self.q, self.s, self.w, self.ids, self.out)
            self._handshake(1, stream)
            st = lib.b200_ep_combine(self._peer_out, N.ptr(ti), N.ptr(result), N.DTYPE_CODE[self.dtype], T, self.T_max,
                                     self.k, H, self.E, self.world, self.rank, stream)
            N.check(st, "ep_combine")
        return result
