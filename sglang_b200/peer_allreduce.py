"""Row-parallel block-FP8 linear whose all-reduce runs over NVLink peer memory, fused with the
GEMM: the GEMM's epilogue stores every finished tile of this rank's partial output straight into
the other ranks' memory while the GEMM is still computing, and one finishing kernel sums the
partials (optionally + residual + RMSNorm). It replaces the GEMM -> ``tensor_model_parallel_all_reduce``
sequence of the reference (python/sglang/srt/layers/linear.py:1543-1558) and its fused
all-reduce + residual + RMSNorm (python/sglang/srt/layers/flashinfer_comm_fusion.py).

Buffers live in ``torch.distributed._symmetric_memory`` (one allocation per rank, every rank's
allocation mapped into every process): PyTorch is the plumbing that hands out the peer pointers;
all data movement and the handshakes are this package's kernels.

Modes
* one-shot (default for 2 ranks): every rank sends its whole partial to every rank; each rank sums
  all slots itself. NVLink egress per rank: (p-1) * M*N elements; one handshake.
* two-shot (default for more ranks): the 128-row block ``mt`` is owned by rank ``mt % p``; partial
  tiles go to their owner only, the owner sums them and writes the result into every rank's
  output. Egress per rank: 2 * (p-1)/p * M*N elements; two handshakes.

Buffer reuse: slot buffers are double-buffered by call parity. A rank can only start the GEMM of
call n+2 after the handshake of call n+1, which every peer enters after it has finished reading
call n's slots, so a buffer is never overwritten while a peer still reads it. The output buffers of
the two-shot mode (result and residual) are returned as views; the next call on the same object
rewrites them.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import _native as N
from .fp8_kernel import _workspace, fp8_dtype, per_token_group_quant_fp8

MAX_RANKS = 8


class PeerAllReduce:
    """Symmetric buffers + epoch state for fused GEMM / all-reduce calls of up to ``max_tokens``
    rows and exactly ``n`` columns, dtype bf16 or fp16."""

    def __init__(self, max_tokens: int, n: int, dtype: torch.dtype = torch.bfloat16, group=None,
                 two_shot: Optional[bool] = None, graph_safe: bool = False, multicast: Optional[bool] = None):
        """``graph_safe``: calls can be captured in a CUDA graph and replayed. Epochs then live on
        the device (advanced by the kernels), one slot buffer is used instead of two, and the
        one-shot mode ends with a second handshake ("I have read my slots") that orders the reuse.
        ``multicast`` (two-shot only; default off; needs an allocation
        with an NVSwitch multicast mapping): the owner of a row block writes its result once to the
        multicast address
        (``multimem.st``) and the switch replicates it into every rank's output, instead of one peer
        store per rank."""
        import torch.distributed._symmetric_memory as symm

        assert dist.is_initialized(), "torch.distributed must be initialised (one process per GPU, NCCL)"
        assert dtype in (torch.bfloat16, torch.float16)
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        assert self.world <= MAX_RANKS
        self.max_tokens, self.n, self.dtype = max_tokens, n, dtype
        self.two_shot = (self.world > 2) if two_shot is None else two_shot
        self.graph_safe = graph_safe
        dev = torch.device("cuda", torch.cuda.current_device())
        self.device = dev
        esz = 2
        self.slot_elems = max_tokens * n
        slots_bytes = 2 * self.world * self.slot_elems * esz            # [parity][src rank][M][N]
        out_bytes = 2 * self.slot_elems * esz if self.two_shot else 0   # output [M][N] + residual output [M][N]
        flag_bytes = 256                                                # [2][8] uint32, padded
        self.off_out = slots_bytes
        self.off_flags = (slots_bytes + out_bytes + 255) // 256 * 256
        total = self.off_flags + flag_bytes
        self.buf = symm.empty(total, dtype=torch.uint8, device=dev)
        self.handle = symm.rendezvous(self.buf, self.group)
        self.base = [int(p) for p in self.handle.buffer_ptrs]
        mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        multicast = bool(multicast)
        self.mc_base = mc if (self.two_shot and mc and multicast) else 0
        assert not (multicast and self.two_shot and not mc), "this allocation has no multicast mapping"
        self.buf[self.off_flags:].zero_()
        torch.cuda.synchronize(dev)
        dist.barrier(self.group)  # every rank's flags are zero before anyone signals
        self.epoch = 0
        self._peer_flags = (ctypes.c_void_p * self.world)(*[b + self.off_flags for b in self.base])

    # -- addresses
    def _slot_ptr(self, owner_rank: int, parity: int, src_rank: int) -> int:
        return self.base[owner_rank] + ((parity * self.world + src_rank) * self.slot_elems) * 2

    def out_view(self, m: int, which: int = 0) -> torch.Tensor:
        off = self.off_out + which * self.slot_elems * 2
        raw = self.buf[off : off + m * self.n * 2]
        return raw.view(self.dtype).view(m, self.n)

    # -- the fused operator
    def linear(self, x_q: torch.Tensor, x_s: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor,
               residual: Optional[torch.Tensor] = None, rms_weight: Optional[torch.Tensor] = None,
               eps: float = 1e-6) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """``sum over ranks of (x_q @ weight^T with block scales)``; with ``residual`` the sum is added
        to it and returned as second result; with ``rms_weight`` the first result is the RMSNorm of
        that sum. ``x_q [M, K_local]`` FP8 with scales ``x_s [M, K_local/128]`` (any strides)."""
        N.require_cuda(x_q, x_s, weight, weight_scale)
        assert x_q.dtype == fp8_dtype and weight.dtype == fp8_dtype
        m, k = x_q.shape
        n = weight.shape[0]
        assert n == self.n and m <= self.max_tokens, f"buffers were sized for [{self.max_tokens}, {self.n}]"
        assert weight.shape[1] == k and x_q.is_contiguous() and weight.is_contiguous()
        lib = N.load()
        self.epoch += 1
        parity = 0 if self.graph_safe else self.epoch & 1
        epoch_arg = 0 if self.graph_safe else self.epoch & 0xFFFFFFFF
        code = N.DTYPE_CODE[self.dtype]
        dests = (ctypes.c_void_p * self.world)(*[self._slot_ptr(d, parity, self.rank) for d in range(self.world)])
        ws_bytes = lib.b200_w8a8_block_fp8_gemm_fanout_workspace_bytes(m, n, k)
        xs = x_s if x_s.dtype == torch.float32 else x_s.float()
        wsc = weight_scale if (weight_scale.dtype == torch.float32 and weight_scale.is_contiguous()) else weight_scale.float().contiguous()
        res_out, res_outs = None, None
        if residual is not None:
            assert residual.shape == (m, n) and residual.dtype == self.dtype and residual.is_contiguous()
            if self.two_shot:
                res_out = self.out_view(m, 1)
                off = self.off_out + self.slot_elems * 2
                res_outs = (ctypes.c_void_p * self.world)(*[b + off for b in self.base])
            else:
                res_out = torch.empty_like(residual)
                res_outs = (ctypes.c_void_p * 1)(res_out.data_ptr())
        if rms_weight is not None:
            assert rms_weight.shape == (n,) and rms_weight.dtype == self.dtype and rms_weight.is_contiguous()
        if self.two_shot:
            out = self.out_view(m)
            outs = (ctypes.c_void_p * self.world)(*[b + self.off_out for b in self.base])
        else:
            out = torch.empty(m, n, dtype=self.dtype, device=x_q.device)
            outs = (ctypes.c_void_p * 1)(out.data_ptr())
        if m == 0:
            return out, res_out
        with N.on_device(x_q):
            stream = N.current_stream()
            ws = _workspace(x_q.device, ws_bytes)
            st = lib.b200_w8a8_block_fp8_gemm_fanout(
                N.ptr(x_q), N.ptr(xs), xs.stride(0), xs.stride(1), N.ptr(weight), N.ptr(wsc), dests, self.world,
                int(self.two_shot), code, m, n, k, N.ptr(ws), ws_bytes, stream,
            )
            N.check(st, "w8a8_block_fp8_gemm_fanout")
            st = lib.b200_allreduce_finish(
                self._slot_ptr(self.rank, parity, 0), self.slot_elems, outs, code, m, n, self.world, self.rank, int(self.two_shot),
                N.ptr(residual), res_outs, N.ptr(rms_weight), float(eps), self.base[self.rank] + self.off_flags,
                self._peer_flags, epoch_arg,
                self.mc_base + self.off_out if self.mc_base else None,
                self.mc_base + self.off_out + self.slot_elems * 2 if self.mc_base else None, stream,
            )
            N.check(st, "allreduce_finish")
            if self.graph_safe and not self.two_shot:
                st = lib.b200_peer_handshake(self.base[self.rank] + self.off_flags, self._peer_flags, self.world,
                                             self.rank, 1, 0, stream)
                N.check(st, "peer_handshake")
        return out, res_out

    def check_status(self) -> None:
        """Synchronise the current stream and raise if a handshake of an earlier call gave up (a rank was
        more than the wait limit late, or gone). The kernels never hang: on expiry they set the device status
        word, fill this rank's result with NaNs and return, so a caller that cannot afford a synchronisation
        per call still sees the failure in its outputs; call this at a cadence of your choice (once per
        model step, say) to turn it into an exception."""
        status = N.read_device_status()
        if status != 0:
            raise RuntimeError(f"peer all-reduce: device status {status}: a bounded device-side wait for another GPU "
                               "ran out; results since the last check are invalid (filled with NaN)")

    def linear_bf16_input(self, x: torch.Tensor, weight, weight_scale, **kw):
        """Quantise ``x [M, K_local]`` per 1x128 group (column-major scales), then ``linear``."""
        x_q, x_s = per_token_group_quant_fp8(x, 128, column_major_scales=True)
        return self.linear(x_q, x_s, weight, weight_scale, **kw)
