"""ctypes binding of the C ABI declared in ``include/b200_blockfp8.h``.

The shared library is the only implementation: if it is missing it is built in-tree with
nvcc, and if that fails the import error propagates. There is no CPU or torch fallback.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_long, c_size_t, c_uint32, c_void_p, POINTER

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
# SGLANG_B200_LIB points at another build of the same library (e.g. one compiled with tuning macros)
LIB_PATH = os.environ.get("SGLANG_B200_LIB") or os.path.join(_PKG, "_lib", "libb200_blockfp8.so")

# Every symbol the header declares: name -> (restype, argtypes)
SIGNATURES = {
    "b200_status_string": (c_char_p, [c_int]),
    "b200_last_error_detail": (c_char_p, []),
    "b200_abi_version": (c_int, []),
    "b200_read_device_status": (c_int, [POINTER(c_int), c_void_p]),
    "b200_set_tuning": (c_int, [c_char_p, c_long]),
    "b200_get_tuning": (c_int, [c_char_p, POINTER(c_long)]),
    "b200_per_token_group_quant_fp8": (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int64, c_int64, c_float, c_int, c_void_p],
    ),
    "b200_per_token_group_quant_fp8_ue8m0": (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int64, c_int, c_void_p, c_int, c_void_p],
    ),
    "b200_w8a8_block_fp8_gemm_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "b200_w8a8_block_fp8_gemm": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64,
         c_void_p, c_size_t, c_void_p],
    ),
    "b200_w8a8_block_fp8_gemm_ue8m0": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_int, c_int64, c_int64, c_int64,
         c_void_p],
    ),
    "b200_w8a8_block_fp8_linear_decode_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "b200_w8a8_block_fp8_linear_decode": (
        c_int,
        [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_float, c_void_p, c_size_t,
         c_void_p, c_void_p],
    ),
    "b200_moe_align_workspace_bytes": (c_size_t, [c_int64, c_int]),
    "b200_moe_align_block_size": (
        c_int,
        [c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int,
         c_void_p, c_size_t, c_void_p],
    ),
    "b200_moe_align_block_size_static": (
        c_int,
        [c_void_p, c_int, c_int64, c_int, c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p],
    ),
    "b200_fused_experts_fp8_workspace_bytes": (c_size_t, [c_int64, c_int, c_int, c_int64, c_int64]),
    "b200_fused_experts_fp8": (
        c_int,
        [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
         c_int, c_int, c_int64, c_int64, c_int, c_int, c_float, c_void_p, c_size_t, c_void_p],
    ),
    "b200_w8a8_block_fp8_gemm_fanout_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64]),
    "b200_w8a8_block_fp8_gemm_fanout": (
        c_int,
        [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, POINTER(c_void_p), c_int, c_int, c_int, c_int64,
         c_int64, c_int64, c_void_p, c_size_t, c_void_p],
    ),
    "b200_allreduce_finish": (
        c_int,
        [c_void_p, c_int64, POINTER(c_void_p), c_int, c_int64, c_int64, c_int, c_int, c_int, c_void_p,
         POINTER(c_void_p), c_void_p, c_float, c_void_p, POINTER(c_void_p), c_uint32, c_void_p, c_void_p, c_void_p],
    ),
    "b200_masked_experts_fp8_workspace_bytes": (c_size_t, [c_int, c_int64, c_int64, c_int64]),
    "b200_masked_experts_fp8": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64,
         c_int64, c_void_p, c_size_t, c_void_p],
    ),
    "b200_ep_dispatch": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_int64, c_int, c_int, c_int,
         POINTER(c_void_p), POINTER(c_void_p), POINTER(c_void_p), POINTER(c_void_p), c_void_p],
    ),
    "b200_peer_handshake": (c_int, [c_void_p, POINTER(c_void_p), c_int, c_int, c_int, c_uint32, c_void_p]),
    "b200_ep_combine": (
        c_int,
        [POINTER(c_void_p), c_void_p, c_void_p, c_int, c_int64, c_int64, c_int, c_int64, c_int, c_int, c_int, c_void_p],
    ),
    "b200_fused_experts_fp8_scatter": (
        c_int,
        [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64,
         c_int64, c_int, c_int, c_int64, c_int64, c_void_p, c_size_t, c_void_p],
    ),
    "b200_moe_sum_reduce": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int64, c_float, c_int, c_int, c_void_p],
    ),
    "b200_route_topk": (
        c_int,
        [c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
         c_void_p, c_void_p, c_void_p],
    ),
    "b200_route_topk_softmax_capped": (
        c_int,
        [c_void_p, c_int, c_float, c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
    ),
}

BF16, F16, F32, I32, I64 = 0, 1, 2, 3, 4
DTYPE_CODE = {
    torch.bfloat16: BF16,
    torch.float16: F16,
    torch.float32: F32,
    torch.int32: I32,
    torch.int64: I64,
}

E_BAD_ARG, E_UNSUPPORTED, E_LAUNCH, E_WORKSPACE, E_TIMEOUT = -1, -2, -3, -4, -5

_lock = threading.Lock()
_lib = None


def load() -> ctypes.CDLL:
    """Load (building first if needed) the native library and bind every declared symbol."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if "SGLANG_B200_LIB" not in os.environ:
            # a no-op when the stamp of the last build names the current sources; otherwise (edited source,
            # missing library) it compiles, so stale kernels never run silently
            from . import build as _build

            _build.build()
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(status: int, what: str) -> None:
    """Map a C-ABI status to the reference's exception types: precondition failures raise
    AssertionError (the reference asserts in Python), everything else RuntimeError."""
    if status == 0:
        return
    lib = load()
    msg = f"{what}: {lib.b200_status_string(status).decode()}: {lib.b200_last_error_detail().decode()}"
    if status == E_BAD_ARG:
        raise AssertionError(msg)
    if status == E_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise RuntimeError(msg)


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "sglang_b200 operators run on CUDA (sm_100a) tensors only; got a tensor on "
                f"{t.device}. There is no CPU path."
            )


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def current_stream(device=None) -> int:
    """Raw cudaStream_t of torch's current stream on ``device`` (default: current device)."""
    if device is None:
        idx = torch.cuda.current_device()
    else:
        idx = device.index if isinstance(device, torch.device) else int(device)
        if idx is None:
            idx = torch.cuda.current_device()
    return torch._C._cuda_getCurrentRawStream(idx)


class on_device:
    """``with on_device(t):`` makes ``t``'s device current for the duration of a launch; a no-op
    (and allocation-free) when it already is, which is the case on every call of a
    one-process-per-GPU server."""

    __slots__ = ("idx", "prev")

    def __init__(self, t: torch.Tensor):
        self.idx = t.device.index
        self.prev = -1

    def __enter__(self):
        cur = torch.cuda.current_device()
        if self.idx is not None and self.idx != cur:
            self.prev = cur
            torch.cuda.set_device(self.idx)
        return self

    def __exit__(self, *a):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


class tuning:
    """``with tuning(gemm_bn=128, gemm_splitk=2): ...`` sets process-wide knobs of the native library
    (``b200_set_tuning``) and restores the previous values on exit. For tests and tuning sweeps."""

    def __init__(self, **knobs: int):
        self.knobs, self.prev = knobs, {}

    def __enter__(self):
        lib = load()
        for name, value in self.knobs.items():
            old = c_long(0)
            check(lib.b200_get_tuning(name.encode(), ctypes.byref(old)), "get_tuning")
            self.prev[name] = old.value
            check(lib.b200_set_tuning(name.encode(), int(value)), "set_tuning")
        return self

    def __exit__(self, *a):
        lib = load()
        for name, value in self.prev.items():
            lib.b200_set_tuning(name.encode(), value)
        return False


def get_tuning(name: str) -> int:
    v = c_long(0)
    check(load().b200_get_tuning(name.encode(), ctypes.byref(v)), "get_tuning")
    return v.value


def read_device_status() -> int:
    """Synchronise the current stream and return (and clear) the device status word."""
    out = c_int(0)
    check(load().b200_read_device_status(ctypes.byref(out), current_stream()), "read_device_status")
    return out.value
