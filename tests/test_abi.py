"""The C-ABI library builds, loads and exports every symbol the header declares (CPU)."""
import os
import re

from conftest import ROOT


def test_library_exports_every_declared_symbol():
    from sglang_b200 import _native

    lib = _native.load()
    header = open(os.path.join(ROOT, "include", "b200_blockfp8.h")).read()
    declared = set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_native.SIGNATURES), declared ^ set(_native.SIGNATURES)
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.b200_abi_version() == 2
    assert lib.b200_status_string(0) == b"ok"
    assert lib.b200_status_string(-5) == b"device-side wait timed out"


def test_workspace_queries_need_no_gpu():
    from sglang_b200 import _native

    lib = _native.load()
    assert lib.b200_moe_align_workspace_bytes(1024, 257) == 0
    assert lib.b200_moe_align_workspace_bytes(131072, 257) == 128 * 257 * 4
    ws = lib.b200_w8a8_block_fp8_gemm_workspace_bytes(64, 2048, 2048)  # split-K fp32 partials
    assert ws > 0 and ws % (64 * 2048 * 4) == 0 and ws // (64 * 2048 * 4) <= 16
    assert lib.b200_w8a8_block_fp8_gemm_workspace_bytes(8192, 4096, 4096) == 0
    assert lib.b200_fused_experts_fp8_workspace_bytes(16, 2, 8, 256, 128) > 0


def test_operators_refuse_cpu_tensors():
    import pytest
    import torch

    import sglang_b200 as S

    with pytest.raises(RuntimeError):
        S.per_token_group_quant_fp8(torch.zeros(2, 256, dtype=torch.bfloat16), 128)
    with pytest.raises(RuntimeError):
        S.moe_align_block_size(torch.zeros(2, 2, dtype=torch.int32), 16, 8)


def test_bad_arguments_return_status_not_crash():
    from sglang_b200 import _native

    lib = _native.load()
    st = lib.b200_per_token_group_quant_fp8(None, 0, None, None, 4, 200, 128, 2, 1, 1e-10, 0, None)
    assert st == _native.E_BAD_ARG and b"null" in lib.b200_last_error_detail()
    st = lib.b200_w8a8_block_fp8_gemm(None, None, 1, 1, None, None, None, 0, 4, 128, 128, None, 0, None)
    assert st == _native.E_BAD_ARG
    st = lib.b200_moe_align_block_size(None, 3, 10, 5000, 16, None, 0, None, 0, None, None, 1, None, 0, None)
    assert st == _native.E_UNSUPPORTED


def test_tuning_knobs_round_trip_without_a_gpu():
    """The knobs are host-side state: settable, readable and restored without any launch."""
    from ctypes import byref, c_long

    from sglang_b200 import _native as N

    lib = N.load()
    v = c_long(0)
    assert lib.b200_get_tuning(b"gemm_bn", byref(v)) == 0 and v.value == -1
    with N.tuning(gemm_bn=128, peer_wait_ms=100):
        assert lib.b200_get_tuning(b"gemm_bn", byref(v)) == 0 and v.value == 128
        assert lib.b200_get_tuning(b"peer_wait_ms", byref(v)) == 0 and v.value == 100
    assert lib.b200_get_tuning(b"gemm_bn", byref(v)) == 0 and v.value == -1
    assert lib.b200_set_tuning(b"no_such_knob", 1) == N.E_BAD_ARG
    # a forced K split is reflected in the workspace the library asks for
    plain = lib.b200_w8a8_block_fp8_gemm_workspace_bytes(4096, 4096, 4096)
    with N.tuning(gemm_splitk=4):
        assert lib.b200_w8a8_block_fp8_gemm_workspace_bytes(4096, 4096, 4096) == 4 * 4096 * 4096 * 4
    assert lib.b200_w8a8_block_fp8_gemm_workspace_bytes(4096, 4096, 4096) == plain
