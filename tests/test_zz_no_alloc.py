"""The workspace-free align entry point (for callers that cannot allocate device memory)
must give exactly what the regular entry point gives. Collected last on purpose."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _align(entry, ids, block, buckets):
    """Call one of the two C-ABI entry points directly and return its four outputs."""
    from sglang_b200 import _native as N

    lib = N.load()
    numel = ids.numel()
    max_pad = numel * block if numel < buckets else numel + buckets * (block - 1)
    max_blocks = (max_pad + block - 1) // block
    dev = ids.device
    sorted_ids = torch.full((max_pad,), -7, dtype=torch.int32, device=dev)
    expert_ids = torch.full((max_blocks,), -7, dtype=torch.int32, device=dev)
    npp = torch.full((1,), -7, dtype=torch.int32, device=dev)
    cumsum = torch.full((buckets + 1,), -7, dtype=torch.int32, device=dev)
    stream = N.current_stream()
    if entry == "static":
        st = lib.b200_moe_align_block_size_static(
            N.ptr(ids), N.DTYPE_CODE[ids.dtype], numel, buckets, block, N.ptr(sorted_ids), max_pad, N.ptr(expert_ids),
            max_blocks, N.ptr(npp), N.ptr(cumsum), stream)
    else:
        ws_bytes = lib.b200_moe_align_workspace_bytes(numel, buckets)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
        st = lib.b200_moe_align_block_size(
            N.ptr(ids), N.DTYPE_CODE[ids.dtype], numel, buckets, block, N.ptr(sorted_ids), max_pad, N.ptr(expert_ids),
            max_blocks, N.ptr(npp), N.ptr(cumsum), 1, N.ptr(ws), ws_bytes, stream)
    N.check(st, f"align ({entry})")
    torch.cuda.synchronize()
    return sorted_ids, expert_ids, npp, cumsum


def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row():
    g = torch.Generator().manual_seed(0)
    # two calls in a row that share the built-in scratch: a large multi-block case, then a
    # smaller one with another bucket count, so stale contents of the first would show
    cases = [(131072, 257, 128, torch.int32), (5000, 33, 64, torch.int64), (131072, 257, 128, torch.int32)]
    for numel, buckets, block, dt in cases:
        ids = torch.randint(-1, buckets - 1, (numel,), generator=g).to(dt).cuda()
        got = _align("static", ids, block, buckets)
        want = _align("workspace", ids, block, buckets)
        for a, b in zip(got, want):
            assert torch.equal(a, b)


def test_static_scratch_entry_rejects_sizes_beyond_its_limit():
    from sglang_b200 import _native as N

    lib = N.load()
    ids = torch.zeros(8, dtype=torch.int32, device="cuda")
    out = torch.zeros(64, dtype=torch.int32, device="cuda")
    st = lib.b200_moe_align_block_size_static(N.ptr(ids), N.I32, 131073, 9, 16, N.ptr(out), 64, N.ptr(out), 4, N.ptr(out),
                                              N.ptr(out), N.current_stream())
    assert st == N.E_UNSUPPORTED and b"limits" in lib.b200_last_error_detail()
    st = lib.b200_moe_align_block_size_static(N.ptr(ids), N.I32, 8, 258, 16, N.ptr(out), 64, N.ptr(out), 4, N.ptr(out),
                                              N.ptr(out), N.current_stream())
    assert st == N.E_UNSUPPORTED
