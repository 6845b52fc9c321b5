"""moe_align_block_size on the GPU vs the oracle: every output bit-exact."""
import pytest
import torch

import oracle as O
from conftest import load_golden

pytestmark = pytest.mark.gpu


def _check(ids_cpu, block, E):
    import sglang_b200 as S

    s, e, n = S.moe_align_block_size(ids_cpu.cuda(), block, E)
    rs, re, rn, rc = O.moe_align_block_size(ids_cpu, block, E)
    assert n.item() == rn.item()
    assert torch.equal(s.cpu(), rs)
    assert torch.equal(e.cpu(), re)


def test_docstring_example():
    import sglang_b200 as S

    c = load_golden("align.npz")["doc"]
    ids = torch.from_numpy(c["topk_ids"])
    s, e, n = S.moe_align_block_size(ids.cuda(), 4, 4)
    assert n.item() == 16 and s[:16].cpu().tolist() == c["sorted_ids"].tolist()
    assert e[:4].cpu().tolist() == [0, 1, 2, 3]


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
@pytest.mark.parametrize("block", [16, 64, 128])
@pytest.mark.parametrize(
    "T,topk,E", [(1, 2, 8), (1, 8, 256), (64, 2, 8), (128, 8, 256), (129, 8, 256), (1024, 2, 8), (2048, 8, 256),
                 (4096, 6, 160), (333, 3, 257), (16384, 8, 256), (700, 4, 1024)]
)
def test_random_routing(T, topk, E, block, dtype):
    g = torch.Generator().manual_seed(T * 31 + E)
    ids = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(min(T, 512))])
    if T > 512:
        ids = ids.repeat((T + 511) // 512, 1)[:T]
        ids = (ids + torch.arange(T).view(-1, 1)) % E
    _check(ids.to(dtype), block, E)


def test_expert_parallel_minus_one_and_skew():
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 256, (5000, 8), generator=g, dtype=torch.int32)
    local = O.ep_local_expert_ids(ids, 256, 8, 3)
    _check(local, 128, 32)
    _check(torch.full((3000, 2), 5, dtype=torch.int32), 64, 8)  # every token to one expert
    _check(torch.full((100, 2), -1, dtype=torch.int32), 64, 8)  # nothing local


def test_cumsum_and_raw_form():
    import sglang_b200 as S

    g = torch.Generator().manual_seed(2)
    ids = torch.randint(-1, 16, (3000,), generator=g, dtype=torch.int32)
    max_pad, max_blocks = O.moe_align_sizes(3000, 32, 16)
    s = torch.empty(max_pad, dtype=torch.int32, device="cuda")
    e = torch.empty(max_blocks, dtype=torch.int32, device="cuda")
    n = torch.empty(1, dtype=torch.int32, device="cuda")
    c = torch.empty(18, dtype=torch.int32, device="cuda")
    S.sgl_moe_align_block_size(ids.cuda(), 17, 32, s, e, n, c, True)
    rs, re, rn, rc = O.moe_align_block_size(ids.view(-1, 1), 32, 16)
    assert torch.equal(s.cpu(), rs) and torch.equal(e.cpu(), re) and torch.equal(c.cpu(), rc)


def test_empty_input():
    import sglang_b200 as S

    s, e, n = S.moe_align_block_size(torch.empty(0, 2, dtype=torch.int32, device="cuda"), 64, 8)
    assert n.item() == 0 and s.numel() == 0
