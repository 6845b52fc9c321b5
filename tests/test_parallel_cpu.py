"""Host logic of the tensor-/expert-parallel path on CPU: sharding arithmetic against the
oracle, and the all-to-all dispatch / combine with two gloo ranks and a stand-in expert."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as O
from conftest import make_weight


def test_column_and_row_shards_reassemble_to_the_full_linear():
    from sglang_b200 import parallel as P

    g = torch.Generator().manual_seed(0)
    x = torch.randn(8, 512, generator=g).bfloat16()
    wq, ws = make_weight(512, 512, 1)
    full = O.w8a8_block_fp8_linear(x, wq, ws, output_dtype=torch.float32)
    cols = []
    rows = torch.zeros_like(full)
    for r in range(2):
        cq, cs = P.shard_column(wq, ws, r, 2)
        cols.append(O.w8a8_block_fp8_linear(x, cq, cs, output_dtype=torch.float32))
        rq, rs = P.shard_row(wq, ws, r, 2)
        rows += O.w8a8_block_fp8_linear(x[:, r * 256 : (r + 1) * 256].contiguous(), rq, rs, output_dtype=torch.float32)
    assert torch.equal(torch.cat(cols, dim=1), full)  # column shards are exact
    assert O.rel_frobenius(rows, full) < 1e-6  # K split only reorders the fp32 sum


def test_moe_tp_and_ep_shards_sum_to_the_full_layer():
    from sglang_b200 import parallel as P

    T, E, topk, H, I = 12, 4, 2, 256, 256
    g = torch.Generator().manual_seed(2)
    x = torch.randn(T, H, generator=g).bfloat16()
    w1 = torch.stack([make_weight(2 * I, H, 10 + e)[0] for e in range(E)])
    w2 = torch.stack([make_weight(H, I, 20 + e)[0] for e in range(E)])
    w1_s = torch.rand(E, 2 * I // 128, H // 128, generator=g) * 2e-4 + 1e-4
    w2_s = torch.rand(E, H // 128, I // 128, generator=g) * 2e-4 + 1e-4
    tw, ti = O.softmax_topk(torch.randn(T, E, generator=g), topk, True)
    full = O.fused_experts_fp8(x, w1, w2, w1_s, w2_s, tw, ti)
    tp = sum(O.fused_experts_fp8(x, *P.shard_moe_tp(w1, w2, w1_s, w2_s, r, 2), tw, ti) for r in range(2))
    ep = sum(
        O.fused_experts_fp8(x, *P.shard_moe_ep(w1, w2, w1_s, w2_s, r, 2), tw, P.local_expert_ids(ti, E, 2, r))
        for r in range(2)
    )
    assert O.rel_frobenius(ep, full) < 1e-6
    # splitting I changes the 1x128 groups' partners in the down GEMM only through fp32 order
    assert O.rel_frobenius(tp, full) < 1e-6
    assert torch.equal(P.local_expert_ids(ti, E, 2, 1), O.ep_local_expert_ids(ti, E, 2, 1))


def test_dispatch_layout_sends_each_token_once_per_owning_rank():
    from sglang_b200.parallel import dispatch_layout

    ids = torch.tensor([[0, 1], [0, 5], [6, 7], [-1, 4]], dtype=torch.int32)
    send_token, counts = dispatch_layout(ids, 8, 2)
    assert counts.tolist() == [2, 3]
    assert send_token.tolist() == [0, 1, 1, 2, 3]


def _a2a_worker(rank, world, port, results):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from sglang_b200 import parallel as P

        E, topk, H, T = 8, 3, 256, 5 + 2 * rank  # ragged: ranks hold different token counts
        g = torch.Generator().manual_seed(100 + rank)
        x = torch.randn(T, H, generator=g).bfloat16()
        tw, ti = O.softmax_topk(torch.randn(T, E, generator=g), topk, True)
        if rank == 1:
            ti[0, :] = -1  # a token routed nowhere
        dummy = torch.zeros(E, 1, 1)

        def expert_fn(q, s, w1, w2, w1s, w2s, w, ids, out_dtype):
            # stand-in for the grouped GEMMs: sum_j w_j * (global expert id + 1) * dequant(row)
            deq = q.float() * s.repeat_interleave(128, dim=1)
            lo = dist.get_rank() * (E // world)
            coef = torch.where(ids >= 0, w * (ids + lo + 1).float(), torch.zeros_like(w)).sum(dim=1, keepdim=True)
            return (deq * coef).to(out_dtype)

        layer = P.FusedMoE(dummy.expand(E, 1, 1), dummy.expand(E, 1, 1), dummy.expand(E, 1, 1), dummy.expand(E, 1, 1),
                           rank, world, mode="ep_a2a", expert_fn=expert_fn)
        layer._quant_fn = lambda t: O.per_token_group_quant_fp8(t, 128)
        out = layer(x, tw, ti)
        q, s = O.per_token_group_quant_fp8(x, 128)
        deq = q.float() * s.repeat_interleave(128, dim=1)
        coef = torch.where(ti >= 0, tw * (ti + 1).float(), torch.zeros_like(tw))
        # per destination rank the partial is rounded to bf16 before the fp32 sum
        expect = torch.zeros(T, H)
        for r in range(world):
            own = (ti >= r * (E // world)) & (ti < (r + 1) * (E // world))
            expect += (deq * torch.where(own, coef, torch.zeros_like(coef)).sum(dim=1, keepdim=True)).bfloat16().float()
        ok = torch.allclose(out.float(), expect.bfloat16().float(), rtol=1e-2, atol=1e-3)
        results[rank] = bool(ok) and out.shape == (T, H)
    finally:
        dist.destroy_process_group()


def test_all_to_all_dispatch_combine_two_gloo_ranks():
    port = 29500 + os.getpid() % 2000
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_a2a_worker, args=(2, port, results), nprocs=2, join=True)
        assert dict(results) == {0: True, 1: True}


def _ar_worker(rank, world, port, results):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from sglang_b200 import parallel as P

        x = torch.full((4, 8), float(rank + 1))
        P.tensor_model_parallel_all_reduce(x)
        results[rank] = bool((x == 3).all())
    finally:
        dist.destroy_process_group()


def test_all_reduce_two_gloo_ranks():
    port = 31500 + os.getpid() % 2000
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_ar_worker, args=(2, port, results), nprocs=2, join=True)
        assert dict(results) == {0: True, 1: True}
