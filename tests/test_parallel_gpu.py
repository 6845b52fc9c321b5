"""Tensor-/expert-parallel path on 2 GPUs (NCCL): every mode against the full-layer oracle."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as O
from conftest import make_activation, make_weight

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    res = {}
    try:
        from sglang_b200 import _native
        from sglang_b200 import parallel as P

        # ---- linears: column-parallel then row-parallel (Llama-70B-like, reduced)
        x = make_activation(96, 1024, 1)
        wq1, ws1 = make_weight(2048, 1024, 2)
        wq2, ws2 = make_weight(1024, 2048, 3)
        col = P.ColumnParallelLinear(wq1.cuda(), ws1.cuda(), rank, world)
        row = P.RowParallelLinear(wq2.cuda(), ws2.cuda(), rank, world)
        h = col(x.cuda())
        y = row(h)
        h_ref = O.w8a8_block_fp8_linear(x, wq1, ws1, output_dtype=torch.bfloat16)
        n = 2048 // world
        res["col"] = O.rel_frobenius(h.float().cpu(), h_ref[:, rank * n : (rank + 1) * n].float())
        y_ref = O.w8a8_block_fp8_linear(h_ref, wq2, ws2, output_dtype=torch.float32)
        res["row"] = O.rel_frobenius(y.float().cpu(), y_ref)
        colg = P.ColumnParallelLinear(wq1.cuda(), ws1.cuda(), rank, world, gather_output=True)
        res["col_gather"] = O.rel_frobenius(colg(x.cuda()).float().cpu(), h_ref.float())

        # ---- MoE: TP over I, standard EP, all-to-all EP
        # the intermediate size must split into whole 128-wide blocks per rank, the experts into whole experts
        T, E, topk, H, I = 64, 8, 2, 512, max(512, 128 * world)
        g = torch.Generator().manual_seed(7)
        xm = torch.randn(T, H, generator=g).bfloat16()
        w1 = torch.stack([make_weight(2 * I, H, 10 + e)[0] for e in range(E)])
        w2 = torch.stack([make_weight(H, I, 30 + e)[0] for e in range(E)])
        w1_s = torch.rand(E, 2 * I // 128, H // 128, generator=g) * 2e-4 + 1e-4
        w2_s = torch.rand(E, H // 128, I // 128, generator=g) * 2e-4 + 1e-4
        tw, ti = O.softmax_topk(torch.randn(T, E, generator=g), topk, True)
        ref = O.fused_experts_fp8(xm, w1, w2, w1_s, w2_s, tw, ti)
        dev = [t.cuda() for t in (w1, w2, w1_s, w2_s)]
        for mode in ("tp", "ep"):
            out = P.FusedMoE(*dev, rank, world, mode=mode)(xm.cuda(), tw.cuda(), ti.cuda())
            res[mode] = O.rel_frobenius(out.float().cpu(), ref)
        per = T // world
        sl = slice(rank * per, (rank + 1) * per)
        out = P.FusedMoE(*dev, rank, world, mode="ep_a2a")(xm[sl].cuda(), tw[sl].cuda(), ti[sl].cuda())
        res["ep_a2a"] = O.rel_frobenius(out.float().cpu(), ref[sl])
        # dispatch / combine by the package's own kernels over peer memory; several calls with
        # different token counts reuse the same areas
        peer = P.FusedMoE(*dev, rank, world, mode="ep_peer", max_tokens=per + 3)
        outs = []
        dist.barrier()  # ranks enter the handshakes together (their wait limit is 2 s)
        for rep, cnt in enumerate([per, per - 5, per]):
            sl = slice(rank * per, rank * per + cnt)
            outs.append((sl, peer(xm[sl].cuda(), tw[sl].cuda(), ti[sl].cuda()).clone()))
        for rep, (sl, out) in enumerate(outs):
            res[f"ep_peer_{rep}"] = O.rel_frobenius(out.float().cpu(), ref[sl])
        # the pull form of the combine (owner pre-reduces, source pulls with peer loads)
        pull = P.FusedMoE(*dev, rank, world, mode="ep_peer", max_tokens=per + 3, peer_combine="pull")
        dist.barrier()
        sl = slice(rank * per, rank * per + per - 2)
        out = pull(xm[sl].cuda(), tw[sl].cuda(), ti[sl].cuda())
        res["ep_peer_pull"] = O.rel_frobenius(out.float().cpu(), ref[sl])
        res["status"] = _native.read_device_status()
        results[rank] = res
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_and_ep_ranks(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = 33500 + os.getpid() % 2000 + world
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        results = dict(results)
    assert set(results) == set(range(world))
    for r, res in results.items():
        assert res.pop("status") == 0
        for k, v in res.items():
            assert v < TOL, (r, k, v)
