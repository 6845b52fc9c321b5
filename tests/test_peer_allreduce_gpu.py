"""Row-parallel linear with the all-reduce fused over peer memory.

One GPU: the fan-out GEMM (every finished tile stored to several destination buffers, or only to
the owner of its 128-row block) must produce exactly the bytes of the plain GEMM in every kernel
path, and the finishing kernel (sum of slots + residual + RMSNorm) must match a torch fp32
restatement. Two GPUs (skipped otherwise): one-shot and two-shot against the full-layer oracle
and against the NCCL path."""
import ctypes
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as O
from conftest import make_activation, make_weight

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _quant(x):
    import sglang_b200 as S

    return S.per_token_group_quant_fp8(x.cuda(), 128, column_major_scales=True)


def _fanout(xq, xs, wq, ws, n_dest, by_tile, dtype, fill):
    from sglang_b200 import _native as N
    from sglang_b200.fp8_kernel import _workspace

    lib = N.load()
    m, k = xq.shape
    n = wq.shape[0]
    bufs = [torch.full((m, n), fill, dtype=dtype, device="cuda") for _ in range(n_dest)]
    dests = (ctypes.c_void_p * n_dest)(*[b.data_ptr() for b in bufs])
    nbytes = lib.b200_w8a8_block_fp8_gemm_fanout_workspace_bytes(m, n, k)
    wsb = _workspace(xq.device, nbytes)
    st = lib.b200_w8a8_block_fp8_gemm_fanout(
        N.ptr(xq), N.ptr(xs), xs.stride(0), xs.stride(1), N.ptr(wq), N.ptr(ws), dests, n_dest, int(by_tile),
        N.DTYPE_CODE[dtype], m, n, k, N.ptr(wsb), nbytes, N.current_stream(),
    )
    N.check(st, "fanout")
    torch.cuda.synchronize()
    assert N.read_device_status() == 0
    return bufs


@pytest.mark.parametrize("M,N,K", [(16, 1024, 512), (1, 256, 2048), (48, 512, 4096), (256, 1024, 2048),
                                   (300, 2048, 1024), (1000, 512, 256), (512, 128, 512), (384, 1032, 384)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fanout_gemm_writes_the_plain_gemm_bytes(M, N, K, dtype):
    import sglang_b200 as S

    x = make_activation(M, K, M + K, dtype=torch.bfloat16)
    wq, ws = make_weight(N, K, N + K)
    xq, xs = _quant(x)
    wq, ws = wq.cuda(), ws.cuda()
    plain = S.w8a8_block_fp8_matmul(xq, wq, xs, ws, [128, 128], dtype)
    for got in _fanout(xq, xs, wq, ws, 3, False, dtype, 7.0):
        assert torch.equal(got, plain)
    # by row block: block mt only in buffer mt % 3, everything else untouched
    bufs = _fanout(xq, xs, wq, ws, 3, True, dtype, 7.0)
    for d, got in enumerate(bufs):
        for mt in range((M + 127) // 128):
            rows = slice(mt * 128, min(M, mt * 128 + 128))
            if mt % 3 == d:
                assert torch.equal(got[rows], plain[rows]), (d, mt)
            else:
                assert torch.all(got[rows] == 7.0), (d, mt)


@pytest.mark.parametrize("M,N", [(1, 256), (37, 1024), (300, 4096)])
@pytest.mark.parametrize("mode", ["sum", "residual", "residual_norm", "norm"])
def test_finish_kernel_single_rank_sum_residual_rmsnorm(M, N, mode):
    """n_ranks = 1: the handshake is with itself, the arithmetic is the whole job."""
    from sglang_b200 import _native as N_

    lib = N_.load()
    g = torch.Generator().manual_seed(M + N)
    slot = torch.randn(M, N, generator=g).bfloat16().cuda()
    residual = torch.randn(M, N, generator=g).bfloat16().cuda() if "residual" in mode else None
    w = (torch.rand(N, generator=g) + 0.5).bfloat16().cuda() if "norm" in mode else None
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    res_out = torch.empty_like(out) if residual is not None else None
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    outs = (ctypes.c_void_p * 1)(out.data_ptr())
    peers = (ctypes.c_void_p * 1)(flags.data_ptr())
    for epoch in (1, 2, 3):  # flags persist: epochs must keep working call after call
        res_outs = (ctypes.c_void_p * 1)(res_out.data_ptr()) if res_out is not None else None
        st = lib.b200_allreduce_finish(slot.data_ptr(), M * N, outs, N_.BF16, M, N, 1, 0, 0, N_.ptr(residual),
                                       res_outs, N_.ptr(w), 1e-6, flags.data_ptr(), peers, epoch, None, None,
                                       N_.current_stream())
        N_.check(st, "finish")
    torch.cuda.synchronize()
    assert N_.read_device_status() == 0
    acc = slot.float()
    if residual is not None:
        acc = acc + residual.float()
        assert torch.equal(res_out, acc.bfloat16())
    if w is not None:
        ref = (acc * torch.rsqrt(acc.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float())
        torch.testing.assert_close(out.float(), ref, rtol=1e-2, atol=1e-2)
        assert O.rel_frobenius(out.float().cpu(), ref.cpu()) < 3e-3
    else:
        assert torch.equal(out, acc.bfloat16())


def test_device_epochs_replay_from_a_cuda_graph_single_rank():
    """epoch = 0: the kernels keep the epoch on the device, so the captured launch replays."""
    from sglang_b200 import _native as N_

    lib = N_.load()
    M, N = 64, 512
    slot = torch.randn(M, N, device="cuda").bfloat16()
    out = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    outs = (ctypes.c_void_p * 1)(out.data_ptr())
    peers = (ctypes.c_void_p * 1)(flags.data_ptr())
    s = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        def call():
            st = lib.b200_allreduce_finish(slot.data_ptr(), M * N, outs, N_.BF16, M, N, 1, 0, 0, None, None, None, 1e-6,
                                           flags.data_ptr(), peers, 0, None, None, N_.current_stream())
            N_.check(st, "finish")
            N_.check(lib.b200_peer_handshake(flags.data_ptr(), peers, 1, 0, 1, 0, N_.current_stream()), "handshake")
        call()
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=s):
            call()
            call()
    for i in range(3):
        slot.copy_(torch.randn(M, N, device="cuda").bfloat16())
        out.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, slot)
    assert N_.read_device_status() == 0
    # 1 eager + 3 replays of 2 calls = 7 epochs on both phases; the block ticket is back at zero
    assert flags[16].item() == 7 and flags[17].item() == 7 and flags[18].item() == 0
    assert flags[0].item() == 7 and flags[8].item() == 7


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    res = {}
    try:
        from sglang_b200 import _native
        from sglang_b200 import parallel as P
        from sglang_b200.peer_allreduce import PeerAllReduce

        Nn, K = 1024, 2048
        wq, ws = make_weight(Nn, K, 3)
        wl, wsl = P.shard_row(wq.cuda(), ws.cuda(), rank, world)
        kl = K // world
        g = torch.Generator().manual_seed(5)
        resid = torch.randn(512, Nn, generator=g).bfloat16()
        gamma = (torch.rand(Nn, generator=g) + 0.5).bfloat16()
        nccl = P.RowParallelLinear(wq.cuda(), ws.cuda(), rank, world)
        # All CPU-side oracle work first: ranks must not drift apart by more than the kernels'
        # wait limit (2 s) between the launches of one collective call.
        cases = []
        for rep, M in enumerate([16, 300, 512, 1, 300, 130]):  # several calls: buffer parity and epochs
            x = make_activation(M, K, 10 + rep)
            ref = O.w8a8_block_fp8_linear(x, wq, ws, output_dtype=torch.float32)
            acc = ref + resid[:M].float()
            normed = acc * torch.rsqrt(acc.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma.float()
            cases.append((M, x[:, rank * kl : (rank + 1) * kl].contiguous().cuda(), ref, acc, normed))
        x = make_activation(96, K, 99)
        layer_x = x[:, rank * kl : (rank + 1) * kl].contiguous().cuda()
        layer_ref = O.w8a8_block_fp8_linear(x, wq, ws, output_dtype=torch.float32)
        got = {}
        for two_shot, multicast, tag in ((False, None, "one"), (True, False, "two"), (True, True, "two_mc")):
            try:
                par = PeerAllReduce(512, Nn, torch.bfloat16, two_shot=two_shot, multicast=multicast)
            except AssertionError:  # no NVSwitch multicast mapping on this box: the peer-store path is the test
                assert multicast
                continue
            dist.barrier()
            for rep, (M, xl, ref, acc, normed) in enumerate(cases):
                out, _ = par.linear_bf16_input(xl, wl, wsl)
                got[f"{tag}_{rep}_sum"] = (out.clone(), ref)
                got[f"{tag}_{rep}_vs_nccl"] = (out.clone(), nccl(xl).float().cpu())
                both = [torch.empty_like(out) for _ in range(world)]
                dist.all_gather(both, out.contiguous())
                # every rank must hold the same bits
                res[f"{tag}_{rep}_same_bits"] = 0.0 if all(torch.equal(both[0], b) for b in both) else 1.0
                r = resid[:M].contiguous().cuda()
                out, r_out = par.linear_bf16_input(xl, wl, wsl, residual=r, rms_weight=gamma.cuda(), eps=1e-6)
                got[f"{tag}_{rep}_resid"] = (r_out.clone(), acc)
                got[f"{tag}_{rep}_norm"] = (out.clone(), normed)
        # captured in a CUDA graph (device-side epochs, single slot buffer): two calls per graph,
        # replayed with new inputs
        import sglang_b200 as S

        M, xl, ref, acc, normed = cases[1]
        for two_shot in (False, True):
            par = PeerAllReduce(512, Nn, torch.bfloat16, two_shot=two_shot, graph_safe=True)
            xq, xs = S.per_token_group_quant_fp8(xl, 128, column_major_scales=True)
            xq_static, xs_static = xq.clone(), xs.clone()
            stream = torch.cuda.Stream()
            graph = torch.cuda.CUDAGraph()
            dist.barrier()
            with torch.cuda.stream(stream):
                par.linear(xq_static, xs_static, wl, wsl)  # warm-up (workspace, module load)
                torch.cuda.synchronize()
                with torch.cuda.graph(graph, stream=stream):
                    o1, _ = par.linear(xq_static, xs_static, wl, wsl)
                    o1 = o1.clone()
                    o2, _ = par.linear(xq_static, xs_static, wl, wsl)
                    o2 = o2.clone()
            for rep in (1, 2, 4):
                M2, xl2, ref2, _, _ = cases[rep]
                if M2 != M:
                    continue
                q2, s2 = S.per_token_group_quant_fp8(xl2, 128, column_major_scales=True)
                xq_static.copy_(q2)
                xs_static.copy_(s2)
                dist.barrier()
                graph.replay()
                torch.cuda.synchronize()
                tag = "two" if two_shot else "one"
                got[f"graph_{tag}_{rep}_a"] = (o1.clone(), ref2)
                got[f"graph_{tag}_{rep}_b"] = (o2.clone(), ref2)
        # through the layer object
        row = P.RowParallelLinear(wq.cuda(), ws.cuda(), rank, world, reduce_mode="peer", max_tokens=128)
        dist.barrier()
        got["layer"] = (row(layer_x).clone(), layer_ref)
        torch.cuda.synchronize()
        for key, (mine, ref) in got.items():
            res[key] = O.rel_frobenius(mine.float().cpu(), ref)
        torch.cuda.synchronize()
        res["status"] = _native.read_device_status()
        results[rank] = res
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_peer_allreduce_ranks(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    port = 35500 + os.getpid() % 2000 + world
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        results = dict(results)
    assert set(results) == set(range(world))
    for r, res in results.items():
        assert res.pop("status") == 0
        for k, v in res.items():
            assert v < TOL, (r, k, v)
