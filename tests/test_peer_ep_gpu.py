"""Expert-parallel dispatch / combine kernels. The C ABI takes one pointer per rank, so p ranks are
emulated on ONE GPU by giving every "rank" its own areas and running the steps rank by rank (no
kernel waits for another: the handshake is a separate kernel and is only exercised against
itself here; the real 2-GPU run is in test_parallel_gpu.py)."""
import ctypes

import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _arr(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


@pytest.mark.parametrize("p,E,k,H,I,T_max,tokens", [(2, 8, 2, 256, 128, 40, [37, 40]), (4, 16, 4, 512, 256, 24, [24, 1, 0, 17]),
                                                   (1, 8, 2, 256, 128, 16, [9])])
def test_dispatch_experts_combine_emulated_ranks(p, E, k, H, I, T_max, tokens):
    import sglang_b200 as S
    from sglang_b200 import _native as N
    from sglang_b200.fused_moe import fused_experts_impl

    lib = N.load()
    g = torch.Generator().manual_seed(p * 100 + E)
    w1 = torch.stack([O.block_quant_weight_fp8((torch.randn(2 * I, H, generator=g) * 0.02).bfloat16())[0] for _ in range(E)])
    w2 = torch.stack([O.block_quant_weight_fp8((torch.randn(H, I, generator=g) * 0.02).bfloat16())[0] for _ in range(E)])
    w1_s = torch.rand(E, 2 * I // 128, H // 128, generator=g) * 2e-4 + 1e-4
    w2_s = torch.rand(E, H // 128, I // 128, generator=g) * 2e-4 + 1e-4
    pos = p * T_max
    dev = "cuda"
    q = [torch.full((pos, H), 0x7F, dtype=torch.uint8, device=dev) for _ in range(p)]  # NaN bytes where nobody writes
    s = [torch.full((pos, H // 128), float("nan"), device=dev) for _ in range(p)]
    w = [torch.full((pos, k), float("nan"), device=dev) for _ in range(p)]
    ids = [torch.full((pos, k), 12345, dtype=torch.int32, device=dev) for _ in range(p)]
    out = [torch.full((pos, H), float("nan"), dtype=torch.bfloat16, device=dev) for _ in range(p)]
    xs, tws, tis = [], [], []
    for r in range(p):
        T = tokens[r]
        x = torch.randn(T, H, generator=g).bfloat16()
        tw, ti = O.softmax_topk(torch.randn(T, E, generator=g), k, True)
        if T > 3:
            ti[1, 0] = -1  # an id that belongs to nobody
        xs.append(x); tws.append(tw); tis.append(ti)
        xq, xsc = S.per_token_group_quant_fp8(x.cuda(), 128) if T else (torch.empty(0, H, dtype=torch.float8_e4m3fn, device=dev), torch.empty(0, H // 128, device=dev))
        tw_d, ti_d = tw.cuda(), ti.cuda()  # named: a temporary would be freed (and its block reused) before the launch
        st = lib.b200_ep_dispatch(N.ptr(xq), N.ptr(xsc), N.ptr(tw_d), N.ptr(ti_d), T, T_max, k, H, E, p, r,
                                  _arr(q), _arr(s), _arr(w), _arr(ids), N.current_stream())
        N.check(st, "dispatch")
        torch.cuda.synchronize()
    per = E // p
    for d in range(p):
        # every position was published: local ids in [-1, per)
        assert int(ids[d].min()) >= -1 and int(ids[d].max()) < per
        for r in range(p):
            blk = ids[d][r * T_max : (r + 1) * T_max].cpu()
            ref = O.ep_local_expert_ids(tis[r], E, p, d)
            assert torch.equal(blk[: tokens[r]], ref) and torch.all(blk[tokens[r] :] == -1)
        lo = d * per
        fused_experts_impl(q[d].view(torch.float8_e4m3fn), w1[lo : lo + per].cuda(), w2[lo : lo + per].cuda(), w[d], ids[d],
                           w1_s[lo : lo + per].cuda(), w2_s[lo : lo + per].cuda(), hidden_states_scale=s[d],
                           output_dtype=torch.bfloat16, out=out[d], skip_unrouted_rows=True)
    for r in range(p):
        T = tokens[r]
        res = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        ti_d = tis[r].cuda()
        st = lib.b200_ep_combine(_arr(out), N.ptr(ti_d), N.ptr(res), N.BF16, T, T_max, k, H, E, p, r,
                                 N.current_stream())
        N.check(st, "combine")
        torch.cuda.synchronize()
        if T == 0:
            continue
        ref = O.fused_experts_fp8(xs[r], w1, w2, w1_s, w2_s, tws[r], tis[r], [128, 128])
        assert not torch.isnan(res.float()).any()
        assert O.rel_frobenius(res.float().cpu(), ref) < TOL, r
    assert N.read_device_status() == 0


@pytest.mark.parametrize("p,E,k,H,I,T_max,tokens", [(2, 8, 2, 256, 128, 40, [37, 40]), (4, 16, 4, 512, 256, 24, [24, 1, 0, 17]),
                                                   (8, 32, 8, 256, 128, 12, [12, 3, 0, 7, 12, 1, 9, 5]), (1, 8, 2, 256, 128, 16, [9])])
def test_dispatch_experts_push_combine_emulated_ranks(p, E, k, H, I, T_max, tokens):
    """Combine by push: the down GEMM of every owner sends its (token, slot) rows into the source rank's inbox
    (here: p inboxes on one GPU), then each source sums its slots. Inboxes start as NaN, so a row sent to the
    wrong place or not at all shows up."""
    import sglang_b200 as S
    from sglang_b200 import _native as N
    from sglang_b200.fused_moe import fused_experts_scatter, moe_sum_reduce

    lib = N.load()
    g = torch.Generator().manual_seed(p * 1000 + E)
    w1 = torch.stack([O.block_quant_weight_fp8((torch.randn(2 * I, H, generator=g) * 0.02).bfloat16())[0] for _ in range(E)])
    w2 = torch.stack([O.block_quant_weight_fp8((torch.randn(H, I, generator=g) * 0.02).bfloat16())[0] for _ in range(E)])
    w1_s = torch.rand(E, 2 * I // 128, H // 128, generator=g) * 2e-4 + 1e-4
    w2_s = torch.rand(E, H // 128, I // 128, generator=g) * 2e-4 + 1e-4
    pos = p * T_max
    dev = "cuda"
    q = [torch.full((pos, H), 0x7F, dtype=torch.uint8, device=dev) for _ in range(p)]
    s = [torch.full((pos, H // 128), float("nan"), device=dev) for _ in range(p)]
    w = [torch.full((pos, k), float("nan"), device=dev) for _ in range(p)]
    ids = [torch.full((pos, k), 12345, dtype=torch.int32, device=dev) for _ in range(p)]
    inbox = [torch.full((T_max, k, H), float("nan"), dtype=torch.bfloat16, device=dev) for _ in range(p)]
    xs, tws, tis = [], [], []
    for r in range(p):
        T = tokens[r]
        x = torch.randn(T, H, generator=g).bfloat16()
        tw, ti = O.softmax_topk(torch.randn(T, E, generator=g), k, True)
        if T > 3:
            ti[1, 0] = -1  # an id that belongs to nobody: its inbox row stays NaN and must not be summed
        xs.append(x); tws.append(tw); tis.append(ti)
        xq, xsc = S.per_token_group_quant_fp8(x.cuda(), 128) if T else (torch.empty(0, H, dtype=torch.float8_e4m3fn, device=dev), torch.empty(0, H // 128, device=dev))
        tw_d, ti_d = tw.cuda(), ti.cuda()
        N.check(lib.b200_ep_dispatch(N.ptr(xq), N.ptr(xsc), N.ptr(tw_d), N.ptr(ti_d), T, T_max, k, H, E, p, r,
                                     _arr(q), _arr(s), _arr(w), _arr(ids), N.current_stream()), "dispatch")
        torch.cuda.synchronize()
    per = E // p
    dests = _arr(inbox)
    for d in range(p):
        lo = d * per
        fused_experts_scatter(q[d].view(torch.float8_e4m3fn), s[d], w1[lo : lo + per].cuda(), w2[lo : lo + per].cuda(), w[d],
                              ids[d], w1_s[lo : lo + per].cuda(), w2_s[lo : lo + per].cuda(), dests, T_max * k, torch.bfloat16)
        torch.cuda.synchronize()
    for r in range(p):
        T = tokens[r]
        if T == 0:
            assert bool(torch.isnan(inbox[r]).all())  # nobody writes into the inbox of a rank without tokens
            continue
        res = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        moe_sum_reduce(inbox[r][:T], tis[r].cuda().to(torch.int32), res, E, poison_on_status=True)
        torch.cuda.synchronize()
        valid = (tis[r] >= 0).cuda()
        got_rows = ~torch.isnan(inbox[r][:T].float()).any(dim=2)
        assert torch.equal(got_rows, valid), "exactly the rows of valid pairs arrive"
        assert bool(torch.isnan(inbox[r][T:]).all())
        ref = O.fused_experts_fp8(xs[r], w1, w2, w1_s, w2_s, tws[r], tis[r], [128, 128])
        assert not torch.isnan(res.float()).any()
        assert O.rel_frobenius(res.float().cpu(), ref) < TOL, r
    assert N.read_device_status() == 0
    # argument checks of the new entry points
    assert lib.b200_fused_experts_fp8_scatter(None, None, N.BF16, None, None, None, None, None, None, dests, p, T_max * k, 4, k,
                                              per, H, I, None, 0, None) == N.E_BAD_ARG
    assert lib.b200_moe_sum_reduce(None, None, None, N.BF16, 4, k, E, H, 1.0, 0, 0, None) == N.E_BAD_ARG


def test_handshake_with_itself_and_argument_checks():
    from sglang_b200 import _native as N

    lib = N.load()
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    peers = (ctypes.c_void_p * 1)(flags.data_ptr())
    for epoch in (1, 2, 3):
        for phase in (0, 1):
            N.check(lib.b200_peer_handshake(flags.data_ptr(), peers, 1, 0, phase, epoch, N.current_stream()), "handshake")
    torch.cuda.synchronize()
    assert N.read_device_status() == 0
    assert flags[0].item() == 3 and flags[8].item() == 3
    assert lib.b200_peer_handshake(flags.data_ptr(), peers, 9, 0, 0, 1, None) == N.E_BAD_ARG
    assert lib.b200_ep_dispatch(None, None, None, None, 4, 2, 2, 256, 8, 1, 0, peers, peers, peers, peers, None) == N.E_BAD_ARG


def test_a_peer_that_never_signals_times_out_and_the_context_survives():
    """Failure detection without a fault: the "other rank" is a flag array that nothing writes. The
    bounded wait gives up after the limit (100 ms here), the device status word reports it, reading
    the word clears it, and the next launches on the same context work."""
    import time

    from sglang_b200 import _native as N

    lib = N.load()
    with N.tuning(peer_wait_ms=100):
        _silent_peer_case(lib, N)


def _silent_peer_case(lib, N):
    import time

    mine = torch.zeros(64, dtype=torch.int32, device="cuda")
    silent_peer = torch.zeros(64, dtype=torch.int32, device="cuda")
    peers = (ctypes.c_void_p * 2)(mine.data_ptr(), silent_peer.data_ptr())
    assert N.read_device_status() == 0
    t0 = time.time()
    N.check(lib.b200_peer_handshake(mine.data_ptr(), peers, 2, 0, 0, 1, N.current_stream()), "handshake")
    status = N.read_device_status()  # synchronises
    waited = time.time() - t0
    assert status == 2, "the expired wait must be reported"
    assert 0.05 < waited < 1.5, waited
    assert silent_peer[0].item() == 1  # our own signal did go out
    assert N.read_device_status() == 0  # cleared by the read
    # the all-reduce finishing kernel gives up the same way and poisons its result with NaNs: a caller
    # that never polls the status word cannot mistake stale bytes for a sum
    slot = torch.ones(2, 8, 256, dtype=torch.bfloat16, device="cuda")
    out = torch.full((8, 256), 7.0, dtype=torch.bfloat16, device="cuda")
    outs = (ctypes.c_void_p * 1)(out.data_ptr())
    N.check(lib.b200_allreduce_finish(slot.data_ptr(), 8 * 256, outs, N.BF16, 8, 256, 2, 0, 0, None, None, None, 1e-6,
                                      mine.data_ptr(), peers, 5, None, None, N.current_stream()), "finish")
    assert N.read_device_status() == 2 and bool(torch.isnan(out).all())
    # two-shot: the owned rows and (second handshake) the rows the silent owner never delivered
    out2 = torch.full((8, 256), 7.0, dtype=torch.bfloat16, device="cuda")
    outs2 = (ctypes.c_void_p * 2)(out2.data_ptr(), out2.data_ptr())
    N.check(lib.b200_allreduce_finish(slot.data_ptr(), 8 * 256, outs2, N.BF16, 8, 256, 2, 0, 1, None, None, None, 1e-6,
                                      mine.data_ptr(), peers, 6, None, None, N.current_stream()), "finish")
    assert N.read_device_status() == 2 and bool(torch.isnan(out2).all())
    # the expert-parallel combine after a handshake that gave up: NaNs, not stale rows
    area = torch.ones(2, 4, 256, dtype=torch.bfloat16, device="cuda")
    areas = (ctypes.c_void_p * 2)(area.data_ptr(), area.data_ptr())
    ids = torch.zeros(4, 2, dtype=torch.int32, device="cuda")
    res = torch.full((4, 256), 7.0, dtype=torch.bfloat16, device="cuda")
    N.check(lib.b200_peer_handshake(mine.data_ptr(), peers, 2, 0, 1, 9, N.current_stream()), "handshake")
    N.check(lib.b200_ep_combine(areas, ids.data_ptr(), res.data_ptr(), N.BF16, 4, 4, 2, 256, 8, 2, 0, N.current_stream()),
            "combine")
    assert N.read_device_status() == 2 and bool(torch.isnan(res).all())
    # the same for the push form: the source's slot sum after a handshake that gave up
    inbox = torch.ones(4, 2, 256, dtype=torch.bfloat16, device="cuda")
    res2 = torch.full((4, 256), 7.0, dtype=torch.bfloat16, device="cuda")
    N.check(lib.b200_peer_handshake(mine.data_ptr(), peers, 2, 0, 1, 10, N.current_stream()), "handshake")
    N.check(lib.b200_moe_sum_reduce(inbox.data_ptr(), ids.data_ptr(), res2.data_ptr(), N.BF16, 4, 2, 8, 256, 1.0, 0, 1,
                                    N.current_stream()), "sum_reduce")
    assert N.read_device_status() == 2 and bool(torch.isnan(res2).all())
    # and with a clear status word the same call sums: two slots of ones
    N.check(lib.b200_moe_sum_reduce(inbox.data_ptr(), ids.data_ptr(), res2.data_ptr(), N.BF16, 4, 2, 8, 256, 1.0, 0, 1,
                                    N.current_stream()), "sum_reduce")
    assert N.read_device_status() == 0 and bool(torch.all(res2 == 2.0))
    # the context is intact: a healthy single-rank call right after
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    self_only = (ctypes.c_void_p * 1)(flags.data_ptr())
    N.check(lib.b200_allreduce_finish(slot.data_ptr(), 8 * 256, outs, N.BF16, 8, 256, 1, 0, 0, None, None, None, 1e-6,
                                      flags.data_ptr(), self_only, 1, None, None, N.current_stream()), "finish")
    assert N.read_device_status() == 0 and torch.all(out == 1.0)
