"""Every operator is launch-only (no allocation, no sync inside the C ABI), so a call captured in
a CUDA graph replays with the same pointers: capture, overwrite the inputs in place, replay and
compare with an eager call on the new inputs."""
import pytest
import torch

import oracle as O
from conftest import make_activation, make_weight

pytestmark = pytest.mark.gpu


def _capture(fn):
    s = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        for _ in range(2):
            fn()  # warm-up on the capture stream (workspaces, lazy set-up)
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=s):
            out = fn()
    torch.cuda.synchronize()
    return g, out


@pytest.mark.parametrize("M", [4, 200, 2048])  # decode kernel + split-K reduce, split-K large tile, plain
def test_linear_replays(M):
    import sglang_b200 as S

    wq, ws = make_weight(1024, 2048, 5)
    wq, ws = wq.cuda(), ws.cuda()
    x = make_activation(M, 2048, 6).cuda()
    g, out = _capture(lambda: S.w8a8_block_fp8_linear(x, wq, [128, 128], ws))
    x2 = make_activation(M, 2048, 7)
    x.copy_(x2.cuda())
    g.replay()
    torch.cuda.synchronize()
    ref = O.w8a8_block_fp8_linear(x2, wq.cpu(), ws.cpu(), output_dtype=torch.float32)
    assert O.rel_frobenius(out.float().cpu(), ref) < 1e-2


def test_fused_experts_and_align_replay():
    import sglang_b200 as S

    T, E, topk, H, I = 300, 16, 4, 512, 256
    gen = torch.Generator().manual_seed(1)
    w1 = torch.stack([make_weight(2 * I, H, 10 + e)[0] for e in range(E)])
    w2 = torch.stack([make_weight(H, I, 40 + e)[0] for e in range(E)])
    w1_s = torch.rand(E, 2 * I // 128, H // 128, generator=gen) * 2e-4 + 1e-4
    w2_s = torch.rand(E, H // 128, I // 128, generator=gen) * 2e-4 + 1e-4
    x = torch.randn(T, H, generator=gen).bfloat16()
    tw, ti = O.softmax_topk(torch.randn(T, E, generator=gen), topk, True)
    xd, twd, tid = x.cuda(), tw.cuda(), ti.cuda()
    dev = [t.cuda() for t in (w1, w2, w1_s, w2_s)]
    cfg = S.MoeRunnerConfig(inplace=False)

    def call():
        return S.fused_experts(xd, dev[0], dev[1], S.StandardTopKOutput(twd, tid, None), cfg, use_fp8_w8a8=True,
                               w1_scale=dev[2], w2_scale=dev[3], block_shape=[128, 128])

    g, out = _capture(call)
    # new tokens AND new routing: the tile schedule is rebuilt on the device at every replay
    x2 = torch.randn(T, H, generator=gen).bfloat16()
    tw2, ti2 = O.softmax_topk(torch.randn(T, E, generator=gen), topk, True)
    xd.copy_(x2.cuda()); twd.copy_(tw2.cuda()); tid.copy_(ti2.cuda())
    g.replay()
    torch.cuda.synchronize()
    ref = O.fused_experts_fp8(x2, w1, w2, w1_s, w2_s, tw2, ti2)
    assert O.rel_frobenius(out.float().cpu(), ref) < 1e-2
