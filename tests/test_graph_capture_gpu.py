"""The operators are plain asynchronous launches on the current stream, so a launch-bound loop of
small calls can be captured once in a CUDA graph and replayed."""
import pytest
import torch

import kermac_b200 as kermac

pytestmark = pytest.mark.gpu


def test_small_calls_replay_from_a_cuda_graph():
    g = torch.Generator().manual_seed(3)
    a = torch.rand(64, 2048, generator=g).cuda().t()
    b = torch.rand(64, 1024, generator=g).cuda().t()
    x = torch.rand(300, 24, generator=g).cuda()
    c = torch.randn(16, 2048, generator=g).cuda()
    gk, gb, gc, gd = torch.rand(96, 260, generator=g).cuda(), torch.randn(40, 96, generator=g).cuda(), \
        torch.randn(4, 96, generator=g).cuda(), torch.randn(40, 260, generator=g).cuda()
    out_d = torch.empty(1024, 2048, device="cuda").t()
    out_s = torch.empty(1, 300, 300, device="cuda")
    out_y = torch.empty(1, 1024, 16, device="cuda")
    out_g = torch.empty(1, 4, 40, 260, device="cuda")

    def work():
        kermac.cdist(a, b, out=out_d, p=2.0)                       # TMA-staged kernel
        kermac.cdist(a, b, out=out_d, p=1.3)
        kermac.cdist(a, b, out=out_d, p=1.0)
        kermac.cdist(x, x, out=out_s, p=2.0)                       # symmetric build
        kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, a, b, c, out=out_y, bandwidth=8.0)   # tcgen05 + TMA
        kermac.cdist_grad(gk, gb, gc, gd, out=out_g, p=1.0)

    work()                                                          # warm-up outside capture (function attributes)
    torch.cuda.synchronize()
    want = [t.clone() for t in (out_d, out_s, out_y, out_g)]
    for t in (out_d, out_s, out_y, out_g):
        t.zero_()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            work()
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        for t in (out_d, out_s, out_y, out_g):
            t.zero_()
        graph.replay()
        torch.cuda.synchronize()
        for got, ref in zip((out_d, out_s, out_y, out_g), want):
            assert torch.equal(got, ref)
