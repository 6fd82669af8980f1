"""kermac_b200_cdist_grad_static: the split-k gradient whose scratch is the array built
into the library, for callers that are not allowed to allocate device memory at the call
site (a plugin living inside another runtime's fixed pool, a latency-bound loop, a
foreign-function layer that can only forward pointers it was handed).

Collected last on purpose: a run that stops at the first failure has then already run
every other test.  The entry point is called through the C-ABI and compared with the
ordinary entry point, which gets its scratch from torch, on two calls in a row that
share the built-in array.
"""
import ctypes

import pytest
import torch

from kermac_b200 import _native
from oracle import kermac_oracle as ko

pytestmark = pytest.mark.gpu
TOL = 5e-5


def _args(a, b, c, d, out, norm, p, split_k):
    K, M = a.shape
    N, O = b.shape[0], c.shape[0]
    g = _native.KmGradArgs()
    g.m, g.n, g.o, g.k, g.l = M, N, O, K, 1
    g.a, g.lda = a.data_ptr(), a.stride(0)
    g.b, g.ldb = b.data_ptr(), b.stride(0)
    g.c, g.ldc = c.data_ptr(), c.stride(0)
    g.d, g.ldd = d.data_ptr(), d.stride(0)
    g.out, g.out_stride_n, g.out_stride_o = out.data_ptr(), out.stride(1), out.stride(0)
    g.norm_type = norm
    g.p = _native.hyper(p)
    g.split_k = split_k
    return g


def _inputs(seed, K, M, N, O):
    gen = torch.Generator().manual_seed(seed)
    a = torch.rand(K, M, generator=gen).cuda()
    b = torch.randn(N, K, generator=gen).cuda()
    c = torch.randn(O, K, generator=gen).cuda()
    d = torch.randn(N, M, generator=gen).cuda()
    return a, b, c, d


def test_static_scratch_matches_caller_scratch_on_two_calls_in_a_row():
    lib = _native.lib()
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: the second call finds the first one's partial
    # sums in the shared array and must not be affected by them
    cases = [(101, 4000, 256, 64, 4, _native.NORM_L1, 1.0, 6), (202, 2500, 192, 48, 3, _native.NORM_P, 1.5, 4)]
    for seed, K, M, N, O, norm, p, split in cases:
        a, b, c, d = _inputs(seed, K, M, N, O)
        want = torch.empty(O, N, M, device="cuda")
        g = _args(a, b, c, d, want, norm, p, split)
        need = lib.kermac_b200_cdist_grad_scratch_bytes(ctypes.byref(g))
        assert 0 < need <= _native.GRAD_STATIC_SCRATCH_BYTES
        scratch = torch.empty(need // 4, device="cuda")
        g.scratch, g.scratch_bytes = scratch.data_ptr(), need
        _native.launch_grad(g, stream)

        got = torch.full((O, N, M), float("nan"), device="cuda")
        gs = _args(a, b, c, d, got, norm, p, split)          # no scratch passed
        _native.launch_grad_static(gs, stream)
        torch.cuda.synchronize()
        assert ko.rel_err_signed(got, want.cpu().double()) < TOL
        assert ko.rel_err_signed(got, ko.cdist_grad_ref(a.cpu(), b.cpu(), c.cpu(), d.cpu(), p=p)[0]) < TOL
    assert _native.device_error_flag() == 0


def test_static_scratch_rejects_what_does_not_fit_and_single_pass_always_fits():
    lib = _native.lib()
    stream = torch.cuda.current_stream().cuda_stream
    a, b, c, d = _inputs(303, 600, 128, 32, 2)
    out = torch.empty(2, 32, 128, device="cuda")
    big = _args(a, b, c, d, out, _native.NORM_L2, 2.0, 4)
    big.m, big.n, big.o = 8192, 4096, 4                     # 4 partials x 512 MiB: far beyond the array
    big.lda = big.ldd = big.out_stride_n = 8192
    big.out_stride_o = 8192 * 4096
    rc = lib.kermac_b200_cdist_grad_static(ctypes.byref(big), ctypes.c_void_p(stream))
    assert rc == -6 and "built-in array" in _native.last_error()
    one = _args(a, b, c, d, out, _native.NORM_L2, 2.0, 1)    # single pass needs no scratch at all
    _native.launch_grad_static(one, stream)
    torch.cuda.synchronize()
    assert ko.rel_err_signed(out, ko.cdist_grad_ref(a.cpu(), b.cpu(), c.cpu(), d.cpu(), p=2.0)[0]) < TOL


def test_automatic_split_is_reduced_to_what_the_array_holds():
    # split_k = 0 on a problem whose preferred split needs more than the built-in array: the ordinary
    # entry point falls back when the caller's scratch is too small, and this one does the same
    # instead of refusing (an explicit split_k that does not fit is still refused)
    lib = _native.lib()
    stream = torch.cuda.current_stream().cuda_stream
    K, M, N, O = 3000, 4096, 320, 4                          # one partial result is 21 MB; 9 are preferred
    a, b, c, d = _inputs(404, K, M, N, O)
    out = torch.full((O, N, M), float("nan"), device="cuda")
    g = _args(a, b, c, d, out, _native.NORM_L1, 1.0, 0)
    wanted = lib.kermac_b200_cdist_grad_scratch_bytes(ctypes.byref(g))
    assert wanted > _native.GRAD_STATIC_SCRATCH_BYTES, "the case must prefer a split that does not fit"
    _native.launch_grad_static(g, stream)
    torch.cuda.synchronize()
    rows = torch.tensor([0, 159, 319])
    ref = ko.cdist_grad_ref(a.cpu(), b.cpu()[rows], c.cpu(), d.cpu()[rows], p=1.0)[0]
    assert ko.rel_err_signed(out[:, rows.cuda()], ref) < TOL
    explicit = _args(a, b, c, d, out, _native.NORM_L1, 1.0, 4)
    rc = lib.kermac_b200_cdist_grad_static(ctypes.byref(explicit), ctypes.c_void_p(stream))
    assert rc == -6 and "built-in array" in _native.last_error()
