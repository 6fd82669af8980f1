"""GPU parity of the tensor-core form of cdist_grad (contraction="tensor") against the float64 CPU
oracle, through the C-ABI.  Tolerance: max |x - ref| / max |ref| <= 5e-5 per output tensor, the same as
for the FP32 kernel; where the test is about the accuracy of the split tf32 products it is tighter and
says so."""
import ctypes

import pytest
import torch

import kermac_b200 as kermac
from kermac_b200 import _native
from oracle import kermac_oracle as ko

pytestmark = pytest.mark.gpu
TOL = 5e-5


def gen(shape, seed, dist="randn"):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn if dist == "randn" else torch.rand)(*shape, generator=g, dtype=torch.float32)


def clean_flag():
    assert _native.device_error_flag() == 0


@pytest.mark.parametrize("p", [1.0, 1.5, 2.0, 3.0, 0.5])
@pytest.mark.parametrize("O", [1, 7, 16, 17, 32, 33, 64, 70])
def test_every_channel_tile_and_norm(p, O):
    # K = 37: one full slab and a ragged one; M, N not multiples of the 32 x 16 / 32 x 8 tiles; channel counts on
    # both sides of the 16-, 32- and 64-channel shapes
    K, M, N = 37, 70, 45
    a, b, c, d = gen((K, M), 5, "rand"), gen((N, K), 6), gen((O, K), 7), gen((N, M), 8)
    got = kermac.cdist_grad(a.cuda(), b.cuda(), c.cuda(), d.cuda(), p=p, contraction="tensor")
    assert tuple(got.shape) == (1, O, N, M)
    assert ko.rel_err_signed(got, ko.cdist_grad_ref(a, b, c, d, p=p)) < TOL
    clean_flag()


@pytest.mark.parametrize("O", [16, 40])
@pytest.mark.parametrize("K", [1, 15, 16, 17, 31, 32, 33, 127, 128, 129, 255, 257, 1000])
def test_k_extents_around_buffers_slabs_and_chains(K, O):
    # 16 k per tensor-memory buffer, 32 per slab, 128 per accumulator chain; 40 channels take the shape with one
    # accumulator set, whose chains hand over differently
    M, N = 40, 20
    a, b, c, d = gen((K, M), 9, "rand"), gen((N, K), 10), gen((O, K), 11), gen((N, M), 12)
    for p in (1.0, 2.0):
        got = kermac.cdist_grad(a.cuda(), b.cuda(), c.cuda(), d.cuda(), p=p, contraction="tensor")
        assert ko.rel_err_signed(got, ko.cdist_grad_ref(a, b, c, d, p=p)) < TOL
    clean_flag()


@pytest.mark.parametrize("shape", [(1, 1, 1, 1), (3, 5, 2, 2), (64, 32, 16, 16), (65, 33, 17, 20), (200, 130, 33, 5)])
def test_odd_shapes_and_unaligned_views(shape):
    K, M, N, O = shape
    big_a = gen((K, M + 3), 13, "rand").cuda()
    big_d = gen((N, M + 5), 14).cuda()
    a, d = big_a[:, 1:M + 1], big_d[:, 2:M + 2]             # unaligned row starts, odd pitches
    b = gen((N, K + 1), 15).cuda()[:, :K]
    c = gen((O, K + 3), 16).cuda()[:, 1:K + 1]              # coefficients that cannot be read 16 bytes at a time
    big_out = torch.full((O, N, M + 2), -3.0, device="cuda")
    out = big_out[:, :, 1:M + 1]
    for p in (1.0, 1.7):
        got = kermac.cdist_grad(a, b, c, d, out=out, p=p, contraction="tensor")
        assert ko.rel_err_signed(got, ko.cdist_grad_ref(a.cpu(), b.cpu(), c.cpu(), d.cpu(), p=p)[0]) < TOL
    assert float(big_out[:, :, 0].max()) == -3.0 and float(big_out[:, :, -1].max()) == -3.0
    clean_flag()


@pytest.mark.parametrize("shape", [(36, 44, 21, 20), (4, 8, 3, 16), (260, 100, 37, 40), (1000, 64, 16, 64)])
def test_tma_staging_and_copy_staging_give_the_same_bits(shape):
    # operands with 16-byte aligned rows are staged by TMA, anything else by 4-byte copies: the arithmetic and
    # its order are the same, so the same numbers behind an unaligned view must give the same bits
    K, M, N, O = shape
    a, b, c, d = gen((K, M), 45, "rand").cuda(), gen((N, K), 46).cuda(), gen((O, K), 47).cuda(), gen((N, M), 48).cuda()
    a_view = torch.zeros(K, M + 3, device="cuda")[:, 1:M + 1]
    b_view = torch.zeros(N, K + 1, device="cuda")[:, :K]
    a_view.copy_(a)
    b_view.copy_(b)
    for p in (1.0, 2.0, 1.7):
        aligned = kermac.cdist_grad(a, b, c, d, p=p, contraction="tensor")
        views = kermac.cdist_grad(a_view, b_view, c, d, p=p, contraction="tensor")
        assert torch.equal(aligned, views)
        assert ko.rel_err_signed(aligned, ko.cdist_grad_ref(a.cpu(), b.cpu(), c.cpu(), d.cpu(), p=p)) < TOL
    clean_flag()


def test_exact_ties_follow_copysign():
    # d[n, m] == b[n, k] for many triples: p = 1 counts them as +1, p > 1 as 0, as the FP32 kernel does
    K, M, N, O = 48, 64, 8, 16
    b = gen((N, K), 17)
    d = b[:, :1].expand(N, M).contiguous()
    a, c = gen((K, M), 18, "rand"), gen((O, K), 19)
    for p in (1.0, 1.5, 2.0):
        got = kermac.cdist_grad(a.cuda(), b.cuda(), c.cuda(), d.cuda(), p=p, contraction="tensor")
        assert ko.rel_err_signed(got, ko.cdist_grad_ref(a, b, c, d, p=p)) < TOL
        assert torch.isfinite(got).all()
    clean_flag()


def test_batching_broadcast_and_per_batch_p():
    L, K, M, N, O = 3, 140, 66, 20, 24
    a, b, c, d = gen((L, K, M), 20, "rand"), gen((N, K), 21), gen((1, O, K), 22), gen((L, N, M), 23)
    p = torch.tensor([1.5, 2.0, 3.0])
    got = kermac.cdist_grad(a.cuda(), b.cuda(), c.cuda(), d.cuda(), p=p.cuda(), contraction="tensor")
    assert ko.rel_err_signed(got, ko.cdist_grad_ref(a, b, c, d, p=p)) < TOL
    clean_flag()


@pytest.mark.parametrize("O", [16, 24, 40])
def test_same_sign_sums_stay_at_fp32_accuracy(O):
    # Every term positive, 20000 of them: a chain of truncating tensor-core additions that long would
    # drift by ~1e-4; cut every 128 k and added up in FP32 the result stays within 3e-6 of the oracle.
    K, M, N = 20000, 64, 32
    a, c = gen((K, M), 24, "rand"), gen((O, K), 25, "rand")
    b, d = gen((N, K), 26, "rand"), gen((N, M), 27, "rand") + 2.0
    for p in (1.0, 2.0):
        got = kermac.cdist_grad(a.cuda(), b.cuda(), c.cuda(), d.cuda(), p=p, contraction="tensor")
        assert ko.rel_err_signed(got, ko.cdist_grad_ref(a, b, c, d, p=p)) < 3e-6
    clean_flag()


@pytest.mark.parametrize("O", [16, 32, 48])
def test_split_k_through_the_c_abi(O):
    K, M, N = 3000, 96, 40
    a, b, c, d = gen((K, M), 28, "rand"), gen((N, K), 29), gen((O, K), 30), gen((N, M), 31)
    ref = ko.cdist_grad_ref(a, b, c, d, p=1.0)[0]
    ad, bd, cd, dd = a.cuda(), b.cuda(), c.cuda(), d.cuda()
    outs = []
    for split in (1, 5):
        out = torch.empty(O, N, M, device="cuda")
        args = _native.KmGradArgs()
        args.m, args.n, args.o, args.k, args.l = M, N, O, K, 1
        args.a, args.lda = ad.data_ptr(), M
        args.b, args.ldb = bd.data_ptr(), K
        args.c, args.ldc = cd.data_ptr(), K
        args.d, args.ldd = dd.data_ptr(), M
        args.out, args.out_stride_n, args.out_stride_o = out.data_ptr(), M, N * M
        args.norm_type = _native.NORM_L1
        args.p = _native.hyper(1.0)
        args.split_k = split
        args.contraction = 2                                 # KM_CONTRACT_TENSOR
        need = _native.lib().kermac_b200_cdist_grad_scratch_bytes(ctypes.byref(args))
        assert need == (0 if split == 1 else split * O * N * M * 4)
        scratch = torch.empty(max(need // 4, 1), device="cuda")
        args.scratch, args.scratch_bytes = scratch.data_ptr(), need
        _native.launch_grad(args, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert ko.rel_err_signed(out, ref) < TOL
        outs.append(out)
    assert float((outs[0] - outs[1]).abs().max() / ref.abs().max()) < 2e-5   # regrouped sums
    clean_flag()


def test_automatic_choice_and_run_to_run_identity():
    # more than 16 channels and 256 k or more: the tensor cores; otherwise the FP32 kernel
    K, M, N = 600, 100, 50
    a, b, d = gen((K, M), 32, "rand").cuda(), gen((N, K), 33).cuda(), gen((N, M), 34).cuda()
    for O, expect in ((16, "fp32"), (17, "tensor"), (40, "tensor")):
        c = gen((O, K), 35).cuda()
        auto = kermac.cdist_grad(a, b, c, d, p=1.0)
        same = kermac.cdist_grad(a, b, c, d, p=1.0, contraction=expect)
        assert torch.equal(auto, same), (O, expect)
        assert torch.equal(auto, kermac.cdist_grad(a, b, c, d, p=1.0))      # fixed summation order
    c = gen((40, 100), 36).cuda()                                            # short k: FP32 whatever O is
    short = kermac.cdist_grad(a[:100], b[:, :100].contiguous(), c, d, p=1.0)
    assert torch.equal(short, kermac.cdist_grad(a[:100], b[:, :100].contiguous(), c, d, p=1.0, contraction="fp32"))
    clean_flag()


def test_wave_filling_split_on_a_long_contraction():
    # few tiles, long k: the launcher splits k over the SMs; checked on sampled rows against the oracle
    K, M, N, O = 9000, 300, 130, 32
    a, b, c, d = gen((K, M), 37, "rand"), gen((N, K), 38), gen((O, K), 39), gen((N, M), 40)
    got = kermac.cdist_grad(a.cuda(), b.cuda(), c.cuda(), d.cuda(), p=1.5, contraction="tensor")[0]
    rows = [0, 7, 8, 64, 129]
    ref = ko.cdist_grad_ref(a, b[rows], c, d[rows], p=1.5)[0]
    assert ko.rel_err_signed(got[:, rows], ref) < TOL
    fp = kermac.cdist_grad(a.cuda(), b.cuda(), c.cuda(), d.cuda(), p=1.5, contraction="fp32")[0]
    assert float((got - fp).abs().max() / fp.abs().max()) < 2e-5
    clean_flag()


def test_static_scratch_entry_point_takes_the_tensor_path_too():
    K, M, N, O = 4000, 64, 32, 20
    a, b, c, d = gen((K, M), 41, "rand").cuda(), gen((N, K), 42).cuda(), gen((O, K), 43).cuda(), gen((N, M), 44).cuda()
    out = torch.empty(O, N, M, device="cuda")
    args = _native.KmGradArgs()
    args.m, args.n, args.o, args.k, args.l = M, N, O, K, 1
    args.a, args.lda = a.data_ptr(), M
    args.b, args.ldb = b.data_ptr(), K
    args.c, args.ldc = c.data_ptr(), K
    args.d, args.ldd = d.data_ptr(), M
    args.out, args.out_stride_n, args.out_stride_o = out.data_ptr(), M, N * M
    args.norm_type = _native.NORM_L2
    args.p = _native.hyper(2.0)
    args.contraction = 2
    rc = _native.lib().kermac_b200_cdist_grad_static(ctypes.byref(args), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, _native.last_error()
    torch.cuda.synchronize()
    ref = ko.cdist_grad_ref(a.cpu(), b.cpu(), c.cpu(), d.cpu(), p=2.0)[0]
    assert ko.rel_err_signed(out, ref) < TOL
    clean_flag()
