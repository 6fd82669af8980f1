"""Parity at the full sizes of the large benchmark configurations, on sampled output rows: the
float64 oracle of a few rows costs the CPU seconds, while the GPU runs the real launch (grid.y
batches with a broadcast operand map; thousands of m-chunks per block and the split over m).
Also `kernel_matvec` pinned to the reference: its kernel matrix materialised by the reference's own
kernels, multiplied in float64."""
import pytest
import torch

import kermac_b200 as kermac
from baseline import ref_kernels
from kermac_b200 import _native
from oracle import kermac_oracle as ko

pytestmark = pytest.mark.gpu

LAPLACE_L2 = dict(inner_operator="DIFF", inner_power="SQUARE", outer_power="SQRT", kernel_type="LAPLACE")


def test_batched_fractional_configuration_full_size_rows_of_every_batch():
    # a[B=4, K=512, M=16384] batched, b[1, K=512, N=16384] broadcast, U(-1,1) seed 2, p = 1.3
    B, K, M, N, p = 4, 512, 16384, 16384, 1.3
    g = torch.Generator().manual_seed(2)
    a_store = 2.0 * torch.rand(B, K, M, generator=g) - 1.0
    b_store = 2.0 * torch.rand(1, K, N, generator=g) - 1.0
    a, b = a_store.cuda().permute(0, 2, 1), b_store.cuda().permute(0, 2, 1)
    out = torch.empty(B, N, M, device="cuda").permute(0, 2, 1)          # (B, M, N), m contiguous
    rows = torch.tensor([0, 127, 128, 8191, 16383])                     # n: tile seams, middle, last
    b_rows = b_store[0].t()[rows]                                       # (R, K)
    for skip in (False, True):
        kermac.cdist(a, b, out=out, p=p, skip_epilogue=skip)
        for l in range(B):
            got = out[l][:, rows.cuda()].t().cpu()                      # (R, M)
            ref = ko.cdist_ref(a_store[l].t(), b_rows, p=p, skip_epilogue=skip)[0].t()
            assert ko.rel_err_nonneg(got, ref) < 5e-5, (skip, l)
    assert _native.device_error_flag() == 0


def test_matvec_configuration_full_size_sampled_rows():
    # a[K=64, M=10^6], c[O=16, M] ~ N(0,1) seed 4, sigma = 8; N cut to two row tiles around five sampled
    # points of the full b: every block still walks all 7,813 m-chunks and the launcher splits over m
    K, M, N, O = 64, 1_000_000, 1_000_000, 16
    g = torch.Generator().manual_seed(4)
    a_store = torch.randn(K, M, generator=g)
    b_store = torch.randn(K, N, generator=g)
    c = torch.randn(O, M, generator=g)
    rows = torch.tensor([0, 127, 128, 500_000, 999_999])
    b_sel = torch.zeros(K, 256)
    b_sel[:, :5] = b_store[:, rows]
    b_sel[:, 5:] = b_store[:, 1000:1251]                                # filler points: keep both tiles full
    a, b = a_store.cuda().t(), b_sel.cuda().t()
    y = kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, a, b, c.cuda(), bandwidth=8.0)[0]
    ref = ko.kernel_matvec_ref(a_store.t(), b_sel.t()[:5], c, **LAPLACE_L2, bandwidth=8.0)[0]
    assert ko.rel_err_signed(y[:5], ref) < 5e-5
    # the same five rows inside a launch over many row tiles (no split over m there): same values to rounding
    b_big = b_store[:, :40_000].clone()
    b_big[:, [0, 1, 2, 3, 4]] = b_store[:, rows]
    y_big = kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, a, b_big.cuda().t(), c.cuda(), bandwidth=8.0)[0]
    assert ko.rel_err_signed(y_big[:5], ref) < 5e-5
    assert _native.device_error_flag() == 0


@pytest.mark.skipif(not ref_kernels.available(), reason="reference cubin not built (baseline/_ref)")
@pytest.mark.parametrize("key, descriptor, hyper, ref_hyper", [
    ("laplace_l2", "kernel_descriptor_laplace_l2", dict(bandwidth=8.0), dict(bandwidth=8.0)),
    ("laplace_l1", "kernel_descriptor_laplace_l1", dict(bandwidth=40.0), dict(bandwidth=40.0)),
    ("gaussian_l2sq", None, dict(bandwidth=9.0), dict(bandwidth=9.0)),
])
def test_kernel_matvec_against_the_reference_kernels_matrix(key, descriptor, hyper, ref_hyper):
    # K(b, a) from the reference's own cute_build_kernel, times c in float64: a reference-produced y
    M, N, K, O = 8192, 4096, 64, 16
    g = torch.Generator().manual_seed(44)
    a = torch.randn(K, M, generator=g).cuda().t()
    b = torch.randn(K, N, generator=g).cuda().t()
    c = torch.randn(O, M, generator=g).cuda()
    kmat = torch.empty(N, M, device="cuda").t()                         # (M, N), m contiguous
    ref_kernels.ref_run_kernel(key, a, b, kmat, **ref_hyper)
    torch.cuda.synchronize()
    expected = (kmat.double().t() @ c.double().t())                     # (N, O)
    if descriptor is None:
        kd = kermac.KernelDescriptor(kermac.InnerOperator.DIFF, kermac.PowerType.SQUARE, kermac.PowerType.NOOP,
                                     kermac.KernelType.GAUSSIAN)
    else:
        kd = getattr(kermac, descriptor)
    for contraction in ("tensor", "fp32"):
        y = kermac.kernel_matvec(kd, a, b, c, contraction=contraction, **hyper)[0]
        err = float((y.double() - expected).abs().max() / expected.abs().max())
        assert err < 5e-5, (key, contraction, err)
    assert _native.device_error_flag() == 0
