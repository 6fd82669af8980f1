"""GPU parity of the fused kernel_matvec against the float64 CPU oracle, through the C-ABI.
Tolerance: max |y - ref| / max |ref| <= 5e-5.  Every test runs once per contraction mode
(tcgen05 tensor cores with three tf32 products per term, and packed FP32 FMAs)."""
import pytest
import torch

import kermac_b200 as kermac
from kermac_b200 import _native
from oracle import kermac_oracle as ko

pytestmark = pytest.mark.gpu
TOL = 5e-5
LAPLACE_L2 = dict(inner_operator="DIFF", inner_power="SQUARE", outer_power="SQRT", kernel_type="LAPLACE")


@pytest.fixture(autouse=True, params=["tensor", "fp32"])
def contraction(request, monkeypatch):
    monkeypatch.setenv("KERMAC_B200_CONTRACTION", request.param)
    return request.param


def gen(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32)


def col_major(t):
    return t.transpose(-1, -2).contiguous().transpose(-1, -2)


@pytest.mark.parametrize("O", [1, 2, 3, 4, 8, 16, 21])
def test_laplace_matvec_equals_build_then_product(O):
    M, N, K = 700, 300, 64
    a, b, c = gen((M, K), 1), gen((N, K), 2), gen((O, M), 3)
    ref = ko.kernel_matvec_ref(a, b, c, **LAPLACE_L2, bandwidth=8.0)
    for a_d, b_d in ((a.cuda(), b.cuda()), (col_major(a).cuda(), col_major(b).cuda())):
        y = kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, a_d, b_d, c.cuda(), bandwidth=8.0)
        assert tuple(y.shape) == (1, N, O)
        assert ko.rel_err_signed(y, ref) < TOL
    # same numbers as materialising the kernel matrix with run_kernel and multiplying
    kmat = kermac.run_kernel(kermac.kernel_descriptor_laplace_l2, a.cuda(), b.cuda(), bandwidth=8.0)[0]
    y2 = (kmat.double().t() @ c.cuda().double().t())
    assert ko.rel_err_signed(y[0], y2.cpu()) < TOL


@pytest.mark.parametrize("shape", [(1, 1, 1), (5, 3, 2), (129, 127, 17), (257, 130, 33), (1000, 5, 64)])
def test_odd_shapes(shape):
    M, N, K = shape
    a, b, c = gen((M, K), 4), gen((N, K), 5), gen((5, M), 6)
    y = kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l1, a.cuda(), b.cuda(), c.cuda(), bandwidth=5.0)
    ref = ko.kernel_matvec_ref(a, b, c, inner_operator="DIFF", inner_power="ABS", outer_power="NOOP",
                               kernel_type="LAPLACE", bandwidth=5.0)
    assert ko.rel_err_signed(y, ref) < TOL


def test_other_descriptors_batches_and_output_views():
    L, M, N, K, O = 2, 400, 150, 20, 6
    a, b, c = gen((L, M, K), 7), gen((N, K), 8), gen((L, O, M), 9)
    gauss = kermac.KernelDescriptor(kermac.InnerOperator.DIFF, kermac.PowerType.SQUARE, kermac.PowerType.NOOP,
                                    kermac.KernelType.GAUSSIAN)
    big = torch.full((L, N, O + 3), -1.0, device="cuda")
    out = big[:, :, 1:O + 1]
    y = kermac.kernel_matvec(gauss, a.cuda(), b.cuda(), c.cuda(), out=out, bandwidth=3.0)
    assert y is out
    ref = ko.kernel_matvec_ref(a, b, c, inner_operator="DIFF", inner_power="SQUARE", outer_power="NOOP",
                               kernel_type="GAUSSIAN", bandwidth=3.0)
    assert ko.rel_err_signed(y, ref) < TOL
    assert float(big[:, :, 0].max()) == -1.0 and float(big[:, :, O + 1:].max()) == -1.0
    y = kermac.kernel_matvec(kermac.kernel_descriptor_p_norm, a.cuda(), b.cuda(), c.cuda(), p=1.5)
    ref = ko.kernel_matvec_ref(a, b, c, inner_operator="DIFF", inner_power="POW", outer_power="POW",
                               kernel_type="NONE", p=1.5)
    assert ko.rel_err_signed(y, ref) < TOL
    y = kermac.kernel_matvec(kermac.kernel_descriptor_mma, a.cuda(), b.cuda(), c.cuda())
    ref = torch.einsum('lmk,nk,lom->lno', a.double(), b.double(), c.double())
    assert ko.rel_err_signed(y, ref) < TOL


@pytest.mark.parametrize("split", [2, 3, 7])
def test_split_m_is_deterministic_and_matches(split):
    M, N, K, O = 5000, 260, 64, 16
    a, b, c = col_major(gen((M, K), 10)), col_major(gen((N, K), 11)), gen((O, M), 12)
    ref = ko.kernel_matvec_ref(a, b, c, **LAPLACE_L2, bandwidth=8.0)
    y1 = kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, a.cuda(), b.cuda(), c.cuda(), bandwidth=8.0,
                              split_m=split)
    y2 = kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, a.cuda(), b.cuda(), c.cuda(), bandwidth=8.0,
                              split_m=split)
    assert torch.equal(y1, y2)
    assert ko.rel_err_signed(y1, ref) < TOL


def test_matvec_configuration_shape_sampled_rows():
    # the fused-matvec configuration scaled in M and N (K=64, O=16, sigma=8, seed 4); linearity in c
    # and the oracle on sampled rows are size-independent checks
    K, M, N, O = 64, 200_000, 4096, 16
    g = torch.Generator().manual_seed(4)
    a_store = torch.randn(K, M, generator=g)
    b_store = torch.randn(K, N, generator=g)
    c = torch.randn(O, M, generator=g)
    a, b = a_store.t(), b_store.t()
    y = kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, a.cuda(), b.cuda(), c.cuda(), bandwidth=8.0)[0]
    rows = torch.tensor([0, 127, 128, 2049, 4095])
    ref = ko.kernel_matvec_ref(a, b, c, n_rows=rows, **LAPLACE_L2, bandwidth=8.0)[0]
    assert ko.rel_err_signed(y[rows.cuda()], ref) < TOL
    y2 = kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, a.cuda(), b.cuda(), (2.0 * c).cuda(), bandwidth=8.0)[0]
    assert torch.equal(y2, 2.0 * y)          # scaling c by a power of two scales every partial sum exactly


def test_tensor_contraction_keeps_fp32_accuracy():
    # One tf32 product per term would be off by ~1e-4 .. 1e-3; the three-product split has to stay
    # at the level of the FP32 contraction.  Coefficients of one sign: no cancellation hides errors.
    M, N, K, O = 6000, 384, 32, 16
    a, b = gen((M, K), 20), gen((N, K), 21)
    c = gen((O, M), 22).abs() + 0.5
    ref = ko.kernel_matvec_ref(a, b, c, **LAPLACE_L2, bandwidth=8.0)
    errs = {}
    for mode in ("tensor", "fp32"):
        y = kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, a.cuda(), b.cuda(), c.cuda(), bandwidth=8.0,
                                 contraction=mode)
        errs[mode] = ko.rel_err_nonneg(y, ref)
    assert errs["fp32"] < 2e-6
    assert errs["tensor"] < 2e-6, errs
    assert _native.device_error_flag() == 0, "a bounded wait inside the kernel ran out"


def test_contraction_argument_is_validated():
    a, b, c = gen((8, 4), 1).cuda(), gen((8, 4), 2).cuda(), gen((2, 8), 3).cuda()
    with pytest.raises(ValueError):
        kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, a, b, c, bandwidth=1.0, contraction="bf16")


@pytest.mark.parametrize("shape", [(1028, 260, 20), (132, 128, 1), (516, 4, 33), (4100, 388, 64)])
def test_m_contiguous_operands(shape):
    # a[K, M] / b[K, N] storage with 16-byte aligned rows: the TMA-staged variant of the tensor kernel
    # (partial m / n tiles, partial and single k slabs), batched with a broadcast b
    M, N, K = shape
    L, O = 2, 7
    a, b, c = col_major(gen((L, M, K), 30)), col_major(gen((N, K), 31)), gen((L, O, M), 32)
    y = kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, a.cuda(), b.cuda(), c.cuda(), bandwidth=6.0)
    ref = ko.kernel_matvec_ref(a, b, c, **LAPLACE_L2, bandwidth=6.0)
    assert ko.rel_err_signed(y, ref) < TOL
    y = kermac.kernel_matvec(kermac.kernel_descriptor_mma, a.cuda(), b.cuda(), c.cuda())
    ref = torch.einsum('lmk,nk,lom->lno', a.double(), b.double(), c.double())
    assert ko.rel_err_signed(y, ref) < TOL
    assert _native.device_error_flag() == 0, "a bounded wait inside the kernel ran out"


@pytest.mark.parametrize("layout", ["row", "col"])
def test_diagonal_rule_gives_regularised_product(layout):
    # square K(X, X): the diagonal becomes 1 + lambda, so y = (K + lambda I) c since K(x, x) = 1
    M, K, O, lam = 900, 24, 5, 0.37
    x, c = gen((M, K), 40), gen((O, M), 41)
    xd = (col_major(x) if layout == "col" else x).cuda()
    y = kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, xd, xd, c.cuda(), bandwidth=4.0, regularization=lam)
    ref = ko.kernel_matvec_ref(x, x, c, **LAPLACE_L2, bandwidth=4.0, regularization=lam)
    assert ko.rel_err_signed(y, ref) < TOL
    plain = ko.kernel_matvec_ref(x, x, c, **LAPLACE_L2, bandwidth=4.0)
    assert ko.rel_err_signed(ref, plain + lam * c.t().double().unsqueeze(0)) < 1e-7     # lambda is rounded to fp32
    # shifted diagonal, rectangular operands, split over m, per-batch lambda
    L, N = 2, 300
    a, b, cc = gen((L, M, K), 42), gen((N, K), 43), gen((L, O, M), 44)
    lam_t = torch.tensor([0.5, -0.25])
    for split in (0, 3):
        y = kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l1, a.cuda(), b.cuda(), cc.cuda(), bandwidth=9.0,
                                 regularization=lam_t.cuda(), regularization_offset_x=-200, regularization_offset_y=57,
                                 split_m=split)
        ref = ko.kernel_matvec_ref(a, b, cc, inner_operator="DIFF", inner_power="ABS", outer_power="NOOP",
                                   kernel_type="LAPLACE", bandwidth=9.0, regularization=lam_t, reg_off_x=-200, reg_off_y=57)
        assert ko.rel_err_signed(y, ref) < TOL
