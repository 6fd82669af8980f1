"""Pins the CPU oracle: against the formulations the reference's own tests use
(torch.cdist, tests/test_cdist.py:75; the einsum pair, tests/test_cdist_grad.py:43-49),
against the committed golden vectors, and against the independent C restatement."""
import os

import numpy as np
import pytest
import torch

from oracle import c_oracle
from oracle import kermac_oracle as ko

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _rand(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32)


@pytest.mark.parametrize("p", [1.0, 1.3, 2.0, 3.0])
def test_cdist_matches_torch_cdist_float64(p):
    a, b = _rand((2, 41, 17), 0), _rand((2, 33, 17), 1)
    ref = torch.cdist(a.double(), b.double(), p=p, compute_mode="donot_use_mm_for_euclid_dist")
    # for fractional p the exponents are float32 values (p and 1/p as the reference passes
    # them to its kernel), which moves the result by ~1e-7 relative to exact exponents
    assert ko.rel_err_nonneg(ko.cdist_ref(a, b, p=p), ref) < (1e-12 if p in (1.0, 2.0) else 5e-7)


@pytest.mark.parametrize("p", [1.0, 1.3, 2.0])
def test_cdist_golden_vectors(p):
    z = np.load(os.path.join(GOLDEN, "cdist_small.npz"))
    a, b = torch.from_numpy(z["a"]), torch.from_numpy(z["b"])
    tol = 1e-12 if p in (1.0, 2.0) else 5e-7
    assert ko.rel_err_nonneg(ko.cdist_ref(a, b, p=p), torch.from_numpy(z[f"cdist_p{p}"])) < tol


def test_skip_epilogue_is_the_raw_sum():
    a, b = _rand((30, 9), 2), _rand((20, 9), 3)
    for p in (1.3, 2.0):
        full = ko.cdist_ref(a, b, p=p)
        raw = ko.cdist_ref(a, b, p=p, skip_epilogue=True)
        # outer power uses float32(1)/float32(p), so compare at float32 resolution of the exponent
        assert torch.allclose(raw.pow(1.0 / p), full, rtol=1e-6, atol=0)


def test_broadcast_over_batch():
    a, b = _rand((3, 12, 7), 4), _rand((1, 10, 7), 5)
    out = ko.cdist_ref(a, b, p=1.3)
    for l in range(3):
        assert torch.equal(out[l], ko.cdist_ref(a[l], b[0], p=1.3)[0])


def test_grad_p2_matches_einsum_pair_and_golden():
    z = np.load(os.path.join(GOLDEN, "grad_small.npz"))
    a, b, c, d = (torch.from_numpy(z[k]) for k in "abcd")
    got = ko.cdist_grad_ref(a, b, c, d, p=2.0)
    assert ko.rel_err_signed(got, torch.from_numpy(z["grad_p2"])) < 1e-12
    coefs, km = c.double(), a.double()
    x, zz = b.double().permute(0, 2, 1), d.double().permute(0, 2, 1)
    ein = (torch.einsum('bli,bij,bjd->bljd', coefs, km, zz) - torch.einsum('bli,bij,bid->bljd', coefs, km, x))
    assert ko.rel_err_signed(got, ein.permute(0, 1, 3, 2)) < 1e-12


def test_grad_sign_convention_on_exact_ties():
    # d[n, m] == b[n, k] exactly: copysign(1, +0) = +1 for p = 1, contribution 0 for p > 1
    a = torch.ones(1, 1)
    b = torch.tensor([[0.5]])
    c = torch.tensor([[2.0]])
    d = torch.tensor([[0.5]])
    assert float(ko.cdist_grad_ref(a, b, c, d, p=1.0)) == 2.0
    assert float(ko.cdist_grad_ref(a, b, c, d, p=1.5)) == 0.0
    d_neg = torch.tensor([[0.25]])
    assert float(ko.cdist_grad_ref(a, b, c, d_neg, p=1.0)) == -2.0


@pytest.mark.parametrize("p", [1.0, 1.5, 2.0, 3.0])
def test_grad_is_the_derivative_of_cdist_pth_power(p):
    # d/dz sum_k |z - x_k|^p = p * sum_k sign(z - x_k) |z - x_k|^(p-1): check against autograd
    g = torch.Generator().manual_seed(7)
    K, M, N, O = 6, 5, 4, 3
    a = torch.rand(K, M, generator=g)
    x = torch.randn(N, K, generator=g)
    c = torch.randn(O, K, generator=g)
    zt = torch.randn(N, M, generator=g)
    z64 = zt.double().requires_grad_(True)
    # f[o, m] = sum_k c[o,k] a[k,m] sum_n |z[n,m] - x[n,k]|^p / p
    diff = z64.unsqueeze(1) - x.double().unsqueeze(2)           # (N, K, M)
    f = torch.einsum('ok,km,nkm->', c.double(), a.double(), diff.abs().pow(p)) / p
    (grad,) = torch.autograd.grad(f, z64)
    got = ko.cdist_grad_ref(a, x, c, zt, p=p)[0].sum(dim=0)      # sum over o matches the scalar f
    assert ko.rel_err_signed(got, grad) < 1e-10


DESCRIPTORS = [
    dict(inner_operator="DIFF", inner_power="ABS", outer_power="NOOP", kernel_type="NONE"),
    dict(inner_operator="DIFF", inner_power="SQUARE", outer_power="SQRT", kernel_type="NONE"),
    dict(inner_operator="DIFF", inner_power="POW", outer_power="POW", kernel_type="NONE"),
    dict(inner_operator="DIFF", inner_power="ABS", outer_power="NOOP", kernel_type="LAPLACE"),
    dict(inner_operator="DIFF", inner_power="SQUARE", outer_power="SQRT", kernel_type="LAPLACE"),
    dict(inner_operator="DIFF", inner_power="SQUARE", outer_power="NOOP", kernel_type="GAUSSIAN"),
    dict(inner_operator="DIFF", inner_power="NOOP", outer_power="ABS", kernel_type="NONE"),
    dict(inner_operator="DOT", inner_power="NOOP", outer_power="NOOP", kernel_type="NONE"),
    dict(inner_operator="DOT", inner_power="SQUARE", outer_power="SQRT", kernel_type="NONE"),
    dict(inner_operator="DOT", inner_power="ABS", outer_power="SQUARE", kernel_type="NONE"),
]


@pytest.mark.parametrize("desc", DESCRIPTORS)
def test_python_oracle_matches_c_restatement(desc):
    a, b = _rand((23, 11), 10), _rand((19, 11), 11)
    a = a.t().contiguous().t()            # column-major a exercises the stride arguments
    kw = {}
    c_kw = {}
    if desc["inner_power"] == "POW":
        kw["p"] = 1.3
        c_kw["p_inner"] = 1.3
        c_kw["p_outer"] = float(np.float32(1.0) / np.float32(1.3))
    if desc["kernel_type"] != "NONE":
        kw.update(bandwidth=2.5, regularization=0.25, reg_off_x=2, reg_off_y=0, epsilon=1e-3)
        c_kw.update(bandwidth=2.5, regularization=0.25, reg_off_x=2, reg_off_y=0, epsilon=1e-3)
    py = ko.build_kernel_ref(a, b, **desc, **kw)[0]
    cc = c_oracle.build_kernel_c(a, b, **desc, **c_kw)
    assert ko.rel_err_nonneg(py, cc) < 1e-12


@pytest.mark.parametrize("p", [1.0, 1.5, 2.0])
def test_python_grad_matches_c_restatement(p):
    a, b, c, d = _rand((9, 13), 20).abs(), _rand((7, 9), 21), _rand((3, 9), 22), _rand((7, 13), 23)
    assert ko.rel_err_signed(ko.cdist_grad_ref(a, b, c, d, p=p)[0], c_oracle.cdist_grad_c(a, b, c, d, p)) < 1e-12


def test_epsilon_mask_and_diagonal_overwrite():
    a = torch.tensor([[0.0, 0.0], [1.0, 0.0], [0.0, 2.0]])
    out = ko.build_kernel_ref(a, a, "DIFF", "SQUARE", "SQRT", "LAPLACE", bandwidth=1.0, regularization=0.5)[0]
    assert torch.equal(out.diagonal(), torch.full((3,), 1.5, dtype=torch.float64))
    out0 = ko.build_kernel_ref(a, a, "DIFF", "SQUARE", "SQRT", "LAPLACE", bandwidth=1.0)[0]
    assert torch.equal(out0.diagonal(), torch.ones(3, dtype=torch.float64))   # distance 0 < eps -> exp(0)
    assert abs(float(out0[0, 1]) - np.exp(-1.0)) < 1e-15
    near = torch.tensor([[1e-6, 0.0]])
    masked = ko.build_kernel_ref(near, torch.zeros(1, 2), "DIFF", "ABS", "NOOP", "LAPLACE", bandwidth=1e-6)[0]
    assert float(masked) == 1.0                                              # 1e-6 < 1e-5 is masked to 0


def test_kernel_matvec_is_build_then_product():
    a, b, c = _rand((31, 5), 30), _rand((17, 5), 31), _rand((4, 31), 32)
    y = ko.kernel_matvec_ref(a, b, c, inner_operator="DIFF", inner_power="SQUARE", outer_power="SQRT",
                             kernel_type="LAPLACE", bandwidth=3.0)
    kmat = torch.exp(-torch.cdist(a.double(), b.double()) / 3.0)
    assert ko.rel_err_signed(y[0], kmat.t() @ c.double().t()) < 1e-12
