"""GPU tests of the symmetric build: when a and b are the same matrix, only the tiles on and above the
diagonal are computed and mirrored.  The result has to equal the full computation bit for bit
(to rounding for the fractional power, whose exp2 takes one of two routes)."""
import pytest
import torch

import kermac_b200 as kermac
from kermac_b200 import _native
from kermac_b200.build_a_kernel import _marshal_build
from oracle import kermac_oracle as ko

pytestmark = pytest.mark.gpu


def gen(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32)


def col_major(t):
    return t.transpose(-1, -2).contiguous().transpose(-1, -2)


def _describe(desc, a, b, **kw):
    args, _, _ = _marshal_build(desc, a, b, None, kw.get("p"), None, None, kw.get("bandwidth"), None,
                                kw.get("regularization"), kw.get("regularization_offset_x", 0),
                                kw.get("regularization_offset_y", 0))
    return _native.describe_build(args)


@pytest.mark.parametrize("layout", ["row", "col"])
@pytest.mark.parametrize("M,K", [(129, 8), (700, 40), (1030, 130)])
@pytest.mark.parametrize("p", [1.0, 2.0, 1.3])
def test_cdist_of_a_matrix_with_itself(monkeypatch, layout, M, K, p):
    x = gen((M, K), 50 + M)
    xd = (col_major(x) if layout == "col" else x).cuda()
    assert "symmetric=1" in _describe(kermac.kernel_descriptor_l1_norm, xd, xd)
    sym = kermac.cdist(xd, xd, p=p)
    monkeypatch.setenv("KERMAC_B200_SYMMETRY", "off")
    full = kermac.cdist(xd, xd, p=p)
    if p in (1.0, 2.0):
        assert torch.equal(sym, full)
        assert torch.equal(sym, sym.transpose(1, 2))
    else:
        # |.|^p evaluates exp2 by one of two routes depending on the element's place in its tile, so a
        # mirrored value can differ from the directly computed one in the last bits
        assert ko.rel_err_nonneg(sym, full.cpu().double()) < 2e-6
    tol = 1e-5 if p in (1.0, 2.0) else 5e-5
    ref = ko.cdist_ref(x, x, p=p)
    # the p = 2 diagonal is sqrt(0) = 0 in both; compare off-diagonal entries relatively
    assert ko.rel_err_nonneg(sym, ref) < tol
    assert _native.device_error_flag() == 0


def test_symmetric_kernel_matrix_with_diagonal_rule_batches_and_views(monkeypatch):
    L, M, K = 3, 520, 33
    x = gen((L, M, K), 60)
    xd = col_major(x).cuda()
    lam = torch.tensor([0.1, 0.0, 2.0]).cuda()
    for out_layout in ("m", "n"):
        outs = []
        for mode in ("auto", "off"):
            monkeypatch.setenv("KERMAC_B200_SYMMETRY", mode)
            big = torch.full((L, M + 8, M + 4), -7.0, device="cuda")
            # (M, N) views of a larger buffer with stride 1 along n, or along m
            out = big[:, 4:M + 4, :M] if out_layout == "n" else big.transpose(1, 2)[:, :M, 4:M + 4]
            kermac.run_kernel(kermac.kernel_descriptor_laplace_l2, xd, xd, out=out, bandwidth=5.0, regularization=lam,
                              regularization_offset_x=3, regularization_offset_y=3)
            outs.append((out.clone(), big))
        assert torch.equal(outs[0][0], outs[1][0])
        assert torch.equal(outs[0][1], outs[1][1])        # nothing outside the view was touched
        ref = ko.build_kernel_ref(x, x, "DIFF", "SQUARE", "SQRT", "LAPLACE", bandwidth=5.0, regularization=lam.cpu(),
                                  reg_off_x=3, reg_off_y=3)
        assert ko.rel_err_nonneg(outs[0][0], ref) < 5e-5
    monkeypatch.setenv("KERMAC_B200_SYMMETRY", "auto")
    # product kernel
    g = kermac.run_kernel(kermac.kernel_descriptor_mma, xd, xd)
    assert ko.rel_err_signed(g, torch.einsum('lmk,lnk->lmn', x.double(), x.double())) < 1e-5
    assert torch.equal(g, g.transpose(1, 2))


def test_symmetry_is_not_assumed_when_it_does_not_hold():
    M, K = 300, 16
    x = gen((M, K), 70).cuda()
    y = x.clone()
    # different storage, signed chain, unequal diagonal offsets, different views of one buffer
    assert "symmetric=0" in _describe(kermac.kernel_descriptor_l1_norm, x, y)
    signed = kermac.KernelDescriptor(kermac.InnerOperator.DIFF, kermac.PowerType.NOOP, kermac.PowerType.NOOP,
                                     kermac.KernelType.NONE)
    assert "symmetric=0" in _describe(signed, x, x)
    assert "symmetric=0" in _describe(kermac.kernel_descriptor_laplace_l2, x, x, bandwidth=1.0, regularization=0.5,
                                      regularization_offset_x=1)
    assert "symmetric=0" in _describe(kermac.kernel_descriptor_l1_norm, x[:200], x[100:])
    assert "symmetric=0" in _describe(kermac.kernel_descriptor_l1_norm, x[:100], x[:100])     # a single tile
    d = kermac.run_kernel(signed, x, x)
    assert ko.rel_err_signed(d, ko.build_kernel_ref(x.cpu(), x.cpu(), "DIFF", "NOOP", "NOOP", "NONE")) < 1e-5
