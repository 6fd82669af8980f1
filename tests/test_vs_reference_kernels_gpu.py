"""Parity against the reference's OWN kernels, run on the same GPU.

baseline/build_ref_cubin.py compiles the reference's CUDA sources (in place, with NVRTC, the way
its JIT does) into baseline/_ref/; baseline/ref_kernels.py launches them through the driver API
with the reference's argument packing.  When that cubin is present these tests compare kermac_b200
with it on the reference's own test shapes; when it is not (no reference checkout at build time)
they are skipped.  Tolerances: 1e-5 (p in {1, 2}), 5e-5 (fractional p, gradients).
"""
import pytest
import torch

import kermac_b200 as kermac
from baseline import ref_kernels

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_kernels.available(), reason="reference cubin not built (baseline/_ref)")]


def gen(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32)


@pytest.mark.parametrize("p", [1.0, 1.3, 2.0])
@pytest.mark.parametrize("aligned", [True, False])
def test_cdist_matches_reference_kernel(p, aligned):
    # L=2, M=N=1000, K=64: the shape of the reference's tests/test_cdist.py, column-major operands
    L, M, N, K = 2, 1000, 1000, 64
    a = gen((L, K, M), 1).cuda().permute(0, 2, 1)
    b = gen((L, K, N), 2).cuda().permute(0, 2, 1)
    out_ref = torch.empty(L, N, M, device="cuda").permute(0, 2, 1)
    out_new = torch.empty(L, N, M, device="cuda").permute(0, 2, 1)
    ref_kernels.ref_cdist(a, b, out_ref, p, aligned=aligned)
    kermac.cdist(a, b, out=out_new, p=p)
    torch.cuda.synchronize()
    rel = ((out_new - out_ref).abs() / out_ref.abs().clamp_min(1e-30)).max().item()
    assert rel < (1e-5 if p in (1.0, 2.0) else 5e-5)


@pytest.mark.parametrize("p", [1.0, 1.5, 2.0])
def test_cdist_grad_matches_reference_kernel(p):
    # K=64, M=N=1000, O=16: the shape of the reference's tests/test_cdist_grad.py (one batch entry)
    K, M, N, O = 64, 1000, 1000, 16
    a, b, c, d = gen((K, M), 3).cuda(), gen((N, K), 4).cuda(), gen((O, K), 5).cuda(), gen((N, M), 6).cuda()
    out_ref = torch.empty(O, N, M, device="cuda")
    ref_kernels.ref_cdist_grad(a, b, c, d, out_ref, p)
    out_new = kermac.cdist_grad(a, b, c, d, p=p)[0]
    torch.cuda.synchronize()
    assert ((out_new - out_ref).abs().max() / out_ref.abs().max()).item() < 5e-5


def _cm(t):
    """Column-major copy: same values, first matrix index contiguous."""
    return t.transpose(-1, -2).contiguous().transpose(-1, -2)


CASES = [
    # key, descriptor, kermac kwargs, reference kwargs
    ("l2_raw", ("DIFF", "SQUARE", "NOOP", "NONE"), {}, {}),
    ("pow_raw", ("DIFF", "POW", "NOOP", "NONE"), dict(inner_p=1.7), dict(p_inner=1.7)),
    ("laplace_l1", ("DIFF", "ABS", "NOOP", "LAPLACE"), dict(bandwidth=5.0), dict(bandwidth=5.0)),
    ("laplace_l2", ("DIFF", "SQUARE", "SQRT", "LAPLACE"),
     dict(bandwidth=3.0, regularization=0.25, regularization_offset_x=3, regularization_offset_y=1, epsilon=1e-3),
     dict(bandwidth=3.0, regularization=0.25, off_x=3, off_y=1, epsilon=1e-3)),
    ("gaussian_l2sq", ("DIFF", "SQUARE", "NOOP", "GAUSSIAN"), dict(bandwidth=6.0), dict(bandwidth=6.0)),
    ("mma", ("DOT", "NOOP", "NOOP", "NONE"), {}, {}),
]


@pytest.mark.parametrize("key, desc, kw, ref_kw", CASES)
def test_run_kernel_descriptors_match_reference_kernel(key, desc, kw, ref_kw):
    # epilogues the reference's own tests never check numerically: compared here with its kernels
    L, M, N, K = 2, 704, 648, 48          # pitches that are multiples of 4: the ALIGN_4 instantiations need them
    a, b = _cm(gen((L, M, K), 7)).cuda(), _cm(gen((L, N, K), 8)).cuda()
    kd = kermac.KernelDescriptor(getattr(kermac.InnerOperator, desc[0]), getattr(kermac.PowerType, desc[1]),
                                 getattr(kermac.PowerType, desc[2]), getattr(kermac.KernelType, desc[3]))
    out_ref = torch.empty(L, N, M, device="cuda").permute(0, 2, 1)
    out_new = torch.empty(L, N, M, device="cuda").permute(0, 2, 1)
    ref_kernels.ref_run_kernel(key, a, b, out_ref, **ref_kw)
    kermac.run_kernel(kd, a, b, out=out_new, **kw)
    torch.cuda.synchronize()
    if key == "mma":
        assert ((out_new - out_ref).abs().max() / out_ref.abs().max()).item() < 1e-5
    else:
        assert ((out_new - out_ref).abs() / out_ref.abs().clamp_min(1e-30)).max().item() < 5e-5


def test_row_major_operands_match_reference_kernel():
    L, M, N, K = 2, 500, 450, 40
    a, b = gen((L, M, K), 9).cuda(), gen((L, N, K), 10).cuda()          # row-major (k contiguous)
    out_ref = torch.empty(L, N, M, device="cuda").permute(0, 2, 1)
    out_new = torch.empty(L, N, M, device="cuda").permute(0, 2, 1)
    ref_kernels.ref_run_kernel("cdist_p2_rowmajor", a, b, out_ref, a_row_major=True, b_row_major=True)
    kermac.cdist(a, b, out=out_new, p=2.0)
    assert ((out_new - out_ref).abs() / out_ref.abs().clamp_min(1e-30)).max().item() < 1e-5
    ref_kernels.ref_run_kernel("cdist_p1_row_col", a, _cm(b), out_ref, a_row_major=True)
    kermac.cdist(a, _cm(b), out=out_new, p=1.0)
    torch.cuda.synchronize()
    assert ((out_new - out_ref).abs() / out_ref.abs().clamp_min(1e-30)).max().item() < 1e-5
