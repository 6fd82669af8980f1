"""Host layer of the kermac API with the launch stubbed at the C-ABI boundary: layout
classification, batch merging, validation errors and the marshalled arguments."""
import numpy as np
import pytest
import torch

import kermac_b200 as kermac
import importlib

from kermac_b200 import _native

# the package re-exports functions named like their modules, so fetch the modules by path
build_a_kernel = importlib.import_module("kermac_b200.build_a_kernel")
cdist_grad_mod = importlib.import_module("kermac_b200.cdist_grad")
matvec_mod = importlib.import_module("kermac_b200.matvec")


@pytest.fixture
def recorder(monkeypatch):
    """CPU tensors stand in for device tensors; launches are recorded, not executed."""
    calls = []
    for mod in (build_a_kernel, cdist_grad_mod, matvec_mod):
        monkeypatch.setattr(mod, "_is_cuda", lambda t: True)
        monkeypatch.setattr(mod, "_current_stream_for", lambda device: 0)
    monkeypatch.setattr(_native, "launch_build", lambda args, stream: calls.append(("build", args)))
    monkeypatch.setattr(_native, "launch_grad", lambda args, stream: calls.append(("grad", args)))
    monkeypatch.setattr(_native, "launch_matvec", lambda args, stream: calls.append(("matvec", args)))
    return calls


# ------------------------------------------------------------------ common helpers
def test_tensor_stats_layouts_and_alignment():
    row = torch.zeros(5, 8)
    s = kermac.tensor_stats(row)
    assert s.majorness is kermac.Majorness.ROW_MAJOR and s.alignment is kermac.Alignment.ALIGN_1
    assert s.shape == (1, 5, 8) and s.leading_dimension_stride == 8 and s.batch_stride == 0
    col = torch.zeros(8, 8).t()[:5]              # shape (5, 8), strides (1, 8)
    s = kermac.tensor_stats(col)
    assert s.majorness is kermac.Majorness.COL_MAJOR and s.alignment is kermac.Alignment.ALIGN_4
    assert s.matrix_strides == (1, 8)
    odd = torch.zeros(8, 9).t()[:5, :8]          # strides (1, 9): pitch not a multiple of 4
    assert kermac.tensor_stats(odd).alignment is kermac.Alignment.ALIGN_1
    batched = torch.zeros(3, 4, 6)
    assert kermac.tensor_stats(batched).batch_stride == 24
    assert kermac.tensor_stats(batched[:1]).batch_stride == 0      # a batch of one broadcasts
    with pytest.raises(ValueError, match="non-standard memory layout"):
        kermac.tensor_stats(torch.zeros(8, 16)[:, ::2])
    with pytest.raises(TypeError):
        kermac.tensor_stats(torch.zeros(4, 4, dtype=torch.float64))
    with pytest.raises(ValueError):
        kermac.tensor_stats(torch.zeros(4))


def test_merge_batch_size_rules():
    m = kermac.merge_batch_size
    assert m('x', 1, None, 0, can_be_none=True) == 1
    assert m('x', 4, 1.5, 0) == 4
    assert m('x', 1, torch.zeros(3, 2, 2), 2) == 3
    assert m('x', 3, torch.zeros(1, 2, 2), 2) == 3
    assert m('x', 3, torch.zeros(2, 2), 2) == 3
    with pytest.raises(ValueError, match="does not match"):
        m('x', 3, torch.zeros(2, 2, 2), 2)
    with pytest.raises(ValueError, match="is none"):
        m('x', 1, None, 0)
    with pytest.raises(ValueError, match="is a float"):
        m('x', 1, 2.0, 2)
    with pytest.raises(ValueError, match="number of dimensions"):
        m('x', 1, torch.zeros(2), 2)
    assert kermac.ceil_div(129, 128) == 2 and kermac.ceil_div(128, 128) == 1


# ------------------------------------------------------------------ run_kernel / cdist
def test_cdist_selects_descriptor_by_p(recorder):
    a, b = torch.zeros(6, 4), torch.zeros(5, 4)
    for p, expect in ((1.0, (_native.POW_ABS, _native.POW_NOOP)), (2.0, (_native.POW_SQUARE, _native.POW_SQRT)),
                      (1.3, (_native.POW_POW, _native.POW_POW))):
        out = kermac.cdist(a, b, p=p)
        args = recorder[-1][1]
        assert (args.inner_power, args.outer_power) == expect
        assert args.inner_operator == _native.INNER_DIFF and args.kernel_type == _native.KERNEL_NONE
        assert tuple(out.shape) == (1, 6, 5)
        assert (args.m, args.n, args.k, args.l) == (6, 5, 4, 1)
    args = recorder[-1][1]
    assert args.p_inner.ptr is None and args.p_inner.value == np.float32(1.3)
    assert args.p_outer.value == np.float32(1.0) / np.float32(1.3)


def test_skip_epilogue_does_not_leak_into_later_calls(recorder):
    a, b = torch.zeros(6, 4), torch.zeros(5, 4)
    kermac.cdist(a, b, p=2.0, skip_epilogue=True)
    assert recorder[-1][1].outer_power == _native.POW_NOOP
    kermac.cdist(a, b, p=2.0)
    assert recorder[-1][1].outer_power == _native.POW_SQRT
    assert kermac.kernel_descriptor_l2_norm._outer_power is kermac.PowerType.SQRT
    kermac.cdist(a, b, p=1.3, skip_epilogue=True)          # raises in the reference; defined here
    args = recorder[-1][1]
    assert (args.inner_power, args.outer_power) == (_native.POW_POW, _native.POW_NOOP)
    assert args.p_inner.value == np.float32(1.3)
    kermac.cdist(a, b, p=1.3)
    assert recorder[-1][1].outer_power == _native.POW_POW


def test_strides_and_batch_strides_are_marshalled(recorder):
    a = torch.zeros(3, 4, 6).permute(0, 2, 1)       # (3, 6, 4) column-major: strides (24, 1, 6)
    b = torch.zeros(5, 4)                           # broadcast over the batch
    out = torch.zeros(3, 5, 6).permute(0, 2, 1)     # (3, 6, 5) with m contiguous
    assert kermac.cdist(a, b, out=out, p=1.0) is out
    args = recorder[-1][1]
    assert (args.a_stride_m, args.a_stride_k, args.a_stride_l) == (1, 6, 24)
    assert (args.b_stride_n, args.b_stride_k, args.b_stride_l) == (4, 1, 0)
    assert (args.out_stride_m, args.out_stride_n, args.out_stride_l) == (1, 6, 30)
    assert args.l == 3 and args.a == a.data_ptr() and args.out == out.data_ptr()


def test_hyper_parameters_scalar_and_tensor(recorder):
    a, b = torch.zeros(2, 6, 4), torch.zeros(2, 5, 4)
    bw = torch.tensor([1.0, 2.0])
    kermac.run_kernel(kermac.kernel_descriptor_laplace_l2, a, b, bandwidth=bw, regularization=0.5,
                      regularization_offset_x=3, epsilon=1e-3)
    args = recorder[-1][1]
    assert args.bandwidth.ptr == bw.data_ptr() and args.bandwidth.batch_stride == 1
    assert args.regularization.ptr is None and args.regularization.value == 0.5
    assert (args.reg_off_x, args.reg_off_y) == (3, 0) and args.epsilon == np.float32(1e-3)
    assert args.kernel_type == _native.KERNEL_LAPLACE
    kermac.run_kernel(kermac.kernel_descriptor_laplace_l1, a, b, bandwidth=4.0)
    assert recorder[-1][1].epsilon == np.float32(1e-5)                 # default epsilon
    p = torch.tensor([1.5, 3.0])
    kermac.run_kernel(kermac.kernel_descriptor_p_norm, a, b, p=p)
    args = recorder[-1][1]
    assert args.p_inner.batch_stride == 1 and args.p_outer.batch_stride == 1 and args.p_outer.ptr is not None
    with pytest.raises(ValueError, match="does not match"):
        kermac.run_kernel(kermac.kernel_descriptor_p_norm, a, b, p=torch.tensor([1.0, 2.0, 3.0]))


@pytest.mark.parametrize("kwargs, message", [
    (dict(desc="p_norm"), "'p' and 'inner_p' is not set"),
    (dict(desc="l2_norm", p=2.0), "is not 'Pow' but 'p' or 'inner_p' is set"),
    (dict(desc="l2_norm", bandwidth=1.0), "'KernelType' is 'None'"),
    (dict(desc="laplace_l2"), "'bandwidth' is not set"),
    (dict(desc="p_norm", p=1.5, inner_p=1.5), "'inner_p' is also not"),
    (dict(desc="p_norm", p=1.5, outer_p=1.5), "'outer_p' is also not"),
])
def test_descriptor_argument_consistency_errors(recorder, kwargs, message):
    desc = getattr(kermac, "kernel_descriptor_" + kwargs.pop("desc"))
    with pytest.raises(ValueError, match=message):
        kermac.run_kernel(desc, torch.zeros(4, 3), torch.zeros(5, 3), **kwargs)
    assert not recorder


def test_operand_validation_errors(recorder):
    d = kermac.kernel_descriptor_l2_norm
    a, b = torch.zeros(4, 3), torch.zeros(5, 3)
    with pytest.raises(TypeError, match="PyTorch tensors"):
        kermac.run_kernel(d, a.numpy(), b)
    with pytest.raises(TypeError, match="float32"):
        kermac.run_kernel(d, a.double(), b)
    with pytest.raises(ValueError, match="K dimensions must match"):
        kermac.run_kernel(d, a, torch.zeros(5, 2))
    with pytest.raises(ValueError, match="out must have shape"):
        kermac.run_kernel(d, a, b, out=torch.zeros(4, 4))
    with pytest.raises(ValueError, match="batch dimension"):
        kermac.run_kernel(d, torch.zeros(3, 4, 3), b, out=torch.zeros(1, 4, 5))
    with pytest.raises(ValueError, match="non-standard memory layout"):
        kermac.run_kernel(d, torch.zeros(4, 6)[:, ::2], b)
    with pytest.raises(TypeError, match="`bandwidth` tensor must have dtype"):
        kermac.run_kernel(kermac.kernel_descriptor_laplace_l2, a, b, bandwidth=torch.tensor(1.0, dtype=torch.float64))
    assert not recorder


def test_cpu_tensors_are_rejected_without_the_stub():
    with pytest.raises(ValueError, match="must be on a CUDA device"):
        kermac.cdist(torch.zeros(4, 3), torch.zeros(5, 3))
    with pytest.raises(ValueError, match="must be on a CUDA device"):
        kermac.cdist_grad(torch.zeros(3, 4), torch.zeros(5, 3), torch.zeros(2, 3), torch.zeros(5, 4))


def test_pre_compile_descriptors_keeps_its_signature():
    kermac.pre_compile_descriptors(device=torch.device('cpu'),
                                   descriptors=[kermac.kernel_descriptor_l1_norm, kermac.kernel_descriptor_p_norm],
                                   try_to_align=True, debug=False)
    kermac.ModuleCache(False).compile_and_cache_functions(device=None, function_names=[])


def test_variant_env_override(recorder, monkeypatch):
    a, b = torch.zeros(6, 4), torch.zeros(5, 4)
    monkeypatch.setenv("KERMAC_B200_VARIANT", "cpasync")
    kermac.cdist(a, b)
    assert recorder[-1][1].variant == _native.VARIANT_CPASYNC
    monkeypatch.setenv("KERMAC_B200_VARIANT", "bogus")
    with pytest.raises(ValueError, match="KERMAC_B200_VARIANT"):
        kermac.cdist(a, b)


# ------------------------------------------------------------------ cdist_grad
def _grad_inputs(L=None, K=7, M=6, N=5, O=3):
    lead = () if L is None else (L,)
    return (torch.zeros(*lead, K, M), torch.zeros(*lead, N, K), torch.zeros(*lead, O, K), torch.zeros(*lead, N, M))


def test_cdist_grad_marshalling_and_norm_selection(recorder, monkeypatch):
    monkeypatch.setattr(_native, "lib", lambda: type("L", (), {
        "kermac_b200_cdist_grad_scratch_bytes": staticmethod(lambda ref: 0)})())
    a, b, c, d = _grad_inputs(L=2)
    out = kermac.cdist_grad(a, b, c, d, p=1.0)
    args = recorder[-1][1]
    assert tuple(out.shape) == (2, 3, 5, 6)
    assert (args.m, args.n, args.o, args.k, args.l) == (6, 5, 3, 7, 2)
    assert args.norm_type == _native.NORM_L1
    assert (args.lda, args.ldb, args.ldc, args.ldd) == (6, 7, 7, 6)
    assert (args.out_stride_n, args.out_stride_o, args.out_stride_l) == (6, 30, 90)
    kermac.cdist_grad(a, b, c, d, p=2.0)
    assert recorder[-1][1].norm_type == _native.NORM_L2
    kermac.cdist_grad(a, b, c, d, p=1.5)
    assert recorder[-1][1].norm_type == _native.NORM_P and recorder[-1][1].p.value == 1.5
    pt = torch.tensor([1.5, 2.5])
    kermac.cdist_grad(a, b, c, d, p=pt)
    assert recorder[-1][1].norm_type == _native.NORM_P and recorder[-1][1].p.ptr == pt.data_ptr()
    # where the products with c run: KM_CONTRACT_AUTO / _FP32 / _TENSOR
    assert recorder[-1][1].contraction == 0
    kermac.cdist_grad(a, b, c, d, p=1.0, contraction="fp32")
    assert recorder[-1][1].contraction == 1
    kermac.cdist_grad(a, b, c, d, p=1.0, contraction="tensor")
    assert recorder[-1][1].contraction == 2
    # a 3-D out with a batch of one is read as unbatched
    a1, b1, c1, d1 = _grad_inputs()
    out3 = torch.zeros(3, 5, 6)
    assert kermac.cdist_grad(a1, b1, c1, d1, out=out3) is out3
    assert recorder[-1][1].out_stride_l == 0


def test_cdist_grad_validation_errors(recorder):
    a, b, c, d = _grad_inputs()
    with pytest.raises(ValueError, match="Expected shape"):
        kermac.cdist_grad(a, torch.zeros(5, 8), c, d)
    with pytest.raises(ValueError, match="stride 1 in last dimension"):
        kermac.cdist_grad(torch.zeros(6, 7).t(), b, c, d)
    with pytest.raises(ValueError, match="3-dimensional or 4-dimensional"):
        kermac.cdist_grad(a, b, c, d, out=torch.zeros(5, 6))
    with pytest.raises(ValueError, match="Expected shape"):
        kermac.cdist_grad(a, b, c, d, out=torch.zeros(3, 5, 7))
    with pytest.raises(TypeError):
        kermac.cdist_grad(a, b, c, d.double())
    with pytest.raises(ValueError, match="contraction must be one of"):
        kermac.cdist_grad(a, b, c, d, contraction="bf16")
    assert not recorder


# ------------------------------------------------------------------ kernel_matvec
def test_kernel_matvec_marshalling(recorder, monkeypatch):
    monkeypatch.setattr(_native, "lib", lambda: type("L", (), {
        "kermac_b200_kernel_matvec_scratch_bytes": staticmethod(lambda ref: 0)})())
    a, b, c = torch.zeros(9, 4), torch.zeros(7, 4), torch.zeros(3, 9)
    y = kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, a, b, c, bandwidth=8.0)
    args = recorder[-1][1]
    assert tuple(y.shape) == (1, 7, 3)
    assert (args.m, args.n, args.k, args.o, args.l) == (9, 7, 4, 3, 1)
    assert (args.y_stride_n, args.y_stride_o) == (3, 1) and args.ldc == 9
    assert args.bandwidth.value == 8.0 and args.kernel_type == _native.KERNEL_LAPLACE
    with pytest.raises(ValueError, match="c must have shape"):
        kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, a, b, torch.zeros(3, 8), bandwidth=8.0)
    with pytest.raises(ValueError, match="'bandwidth' is not set"):
        kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, a, b, c)
    # contraction mode, diagonal rule
    assert args.contraction == 0 and args.regularization.value == 0.0
    monkeypatch.setenv("KERMAC_B200_CONTRACTION", "fp32")
    kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, a, b, c, bandwidth=8.0, regularization=0.5,
                         regularization_offset_x=3, regularization_offset_y=-2)
    args = recorder[-1][1]
    assert args.contraction == 1 and args.regularization.value == 0.5 and (args.reg_off_x, args.reg_off_y) == (3, -2)
    kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, a, b, c, bandwidth=8.0, contraction="tensor")
    assert recorder[-1][1].contraction == 2
    with pytest.raises(ValueError, match="contraction must be one of"):
        kermac.kernel_matvec(kermac.kernel_descriptor_laplace_l2, a, b, c, bandwidth=8.0, contraction="bf16")
    with pytest.raises(ValueError, match="'KernelType' is 'None'"):
        kermac.kernel_matvec(kermac.kernel_descriptor_l2_norm, a, b, c, regularization=0.1)


def test_host_pipeline_slab_plan_covers_the_rows():
    from kermac_b200.host import HostCdist
    assert HostCdist.slab_plan(30000, 8) == [3840] * 7 + [3120]
    assert HostCdist.slab_plan(30000, 47) == [640] * 46 + [560]
    assert HostCdist.slab_plan(1100, 5) == [256, 256, 256, 256, 76]
    assert HostCdist.slab_plan(100, 4) == [100] and HostCdist.slab_plan(0, 3) == []
    for n, slabs in [(1, 1), (129, 2), (4097, 3), (100000, 16), (30000, 32)]:
        plan = HostCdist.slab_plan(n, slabs)
        assert sum(plan) == n and all(s > 0 for s in plan)
        assert all(s % 128 == 0 for s in plan[:-1])            # every slab but the last starts on a tile boundary
