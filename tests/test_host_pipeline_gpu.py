"""HostCdist: cdist with operands and result in (pinned) host memory, slabs overlapped."""
import pytest
import torch

from kermac_b200.host import HostCdist
from oracle import kermac_oracle as ko

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("p", [1.0, 2.0, 1.3])
def test_host_pipeline_matches_oracle_and_reuses_its_buffers(p):
    K, M, N = 48, 900, 1100                     # 1100 rows -> slabs of 256 / 256 / 256 / 256 / 76
    g = torch.Generator().manual_seed(5)
    a_store = torch.randn(K, M, generator=g).pin_memory()
    b_store = torch.randn(K, N, generator=g).pin_memory()
    out = torch.empty(N, M).pin_memory()
    pipe = HostCdist(M, N, K, slabs=5)
    assert pipe.h2d_bytes == 4 * K * (M + N) and pipe.d2h_bytes == 4 * N * M
    ref = ko.cdist_ref(a_store.t(), b_store.t(), p=p)[0].t()          # [n][m]
    for _ in range(2):                                                # second run reuses streams and buffers
        out.fill_(-1.0)
        assert pipe.run(a_store, b_store, out, p=p) is out
        assert ko.rel_err_nonneg(out, ref) < (1e-5 if p in (1.0, 2.0) else 5e-5)
    with pytest.raises(ValueError):
        pipe.run(a_store[:, :10], b_store, out)


def test_unpinned_operands_take_the_contiguous_copy():
    # pageable host memory: b goes up in one contiguous copy instead of per-slab strided ones; same result
    K, M, N = 32, 300, 700
    g = torch.Generator().manual_seed(6)
    a_store, b_store = torch.randn(K, M, generator=g), torch.randn(K, N, generator=g)
    out = torch.empty(N, M)
    HostCdist(M, N, K, slabs=3).run(a_store, b_store, out, p=2.0)
    assert ko.rel_err_nonneg(out, ko.cdist_ref(a_store.t(), b_store.t(), p=2.0)[0].t()) < 1e-5


def test_strided_copy_helper_round_trip():
    from kermac_b200 import _native
    src = torch.arange(40 * 100, dtype=torch.float32).reshape(40, 100).pin_memory()
    dev = torch.zeros(40, 100, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    _native.copy_2d_async(dev.data_ptr() + 4 * 10, 400, src.data_ptr() + 4 * 10, 400, 4 * 25, 40, False, stream)
    torch.cuda.synchronize()
    want = torch.zeros(40, 100)
    want[:, 10:35] = src[:, 10:35]
    assert torch.equal(dev.cpu(), want)
    back = torch.zeros(40, 100).pin_memory()
    _native.copy_2d_async(back.data_ptr() + 4 * 10, 400, dev.data_ptr() + 4 * 10, 400, 4 * 25, 40, True, stream)
    torch.cuda.synchronize()
    assert torch.equal(back, want)
    with pytest.raises(ValueError):
        _native.copy_2d_async(dev.data_ptr(), 8, src.data_ptr(), 400, 100, 4, False, stream)     # pitch < row
