"""A build launch restricted to a range of the launcher's tile order (KmBuildArgs.tile_first /
tile_count) writes exactly those tiles: ranges that partition the tile order reproduce the full
launch bit for bit, which is what the multi-GPU cdist relies on."""
import ctypes

import pytest
import torch

import kermac_b200 as kermac
from kermac_b200 import _native
from kermac_b200.build_a_kernel import _current_stream_for, _marshal_build
from kermac_b200.cdist import descriptor_for
from kermac_b200.dist import tile_ranges

pytestmark = pytest.mark.gpu


def _launch(a, b, out, p, first=0, count=0):
    descriptor, powers = descriptor_for(p, False)
    args, _, keep = _marshal_build(descriptor, a, b, out, powers.get("p"), powers.get("inner_p"),
                                   None, None, None, None, 0, 0)
    total = _native.build_tile_count(args)
    args.tile_first, args.tile_count = first, count
    _native.launch_build(args, _current_stream_for(a.device))
    del keep
    return total


@pytest.mark.parametrize("p", [1.0, 2.0, 1.3])
@pytest.mark.parametrize("layout", ["m_contiguous", "k_contiguous", "out_n_contiguous"])
def test_tile_ranges_reproduce_the_full_launch(p, layout):
    M, N, K = 2100, 2500, 72                      # 17 x 20 tiles, ragged edges, more than one raster panel
    g = torch.Generator().manual_seed(21)
    a_store, b_store = torch.randn(K, M, generator=g).cuda(), torch.randn(K, N, generator=g).cuda()
    if layout == "k_contiguous":
        a, b = a_store.t().contiguous(), b_store.t().contiguous()
    else:
        a, b = a_store.t(), b_store.t()
    def fresh():
        if layout == "out_n_contiguous":
            return torch.full((M, N), -3.0, device="cuda")            # (M, N) with n contiguous
        return torch.full((N, M), -3.0, device="cuda").t()            # (M, N) with m contiguous
    whole = fresh()
    total = _launch(a, b, whole, p)
    assert total == 17 * 20
    for world in (3, 8):
        parts = fresh()
        for first, count in tile_ranges(total, world):
            _launch(a, b, parts, p, first, count)
        assert torch.equal(parts, whole)
    # a single range touches only its own tiles
    one = fresh()
    _launch(a, b, one, p, 40, 5)
    written = (one != -3.0)
    assert int(written.sum()) > 0 and int(written.sum()) <= 5 * 128 * 128
    assert torch.equal(one[written], whole[written])
    assert _native.device_error_flag() == 0


def test_empty_range_is_a_no_op():
    a = torch.rand(64, 300, device="cuda").t()
    out = torch.full((300, 300), -3.0, device="cuda").t()
    total = _launch(a, a, out, 2.0)
    assert total == 9
    out.fill_(-3.0)
    descriptor, _ = descriptor_for(2.0, False)
    args, _, keep = _marshal_build(descriptor, a, a, out, None, None, None, None, None, None, 0, 0)
    args.tile_first, args.tile_count = 9, 0       # from the end on: nothing left
    assert _native.lib().kermac_b200_build_kernel(ctypes.byref(args), None) == 0
    torch.cuda.synchronize()
    assert float(out.max()) == -3.0
