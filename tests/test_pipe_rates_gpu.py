"""The pipe-rate measurements that the bench's rooflines divide by (kermac_b200_measure_pipe), on a GPU:
every kind runs, returns a plausible rate, and the tensor-pipe kinds show the rule the tensor-core
gradient kernel is planned around (an MMA of up to 64 columns costs as much as one of 32)."""
import pytest

from kermac_b200 import _native

pytestmark = pytest.mark.gpu


def test_fp32_and_mufu_kinds_return_rates():
    packed = _native.measure_pipe(1, 2048)[0]
    scalar = _native.measure_pipe(0, 2048)[0]
    mufu = _native.measure_pipe(2, 1024)[0]
    assert 1e13 < scalar <= packed * 1.05 and packed < 1e14
    assert 1e12 < mufu < 1e13
    for kind in (3, 4, 5, 6, 7):
        assert _native.measure_pipe(kind, 512)[0] > 1e12


def test_narrow_tensor_mmas_cost_the_same_up_to_64_columns():
    r32, r64, r128, r256 = (_native.measure_pipe(kind, 2048)[0] for kind in (8, 9, 10, 11))
    assert _native.device_error_flag() == 0
    assert 1e9 < r256 < r128 < r64 * 1.02 and r64 < 1e10
    assert abs(r32 / r64 - 1.0) < 0.05            # 128 x 32 x 8 and 128 x 64 x 8: the same time per MMA
    assert 1.6 < r128 / r256 < 2.4                # from 128 columns on the time follows the width


def test_rejects_unknown_kind():
    with pytest.raises(ValueError):
        _native.measure_pipe(12, 16)
