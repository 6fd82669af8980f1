"""The report path of a bounded device-side wait, made to run out on purpose and safely: a one-block
kernel waits a thousand attempts on an mbarrier that nothing arrives at, gives up, raises the device
error flag and ends (kermac_b200_selftest_wait_expiry).  No fault, no trap, no hang: the loop is
bounded by construction."""
import pytest
import torch

from kermac_b200 import _native

pytestmark = pytest.mark.gpu


def test_an_expired_wait_raises_the_flag_once_and_the_context_stays_usable():
    assert _native.device_error_flag() == 0
    _native.selftest_wait_expiry(1024, torch.cuda.current_stream().cuda_stream)
    assert _native.device_error_flag() == 1          # reads the flag back and clears it
    assert _native.device_error_flag() == 0
    # the context is intact: an ordinary operator still runs and still leaves the flag clear
    import kermac_b200 as kermac
    a = torch.rand(64, 300, device="cuda").t()
    d = kermac.cdist(a, a, p=2.0)
    assert torch.isfinite(d).all()
    assert _native.device_error_flag() == 0


def test_selftest_rejects_unbounded_requests():
    with pytest.raises(ValueError):
        _native.selftest_wait_expiry(0)
    with pytest.raises(ValueError):
        _native.selftest_wait_expiry(1 << 21)
