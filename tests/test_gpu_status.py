"""Device-side failure reporting: a bounded wait that runs out sets the per-device status word and the
kernel returns normally.  The wait is made to run out in a harmless way: the self-test kernel's only bulk
copy completes, but its barrier was armed for more bytes than the copy delivers, so the phase never
completes and the (shortened) wait gives up.  Nothing faults, traps or hangs, and the context stays usable."""
import pytest
import torch

from tests.gpu_common import ops

pytestmark = pytest.mark.gpu


def test_wait_timeout_is_reported_and_the_context_stays_usable():
    C = ops()
    dev = torch.cuda.current_device()
    stream = C.stream_of(torch.zeros(1, device="cuda"))
    C.device_status(dev, reset=True)
    # control: the barrier is armed for exactly the copied bytes, the wait succeeds
    C.check(C.lib.rn_selftest_wait_timeout(0, 16, dev, stream))
    assert C.device_status(dev, reset=False) == 0
    # armed for 16 bytes more than the copy delivers: the wait of 2^16 cycles runs out
    C.check(C.lib.rn_selftest_wait_timeout(16, 16, dev, stream))
    assert C.device_status(dev, reset=False) == 1      # sticky until reset
    assert C.device_status(dev, reset=True) == 1
    assert C.device_status(dev, reset=False) == 0
    # the context is intact: a product kernel still runs and reports nothing
    q = torch.randn(2, 4, 2, 2, 16, device="cuda").bfloat16()
    import ramnet_ops
    y, _ = ramnet_ops.random_access_memory_attention(q, q, torch.randn(2, 4, 2, 8, device="cuda").bfloat16(), top_k=4,
                                                     impl_backend="cuda")
    torch.cuda.synchronize()
    assert torch.isfinite(y.float()).all() and C.device_status(dev) == 0


def test_debug_mode_turns_a_reported_failure_into_an_exception(monkeypatch):
    C = ops()
    dev = torch.cuda.current_device()
    monkeypatch.setattr(C, "CHECK_STATUS", True)
    C.device_status(dev, reset=True)
    C.check(C.lib.rn_selftest_wait_timeout(32, 14, dev, C.stream_of(torch.zeros(1, device="cuda"))))
    with pytest.raises(RuntimeError, match="device status 1"):
        C.check_device(torch.zeros(1, device="cuda"))
    assert C.device_status(dev) == 0
