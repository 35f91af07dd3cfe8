"""A device-side wait that runs out: the kernel gives up after its (millisecond) limit, returns, leaves the self-test
code in the status word, ``check_status`` raises, and the stream keeps working.  Nothing faults, traps or hangs."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_on_a_flag_nobody_raises_times_out_cleanly():
    from dttt_b200.ops import _lib, gemm
    dev = torch.device("cuda", 0)
    _lib.check_status(dev)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    waited = _lib.wait_selftest(flag, target=1, limit_ms=3.0)
    torch.cuda.synchronize()
    assert 2500 <= int(waited.item()) < 200_000, int(waited.item())
    with pytest.raises(_lib.KernelError, match="self-test"):
        _lib.check_status(dev)
    _lib.check_status(dev)                                     # the word was reset by the failed check
    # the context is intact: the next launches on the same stream run and are correct
    a = torch.randn(256, 128, device=dev).to(torch.bfloat16)
    b = torch.randn(128, 256, device=dev).to(torch.bfloat16)
    c = gemm.gemm_raw(a, b, False, False)
    torch.cuda.synchronize()
    assert (c.float() - a.float() @ b.float()).abs().max().item() < 0.5
    _lib.check_status(dev)


def test_wait_that_is_satisfied_reports_nothing():
    from dttt_b200.ops import _lib
    dev = torch.device("cuda", 0)
    flag = torch.ones(1, dtype=torch.int32, device=dev)
    waited = _lib.wait_selftest(flag, target=1, limit_ms=3.0)
    torch.cuda.synchronize()
    assert int(waited.item()) < 2000
    _lib.check_status(dev)
