"""GPU: the failure path of the device-side waits, exercised without faulting or hanging anything.

Every wait inside the tcgen05 kernels is bounded: when it runs out, the kernel records
``{KB_ERR_DEVICE_TIMEOUT, wait site, block}`` in the status words, raises its CTA-wide abort flag and
returns; the host finds the words after synchronising and raises.  ``kb_selftest_wait_timeout`` runs that
very wait (one small CTA, a barrier nobody arrives on, a limit of 1 024 polls) so the whole chain can be
checked: the wait returns, the status words are set, ``check_device_status()`` raises and clears them,
and the context is still good for the next call.
"""

import pytest
import torch

from kernels_b200 import _lib

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_and_reports():
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    status = _lib.status_words()
    status.zero_()
    seen = torch.full((3,), -1, dtype=torch.int32).pin_memory()
    stream = torch.cuda.current_stream(dev)
    rc = lib.kb_selftest_wait_timeout(status.data_ptr(), seen.data_ptr(), stream.cuda_stream)
    _lib.check(rc, "kb_selftest_wait_timeout")
    stream.synchronize()  # returns: the kernel ended by itself
    assert seen.tolist() == [0, 0, 1], "short wait gave up, second role left on the abort flag, flag raised"
    assert status.tolist()[:3] == [4, 900, 0]  # KB_ERR_DEVICE_TIMEOUT, wait site, block
    with pytest.raises(RuntimeError, match="timed out"):
        _lib.check_device_status()
    assert status.tolist() == [0, 0, 0, 0], "reading the status clears it"
    _lib.check_device_status()  # nothing pending now

    # the context is still usable and an ordinary call reports no timeout
    from kernels_b200.softmax import softmax

    x = torch.randn(8, 256, device=dev)
    torch.testing.assert_close(softmax(x), torch.softmax(x, -1), atol=1e-6, rtol=0)
    torch.cuda.synchronize()
    _lib.check_device_status()


def test_selftest_rejects_null_pointers():
    lib = _lib.load()
    assert lib.kb_selftest_wait_timeout(None, None, None) == 1
