"""The caching device allocator hands a freed block out again only when the work that was queued
when it was freed has finished, on whichever stream that work runs."""
import ctypes

import numpy as np
import pytest

from tessera_b200 import _lib, device
from tessera_b200.device import DeviceArray, Stream

pytestmark = pytest.mark.gpu


def _alloc(nbytes):
    h = ctypes.c_void_p()
    _lib.call("tessera_sm100_pool_alloc", ctypes.byref(h), nbytes)
    return int(h.value)


@pytest.mark.parametrize("how", ["known_streams", "given_stream"])
def test_block_is_not_reused_while_a_stream_still_uses_it(how):
    device.set_device(0)
    _lib.call("tessera_sm100_pool_release")
    nbytes = 48 << 20
    s = Stream()                        # non-blocking: does not order with the default stream
    p = _alloc(nbytes)
    for _ in range(40):                 # a few milliseconds of queued work ahead of the last use of p
        device.flush_l2(s)
    _lib.call("tessera_sm100_device_memset", p, 7, nbytes, s.handle)
    if how == "known_streams":
        _lib.call("tessera_sm100_pool_free", p)          # ordered after every stream the library made
    else:
        _lib.call("tessera_sm100_pool_free_async", p, s.handle)
    q = _alloc(nbytes)                  # the memset has not run yet: p must not come back
    assert q != p
    s.synchronize()
    check = DeviceArray((nbytes,), np.uint8, ptr=p).download()
    assert (check == 7).all()
    r = _alloc(nbytes)                  # now it may, and it is the only cached block of this size
    assert r == p
    for ptr in (q, r):
        _lib.call("tessera_sm100_pool_free_async", ptr, None)
    s.close()
    device.synchronize()
    _lib.call("tessera_sm100_pool_release")
