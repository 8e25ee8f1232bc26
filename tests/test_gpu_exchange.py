"""GPU (one is enough): the device-side exchange barrier gives up a wait that nothing ends.

The barrier is given two flag blocks in this GPU's own memory, as if a second rank existed; nobody ever
writes that rank's arrival, so the wait runs out after about a second, the kernel ends by itself and the
next synchronize reports SHREWQ_ERR_TIMEOUT naming the missing rank.  Nothing faults or traps, the
context stays usable, and a world of one passes at once.  (The barrier between real ranks is exercised in
test_gpu_multi.py and, as host threads, in test_exchange_barrier.py.)"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_missing_peer_ends_the_wait_with_a_timeout_status():
    from shrew_b200 import ShrewError, _lib
    from shrew_b200.quantize import Device
    L = _lib.lib()
    dev = Device.get("cuda:0")
    flags = torch.zeros(2, _lib.EXCHANGE_FLAG_BYTES // 4, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    blocks = (ctypes.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
    ex = ctypes.c_void_p()
    _lib.check(L.shrewq_exchange_create(dev.handle, 0, 2, blocks, ctypes.byref(ex)), dev.handle)
    try:
        dev.bind_stream()
        _lib.check(L.shrewq_exchange_barrier(ex), dev.handle)
        with pytest.raises(ShrewError) as e:
            dev.synchronize()
        assert e.value.code == _lib.ERR_TIMEOUT
        # this rank did announce itself to the "peer" before it gave up
        assert int(flags[1, 0].item()) == 1
        # the status is cleared by the failed synchronize; the context works on
        dev.synchronize()
        y = torch.ones(4, device="cuda") * 2
        assert float(y.sum().item()) == 8.0
    finally:
        L.shrewq_exchange_destroy(ex)


def test_world_of_one_passes_at_once_and_counts_on():
    from shrew_b200 import _lib
    from shrew_b200.quantize import Device
    L = _lib.lib()
    dev = Device.get("cuda:0")
    flags = torch.zeros(_lib.EXCHANGE_FLAG_BYTES // 4, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    blocks = (ctypes.c_void_p * 1)(flags.data_ptr())
    ex = ctypes.c_void_p()
    _lib.check(L.shrewq_exchange_create(dev.handle, 0, 1, blocks, ctypes.byref(ex)), dev.handle)
    try:
        dev.bind_stream()
        for _ in range(3):
            _lib.check(L.shrewq_exchange_barrier(ex), dev.handle)
        dev.synchronize()
        assert int(flags[32].item()) == 3      # the barrier count lives in device memory
    finally:
        L.shrewq_exchange_destroy(ex)
    assert L.shrewq_exchange_create(dev.handle, 2, 2, blocks, ctypes.byref(ex)) == _lib.ERR_INVALID_ARG
    assert L.shrewq_exchange_create(dev.handle, 0, 9, blocks, ctypes.byref(ex)) == _lib.ERR_INVALID_ARG
