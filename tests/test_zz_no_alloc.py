"""GPU: shrewq_linear_forward_noalloc, the forward for callers that cannot allocate device
memory (a process whose HBM is fully reserved by its own pools, or a loop that cannot take
the device-wide synchronisation an allocation implies).  It keeps its split-K partial sums
in an array inside the library image.  The test calls it through the C ABI twice in a row
— the second call meets the first call's leftovers in the shared array — and compares each
result with the allocating entry point on the same inputs.  Collected last on purpose."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL_BF16 = 1e-2  # max|y - y_ref| / max|y_ref|, the bf16-path tolerance of the other GPU tests


def _rel_err(y, ref):
    y, ref = y.double(), ref.double()
    return float((y - ref).abs().max() / ref.abs().max())


def _make(N, K, seed):
    from shrew_b200 import Linear, QuantConfig, QuantizedLinear
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.02
    b = torch.randn(N, device="cuda", generator=g) * 0.1
    return QuantizedLinear.from_linear(Linear(w, b), QuantConfig.int8_per_channel())


@pytest.mark.parametrize("M,N,K", [(16, 1024, 4096), (48, 512, 2048), (32, 2048, 4096), (300, 384, 1024)])
def test_noalloc_matches_allocating_forward_twice(M, N, K):
    from shrew_b200 import _lib
    from shrew_b200.quantize import Device
    L = _lib.lib()
    dev = Device.get("cuda:0")
    ql = _make(N, K, seed=M + N)
    g = torch.Generator(device="cuda").manual_seed(7)
    try:
        for call in range(2):
            x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
            L.shrewq_force_kernel(b"tcgen05")
            ref = ql.forward(x)                       # existing entry point (may allocate scratch)
            dev.synchronize()
            y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
            dev.bind_stream()
            rc = L.shrewq_linear_forward_noalloc(ql._h, ctypes.c_void_p(x.data_ptr()), M, ctypes.c_void_p(y.data_ptr()),
                                                 _lib.BF16, N, _lib.EPILOGUE_NONE)
            _lib.check(rc, dev.handle)
            dev.synchronize()
            assert not torch.isnan(y.float()).any(), f"call {call}: output not fully written"
            err = _rel_err(y, ref)
            assert err <= TOL_BF16, f"call {call}: rel err {err:.3e}"
    finally:
        L.shrewq_force_kernel(b"auto")


@pytest.mark.parametrize("M,N,K", [(16, 1024, 4096), (300, 384, 1024)])
def test_noalloc_leaves_free_device_memory_unchanged(M, N, K):
    # the claim itself: once the module is loaded (the first call may load it), a call allocates nothing on the
    # device.  cudaMemGetInfo (torch.cuda.mem_get_info) before and after a run of warmed calls must agree, with
    # every input and output allocated beforehand.
    from shrew_b200 import _lib
    from shrew_b200.quantize import Device
    L = _lib.lib()
    dev = Device.get("cuda:0")
    ql = _make(N, K, seed=3)
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")

    def call():
        dev.bind_stream()
        _lib.check(L.shrewq_linear_forward_noalloc(ql._h, ctypes.c_void_p(x.data_ptr()), M, ctypes.c_void_p(y.data_ptr()),
                                                   _lib.BF16, N, _lib.EPILOGUE_NONE), dev.handle)

    call()                                  # warm: module load, function attributes
    dev.synchronize()
    torch.cuda.synchronize()
    free_before, total = torch.cuda.mem_get_info()
    for _ in range(5):
        call()
    dev.synchronize()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, f"free device memory changed by {free_before - free_after} bytes of {total}"


def test_noalloc_refuses_shapes_beyond_its_scratch_and_wrong_inputs():
    from shrew_b200 import _lib
    from shrew_b200.quantize import Device
    L = _lib.lib()
    dev = Device.get("cuda:0")
    # a shape whose partial sums exceed the 4 MiB array: 64 tokens, N = 1024 (8 channel
    # tiles), K = 8192 -> 16 splits: 8*16 slices of 64*128 f32 = 4.19 MB (+ counters)
    ql = _make(1024, 8192, seed=1)
    x = torch.zeros(64, 8192, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(64, 1024, dtype=torch.bfloat16, device="cuda")
    dev.bind_stream()
    rc = L.shrewq_linear_forward_noalloc(ql._h, ctypes.c_void_p(x.data_ptr()), 64, ctypes.c_void_p(y.data_ptr()),
                                         _lib.BF16, 1024, 0)
    assert rc == _lib.ERR_UNSUPPORTED
    msg = L.shrewq_last_error(dev.handle).decode()
    assert "built-in array" in msg and "4194304" in msg
    assert L.shrewq_linear_forward_noalloc(None, None, 1, None, 1, 1, 0) == _lib.ERR_INVALID_ARG
    odd = _make(64, 72, seed=2)  # in_features not a multiple of 16
    rc = L.shrewq_linear_forward_noalloc(odd._h, ctypes.c_void_p(x.data_ptr()), 4, ctypes.c_void_p(y.data_ptr()),
                                         _lib.BF16, 64, 0)
    assert rc == _lib.ERR_UNSUPPORTED
