"""CPU: the C-ABI library loads, exports every symbol include/shrewq.h declares, refuses
to compute without a GPU, and the host-side mirror keeps the reference's semantics."""
import ctypes
import os
import re

import pytest
import torch

from tests.conftest import ROOT


@pytest.fixture(scope="module")
def shrewq():
    from shrew_b200 import build
    build.build_library()
    from shrew_b200 import _lib
    return _lib


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "shrewq.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(shrewq_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_all_exported(shrewq):
    names = _declared_functions()
    assert len(names) >= 18
    L = ctypes.CDLL(shrewq.LIB_PATH)
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, f"declared in shrewq.h but not exported: {missing}"
    # and the binding table covers the header exactly
    assert sorted(shrewq.SIGNATURES) == names


def test_version_names_architecture(shrewq):
    assert b"sm_100a" in shrewq.lib().shrewq_version()


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_no_device_fails_loudly(shrewq):
    h = ctypes.c_void_p()
    rc = shrewq.lib().shrewq_ctx_create(0, None, ctypes.byref(h))
    assert rc == shrewq.ERR_NO_DEVICE
    assert not h.value
    msg = shrewq.lib().shrewq_last_error(None).decode()
    assert "no CPU path" in msg
    with pytest.raises(shrewq.ShrewError):
        shrewq.check(rc, None)


def test_null_handles_are_rejected_not_crashed(shrewq):
    L = shrewq.lib()
    assert L.shrewq_quantize_f32(None, None, 1, 1, 0, None, None) == shrewq.ERR_INVALID_ARG
    assert L.shrewq_dequantize(None, None, None, 1, 1, 0, 0, None) == shrewq.ERR_INVALID_ARG
    assert L.shrewq_linear_forward(None, None, 0, 1, None, 0, 1, 0) == shrewq.ERR_INVALID_ARG
    assert L.shrewq_ctx_create(0, None, None) == shrewq.ERR_INVALID_ARG
    assert L.shrewq_force_kernel(b"bogus") == shrewq.ERR_INVALID_ARG
    assert L.shrewq_force_kernel(b"auto") == shrewq.OK
    assert L.shrewq_linear_in_features(None) == 0
    L.shrewq_linear_destroy(None)
    L.shrewq_ctx_destroy(None)
    # the later entry points too
    out = ctypes.c_void_p()
    assert L.shrewq_quantize_f32_ex(None, None, 1, 1, 0, 8, 0, None, None, None) == shrewq.ERR_INVALID_ARG
    assert L.shrewq_quantize_any(None, None, 0, 1, 1, 0, 8, 0, None, None, None) == shrewq.ERR_INVALID_ARG
    assert L.shrewq_dequantize_ex(None, None, None, None, 1, 1, 0, 0, None) == shrewq.ERR_INVALID_ARG
    assert L.shrewq_absmax_f32(None, None, 1, None) == shrewq.ERR_INVALID_ARG
    assert L.shrewq_quantize_f32_given_amax(None, None, 1, None, None, None) == shrewq.ERR_INVALID_ARG
    assert L.shrewq_linear_create_ex(None, None, None, None, None, 1, 1, 0, ctypes.byref(out)) == shrewq.ERR_INVALID_ARG
    assert L.shrewq_linear_forward_noalloc(None, None, 1, None, 0, 1, 0) == shrewq.ERR_INVALID_ARG
    for kind in (b"gemv", b"tcgen05", b"simt", b"mma", b"mma-ring", b"tcgen05-f32", b"tcgen05-2cta", b"auto"):
        assert L.shrewq_force_kernel(kind) == shrewq.OK


def test_quant_config_mirror():
    # quantize.rs:74-139
    from shrew_b200 import QuantBits, QuantConfig, QuantGranularity, QuantMode
    c = QuantConfig.int8()
    assert (c.bits, c.mode, c.granularity) == (QuantBits.Int8, QuantMode.Symmetric, QuantGranularity.PerTensor)
    assert c == QuantConfig()
    pc = QuantConfig.int8_per_channel()
    assert pc.granularity is QuantGranularity.PerChannel
    assert (c.qmax(), c.qmin()) == (127.0, -127.0)
    assert c.asymmetric().qmin() == -128.0
    assert (QuantConfig.int4().qmax(), QuantConfig.int4().qmin()) == (7.0, -7.0)
    assert QuantConfig.int4_per_channel().asymmetric().qmin() == -8.0


def test_cpu_tensor_is_rejected_loudly(shrewq):
    from shrew_b200 import QuantConfig, ShrewError, quantize_tensor
    with pytest.raises(ShrewError) as e:
        quantize_tensor(torch.zeros(2, 3), QuantConfig.int8())
    assert e.value.code == shrewq.ERR_NO_DEVICE


def test_unsupported_modes_are_errors():
    from shrew_b200 import QuantConfig, ShrewError, quantize_tensor
    for cfg in (QuantConfig.int4(), QuantConfig.int8().asymmetric()):
        with pytest.raises(ShrewError):
            quantize_tensor(torch.zeros(2, 3), cfg)


def test_quantization_stats_bias_is_rank2():
    # quantize.rs:768-776: weight [32,64] and bias [1,32] both count as quantized
    from shrew_b200 import Linear, QuantConfig, quantization_stats
    lin = Linear(torch.zeros(32, 64), torch.zeros(32))
    st = quantization_stats(lin, QuantConfig.int8())
    assert st.num_quantized == 2 and st.num_fp32 == 0
    assert st.compression_ratio > 3.0
    assert st.fp32_bytes == (32 * 64 + 32) * 4
    assert st.quantized_bytes == 32 * 64 + 16 + 32 + 16
    st_pc = quantization_stats(lin, QuantConfig.int8_per_channel())
    assert st_pc.quantized_bytes == 32 * 64 + 32 * 16 + 32 + 1 * 16


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "shrew_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower() or f == "bench_support.py", f"{f} mentions the oracle"
