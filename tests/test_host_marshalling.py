"""Host-side marshalling of the Python mirror that only a GPU run would otherwise exercise: the calls are
made against a recording stand-in for the library (CPU tensors carry the pointers), so a wrong field
order or a dropped tensor shows up here and not in a GPU session."""
import ctypes

import pytest
import torch

from shrew_b200 import QuantConfig, QuantGranularity, _lib
from shrew_b200 import quantize as Q


class _FakeDevice:
    handle = ctypes.c_void_p(0x1234)

    def bind_stream(self):
        pass


class _FakeLib:
    def __init__(self):
        self.calls = []

    def shrewq_quantize_f32_batch(self, handle, items, n, gran):
        arr = ctypes.cast(items, ctypes.POINTER(_lib.QuantItem * n)).contents
        self.calls.append((gran, [(it.w_dev, it.rows, it.cols, it.q_dev, it.scales_dev) for it in arr]))
        return 0


@pytest.fixture
def fake(monkeypatch):
    lib = _FakeLib()
    monkeypatch.setattr(Q.Device, "get", classmethod(lambda cls, dev: _FakeDevice()))
    monkeypatch.setattr(_lib, "lib", lambda: lib)
    return lib


def test_quantize_tensors_builds_one_table_per_granularity(fake):
    ws = [torch.zeros(6, 10), torch.zeros(3, 4, 5), torch.zeros(()), torch.zeros(0, 7), torch.zeros(1, 9)]
    out = Q.quantize_tensors(ws, QuantConfig.int8_per_channel())
    assert [t.shape for t in out] == [[6, 10], [3, 4, 5], [], [0, 7], [1, 9]]
    assert [t.scales.numel() for t in out] == [6, 3, 1, 0, 1]
    assert [t.data.numel() for t in out] == [60, 60, 1, 0, 9]
    # the rank-0 tensor goes in a per-tensor call of its own (quantize.rs:276-278), the others in one per-channel call
    assert [g for g, _ in fake.calls] == [QuantGranularity.PerChannel.value, QuantGranularity.PerTensor.value]
    main, single = fake.calls[0][1], fake.calls[1][1]
    assert [(r, c) for _, r, c, _, _ in main] == [(6, 10), (3, 20), (0, 7), (1, 9)]
    assert [(r, c) for _, r, c, _, _ in single] == [(1, 1)]
    for (w_ptr, _, _, q_ptr, s_ptr), w, t in zip(main, [ws[0], ws[1], ws[3], ws[4]], [out[0], out[1], out[3], out[4]]):
        assert w_ptr == (w.data_ptr() or None) and q_ptr == (t.data.data_ptr() or None) and s_ptr == (t.scales.data_ptr() or None)
    assert single[0][0] == ws[2].data_ptr() and single[0][3] == out[2].data.data_ptr()


def test_quantize_tensors_per_tensor_config_is_one_call(fake):
    out = Q.quantize_tensors([torch.zeros(4, 4), torch.zeros(())], QuantConfig.int8())
    assert len(fake.calls) == 1 and fake.calls[0][0] == QuantGranularity.PerTensor.value
    assert [t.scales.numel() for t in out] == [1, 1]


def test_quantize_tensors_refuses_what_the_kernels_do_not_take(fake):
    with pytest.raises(Q.ShrewError):
        Q.quantize_tensors([torch.zeros(2, 2, dtype=torch.bfloat16)], QuantConfig.int8())
    with pytest.raises(Q.ShrewError):
        Q.quantize_tensors([torch.zeros(2, 2)], QuantConfig.int4())
    assert Q.quantize_tensors([], QuantConfig.int8()) == [] and fake.calls == []


def test_named_parameters_walk_goes_out_as_one_batch(fake):
    class M:
        def named_parameters(self):
            return [("weight", torch.zeros(4, 8)), ("bias", torch.zeros(1, 4)), ("gain", torch.zeros(4))]

    out = Q.quantize_named_parameters(M(), QuantConfig.int8())
    assert [n for n, _ in out] == ["weight", "bias"]            # rank >= 2 only, the [1, out] bias included (quantize.rs:507-513)
    assert len(fake.calls) == 1 and len(fake.calls[0][1]) == 2


class _SignatureCheckingLib:
    """Stands in for libshrewq: every call must carry as many arguments as the C declaration has parameters,
    each acceptable to its ctypes type; returns success."""

    def __init__(self):
        self.calls = []

    def __getattr__(self, name):
        if name not in _lib.SIGNATURES:
            raise AttributeError(name)
        res, argtypes = _lib.SIGNATURES[name]

        def call(*args):
            assert len(args) == len(argtypes), f"{name}: {len(args)} arguments for {len(argtypes)} parameters"
            for a, t in zip(args, argtypes):
                t.from_param(a)
            self.calls.append(name)
            return b"stand-in" if res is ctypes.c_char_p else 0
        return call


def test_every_mode_of_the_python_mirror_marshals_its_call(monkeypatch):
    # the experimental modes (asymmetric, INT4, other storage types, packed INT4, shard entry points) have not
    # run on a GPU; their host side at least calls the C ABI with the declared arity and types
    from shrew_b200 import Linear, quantization_stats, quantize_named_parameters
    lib = _SignatureCheckingLib()
    monkeypatch.setattr(Q.Device, "get", classmethod(lambda cls, dev: _FakeDevice()))
    monkeypatch.setattr(_lib, "lib", lambda: lib)
    w = torch.randn(8, 128)
    for cfg in (QuantConfig.int8(), QuantConfig.int8_per_channel(), QuantConfig.int4_per_channel(), QuantConfig.int8().asymmetric()):
        for dt in (torch.float32, torch.bfloat16, torch.float16, torch.float64):
            qt = Q.quantize_tensor(w.to(dt), cfg)
            back = Q.dequantize_tensor(qt)
            assert list(back.shape) == [8, 128] and back.dtype == dt
            assert (qt.zero_points_t is not None) == (cfg.mode is Q.QuantMode.Asymmetric)
    shard = Q.quantize_tensor_given_amax(w, Q.absmax(w))
    assert shard.scales.numel() == 1
    Q.QuantizedLinear.new(Q.quantize_tensor(w, QuantConfig.int8_per_channel()), torch.zeros(8))
    Q.QuantizedLinear.new(Q.quantize_tensor(w, QuantConfig.int8_per_channel().asymmetric()), None)
    q4 = Q.quantize_tensor(w, QuantConfig.int4_per_channel())
    assert Q.pack_int4(q4).numel() == 8 * 128 // 2
    Q.QuantizedLinear.new_int4_packed(q4, None)
    lin = Linear(w, torch.zeros(8))
    assert len(quantize_named_parameters(lin, QuantConfig.int8())) == 2
    assert quantization_stats(lin, QuantConfig.int8()).num_quantized == 2
    assert {"shrewq_quantize_f32", "shrewq_quantize_f32_ex", "shrewq_quantize_any", "shrewq_dequantize", "shrewq_dequantize_ex",
            "shrewq_absmax_f32", "shrewq_quantize_f32_given_amax", "shrewq_linear_create", "shrewq_linear_create_ex",
            "shrewq_pack_int4", "shrewq_linear_create_int4"} <= set(lib.calls)


def test_quantized_linear_module_surface_without_a_device():
    # the Module methods a QuantizedLinear inherits (quantize.rs:462-482 overrides only forward and parameters):
    # pure host state, checked on an instance that never touched the library
    ql = object.__new__(Q.QuantizedLinear)
    ql._h = None
    assert ql.parameters() == [] and ql.named_parameters() == []
    assert ql.num_parameters() == 0 and ql.trainable_params_count() == 0
    assert ql.is_training() is True
    ql.set_training(False)
    assert ql.is_training() is False


def test_forward_host_marshals_host_pointers_and_checks_its_input(monkeypatch):
    calls = []

    class Lib:
        def shrewq_linear_forward_host(self, h, x, x_dtype, M, y, y_dtype, epilogue):
            calls.append((h, x.value, x_dtype, M, y.value, y_dtype, epilogue))
            return 0

    monkeypatch.setattr(_lib, "lib", lambda: Lib())
    ql = object.__new__(Q.QuantizedLinear)
    ql._h, ql.in_features, ql.out_features, ql.device = 0x77, 8, 3, _FakeDevice()
    x = torch.zeros(5, 8, dtype=torch.bfloat16)
    y = ql.forward_host(x, epilogue=1, out_dtype=torch.float32)
    assert y.shape == (5, 3) and y.dtype == torch.float32 and y.device.type == "cpu"
    (h, xp, xd, M, yp, yd, ep), = calls
    assert (h, xp, xd, M, yp, yd, ep) == (0x77, x.data_ptr(), _lib.BF16, 5, y.data_ptr(), _lib.F32, 1)
    with pytest.raises(Q.ShrewError):
        ql.forward_host(torch.zeros(5, 7))                       # wrong in_features
    with pytest.raises(Q.ShrewError):
        ql.forward_host(torch.zeros(5, 8, dtype=torch.float64))  # unsupported dtype
    ql._h = None
