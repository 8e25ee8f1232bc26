"""GPU parity: quantize / dequantize kernels against the oracle, bit-exact
(crates/shrew/src/quantize.rs:194-366)."""
import numpy as np
import pytest
import torch

from tests.conftest import GOLDEN

pytestmark = pytest.mark.gpu


def _cfg(gran):
    from shrew_b200 import QuantConfig
    return QuantConfig.int8_per_channel() if gran == 1 else QuantConfig.int8()


def _quantize_gpu(w_np, gran):
    from shrew_b200 import quantize_tensor
    t = torch.from_numpy(np.require(w_np, dtype=np.float32, requirements="C")).cuda()
    qt = quantize_tensor(t, _cfg(gran))
    torch.cuda.synchronize()
    return qt, qt.data.cpu().numpy().reshape(w_np.shape), qt.scales.cpu().numpy()


@pytest.mark.parametrize("case", GOLDEN, ids=[c["name"] for c in GOLDEN])
def test_golden_vectors(case):
    qt, q, s = _quantize_gpu(case["data"], case["granularity"])
    np.testing.assert_array_equal(q, case["codes"])
    assert s.tobytes() == case["scales"].tobytes()
    assert qt.zero_points == [0.0] * len(case["scales"])
    assert qt.shape == list(case["shape"])


def _outlier_matrix(rows, cols, seed, std=1.0):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((rows, cols)) * std).astype(np.float32)
    mask = rng.random((rows, cols)) < 0.01
    w[mask] *= 50.0
    return w


# every register-tile width of the per-channel kernel, ragged widths, the generic fallback
@pytest.mark.parametrize("rows,cols", [
    (5, 32), (300, 128), (33, 132), (64, 256), (10, 260), (784, 256), (256, 784), (77, 1024), (50, 1100),
    (40, 2048), (33, 4096), (17, 5000), (9, 8192), (6, 16384), (3, 20000), (3, 32768), (2, 40000),
    (100, 7), (1000, 1), (3, 33), (1, 4096), (4096, 1024),
])
def test_per_channel_bit_exact(oracle, rows, cols):
    w = _outlier_matrix(rows, cols, seed=rows * 131 + cols)
    _, q, s = _quantize_gpu(w, 1)
    q_ref, s_ref = oracle.quantize_f32(w, oracle.PER_CHANNEL)
    assert s.tobytes() == s_ref.tobytes()
    np.testing.assert_array_equal(q, q_ref)


@pytest.mark.parametrize("shape", [(1,), (7,), (64, 96), (1000, 1000), (333, 777), (2, 3, 5, 7), (4096, 4096)])
def test_per_tensor_bit_exact(oracle, shape):
    w = _outlier_matrix(int(np.prod(shape)), 1, seed=len(shape) * 7 + shape[0], std=0.02).reshape(shape)
    _, q, s = _quantize_gpu(w, 0)
    q_ref, s_ref = (oracle.np_quantize_f32 if w.size > 1 << 22 else oracle.quantize_f32)(w, oracle.PER_TENSOR)
    assert s.tobytes() == s_ref.tobytes()
    np.testing.assert_array_equal(q, q_ref)


def test_ties_and_near_ties_take_the_exact_path(oracle):
    # products sitting on, or one f32 ulp away from, a .5 boundary: the f32 fast path must
    # hand these to the f64 path.  Row amax is 127 so inv_scale = 1/(127/127) = 1 exactly.
    base = np.arange(-126, 127, dtype=np.float32) + 0.5
    near = np.concatenate([base, np.nextafter(base, np.float32(1e9)), np.nextafter(base, np.float32(-1e9))])
    row = np.concatenate([[127.0], near]).astype(np.float32)
    row = np.pad(row, (0, (-len(row)) % 4))
    w = np.stack([row, row * np.float32(0.37), row * np.float32(1e-20), row * np.float32(3e30)])
    _, q, s = _quantize_gpu(w, 1)
    q_ref, s_ref = oracle.quantize_f32(w, oracle.PER_CHANNEL)
    assert s.tobytes() == s_ref.tobytes()
    np.testing.assert_array_equal(q, q_ref)


def test_reference_weight_distribution_4096(oracle):
    # N(0, 0.02) weights: the case where an all-f32 quantizer differs from the reference
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((4096, 4096)) * 0.02).astype(np.float32)
    _, q, s = _quantize_gpu(w, 1)
    q_ref, s_ref = oracle.np_quantize_f32(w, oracle.PER_CHANNEL)
    assert s.tobytes() == s_ref.tobytes()
    assert int((q != q_ref).sum()) == 0
    # the C oracle on a slice, so the numpy twin is not the only witness at this size
    q_c, s_c = oracle.quantize_f32(w[:128], oracle.PER_CHANNEL)
    np.testing.assert_array_equal(q[:128], q_c)


def test_full_size_properties():
    # largest sweep shape that the CPU oracle cannot finish in seconds: size-independent
    # properties.  (1) |code| <= 127 and every row reaches +-127; (2) scale = amax/127 in f64;
    # (3) quantizing the dequantized tensor again returns the same codes (idempotence).
    from shrew_b200 import QuantConfig, dequantize_tensor, quantize_tensor
    rows, cols = 16384, 8192
    g = torch.Generator(device="cuda").manual_seed(0)
    w = torch.randn(rows, cols, device="cuda", generator=g)
    qt = quantize_tensor(w, QuantConfig.int8_per_channel())
    codes = qt.data.view(rows, cols)
    assert int(codes.abs().max()) == 127 and int(codes.min()) >= -127
    assert bool((codes.abs().amax(dim=1) == 127).all())
    amax = w.abs().amax(dim=1).double().cpu().numpy()  # divide on the host: IEEE f64 division
    assert qt.scales.cpu().numpy().tobytes() == (amax / 127.0).tobytes()
    back = dequantize_tensor(qt)
    assert float((back - w).abs().max()) <= float(qt.scales.max()) * 0.5 + 1e-6
    again = quantize_tensor(back, QuantConfig.int8_per_channel())
    assert torch.equal(again.data, qt.data)


@pytest.mark.parametrize("rows,cols,gran", [(64, 96, 0), (64, 96, 1), (7, 33, 1), (1, 5, 0), (300, 4096, 1), (3, 0, 1)])
def test_dequantize_bit_exact(oracle, rows, cols, gran):
    from shrew_b200 import dequantize_tensor
    w = _outlier_matrix(rows, cols, seed=rows + cols, std=0.02)
    qt, q, s = _quantize_gpu(w, gran)
    back = dequantize_tensor(qt)
    torch.cuda.synchronize()
    ref = oracle.dequantize(q, s, gran, "f32")
    assert back.dtype == torch.float32 and list(back.shape) == [rows, cols]
    assert back.cpu().numpy().tobytes() == ref.tobytes()
    qt.original_dtype = torch.bfloat16
    back16 = dequantize_tensor(qt)
    ref16 = oracle.dequantize(q, s, gran, "bf16")
    assert back16.view(torch.int16).cpu().numpy().view(np.uint16).tobytes() == ref16.tobytes()


def test_host_buffer_entry_point(oracle):
    import ctypes
    from shrew_b200 import _lib
    from shrew_b200.quantize import Device
    dev = Device.get("cuda:0")
    w = _outlier_matrix(300, 1024, seed=3)
    q = np.empty(w.shape, dtype=np.int8)
    s = np.empty(300, dtype=np.float64)
    rc = _lib.lib().shrewq_quantize_f32_host(dev.handle, ctypes.c_void_p(w.ctypes.data), 300, 1024, 1,
                                             ctypes.c_void_p(q.ctypes.data), ctypes.c_void_p(s.ctypes.data))
    _lib.check(rc, dev.handle)
    q_ref, s_ref = oracle.quantize_f32(w, oracle.PER_CHANNEL)
    np.testing.assert_array_equal(q, q_ref)
    assert s.tobytes() == s_ref.tobytes()


def test_bad_arguments_return_errors():
    from shrew_b200 import _lib
    from shrew_b200.quantize import Device
    dev = Device.get("cuda:0")
    L = _lib.lib()
    t = torch.zeros(16, device="cuda")
    assert L.shrewq_quantize_f32(dev.handle, t.data_ptr(), 4, 4, 7, t.data_ptr(), t.data_ptr()) == _lib.ERR_INVALID_ARG
    assert L.shrewq_quantize_f32(dev.handle, None, 4, 4, 1, None, t.data_ptr()) == _lib.ERR_INVALID_ARG
    assert b"NULL" in L.shrewq_last_error(dev.handle)
    assert L.shrewq_dequantize(dev.handle, t.data_ptr(), t.data_ptr(), 4, 4, 1, 9, t.data_ptr()) == _lib.ERR_INVALID_ARG


@pytest.mark.parametrize("rows,cols,split", [(64, 128, 40), (1000, 333, 1), (7, 5, 7), (2048, 4096, 1024)])
def test_per_tensor_quantization_of_row_shards(oracle, rows, cols, split):
    # two "ranks" on one GPU: amax per shard, max of the two on the host (the all-reduce), then each
    # shard quantized with the global amax == the rows of the unsplit per-tensor quantization
    from shrew_b200.quantize import absmax, quantize_tensor_given_amax
    w = _outlier_matrix(rows, cols, seed=rows + cols, std=0.05)
    w[0, 0] = np.nan
    q_ref, s_ref = oracle.np_quantize_f32(w, oracle.PER_TENSOR)
    shards = [torch.from_numpy(w[:split].copy()).cuda(), torch.from_numpy(w[split:].copy()).cuda()]
    amax = torch.maximum(absmax(shards[0]), absmax(shards[1]))
    assert float(amax) == float(np.fmax.reduce(np.abs(w).reshape(-1)))
    got = [quantize_tensor_given_amax(s, amax) for s in shards]
    torch.cuda.synchronize()
    q = np.concatenate([g.data.cpu().numpy().reshape(s.shape) for g, s in zip(got, shards)], axis=0)
    np.testing.assert_array_equal(q, q_ref)
    for g in got:
        assert g.scales.cpu().numpy().tobytes() == s_ref.tobytes()


@pytest.mark.parametrize("gran", [0, 1])
def test_many_tensors_per_launch_match_one_by_one(oracle, gran, monkeypatch):
    # the parameter list of config 2's model shape (4 blocks of 256-wide layers, scaled-down head), plus
    # ragged, empty and rank-0 tensors, and more tensors than one table holds
    from shrew_b200 import Linear, QuantConfig, quantize_named_parameters, quantize_tensor, quantize_tensors
    cfg = QuantConfig.int8_per_channel() if gran == 1 else QuantConfig.int8()
    rng = np.random.default_rng(gran)
    shapes = ([(256, 256)] * 4 + [(1024, 256), (1, 1024), (256, 1024), (1, 256)]) * 4 + [(5025, 256), (7, 5), (0, 4), (3, 0), (), (2, 3, 4)]
    shapes += [(3, 20)] * 70
    ws = [torch.from_numpy(np.asarray(rng.standard_normal(s) * 0.02, dtype=np.float32)).cuda() for s in shapes]
    ws[0][0, 0] = float("nan")
    got = quantize_tensors(ws, cfg)
    torch.cuda.synchronize()
    for w, g in zip(ws, got):
        one = quantize_tensor(w, cfg)
        assert torch.equal(g.data, one.data) and g.shape == one.shape, tuple(w.shape)
        assert g.scales.cpu().numpy().tobytes() == one.scales.cpu().numpy().tobytes(), tuple(w.shape)
    q_ref, s_ref = oracle.np_quantize_f32(ws[4].cpu().numpy(), gran)
    np.testing.assert_array_equal(got[4].data.cpu().numpy().reshape(1024, 256), q_ref)
    assert got[4].scales.cpu().numpy().tobytes() == s_ref.tobytes()
    # and through the model-level helper
    lin = Linear(ws[1], torch.randn(256, device="cuda"))
    a = quantize_named_parameters(lin, cfg)                  # one batched call
    b = quantize_named_parameters(lin, cfg, batched=False)   # tensor by tensor
    assert [n for n, _ in a] == [n for n, _ in b] and all(torch.equal(x.data, y.data) and torch.equal(x.scales, y.scales)
                                                          for (_, x), (_, y) in zip(a, b))
