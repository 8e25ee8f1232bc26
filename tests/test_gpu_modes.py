"""GPU: the reference's other quantization modes (asymmetric INT8, INT4: quantize.rs:99-139,353-364) through the C ABI
against the oracle and its golden vectors: codes, scales and zero points bit for bit, the zero-point forward and the
packed INT4 forward within the layer tolerances."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

def _cfg(bits, mode, gran):
    from shrew_b200.quantize import QuantBits, QuantConfig, QuantGranularity, QuantMode
    return QuantConfig(QuantBits.Int8 if bits == 8 else QuantBits.Int4,
                       QuantMode.Asymmetric if mode else QuantMode.Symmetric,
                       QuantGranularity.PerChannel if gran else QuantGranularity.PerTensor)


def _modes_golden():
    from tests.test_oracle_modes import MODES
    return MODES


@pytest.mark.parametrize("case", _modes_golden(), ids=[c["name"] for c in _modes_golden()])
def test_quantize_modes_match_golden(case):
    from shrew_b200 import quantize_tensor
    w = torch.from_numpy(np.require(case["data"], dtype=np.float32, requirements="C")).cuda()
    qt = quantize_tensor(w, _cfg(case["bits"], case["mode"], case["granularity"]))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(qt.data.cpu().numpy().reshape(case["codes"].shape), case["codes"])
    assert qt.scales.cpu().numpy().tobytes() == case["scales"].tobytes()
    zps = np.zeros_like(case["scales"]) if qt.zero_points_t is None else qt.zero_points_t.cpu().numpy()
    assert zps.tobytes() == case["zps"].tobytes()


@pytest.mark.parametrize("bits,mode", [(8, 1), (4, 0), (4, 1)])
@pytest.mark.parametrize("shape,gran", [((64, 300), 1), ((1000, 33), 1), ((257, 129), 0), ((3, 100000), 1), ((1 << 20,), 0)])
def test_quantize_dequantize_modes_match_oracle(oracle, bits, mode, shape, gran):
    from shrew_b200 import dequantize_tensor, quantize_tensor
    rng = np.random.default_rng(bits * 10 + mode)
    w = (rng.standard_normal(shape) * 0.3 + (0.2 if mode else 0.0)).astype(np.float32)
    w.reshape(-1)[::997] *= 40.0
    qt = quantize_tensor(torch.from_numpy(w).cuda(), _cfg(bits, mode, gran))
    q_ref, s_ref, z_ref = oracle.np_quantize_f32_ex(w, gran, bits, mode)
    np.testing.assert_array_equal(qt.data.cpu().numpy().reshape(shape), q_ref)
    assert qt.scales.cpu().numpy().tobytes() == s_ref.tobytes()
    zps = np.zeros_like(s_ref) if qt.zero_points_t is None else qt.zero_points_t.cpu().numpy()
    assert zps.tobytes() == z_ref.tobytes()
    back = dequantize_tensor(qt).cpu().numpy()
    g = gran if len(shape) > 1 else 0
    ref = oracle.dequantize_f64_ex(q_ref, s_ref, z_ref, g).astype(np.float32)
    np.testing.assert_array_equal(back, ref)


@pytest.mark.parametrize("M,dtype", [(1, "bf16"), (7, "f32"), (48, "bf16"), (300, "bf16")])
def test_forward_with_zero_points(oracle, M, dtype):
    # QuantizedLinear::forward with an asymmetric weight (quantize.rs:463-476): x . dequant(W)^T + bias
    from shrew_b200 import Linear, QuantizedLinear, _lib
    from shrew_b200.quantize import Device
    rng = np.random.default_rng(M)
    N, K = 384, 1024
    w = (rng.standard_normal((N, K)) * 0.05 + 0.1).astype(np.float32)      # one-sided-ish: large zero points
    b = (rng.standard_normal(N) * 0.1).astype(np.float32)
    ql = QuantizedLinear.from_linear(Linear(torch.from_numpy(w).cuda(), torch.from_numpy(b).cuda()), _cfg(8, 1, 1))
    x = rng.standard_normal((M, K)).astype(np.float32)
    x_t = torch.from_numpy(x).cuda()
    if dtype == "bf16":
        x_t = x_t.to(torch.bfloat16)
        x = x_t.float().cpu().numpy()
    y = ql.forward(x_t, epilogue=_lib.EPILOGUE_RELU)
    Device.get("cuda:0").synchronize()
    qt = ql.weight_q
    wd = oracle.dequantize_f64_ex(qt.data.cpu().numpy().reshape(N, K), qt.scales.cpu().numpy(), qt.zero_points_t.cpu().numpy(), 1)
    ref = (x.astype(np.float64) @ wd.astype(np.float32).astype(np.float64).T).astype(np.float32) + b.reshape(1, -1)
    ref = np.maximum(ref, 0.0)
    assert oracle.rel_err(y.float().cpu().numpy(), ref) < (1e-2 if dtype == "bf16" else 1e-4)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float64])
@pytest.mark.parametrize("gran", [0, 1])
def test_quantize_any_storage_type(oracle, dtype, gran):
    # quantize_tensor widens every storage type to f64 (quantize.rs:198); dequantize_tensor narrows back
    from shrew_b200 import dequantize_tensor, quantize_tensor
    rng = np.random.default_rng(gran)
    w64 = rng.standard_normal((40, 700)) * 0.2
    t = torch.from_numpy(w64).to(dtype).cuda()
    exact = t.double().cpu().numpy()
    qt = quantize_tensor(t, _cfg(8, 0, gran))
    torch.cuda.synchronize()
    # reference arithmetic on the exactly widened values
    data = exact if gran else exact.reshape(1, -1)
    amax = np.abs(data).max(axis=1)
    scale = np.where(amax < 1e-30, 1.0, amax / 127.0)
    tq = oracle.np_round_half_away(data * (1.0 / scale)[:, None])
    q_ref = np.clip(tq, -127, 127).astype(np.int8).reshape(40, 700)
    np.testing.assert_array_equal(qt.data.cpu().numpy().reshape(40, 700), q_ref)
    assert qt.scales.cpu().numpy().tobytes() == scale.tobytes()
    back = dequantize_tensor(qt)
    assert back.dtype == dtype
    ref = torch.from_numpy(q_ref.astype(np.float64) * (scale[:, None] if gran else scale[0])).to(dtype)
    assert torch.equal(back.cpu(), ref)


@pytest.mark.parametrize("M,N,K", [(1, 4096, 4096), (3, 300, 1024), (16, 523, 2048), (32, 1000, 1152)])
def test_packed_int4_forward(oracle, M, N, K):
    # INT4 symmetric per-channel codes packed two per byte, small-batch forward on the warp-MMA kernel
    from shrew_b200 import quantize_tensor
    from shrew_b200.quantize import Device, QuantizedLinear
    rng = np.random.default_rng(M + N)
    w = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(N) * 0.1).astype(np.float32)
    qt = quantize_tensor(torch.from_numpy(w).cuda(), _cfg(4, 0, 1))
    ql = QuantizedLinear.new_int4_packed(qt, torch.from_numpy(b).cuda())
    x_t = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).cuda().to(torch.bfloat16)
    y = ql.forward(x_t, out_dtype=torch.float32)
    Device.get("cuda:0").synchronize()
    assert ql.last_kernel() == "mma-w4"
    q_ref, s_ref, _ = oracle.np_quantize_f32_ex(w, 1, 4, 0)
    np.testing.assert_array_equal(qt.data.cpu().numpy().reshape(N, K), q_ref)
    ref = oracle.np_linear_forward(q_ref, s_ref, 1, b, x_t.float().cpu().numpy())
    assert oracle.rel_err(y.cpu().numpy(), ref) < 1e-4

