"""CPU: the oracle against the golden vectors and the reference's own test assertions
(crates/shrew/src/quantize.rs:601-789)."""
import numpy as np
import pytest

from tests.conftest import GOLDEN


@pytest.mark.parametrize("case", GOLDEN, ids=[c["name"] for c in GOLDEN])
def test_c_oracle_matches_golden(oracle, case):
    q, s = oracle.quantize_f32(case["data"], case["granularity"])
    assert q.shape == case["codes"].shape
    np.testing.assert_array_equal(q, case["codes"])
    assert s.tobytes() == case["scales"].tobytes()  # bit-exact f64 scales


@pytest.mark.parametrize("case", GOLDEN, ids=[c["name"] for c in GOLDEN])
def test_numpy_twin_matches_golden(oracle, case):
    q, s = oracle.np_quantize_f32(case["data"], case["granularity"])
    np.testing.assert_array_equal(q, case["codes"])
    assert s.tobytes() == case["scales"].tobytes()


def _case(name):
    return next(c for c in GOLDEN if c["name"] == name)


def test_ref_int8_symmetric_per_tensor(oracle):
    # quantize.rs:601-625
    c = _case("ref_int8_symmetric_per_tensor")
    q, s = oracle.quantize_f32(c["data"], oracle.PER_TENSOR)
    assert list(q.shape) == [2, 3]
    assert len(s) == 1
    rec = oracle.dequantize(q, s, oracle.PER_TENSOR, "f32").astype(np.float64)
    assert np.all(np.abs(c["data"].astype(np.float64) - rec) < 0.02)


def test_ref_int8_per_channel(oracle):
    # quantize.rs:651-673
    c = _case("ref_int8_per_channel")
    q, s = oracle.quantize_f32(c["data"], oracle.PER_CHANNEL)
    assert len(s) == 3
    rec = oracle.dequantize(q, s, oracle.PER_CHANNEL, "f32").astype(np.float64)
    assert np.all(np.abs(c["data"].astype(np.float64) - rec) < 0.01)


def test_ref_zero_tensor(oracle):
    # quantize.rs:780-789
    c = _case("ref_zero_tensor")
    q, s = oracle.quantize_f32(c["data"], oracle.PER_TENSOR)
    assert s[0] == 1.0
    rec = oracle.dequantize(q, s, oracle.PER_TENSOR, "f32")
    assert np.all(rec == 0.0)


def test_ref_quantized_linear_forward_close_to_float(oracle):
    # quantize.rs:714-739: Linear(4 -> 3, bias), x [2,4], |quantized - float| < 0.5
    rng = np.random.default_rng(0)
    w = rng.standard_normal((3, 4)).astype(np.float32) * 0.5
    b = rng.standard_normal((1, 3)).astype(np.float32) * 0.1
    x = rng.standard_normal((2, 4)).astype(np.float32)
    q, s = oracle.quantize_f32(w, oracle.PER_TENSOR)
    y = oracle.linear_forward_f32(q, s, oracle.PER_TENSOR, b, x)
    y_float = x.astype(np.float64) @ w.astype(np.float64).T + b
    assert np.all(np.abs(y - y_float) < 0.5)


def test_float_linear_known_answers(oracle):
    # the reference's exact Linear / matmul cases at the boundary of this path, run with
    # weights that quantize losslessly (integers with amax 127 -> scale exactly 1)
    # exec_tests.rs:617-648: ones weights, x rows of ones -> 4 and 8 (+ zero bias)
    w = np.zeros((2, 4), dtype=np.float32)
    w[:, :] = 127.0
    q, s = oracle.quantize_f32(w, oracle.PER_TENSOR)
    assert s[0] == 1.0 and np.all(q == 127)
    x = np.array([[1, 1, 1, 1], [2, 2, 2, 2]], dtype=np.float32) / 127.0
    y = oracle.linear_forward_f32(q, s, oracle.PER_TENSOR, None, x)
    np.testing.assert_allclose(y, [[4, 4], [8, 8]], rtol=1e-6)


def test_rounding_convention_of_the_reference(oracle):
    # nn_tests.rs:2413-2420: f64::round rounds half away from zero; the vector and its expected result
    t = np.array([-1.7, -0.5, 0.0, 0.3, 1.5, 2.9])
    np.testing.assert_array_equal(oracle.np_round_half_away(t), [-2.0, -1.0, 0.0, 0.0, 2.0, 3.0])
    # and through the C restatement: values that are exactly these after the multiply by 1/scale (scale 1.0:
    # amax 127 puts the codes on the values themselves)
    w = np.array([[127.0, -1.5, -0.5, 0.5, 1.5, 2.5, -2.5, 0.49999997]], dtype=np.float32)
    q, s = oracle.quantize_f32(w, oracle.PER_TENSOR)
    assert s[0] == 1.0
    np.testing.assert_array_equal(q, [[127, -2, -1, 1, 2, 3, -3, 0]])


def test_linear_from_tensors_known_answer(oracle):
    # nn_tests.rs:68-79: W = identity (2 x 2), b = [0.5, -0.5], x = [3, 7] -> [3.5, 6.5]; quantized per channel
    # the identity's rows have amax 1, codes {127, 0}, and 127 * (1 / 127) narrows to exactly 1.0f
    w = np.eye(2, dtype=np.float32)
    b = np.array([[0.5, -0.5]], dtype=np.float32)
    x = np.array([[3.0, 7.0]], dtype=np.float32)
    for gran in (oracle.PER_CHANNEL, oracle.PER_TENSOR):
        q, s = oracle.quantize_f32(w, gran)
        np.testing.assert_array_equal(q, [[127, 0], [0, 127]])
        np.testing.assert_array_equal(oracle.dequantize(q, s, gran, "f32"), w)
        np.testing.assert_allclose(oracle.linear_forward_f32(q, s, gran, b, x), [[3.5, 6.5]], rtol=1e-7)


def test_matmul_known_answer_within_quantization_error(oracle):
    # exec_tests.rs:132-173: a [2,3] = rows of the identity, b [3,2] = [[1,2],[3,4],[5,6]] -> [[1,2],[3,4]].
    # As a Linear the weight is b^T; its entries are not multiples of amax / 127, so the quantized result
    # is off by at most half a step per weight: |error| <= 0.5 * amax / 127
    wt = np.array([[1.0, 3.0, 5.0], [2.0, 4.0, 6.0]], dtype=np.float32)
    a = np.array([[1.0, 0.0, 0.0], [0.0, 1.0, 0.0]], dtype=np.float32)
    q, s = oracle.quantize_f32(wt, oracle.PER_CHANNEL)
    y = oracle.linear_forward_f32(q, s, oracle.PER_CHANNEL, None, a)
    assert np.all(np.abs(y - np.array([[1.0, 2.0], [3.0, 4.0]])) <= 0.5 * np.array([5.0, 6.0]) / 127 + 1e-6)
    np.testing.assert_array_equal(q, [[25, 76, 127], [42, 85, 127]])   # round(v * 127 / amax): 25.4, 76.2 | 42.33, 84.67


@pytest.mark.parametrize("shape,gran", [((64, 96), 0), ((64, 96), 1), ((7, 33), 1), ((5, 3, 11), 1), ((1, 513), 0)])
def test_c_oracle_equals_numpy_twin_random(oracle, shape, gran):
    rng = np.random.default_rng(123)
    w = (rng.standard_normal(shape) * 0.02).astype(np.float32)
    w.reshape(-1)[::17] *= 50.0
    qc, sc = oracle.quantize_f32(w, gran)
    qn, sn = oracle.np_quantize_f32(w, gran)
    np.testing.assert_array_equal(qc, qn)
    assert sc.tobytes() == sn.tobytes()
    d64 = oracle.dequantize(qc, sc, gran, "f64")
    np.testing.assert_array_equal(d64, oracle.np_dequantize_f64(qc, sc, gran))
    np.testing.assert_array_equal(oracle.dequantize(qc, sc, gran, "f32"), d64.astype(np.float32))


def test_compression_ratio_and_savings_arithmetic():
    # quantize.rs:701-710 (ratio 4.0 for INT8) and :749-755 (savings 98304 bytes)
    assert (256 * 128 * 4) / (256 * 128) == 4.0
    assert 256 * 128 * 4 - 256 * 128 == 98304


def test_bf16_rounding_matches_torch(oracle):
    import torch
    rng = np.random.default_rng(5)
    vals = np.concatenate([rng.standard_normal(2000) * 10.0 ** rng.integers(-20, 20, 2000),
                           [0.0, -0.0, 1.0, 1.00390625, 1.01171875, 3.3895313892515355e38, 3.4e38, 1e-45, 9.2e-41]])
    got = np.array([oracle.f64_to_bf16_bits(v) for v in vals], dtype=np.uint16)
    # values exactly representable in f32 first, so torch's f32->bf16 RNE is a fair check
    v32 = vals.astype(np.float32)
    got32 = np.array([oracle.f64_to_bf16_bits(float(v)) for v in v32], dtype=np.uint16)
    ref = torch.from_numpy(v32).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    np.testing.assert_array_equal(got32, ref)
    np.testing.assert_array_equal(oracle.f32_to_bf16_bits(v32), ref)
    assert got.shape == vals.shape


def test_forward_c_loop_equals_blas_twin(oracle):
    rng = np.random.default_rng(9)
    w = (rng.standard_normal((37, 64)) * 0.02).astype(np.float32)
    b = rng.standard_normal(37).astype(np.float32)
    x = rng.standard_normal((5, 64)).astype(np.float32)
    for gran in (0, 1):
        q, s = oracle.quantize_f32(w, gran)
        y_c = oracle.linear_forward_f32(q, s, gran, b, x, relu=True)
        y_np = oracle.np_linear_forward(q, s, gran, b, x, relu=True)
        assert oracle.rel_err(y_c, y_np) < 1e-6


def test_committed_golden_file_matches_its_generator(tmp_path, monkeypatch):
    # the fixture is exactly what tests/golden/make_golden.py produces
    import importlib.util
    import json
    import os
    from tests.conftest import ROOT
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(ROOT, "tests", "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = tmp_path / "quantize_golden.json"
    monkeypatch.setattr(mod.os.path, "dirname", lambda p: str(tmp_path))
    mod.main()
    fresh = json.load(open(out))
    committed = json.load(open(os.path.join(ROOT, "tests", "golden", "quantize_golden.json")))
    assert fresh == committed


def test_oracle_property_random_shapes_and_specials(oracle):
    # C oracle == numpy twin over random shapes, scales and injected special values
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=150, deadline=None, derandomize=True)
    @given(rows=st.integers(1, 9), cols=st.integers(0, 40), gran=st.integers(0, 1),
           log_scale=st.floats(-35, 35), seed=st.integers(0, 2 ** 31 - 1),
           special=st.sampled_from([None, np.nan, np.inf, -np.inf, 0.0, -0.0]))
    def check(rows, cols, gran, log_scale, seed, special):
        rng = np.random.default_rng(seed)
        with np.errstate(over="ignore"):
            w = (rng.standard_normal((rows, cols)) * 10.0 ** log_scale).astype(np.float32)
        if special is not None and w.size:
            w.reshape(-1)[rng.integers(0, w.size)] = special
        qc, sc = oracle.quantize_f32(w, gran)
        qn, sn = oracle.np_quantize_f32(w, gran)
        np.testing.assert_array_equal(qc, qn)
        assert sc.tobytes() == sn.tobytes()
        assert np.abs(qc.astype(np.int32)).max(initial=0) <= 127
        d32 = oracle.dequantize(qc, sc, gran, "f32")
        with np.errstate(over="ignore", invalid="ignore"):
            np.testing.assert_array_equal(d32, oracle.np_dequantize_f64(qc, sc, gran).astype(np.float32))

    check()
