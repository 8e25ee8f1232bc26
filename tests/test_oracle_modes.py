"""CPU: the oracle's restatement of the reference's other quantization modes (asymmetric INT8,
INT4 symmetric / asymmetric; crates/shrew/src/quantize.rs:124-139, :339-366) against golden
vectors from the independent pure-Python restatement, and against the reference's own test
assertions for those modes (quantize.rs:626-650, :676-699)."""
import json
import os
import struct

import numpy as np
import pytest

from tests.conftest import ROOT


def _load():
    with open(os.path.join(ROOT, "tests", "golden", "quantize_modes_golden.json")) as f:
        cases = json.load(f)["cases"]
    f64 = lambda bits: np.array([struct.unpack("<d", struct.pack("<Q", b))[0] for b in bits], dtype=np.float64)  # noqa: E731
    out = []
    for c in cases:
        data = np.array([struct.unpack("<f", struct.pack("<I", b))[0] for b in c["data_f32_bits"]],
                        dtype=np.float32).reshape(c["shape"])
        out.append(dict(name=c["name"], data=data, codes=np.array(c["codes"], dtype=np.int8).reshape(c["shape"]),
                        scales=f64(c["scales_f64_bits"]), zps=f64(c["zero_points_f64_bits"]),
                        granularity=1 if c["granularity"] == "per_channel" else 0, bits=c["bits"],
                        mode=1 if c["mode"] == "asymmetric" else 0))
    return out


MODES = _load()


@pytest.mark.parametrize("impl", ["c", "numpy"])
@pytest.mark.parametrize("case", MODES, ids=[c["name"] for c in MODES])
def test_oracle_matches_mode_golden(oracle, case, impl):
    fn = oracle.quantize_f32_ex if impl == "c" else oracle.np_quantize_f32_ex
    q, s, z = fn(case["data"], case["granularity"], case["bits"], case["mode"])
    np.testing.assert_array_equal(q, case["codes"])
    assert s.tobytes() == case["scales"].tobytes()       # bit-exact f64, NaN and Inf included
    assert z.tobytes() == case["zps"].tobytes()


def test_symmetric_int8_is_the_plain_quantizer(oracle):
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((7, 33)) * 0.3).astype(np.float32)
    for gran in (0, 1):
        q, s = oracle.quantize_f32(w, gran)
        q2, s2, z2 = oracle.quantize_f32_ex(w, gran, 8, oracle.SYMMETRIC)
        np.testing.assert_array_equal(q, q2)
        assert s.tobytes() == s2.tobytes() and not z2.any()


def test_ref_int8_asymmetric_round_trip(oracle):
    # quantize.rs:676-699
    data = np.array([[-1.0, -0.5, 0.0, 0.5, 1.0]], dtype=np.float32)
    q, s, z = oracle.quantize_f32_ex(data, oracle.PER_TENSOR, 8, oracle.ASYMMETRIC)
    assert len(s) == 1
    rec = oracle.dequantize_f64_ex(q, s, z, oracle.PER_TENSOR)
    assert np.all(np.abs(data.astype(np.float64) - rec) < 0.02)
    # scale = 2/255; zero point = round(-128 + 127.5) = round(-0.5) = -1 (half away from zero)
    assert s[0] == 2.0 / 255.0 and z[0] == -1.0


def test_ref_int4_symmetric_round_trip(oracle):
    # quantize.rs:626-650: INT4 has max 7, scale = 1/7
    data = np.array([[1.0, -0.5], [0.25, -1.0]], dtype=np.float32)
    q, s, z = oracle.quantize_f32_ex(data, oracle.PER_TENSOR, 4, oracle.SYMMETRIC)
    assert len(s) == 1 and s[0] == 1.0 / 7.0 and z[0] == 0.0
    assert q.min() >= -7 and q.max() <= 7
    rec = oracle.dequantize_f64_ex(q, s, z, oracle.PER_TENSOR)
    assert np.all(np.abs(data.astype(np.float64) - rec) < 0.2)


def test_modes_property_c_equals_numpy(oracle):
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=150, deadline=None, derandomize=True)
    @given(rows=st.integers(1, 7), cols=st.integers(0, 30), gran=st.integers(0, 1), bits=st.sampled_from([4, 8]),
           mode=st.integers(0, 1), log_scale=st.floats(-33, 33), shift=st.floats(-3, 3), seed=st.integers(0, 2 ** 31 - 1),
           special=st.sampled_from([None, np.nan, np.inf, -np.inf, -0.0]))
    def check(rows, cols, gran, bits, mode, log_scale, shift, seed, special):
        rng = np.random.default_rng(seed)
        with np.errstate(over="ignore"):
            w = ((rng.standard_normal((rows, cols)) + shift) * 10.0 ** log_scale).astype(np.float32)
        if special is not None and w.size:
            w.reshape(-1)[rng.integers(0, w.size)] = special
        qc, sc, zc = oracle.quantize_f32_ex(w, gran, bits, mode)
        qn, sn, zn = oracle.np_quantize_f32_ex(w, gran, bits, mode)
        np.testing.assert_array_equal(qc, qn)
        assert sc.tobytes() == sn.tobytes() and zc.tobytes() == zn.tobytes()
        qmax = 7 if bits == 4 else 127
        qmin = -(qmax + 1) if mode else -qmax
        assert qc.min(initial=0) >= qmin and qc.max(initial=0) <= qmax
        if np.isfinite(w).all() and w.size and np.all(np.abs(sc) >= 1e-30):
            # round trip within one quantization step of every element (finite inputs; a scale under
            # 1e-30 makes the reference use an inverse of 0, i.e. every code 0: quantize.rs:236-240)
            rec = oracle.dequantize_f64_ex(qc, sc, zc, gran)
            step = (sc.reshape(-1, 1) if gran else sc.reshape(1, 1)) * np.ones((rows, 1))
            with np.errstate(invalid="ignore", over="ignore"):
                assert np.all(np.abs(rec - w.astype(np.float64)) <= 1.0001 * np.broadcast_to(step, (rows, 1)) + 0.0 * rec)

    check()


def test_committed_modes_file_matches_its_generator(tmp_path, monkeypatch):
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(ROOT, "tests", "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    monkeypatch.setattr(mod.os.path, "dirname", lambda p: str(tmp_path))
    mod.main()
    fresh = json.load(open(tmp_path / "quantize_modes_golden.json"))
    committed = json.load(open(os.path.join(ROOT, "tests", "golden", "quantize_modes_golden.json")))
    assert fresh == committed
