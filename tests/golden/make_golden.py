"""Generates tests/golden/quantize_golden.json.

The reference (Rust) cannot be executed here and its tests hold no golden INT8 code
vectors, only small fixed inputs with tolerance and metadata assertions
(crates/shrew/src/quantize.rs:601-789).  This script replays those inputs, plus the edge
cases the reference's code branches on, through a THIRD restatement of the quantizer that
shares no code with oracle/: plain Python floats (IEEE binary64, the same arithmetic as
Rust f64) and math.trunc for the rounding.  The resulting codes and scales are the
committed golden vectors; tests check the C oracle, its numpy twin and the CUDA kernels
against them, and check the reference's own assertions on them.

Run:  python tests/golden/make_golden.py
"""
import json
import math
import os
import struct


def f32(v: float) -> float:
    """Value after storing in an F32 tensor (Tensor::from_f64_slice with DType::F32)."""
    return struct.unpack("<f", struct.pack("<f", v))[0]


def exact_round_half_away(t: float) -> float:
    """f64::round.  floor(t+0.5) can be off when t+0.5 itself rounds (0.49999999999999994),
    so decide on t - trunc(t), which is exact."""
    if t != t or math.isinf(t):
        return t
    r = float(math.trunc(t))
    if abs(t - r) >= 0.5:
        r += 1.0 if t > 0 else -1.0
    return math.copysign(r, t)  # f64::round keeps the sign: round(-0.3) is -0.0


def scale_of(vals):
    if not vals:
        return 1.0
    amax = 0.0
    for v in vals:
        a = abs(v)
        if a == a and (amax != amax or a > amax):  # f64::max ignores a NaN operand
            amax = a
    return 1.0 if amax < 1e-30 else amax / 127.0


def quantize(vals, scale):
    inv = 0.0 if abs(scale) < 1e-30 else 1.0 / scale
    out = []
    for v in vals:
        t = v * inv + 0.0
        t = exact_round_half_away(t)
        if t != t:
            out.append(0)  # NaN as i8
            continue
        t = min(max(t, -127.0), 127.0)
        out.append(int(t))
    return out


def case(name, shape, data, granularity, note):
    data = [f32(v) for v in data]
    rows = shape[0] if shape else 1
    cols = 1
    for s in shape[1:]:
        cols *= s
    if granularity == "per_channel" and shape:
        scales, codes = [], []
        for r in range(rows):
            row = data[r * cols:(r + 1) * cols]
            s = scale_of(row)
            scales.append(s)
            codes += quantize(row, s)
    else:
        s = scale_of(data)
        scales, codes = [s], quantize(data, s)
    return {
        "name": name, "note": note, "shape": shape, "granularity": granularity,
        # inputs as f32 bit patterns so NaN / inf / -0.0 survive JSON
        "data_f32_bits": [struct.unpack("<I", struct.pack("<f", v))[0] for v in data],
        "codes": codes,
        "scales_f64_bits": [struct.unpack("<Q", struct.pack("<d", s))[0] for s in scales],
    }


# ---- the other modes: asymmetric INT8, INT4 symmetric / asymmetric (quantize.rs:124-139, :339-366) ----
def qrange(bits, mode):
    qmax = 7.0 if bits == 4 else 127.0
    if bits == 4:
        return (-8.0 if mode == "asymmetric" else -7.0), qmax
    return (-128.0 if mode == "asymmetric" else -127.0), qmax


def scale_zp_of(vals, bits, mode):
    if not vals:
        return 1.0, 0.0
    qmin, qmax = qrange(bits, mode)
    if mode == "symmetric":
        amax = 0.0
        for v in vals:
            a = abs(v)
            if a == a and a > amax:
                amax = a
        return (1.0 if amax < 1e-30 else amax / qmax), 0.0
    lo, hi = float("inf"), float("-inf")
    for v in vals:  # f64::min / f64::max keep the other operand when one is NaN
        if v == v:
            lo = v if v < lo else lo
            hi = v if v > hi else hi
    rng = hi - lo
    scale = 1.0 if rng < 1e-30 else rng / (qmax - qmin)
    return scale, exact_round_half_away(qmin - div(lo, scale))


def div(a, b):
    """IEEE division (Python raises on a zero divisor; not reachable here, scale is never 0)."""
    return a / b


def quantize_mode(vals, scale, zp, bits, mode):
    qmin, qmax = qrange(bits, mode)
    inv = 0.0 if abs(scale) < 1e-30 else 1.0 / scale
    out = []
    for v in vals:
        t = exact_round_half_away(v * inv + zp)
        if t != t:
            out.append(0)
            continue
        out.append(int(min(max(t, qmin), qmax)))
    return out


def mode_case(name, shape, data, granularity, bits, mode, note):
    data = [f32(v) for v in data]
    rows = shape[0] if shape else 1
    cols = 1
    for s in shape[1:]:
        cols *= s
    groups = [data[r * cols:(r + 1) * cols] for r in range(rows)] if (granularity == "per_channel" and shape) else [data]
    scales, zps, codes = [], [], []
    for g in groups:
        s, z = scale_zp_of(g, bits, mode)
        scales.append(s)
        zps.append(z)
        codes += quantize_mode(g, s, z, bits, mode)
    bits64 = lambda v: struct.unpack("<Q", struct.pack("<d", v))[0]  # noqa: E731
    return {"name": name, "note": note, "shape": shape, "granularity": granularity, "bits": bits, "mode": mode,
            "data_f32_bits": [struct.unpack("<I", struct.pack("<f", v))[0] for v in data], "codes": codes,
            "scales_f64_bits": [bits64(s) for s in scales], "zero_points_f64_bits": [bits64(z) for z in zps]}


def mode_cases():
    inf, nan = float("inf"), float("nan")
    ramp = [(i - 6.0) * 0.1 for i in range(12)]
    out = []
    for bits in (8, 4):
        for mode in ("symmetric", "asymmetric"):
            tag = f"int{bits}_{mode}"
            out += [
                mode_case(f"{tag}_ref_asymmetric_input", [1, 5], [-1.0, -0.5, 0.0, 0.5, 1.0], "per_tensor", bits, mode,
                          "input of quantize.rs:676-699 (the reference asserts round-trip < 0.02 in INT8 asymmetric)"),
                mode_case(f"{tag}_ref_int4_input", [2, 2], [1.0, -0.5, 0.25, -1.0], "per_tensor",
                          bits, mode, "input of quantize.rs:626-650 (the reference asserts round-trip < 0.2 in INT4 symmetric)"),
                mode_case(f"{tag}_ramp_per_channel", [3, 4], ramp, "per_channel", bits, mode, "three rows, own scale and zero point each"),
                mode_case(f"{tag}_constant_rows", [2, 3], [3.0, 3.0, 3.0, -2.0, -2.0, -2.0], "per_channel", bits, mode,
                          "range < 1e-30 -> scale 1.0, zero point qmin - min"),
                mode_case(f"{tag}_positive_only", [1, 6], [0.1, 0.2, 0.4, 0.8, 1.6, 3.2], "per_tensor", bits, mode,
                          "one-sided data: the asymmetric range starts at the minimum"),
                mode_case(f"{tag}_zeros", [2, 2], [0.0] * 4, "per_tensor", bits, mode, "all zero"),
                mode_case(f"{tag}_nan_inf", [2, 3], [nan, 1.0, -2.0, inf, -1.0, 0.5], "per_channel", bits, mode,
                          "NaN skipped by min/max, code 0; a row holding Inf: scale Inf, inverse 0"),
                mode_case(f"{tag}_all_nan", [1, 3], [nan, nan, nan], "per_tensor", bits, mode, "min=+Inf, max=-Inf, range=-Inf < 1e-30"),
                mode_case(f"{tag}_empty", [0, 3], [], "per_channel", bits, mode, "no channels"),
                mode_case(f"{tag}_empty_cols", [2, 0], [], "per_channel", bits, mode, "empty channels -> (1.0, 0.0)"),
                mode_case(f"{tag}_rank0", [], [2.5], "per_channel", bits, mode, "rank 0 falls back to per-tensor"),
                mode_case(f"{tag}_negative_zero_point", [1, 2], [0.12573022, -0.13210486], "per_tensor", bits, mode,
                          "INT4 asymmetric: qmin - min/scale = -0.31 rounds to -0.0, sign kept in the zero point"),
                mode_case(f"{tag}_ties", [1, 6], [7.0, 3.5, -3.5, 0.5, -0.5, 1.5], "per_tensor", bits, mode, "products on .5"),
            ]
    return out


def main():
    inf, nan = float("inf"), float("nan")
    cases = [
        case("ref_int8_symmetric_per_tensor", [2, 3], [1.0, -0.5, 0.25, -1.0, 0.0, 0.75], "per_tensor",
             "quantize.rs:603-611: scales.len()==1, zero_points==[0.0], round-trip < 0.02"),
        case("ref_int8_per_channel", [3, 4], [(i - 6.0) * 0.1 for i in range(12)], "per_channel",
             "quantize.rs:654-673: 3 scales, round-trip < 0.01"),
        case("ref_zero_tensor", [2, 3], [0.0] * 6, "per_tensor",
             "quantize.rs:781-789: amax < 1e-30 -> scale 1.0, exact zeros back"),
        case("ref_zero_tensor_per_channel", [2, 3], [0.0] * 6, "per_channel", "same branch per row"),
        case("ref_asym_data_symmetric_mode", [1, 5], [-1.0, -0.5, 0.0, 0.5, 1.0], "per_tensor",
             "input of quantize.rs:677 run in symmetric mode"),
        case("half_ties", [1, 8], [127.0, 63.5, -63.5, 0.5, -0.5, 1.5, -2.5, 126.5], "per_tensor",
             "exact .5 products: round half away from zero (nn_tests.rs:2413-2420)"),
        case("tiny_amax", [2, 2], [1e-31, -5e-32, 1e-29, -1e-29], "per_channel",
             "row 0 below 1e-30 -> scale 1.0; row 1 above"),
        case("nan_ignored_in_amax", [1, 4], [nan, 1.0, -2.0, 0.5], "per_tensor",
             "f64::max skips NaN; NaN as i8 == 0"),
        case("inf_input", [2, 3], [inf, 1.0, -1.0, 2.0, -inf, nan], "per_channel",
             "scale=inf -> inv=0 -> finite*0=0, inf*0=NaN -> 0"),
        case("negative_zero", [1, 3], [-0.0, 0.0, -1.0], "per_tensor", "-0.0 -> code 0"),
        case("rank1_per_channel", [5], [0.5, -0.25, 0.0, 3.0, -7.0], "per_channel",
             "rank 1: channel_size = empty product = 1, every element its own channel"),
        case("rank0", [], [2.5], "per_channel", "quantize.rs:276-278: rank 0 falls back to per-tensor"),
        case("rank3_per_channel", [2, 2, 3], [0.1 * i - 0.55 for i in range(12)], "per_channel",
             "channel_size = product(shape[1..]) = 6"),
        case("empty_rows", [0, 4], [], "per_channel", "no channels"),
        case("empty_cols", [3, 0], [], "per_channel", "empty channel -> (1.0, 0.0) (quantize.rs:340-342)"),
        case("empty_per_tensor", [0], [], "per_tensor", "empty tensor -> scale 1.0"),
        case("bias_like_1xN", [1, 4], [0.01, -0.02, 0.03, 0.0], "per_tensor",
             "quantize.rs:760-776: a [1,out] bias is rank 2 and gets quantized too"),
        case("large_magnitude", [1, 3], [3.0e38, -1.5e38, 1.0e30], "per_channel", "near f32 max"),
        case("subnormal_f32", [1, 3], [1e-40, -1e-41, 0.0], "per_tensor", "f32 subnormals widen exactly"),
    ]
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "quantize_golden.json")
    with open(out, "w") as f:
        json.dump({"generator": "tests/golden/make_golden.py", "cases": cases}, f, indent=1)
    print("wrote", out, len(cases), "cases")
    out2 = os.path.join(os.path.dirname(os.path.abspath(__file__)), "quantize_modes_golden.json")
    mc = mode_cases()
    with open(out2, "w") as f:
        json.dump({"generator": "tests/golden/make_golden.py", "cases": mc}, f, indent=1)
    print("wrote", out2, len(mc), "cases")


if __name__ == "__main__":
    main()
