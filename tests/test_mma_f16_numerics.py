"""CPU model of the arithmetic of the f16 warp-MMA kernel (shrew_b200/csrc/gemv_mma.cu, "mma-f16").

Three claims of that kernel are checked here without a GPU:
1. the two-instruction widening of INT8 codes to f16 is exact for all 256 byte values
   (byte-permute into halves 0x6400 | u, packed subtract of 1152);
2. the per-token power-of-two rescale puts every row's largest magnitude into [2^14, 2^15) and
   converts every element within 2^-31 of it to f16 without error;
3. a dot product computed from the rescaled f16 activations and scaled back by 2^-s agrees with
   the f64 dot product of the original bf16 activations far inside the f32 tolerance, for
   activations spread over 70 orders of magnitude.
The fragment/index mapping of the kernel is shared with the bf16 variant and covered by
tests/test_mma_layout.py."""
import numpy as np
import pytest


def byte_perm(x, y, sel):
    """__byte_perm(x, y, s): result byte i = byte (nibble i of s) of the 8-byte value y:x."""
    src = [(x >> (8 * i)) & 0xFF for i in range(4)] + [(y >> (8 * i)) & 0xFF for i in range(4)]
    out = 0
    for i in range(4):
        out |= src[(sel >> (4 * i)) & 0x7] << (8 * i)
    return out


def halves(word):
    return np.array([word & 0xFFFF, word >> 16], dtype=np.uint16).view(np.float16)


def test_code_widening_is_exact_for_every_byte():
    assert np.array([0x6480], np.uint16).view(np.float16)[0] == np.float16(1152.0)
    codes = np.arange(-128, 128, dtype=np.int8)
    for i in range(0, 256, 4):
        b = codes[i:i + 4]
        w = int(b.view(np.uint8)[0]) | int(b.view(np.uint8)[1]) << 8 | int(b.view(np.uint8)[2]) << 16 | int(b.view(np.uint8)[3]) << 24
        u = w ^ 0x80808080
        h01 = byte_perm(u, 0x64646464, 0x4140)
        h23 = byte_perm(u, 0x64646464, 0x4342)
        lo = halves(h01) - np.float16(1152.0)
        hi = halves(h23) - np.float16(1152.0)
        assert lo.dtype == np.float16
        np.testing.assert_array_equal(np.concatenate([lo, hi]).astype(np.int32), b.astype(np.int32))


def to_bf16(x):
    """round-to-nearest-even f32 -> bf16, returned as f32"""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32)


def rescale_row(x_row):
    """the kernel's x_to_f16 step for one token row of bf16 values (held as f32)"""
    finite = x_row[~np.isnan(x_row)]
    amax = float(np.max(np.abs(finite))) if finite.size else 0.0
    if amax == 0.0:
        e = 0
    elif np.isinf(amax):
        e = 127
    else:
        e = int(np.floor(np.log2(amax)))
        # ilogb semantics, robust against log2 rounding at powers of two
        while np.ldexp(1.0, e) > amax:
            e -= 1
        while np.ldexp(1.0, e + 1) <= amax:
            e += 1
    s = 14 - e
    with np.errstate(over="ignore"):
        x16 = np.ldexp(x_row.astype(np.float32), s).astype(np.float16)
    return x16, s, amax


@pytest.mark.parametrize("scale", [1e-37, 1e-30, 1e-12, 1e-3, 1.0, 123.0, 6e4, 1e9, 1e20, 3e38])
def test_rescale_places_amax_and_is_exact_near_it(scale):
    rng = np.random.default_rng(5)
    x = to_bf16((rng.standard_normal(4096) * scale / 4).astype(np.float32))
    x = x[np.isfinite(x)]
    x16, s, amax = rescale_row(x)
    top = np.ldexp(np.float64(amax), s)
    assert 2.0 ** 14 <= top < 2.0 ** 15
    back = np.ldexp(x16.astype(np.float64), -s)
    near = np.abs(x) >= amax * 2.0 ** -31
    np.testing.assert_array_equal(back[near], x[near].astype(np.float64))
    assert np.max(np.abs(back - x.astype(np.float64))) <= amax * 2.0 ** -39


def test_rescale_wide_spread_inside_one_row():
    # one row holding values from 2^-60 to 2^20 of its amax scale: the small ones are rounded, by
    # at most amax * 2^-39 each
    rng = np.random.default_rng(6)
    expo = rng.integers(-60, 21, size=2048)
    x = to_bf16((rng.standard_normal(2048) * np.exp2(expo)).astype(np.float32))
    x16, s, amax = rescale_row(x)
    back = np.ldexp(x16.astype(np.float64), -s)
    assert np.max(np.abs(back - x.astype(np.float64))) <= amax * 2.0 ** -39
    near = np.abs(x) >= amax * 2.0 ** -31
    np.testing.assert_array_equal(back[near], x[near].astype(np.float64))


@pytest.mark.parametrize("row_scales", [
    [1.0, 1e-6, 1e3, 0.0, 1e-30, 1e30],
    [3e4, 7e4, 65504.0, 65520.0, 1e5, 6e-8],   # around f16's own limits
])
def test_dot_products_match_f64(row_scales):
    rng = np.random.default_rng(7)
    K, N = 1024, 64
    q = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
    w_scale = (rng.random(N) * 1e-3 + 1e-5)
    x = to_bf16((rng.standard_normal((len(row_scales), K)) * np.array(row_scales)[:, None]).astype(np.float32))
    for m in range(x.shape[0]):
        x16, s, amax = rescale_row(x[m])
        # tensor-core products are exact (8-bit x 11-bit); model the f32 accumulation by f64 sums
        # rounded once, the centre of any f32 summation order
        acc = (q.astype(np.float64) @ x16.astype(np.float64)).astype(np.float32)
        y = np.ldexp(acc, -s).astype(np.float64) * w_scale
        ref = (q.astype(np.float64) @ x[m].astype(np.float64)) * w_scale
        denom = np.max(np.abs(ref))
        if denom == 0.0:
            assert np.all(y == 0.0)
        else:
            assert np.max(np.abs(y - ref)) / denom < 1e-6


def test_special_values_follow_ieee():
    x = to_bf16(np.array([1.0, -2.0, np.inf, 3.0], np.float32))
    x16, s, _ = rescale_row(x)
    assert s == 14 - 127 and np.isinf(x16[2])           # Inf stays Inf, finite neighbours underflow
    x = to_bf16(np.array([1.0, np.nan, -4.0], np.float32))
    x16, s, amax = rescale_row(x)
    assert amax == 4.0 and s == 12 and np.isnan(x16[1]) and x16[2] == np.float16(-16384.0)
    x16, s, _ = rescale_row(np.zeros(8, np.float32))
    assert s == 14 and not x16.any()
