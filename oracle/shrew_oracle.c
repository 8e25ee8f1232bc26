/*
 * shrew_oracle.c — CPU restatement of Shrew's INT8 symmetric quantization path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are compared
 * against.  Nothing in the shipped library links, loads or calls it; only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg may.
 *
 * What is pinned and what is not:
 *   - The quantizer / dequantizer arithmetic below follows the reference source line by
 *     line (std f64 operations only), so codes and scales are expected bit-exact.  The
 *     reference's own tests hold no golden INT8 code vectors; they hold small fixed
 *     inputs with tolerance / metadata assertions (crates/shrew/src/quantize.rs:601-789).
 *     Those fixtures are replayed against this file in tests/test_oracle.py, and a third
 *     independent restatement (pure Python floats, tests/golden/make_golden.py) pins the
 *     exact codes for them.
 *   - The matmul inside QuantizedLinear::forward (quantize.rs:469) is computed by the
 *     third-party `gemm` crate 0.18.2 (Cargo.lock:439-440), reached through the
 *     un-vendored shrew-cpu crate: its summation order is PARITY UNPINNED.  The forward
 *     here accumulates in f64 and rounds once, the centre of every valid f32 ordering;
 *     kernels are compared to it under a stated tolerance, never bit-exactly.
 *
 *   - The *_ex functions restate the reference's other modes (asymmetric INT8, INT4 symmetric
 *     and asymmetric, quantize.rs:124-139, :339-366) the same way; tests/test_oracle_modes.py
 *     pins them.  They are ahead of the CUDA library, which implements INT8 symmetric only.
 *
 * The reference cannot be compiled here (Rust, sibling crates absent), so there is no
 * oracle/_ref build of it.
 *
 * Build: make -C oracle      (gcc -O2 -ffp-contract=off: no FMA contraction, so every
 * f64 multiply and add rounds exactly as the reference's separate operations do)
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define SHREW_PER_TENSOR 0
#define SHREW_PER_CHANNEL 1
#define SHREW_SYMMETRIC 0
#define SHREW_ASYMMETRIC 1

/* Rust f64::round: round half away from zero (pinned by
 * crates/shrew/tests/nn_tests.rs:2413-2420).  C99 round() has the same definition. */
static inline double round_half_away(double v) { return round(v); }

/* Rust `f64 as i8`: saturating, NaN -> 0.  After clamp(-127,127) only NaN is special. */
static inline int8_t f64_as_i8(double v) {
    if (v != v) return 0;
    if (v >= 127.0) return 127;
    if (v <= -128.0) return -128;
    return (int8_t)v; /* truncation toward zero; v is integral here */
}

/* Rust f64::clamp(min,max): NaN stays NaN. */
static inline double clamp_f64(double v, double lo, double hi) {
    if (v < lo) return lo;
    if (v > hi) return hi;
    return v;
}

/* Rust f64::max(a,b): if one operand is NaN the other is returned. */
static inline double max_ignore_nan(double a, double b) {
    if (a != a) return b;
    if (b != b) return a;
    return a > b ? a : b;
}

/* compute_scale_zp, symmetric branch — quantize.rs:339-352.
 * Empty slice -> (1.0, 0.0) (quantize.rs:340-342); amax < 1e-30 -> scale 1.0 (:350). */
static double scale_symmetric_int8(const double *data, size_t n) {
    if (n == 0) return 1.0;
    double amax = 0.0;
    for (size_t i = 0; i < n; ++i) amax = max_ignore_nan(amax, fabs(data[i]));
    return amax < 1e-30 ? 1.0 : amax / 127.0;
}

/* inv_scale guard — quantize.rs:236-240 and :295-299. */
static inline double inv_scale_of(double scale) { return fabs(scale) < 1e-30 ? 0.0 : 1.0 / scale; }

/* The element map — quantize.rs:244-250 and :301-304 with zero_point = 0.0. */
static inline int8_t quantize_one(double v, double inv_scale) {
    double q = clamp_f64(round_half_away(v * inv_scale + 0.0), -127.0, 127.0);
    return f64_as_i8(q);
}

/* quantize_per_tensor — quantize.rs:229-260. */
static void quantize_per_tensor_f64(const double *data, size_t n, int8_t *q, double *scale_out) {
    double scale = scale_symmetric_int8(data, n);
    double inv = inv_scale_of(scale);
    for (size_t i = 0; i < n; ++i) q[i] = quantize_one(data[i], inv);
    *scale_out = scale;
}

/* quantize_per_channel — quantize.rs:270-318.  channels = shape[0],
 * channel_size = product(shape[1..]) (:280-281). */
static void quantize_per_channel_f64(const double *data, size_t channels, size_t channel_size,
                                     int8_t *q, double *scales) {
    for (size_t ch = 0; ch < channels; ++ch) {
        const double *row = data + ch * channel_size;
        double scale = scale_symmetric_int8(row, channel_size);
        double inv = inv_scale_of(scale);
        for (size_t i = 0; i < channel_size; ++i) q[ch * channel_size + i] = quantize_one(row[i], inv);
        scales[ch] = scale;
    }
}

/*
 * quantize_tensor for an F32 tensor — quantize.rs:194-205.  The tensor is first widened
 * to a Vec<f64> copy (to_f64_vec, :198), then dispatched on granularity.
 * `rows` = shape[0], `cols` = product(shape[1..]).  scales receives 1 (per-tensor) or
 * `rows` (per-channel) values.  Returns 0, or -1 if the f64 copy cannot be allocated.
 */
int shrew_oracle_quantize_f32(const float *w, size_t rows, size_t cols, int granularity,
                              int8_t *q, double *scales) {
    size_t n = rows * cols;
    double *data = (double *)malloc((n ? n : 1) * sizeof(double));
    if (!data) return -1;
    for (size_t i = 0; i < n; ++i) data[i] = (double)w[i];
    if (granularity == SHREW_PER_CHANNEL)
        quantize_per_channel_f64(data, rows, cols, q, scales);
    else
        quantize_per_tensor_f64(data, n, q, scales);
    free(data);
    return 0;
}

/* ---- every mode: INT8 / INT4 codes (one per byte, as the reference stores them), symmetric or
 * asymmetric.  qmax / qmin — quantize.rs:124-139. */
static double qmax_of(int bits) { return bits == 4 ? 7.0 : 127.0; }
static double qmin_of(int bits, int mode) {
    if (bits == 4) return mode == SHREW_ASYMMETRIC ? -8.0 : -7.0;
    return mode == SHREW_ASYMMETRIC ? -128.0 : -127.0;
}

/* compute_scale_zp, both branches — quantize.rs:339-366.  f64::min / f64::max return the other
 * operand when one is NaN, which is fmin / fmax. */
static void scale_zp_of(const double *data, size_t n, int bits, int mode, double *scale, double *zp) {
    if (n == 0) { *scale = 1.0; *zp = 0.0; return; }
    const double qmin = qmin_of(bits, mode), qmax = qmax_of(bits);
    if (mode != SHREW_ASYMMETRIC) {
        double amax = 0.0;
        for (size_t i = 0; i < n; ++i) amax = max_ignore_nan(amax, fabs(data[i]));
        *scale = amax < 1e-30 ? 1.0 : amax / qmax;
        *zp = 0.0;
        return;
    }
    double min_val = INFINITY, max_val = -INFINITY;
    for (size_t i = 0; i < n; ++i) {
        min_val = fmin(min_val, data[i]);
        max_val = fmax(max_val, data[i]);
    }
    const double range = max_val - min_val;
    *scale = range < 1e-30 ? 1.0 : range / (qmax - qmin);
    *zp = round_half_away(qmin - min_val / *scale);
}

/* The element map with a zero point and the mode's clamp range — quantize.rs:244-250, :301-304.
 * f64::clamp keeps a NaN, and NaN as i8 is 0. */
static inline int8_t quantize_one_ex(double v, double inv_scale, double zp, double qmin, double qmax) {
    double t = round_half_away(v * inv_scale + zp);
    if (t != t) return 0;
    return f64_as_i8(clamp_f64(t, qmin, qmax));
}

/* quantize_tensor for an F32 tensor in any mode — quantize.rs:194-205, :229-260, :270-318.
 * scales and zero_points receive 1 (per-tensor) or `rows` (per-channel) values. */
int shrew_oracle_quantize_f32_ex(const float *w, size_t rows, size_t cols, int granularity, int bits, int mode,
                                 int8_t *q, double *scales, double *zero_points) {
    size_t n = rows * cols;
    double *data = (double *)malloc((n ? n : 1) * sizeof(double));
    if (!data) return -1;
    for (size_t i = 0; i < n; ++i) data[i] = (double)w[i];
    const double qmin = qmin_of(bits, mode), qmax = qmax_of(bits);
    const size_t groups = granularity == SHREW_PER_CHANNEL ? rows : 1;
    const size_t len = granularity == SHREW_PER_CHANNEL ? cols : n;
    for (size_t g = 0; g < groups; ++g) {
        const double *src = data + g * len;
        double scale, zp;
        scale_zp_of(src, len, bits, mode, &scale, &zp);
        const double inv = inv_scale_of(scale);
        for (size_t i = 0; i < len; ++i) q[g * len + i] = quantize_one_ex(src[i], inv, zp, qmin, qmax);
        scales[g] = scale;
        zero_points[g] = zp;
    }
    free(data);
    return 0;
}

/* dequantize with zero points — quantize.rs:262-266, :320-335: (q as f64 - zp) * scale. */
void shrew_oracle_dequantize_f64_ex(const int8_t *q, const double *scales, const double *zero_points, size_t rows,
                                    size_t cols, int granularity, double *out) {
    for (size_t r = 0; r < rows; ++r) {
        const double s = granularity == SHREW_PER_CHANNEL ? scales[r] : scales[0];
        const double zp = granularity == SHREW_PER_CHANNEL ? zero_points[r] : zero_points[0];
        for (size_t c = 0; c < cols; ++c) out[r * cols + c] = ((double)q[r * cols + c] - zp) * s;
    }
}

/* dequantize_per_tensor / dequantize_per_channel — quantize.rs:262-266, :320-335:
 * (q as f64 - zp) * scale with zp = 0.0, as f64. */
void shrew_oracle_dequantize_f64(const int8_t *q, const double *scales, size_t rows, size_t cols,
                                 int granularity, double *out) {
    for (size_t r = 0; r < rows; ++r) {
        double s = granularity == SHREW_PER_CHANNEL ? scales[r] : scales[0];
        for (size_t c = 0; c < cols; ++c) out[r * cols + c] = ((double)q[r * cols + c] - 0.0) * s;
    }
}

/* dequantize_tensor to an F32 tensor — quantize.rs:210-225: the f64 values are narrowed
 * by Tensor::from_f64_slice (round to nearest even, the `as f32` cast). */
void shrew_oracle_dequantize_f32(const int8_t *q, const double *scales, size_t rows, size_t cols,
                                 int granularity, float *out) {
    for (size_t r = 0; r < rows; ++r) {
        double s = granularity == SHREW_PER_CHANNEL ? scales[r] : scales[0];
        for (size_t c = 0; c < cols; ++c) out[r * cols + c] = (float)(((double)q[r * cols + c] - 0.0) * s);
    }
}

/* f64 -> bf16, round to nearest even in one step, as half::bf16::from_f64 does
 * (half 2.7.1, Cargo.lock:591-592; used by the reference at safetensors.rs:102-104). */
uint16_t shrew_oracle_f64_to_bf16(double v) {
    if (v != v) return 0x7FC0;
    uint64_t b;
    memcpy(&b, &v, 8);
    uint16_t sign = (uint16_t)((b >> 48) & 0x8000u);
    double a = fabs(v);
    if (a == 0.0) return sign;
    if (isinf(a)) return sign | 0x7F80u;
    /* scale so that one bf16 ulp at this magnitude equals 1.0, then round half even */
    int e;
    (void)frexp(a, &e);        /* a = m * 2^e, m in [0.5,1) ; unbiased exponent = e-1 */
    int ex = e - 1;
    if (ex < -126) ex = -126;  /* subnormal range shares the ulp of 2^-126 */
    double ulp = ldexp(1.0, ex - 7);
    double n = nearbyint(a / ulp); /* default rounding mode: to nearest even; a/ulp is exact */
    double r = n * ulp;
    if (r > 3.3895313892515355e38) return sign | 0x7F80u; /* beyond max finite bf16 */
    float f = (float)r; /* exact: r has at most 8 significant bits */
    uint32_t fb;
    memcpy(&fb, &f, 4);
    return sign | (uint16_t)(fb >> 16);
}

float shrew_oracle_bf16_to_f32(uint16_t h) {
    uint32_t b = (uint32_t)h << 16;
    float f;
    memcpy(&f, &b, 4);
    return f;
}

void shrew_oracle_dequantize_bf16(const int8_t *q, const double *scales, size_t rows, size_t cols,
                                  int granularity, uint16_t *out) {
    for (size_t r = 0; r < rows; ++r) {
        double s = granularity == SHREW_PER_CHANNEL ? scales[r] : scales[0];
        for (size_t c = 0; c < cols; ++c)
            out[r * cols + c] = shrew_oracle_f64_to_bf16(((double)q[r * cols + c] - 0.0) * s);
    }
}

/*
 * QuantizedLinear::forward — quantize.rs:463-476.
 *   weight = dequantize_tensor(weight_q)      f32 [N,K]        (:465)
 *   out    = x.matmul(weight.t())             [M,K]x[K,N]      (:468-469)
 *   out    = out.add(bias)  if bias           bias [1,N]       (:471-472)
 * x is f32 [M,K] (bf16 activations are widened exactly by the caller).  The product is
 * accumulated in f64 over the f32 weights and rounded to f32 once; the bias is then added
 * in f32 as the reference's separate `add` does.  `relu` != 0 applies max(.,0) after the
 * bias (the tensor op a caller applies between layers).
 */
void shrew_oracle_linear_forward_f32(const int8_t *q, const double *scales, int granularity,
                                     const float *bias, const float *x, size_t M, size_t N,
                                     size_t K, int relu, float *y) {
    size_t nk = N * K;
    float *w = (float *)malloc((nk ? nk : 1) * sizeof(float));
    if (!w) return;
    shrew_oracle_dequantize_f32(q, scales, N, K, granularity, w);
    for (size_t m = 0; m < M; ++m) {
        for (size_t n = 0; n < N; ++n) {
            double acc = 0.0;
            const float *xr = x + m * K, *wr = w + n * K;
            for (size_t k = 0; k < K; ++k) acc += (double)xr[k] * (double)wr[k];
            float o = (float)acc;
            if (bias) o = o + bias[n];
            if (relu && o < 0.0f) o = 0.0f;
            y[m * N + n] = o;
        }
    }
    free(w);
}

/* The dequantize step of one forward call exactly as the reference performs it: a fresh
 * Vec<f64> (8 B/element) then a narrowing copy to f32 (quantize.rs:214-224).  Used by the
 * benchmark's CPU baseline so the per-call dequantization cost is timed as the reference
 * pays it (single thread, two passes). */
int shrew_oracle_dequantize_like_reference(const int8_t *q, const double *scales, size_t rows,
                                           size_t cols, int granularity, float *out) {
    size_t n = rows * cols;
    double *tmp = (double *)malloc((n ? n : 1) * sizeof(double));
    if (!tmp) return -1;
    shrew_oracle_dequantize_f64(q, scales, rows, cols, granularity, tmp);
    for (size_t i = 0; i < n; ++i) out[i] = (float)tmp[i];
    free(tmp);
    return 0;
}
