"""CPU oracle for Shrew's INT8 symmetric quantization path (TEST INFRASTRUCTURE ONLY).

Two independent restatements of crates/shrew/src/quantize.rs live here:

* the C library built from ``shrew_oracle.c`` (loaded through ctypes) — scalar f64 loops in
  the reference's own order; this is the checker the CUDA kernels are compared with and
  the thing the benchmark times as the CPU baseline;
* a vectorised numpy twin (functions prefixed ``np_``) used to cross-check the C code.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may import this
module.  The shipped package never does.

Pinning: quantizer arithmetic is pinned by the reference source (std f64 ops) and by the
reference's own test fixtures (quantize.rs:601-789, replayed in tests/test_oracle.py).
The matmul summation order inside QuantizedLinear::forward is PARITY UNPINNED (third-party
`gemm` 0.18.2, not vendored); the forward here accumulates in f64 and rounds once.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

PER_TENSOR = 0
PER_CHANNEL = 1

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libshrew_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile shrew_oracle.c with gcc (see the Makefile beside this file)."""
    src = os.path.join(_HERE, "shrew_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B", "libshrew_oracle.so"])
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        sz, vp, ci = ctypes.c_size_t, ctypes.c_void_p, ctypes.c_int
        L.shrew_oracle_quantize_f32.argtypes = [vp, sz, sz, ci, vp, vp]
        L.shrew_oracle_quantize_f32.restype = ci
        L.shrew_oracle_quantize_f32_ex.argtypes = [vp, sz, sz, ci, ci, ci, vp, vp, vp]
        L.shrew_oracle_quantize_f32_ex.restype = ci
        L.shrew_oracle_dequantize_f64_ex.argtypes = [vp, vp, vp, sz, sz, ci, vp]
        L.shrew_oracle_dequantize_f64_ex.restype = None
        for name in ("f64", "f32", "bf16"):
            fn = getattr(L, f"shrew_oracle_dequantize_{name}")
            fn.argtypes = [vp, vp, sz, sz, ci, vp]
            fn.restype = None
        L.shrew_oracle_dequantize_like_reference.argtypes = [vp, vp, sz, sz, ci, vp]
        L.shrew_oracle_dequantize_like_reference.restype = ci
        L.shrew_oracle_linear_forward_f32.argtypes = [vp, vp, ci, vp, vp, sz, sz, sz, ci, vp]
        L.shrew_oracle_linear_forward_f32.restype = None
        L.shrew_oracle_f64_to_bf16.argtypes = [ctypes.c_double]
        L.shrew_oracle_f64_to_bf16.restype = ctypes.c_uint16
        _lib = L
    return _lib


def _p(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


def _rows_cols(shape) -> tuple[int, int]:
    """rows = shape[0]; cols = product(shape[1..]) (quantize.rs:280-281).  Rank 0 is a
    single per-tensor element (quantize.rs:276-278)."""
    shape = tuple(int(s) for s in shape)
    if len(shape) == 0:
        return 1, 1
    cols = 1
    for s in shape[1:]:
        cols *= s
    return shape[0], cols


# --------------------------------------------------------------------------------------
# C oracle
# --------------------------------------------------------------------------------------
def quantize_f32(w: np.ndarray, granularity: int) -> tuple[np.ndarray, np.ndarray]:
    """quantize_tensor on an F32 tensor (quantize.rs:194-205).  Returns (codes i8 with the
    shape of ``w``, scales f64 of length 1 or shape[0])."""
    w = np.require(w, dtype=np.float32, requirements="C")  # keeps rank 0, unlike ascontiguousarray
    rows, cols = _rows_cols(w.shape)
    if w.ndim == 0:
        granularity = PER_TENSOR
    q = np.empty(w.shape, dtype=np.int8)
    scales = np.empty(rows if granularity == PER_CHANNEL else 1, dtype=np.float64)
    rc = lib().shrew_oracle_quantize_f32(_p(w), rows, cols, granularity, _p(q), _p(scales))
    if rc != 0:
        raise MemoryError("oracle: f64 widening copy failed")
    return q, scales


SYMMETRIC, ASYMMETRIC = 0, 1


def quantize_f32_ex(w: np.ndarray, granularity: int, bits: int = 8, mode: int = SYMMETRIC):
    """quantize_tensor in any of the reference's modes (quantize.rs:124-139, :339-366): INT8 or
    INT4 codes (one per byte), symmetric or asymmetric.  Returns (codes, scales, zero_points)."""
    w = np.require(w, dtype=np.float32, requirements="C")
    rows, cols = _rows_cols(w.shape)
    if w.ndim == 0:
        granularity = PER_TENSOR
    q = np.empty(w.shape, dtype=np.int8)
    n = rows if granularity == PER_CHANNEL else 1
    scales, zps = np.empty(n, dtype=np.float64), np.empty(n, dtype=np.float64)
    rc = lib().shrew_oracle_quantize_f32_ex(_p(w), rows, cols, granularity, bits, mode, _p(q), _p(scales), _p(zps))
    if rc != 0:
        raise MemoryError("oracle: f64 widening copy failed")
    return q, scales, zps


def dequantize_f64_ex(q: np.ndarray, scales: np.ndarray, zero_points: np.ndarray, granularity: int) -> np.ndarray:
    """(q as f64 - zp) * scale (quantize.rs:262-266, :320-335), the intermediate Vec<f64>."""
    q = np.ascontiguousarray(q, dtype=np.int8)
    rows, cols = _rows_cols(q.shape)
    out = np.empty(q.shape, dtype=np.float64)
    lib().shrew_oracle_dequantize_f64_ex(_p(q), _p(np.ascontiguousarray(scales, dtype=np.float64)),
                                         _p(np.ascontiguousarray(zero_points, dtype=np.float64)), rows, cols,
                                         granularity if q.ndim else PER_TENSOR, _p(out))
    return out


def dequantize(q: np.ndarray, scales: np.ndarray, granularity: int, dtype: str = "f32") -> np.ndarray:
    """dequantize_tensor (quantize.rs:210-225).  dtype 'f64' = the intermediate Vec<f64>;
    'f32' / 'bf16' = after Tensor::from_f64_slice narrowing.  bf16 is returned as uint16."""
    q = np.ascontiguousarray(q, dtype=np.int8)
    scales = np.ascontiguousarray(scales, dtype=np.float64)
    rows, cols = _rows_cols(q.shape)
    out = np.empty(q.shape, dtype={"f64": np.float64, "f32": np.float32, "bf16": np.uint16}[dtype])
    getattr(lib(), f"shrew_oracle_dequantize_{dtype}")(_p(q), _p(scales), rows, cols, granularity, _p(out))
    return out


def linear_forward_f32(q, scales, granularity, bias, x, relu: bool = False) -> np.ndarray:
    """QuantizedLinear::forward (quantize.rs:463-476) on f32 activations [M,K]."""
    q = np.ascontiguousarray(q, dtype=np.int8)
    scales = np.ascontiguousarray(scales, dtype=np.float64)
    x = np.ascontiguousarray(x, dtype=np.float32)
    N, K = q.shape
    M = x.shape[0]
    assert x.shape[1] == K
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32).reshape(-1)
    y = np.empty((M, N), dtype=np.float32)
    lib().shrew_oracle_linear_forward_f32(_p(q), _p(scales), granularity, None if b is None else _p(b),
                                          _p(x), M, N, K, int(relu), _p(y))
    return y


def dequantize_like_reference(q, scales, granularity, out: np.ndarray) -> None:
    """One forward call's dequantization with the reference's memory behaviour (fresh f64
    vector, then narrowing copy): the part of the CPU baseline that is single-threaded."""
    rows, cols = _rows_cols(q.shape)
    rc = lib().shrew_oracle_dequantize_like_reference(_p(q), _p(scales), rows, cols, granularity, _p(out))
    if rc != 0:
        raise MemoryError("oracle: f64 dequantize buffer failed")


def f64_to_bf16_bits(v: float) -> int:
    return int(lib().shrew_oracle_f64_to_bf16(float(v)))


# --------------------------------------------------------------------------------------
# numpy twin (cross-check of the C code; also handy for big tensors)
# --------------------------------------------------------------------------------------
def np_round_half_away(t: np.ndarray) -> np.ndarray:
    """f64::round.  trunc(t) plus one step when the exact fractional part is >= 0.5
    (t - trunc(t) is exact in binary floating point)."""
    r = np.trunc(t)
    return np.copysign(r + np.where(np.abs(t - r) >= 0.5, np.sign(t), 0.0), t)  # round(-0.3) is -0.0


def np_quantize_f32(w: np.ndarray, granularity: int) -> tuple[np.ndarray, np.ndarray]:
    w = np.require(w, dtype=np.float32, requirements="C")
    rows, cols = _rows_cols(w.shape)
    data = w.astype(np.float64).reshape(rows, cols)
    if granularity == PER_TENSOR or w.ndim == 0:
        data = data.reshape(1, -1)
    with np.errstate(all="ignore"):
        if data.shape[1] == 0:
            amax = np.zeros(data.shape[0])
        else:
            amax = np.fmax.reduce(np.abs(data), axis=1, initial=0.0)  # fmax ignores NaN like f64::max
        scale = np.where(amax < 1e-30, 1.0, amax / 127.0)
        inv = np.where(np.abs(scale) < 1e-30, 0.0, 1.0 / scale)
        t = np_round_half_away(data * inv[:, None] + 0.0)
        t = np.where(np.isnan(t), 0.0, np.clip(t, -127.0, 127.0))  # NaN as i8 == 0
    return t.astype(np.int8).reshape(w.shape), scale.astype(np.float64)


def np_quantize_f32_ex(w: np.ndarray, granularity: int, bits: int = 8, mode: int = SYMMETRIC):
    """numpy twin of quantize_f32_ex."""
    w = np.require(w, dtype=np.float32, requirements="C")
    rows, cols = _rows_cols(w.shape)
    data = w.astype(np.float64).reshape(rows, cols)
    if granularity == PER_TENSOR or w.ndim == 0:
        data = data.reshape(1, -1)
    qmax = 7.0 if bits == 4 else 127.0
    qmin = (-8.0 if mode == ASYMMETRIC else -7.0) if bits == 4 else (-128.0 if mode == ASYMMETRIC else -127.0)
    g = data.shape[0]
    with np.errstate(all="ignore"):
        if data.shape[1] == 0:
            scale, zp = np.ones(g), np.zeros(g)
        elif mode == ASYMMETRIC:
            lo = np.fmin.reduce(data, axis=1, initial=np.inf)     # fmin / fmax skip NaN like f64::min / max
            hi = np.fmax.reduce(data, axis=1, initial=-np.inf)
            rng = hi - lo
            scale = np.where(rng < 1e-30, 1.0, rng / (qmax - qmin))
            zp = np_round_half_away(qmin - lo / scale)
        else:
            amax = np.fmax.reduce(np.abs(data), axis=1, initial=0.0)
            scale = np.where(amax < 1e-30, 1.0, amax / qmax)
            zp = np.zeros(g)
        inv = np.where(np.abs(scale) < 1e-30, 0.0, 1.0 / scale)
        t = np_round_half_away(data * inv[:, None] + zp[:, None])
        t = np.where(np.isnan(t), 0.0, np.clip(t, qmin, qmax))
    return t.astype(np.int8).reshape(w.shape), scale.astype(np.float64), zp.astype(np.float64)


def np_dequantize_f64(q: np.ndarray, scales: np.ndarray, granularity: int) -> np.ndarray:
    rows, cols = _rows_cols(q.shape)
    s = scales.reshape(-1, 1) if granularity == PER_CHANNEL else scales.reshape(1, 1)
    return ((q.astype(np.float64).reshape(rows, cols) - 0.0) * s).reshape(q.shape)


def np_linear_forward(q, scales, granularity, bias, x, relu: bool = False) -> np.ndarray:
    """Twin of linear_forward_f32 for sizes the scalar C loop is too slow for: the same
    f32 dequantized weight, product accumulated in f64 (BLAS order, still f64), rounded to
    f32 once, then the f32 bias add."""
    w = dequantize(q, scales, granularity, "f32").astype(np.float64)
    y = (np.ascontiguousarray(x, dtype=np.float32).astype(np.float64) @ w.T).astype(np.float32)
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float32).reshape(1, -1)
    if relu:
        y = np.maximum(y, np.float32(0))
    return y.astype(np.float32)


def rel_err(y: np.ndarray, y_ref: np.ndarray) -> float:
    """max|y - y_ref| / max|y_ref| over one output tensor: the figure the tolerances
    (1e-2 bf16 path, 1e-4 f32-accumulate path) are stated on."""
    y = np.asarray(y, dtype=np.float64)
    y_ref = np.asarray(y_ref, dtype=np.float64)
    denom = float(np.max(np.abs(y_ref))) if y_ref.size else 0.0
    if denom == 0.0:
        return float(np.max(np.abs(y - y_ref))) if y.size else 0.0
    return float(np.max(np.abs(y - y_ref)) / denom)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """f32 -> bf16 round to nearest even (used to make bf16 test activations)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = b + (0x7FFF + ((b >> 16) & 1))
    out = (rounded >> 16).astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        out = np.where(nan, np.uint16(0x7FC0), out)
    return out
