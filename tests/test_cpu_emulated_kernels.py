"""CPU: the library's scalar CUDA kernels, executed thread by thread under a small stand-in for the
CUDA execution model (tests/cpu_emu/cuda_shim.h), against the golden vectors and the oracle.

The device code of the quantize / dequantize families, of the warp-MMA small-batch forward and of the
tcgen05 kernels lives in headers without launch syntax (shrew_b200/csrc/*_kernels.cuh,
activation_f16.cuh; their PTX instructions sit behind ptx_small.cuh, ptx_tcgen05.cuh and
ptx_tcgen05_pair.cuh); g++ compiles them here as plain C++, with mma.sync, mbarriers, TMA, tensor memory
and tcgen05.mma modelled from their documented behaviour.  This is a check of kernel LOGIC (indexing, block and warp reductions, the
f32 shortcut and its f64 replay, special values); it says nothing about speed and is no substitute
for the GPU parity tests.  The kernels have run on B200s and pass the same golden vectors there, which is
what validates the stand-in itself."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from tests.conftest import GOLDEN, ROOT
from tests.test_oracle_modes import MODES

EMU_DIR = os.path.join(ROOT, "tests", "cpu_emu")
BUILD_DIR = os.path.join(EMU_DIR, "_build")
_vp, _sz, _ci, _cu = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_uint


def _build(name):
    os.makedirs(BUILD_DIR, exist_ok=True)
    src = os.path.join(EMU_DIR, name + ".cpp")
    out = os.path.join(BUILD_DIR, "lib" + name + ".so")
    deps = [src, os.path.join(EMU_DIR, "cuda_shim.h")] + [
        os.path.join(ROOT, "shrew_b200", "csrc", h) for h in os.listdir(os.path.join(ROOT, "shrew_b200", "csrc")) if h.endswith(".cuh")] + [
        os.path.join(EMU_DIR, h) for h in os.listdir(EMU_DIR) if h.endswith(".h")]
    if not os.path.exists(out) or any(os.path.getmtime(d) > os.path.getmtime(out) for d in deps):
        subprocess.run(["g++", "-std=c++20", "-O1", "-pthread", "-fPIC", "-shared", "-ffp-contract=off", "-fno-fast-math",
                        "-Wno-unknown-pragmas", "-o", out, src], check=True, cwd=EMU_DIR)
    return ctypes.CDLL(out)


@pytest.fixture(scope="module")
def emu():
    L = _build("emu_quantize")
    L.emu_quantize_rows.argtypes = [_vp, _sz, _sz, _ci, _vp, _vp]
    L.emu_quantize_tensor.argtypes = [_vp, _sz, _cu, _vp, _vp]
    L.emu_quantize_given_amax.argtypes = [_vp, _sz, _vp, _cu, _vp, _vp]
    L.emu_absmax.argtypes = [_vp, _sz, _cu, _vp]
    L.emu_dequantize.argtypes = [_vp, _vp, _sz, _sz, _ci, _ci, _ci, _cu, _vp]
    return L


@pytest.fixture(scope="module")
def emu_modes():
    L = _build("emu_quantize_modes")
    L.emu_quantize_ex.argtypes = [_vp, _sz, _sz, _ci, _ci, _ci, _cu, _vp, _vp, _vp]
    L.emu_dequantize_ex.argtypes = [_vp, _vp, _vp, _sz, _sz, _ci, _ci, _cu, _vp]
    L.emu_scale_zp_to_f32.argtypes = [_vp, _vp, _ci, _sz, _vp]
    L.emu_row_sums.argtypes = [_vp, _ci, _sz, _sz, _vp]
    L.emu_zero_point_fix.argtypes = [_vp, _vp, _vp, _sz, _sz, _sz, _ci, _ci, _cu, _vp]
    L.emu_x_to_f16.argtypes = [_vp, _sz, _ci, _vp, _vp]
    return L


def _p(a):
    return ctypes.c_void_p(a.ctypes.data)


def _aligned(shape, dtype, align=64):
    """numpy array whose data pointer is `align`-byte aligned (the launcher's vector paths check it)."""
    n = int(np.prod(shape)) if len(shape) else 1
    raw = np.empty(n * np.dtype(dtype).itemsize + align, dtype=np.uint8)
    off = (-raw.ctypes.data) % align
    return raw[off:off + n * np.dtype(dtype).itemsize].view(dtype).reshape(shape)


def _rows_cols(shape):
    if len(shape) == 0:
        return 1, 1
    return int(shape[0]), int(np.prod(shape[1:], dtype=np.int64))


def _quantize_rows(emu, w, variant):
    rows, cols = _rows_cols(w.shape)
    wa = _aligned(w.shape, np.float32)
    wa[...] = w
    q = _aligned(w.shape, np.int8)
    q[...] = 99
    s = np.full(rows, -1.0)
    rc = emu.emu_quantize_rows(_p(wa), rows, cols, variant, _p(q), _p(s))
    return rc, q, s


# ---- INT8 symmetric (GPU-validated kernels: this validates the stand-in) ----------------------------
@pytest.mark.parametrize("case", [c for c in GOLDEN if c["granularity"] == 1 and len(c["shape"]) >= 1],
                         ids=lambda c: c["name"])
def test_golden_per_channel_generic_kernel(emu, case):
    rc, q, s = _quantize_rows(emu, case["data"], 0)
    assert rc == 0
    np.testing.assert_array_equal(q, case["codes"])
    assert s.tobytes() == case["scales"].tobytes()


@pytest.mark.parametrize("case", [c for c in GOLDEN if c["granularity"] == 0 or len(c["shape"]) == 0], ids=lambda c: c["name"])
@pytest.mark.parametrize("grid", [1, 3])
def test_golden_per_tensor_chain(emu, case, grid):
    w = _aligned(case["data"].shape, np.float32)
    w[...] = case["data"]
    q = _aligned(w.shape, np.int8)
    s = np.full(1, -1.0)
    emu.emu_quantize_tensor(_p(w), w.size, grid, _p(q), _p(s))
    np.testing.assert_array_equal(q, case["codes"])
    assert s.tobytes() == case["scales"].tobytes()


class _EmuQuantItem(ctypes.Structure):
    _fields_ = [("w", ctypes.c_void_p), ("rows", ctypes.c_size_t), ("cols", ctypes.c_size_t), ("q", ctypes.c_void_p),
                ("scales", ctypes.c_void_p)]


def _quantize_batch(emu, tensors, per_channel, grid, misalign=False):
    emu.emu_quantize_batch.argtypes = [_vp, _sz, _ci, _cu]
    items = (_EmuQuantItem * len(tensors))()
    bufs = []
    for i, w in enumerate(tensors):
        rows, cols = _rows_cols(w.shape)
        pad = 1 if misalign and i % 2 else 0              # every other tensor off the 16-byte boundary: scalar path
        wa = _aligned((w.size + pad,), np.float32)[pad:]
        wa[...] = w.reshape(-1)
        q = _aligned((w.size + pad,), np.int8)[pad:]
        q[...] = 99
        s = np.full(rows if per_channel else 1, -1.0)
        items[i] = _EmuQuantItem(wa.ctypes.data, rows, cols, q.ctypes.data, s.ctypes.data)
        bufs.append((wa, q, s))
    assert emu.emu_quantize_batch(ctypes.cast(items, ctypes.c_void_p), len(tensors), int(per_channel), grid) == 0
    return [(q.reshape(w.shape), s) for (wa, q, s), w in zip(bufs, tensors)]


@pytest.mark.parametrize("per_channel", [1, 0], ids=["per_channel", "per_tensor"])
def test_batched_quantizer_on_the_golden_vectors(emu, per_channel):
    # every golden tensor of the granularity, all in one table
    cases = [c for c in GOLDEN if len(c["shape"]) >= 1 and c["granularity"] == per_channel]
    assert len(cases) >= 5
    for grid in (1, 7):
        got = _quantize_batch(emu, [c["data"] for c in cases], per_channel, grid)
        for c, (q, s) in zip(cases, got):
            np.testing.assert_array_equal(q, c["codes"], err_msg=c["name"])
            assert s.tobytes() == c["scales"].tobytes(), c["name"]


@pytest.mark.parametrize("per_channel", [1, 0], ids=["per_channel", "per_tensor"])
def test_batched_quantizer_matches_oracle_on_a_model(oracle, emu, per_channel):
    # a small GPT's parameter list (scaled down), empty and ragged tensors, special values, more tensors
    # than one table holds (64), odd alignments
    rng = np.random.default_rng(3)
    shapes = [(64, 64)] * 4 + [(256, 64), (64, 256), (1, 64), (0, 5), (3, 0), (1, 1), (5, 3), (2, 4100), (50, 33)]
    tensors = [_special_matrix(r, c, i) if r * c else np.zeros((r, c), np.float32) for i, (r, c) in enumerate(shapes)]
    tensors += [(rng.standard_normal((3, 20)) * 10.0 ** rng.integers(-38, 38)).astype(np.float32) for _ in range(70)]
    for misalign in (False, True):
        got = _quantize_batch(emu, tensors, per_channel, 5, misalign=misalign)
        for i, (w, (q, s)) in enumerate(zip(tensors, got)):
            rq, rs = oracle.quantize_f32(w, oracle.PER_CHANNEL if per_channel else oracle.PER_TENSOR)
            np.testing.assert_array_equal(q, rq, err_msg=f"tensor {i} shape {w.shape}")
            assert s.tobytes() == rs.tobytes(), f"tensor {i} shape {w.shape}"


def _special_matrix(rows, cols, seed, scale=1.0):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((rows, cols)) * scale).astype(np.float32)
    flat = w.reshape(-1)
    if flat.size > 8:
        flat[rng.integers(0, flat.size, 4)] = [np.nan, np.inf, -0.0, 0.0][: 4]
        flat[1] = flat[0] * 0.5           # an exact .5 product when flat[0] is the row's amax? not guaranteed; ties are in the goldens
    return w


@pytest.mark.parametrize("variant,rows,cols", [
    (1, 9, 32), (1, 20, 128), (2, 11, 200), (3, 9, 512), (4, 17, 1000), (5, 3, 1028), (5, 2, 2048), (6, 2, 4096),
    (7, 2, 6000), (8, 2, 16384), (8, 1, 9000), (9, 1, 20000), (0, 7, 33), (0, 3, 5000), (0, 12, 1)])
def test_register_tile_kernels_match_oracle(oracle, emu, variant, rows, cols):
    for seed, scale in ((0, 1.0), (1, 1e-35), (2, 3e37)):
        w = _special_matrix(rows, cols, seed + variant, scale)
        if seed == 0:
            w[rows - 1] = 0.0                      # an all-zero row: amax < 1e-30 -> scale 1.0
        rc, q, s = _quantize_rows(emu, w, variant)
        assert rc == 0
        q_ref, s_ref = oracle.np_quantize_f32(w, oracle.PER_CHANNEL)
        np.testing.assert_array_equal(q, q_ref)
        assert s.tobytes() == s_ref.tobytes()


def test_variant_rejects_what_the_launcher_would_not_choose(emu):
    assert _quantize_rows(emu, np.zeros((2, 130), np.float32), 1)[0] == -1    # cols not a multiple of 4
    assert _quantize_rows(emu, np.zeros((2, 256), np.float32), 1)[0] == -1    # too wide for 32 x 1 float4


@pytest.mark.parametrize("n,grid", [(1, 1), (1023, 2), (4096 + 3, 3), (100000, 4)])
def test_per_tensor_chain_and_shard_entry_points(oracle, emu, n, grid):
    w = _special_matrix(1, n, n).reshape(-1)
    wa = _aligned((n,), np.float32)
    wa[...] = w
    q = _aligned((n,), np.int8)
    s = np.zeros(1)
    emu.emu_quantize_tensor(_p(wa), n, grid, _p(q), _p(s))
    q_ref, s_ref = oracle.np_quantize_f32(w, oracle.PER_TENSOR)
    np.testing.assert_array_equal(q, q_ref)
    assert s.tobytes() == s_ref.tobytes()
    # two shards, each with the global amax
    cut = n // 3
    am = np.zeros(2, np.float32)
    for i, part in enumerate((wa[:cut], wa[cut:])):
        pa = _aligned(part.shape, np.float32)
        pa[...] = part
        emu.emu_absmax(_p(pa), pa.size, grid, ctypes.c_void_p(am.ctypes.data + 4 * i))
    g = np.array([max(am)], np.float32)
    assert float(g[0]) == float(np.fmax.reduce(np.abs(w), initial=0.0))
    off = 0
    for part in (wa[:cut], wa[cut:]):
        pa = _aligned(part.shape, np.float32)
        pa[...] = part
        qs, ss = _aligned(part.shape, np.int8), np.zeros(1)
        emu.emu_quantize_given_amax(_p(pa), pa.size, _p(g), grid, _p(qs), _p(ss))
        np.testing.assert_array_equal(qs, q_ref[off:off + part.size])
        assert ss.tobytes() == s_ref.tobytes()
        off += part.size


@pytest.mark.parametrize("rows,cols,gran", [(5, 64, 1), (7, 33, 1), (3, 100, 0), (1, 4, 0)])
@pytest.mark.parametrize("bf16", [0, 1])
def test_dequantize_kernels_match_oracle(oracle, emu, rows, cols, gran, bf16):
    rng = np.random.default_rng(rows * cols)
    q = _aligned((rows, cols), np.int8)
    q[...] = rng.integers(-127, 128, size=(rows, cols))
    s = (rng.random(rows if gran else 1) * 10.0 ** rng.integers(-30, 30)).astype(np.float64)
    ref = oracle.dequantize(q, s, gran, "bf16" if bf16 else "f32")
    for vec in ((1, 0) if cols % 4 == 0 else (0,)):
        out = _aligned((rows, cols), np.uint16 if bf16 else np.float32)
        assert emu.emu_dequantize(_p(q), _p(s), rows, cols, gran, bf16, vec, 2, _p(out)) == 0
        np.testing.assert_array_equal(out, ref)


# ---- the other modes: first execution of these kernels ---------------------------------------------------
@pytest.mark.parametrize("case", MODES, ids=lambda c: c["name"])
def test_modes_golden(emu_modes, case):
    w = _aligned(case["data"].shape, np.float32)
    w[...] = case["data"]
    rows, cols = _rows_cols(w.shape)
    gran = case["granularity"] if len(w.shape) else 0
    n = rows if gran else 1
    q = _aligned(w.shape, np.int8)
    s, z = np.full(n, -1.0), np.full(n, -1.0)
    emu_modes.emu_quantize_ex(_p(w), rows, cols, gran, case["bits"], case["mode"], 3, _p(q), _p(s), _p(z))
    np.testing.assert_array_equal(q, case["codes"])
    assert s.tobytes() == case["scales"].tobytes()
    assert z.tobytes() == case["zps"].tobytes()


@pytest.mark.parametrize("bits,mode", [(8, 1), (4, 0), (4, 1), (8, 0)])
@pytest.mark.parametrize("rows,cols,gran", [(9, 300, 1), (4, 1000, 1), (3, 777, 0), (1, 5000, 0), (600, 3, 1)])
def test_modes_match_oracle_and_round_trip(oracle, emu_modes, bits, mode, rows, cols, gran):
    for seed, scale, shift in ((0, 1.0, 0.3), (1, 1e-33, 0.0), (2, 1e36, -2.0)):
        w = _special_matrix(rows, cols, seed + bits + mode, 1.0)
        w = ((w + shift) * scale).astype(np.float32)
        wa = _aligned(w.shape, np.float32)
        wa[...] = w
        n = rows if gran else 1
        q = _aligned(w.shape, np.int8)
        s, z = np.zeros(n), np.zeros(n)
        emu_modes.emu_quantize_ex(_p(wa), rows, cols, gran, bits, mode, 4, _p(q), _p(s), _p(z))
        q_ref, s_ref, z_ref = oracle.np_quantize_f32_ex(w, gran, bits, mode)
        np.testing.assert_array_equal(q, q_ref)
        assert s.tobytes() == s_ref.tobytes() and z.tobytes() == z_ref.tobytes()
        with np.errstate(all="ignore"):
            ref64 = oracle.dequantize_f64_ex(q_ref, s_ref, z_ref, gran)
            out = _aligned(w.shape, np.float32)
            emu_modes.emu_dequantize_ex(_p(q), _p(s), _p(z), rows, cols, gran, 0, 3, _p(out))
            np.testing.assert_array_equal(out, ref64.astype(np.float32))
            out16 = _aligned(w.shape, np.uint16)
            emu_modes.emu_dequantize_ex(_p(q), _p(s), _p(z), rows, cols, gran, 1, 3, _p(out16))
            want16 = np.array([oracle.f64_to_bf16_bits(v) for v in ref64.reshape(-1)[:200]], dtype=np.uint16)
            np.testing.assert_array_equal(out16.reshape(-1)[:200], want16)


def test_zero_point_forward_pieces(emu_modes):
    rng = np.random.default_rng(5)
    M, N, K = 5, 37, 300
    x = rng.standard_normal((M, K)).astype(np.float32)
    sums = np.zeros(M, np.float32)
    emu_modes.emu_row_sums(_p(x), 0, M, K, _p(sums))
    np.testing.assert_array_equal(sums, x.astype(np.float64).sum(axis=1).astype(np.float32))
    xb = (x.view(np.uint32) >> 16).astype(np.uint16)          # truncated bf16 copies of x
    emu_modes.emu_row_sums(_p(xb), 1, M, K, _p(sums))
    xb_f = (xb.astype(np.uint32) << 16).view(np.float32)
    np.testing.assert_allclose(sums, xb_f.astype(np.float64).sum(axis=1), rtol=1e-6)
    scales, zps = rng.random(N) * 1e-2, np.round(rng.standard_normal(N) * 50)
    czp = np.zeros(N, np.float32)
    emu_modes.emu_scale_zp_to_f32(_p(scales), _p(zps), 1, N, _p(czp))
    np.testing.assert_array_equal(czp, (scales * zps).astype(np.float32))
    emu_modes.emu_scale_zp_to_f32(_p(scales), _p(zps), 0, N, _p(czp))
    np.testing.assert_array_equal(czp, np.full(N, np.float32(scales[0] * zps[0])))
    acc = rng.standard_normal((M, N)).astype(np.float32)
    ldy = N + 3
    for relu in (0, 1):
        y = np.full((M, ldy), 7.0, np.float32)
        emu_modes.emu_zero_point_fix(_p(acc), _p(czp), _p(sums), M, N, ldy, relu, 0, 2, _p(y))
        want = acc - czp[None, :] * sums[:, None]
        if relu:
            want = np.maximum(want, 0.0)
        np.testing.assert_array_equal(y[:, :N], want.astype(np.float32))
        assert np.all(y[:, N:] == 7.0)                          # the row stride's padding is untouched


@pytest.mark.parametrize("scale", [1e-37, 1e-12, 1.0, 6e4, 1e20, 3e38])
def test_activation_rescale_kernel_matches_its_model(emu_modes, scale):
    from tests.test_mma_f16_numerics import rescale_row, to_bf16
    rng = np.random.default_rng(9)
    M, K = 4, 1088
    x = to_bf16((rng.standard_normal((M, K)) * scale / 4).astype(np.float32))
    x[1] *= np.float32(1e-6)
    x[2] = 0.0
    x[3, 5] = np.nan
    x = to_bf16(np.where(np.isinf(x), np.float32(1e38), x))
    bits = (x.view(np.uint32) >> 16).astype(np.uint16)
    x16 = np.zeros((M, K), np.uint16)
    shift = np.zeros(M, np.int32)
    emu_modes.emu_x_to_f16(_p(bits), M, K, _p(x16), _p(shift))
    for m in range(M):
        ref16, s, _ = rescale_row(x[m])
        assert int(shift[m]) == s
        got = x16[m].view(np.float16)
        np.testing.assert_array_equal(np.isnan(got), np.isnan(ref16))
        ok = ~np.isnan(ref16)
        np.testing.assert_array_equal(got[ok], ref16[ok])


# ---- the warp-MMA small-batch forward (never run on a GPU): whole kernels, mma.sync emulated --------
@pytest.fixture(scope="module")
def emu_mma():
    L = _build("emu_gemv_mma")
    L.emu_gemv_mma.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _sz, _ci, _ci, _ci, _vp]
    return L


def _bf16_bits(x32):
    """f32 -> (bf16 bits, the bf16 values as f32), round to nearest even"""
    b = np.ascontiguousarray(x32, dtype=np.float32).view(np.uint32).astype(np.uint64)
    b = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)
    return b, (b.astype(np.uint32) << 16).view(np.float32)


def _gated_ref(oracle, qg, sg, bg, qu, su, bu, x):
    g = oracle.np_linear_forward(qg, sg, 1, bg, x).astype(np.float64)
    u = oracle.np_linear_forward(qu, su, 1, bu, x).astype(np.float64)
    with np.errstate(over="ignore"):
        return (g / (1.0 + np.exp(-g)) * u).astype(np.float32)


def _mma_forward(emu_mma, q, scales, bias, x_bits, f16, y_bf16, relu=False, up=None, ldy=None):
    N, K = q.shape
    M = x_bits.shape[0]
    ldy = ldy or N
    qa = _aligned(q.shape, np.int8)
    qa[...] = q
    xa = _aligned(x_bits.shape, np.uint16)
    xa[...] = x_bits
    y = np.full((M, ldy), 7.0, np.float32) if not y_bf16 else np.full((M, ldy), 0x4100, np.uint16)
    s32 = scales.astype(np.float32)
    staged = ctypes.c_int(-1)
    if up is None:
        args = (_p(qa), _p(s32), None if bias is None else _p(bias), None, None, None)
    else:
        qu = _aligned(q.shape, np.int8)
        qu[...] = up[0]
        su = up[1].astype(np.float32)
        args = (_p(qa), _p(s32), None if bias is None else _p(bias), _p(qu), _p(su), None if up[2] is None else _p(up[2]))
    rc = emu_mma.emu_gemv_mma(*args, _p(xa), _p(y), M, N, K, ldy, 1 if relu else 0, int(f16), int(y_bf16), ctypes.byref(staged))
    assert rc == 0
    return y, staged.value


@pytest.mark.parametrize("seed", range(30))
def test_warp_mma_random_configurations(oracle, emu_mma, seed):
    # seeded sweep: batch 1..64 (staged in the CTA up to 4, else the separate conversion kernel), ragged N,
    # K a multiple of 64, bf16 or f16 operands, plain or gate/up, either output type, activations of any scale
    rng = np.random.default_rng(3000 + seed)
    M = int(rng.choice([1, 2, 3, 4, 5, 8, 15, 16, 17, 31, 32, 33, 48, 64]))
    N = int(rng.integers(1, 70))
    K = 64 * int(rng.integers(1, 40 if M <= 4 else 12))
    f16 = int(rng.integers(0, 2))
    gated = bool(rng.integers(0, 2))
    y_bf16 = bool(rng.integers(0, 2))
    relu = (not gated) and bool(rng.integers(0, 2))
    q, scales, bias, x_bits, x = _tc_case(M, N, K, seed)
    xs = (x * np.float32(2.0) ** rng.integers(-30, 30, size=(M, 1))).astype(np.float32)   # per-row scales: the f16 rescale
    x_bits, x = _bf16_bits(xs)
    up = None
    if gated:
        qu = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
        su = rng.random(N) * 1e-2 + 1e-4
        bu = (rng.standard_normal(N) * 0.1).astype(np.float32)
        up = (qu, su, bu)
        ref = _gated_ref(oracle, q, scales, bias, qu, su, bu, x)
    else:
        ref = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, x, relu=relu)
    y, staged = _mma_forward(emu_mma, q, scales, bias, x_bits, f16, y_bf16, relu=relu, up=up)
    assert staged == int(bool(f16) and M <= 4 and M * K * 2 <= 36864)
    if y_bf16:
        y = (y.astype(np.uint32) << 16).view(np.float32)
    with np.errstate(invalid="ignore"):
        ok = np.isfinite(ref)
    assert np.array_equal(np.isfinite(y), ok)
    what = dict(M=M, N=N, K=K, f16=f16, gated=gated, y_bf16=y_bf16, relu=relu)
    assert oracle.rel_err(np.where(ok, y, 0), np.where(ok, ref, 0)) < (1e-2 if y_bf16 else 1e-5), what


@pytest.mark.parametrize("f16", [0, 1], ids=["bf16", "f16"])
@pytest.mark.parametrize("M,N,K", [(1, 16, 64), (1, 40, 512), (3, 21, 128), (4, 16, 4608), (4, 16, 4672), (5, 16, 64), (16, 32, 192),
                                   (17, 24, 128), (33, 16, 128), (64, 17, 64)])
def test_warp_mma_forward_matches_oracle(oracle, emu_mma, f16, M, N, K):
    rng = np.random.default_rng(M * 1000 + N + K)
    q = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
    scales = rng.random(N) * 1e-2 + 1e-4
    bias = (rng.standard_normal(N) * 0.1).astype(np.float32)
    x_bits, x = _bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    ref = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, x, relu=True)
    y, staged = _mma_forward(emu_mma, q, scales, bias, x_bits, f16, y_bf16=False, relu=True, ldy=N + 5)
    assert staged == int(bool(f16) and M <= 4 and M * K * 2 <= 36864)
    assert oracle.rel_err(y[:, :N], ref) < 2e-6        # exact products, f32-level accumulation
    assert np.all(y[:, N:] == 7.0)                     # nothing written outside [M, N]
    y16, _ = _mma_forward(emu_mma, q, scales, None, x_bits, f16, y_bf16=True)
    ref_nb = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, None, x)
    got = (y16.astype(np.uint32) << 16).view(np.float32)
    assert oracle.rel_err(got, ref_nb) < 1e-2          # the bf16 output rounding


@pytest.mark.parametrize("f16", [0, 1], ids=["bf16", "f16"])
@pytest.mark.parametrize("M,N,K", [(2, 24, 128), (12, 9, 192)])
def test_warp_mma_gate_up_matches_oracle(oracle, emu_mma, f16, M, N, K):
    rng = np.random.default_rng(N + K)
    qg, qu = (rng.integers(-127, 128, size=(N, K)).astype(np.int8) for _ in range(2))
    sg, su = rng.random(N) * 1e-2 + 1e-4, rng.random(N) * 1e-2 + 1e-4
    bg = (rng.standard_normal(N) * 0.1).astype(np.float32)
    x_bits, x = _bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    g = oracle.np_linear_forward(qg, sg, 1, bg, x).astype(np.float64)
    u = oracle.np_linear_forward(qu, su, 1, None, x).astype(np.float64)
    ref = (g / (1.0 + np.exp(-g)) * u).astype(np.float32)
    y, _ = _mma_forward(emu_mma, qg, sg, bg, x_bits, f16, y_bf16=False, up=(qu, su, None))
    assert oracle.rel_err(y, ref) < 1e-5


@pytest.mark.parametrize("rows", [3, 7], ids=["staged_in_kernel", "staging_kernel"])
def test_warp_mma_f16_activation_range(oracle, emu_mma, rows):
    # rows of very different magnitude, far outside f16's range, each rescaled by its own power of two
    rng = np.random.default_rng(2)
    N, K = 16, 256
    q = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
    scales = rng.random(N) * 1e-3 + 1e-5
    x = rng.standard_normal((7, K)).astype(np.float32)
    x *= np.array([1e-25, 1e30, 0.0, 3e4, 1e-12, 1.0, 1e20], np.float32)[:, None]
    x_bits, xb = _bf16_bits(x[:rows])
    y, staged = _mma_forward(emu_mma, q, scales, None, x_bits, 1, y_bf16=False)
    assert staged == int(rows <= 4)
    ref = oracle.np_linear_forward(q, scales, 1, None, xb)
    for m in range(rows):
        assert oracle.rel_err(y[m:m + 1], ref[m:m + 1]) < 2e-6, m


def test_warp_mma_refuses_unsupported_shapes(emu_mma):
    q = _aligned((16, 96), np.int8)
    x = _aligned((2, 96), np.uint16)
    y = np.zeros((2, 16), np.float32)
    s = np.ones(16, np.float32)
    st = ctypes.c_int(0)
    assert emu_mma.emu_gemv_mma(_p(q), _p(s), None, None, None, None, _p(x), _p(y), 2, 16, 96, 16, 0, 0, 0, ctypes.byref(st)) == -1


# ---- the tcgen05 forward kernel: mbarriers, TMA, tensor memory and tcgen05.mma modelled ---------------
# (tests/cpu_emu/cuda_shim_tcgen05.h).  This kernel has passed its parity tests on B200s; that it
# also produces the oracle's results on top of the model is what ties the model to the hardware.
@pytest.fixture(scope="module")
def emu_tc():
    L = _build("emu_gemm_tcgen05")
    L.emu_gemm_tcgen05.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _sz, _ci, _ci, _ci, _ci, _ci, _ci]
    return L


def _tc_forward(emu_tc, q, scales, bias, x_bits, tok, groups, splits=1, y_bf16=False, epilogue=0, up=None, ldy=None,
                tile_list=0, y_init=None):
    N, K = q.shape
    M = x_bits.shape[0]
    ldy = ldy or N
    qa = _aligned(q.shape, np.int8)
    qa[...] = q
    xa = _aligned(x_bits.shape, np.uint16)
    xa[...] = x_bits
    if y_init is not None:
        y = y_init.copy()
    else:
        y = np.full((M, ldy), 0x4100, np.uint16) if y_bf16 else np.full((M, ldy), 7.0, np.float32)
    s32 = scales.astype(np.float32)
    if up is None:
        args = (_p(qa), _p(s32), None if bias is None else _p(bias), None, None, None)
    else:
        qu = _aligned(q.shape, np.int8)
        qu[...] = up[0]
        su = up[1].astype(np.float32)
        args = (_p(qa), _p(s32), None if bias is None else _p(bias), _p(qu), _p(su), None if up[2] is None else _p(up[2]))
    rc = emu_tc.emu_gemm_tcgen05(*args, _p(xa), _p(y), M, N, K, ldy, epilogue, int(y_bf16), tok, groups, splits, tile_list)
    if rc == -4:
        emu_tc.emu_fail_message.restype = ctypes.c_char_p
        raise AssertionError("the model's rules were violated: " + emu_tc.emu_fail_message().decode())
    assert rc == 0, f"emulated kernel returned {rc} (-2: a bounded wait gave up, -3: a tile counter was left set)"
    return y


def _tc_case(M, N, K, seed):
    rng = np.random.default_rng(seed)
    q = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
    scales = rng.random(N) * 1e-2 + 1e-4
    bias = (rng.standard_normal(N) * 0.1).astype(np.float32)
    x_bits, x = _bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    return q, scales, bias, x_bits, x


# every (token tile, converter groups) pair the launcher can choose: 7 pipeline stages at 16 and 32
# tokens, 6 at 64, 4 at 128, 5 at 256; converter groups own stages (stage s -> group s % G)
@pytest.mark.parametrize("groups", [1, 2, 3])
@pytest.mark.parametrize("tok,M,N,K", [(16, 5, 130, 1088), (32, 30, 128, 960), (64, 64, 200, 1024), (128, 100, 129, 1280),
                                       (256, 300, 140, 704)])
def test_tcgen05_forward_matches_oracle(oracle, emu_tc, tok, groups, M, N, K):
    q, scales, bias, x_bits, x = _tc_case(M, N, K, tok + groups)
    ref = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, x, relu=True)
    y = _tc_forward(emu_tc, q, scales, bias, x_bits, tok, groups, epilogue=1, ldy=N + 3)
    assert oracle.rel_err(y[:, :N], ref) < 2e-6
    assert np.all(y[:, N:] == 7.0)


@pytest.mark.parametrize("tok,M,N,K,splits", [(16, 3, 128, 1024, 4), (64, 40, 130, 768, 3), (32, 20, 64, 1100 // 4 * 4, 2),
                                              (128, 100, 200, 2048, 3),      # large-tile split-K
                                              (256, 260, 128, 1024, 2)])     # large-tile split-K
def test_tcgen05_split_k(oracle, emu_tc, tok, M, N, K, splits):
    K = K // 16 * 16
    q, scales, bias, x_bits, x = _tc_case(M, N, K, splits)
    ref = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, x)
    y = _tc_forward(emu_tc, q, scales, bias, x_bits, tok, 3, splits=splits)
    assert oracle.rel_err(y, ref) < 2e-6
    y2 = _tc_forward(emu_tc, q, scales, bias, x_bits, tok, 3, splits=splits)
    np.testing.assert_array_equal(y, y2)               # slices are summed in split order: same bits every run


@pytest.mark.parametrize("tok,M,N,K,splits", [(16, 8, 100, 512, 1), (64, 50, 64, 640, 2), (128, 128, 130, 256, 1), (256, 257, 70, 320, 1)])
def test_tcgen05_gate_up_tile(oracle, emu_tc, tok, M, N, K, splits):
    rng = np.random.default_rng(tok)
    qg, qu = (rng.integers(-127, 128, size=(N, K)).astype(np.int8) for _ in range(2))
    sg, su = rng.random(N) * 1e-2 + 1e-4, rng.random(N) * 1e-2 + 1e-4
    bg, bu = ((rng.standard_normal(N) * 0.1).astype(np.float32) for _ in range(2))
    x_bits, x = _bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    g = oracle.np_linear_forward(qg, sg, 1, bg, x).astype(np.float64)
    u = oracle.np_linear_forward(qu, su, 1, bu, x).astype(np.float64)
    ref = (g / (1.0 + np.exp(-g)) * u).astype(np.float32)
    y = _tc_forward(emu_tc, qg, sg, bg, x_bits, tok, 3, splits=splits, up=(qu, su, bu))
    assert oracle.rel_err(y, ref) < 1e-5


def test_tcgen05_bf16_output(oracle, emu_tc):
    q, scales, bias, x_bits, x = _tc_case(70, 130, 384, 11)
    ref = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, x)
    y16 = _tc_forward(emu_tc, q, scales, bias, x_bits, 128, 3, y_bf16=True)
    assert oracle.rel_err((y16.astype(np.uint32) << 16).view(np.float32), ref) < 1e-2


@pytest.mark.parametrize("M,N,K,ldy,y_bf16", [(70, 130, 384, 130, True), (33, 129, 128, 133, False), (40, 64, 192, 72, True),
                                              (20, 200, 64, 203, True)])
def test_tcgen05_rows_that_do_not_start_on_16_bytes(oracle, emu_tc, M, N, K, ldy, y_bf16):
    # the epilogue's wide stores need 16-byte aligned rows; an odd row stride (or a ragged last channel
    # segment) takes the element-wise stores out of the same staging tile, and nothing outside [M, N] is touched
    q, scales, bias, x_bits, x = _tc_case(M, N, K, ldy)
    ref = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, x)
    y = _tc_forward(emu_tc, q, scales, bias, x_bits, 64 if M <= 64 else 128, 3, y_bf16=y_bf16, ldy=ldy)
    got = (y.astype(np.uint32) << 16).view(np.float32) if y_bf16 else y
    assert oracle.rel_err(got[:, :N], ref) < (1e-2 if y_bf16 else 2e-6)
    fill = 0x4100 if y_bf16 else np.float32(7.0)
    assert np.all(y[:, N:] == fill)


@pytest.mark.parametrize("seed", range(36))
def test_tcgen05_random_configurations(oracle, emu_tc, seed):
    # a seeded sweep over what the launcher can combine: token tile, converter groups, K splits, plain or
    # gate/up tile, output type, elementwise op, grid or tile list,
    # ragged M / N / K (K a multiple of 16 only)
    rng = np.random.default_rng(1000 + seed)
    tok = int(rng.choice([16, 32, 64, 128, 256]))
    M = int(rng.integers(1, tok + tok // 2 + 2))
    N = int(rng.integers(1, 280))
    K = 16 * int(rng.integers(1, 72))
    groups = int(rng.integers(1, 4))
    gated = bool(rng.integers(0, 2))
    y_bf16 = bool(rng.integers(0, 2))
    relu = (not gated) and bool(rng.integers(0, 2))
    kblk = 64 if tok == 256 else 128
    rounds = -(-K // kblk)
    splits = int(rng.integers(1, min(4, rounds) + 1))
    tile_list = int(rng.integers(0, 2))
    q, scales, bias, x_bits, x = _tc_case(M, N, K, seed)
    up = None
    if gated:
        qu = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
        su = rng.random(N) * 1e-2 + 1e-4
        bu = (rng.standard_normal(N) * 0.1).astype(np.float32)
        up = (qu, su, bu)
        ref = _gated_ref(oracle, q, scales, bias, qu, su, bu, x)
    else:
        ref = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, x, relu=relu)
    what = dict(tok=tok, M=M, N=N, K=K, groups=groups, gated=gated, y_bf16=y_bf16, relu=relu, splits=splits,
                tile_list=tile_list)
    emu_tc.emu_tma_async.argtypes = [_cu, _cu]
    if seed % 3 == 0:                                  # loads land late and newest first
        emu_tc.emu_tma_async(seed + 1, int(rng.choice([8, 200, 1500])))
        what["late_loads"] = True
    try:
        y = _tc_forward(emu_tc, q, scales, bias, x_bits, tok, groups, splits=splits, y_bf16=y_bf16, epilogue=int(relu), up=up,
                        tile_list=tile_list)
    finally:
        emu_tc.emu_tma_async(0, 0)
    if y_bf16:
        y = (y.astype(np.uint32) << 16).view(np.float32)
    assert oracle.rel_err(y, ref) < (1e-2 if y_bf16 else 1e-5), what


def test_tcgen05_tile_list_grid(oracle, emu_tc):
    # the 1-D tile list of the two-launch tail-split scheme
    q, scales, bias, x_bits, x = _tc_case(300, 260, 512, 5)
    ref = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, x)
    for splits in (1, 2):
        y = _tc_forward(emu_tc, q, scales, bias, x_bits, 128, 3, splits=splits, tile_list=1)
        assert oracle.rel_err(y, ref) < 2e-6


@pytest.mark.parametrize("M,N,K,splits,y_bf16,tok", [(90, 140, 784 // 16 * 16, 1, False, 128), (200, 129, 256, 1, False, 128),
                                                      (130, 64, 1024, 2, False, 128), (17, 300, 128, 1, True, 128),
                                                      (300, 129, 256, 1, False, 256), (260, 70, 512, 2, True, 256)])
def test_f32_activations_as_hi_lo_pair_on_the_tensor_cores(oracle, emu, emu_tc, M, N, K, splits, y_bf16, tok):
    # forward_f32_on_tensor_cores: x = hi + lo in bf16, both token tiles in one stage, two MMAs per k-step
    # into the same accumulator; the lo rows sit under the M hi rows of one array
    emu.emu_split_f32.argtypes = [_vp, _sz, _cu, _vp, _vp]
    emu_tc.emu_gemm_tcgen05_xsplit.argtypes = [_vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _sz, _ci, _ci, _ci, _ci]
    rng = np.random.default_rng(3 + M)
    q = _aligned((N, K), np.int8)
    q[...] = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
    scales = rng.random(N) * 1e-2 + 1e-4
    bias = (rng.standard_normal(N) * 0.1).astype(np.float32)
    x = rng.random((M, K)).astype(np.float32)                 # U(0,1) like the MLP config's inputs
    pair = _aligned((2 * M, K), np.uint16)
    hi, lo = np.zeros((M, K), np.uint16), np.zeros((M, K), np.uint16)
    emu.emu_split_f32(_p(x), x.size, 3, _p(hi), _p(lo))
    pair[:M], pair[M:] = hi, lo
    hi_f, lo_f = (hi.astype(np.uint32) << 16).view(np.float32), (lo.astype(np.uint32) << 16).view(np.float32)
    assert np.max(np.abs((hi_f.astype(np.float64) + lo_f) - x)) <= 2.0 ** -16 * np.max(np.abs(x))
    s32 = scales.astype(np.float32)
    y = np.full((M, N), 0x4100, np.uint16) if y_bf16 else np.full((M, N), 7.0, np.float32)
    rc = emu_tc.emu_gemm_tcgen05_xsplit(_p(q), _p(s32), _p(bias), _p(pair), _p(y), M, N, K, N, 1, int(y_bf16), splits, tok)
    assert rc == 0
    ref = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, x, relu=True)
    got = (y.astype(np.uint32) << 16).view(np.float32) if y_bf16 else y
    assert oracle.rel_err(got, ref) < (1e-2 if y_bf16 else 1e-4)   # the f32 path's tolerance


# ---- the CTA-pair kernel (cta_group::2): two blocks of a cluster run concurrently over modelled cluster
# shared memory.  The cta_group::2 parts of the model (tests/cpu_emu/cuda_shim_tcgen05_pair.h) state how the
# documentation is read here; the kernel's GPU parity tests have since confirmed that reading.
@pytest.fixture(scope="module")
def emu_pair():
    L = _build("emu_gemm_tcgen05_pair")
    L.emu_gemm_tcgen05_pair.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _sz, _ci, _ci, _ci, _ci]
    return L


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (300, 300, 320), (100, 130, 128), (513, 512, 1088), (1, 256, 1024), (260, 1000, 64)])
def test_cta_pair_forward_matches_oracle(oracle, emu_pair, M, N, K):
    q, scales, bias, x_bits, x = _tc_case(M, N, K, M + N)
    qa = _aligned(q.shape, np.int8)
    qa[...] = q
    xa = _aligned(x_bits.shape, np.uint16)
    xa[...] = x_bits
    s32 = scales.astype(np.float32)
    ref = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, x, relu=True)
    ldy = N + 2
    y = np.full((M, ldy), 7.0, np.float32)
    assert emu_pair.emu_gemm_tcgen05_pair(_p(qa), _p(s32), _p(bias), None, None, None, _p(xa), _p(y), M, N, K, ldy, 1, 0, 1, 0) == 0
    assert oracle.rel_err(y[:, :N], ref) < 2e-6
    assert np.all(y[:, N:] == 7.0)
    y16 = np.full((M, N), 0x4100, np.uint16)
    assert emu_pair.emu_gemm_tcgen05_pair(_p(qa), _p(s32), None, None, None, None, _p(xa), _p(y16), M, N, K, N, 0, 1, 1, 0) == 0
    ref_nb = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, None, x)
    assert oracle.rel_err((y16.astype(np.uint32) << 16).view(np.float32), ref_nb) < 1e-2


@pytest.mark.parametrize("seed", range(15))
def test_cta_pair_random_configurations(oracle, emu_pair, seed):
    rng = np.random.default_rng(2000 + seed)
    M = int(rng.integers(1, 560))
    N = int(rng.integers(1, 560))
    K = 16 * int(rng.integers(1, 60))
    gated = bool(rng.integers(0, 2))
    y_bf16 = bool(rng.integers(0, 2))
    relu = (not gated) and bool(rng.integers(0, 2))
    rounds = -(-K // 128)
    splits = int(rng.integers(1, min(3, rounds) + 1))
    tile_list = int(rng.integers(0, 2))
    q, scales, bias, x_bits, x = _tc_case(M, N, K, seed)
    qa, xa = _aligned(q.shape, np.int8), _aligned(x_bits.shape, np.uint16)
    qa[...] = q
    xa[...] = x_bits
    s32 = scales.astype(np.float32)
    up = (None, None, None)
    if gated:
        qu = _aligned(q.shape, np.int8)
        qu[...] = rng.integers(-127, 128, size=q.shape).astype(np.int8)
        su = rng.random(N) * 1e-2 + 1e-4
        bu = (rng.standard_normal(N) * 0.1).astype(np.float32)
        su32 = su.astype(np.float32)
        up = (_p(qu), _p(su32), _p(bu))
        ref = _gated_ref(oracle, q, scales, bias, qu, su, bu, x)
    else:
        ref = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, x, relu=relu)
    what = dict(M=M, N=N, K=K, gated=gated, y_bf16=y_bf16, relu=relu, splits=splits, tile_list=tile_list)
    y = np.full((M, N), 0x4100, np.uint16) if y_bf16 else np.full((M, N), 7.0, np.float32)
    emu_pair.emu_tma_async.argtypes = [_cu, _cu]
    if seed % 3 == 0:                                  # loads land late and newest first
        emu_pair.emu_tma_async(seed + 1, int(rng.choice([8, 200, 1500])))
        what["late_loads"] = True
    try:
        rc = emu_pair.emu_gemm_tcgen05_pair(_p(qa), _p(s32), _p(bias), *up, _p(xa), _p(y), M, N, K, N, int(relu), int(y_bf16), splits,
                                            tile_list)
    finally:
        emu_pair.emu_tma_async(0, 0)
    if rc == -4:
        emu_pair.emu_fail_message.restype = ctypes.c_char_p
        raise AssertionError(emu_pair.emu_fail_message().decode() + f" {what}")
    assert rc == 0, what
    if y_bf16:
        y = (y.astype(np.uint32) << 16).view(np.float32)
    assert oracle.rel_err(y, ref) < (1e-2 if y_bf16 else 1e-5), what


@pytest.mark.parametrize("gated", [False, True])
def test_cta_pair_tile_list_and_tail_split(oracle, emu_pair, gated):
    # the tail split (option tc_tailsplit) on the pair kernel: the 1-D list of pair tiles as one launch,
    # then the two-launch scheme with 4 (5) pair tiles "resident at once": 4 (5) whole-K tiles in the first
    # launch, the remaining 2 (1) split 2 (3) ways along K in the second
    M, N, K = 300, (300 if gated else 600), 2048           # 3 channel pairs x 2 token tiles = 6 pair tiles
    q, scales, bias, x_bits, x = _tc_case(M, N, K, 77)
    qa, xa = _aligned(q.shape, np.int8), _aligned(x_bits.shape, np.uint16)
    qa[...] = q
    xa[...] = x_bits
    s32 = scales.astype(np.float32)
    ref = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, x)
    up = (None, None, None)
    if gated:
        rng = np.random.default_rng(5)
        qu = _aligned(q.shape, np.int8)
        qu[...] = rng.integers(-127, 128, size=q.shape).astype(np.int8)
        su = rng.random(N) * 1e-2 + 1e-4
        su32 = su.astype(np.float32)
        up = (_p(qu), _p(su32), None)
        u = oracle.np_linear_forward(qu, su, oracle.PER_CHANNEL, None, x).astype(np.float64)
        g = ref.astype(np.float64)
        ref = (g / (1.0 + np.exp(-g)) * u).astype(np.float32)
    for tile_list, splits in ((1, 1), (1, 2), (4, 2), (5, 3)):
        y = np.full((M, N), 7.0, np.float32)
        rc = emu_pair.emu_gemm_tcgen05_pair(_p(qa), _p(s32), _p(bias), *up, _p(xa), _p(y), M, N, K, N, 0, 0, splits, tile_list)
        if rc == -4:
            emu_pair.emu_fail_message.restype = ctypes.c_char_p
            raise AssertionError(emu_pair.emu_fail_message().decode())
        assert rc == 0
        assert oracle.rel_err(y, ref) < (1e-5 if gated else 2e-6), (tile_list, splits)


# ---- bounded waits: a wait that runs out must end the kernel, not hang it -------------------------------
# On the GPU no wait has ever expired, so the give-up path (record where, raise the CTA-wide abort flag,
# every role falls through to the teardown that frees tensor memory) had only been read, never run.  Here a
# TMA load is dropped on purpose (host-side injection, nothing faults) and the kernel, compiled with small
# wait limits (so small that other roles give up at about the same time, wherever they happen to be), has
# to return with the status set while its 448 threads sit in barriers of every kind.
def _build_short_waits(name):
    src = os.path.join(EMU_DIR, name + ".cpp")
    out = os.path.join(BUILD_DIR, "lib" + name + "_short_waits.so")
    os.makedirs(BUILD_DIR, exist_ok=True)
    deps = [src] + [os.path.join(ROOT, "shrew_b200", "csrc", h) for h in os.listdir(os.path.join(ROOT, "shrew_b200", "csrc")) if h.endswith(".cuh")] + [
        os.path.join(EMU_DIR, h) for h in os.listdir(EMU_DIR) if h.endswith(".h")]
    if not os.path.exists(out) or any(os.path.getmtime(d) > os.path.getmtime(out) for d in deps):
        subprocess.run(["g++", "-std=c++20", "-O1", "-pthread", "-fPIC", "-shared", "-ffp-contract=off", "-fno-fast-math",
                        "-Wno-unknown-pragmas", "-DSHREWQ_SPIN_FAST_LIMIT=64", "-DSHREWQ_SPIN_SLOW_LIMIT=40", "-o", out, src],
                       check=True, cwd=EMU_DIR)
    return ctypes.CDLL(out)


@pytest.mark.parametrize("tok,M,N,K,splits,gated,drop", [
    (64, 40, 128, 1024, 1, False, 0), (64, 40, 128, 1024, 1, False, 7), (256, 300, 128, 512, 1, False, 3),
    (128, 100, 64, 768, 1, True, 4), (32, 20, 128, 1024, 2, False, 5), (16, 8, 128, 2048, 1, False, 31)])
@pytest.mark.timeout(300)   # a deadlock in the give-up path would otherwise hang the suite
def test_tcgen05_wait_that_runs_out_ends_the_kernel(tok, M, N, K, splits, gated, drop):
    L = _build_short_waits("emu_gemm_tcgen05")
    L.emu_gemm_tcgen05.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _sz, _ci, _ci, _ci, _ci, _ci, _ci]
    L.emu_drop_tma.argtypes = [_ci]
    q, scales, bias, x_bits, x = _tc_case(M, N, K, drop)
    qa = _aligned(q.shape, np.int8)
    qa[...] = q
    xa = _aligned(x_bits.shape, np.uint16)
    xa[...] = x_bits
    s32 = scales.astype(np.float32)
    y = np.zeros((M, N), np.float32)
    up = (_p(qa), _p(s32), None) if gated else (None, None, None)
    L.emu_drop_tma(drop)
    try:
        rc = L.emu_gemm_tcgen05(_p(qa), _p(s32), _p(bias), *up, _p(xa), _p(y), M, N, K, N, 0, 0, tok, 3, splits, 0)
    finally:
        L.emu_drop_tma(-1)
    assert rc in (-2, -3, -4)   # a bounded wait gave up and was reported (a tile counter may stay set, and an
    # arrival may find its barrier's phase already spent by roles that gave up)


@pytest.mark.timeout(300)
def test_cta_pair_wait_that_runs_out_ends_both_blocks():
    L = _build_short_waits("emu_gemm_tcgen05_pair")
    L.emu_gemm_tcgen05_pair.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _sz, _ci, _ci, _ci, _ci]
    L.emu_drop_tma.argtypes = [_ci]
    q, scales, bias, x_bits, x = _tc_case(256, 256, 1024, 1)
    qa = _aligned(q.shape, np.int8)
    qa[...] = q
    xa = _aligned(x_bits.shape, np.uint16)
    xa[...] = x_bits
    s32 = scales.astype(np.float32)
    y = np.zeros((256, 256), np.float32)
    for drop in (0, 1, 9, 14):   # a code load or an activation load, of the leader or of the peer
        L.emu_drop_tma(drop)
        try:
            rc = L.emu_gemm_tcgen05_pair(_p(qa), _p(s32), _p(bias), None, None, None, _p(xa), _p(y), 256, 256, 1024, 256, 0, 0, 1, 0)
        finally:
            L.emu_drop_tma(-1)
        assert rc == -2, drop


def test_tcgen05_two_launch_tail_split(oracle, emu_tc):
    # the tail split (option tc_tailsplit): with "5 SMs", 12 tiles = two full waves as whole-K tiles
    # plus 2 tiles split along K in a second launch; both launches index tiles through the 1-D list
    q, scales, bias, x_bits, x = _tc_case(260, 500, 1024, 21)       # 4 channel tiles x 3 token tiles
    ref = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, x, relu=True)
    for splits in (2, 3):
        y = _tc_forward(emu_tc, q, scales, bias, x_bits, 128, 3, splits=splits, epilogue=1, tile_list=5)
        assert oracle.rel_err(y, ref) < 2e-6


def test_tcgen05_peer_destinations(oracle, emu_tc):
    # the all-gather fused into the epilogue: every value also lands at the same offset of each peer buffer
    emu_tc.emu_set_peers.argtypes = [_vp, _ci]
    q, scales, bias, x_bits, x = _tc_case(70, 140, 256, 8)
    ref = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, x)
    ldy = 300                                                           # the shard writes columns [0, 140) of a wider row
    peers = [np.full((70, ldy), 5.0, np.float32) for _ in range(3)]
    arr = (ctypes.c_void_p * 3)(*[p.ctypes.data for p in peers])
    for tok, splits in ((128, 1), (64, 2)):
        emu_tc.emu_set_peers(arr, 3)
        try:
            y = _tc_forward(emu_tc, q, scales, bias, x_bits, tok, 3, splits=splits, ldy=ldy)
        finally:
            emu_tc.emu_set_peers(None, 0)
        for buf in [y] + peers:
            assert oracle.rel_err(buf[:, :140], ref) < 2e-6
            assert np.all(buf[:, 140:] == (7.0 if buf is y else 5.0))


def test_tcgen05_down_projection_shard_split_along_k_with_peers(oracle, emu_tc):
    # the sharded block's second layer: few channel tiles per rank (4096 / 4 = 1024 rows = 8 tiles) over the FULL
    # hidden width, so its k-loop does not shrink with the number of GPUs; split-K on 128-token tiles is what lets it
    # use the idle SMs.  Reduced: 2 channel tiles (the second ragged), 2 token tiles (the second ragged), 11 rounds of
    # 128 k in 3 splits (4 + 4 + 3), bf16 into a column slice of a wider row and into three peer buffers.
    emu_tc.emu_set_peers.argtypes = [_vp, _ci]
    M, N, K, world, rank = 130, 200, 1408, 4, 1
    q, scales, bias, x_bits, x = _tc_case(M, N, K, 17)
    ref = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, x)
    ldy, n0 = world * N, rank * N
    full = [np.full((M, ldy), 0x4100, np.uint16) for _ in range(world)]
    arr = (ctypes.c_void_p * 3)(*[f[:, n0:].ctypes.data for i, f in enumerate(full) if i != rank])
    emu_tc.emu_set_peers(arr, 3)
    try:
        y = _tc_forward(emu_tc, q, scales, bias, x_bits, 128, 3, splits=3, y_bf16=True, ldy=ldy,
                        y_init=np.full((M, ldy), 0x4100, np.uint16))
    finally:
        emu_tc.emu_set_peers(None, 0)
    got = [y[:, :N]] + [f[:, n0:n0 + N] for i, f in enumerate(full) if i != rank]
    for g in got:
        assert oracle.rel_err((g.astype(np.uint32) << 16).view(np.float32), ref) < 1e-2
        assert np.array_equal(g, got[0])
    assert np.all(y[:, N:] == 0x4100) and all(np.all(np.delete(f, np.s_[n0:n0 + N], axis=1) == 0x4100) for i, f in enumerate(full) if i != rank)
    assert np.all(full[rank] == 0x4100)        # the own copy is the kernel's y, not a peer


def test_tcgen05_gated_shard_of_eight_ranks_with_seven_peers(oracle, emu_tc):
    # the benchmark's MLP block over 8 GPUs: each rank owns 11008 / 8 = 1376 = 21 x 64 + 32 hidden channels, so its
    # gated launch ends in a half-full channel tile, writes bf16 into columns [n0, n0 + n_local) of the full-width
    # row and into the same columns of seven peer buffers.  Same structure at reduced size: 2 x 64 + 32 channels,
    # two token tiles (the second ragged), row stride 8 x n_local.
    emu_tc.emu_set_peers.argtypes = [_vp, _ci]
    rng = np.random.default_rng(88)
    M, N, K, world, rank = 130, 160, 256, 8, 3
    ldy = world * N
    qg, qu = (rng.integers(-127, 128, size=(N, K)).astype(np.int8) for _ in range(2))
    sg, su = rng.random(N) * 1e-2 + 1e-4, rng.random(N) * 1e-2 + 1e-4
    x_bits, x = _bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    g = oracle.np_linear_forward(qg, sg, 1, None, x).astype(np.float64)
    u = oracle.np_linear_forward(qu, su, 1, None, x).astype(np.float64)
    ref = (g / (1.0 + np.exp(-g)) * u).astype(np.float32)
    # every buffer is the full [M, ldy] matrix; the kernel is handed the address of column n0 in each
    full = [np.full((M, ldy), 0x4100, np.uint16) for _ in range(world)]
    n0 = rank * N
    views = [f[:, n0:] for f in full]
    arr = (ctypes.c_void_p * 7)(*[v.ctypes.data for i, v in enumerate(views) if i != rank])
    own = np.full((M, ldy), 0x4100, np.uint16)
    emu_tc.emu_set_peers(arr, 7)
    try:
        y = _tc_forward(emu_tc, qg, sg, None, x_bits, 128, 3, y_bf16=True, up=(qu, su, None), ldy=ldy, y_init=own)
    finally:
        emu_tc.emu_set_peers(None, 0)
    # _tc_forward's own buffer starts at column 0: compare its first N columns, and columns [n0, n0 + N) of the peers
    got = [(y[:, :N], y[:, N:])] + [(f[:, n0:n0 + N], np.delete(f, np.s_[n0:n0 + N], axis=1)) for i, f in enumerate(full) if i != rank]
    for inside, outside in got:
        assert oracle.rel_err((inside.astype(np.uint32) << 16).view(np.float32), ref) < 1e-2
        assert np.all(outside == 0x4100)                       # nothing written outside the shard's columns
    assert all(np.array_equal(inside, got[0][0]) for inside, _ in got)   # every copy holds the same bits


# ---- the CUDA-core forward kernels (GPU-validated; here for the stand-in's sake and for the paths the GPU
# tests reach only on several GPUs: peer destinations) ---------------------------------------------------
@pytest.fixture(scope="module")
def emu_cc():
    L = _build("emu_forward_cuda_cores")
    L.emu_forward_cuda_cores.argtypes = [_ci, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _sz, _ci, _ci, _ci, _ci]
    L.emu_set_peers.argtypes = [_vp, _ci]
    return L


def _cc_forward(emu_cc, kernel, q, scales, bias, x, x_bf16, y_bf16, relu=False, up=None, ldy=None, pdl=0, unaligned=False):
    N, K = q.shape
    M = x.shape[0]
    ldy = ldy or N
    pad = 1 if unaligned else 0
    qbuf = _aligned((N * K + pad,), np.int8)
    qa = qbuf[pad:].reshape(N, K)
    qa[...] = q
    xa = _aligned(x.shape, x.dtype)
    xa[...] = x
    y = np.full((M, ldy), 0x4100, np.uint16) if y_bf16 else np.full((M, ldy), 7.0, np.float32)
    s32 = scales.astype(np.float32)
    if up is None:
        args = (_p(qa), _p(s32), None if bias is None else _p(bias), None, None, None)
    else:
        qub = _aligned((N * K + pad,), np.int8)
        qu = qub[pad:].reshape(N, K)
        qu[...] = up[0]
        su = up[1].astype(np.float32)
        args = (_p(qa), _p(s32), None if bias is None else _p(bias), _p(qu), _p(su), None if up[2] is None else _p(up[2]))
    rc = emu_cc.emu_forward_cuda_cores(kernel, *args, _p(xa), _p(y), M, N, K, ldy, 1 if relu else 0, int(x_bf16), int(y_bf16), pdl)
    assert rc == 0
    return y


@pytest.mark.parametrize("M", [1, 2, 3, 4, 7, 8, 16, 17, 40, 64])
@pytest.mark.parametrize("x_bf16", [0, 1], ids=["f32", "bf16"])
def test_gemv_matches_oracle(oracle, emu_cc, M, x_bf16):
    # above 16 tokens the launch is sliced along grid.y (16 tokens per slice, a ragged last slice)
    rng = np.random.default_rng(M)
    N, K = 37, 528
    q = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
    scales = rng.random(N) * 1e-2 + 1e-4
    bias = (rng.standard_normal(N) * 0.1).astype(np.float32)
    x32 = rng.standard_normal((M, K)).astype(np.float32)
    bits, xb = _bf16_bits(x32)
    x_in, x_ref = (bits, xb) if x_bf16 else (x32, x32)
    ref = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, x_ref, relu=True)
    y = _cc_forward(emu_cc, 0, q, scales, bias, x_in, x_bf16, 0, relu=True, ldy=N + 1, pdl=M & 1)
    assert oracle.rel_err(y[:, :N], ref) < 2e-6 and np.all(y[:, N:] == 7.0)


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("y_bf16", [0, 1], ids=["f32-out", "bf16-out"])
@pytest.mark.parametrize("N,K,kc", [(37, 576, 512), (20, 64 * 137, 512), (20, 64 * 137, 1024), (18, 64 * 137, 2048), (5, 64, 1024)],
                         ids=["one-partial-stage", "ring-reused-512", "ring-reused-1024", "ring-reused-2048", "one-k-block"])
def test_ring_kernel_matches_oracle(oracle, emu_cc, M, y_bf16, N, K, kc):
    # bulk copies into the ring + warp MMA: ragged last CTA (rows clamped), a last stage shorter than 512 codes, a
    # K longer than the ring (8 stages of 512: slots are reused through the empty barriers), a row pitch wider
    # than N, relu; several sizes of bulk copy (the launcher instantiates 2048)
    rng = np.random.default_rng(M + K)
    q = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
    scales = rng.random(N) * 1e-2 + 1e-4
    bias = (rng.standard_normal(N) * 0.1).astype(np.float32)
    bits, xb = _bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    ref = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, xb, relu=True)
    emu_cc.emu_set_ring_kc(kc)
    try:
        y = _cc_forward(emu_cc, 2, q, scales, bias, bits, 1, y_bf16, relu=True, ldy=N + 1)
    finally:
        emu_cc.emu_set_ring_kc(2048)
    if y_bf16:
        assert oracle.rel_err((y[:, :N].astype(np.uint32) << 16).view(np.float32), ref) < 1e-2 and np.all(y[:, N:] == 0x4100)
    else:
        assert oracle.rel_err(y[:, :N], ref) < 2e-6 and np.all(y[:, N:] == 7.0)


@pytest.mark.parametrize("M,gated", [(5, False), (16, True), (32, False)])
def test_ring_kernel_with_two_stages(oracle, emu_cc, M, gated):
    # the launcher's choice for grids of several waves: a ring of two 2 KB stages, reused many times over a long K
    rng = np.random.default_rng(M)
    N, K = 21, 64 * 170
    q, qu = (rng.integers(-127, 128, size=(N, K)).astype(np.int8) for _ in range(2))
    scales, su = rng.random(N) * 1e-2 + 1e-4, rng.random(N) * 1e-2 + 1e-4
    bits, xb = _bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    emu_cc.emu_set_ring_kc(2048)
    emu_cc.emu_set_ring_two_stages(1)
    try:
        y = _cc_forward(emu_cc, 2, q, scales, None, bits, 1, 0, up=(qu, su, None) if gated else None)
    finally:
        emu_cc.emu_set_ring_two_stages(0)
    ref = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, None, xb)
    if gated:
        g, u = ref.astype(np.float64), oracle.np_linear_forward(qu, su, 1, None, xb).astype(np.float64)
        ref = (g / (1.0 + np.exp(-g)) * u).astype(np.float32)
    assert oracle.rel_err(y, ref) < 1e-5


@pytest.mark.parametrize("M", [3, 12])
def test_ring_kernel_gate_up_and_peer_destinations(oracle, emu_cc, M):
    rng = np.random.default_rng(14 + M)
    N, K = 50, 1280
    qg, qu = (rng.integers(-127, 128, size=(N, K)).astype(np.int8) for _ in range(2))
    sg, su = rng.random(N) * 1e-2 + 1e-4, rng.random(N) * 1e-2 + 1e-4
    bg, bu = ((rng.standard_normal(N) * 0.1).astype(np.float32) for _ in range(2))
    bits, xb = _bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    g = oracle.np_linear_forward(qg, sg, 1, bg, xb).astype(np.float64)
    u = oracle.np_linear_forward(qu, su, 1, bu, xb).astype(np.float64)
    ref = (g / (1.0 + np.exp(-g)) * u).astype(np.float32)
    peers = [np.full((M, N), 5.0, np.float32) for _ in range(7)]
    arr = (ctypes.c_void_p * 7)(*[p.ctypes.data for p in peers])
    emu_cc.emu_set_peers(arr, 7)
    try:
        y = _cc_forward(emu_cc, 2, qg, sg, bg, bits, 1, 0, up=(qu, su, bu))
    finally:
        emu_cc.emu_set_peers(None, 0)
    for buf in [y] + peers:
        assert oracle.rel_err(buf, ref) < 1e-5


def test_ring_kernel_refuses_what_its_launcher_would(emu_cc):
    q = _aligned((4, 96), np.int8); q[...] = 1
    x = _aligned((33, 96), np.uint16); x[...] = 0x3F80
    s = np.ones(4, np.float32); y = np.zeros((33, 4), np.float32)
    args = (_p(q), _p(s), None, None, None, None, _p(x), _p(y))
    assert emu_cc.emu_forward_cuda_cores(2, *args, 33, 4, 64, 4, 0, 1, 0, 0) == -1   # more than 32 tokens
    assert emu_cc.emu_forward_cuda_cores(2, *args, 1, 4, 96, 4, 0, 1, 0, 0) == -1    # K not a multiple of 64
    assert emu_cc.emu_forward_cuda_cores(2, *args, 1, 4, 64, 4, 0, 0, 0, 0) == -1    # f32 activations


@pytest.mark.parametrize("M,K", [(1, 16 * 296), (4, 16 * 130), (8, 16 * 128), (2, 16 * 5)])
def test_gemv_pdl_variant_gives_the_same_bits(oracle, emu_cc, M, K):
    # the programmatic-dependent-launch variant: the first weights are fetched before the wait for the
    # previous kernel, the remaining chunks in the usual loop; same operations in the same order
    rng = np.random.default_rng(K)
    N = 9
    q = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
    scales = rng.random(N) * 1e-2 + 1e-4
    bits, xb = _bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    ys = [_cc_forward(emu_cc, 0, q, scales, None, bits, 1, 0, pdl=p) for p in (0, 1)]
    np.testing.assert_array_equal(ys[0], ys[1])
    assert oracle.rel_err(ys[1], oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, None, xb)) < 2e-6
    qu = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
    yg = [_cc_forward(emu_cc, 0, q, scales, None, bits, 1, 0, up=(qu, scales, None), pdl=p) for p in (0, 1)]
    np.testing.assert_array_equal(yg[0], yg[1])


def test_gemv_gate_up_and_peer_destinations(oracle, emu_cc):
    rng = np.random.default_rng(4)
    M, N, K = 3, 50, 256
    qg, qu = (rng.integers(-127, 128, size=(N, K)).astype(np.int8) for _ in range(2))
    sg, su = rng.random(N) * 1e-2 + 1e-4, rng.random(N) * 1e-2 + 1e-4
    bits, xb = _bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    g = oracle.np_linear_forward(qg, sg, 1, None, xb).astype(np.float64)
    u = oracle.np_linear_forward(qu, su, 1, None, xb).astype(np.float64)
    ref = (g / (1.0 + np.exp(-g)) * u).astype(np.float32)
    peers = [np.full((M, N), 5.0, np.float32) for _ in range(7)]      # the most a launch takes
    arr = (ctypes.c_void_p * 7)(*[p.ctypes.data for p in peers])
    emu_cc.emu_set_peers(arr, 7)
    try:
        y = _cc_forward(emu_cc, 0, qg, sg, None, bits, 1, 0, up=(qu, su, None))
    finally:
        emu_cc.emu_set_peers(None, 0)
    for buf in [y] + peers:
        assert oracle.rel_err(buf, ref) < 1e-5


@pytest.mark.parametrize("M,N,K,x_bf16,unaligned", [(64, 256, 784, 0, False), (5, 3, 37, 0, True), (130, 70, 100, 1, True), (257, 65, 16, 0, False)])
def test_general_f32_kernel_matches_oracle(oracle, emu_cc, M, N, K, x_bf16, unaligned):
    rng = np.random.default_rng(N)
    q = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
    scales = rng.random(N) * 1e-2 + 1e-4
    bias = (rng.standard_normal(N) * 0.1).astype(np.float32)
    x32 = rng.random((M, K)).astype(np.float32)
    bits, xb = _bf16_bits(x32)
    x_in, x_ref = (bits, xb) if x_bf16 else (x32, x32)
    ref = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, x_ref, relu=True)
    y = _cc_forward(emu_cc, 1, q, scales, bias, x_in, x_bf16, 0, relu=True, unaligned=unaligned)
    assert oracle.rel_err(y, ref) < 1e-5


@pytest.mark.parametrize("seed,one_in", [(1, 8), (2, 300), (3, 3000), (4, 3000)])
@pytest.mark.parametrize("tok,groups,M,N,K,splits,gated", [
    (256, 3, 300, 130, 1536, 1, False),    # 5 stages, 3 groups: a group meets a stage every few phases
    (128, 3, 100, 200, 2048, 1, False),    # 4 stages, 3 groups
    (16, 3, 8, 128, 4096, 1, False),       # 7 stages
    (32, 2, 20, 128, 2048, 2, False),
    (128, 3, 128, 64, 1024, 1, True)])
def test_tcgen05_with_loads_landing_late_and_out_of_order(oracle, emu_tc, seed, one_in, tok, groups, M, N, K, splits, gated):
    # TMA loads are queued at issue and land later, mostly NEWEST FIRST, one per `one_in` barrier polls: the
    # kernel may not rely on loads completing in the order they were issued.  With rounds dealt round-robin
    # to the converter groups (the mapping this kernel had when it was measured) the slow settings of this
    # test fail, with wrong results or a wait that runs out: a group polled a stage barrier whose previous
    # phase was still open and the parity bit answered for the phase two back.  Groups own stages now.
    emu_tc.emu_tma_async.argtypes = [_cu, _cu]
    q, scales, bias, x_bits, x = _tc_case(M, N, K, seed)
    emu_tc.emu_tma_async(seed, one_in)
    try:
        if gated:
            rng = np.random.default_rng(seed)
            qu = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
            su = rng.random(N) * 1e-2 + 1e-4
            y = _tc_forward(emu_tc, q, scales, bias, x_bits, tok, groups, splits=splits, up=(qu, su, None))
            g = oracle.np_linear_forward(q, scales, 1, bias, x).astype(np.float64)
            u = oracle.np_linear_forward(qu, su, 1, None, x).astype(np.float64)
            ref, tol = (g / (1.0 + np.exp(-g)) * u).astype(np.float32), 1e-5
        else:
            y = _tc_forward(emu_tc, q, scales, bias, x_bits, tok, groups, splits=splits)
            ref, tol = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, x), 2e-6
    finally:
        emu_tc.emu_tma_async(0, 0)
    assert oracle.rel_err(y, ref) < tol


def test_cta_pair_with_loads_landing_late_and_out_of_order(oracle, emu_pair):
    emu_pair.emu_tma_async.argtypes = [_cu, _cu]
    q, scales, bias, x_bits, x = _tc_case(300, 260, 2048, 3)
    qa = _aligned(q.shape, np.int8)
    qa[...] = q
    xa = _aligned(x_bits.shape, np.uint16)
    xa[...] = x_bits
    s32 = scales.astype(np.float32)
    ref = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, x)
    for seed, one_in in ((1, 8), (2, 3000)):
        y = np.zeros((300, 260), np.float32)
        emu_pair.emu_tma_async(seed, one_in)
        try:
            assert emu_pair.emu_gemm_tcgen05_pair(_p(qa), _p(s32), _p(bias), None, None, None, _p(xa), _p(y), 300, 260, 2048, 260, 0, 0, 1, 0) == 0
        finally:
            emu_pair.emu_tma_async(0, 0)
        assert oracle.rel_err(y, ref) < 2e-6


@pytest.mark.parametrize("M,N,K", [(256, 128, 256), (300, 200, 384), (40, 70, 1024), (513, 300, 128)])
def test_cta_pair_gate_up_tile(oracle, emu_pair, M, N, K):
    # gate/up on CTA pairs: each block carries 64 gate + 64 up rows, the pair 128 channels x 256 tokens
    rng = np.random.default_rng(M + K)
    qg, qu = (rng.integers(-127, 128, size=(N, K)).astype(np.int8) for _ in range(2))
    sg, su = rng.random(N) * 1e-2 + 1e-4, rng.random(N) * 1e-2 + 1e-4
    bg, bu = ((rng.standard_normal(N) * 0.1).astype(np.float32) for _ in range(2))
    x_bits, x = _bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    g = oracle.np_linear_forward(qg, sg, 1, bg, x).astype(np.float64)
    u = oracle.np_linear_forward(qu, su, 1, bu, x).astype(np.float64)
    ref = (g / (1.0 + np.exp(-g)) * u).astype(np.float32)
    qga, qua = _aligned(qg.shape, np.int8), _aligned(qu.shape, np.int8)
    qga[...] = qg
    qua[...] = qu
    xa = _aligned(x_bits.shape, np.uint16)
    xa[...] = x_bits
    sg32, su32 = sg.astype(np.float32), su.astype(np.float32)
    y = np.full((M, N), 7.0, np.float32)
    rc = emu_pair.emu_gemm_tcgen05_pair(_p(qga), _p(sg32), _p(bg), _p(qua), _p(su32), _p(bu), _p(xa), _p(y), M, N, K, N, 0, 0, 1, 0)
    assert rc == 0
    assert oracle.rel_err(y, ref) < 1e-5


@pytest.mark.parametrize("M,N,K,splits,gated", [(300, 256, 2048, 2, False), (256, 130, 3072, 3, False), (100, 128, 2048, 4, True)])
def test_cta_pair_split_k(oracle, emu_pair, M, N, K, splits, gated):
    # K split over blockIdx.z; every CTA of a pair reduces its own 128 lanes x 256 tokens
    rng = np.random.default_rng(K + splits)
    q, scales, bias, x_bits, x = _tc_case(M, N, K, splits)
    qa = _aligned(q.shape, np.int8)
    qa[...] = q
    xa = _aligned(x_bits.shape, np.uint16)
    xa[...] = x_bits
    s32 = scales.astype(np.float32)
    y = np.full((M, N), 7.0, np.float32)
    if gated:
        qu = _aligned(q.shape, np.int8)
        qu[...] = rng.integers(-127, 128, size=q.shape)
        su = rng.random(N) * 1e-2 + 1e-4
        su32 = su.astype(np.float32)
        rc = emu_pair.emu_gemm_tcgen05_pair(_p(qa), _p(s32), _p(bias), _p(qu), _p(su32), None, _p(xa), _p(y), M, N, K, N, 0, 0, splits, 0)
        g = oracle.np_linear_forward(q, scales, 1, bias, x).astype(np.float64)
        u = oracle.np_linear_forward(np.array(qu), su, 1, None, x).astype(np.float64)
        ref, tol = (g / (1.0 + np.exp(-g)) * u).astype(np.float32), 1e-5
    else:
        rc = emu_pair.emu_gemm_tcgen05_pair(_p(qa), _p(s32), _p(bias), None, None, None, _p(xa), _p(y), M, N, K, N, 1, 0, splits, 0)
        ref, tol = oracle.np_linear_forward(q, scales, oracle.PER_CHANNEL, bias, x, relu=True), 2e-6
    assert rc == 0
    assert oracle.rel_err(y, ref) < tol



# ---- any float storage type (quantize_tensor widens every dtype with to_f64_vec, quantize.rs:198) ------
@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16", "f64"])
@pytest.mark.parametrize("bits,mode", [(8, 0), (8, 1), (4, 0)])
@pytest.mark.parametrize("gran", [0, 1])
def test_quantize_any_storage_type(oracle, emu_modes, dtype, bits, mode, gran):
    emu_modes.emu_quantize_any.argtypes = [_vp, _ci, _sz, _sz, _ci, _ci, _ci, _cu, _vp, _vp, _vp]
    emu_modes.emu_dequantize_any.argtypes = [_vp, _vp, _vp, _sz, _sz, _ci, _ci, _cu, _vp]
    rng = np.random.default_rng(bits + mode + gran)
    rows, cols = 5, 333
    w64 = rng.standard_normal((rows, cols)) * 0.3 + (0.1 if mode else 0.0)
    w64[0, 0], w64[1, 1], w64[2, 2] = np.nan, -0.0, 0.0
    if dtype == "f32":
        stored, code = w64.astype(np.float32), 0
        exact = stored.astype(np.float64)
    elif dtype == "bf16":
        bits16, f = _bf16_bits(w64.astype(np.float32))
        stored, code, exact = bits16, 1, f.astype(np.float64)
    elif dtype == "f16":
        h = w64.astype(np.float16)
        stored, code, exact = h.view(np.uint16).copy(), 2, h.astype(np.float64)
    else:
        w64[3, 3] = 0.1 + 2.0 ** -40          # not representable in f32: the f64 path must not narrow
        stored, code, exact = w64.copy(), 3, w64
    # the oracle restates the arithmetic on f64 data; feed it the exactly widened values (f32 inputs of the
    # oracle are widened the same way, so for the narrower types go through its f64 twin directly)
    n = rows if gran else 1
    q = _aligned((rows, cols), np.int8)
    s, z = np.zeros(n), np.zeros(n)
    sa = _aligned(stored.shape, stored.dtype)
    sa[...] = stored
    assert emu_modes.emu_quantize_any(_p(sa), code, rows, cols, gran, bits, mode, 3, _p(q), _p(s), _p(z)) == 0
    q_ref, s_ref, z_ref = _np_quantize_f64(oracle, exact, gran, bits, mode)
    np.testing.assert_array_equal(q, q_ref)
    assert s.tobytes() == s_ref.tobytes() and z.tobytes() == z_ref.tobytes()
    # dequantize_tensor narrows to the original dtype with one rounding
    back64 = (q_ref.astype(np.float64) - (z_ref.reshape(-1, 1) if gran else z_ref[0])) * (s_ref.reshape(-1, 1) if gran else s_ref[0])
    for out_code, np_dt in ((2, np.float16), (3, np.float64), (0, np.float32)):
        out = _aligned((rows, cols), np_dt)
        zp_arg = _p(z) if mode else None       # symmetric: no zero-point array
        assert emu_modes.emu_dequantize_any(_p(q), _p(s), zp_arg, rows, cols, gran, out_code, 2, _p(out)) == 0
        with np.errstate(over="ignore"):
            np.testing.assert_array_equal(out, back64.astype(np_dt))


def _np_quantize_f64(oracle, data64, gran, bits, mode):
    """the oracle's numpy twin on f64 data (it widens f32 itself; here the data are already f64)"""
    rows, cols = data64.shape
    data = data64 if gran else data64.reshape(1, -1)
    qmax = 7.0 if bits == 4 else 127.0
    qmin = (-8.0 if mode else -7.0) if bits == 4 else (-128.0 if mode else -127.0)
    with np.errstate(all="ignore"):
        if mode:
            lo = np.fmin.reduce(data, axis=1, initial=np.inf)
            hi = np.fmax.reduce(data, axis=1, initial=-np.inf)
            rng_ = hi - lo
            scale = np.where(rng_ < 1e-30, 1.0, rng_ / (qmax - qmin))
            zp = oracle.np_round_half_away(qmin - lo / scale)
        else:
            amax = np.fmax.reduce(np.abs(data), axis=1, initial=0.0)
            scale = np.where(amax < 1e-30, 1.0, amax / qmax)
            zp = np.zeros(data.shape[0])
        inv = np.where(np.abs(scale) < 1e-30, 0.0, 1.0 / scale)
        t = oracle.np_round_half_away(data * inv[:, None] + zp[:, None])
        t = np.where(np.isnan(t), 0.0, np.clip(t, qmin, qmax))
    return t.astype(np.int8).reshape(rows, cols), scale.astype(np.float64), zp.astype(np.float64)


# ---- INT4 codes packed two per byte and their small-batch forward (beyond the reference, never run on a GPU)
def _pack_int4(codes):
    u = (codes.astype(np.int16) + 8).astype(np.uint8) & 0xF
    return (u[:, 0::2] | (u[:, 1::2] << 4)).astype(np.uint8)


def test_pack_int4_kernel(emu_modes):
    emu_modes.emu_pack_int4.argtypes = [_vp, _sz, _cu, _vp]
    rng = np.random.default_rng(0)
    codes = rng.integers(-8, 8, size=(7, 130)).astype(np.int8)
    out = np.zeros((7, 65), np.uint8)
    emu_modes.emu_pack_int4(_p(codes), codes.size // 2, 3, _p(out))
    np.testing.assert_array_equal(out, _pack_int4(codes))


@pytest.mark.parametrize("M,N,K", [(1, 16, 128), (1, 40, 1024), (3, 21, 256), (4, 16, 5120), (5, 16, 128), (16, 24, 384), (17, 17, 256),
                                   (32, 16, 128)])
def test_packed_int4_forward_matches_oracle(oracle, emu_mma, M, N, K):
    emu_mma.emu_gemv_mma_w4.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _sz, _ci, _ci, _vp]
    rng = np.random.default_rng(M * 100 + N + K)
    codes = rng.integers(-8, 8, size=(N, K)).astype(np.int8)       # the asymmetric range too: -8 is representable
    scales = rng.random(N) * 1e-1 + 1e-3
    bias = (rng.standard_normal(N) * 0.1).astype(np.float32)
    x_bits, x = _bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
    ref = oracle.np_linear_forward(codes, scales, oracle.PER_CHANNEL, bias, x, relu=True)
    packed = _aligned((N, K // 2), np.uint8)
    packed[...] = _pack_int4(codes)
    xa = _aligned(x_bits.shape, np.uint16)
    xa[...] = x_bits
    s32 = scales.astype(np.float32)
    y = np.full((M, N + 2), 7.0, np.float32)
    staged = ctypes.c_int(-1)
    rc = emu_mma.emu_gemv_mma_w4(_p(packed), _p(s32), _p(bias), None, None, None, _p(xa), _p(y), M, N, K, N + 2, 1, 0, ctypes.byref(staged))
    assert rc == 0
    assert staged.value == int(M <= 4 and M * K * 2 <= 36864)
    assert oracle.rel_err(y[:, :N], ref) < 2e-6 and np.all(y[:, N:] == 7.0)


def test_packed_int4_gate_up(oracle, emu_mma):
    emu_mma.emu_gemv_mma_w4.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ci, _ci, _ci, _sz, _ci, _ci, _vp]
    rng = np.random.default_rng(9)
    for M, N, K in ((2, 24, 256), (12, 9, 384)):
        cg, cu = (rng.integers(-7, 8, size=(N, K)).astype(np.int8) for _ in range(2))
        sg, su = rng.random(N) * 1e-1 + 1e-3, rng.random(N) * 1e-1 + 1e-3
        x_bits, x = _bf16_bits(rng.standard_normal((M, K)).astype(np.float32))
        g = oracle.np_linear_forward(cg, sg, 1, None, x).astype(np.float64)
        u = oracle.np_linear_forward(cu, su, 1, None, x).astype(np.float64)
        ref = (g / (1.0 + np.exp(-g)) * u).astype(np.float32)
        pg, pu = _aligned((N, K // 2), np.uint8), _aligned((N, K // 2), np.uint8)
        pg[...] = _pack_int4(cg)
        pu[...] = _pack_int4(cu)
        xa = _aligned(x_bits.shape, np.uint16)
        xa[...] = x_bits
        sg32, su32 = sg.astype(np.float32), su.astype(np.float32)
        y = np.zeros((M, N), np.float32)
        staged = ctypes.c_int(-1)
        assert emu_mma.emu_gemv_mma_w4(_p(pg), _p(sg32), None, _p(pu), _p(su32), None, _p(xa), _p(y), M, N, K, N, 0, 0, ctypes.byref(staged)) == 0
        assert oracle.rel_err(y, ref) < 1e-5
