"""Host-side launch planning of the QuantizedLinear forward (kernel family, token tile, tile grid, K splits).

`shrewq_plan_forward` is pure host arithmetic, so the choice the library would make on a 148-SM GPU is
checked here without one.  The forward it plans replaces QuantizedLinear::forward
(crates/shrew/src/quantize.rs:208-223 of the reference), which has one code path for every shape.
"""
import ctypes
import itertools

import pytest

from shrew_b200 import _lib

SMS = 148


def plan(M, N, K, bf16=1, gated=0, sms=SMS):
    name = ctypes.create_string_buffer(32)
    out = [ctypes.c_int(-1) for _ in range(5)]
    rc = _lib.lib().shrewq_plan_forward(M, N, K, bf16, gated, sms, name, 32, *[ctypes.byref(v) for v in out])
    return rc, name.value.decode(), dict(zip(("tok", "n_tiles", "m_tiles", "splits", "rounds"), (v.value for v in out)))


def test_small_batches_go_to_the_streaming_kernels():
    for M in (1, 2):
        rc, name, p = plan(M, 4096, 4096)
        assert (rc, name) == (0, "gemv") and not any(p.values())
    for M in (3, 4, 8, 16):
        rc, name, p = plan(M, 4096, 4096)        # 256 CTAs of 16 rows: resident at once on 148 SMs
        assert (rc, name) == (0, "mma-ring") and not any(p.values())
        assert plan(M, 4096, 11008)[1] == "mma-ring"
        assert plan(M, 11008, 4096)[1] == "mma-ring"          # 688 CTAs: the two-stage ring
        assert plan(M, 5920, 4096, gated=1)[1] == "mma-ring"  # gated: 8 channels per CTA, 740 CTAs = five per SM
        assert plan(M, 5928, 4096, gated=1)[1] == "mma"
        assert plan(M, 32000, 4096)[1] == "mma"               # 2000 CTAs: the register-streaming kernel
        assert plan(M, 4096, 4096, sms=50)[1] == "mma"
    for M in (17, 32):
        rc, name, p = plan(M, 4096, 4096)
        assert (rc, name) == (0, "mma") and not any(p.values())
    assert plan(33, 4096, 4096)[1] == "tcgen05"
    assert plan(8, 4096, 4112)[1] == "tcgen05"          # the warp-MMA kernel wants in_features in blocks of 64
    assert plan(4, 4096, 4112)[1] == "gemv"


def test_f32_activations_take_the_hi_lo_pass_on_the_tensor_cores():
    assert plan(8, 4096, 4096, bf16=0)[1] == "gemv"
    assert plan(16, 4096, 4096, bf16=0)[1] == "gemv"
    assert plan(17, 4096, 4096, bf16=0)[1] == "tcgen05-f32"
    assert plan(64, 256, 784, bf16=0)[1] == "gemv"       # config 1: a few MFLOP, one short sliced launch
    assert plan(64, 10, 256, bf16=0)[1] == "gemv"
    assert plan(129, 256, 784, bf16=0)[1] == "tcgen05-f32"
    assert plan(128, 1024, 1024, bf16=0)[1] == "tcgen05-f32"
    assert plan(512, 4096, 4096, bf16=0)[1] == "tcgen05-f32"
    assert plan(512, 4096, 4100, bf16=0)[1] == "simt"    # ragged in_features: the general kernel
    assert plan(512, 4096, 4096, bf16=0, gated=1)[1] == "simt"


def test_ragged_in_features_fall_back_to_the_general_kernel():
    for K in (4100, 17, 1):
        assert plan(8, 4096, K)[1] == "simt"
        assert plan(1, 4096, K)[1] == "simt"


@pytest.mark.parametrize("gated", [0, 1])
@pytest.mark.parametrize("M,N,K", list(itertools.product(
    (33, 64, 100, 128, 129, 256, 512, 1000, 2048, 8192),
    (128, 1000, 4096, 11008, 32000),
    (16, 64, 128, 4096, 11008))))
def test_the_plan_covers_the_problem(M, N, K, gated):
    rc, name, p = plan(M, N, K, gated=gated)
    assert rc == 0 and name in ("tcgen05", "tcgen05-2cta")
    if name == "tcgen05-2cta":          # CTA pairs: at least a full wave of pair tiles, or a quarter wave over a long K
        pair_tiles = -(-N // (128 if gated else 256)) * -(-M // 256)
        assert M > 128 and (pair_tiles >= 64 or (pair_tiles >= 16 and K >= 8192))
        return
    chan = 64 if gated else 128
    assert p["tok"] in (16, 32, 64, 128, 256)
    assert p["n_tiles"] == -(-N // chan)
    assert p["m_tiles"] == -(-M // p["tok"])
    # the token tile is not a size larger than the batch needs
    assert p["tok"] == 16 or p["tok"] // 2 < M
    # every 64-wide block of in_features belongs to exactly one split
    kblk = 64 if p["tok"] == 256 else 128
    rounds_total = -(-K // kblk)
    assert p["splits"] >= 1 and p["rounds"] >= 1
    assert p["splits"] * p["rounds"] >= rounds_total
    assert (p["splits"] - 1) * p["rounds"] < rounds_total
    # K is split only to fill SMs that the tile grid leaves idle, and never below a useful pipeline length
    tiles = p["n_tiles"] * p["m_tiles"]
    if p["splits"] > 1:
        assert tiles * p["splits"] <= SMS          # all splits of all tiles run in one wave
        assert p["rounds"] >= (2 if p["tok"] <= 64 else 8)


def test_headline_shapes():
    # a 4096x4096 projection at 64 tokens: 32 channel tiles cannot fill 148 SMs, so K is split
    assert plan(64, 4096, 4096)[2] == dict(tok=64, n_tiles=32, m_tiles=1, splits=4, rounds=8)
    # wide projections fill the GPU by themselves
    assert plan(64, 11008, 4096)[2] == dict(tok=64, n_tiles=86, m_tiles=1, splits=1, rounds=32)
    # prefill: 128-token tiles until the grid is several waves deep, then 256
    assert plan(512, 4096, 4096)[2]["tok"] == 128
    assert plan(768, 4096, 4096)[2] == dict(tok=256, n_tiles=32, m_tiles=3, splits=1, rounds=64)
    # the benchmark's block at batch 512 runs on CTA pairs: 172 pair tiles (gate/up), 32 pair tiles over K = 11008 (down)
    assert plan(512, 11008, 4096, gated=1)[1] == "tcgen05-2cta"
    assert plan(512, 4096, 11008)[1] == "tcgen05-2cta"
    assert plan(512, 4096, 4096)[1] == "tcgen05"
    assert plan(2048, 4096, 4096)[1] == "tcgen05-2cta"
    # one rank's share of that block sharded over 4 GPUs stays on the single-CTA kernel: gate and up halves share a
    # tile (twice the channel tiles), 256 tokens above a batch of 128
    assert plan(512, 2752, 4096, gated=1) == (0, "tcgen05", dict(tok=256, n_tiles=43, m_tiles=2, splits=1, rounds=64))
    assert plan(128, 11008, 4096, gated=1)[2]["tok"] == 128
    # the down projection of a block sharded over 8 GPUs: 4 channel tiles x 4 token tiles, K split to fill the SMs
    p = plan(512, 512, 11008)[2]
    assert p["tok"] == 128 and p["splits"] == 9 and p["rounds"] == 10


def test_fewer_sms_split_less():
    full = plan(64, 4096, 4096, sms=148)[2]["splits"]
    small = plan(64, 4096, 4096, sms=40)[2]["splits"]
    assert small <= full and small == 1


def test_bad_arguments_are_refused():
    L = _lib.lib()
    name = ctypes.create_string_buffer(32)
    v = [ctypes.c_int() for _ in range(5)]
    refs = [ctypes.byref(x) for x in v]
    assert L.shrewq_plan_forward(8, 4096, 4096, 1, 0, 148, None, 32, *refs) != 0
    assert L.shrewq_plan_forward(8, 4096, 4096, 1, 0, 148, name, 4, *refs) != 0
    assert L.shrewq_plan_forward(8, 4096, 4096, 1, 0, 0, name, 32, *refs) != 0
    assert L.shrewq_plan_forward(8, 0, 4096, 1, 0, 148, name, 32, *refs) != 0
    assert L.shrewq_plan_forward(8, 4096, 0, 1, 0, 148, name, 32, *refs) != 0
    assert L.shrewq_plan_forward(8, 4096, 4096, 1, 0, 148, name, 32, None, *refs[1:]) != 0
