"""CPU: the C++ host mirror (include/shrewq.hpp, shrewq_checkpoint.hpp) exercised end to end without a GPU.

tests/cpp/test_quantize_api.cpp — the reference's nine quantization unit tests (crates/shrew/src/quantize.rs:601-789)
restated in C++, plus the save / load round trip — is linked against a stand-in for libshrewq.so and the CUDA
runtime (tests/cpp/standin_libshrewq.cpp: host memory as device memory, the oracle's arithmetic behind the C ABI).
A mistake in the host code above the C ABI (argument order, shapes, ownership, the on-disk record) then shows up
here and not first in a GPU session.  The same binary source runs against the real library in
tests/test_gpu_cpp_api.py."""
import os
import subprocess

import pytest

from tests.conftest import ROOT


@pytest.fixture(scope="module")
def exe():
    from oracle import shrew_oracle
    shrew_oracle.build()
    out = os.path.join(ROOT, "tests", "cpp", "build", "standin")
    os.makedirs(out, exist_ok=True)
    inc = ["-I", os.path.join(ROOT, "include"), "-I", "/usr/local/cuda/include"]
    lib = os.path.join(out, "libshrewq.so")
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-fPIC", "-shared", *inc,
                           os.path.join(ROOT, "tests", "cpp", "standin_libshrewq.cpp"),
                           "-x", "c", "-ffp-contract=off", os.path.join(ROOT, "oracle", "shrew_oracle.c"), "-o", lib, "-lm"])
    binary = os.path.join(out, "test_quantize_api")
    subprocess.check_call(["g++", "-std=c++17", "-O1", *inc, os.path.join(ROOT, "tests", "cpp", "test_quantize_api.cpp"),
                           "-o", binary, "-L", out, "-lshrewq", "-Wl,-rpath," + out])
    return binary


def test_reference_unit_tests_in_cpp_against_the_standin(exe):
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "9 reference tests passed" in r.stdout


def test_cpp_checkpoint_round_trip_against_the_standin(exe, tmp_path):
    path = str(tmp_path / "ckpt.safetensors")
    r = subprocess.run([exe, path], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "checkpoint round trip passed" in r.stdout
    # the same assertions the GPU test makes on the file
    from shrew_b200 import qsafetensors as qs
    back = qs.unpack_records(*qs.read_file(path))
    assert list(back) == ["fc.weight", "fc_pt.weight"]
    assert back["fc.weight"].codes.shape == (24, 16) and back["fc.weight"].granularity == "per_channel"
    assert back["fc_pt.weight"].scales.size == 1
    # and the codes in the file are the oracle's for the weight the C++ test builds
    import numpy as np
    from oracle import shrew_oracle as oracle
    w = (np.sin(0.37 * np.arange(24 * 16, dtype=np.float64)) * 0.4).astype(np.float32).reshape(24, 16)
    q, s = oracle.np_quantize_f32(w, oracle.PER_CHANNEL)
    np.testing.assert_array_equal(back["fc.weight"].codes, q)
    assert back["fc.weight"].scales.tobytes() == s.tobytes()
