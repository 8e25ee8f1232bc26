"""GPU: the reference's quantization unit tests, restated in C++ against include/shrewq.hpp,
compiled with g++ and run against libshrewq.so."""
import os
import subprocess

import pytest

from tests.conftest import ROOT


def _compile():
    from shrew_b200 import build
    lib = build.build_library()
    out_dir = os.path.join(ROOT, "tests", "cpp", "build")
    os.makedirs(out_dir, exist_ok=True)
    exe = os.path.join(out_dir, "test_quantize_api")
    src = os.path.join(ROOT, "tests", "cpp", "test_quantize_api.cpp")
    cmd = ["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), "-I", "/usr/local/cuda/include", src,
           "-o", exe, "-L", os.path.dirname(lib), "-lshrewq", "-L", "/usr/local/cuda/lib64", "-lcudart",
           "-Wl,-rpath," + os.path.dirname(lib), "-Wl,-rpath,/usr/local/cuda/lib64"]
    subprocess.check_call(cmd)
    return exe


def test_cpp_mirror_compiles():
    # CPU-side: the header and the test translate against the C ABI
    assert os.path.exists(_compile())


@pytest.mark.gpu
def test_reference_unit_tests_in_cpp():
    exe = _compile()
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "9 reference tests passed" in r.stdout


@pytest.mark.gpu
def test_cpp_checkpoint_round_trip(tmp_path):
    # the C++ host's save / load of quantized tensors (include/shrewq_checkpoint.hpp): quantize, save, load,
    # same forward bits; the Python reader opens the file too
    exe = _compile()
    r = subprocess.run([exe, str(tmp_path / "ckpt.safetensors")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "checkpoint round trip passed" in r.stdout
    from shrew_b200 import qsafetensors as qs
    back = qs.unpack_records(*qs.read_file(str(tmp_path / "ckpt.safetensors")))
    assert list(back) == ["fc.weight", "fc_pt.weight"]
    assert back["fc.weight"].codes.shape == (24, 16) and back["fc.weight"].granularity == "per_channel"
    assert back["fc_pt.weight"].scales.size == 1
