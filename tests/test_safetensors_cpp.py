"""The C++ reader / writer of the quantized on-disk record (include/shrewq_safetensors.hpp) against the
Python one (shrew_b200/qsafetensors.py): files of either side are read by the other, and the C++ reader
refuses the same malformed files.  Host only."""
import json
import os
import struct
import subprocess

import numpy as np
import pytest

from shrew_b200 import qsafetensors as qs
from tests.conftest import ROOT


@pytest.fixture(scope="module")
def tool():
    out_dir = os.path.join(ROOT, "tests", "cpp", "build")
    os.makedirs(out_dir, exist_ok=True)
    exe = os.path.join(out_dir, "st_tool")
    src = os.path.join(ROOT, "tests", "cpp", "st_tool.cpp")
    hdr = os.path.join(ROOT, "include", "shrewq_safetensors.hpp")
    if not os.path.exists(exe) or max(os.path.getmtime(src), os.path.getmtime(hdr)) > os.path.getmtime(exe):
        subprocess.check_call(["g++", "-std=c++17", "-O1", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"),
                               src, "-o", exe])
    return exe


def _fnv(b: bytes) -> str:
    h = 1469598103934665603
    for c in b:
        h = ((h ^ c) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return f"{h:016x}"


def _record(rows, cols, gran, seed, mode="symmetric", bits=8):
    rng = np.random.default_rng(seed)
    lim = 127 if bits == 8 else 7
    codes = rng.integers(-lim, lim + 1, size=(rows, cols)).astype(np.int8)
    s = rows if gran == "per_channel" else 1
    zp = np.zeros(s) if mode == "symmetric" else np.round(rng.standard_normal(s) * 10)
    return qs.HostQuantized(codes, rng.random(s) * 1e-2 + 1e-9, zp, bits, mode, gran, "F32")


def _model():
    return [("fc1.weight", _record(6, 10, "per_channel", 0)),
            ("fc1.bias", qs.Entry("F32", [1, 6], np.arange(6, dtype=np.float32).reshape(1, 6))),
            ("fc2.weight", _record(3, 6, "per_tensor", 1, mode="asymmetric")),
            ("emb é\"x", qs.Entry("BF16", [2, 3], np.arange(6, dtype=np.uint16).reshape(2, 3))),   # a name that needs escaping
            ("fc3.weight", _record(5, 4, "per_channel", 2, bits=4)),
            ("step", qs.Entry("I64", [], np.array(7, dtype=np.int64))),
            ("empty", qs.Entry("F32", [0, 4], np.zeros((0, 4), np.float32)))]


def _dump(tool, path):
    r = subprocess.run([tool, "dump", path], capture_output=True, text=True)
    return r.returncode, r.stdout


def test_cpp_reads_what_python_writes(tool, tmp_path):
    p = str(tmp_path / "m.safetensors")
    named = _model()
    entries, md = qs.pack_records(named)
    qs.write_file(p, entries, md)
    rc, out = _dump(tool, p)
    assert rc == 0, out
    lines = out.splitlines()
    assert "meta format shrew" in lines
    want = [f"tensor {name} {e.dtype} [{','.join(str(d) for d in e.shape)}] {e.data.nbytes} {_fnv(e.data.tobytes())}"
            for name, e in entries]
    assert [l for l in lines if l.startswith("tensor ")] == want          # every entry, in header order
    quant = [l for l in lines if l.startswith("quant ")]
    assert len(quant) == 3
    for name, t in named:
        if isinstance(t, qs.HostQuantized):
            shape = f"[{','.join(str(d) for d in t.codes.shape)}]"
            want = (f"quant {name} {t.bits} {t.mode} {t.granularity} F32 {shape} {t.scales.size} {_fnv(t.codes.tobytes())} "
                    f"{_fnv(t.scales.astype('<f8').tobytes())} {_fnv(t.zero_points.astype('<f8').tobytes())}")
            assert want in quant, (want, quant)


def test_python_reads_what_cpp_writes(tool, tmp_path):
    p, p2 = str(tmp_path / "m.safetensors"), str(tmp_path / "copy.safetensors")
    named = _model()
    entries, md = qs.pack_records(named)
    md["note"] = "line\nbreak é \"quoted\" \\ tab\t"
    qs.write_file(p, entries, md)
    r = subprocess.run([tool, "copy", p, p2], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    raw = open(p2, "rb").read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    assert hlen % 8 == 0                                     # data section (and the f64 scales in it) stays aligned
    json.loads(raw[8:8 + hlen])                              # a plain JSON header
    metadata, got = qs.read_file(p2)
    assert metadata["format"] == "shrew" and metadata["note"] == md["note"]
    assert json.loads(metadata["shrew.quantized"]) == json.loads(md["shrew.quantized"])
    back = qs.unpack_records(metadata, got)
    for name, t in named:
        b = back[name]
        if isinstance(t, qs.HostQuantized):
            np.testing.assert_array_equal(b.codes, t.codes)
            np.testing.assert_array_equal(b.scales, t.scales)
            np.testing.assert_array_equal(b.zero_points, t.zero_points)
            assert (b.bits, b.mode, b.granularity, b.original_dtype) == (t.bits, t.mode, t.granularity, "F32")
        else:
            assert (b.dtype, b.shape) == (t.dtype, t.shape)
            np.testing.assert_array_equal(b.data, t.data)
    # and the safetensors package reads it too
    safetensors = pytest.importorskip("safetensors")
    with safetensors.safe_open(p2, framework="np") as f:        # (its numpy loader has no bf16: one entry at a time)
        assert set(f.keys()) == set(got)
        np.testing.assert_array_equal(f.get_tensor("fc1.weight.qweight"), named[0][1].codes)
        np.testing.assert_array_equal(f.get_tensor("fc2.weight.zero_points"), named[2][1].zero_points)


def _write_raw(path, header: bytes, data: bytes):
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(header)) + header + data)


@pytest.mark.parametrize("header,data,msg", [
    (b'{"a":{"dtype":"F32","shape":[2],"data_offsets":[0,8]}}', b"\0" * 4, "outside"),
    (b'{"a":{"dtype":"F32","shape":[3],"data_offsets":[0,8]}}', b"\0" * 8, "expected 12 bytes"),
    (b'{"a":{"dtype":"F32","shape":[1],"data_offsets":[4,8]}}', b"\0" * 8, "hole"),
    (b'{"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}', b"\0" * 8, "trailing"),
    (b'{"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},"b":{"dtype":"F32","shape":[1],"data_offsets":[2,6]}}', b"\0" * 6, "overlap"),
    (b'{"a":{"dtype":"Q4","shape":[1],"data_offsets":[0,4]}}', b"\0" * 4, "unsupported dtype"),
    (b'{"a":{"dtype":"F32","shape":[-1],"data_offsets":[0,4]}}', b"\0" * 4, "bad shape"),
    (b'{"a":{"dtype":"F32","shape":[1.5],"data_offsets":[0,4]}}', b"\0" * 4, "bad shape"),
    (b'{"a":{"dtype":"F32","shape":[4611686018427387904,4],"data_offsets":[0,0]}}', b"", "bad shape"),
    (b'{"a":{"dtype":"F32","shape":[1],"data_offsets":[0]}}', b"\0" * 4, "data_offsets"),
    (b'{"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}', b"\0" * 4, "duplicate"),
    (b'[1,2]', b"", "not a JSON object"),
    (b'{"a":', b"", "invalid header"),
    (b'{"a":1} x', b"", "invalid header"),
    (b'\xff\xfe{}', b"", "invalid header"),
    (b'{"__metadata__":{"k":1}}', b"", "must be strings"),
    (b'{"__metadata__":{"shrew.quantized":"{\\"w\\":{\\"bits\\":8,\\"mode\\":\\"symmetric\\",\\"granularity\\":\\"per_channel\\",'
     b'\\"original_dtype\\":\\"F32\\"}}"}}', b"", "is missing"),
    (b'{"__metadata__":{"shrew.quantized":"[1]"}}', b"", "not an object"),
])
def test_cpp_reader_refuses_malformed_files(tool, tmp_path, header, data, msg):
    p = str(tmp_path / "bad.safetensors")
    _write_raw(p, header, data)
    rc, out = _dump(tool, p)
    assert rc == 2 and msg in out, out


def test_cpp_reader_header_limits_and_record_checks(tool, tmp_path):
    p = str(tmp_path / "bad.safetensors")
    open(p, "wb").write(b"\x01\x02")
    assert "shorter" in _dump(tool, p)[1]
    open(p, "wb").write(struct.pack("<Q", 200_000_000) + b"{}")
    assert "unreasonably large" in _dump(tool, p)[1]           # the reference's limit, safetensors.rs:383-388
    open(p, "wb").write(struct.pack("<Q", 50) + b"{}")
    assert "past the end" in _dump(tool, p)[1]
    rec = _record(4, 4, "per_channel", 0)
    entries, md = qs.pack_records([("w", rec)])
    bad = dict(md)
    bad["shrew.quantized"] = json.dumps({"w": {"bits": 2, "mode": "symmetric", "granularity": "per_channel", "original_dtype": "F32"}})
    qs.write_file(p, entries, bad)
    assert "bad description" in _dump(tool, p)[1]
    bad["shrew.quantized"] = json.dumps({"w": {"bits": 8, "mode": "symmetric", "granularity": "per_tensor", "original_dtype": "F32"}})
    qs.write_file(p, entries, bad)
    assert "wrong number of scales" in _dump(tool, p)[1]
    wrong = [(n, qs.Entry("F32", e.shape, e.data.astype(np.float32)) if n.endswith(".scales") else e) for n, e in entries]
    qs.write_file(p, wrong, md)
    assert "expected F64" in _dump(tool, p)[1]
    qs.write_file(p, [])
    assert _dump(tool, p) == (0, "meta format shrew\n")
