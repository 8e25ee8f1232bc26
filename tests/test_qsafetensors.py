"""The on-disk record for quantized tensors (shrew_b200/qsafetensors.py): host layer on the CPU,
cross-checked against the `safetensors` package in both directions; device round trip on a GPU."""
import json
import struct

import numpy as np
import pytest

from shrew_b200 import qsafetensors as qs

st_numpy = pytest.importorskip("safetensors.numpy")


def _record(rows=6, cols=10, gran="per_channel", seed=0):
    rng = np.random.default_rng(seed)
    codes = rng.integers(-127, 128, size=(rows, cols)).astype(np.int8)
    s = rows if gran == "per_channel" else 1
    return qs.HostQuantized(codes, rng.random(s) * 1e-2 + 1e-9, np.zeros(s), 8, "symmetric", gran, "F32")


def test_round_trip_host(tmp_path):
    p = str(tmp_path / "m.safetensors")
    named = [("fc1.weight", _record(6, 10)), ("fc1.bias", qs.Entry("F32", [1, 6], np.arange(6, dtype=np.float32).reshape(1, 6))),
             ("fc2.weight", _record(3, 6, "per_tensor", seed=1)), ("step", qs.Entry("I64", [], np.array(7, dtype=np.int64)))]
    entries, md = qs.pack_records(named)
    qs.write_file(p, entries, md)
    metadata, got = qs.read_file(p)
    assert metadata["format"] == "shrew"            # as the reference's writer tags its files
    back = qs.unpack_records(metadata, got)
    assert list(back)[:2] == ["fc1.weight", "fc2.weight"]
    for name, t in named:
        b = back[name]
        if isinstance(t, qs.HostQuantized):
            np.testing.assert_array_equal(b.codes, t.codes)
            np.testing.assert_array_equal(b.scales, t.scales)      # f64 scales survive bit for bit
            np.testing.assert_array_equal(b.zero_points, t.zero_points)
            assert (b.bits, b.mode, b.granularity, b.original_dtype) == (8, "symmetric", t.granularity, "F32")
        else:
            assert b.dtype == t.dtype and b.shape == t.shape
            np.testing.assert_array_equal(b.data, t.data)


def test_file_is_plain_safetensors(tmp_path):
    # the reference library of the format reads what we write ...
    p = str(tmp_path / "m.safetensors")
    rec = _record(5, 8)
    entries, md = qs.pack_records([("w", rec)])
    qs.write_file(p, entries, md)
    theirs = st_numpy.load_file(p)
    assert theirs["w.qweight"].dtype == np.int8 and theirs["w.scales"].dtype == np.float64
    np.testing.assert_array_equal(theirs["w.qweight"], rec.codes)
    np.testing.assert_array_equal(theirs["w.scales"], rec.scales)
    # ... and we read what it writes, including its own header padding and metadata
    p2 = str(tmp_path / "theirs.safetensors")
    st_numpy.save_file({"a": np.arange(12, dtype=np.float32).reshape(3, 4), "b": np.array([1, -2, 3], dtype=np.int8)}, p2,
                       metadata={"k": "v"})
    metadata, got = qs.read_file(p2)
    assert metadata == {"k": "v"}
    np.testing.assert_array_equal(got["a"].data, np.arange(12, dtype=np.float32).reshape(3, 4))
    assert got["b"].dtype == "I8" and got["b"].data.tolist() == [1, -2, 3]
    assert qs.unpack_records(metadata, got).keys() == {"a", "b"}   # no quantized records described: all plain


def test_layout_matches_the_reference_writer(tmp_path):
    # 8-byte little-endian header length, JSON header, data; offsets relative to the data section,
    # entries back to back in the order given (safetensors.rs:336-377)
    p = str(tmp_path / "m.safetensors")
    a = np.array([1.5, -2.0], dtype=np.float32)
    b = np.array([[1, 2, 3]], dtype=np.int8)
    qs.write_file(p, [("a", qs.Entry("F32", [2], a)), ("b", qs.Entry("I8", [1, 3], b))])
    raw = open(p, "rb").read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    assert hlen % 8 == 0
    header = json.loads(raw[8:8 + hlen])
    assert header["a"] == {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}
    assert header["b"] == {"dtype": "I8", "shape": [1, 3], "data_offsets": [8, 11]}
    assert raw[8 + hlen:] == a.tobytes() + b.tobytes()


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
    (b'{"a":{"dtype":"F32","shape":[1],"data_offsets":[0]}}', b"\0" * 4, "data_offsets"),
    (b'{"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]}}', b"\0" * 4, "duplicate"),
    (b'[1,2]', b"", "not a JSON object"),
    (b'{"a":', b"", "invalid header"),
    (b'\xff\xfe{}', b"", "invalid header"),
    (b'{"__metadata__":{"k":1}}', b"", "must be strings"),
])
def test_malformed_files_are_rejected(tmp_path, header, data, msg):
    p = str(tmp_path / "bad.safetensors")
    _write_raw(p, header, data)
    with pytest.raises(qs.FormatError, match=msg):
        qs.read_file(p)


def test_header_length_limits(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    open(p, "wb").write(b"\x01\x02")
    with pytest.raises(qs.FormatError, match="shorter"):
        qs.read_file(p)
    open(p, "wb").write(struct.pack("<Q", 200_000_000) + b"{}")
    with pytest.raises(qs.FormatError, match="unreasonably large"):   # the reference's limit, safetensors.rs:383-388
        qs.read_file(p)
    open(p, "wb").write(struct.pack("<Q", 50) + b"{}")
    with pytest.raises(qs.FormatError, match="past the end"):
        qs.read_file(p)


def test_broken_quantized_records_are_rejected(tmp_path):
    p = str(tmp_path / "m.safetensors")
    rec = _record(4, 4)
    entries, md = qs.pack_records([("w", rec)])
    # a described record with a missing part
    qs.write_file(p, [e for e in entries if not e[0].endswith(".scales")], md)
    with pytest.raises(qs.FormatError, match="missing"):
        qs.unpack_records(*qs.read_file(p))
    # scales of the wrong length for the granularity
    bad = qs.HostQuantized(rec.codes, rec.scales[:2], rec.zero_points[:2], 8, "symmetric", "per_channel", "F32")
    with pytest.raises(qs.FormatError, match="scales"):
        qs.pack_records([("w", bad)])
    # a description that is not what this format defines
    qs.write_file(p, entries, {"shrew.quantized": json.dumps({"w": {"bits": 2, "mode": "symmetric",
                                                                      "granularity": "per_channel", "original_dtype": "F32"}})})
    with pytest.raises(qs.FormatError, match="bad description"):
        qs.unpack_records(*qs.read_file(p))
    # a plain tensor squatting on a record's suffix
    with pytest.raises(qs.FormatError, match="suffix"):
        qs.pack_records([("w.scales", qs.Entry("F32", [1], np.zeros(1, np.float32)))])
    with pytest.raises(qs.FormatError, match="duplicate"):
        qs.write_file(p, [("a", qs.Entry("U8", [1], np.zeros(1, np.uint8)))] * 2)


def test_empty_and_rank0_records(tmp_path):
    p = str(tmp_path / "m.safetensors")
    r0 = qs.HostQuantized(np.array(5, dtype=np.int8), np.array([0.25]), np.zeros(1), 8, "symmetric", "per_channel", "F32")
    empty = qs.HostQuantized(np.zeros((0, 7), np.int8), np.zeros(0), np.zeros(0), 8, "symmetric", "per_channel", "F32")
    entries, md = qs.pack_records([("scalar", r0), ("empty", empty)])
    qs.write_file(p, entries, md)
    back = qs.unpack_records(*qs.read_file(p))
    assert back["scalar"].codes.shape == () and int(back["scalar"].codes) == 5   # rank 0: one per-tensor scale (quantize.rs:276-278)
    assert back["empty"].codes.shape == (0, 7) and back["empty"].scales.size == 0
    qs.write_file(p, [])
    assert qs.read_file(p) == ({"format": "shrew"}, {})


@pytest.mark.gpu
def test_device_round_trip(tmp_path):
    import torch

    from shrew_b200 import Linear, QuantConfig, QuantizedLinear, quantize_tensor
    from shrew_b200.quantize import Device
    rng = np.random.default_rng(0)
    w = torch.from_numpy((rng.standard_normal((96, 256)) * 0.05).astype(np.float32)).cuda()
    b = torch.from_numpy(rng.standard_normal(96).astype(np.float32)).cuda()
    x = torch.from_numpy(rng.standard_normal((5, 256)).astype(np.float32)).cuda().to(torch.bfloat16)
    ql = QuantizedLinear.from_linear(Linear(w, b), QuantConfig.int8_per_channel())
    qt2 = quantize_tensor(w, QuantConfig.int8())
    p = str(tmp_path / "m.safetensors")
    qs.save(p, [("fc.weight", ql.weight_q), ("fc.bias", ql.bias), ("fc_pt.weight", qt2), ("emb", x)])
    got = dict(qs.load(p, "cuda:0"))
    assert torch.equal(got["fc.weight"].data, ql.weight_q.data) and torch.equal(got["fc.weight"].scales, ql.weight_q.scales)
    assert got["fc.weight"].shape == [96, 256] and got["fc.weight"].original_dtype == torch.float32
    assert torch.equal(got["fc_pt.weight"].data, qt2.data) and got["fc_pt.weight"].scales.numel() == 1
    assert torch.equal(got["emb"], x) and torch.equal(got["fc.bias"], ql.bias)
    ql2 = QuantizedLinear.new(got["fc.weight"], got["fc.bias"])
    y1, y2 = ql.forward(x), ql2.forward(x)
    Device.get("cuda:0").synchronize()
    assert torch.equal(y1, y2)


def test_device_layer_round_trip_on_cpu_tensors(tmp_path):
    # `save` / `load` are plain torch + numpy: with CPU tensors they run without a GPU (the GPU test above
    # adds the forward through the loaded layer)
    import torch

    from shrew_b200 import QuantConfig
    from shrew_b200.quantize import QuantizedTensor
    rng = np.random.default_rng(1)
    codes = torch.from_numpy(rng.integers(-127, 128, size=96 * 32).astype(np.int8))
    pc = QuantizedTensor(codes, torch.from_numpy(rng.random(96) * 1e-2), [96, 32], torch.float32, QuantConfig.int8_per_channel())
    pt = QuantizedTensor(codes[:64].clone(), torch.tensor([0.125], dtype=torch.float64), [2, 4, 8], torch.bfloat16, QuantConfig.int8())
    asym = QuantizedTensor(codes[:12].clone(), torch.from_numpy(rng.random(3)), [3, 4], torch.float32,
                           QuantConfig.int8_per_channel().asymmetric(), torch.tensor([-3.0, 0.0, 17.0], dtype=torch.float64))
    bias = torch.arange(96, dtype=torch.float32)
    emb = torch.arange(12, dtype=torch.float32).reshape(3, 4).to(torch.bfloat16)
    p = str(tmp_path / "m.safetensors")
    qs.save(p, [("fc.weight", pc), ("fc.bias", bias), ("pt.weight", pt), ("asym.weight", asym), ("emb", emb)])
    got = dict(qs.load(p, "cpu"))
    for name, t in (("fc.weight", pc), ("pt.weight", pt), ("asym.weight", asym)):
        g = got[name]
        assert torch.equal(g.data, t.data) and torch.equal(g.scales, t.scales) and g.shape == t.shape
        assert g.original_dtype == t.original_dtype and g.config == t.config
    assert got["fc.weight"].zero_points_t is None and got["pt.weight"].zero_points_t is None
    assert torch.equal(got["asym.weight"].zero_points_t, asym.zero_points_t)
    assert torch.equal(got["fc.bias"], bias) and torch.equal(got["emb"], emb) and got["emb"].dtype == torch.bfloat16
