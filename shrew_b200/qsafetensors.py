"""On-disk record for quantized tensors, in the safetensors container the reference uses for
float tensors (crates/shrew/src/safetensors.rs:1-28: 8-byte little-endian header length, a
JSON header, then the raw little-endian tensor bytes with offsets relative to their start).

The reference has no record for `QuantizedTensor` (its `DType` has no 8-bit signed type and
its loader maps "I8" to a 4-byte type, safetensors.rs:61-75), so a quantized model has to be
re-quantized from floats at every start.  This module stores the struct's fields
(quantize.rs:150-185) as ordinary safetensors entries:

    <name>.qweight       I8    the tensor's shape      codes, source order
    <name>.scales        F64   [1] or [shape[0]]
    <name>.zero_points   F64   same length             all 0.0 in symmetric mode

and describes each record in the header's `__metadata__` (string values only, as the format
requires): `"format": "shrew"` like the reference's writer (safetensors.rs:360-361) plus
`"shrew.quantized"`, a JSON object  name -> {bits, mode, granularity, original_dtype}.  Float
tensors (biases, norms) sit beside them under their own names.  Any safetensors reader can
open the file; the entries are contiguous and cover the data section, as the format demands.

Two layers: `write_file` / `read_file` work on host bytes only (numpy, no GPU); `save` /
`load` move `QuantizedTensor`s between the file and a CUDA device.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple, Union

import numpy as np

# safetensors dtype string -> numpy dtype (little-endian); bf16 has no numpy type: raw uint16
_NP = {"F64": "<f8", "F32": "<f4", "F16": "<f2", "BF16": "<u2", "I64": "<i8", "I32": "<i4", "I16": "<i2",
       "I8": "i1", "U8": "u1", "U16": "<u2", "U32": "<u4", "U64": "<u8", "BOOL": "u1"}
_MAX_HEADER = 100_000_000          # the reference's sanity limit (safetensors.rs:383-388)
_QKEY = "shrew.quantized"
_SUFFIXES = (".qweight", ".scales", ".zero_points")


class FormatError(ValueError):
    """The file is not a well-formed safetensors file, or a quantized record in it is broken."""


@dataclass
class Entry:
    dtype: str                 # safetensors dtype string
    shape: List[int]
    data: np.ndarray           # host array of the numpy dtype in _NP (a view into the mapping when read)


def _nbytes(dtype: str, shape: Sequence[int]) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n * np.dtype(_NP[dtype]).itemsize


def write_file(path: str, entries: Sequence[Tuple[str, Entry]], metadata: Optional[Dict[str, str]] = None) -> None:
    """Writes entries in the given order, contiguously.  The header is padded with spaces to a
    multiple of 8 bytes so that the data section starts aligned."""
    header: Dict[str, object] = {}
    md = {"format": "shrew"}
    md.update(metadata or {})
    for k, v in md.items():
        if not isinstance(k, str) or not isinstance(v, str):
            raise FormatError("safetensors metadata keys and values must be strings")
    header["__metadata__"] = md
    off = 0
    blobs = []
    for name, e in entries:
        if name in header:
            raise FormatError(f"duplicate tensor name '{name}'")
        if e.dtype not in _NP:
            raise FormatError(f"unsupported dtype '{e.dtype}' for '{name}'")
        arr = np.ascontiguousarray(e.data, dtype=_NP[e.dtype]) if e.data.ndim else np.asarray(e.data, dtype=_NP[e.dtype])
        n = _nbytes(e.dtype, e.shape)
        if arr.nbytes != n:
            raise FormatError(f"'{name}': {arr.nbytes} bytes of data for shape {list(e.shape)} of {e.dtype}")
        header[name] = {"dtype": e.dtype, "shape": [int(d) for d in e.shape], "data_offsets": [off, off + n]}
        off += n
        blobs.append(arr)
    raw = json.dumps(header, separators=(",", ":"), ensure_ascii=False).encode("utf-8")
    raw += b" " * (-len(raw) % 8)
    tmp = f"{path}.tmp.{os.getpid()}"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for arr in blobs:
            if arr.size:
                f.write(arr.tobytes() if arr.ndim == 0 else memoryview(arr.reshape(-1)).cast("B"))
    os.replace(tmp, path)  # a reader never sees a half-written file


def read_file(path: str) -> Tuple[Dict[str, str], Dict[str, Entry]]:
    """Maps the file and returns (metadata, name -> Entry) with zero-copy views.  Checks what the
    reference's reader checks (header size, UTF-8, JSON object, dtype, byte count per entry,
    safetensors.rs:132-140,383-403) and, beyond it, that offsets lie inside the file, do not
    overlap and leave no hole."""
    size = os.path.getsize(path)
    if size < 8:
        raise FormatError("file shorter than the 8-byte header length")
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        if hlen > _MAX_HEADER:
            raise FormatError(f"header size {hlen} bytes is unreasonably large")
        if 8 + hlen > size:
            raise FormatError("header runs past the end of the file")
        raw = f.read(hlen)
        try:
            pairs = json.loads(raw.decode("utf-8"), object_pairs_hook=list)
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise FormatError(f"invalid header: {e}") from None
        if not isinstance(pairs, list) or (pairs and not isinstance(pairs[0], tuple)):
            raise FormatError("header is not a JSON object")
        data_len = size - 8 - hlen
        buf = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
    base = 8 + hlen
    metadata: Dict[str, str] = {}
    out: Dict[str, Entry] = {}
    spans = []
    for key, val in pairs:
        if key == "__metadata__":
            if not isinstance(val, list):
                raise FormatError("__metadata__ is not an object")
            for k, v in val:
                if not isinstance(v, str):
                    raise FormatError("__metadata__ values must be strings")
                metadata[k] = v
            continue
        if key in out:
            raise FormatError(f"duplicate tensor name '{key}'")
        if not isinstance(val, list):
            raise FormatError(f"entry '{key}' is not an object")
        obj = dict(val)
        dtype, shape, offs = obj.get("dtype"), obj.get("shape"), obj.get("data_offsets")
        if not isinstance(dtype, str) or dtype not in _NP:
            raise FormatError(f"'{key}': unsupported dtype {dtype!r}")
        if not isinstance(shape, list) or any(not isinstance(d, int) or isinstance(d, bool) or d < 0 for d in shape):
            raise FormatError(f"'{key}': bad shape")
        if (not isinstance(offs, list) or len(offs) != 2
                or any(not isinstance(o, int) or isinstance(o, bool) or o < 0 for o in offs)):
            raise FormatError(f"'{key}': data_offsets must be two non-negative integers")
        start, end = offs
        if end < start or end > data_len:
            raise FormatError(f"'{key}': data_offsets [{start},{end}] outside the {data_len}-byte data section")
        if end - start != _nbytes(dtype, shape):
            raise FormatError(f"'{key}': expected {_nbytes(dtype, shape)} bytes for shape {shape} of {dtype}, got {end - start}")
        arr = np.frombuffer(buf, dtype=_NP[dtype], count=(end - start) // np.dtype(_NP[dtype]).itemsize,
                            offset=base + start).reshape(shape)
        out[key] = Entry(dtype, list(shape), arr)
        spans.append((start, end, key))
    spans.sort()
    pos = 0
    for start, end, key in spans:
        if start != pos:
            raise FormatError(f"'{key}': data section has a hole or an overlap at byte {pos}")
        pos = end
    if pos != data_len:
        raise FormatError(f"{data_len - pos} trailing bytes not covered by any entry")
    return metadata, out


# ---- quantized records on the host -----------------------------------------------------------------
@dataclass
class HostQuantized:
    """The fields of `QuantizedTensor` (quantize.rs:150-185) as host arrays."""
    codes: np.ndarray          # int8, the tensor's shape
    scales: np.ndarray         # float64 [S]
    zero_points: np.ndarray    # float64 [S]
    bits: int = 8
    mode: str = "symmetric"            # "symmetric" | "asymmetric"
    granularity: str = "per_tensor"    # "per_tensor" | "per_channel"
    original_dtype: str = "F32"


def pack_records(named: Sequence[Tuple[str, Union[HostQuantized, Entry]]]):
    """(entries, metadata) for write_file."""
    entries: List[Tuple[str, Entry]] = []
    desc: Dict[str, dict] = {}
    for name, t in named:
        if isinstance(t, Entry):
            if name.endswith(_SUFFIXES):
                raise FormatError(f"'{name}': a plain tensor may not use a quantized record's suffix")
            entries.append((name, t))
            continue
        s = int(t.scales.size)
        rows = int(t.codes.shape[0]) if t.codes.ndim else 1
        want = rows if (t.granularity == "per_channel" and t.codes.ndim) else 1
        if s != want or int(t.zero_points.size) != s:
            raise FormatError(f"'{name}': {s} scales / {int(t.zero_points.size)} zero points for granularity "
                              f"{t.granularity} and shape {list(t.codes.shape)}")
        if t.bits not in (4, 8):
            raise FormatError(f"'{name}': records hold 8-bit or 4-bit codes (one per byte)")
        entries.append((name + ".qweight", Entry("I8", list(t.codes.shape), np.asarray(t.codes, dtype=np.int8))))
        entries.append((name + ".scales", Entry("F64", [s], np.asarray(t.scales, dtype=np.float64).reshape(s))))
        entries.append((name + ".zero_points", Entry("F64", [s], np.asarray(t.zero_points, dtype=np.float64).reshape(s))))
        desc[name] = {"bits": t.bits, "mode": t.mode, "granularity": t.granularity, "original_dtype": t.original_dtype}
    return entries, {_QKEY: json.dumps(desc, separators=(",", ":"), sort_keys=True)}


def unpack_records(metadata: Dict[str, str], entries: Dict[str, Entry]):
    """name -> HostQuantized | Entry, quantized records reassembled and checked."""
    try:
        desc = json.loads(metadata.get(_QKEY, "{}"))
    except json.JSONDecodeError as e:
        raise FormatError(f"metadata '{_QKEY}' is not JSON: {e}") from None
    if not isinstance(desc, dict):
        raise FormatError(f"metadata '{_QKEY}' is not an object")
    out: Dict[str, Union[HostQuantized, Entry]] = {}
    used = set()
    for name, d in desc.items():
        parts = []
        for suf, dt in zip(_SUFFIXES, ("I8", "F64", "F64")):
            e = entries.get(name + suf)
            if e is None:
                raise FormatError(f"quantized record '{name}': entry '{name + suf}' is missing")
            if e.dtype != dt:
                raise FormatError(f"quantized record '{name}': '{name + suf}' has dtype {e.dtype}, expected {dt}")
            parts.append(e)
            used.add(name + suf)
        if not isinstance(d, dict) or d.get("bits") not in (4, 8) or d.get("mode") not in ("symmetric", "asymmetric") \
                or d.get("granularity") not in ("per_tensor", "per_channel") or d.get("original_dtype") not in _NP:
            raise FormatError(f"quantized record '{name}': bad description {d!r}")
        q, sc, zp = parts
        rows = q.shape[0] if q.shape else 1
        want = rows if (d["granularity"] == "per_channel" and q.shape) else 1
        if sc.shape != [want] or zp.shape != [want]:
            raise FormatError(f"quantized record '{name}': {sc.shape} scales for granularity {d['granularity']} "
                              f"and shape {q.shape}")
        out[name] = HostQuantized(q.data, sc.data, zp.data, d["bits"], d["mode"], d["granularity"], d["original_dtype"])
    for name, e in entries.items():
        if name not in used:
            out[name] = e
    return out


# ---- device layer ---------------------------------------------------------------------------------
def save(path: str, named) -> None:
    """named: sequence of (name, QuantizedTensor | torch.Tensor).  Device tensors are copied to
    the host first; float tensors keep their dtype (f32, f64, f16, bf16)."""
    import torch

    from .quantize import QuantGranularity, QuantizedTensor, QuantMode
    st = {torch.float32: "F32", torch.float64: "F64", torch.float16: "F16", torch.bfloat16: "BF16",
          torch.int64: "I64", torch.uint8: "U8", torch.int8: "I8", torch.int32: "I32"}
    host = []
    for name, t in named:
        if isinstance(t, QuantizedTensor):
            gran = "per_channel" if (t.config.granularity is QuantGranularity.PerChannel and len(t.shape)) else "per_tensor"
            mode = "symmetric" if t.config.mode is QuantMode.Symmetric else "asymmetric"
            codes = t.data.detach().cpu().numpy().reshape(t.shape)
            scales = t.scales.detach().cpu().numpy()
            zps = np.zeros_like(scales) if t.zero_points_t is None else t.zero_points_t.detach().cpu().numpy()
            host.append((name, HostQuantized(codes, scales, zps, t.config.bits.value, mode, gran, st[t.original_dtype])))
        else:
            if t.dtype not in st:
                raise FormatError(f"'{name}': dtype {t.dtype} cannot be stored")
            c = t.detach().contiguous().cpu()
            arr = c.view(torch.uint16).numpy() if c.dtype is torch.bfloat16 else c.numpy()
            host.append((name, Entry(st[t.dtype], list(t.shape), arr)))
    entries, md = pack_records(host)
    write_file(path, entries, md)


def load(path: str, device):
    """Returns a list of (name, QuantizedTensor | torch.Tensor) on `device`, quantized records
    first in the order of their description, ready for `QuantizedLinear.new`."""
    import torch

    from .quantize import QuantBits, QuantConfig, QuantGranularity, QuantizedTensor, QuantMode
    ts = {"F32": torch.float32, "F64": torch.float64, "F16": torch.float16, "BF16": torch.bfloat16,
          "I64": torch.int64, "U8": torch.uint8, "I8": torch.int8, "I32": torch.int32}
    metadata, entries = read_file(path)
    out = []
    for name, t in unpack_records(metadata, entries).items():
        if isinstance(t, HostQuantized):
            cfg = QuantConfig(QuantBits.Int8 if t.bits == 8 else QuantBits.Int4,
                              QuantMode.Symmetric if t.mode == "symmetric" else QuantMode.Asymmetric,
                              QuantGranularity.PerChannel if t.granularity == "per_channel" else QuantGranularity.PerTensor)
            q = torch.from_numpy(np.array(t.codes, copy=True).reshape(-1)).to(device)
            s = torch.from_numpy(np.array(t.scales, copy=True)).to(device)
            z = None if t.mode == "symmetric" else torch.from_numpy(np.array(t.zero_points, copy=True)).to(device)
            out.append((name, QuantizedTensor(q, s, [int(d) for d in t.codes.shape], ts[t.original_dtype], cfg, z)))
        else:
            if t.dtype not in ts:
                raise FormatError(f"'{name}': dtype {t.dtype} has no device tensor type here")
            arr = np.array(t.data, copy=True)
            tt = torch.from_numpy(arr).view(torch.bfloat16) if t.dtype == "BF16" else torch.from_numpy(arr)
            out.append((name, tt.to(device)))
    return out
