"""The `@inference` block of a `.sw` program, read for its `quantization` settings.

Shrew's DSL lets a model file say how it wants to be served (docs/src/dsl/grammar.md:146-154 of the
reference; examples/tiny_gpt.sw:158-164 asks for `mode: "int8"; calibration: "dynamic";`), but the
reference's executors never look at the block: `OpKind::Linear` and `Instruction::Linear` always build a
float `Linear` (crates/shrew/src/exec/engine.rs:411-422, jit.rs:1290-1301).  This module is the front
half of the missing seam: it turns the block into the `QuantConfig` that `QuantizedLinear.from_linear`
takes, so that a host which walks a `.sw` graph can swap each Linear for its quantized form.

Attribute meanings (the reference defines none beyond the grammar; these follow its `QuantConfig`,
quantize.rs:64-121):

    mode:        "int8" | "int4" | "none"           bits; "none" / "fp32" / "off" disables quantization
    granularity: "per_tensor" | "per_channel"        default per_tensor, the reference's default
    per_channel: true | false                        the same as a flag
    symmetric:   true | false                        default true; false = asymmetric (zero points)
    calibration: "dynamic" | "static" | ...          accepted and reported; weights are quantized from
                                                     their own values, no activation calibration exists

Pure text processing: no GPU, no library call.
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Dict, Optional, Union

from .quantize import QuantBits, QuantConfig, QuantGranularity, QuantMode

Value = Union[str, float, int, bool, dict, list]


class SwSyntaxError(ValueError):
    """The text is not what the DSL's grammar allows inside an `@inference` block."""


_TOKEN = re.compile(r"""
    \s+ | //[^\n]* | /\*.*?\*/                                    # blanks and comments
  | (?P<str>"(?:[^"\\]|\\.)*")
  | (?P<num>[-+]?(?:\d+\.\d*|\.\d+|\d+)(?:[eE][-+]?\d+)?)
  | (?P<id>[A-Za-z_][A-Za-z_0-9.]*)
  | (?P<sym>[{}\[\]:;,@])
""", re.VERBOSE | re.DOTALL)


def _tokens(text: str):
    pos, out = 0, []
    while pos < len(text):
        m = _TOKEN.match(text, pos)
        if not m:
            raise SwSyntaxError(f"unexpected character {text[pos]!r} at offset {pos}")
        pos = m.end()
        if m.lastgroup:
            out.append((m.lastgroup, m.group(m.lastgroup), m.start()))
    return out


class _Parser:
    def __init__(self, toks, i):
        self.t, self.i = toks, i

    def peek(self):
        return self.t[self.i] if self.i < len(self.t) else ("eof", "", -1)

    def take(self, kind=None, val=None):
        k, v, at = self.peek()
        if (kind and k != kind) or (val is not None and v != val):
            raise SwSyntaxError(f"expected {val or kind}, found {v or 'end of text'!r} at offset {at}")
        self.i += 1
        return v

    def value(self) -> Value:
        k, v, at = self.peek()
        if k == "str":
            self.i += 1
            return bytes(v[1:-1], "utf-8").decode("unicode_escape") if "\\" in v else v[1:-1]
        if k == "num":
            self.i += 1
            return float(v) if re.search(r"[.eE]", v) else int(v)
        if k == "id":
            self.i += 1
            return {"true": True, "false": False}.get(v, v)
        if k == "sym" and v == "{":
            return self.block()
        if k == "sym" and v == "[":
            self.i += 1
            items = []
            while self.peek()[1] != "]":
                items.append(self.value())
                if self.peek()[1] == ",":
                    self.i += 1
            self.take("sym", "]")
            return items
        raise SwSyntaxError(f"expected a value, found {v or 'end of text'!r} at offset {at}")

    def block(self) -> Dict[str, Value]:
        """"{" { identifier ":" value ";" } "}" """
        self.take("sym", "{")
        out: Dict[str, Value] = {}
        while self.peek()[1] != "}":
            key = self.take("id")
            self.take("sym", ":")
            out[key] = self.value()
            if self.peek()[1] == ";":      # a nested block may omit the ';' (tiny_gpt.sw does)
                self.i += 1
        self.take("sym", "}")
        return out


def parse_inference_block(text: str) -> Optional[Dict[str, Value]]:
    """The attributes of the first `@inference { ... }` block of a `.sw` text as a dict (nested blocks as
    dicts, lists as lists, numbers as int / float, `true` / `false` as bool, identifiers and strings as
    str), or None if the text has no such block."""
    # the other blocks of a program hold expression syntax this reader does not need to understand:
    # cut out the block first (strings and comments may hold braces), then read only that
    skip = re.compile(r'"(?:[^"\\]|\\.)*"|//[^\n]*|/\*.*?\*/', re.DOTALL)
    pos, start = 0, None
    while pos < len(text):
        m = skip.match(text, pos)
        if m:
            pos = m.end()
            continue
        m = re.compile(r"@inference\b").match(text, pos)
        if m:
            start = m.end()
            break
        pos += 1
    if start is None:
        return None
    depth, pos, opened = 0, start, False
    while pos < len(text):
        m = skip.match(text, pos)
        if m:
            pos = m.end()
            continue
        c = text[pos]
        pos += 1
        if c == "{":
            depth += 1
            opened = True
        elif c == "}":
            depth -= 1
            if opened and depth == 0:
                break
    return _Parser(_tokens(text[start:pos]), 0).block()


@dataclass
class InferenceQuantization:
    config: Optional[QuantConfig]      # None: the block asks for no quantization
    calibration: Optional[str]         # reported as written; not used (weight-only quantization)


def quantization_from_sw(text: str) -> Optional[InferenceQuantization]:
    """What the `.sw` text's `@inference { quantization: {...} }` asks for, or None when it does not say."""
    blk = parse_inference_block(text)
    if not blk or "quantization" not in blk:
        return None
    q = blk["quantization"]
    if not isinstance(q, dict):
        raise SwSyntaxError("quantization must be a block of `name: value;` attributes")
    known = {"mode", "granularity", "per_channel", "symmetric", "calibration"}
    for k in q:
        if k not in known:
            raise SwSyntaxError(f"quantization: unknown attribute '{k}' (known: {', '.join(sorted(known))})")
    calibration = q.get("calibration")
    if calibration is not None and not isinstance(calibration, str):
        raise SwSyntaxError("quantization.calibration must be a string")
    mode = q.get("mode", "int8")
    if not isinstance(mode, str) or mode.lower() not in ("int8", "int4", "none", "fp32", "off"):
        raise SwSyntaxError(f"quantization.mode must be \"int8\", \"int4\" or \"none\", not {mode!r}")
    if mode.lower() in ("none", "fp32", "off"):
        return InferenceQuantization(None, calibration)
    gran = q.get("granularity")
    if gran is not None and gran not in ("per_tensor", "per_channel"):
        raise SwSyntaxError(f"quantization.granularity must be \"per_tensor\" or \"per_channel\", not {gran!r}")
    flag = q.get("per_channel")
    if flag is not None and not isinstance(flag, bool):
        raise SwSyntaxError("quantization.per_channel must be true or false")
    if gran is not None and flag is not None and (gran == "per_channel") != flag:
        raise SwSyntaxError("quantization: granularity and per_channel contradict each other")
    per_channel = (gran == "per_channel") if gran is not None else bool(flag)
    sym = q.get("symmetric", True)
    if not isinstance(sym, bool):
        raise SwSyntaxError("quantization.symmetric must be true or false")
    cfg = QuantConfig(QuantBits.Int8 if mode.lower() == "int8" else QuantBits.Int4,
                      QuantMode.Symmetric if sym else QuantMode.Asymmetric,
                      QuantGranularity.PerChannel if per_channel else QuantGranularity.PerTensor)
    return InferenceQuantization(cfg, calibration)
