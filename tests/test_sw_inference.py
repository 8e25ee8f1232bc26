"""The `@inference` block of a `.sw` program -> QuantConfig (shrew_b200/sw_inference.py).  Text only."""
import pytest

from shrew_b200 import QuantBits, QuantGranularity, QuantMode
from shrew_b200.sw_inference import SwSyntaxError, parse_inference_block, quantization_from_sw

# a program in the DSL's grammar (docs/src/dsl/grammar.md:146-154 of the reference), written for this test
PROGRAM = '''
@model { name: "TwoLayer"; version: "0.1"; }
@config { d_model: 64; d_ff: 64 * 4; }
@graph Forward(x: Tensor<[Batch, 64], f32>) -> Tensor<[Batch, 10], f32> {
    input x: Tensor<[Batch, 64], f32>;
    param w1: Tensor<[256, 64], f32> { init: "normal(0, 0.02)"; };
    node h { op: relu(linear(x, w1)); };
    output h;
}
// how the model wants to be served
@inference {
    model: Forward;
    optimizations: ["fuse_matmul_add", "constant_folding"];
    quantization: {
        mode: "int8";            /* weight-only */
        calibration: "dynamic";
    }
    generation: { strategy: "top_p"; temperature: 0.9; top_p: 0.95; max_tokens: 256; }
    batch_size: 8;
}
@metrics M { track loss { source: loss; } }
'''


def test_block_is_read_as_written():
    blk = parse_inference_block(PROGRAM)
    assert blk["model"] == "Forward"
    assert blk["optimizations"] == ["fuse_matmul_add", "constant_folding"]
    assert blk["quantization"] == {"mode": "int8", "calibration": "dynamic"}
    assert blk["generation"] == {"strategy": "top_p", "temperature": 0.9, "top_p": 0.95, "max_tokens": 256}
    assert blk["batch_size"] == 8
    assert parse_inference_block("@model { name: \"x\"; }") is None


def test_default_request_is_the_reference_default_config():
    got = quantization_from_sw(PROGRAM)
    # QuantConfig::int8(): symmetric, per-tensor (quantize.rs:64-75)
    assert (got.config.bits, got.config.mode, got.config.granularity) == (QuantBits.Int8, QuantMode.Symmetric, QuantGranularity.PerTensor)
    assert got.calibration == "dynamic"
    assert quantization_from_sw("@inference { model: Forward; }") is None
    assert quantization_from_sw("@graph G() {}") is None


@pytest.mark.parametrize("attrs,bits,mode,gran", [
    ('mode: "int8"; granularity: "per_channel";', QuantBits.Int8, QuantMode.Symmetric, QuantGranularity.PerChannel),
    ('mode: "int8"; per_channel: true;', QuantBits.Int8, QuantMode.Symmetric, QuantGranularity.PerChannel),
    ('mode: "int4"; symmetric: false;', QuantBits.Int4, QuantMode.Asymmetric, QuantGranularity.PerTensor),
    ('mode: "INT8"; symmetric: true; per_channel: false;', QuantBits.Int8, QuantMode.Symmetric, QuantGranularity.PerTensor),
    ('', QuantBits.Int8, QuantMode.Symmetric, QuantGranularity.PerTensor),
])
def test_attributes_map_to_quant_config(attrs, bits, mode, gran):
    got = quantization_from_sw("@inference { quantization: { %s } }" % attrs)
    assert (got.config.bits, got.config.mode, got.config.granularity) == (bits, mode, gran)


def test_quantization_can_be_switched_off():
    for m in ("none", "fp32", "off"):
        got = quantization_from_sw('@inference { quantization: { mode: "%s"; }; }' % m)
        assert got is not None and got.config is None


@pytest.mark.parametrize("text,msg", [
    ('@inference { quantization: { mode: "int2"; } }', "mode"),
    ('@inference { quantization: { mode: 8; } }', "mode"),
    ('@inference { quantization: { bits: 8; } }', "unknown attribute"),
    ('@inference { quantization: { granularity: "per_row"; } }', "granularity"),
    ('@inference { quantization: { granularity: "per_channel"; per_channel: false; } }', "contradict"),
    ('@inference { quantization: { symmetric: "yes"; } }', "symmetric"),
    ('@inference { quantization: "int8"; }', "block"),
    ('@inference { quantization: { mode "int8"; } }', "expected"),
    ('@inference { quantization: { mode: "int8"; ', "expected"),
    ('@inference { quantization: { mode: # } }', "unexpected character"),
])
def test_malformed_requests_are_refused(text, msg):
    with pytest.raises(SwSyntaxError, match=msg):
        quantization_from_sw(text)
