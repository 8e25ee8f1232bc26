"""shrew_b200 — B200-native INT8 quantization path for Shrew (quantize / dequantize /
quantized Linear forward), hand-written sm_100a kernels behind a C ABI.

The names re-exported here are the ones the reference's facade crate re-exports for this
path (crates/shrew/src/lib.rs:120-124)."""
from .quantize import (  # noqa: F401
    Linear,
    QuantBits,
    QuantConfig,
    QuantGranularity,
    QuantMode,
    QuantStats,
    QuantizedLinear,
    QuantizedTensor,
    ShrewError,
    dequantize_tensor,
    quantization_stats,
    quantize_named_parameters,
    quantize_tensor,
    quantize_tensors,
)
