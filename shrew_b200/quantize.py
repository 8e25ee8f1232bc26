"""Host-side mirror of the reference's `quantize` module (crates/shrew/src/quantize.rs)
over the libshrewq C ABI.

Same names, argument meaning and error behaviour as the Rust API, so tests read like the
reference's own.  Tensors are torch CUDA tensors (torch is plumbing here: device memory
and streams); every computation is a libshrewq kernel.  There is no CPU path: a tensor
that is not on a CUDA device is rejected.
"""
from __future__ import annotations

import ctypes
import enum
import os
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib
from ._lib import ShrewError

__all__ = [
    "QuantBits", "QuantMode", "QuantGranularity", "QuantConfig", "QuantizedTensor", "quantize_tensor",
    "dequantize_tensor", "absmax", "quantize_tensor_given_amax", "QuantizedLinear", "quantize_named_parameters", "QuantStats", "quantization_stats",
    "Linear", "ShrewError", "Device",
]


# ---- configuration (quantize.rs:35-140) ---------------------------------------------------
class QuantBits(enum.Enum):
    Int8 = 8
    Int4 = 4


class QuantMode(enum.Enum):
    Symmetric = 0
    Asymmetric = 1


class QuantGranularity(enum.Enum):
    PerTensor = _lib.PER_TENSOR
    PerChannel = _lib.PER_CHANNEL


@dataclass
class QuantConfig:
    """quantize.rs:64-121.  Default = INT8 symmetric per-tensor."""
    bits: QuantBits = QuantBits.Int8
    mode: QuantMode = QuantMode.Symmetric
    granularity: QuantGranularity = QuantGranularity.PerTensor

    @staticmethod
    def int8() -> "QuantConfig":
        return QuantConfig()

    @staticmethod
    def int8_per_channel() -> "QuantConfig":
        return QuantConfig(QuantBits.Int8, QuantMode.Symmetric, QuantGranularity.PerChannel)

    @staticmethod
    def int4() -> "QuantConfig":
        return QuantConfig(QuantBits.Int4, QuantMode.Symmetric, QuantGranularity.PerTensor)

    @staticmethod
    def int4_per_channel() -> "QuantConfig":
        return QuantConfig(QuantBits.Int4, QuantMode.Symmetric, QuantGranularity.PerChannel)

    def asymmetric(self) -> "QuantConfig":
        return QuantConfig(self.bits, QuantMode.Asymmetric, self.granularity)

    def qmax(self) -> float:
        return 127.0 if self.bits is QuantBits.Int8 else 7.0

    def qmin(self) -> float:
        if self.bits is QuantBits.Int8:
            return -127.0 if self.mode is QuantMode.Symmetric else -128.0
        return -7.0 if self.mode is QuantMode.Symmetric else -8.0

    def _is_int8_symmetric(self) -> bool:
        return self.bits is QuantBits.Int8 and self.mode is QuantMode.Symmetric

    def _require_int8_symmetric(self) -> None:
        if not self._is_int8_symmetric():
            raise ShrewError(_lib.ERR_UNSUPPORTED,
                             "this entry point takes INT8 symmetric quantization only")

    def _abi_mode(self) -> Tuple[int, int]:
        return (8 if self.bits is QuantBits.Int8 else 4, _lib.SYMMETRIC if self.mode is QuantMode.Symmetric else _lib.ASYMMETRIC)


# ---- device / context ------------------------------------------------------------------------
class Device:
    """One libshrewq context per CUDA device (the role of `B::Device`).  Work is enqueued on
    torch's current stream for that device."""
    _by_index: dict = {}

    def __init__(self, index: int):
        self.index = index
        h = ctypes.c_void_p()
        rc = _lib.lib().shrewq_ctx_create(index, None, ctypes.byref(h))
        _lib.check(rc, None)
        self.handle = h

    @classmethod
    def get(cls, device) -> "Device":
        dev = torch.device(device)
        if dev.type != "cuda":
            raise ShrewError(_lib.ERR_NO_DEVICE, f"tensor is on '{dev}'; this path runs on CUDA devices only (no CPU fallback)")
        idx = dev.index if dev.index is not None else torch.cuda.current_device()
        d = cls._by_index.get(idx)
        if d is None:
            d = cls._by_index[idx] = Device(idx)
        return d

    def bind_stream(self) -> None:
        s = torch.cuda.current_stream(self.index).cuda_stream
        _lib.check(_lib.lib().shrewq_ctx_set_stream(self.handle, ctypes.c_void_p(s)), self.handle)

    def synchronize(self) -> None:
        """Waits for the stream and surfaces a kernel that gave up a bounded wait."""
        self.bind_stream()
        _lib.check(_lib.lib().shrewq_ctx_synchronize(self.handle), self.handle)

    def launch_count(self) -> int:
        return int(_lib.lib().shrewq_ctx_launch_count(self.handle))

    def set_option(self, name: str, value: int) -> None:
        """A launch option of this device's context (shrewq_ctx_set_option: "tc_pair", "tc_tailsplit", ...)."""
        _lib.check(_lib.lib().shrewq_ctx_set_option(self.handle, name.encode(), int(value)), self.handle)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _rows_cols(shape: Sequence[int]) -> Tuple[int, int]:
    """rows = shape[0], cols = product(shape[1..]) (quantize.rs:280-281); rank 0 is one
    per-tensor element (quantize.rs:276-278)."""
    if len(shape) == 0:
        return 1, 1
    cols = 1
    for s in shape[1:]:
        cols *= int(s)
    return int(shape[0]), cols


_DTYPE_CODE = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}
# storage types of quantize_tensor / dequantize_tensor (the forward takes f32 and bf16 only)
_STORAGE_CODE = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16, torch.float64: _lib.F64}


# ---- QuantizedTensor (quantize.rs:150-185) -----------------------------------------------------
@dataclass
class QuantizedTensor:
    data: torch.Tensor            # int8 codes on the device, flat, source order
    scales: torch.Tensor          # float64 on the device, len 1 or shape[0]
    shape: List[int]
    original_dtype: torch.dtype
    config: QuantConfig = field(default_factory=QuantConfig)
    zero_points_t: Optional[torch.Tensor] = None   # float64 on the device; None = all 0.0 (symmetric)

    @property
    def zero_points(self) -> List[float]:
        """All 0.0 in symmetric mode (quantize.rs:351); round(qmin - min/scale) per group otherwise."""
        if self.zero_points_t is not None:
            return [float(v) for v in self.zero_points_t.cpu().tolist()]
        return [0.0] * int(self.scales.numel())

    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= int(s)
        return n

    def size_bytes(self) -> int:
        return self.numel() if self.config.bits is QuantBits.Int8 else (self.numel() + 1) // 2

    def compression_ratio(self) -> float:
        return (self.numel() * 4) / self.size_bytes()


def quantize_tensor(tensor: torch.Tensor, config: QuantConfig) -> QuantizedTensor:
    """quantize.rs:194-205 on the GPU.  `tensor` is a float CUDA tensor.  f32 INT8 symmetric runs the
    tuned kernels (shrewq_quantize_f32); the other modes and storage types go through
    shrewq_quantize_f32_ex / shrewq_quantize_any."""
    dev = Device.get(tensor.device)
    if tensor.dtype not in _STORAGE_CODE:
        raise ShrewError(_lib.ERR_UNSUPPORTED, f"quantize_tensor: dtype {tensor.dtype} is not a float storage type")
    w = tensor.contiguous()
    shape = list(w.shape)
    rows, cols = _rows_cols(shape)
    gran = config.granularity
    if len(shape) == 0:
        gran = QuantGranularity.PerTensor
    n_scales = rows if gran is QuantGranularity.PerChannel else 1
    q = torch.empty(w.numel(), dtype=torch.int8, device=w.device)
    scales = torch.empty(n_scales, dtype=torch.float64, device=w.device)
    dev.bind_stream()
    if config._is_int8_symmetric() and w.dtype is torch.float32:
        rc = _lib.lib().shrewq_quantize_f32(dev.handle, _ptr(w), rows, cols, gran.value, _ptr(q), _ptr(scales))
        _lib.check(rc, dev.handle)
        return QuantizedTensor(q, scales, shape, tensor.dtype, config)
    bits, mode = config._abi_mode()
    zps = torch.empty(n_scales, dtype=torch.float64, device=w.device)
    if w.dtype is torch.float32:
        rc = _lib.lib().shrewq_quantize_f32_ex(dev.handle, _ptr(w), rows, cols, gran.value, bits, mode, _ptr(q), _ptr(scales),
                                               _ptr(zps))
    else:  # bf16 / f16 / f64 storage: every element is widened to f64 like the reference's to_f64_vec
        rc = _lib.lib().shrewq_quantize_any(dev.handle, _ptr(w), _STORAGE_CODE[w.dtype], rows, cols, gran.value, bits, mode,
                                            _ptr(q), _ptr(scales), _ptr(zps))
    _lib.check(rc, dev.handle)
    return QuantizedTensor(q, scales, shape, tensor.dtype, config, zps if config.mode is QuantMode.Asymmetric else None)


def quantize_tensors(tensors: Sequence[torch.Tensor], config: QuantConfig) -> List[QuantizedTensor]:
    """`quantize_tensor` for many tensors in a few launches in all (shrewq_quantize_f32_batch): what a model
    of many small matrices needs, where a launch per tensor costs more than the data.  F32 CUDA tensors on
    one device, INT8 symmetric; same codes and scales as `quantize_tensor`."""
    if not tensors:
        return []
    if not config._is_int8_symmetric():
        raise ShrewError(_lib.ERR_UNSUPPORTED, "quantize_tensors: INT8 symmetric only")
    dev = Device.get(tensors[0].device)
    items = (_lib.QuantItem * len(tensors))()
    out, keep = [], []
    per_tensor_group: List[int] = []     # rank-0 tensors fall back to per-tensor (quantize.rs:276-278)
    for i, t in enumerate(tensors):
        if t.dtype is not torch.float32 or t.device != tensors[0].device:
            raise ShrewError(_lib.ERR_UNSUPPORTED, "quantize_tensors: f32 tensors on one CUDA device")
        w = t.contiguous()
        shape = list(w.shape)
        rows, cols = _rows_cols(shape)
        gran = config.granularity if shape else QuantGranularity.PerTensor
        if gran is not config.granularity:
            per_tensor_group.append(i)
        q = torch.empty(w.numel(), dtype=torch.int8, device=w.device)
        scales = torch.empty(rows if gran is QuantGranularity.PerChannel else 1, dtype=torch.float64, device=w.device)
        items[i] = _lib.QuantItem(_ptr(w), rows, cols, _ptr(q), _ptr(scales))
        keep.append(w)
        out.append(QuantizedTensor(q, scales, shape, t.dtype, config))
    dev.bind_stream()
    main = [i for i in range(len(tensors)) if i not in per_tensor_group]
    for idx, gran in ((main, config.granularity), (per_tensor_group, QuantGranularity.PerTensor)):
        if idx:
            sub = (_lib.QuantItem * len(idx))(*[items[i] for i in idx])
            _lib.check(_lib.lib().shrewq_quantize_f32_batch(dev.handle, ctypes.cast(sub, ctypes.c_void_p), len(idx), gran.value),
                       dev.handle)
    return out


def absmax(tensor: torch.Tensor) -> torch.Tensor:
    """max |w| of an f32 CUDA tensor (NaN ignored) as a 1-element f32 tensor on its device: the value
    a per-tensor scale derives from (quantize.rs:349-351).  For shards: reduce it over the ranks with
    MAX, then `quantize_tensor_given_amax`."""
    dev = Device.get(tensor.device)
    if tensor.dtype != torch.float32:
        raise ShrewError(_lib.ERR_UNSUPPORTED, f"absmax: dtype {tensor.dtype} not supported (f32 only)")
    w = tensor.contiguous()
    out = torch.empty(1, dtype=torch.float32, device=w.device)
    dev.bind_stream()
    _lib.check(_lib.lib().shrewq_absmax_f32(dev.handle, _ptr(w), w.numel(), _ptr(out)), dev.handle)
    return out


def quantize_tensor_given_amax(tensor: torch.Tensor, amax: torch.Tensor) -> QuantizedTensor:
    """INT8 symmetric per-tensor quantization of a shard with the whole tensor's amax supplied
    (a 1-element f32 tensor on the same device)."""
    dev = Device.get(tensor.device)
    if tensor.dtype != torch.float32 or amax.dtype != torch.float32 or amax.numel() != 1 or amax.device != tensor.device:
        raise ShrewError(_lib.ERR_INVALID_ARG, "quantize_tensor_given_amax: f32 tensor and a 1-element f32 amax on its device")
    w = tensor.contiguous()
    q = torch.empty(w.numel(), dtype=torch.int8, device=w.device)
    scale = torch.empty(1, dtype=torch.float64, device=w.device)
    dev.bind_stream()
    rc = _lib.lib().shrewq_quantize_f32_given_amax(dev.handle, _ptr(w), w.numel(), _ptr(amax.contiguous()), _ptr(q), _ptr(scale))
    _lib.check(rc, dev.handle)
    return QuantizedTensor(q, scale, list(w.shape), tensor.dtype, QuantConfig.int8())


def pack_int4(qtensor: QuantizedTensor) -> torch.Tensor:
    """INT4 codes (one per i8, as quantize_tensor returns them) -> two per byte: a uint8 tensor
    [shape[0], cols / 2], byte j of a row = code 2j + 8 in the low and code 2j+1 + 8 in the high nibble."""
    dev = Device.get(qtensor.data.device)
    rows, cols = _rows_cols(qtensor.shape)
    out = torch.empty((rows, cols // 2), dtype=torch.uint8, device=qtensor.data.device)
    dev.bind_stream()
    _lib.check(_lib.lib().shrewq_pack_int4(dev.handle, _ptr(qtensor.data), rows, cols, _ptr(out)), dev.handle)
    return out


def dequantize_tensor(qtensor: QuantizedTensor, device=None) -> torch.Tensor:
    """quantize.rs:210-225 on the GPU: a tensor of the original dtype and shape."""
    dev_t = qtensor.data.device if device is None else torch.device(device)
    dev = Device.get(dev_t)
    out_dtype = qtensor.original_dtype
    if out_dtype not in _STORAGE_CODE:
        raise ShrewError(_lib.ERR_UNSUPPORTED, f"dequantize_tensor: target dtype {out_dtype} not supported")
    rows, cols = _rows_cols(qtensor.shape)
    gran = qtensor.config.granularity if len(qtensor.shape) else QuantGranularity.PerTensor
    out = torch.empty(qtensor.shape, dtype=out_dtype, device=qtensor.data.device)
    dev.bind_stream()
    if qtensor.zero_points_t is not None or out_dtype not in _DTYPE_CODE:
        rc = _lib.lib().shrewq_dequantize_ex(dev.handle, _ptr(qtensor.data), _ptr(qtensor.scales), _ptr(qtensor.zero_points_t),
                                             rows, cols, gran.value, _STORAGE_CODE[out_dtype], _ptr(out))
    else:
        rc = _lib.lib().shrewq_dequantize(dev.handle, _ptr(qtensor.data), _ptr(qtensor.scales), rows, cols, gran.value,
                                          _DTYPE_CODE[out_dtype], _ptr(out))
    _lib.check(rc, dev.handle)
    return out


# ---- a minimal shrew_nn::Linear stand-in --------------------------------------------------------
class Linear:
    """Holds what QuantizedLinear::from_linear reads from shrew_nn::Linear: weight [out,in]
    and an optional bias stored as [1,out] (crates/shrew/tests/nn_tests.rs:43-44)."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, name: str = ""):
        assert weight.dim() == 2
        self.weight = weight
        self.bias = None if bias is None else bias.reshape(1, -1)
        self.name = name

    def parameters(self) -> List[torch.Tensor]:
        return [self.weight] + ([self.bias] if self.bias is not None else [])

    def named_parameters(self) -> List[Tuple[str, torch.Tensor]]:
        p = self.name + "." if self.name else ""
        return [(p + "weight", self.weight)] + ([(p + "bias", self.bias)] if self.bias is not None else [])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise ShrewError(_lib.ERR_UNSUPPORTED, "the float Linear forward is outside this library's path")


# ---- QuantizedLinear (quantize.rs:384-482) --------------------------------------------------------
class QuantizedLinear:
    def __init__(self, weight_q: QuantizedTensor, bias: Optional[torch.Tensor], device=None):
        """QuantizedLinear::new (quantize.rs:437-447).  A weight carrying zero points (asymmetric
        mode) goes through shrewq_linear_create_ex; INT4 codes are ordinary i8 codes within [-8, 7]."""
        if weight_q.config.mode is QuantMode.Asymmetric and weight_q.zero_points_t is None:
            raise ShrewError(_lib.ERR_INVALID_ARG, "QuantizedLinear: an asymmetric weight needs its zero points")
        if len(weight_q.shape) != 2:
            raise ShrewError(_lib.ERR_INVALID_ARG, "QuantizedLinear needs a rank-2 weight [out,in]")
        self.weight_q = weight_q
        self.bias = bias
        self.out_features, self.in_features = int(weight_q.shape[0]), int(weight_q.shape[1])
        self.device = Device.get(weight_q.data.device if device is None else device)
        self._bias_flat = None
        if bias is not None:
            if bias.numel() != self.out_features:
                raise ShrewError(_lib.ERR_INVALID_ARG, "bias must have out_features elements")
            self._bias_flat = bias.reshape(-1).to(torch.float32).contiguous()
        h = ctypes.c_void_p()
        self.device.bind_stream()
        if weight_q.zero_points_t is not None and weight_q.config.mode is QuantMode.Asymmetric:
            rc = _lib.lib().shrewq_linear_create_ex(self.device.handle, _ptr(weight_q.data), _ptr(weight_q.scales),
                                                    _ptr(weight_q.zero_points_t), _ptr(self._bias_flat), self.out_features,
                                                    self.in_features, weight_q.config.granularity.value, ctypes.byref(h))
        else:
            rc = _lib.lib().shrewq_linear_create(self.device.handle, _ptr(weight_q.data), _ptr(weight_q.scales),
                                                 _ptr(self._bias_flat), self.out_features, self.in_features,
                                                 weight_q.config.granularity.value, ctypes.byref(h))
        _lib.check(rc, self.device.handle)
        self._h = h

    @classmethod
    def new(cls, weight_q: QuantizedTensor, bias: Optional[torch.Tensor], device=None) -> "QuantizedLinear":
        return cls(weight_q, bias, device)

    @classmethod
    def new_int4_packed(cls, weight_q: QuantizedTensor, bias: Optional[torch.Tensor] = None) -> "QuantizedLinear":
        """A layer over INT4 codes packed two per byte (beyond the reference, whose INT4 tensors keep one
        code per i8): half the weight bytes of INT8 for the small-batch forward (bf16 activations, M <= 32,
        in_features a multiple of 128).  `weight_q` is an INT4 symmetric QuantizedTensor."""
        if weight_q.config.bits is not QuantBits.Int4 or weight_q.config.mode is not QuantMode.Symmetric:
            raise ShrewError(_lib.ERR_INVALID_ARG, "new_int4_packed: needs an INT4 symmetric weight")
        self = cls.__new__(cls)
        self.weight_q, self.bias = weight_q, bias
        self.out_features, self.in_features = int(weight_q.shape[0]), int(weight_q.shape[1])
        self.device = Device.get(weight_q.data.device)
        self.packed = pack_int4(weight_q)
        self._bias_flat = None if bias is None else bias.reshape(-1).to(torch.float32).contiguous()
        h = ctypes.c_void_p()
        self.device.bind_stream()
        rc = _lib.lib().shrewq_linear_create_int4(self.device.handle, _ptr(self.packed), _ptr(weight_q.scales), _ptr(self._bias_flat),
                                                  self.out_features, self.in_features, weight_q.config.granularity.value,
                                                  ctypes.byref(h))
        _lib.check(rc, self.device.handle)
        self._h = h
        return self

    @classmethod
    def from_linear(cls, linear, config: QuantConfig) -> "QuantizedLinear":
        """quantize.rs:413-434: params[0] is the weight, params[1] the bias if present."""
        params = list(linear.parameters())
        weight = params[0]
        bias = params[1] if len(params) > 1 else None
        return cls(quantize_tensor(weight.detach(), config), None if bias is None else bias.detach(), weight.device)

    def weight_quantized(self) -> QuantizedTensor:
        return self.weight_q

    def memory_savings_bytes(self) -> int:
        return int(_lib.lib().shrewq_linear_memory_savings_bytes(self._h))

    def parameters(self) -> list:
        """Inference only: no trainable parameters (quantize.rs:478-481)."""
        return []

    # The rest of the Module surface a QuantizedLinear inherits from the trait's defaults (the reference
    # overrides only forward and parameters, quantize.rs:462-482; containers such as DataParallel forward
    # these calls to the module they wrap, distributed.rs:203-218).  They follow from parameters() being
    # empty; the mode flag is kept and returned as set, the forward does not depend on it.
    def named_parameters(self) -> list:
        return []

    def num_parameters(self) -> int:
        return 0

    def trainable_params_count(self) -> int:
        return 0

    def set_training(self, training: bool) -> None:
        self._training = bool(training)

    def is_training(self) -> bool:
        return getattr(self, "_training", True)

    def last_kernel(self) -> str:
        return _lib.lib().shrewq_linear_last_kernel(self._h).decode()

    def forward(self, x: torch.Tensor, epilogue: int = _lib.EPILOGUE_NONE, out: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """Module::forward (quantize.rs:463-476).  x is [M, in_features] f32 or bf16 on the
        layer's device; the result has x's dtype.  `out` may be a column slice of a wider
        row-major buffer (last stride 1): the shard-writes-its-slice case."""
        if x.dim() != 2 or x.shape[1] != self.in_features:
            raise ShrewError(_lib.ERR_INVALID_ARG,
                             f"forward: expected x of shape [M,{self.in_features}], got {list(x.shape)}")
        if x.dtype not in _DTYPE_CODE:
            raise ShrewError(_lib.ERR_UNSUPPORTED, f"forward: activation dtype {x.dtype} not supported")
        if x.device.type != "cuda" or x.device.index != self.device.index:
            raise ShrewError(_lib.ERR_INVALID_ARG, "forward: x is not on the layer's device")
        x = x.contiguous()
        M = x.shape[0]
        if out is None:
            out = torch.empty((M, self.out_features), dtype=out_dtype or x.dtype, device=x.device)
        if out.dim() != 2 or out.shape[0] != M or out.shape[1] != self.out_features or (M > 0 and out.stride(1) != 1):
            raise ShrewError(_lib.ERR_INVALID_ARG, "forward: bad output buffer")
        ldy = out.stride(0) if M > 1 else max(out.stride(0), self.out_features)
        self.device.bind_stream()
        rc = _lib.lib().shrewq_linear_forward(self._h, _ptr(x), _DTYPE_CODE[x.dtype], M, _ptr(out),
                                              _DTYPE_CODE[out.dtype], ldy, epilogue)
        _lib.check(rc, self.device.handle)
        return out

    __call__ = forward

    def forward_host(self, x: torch.Tensor, epilogue: int = _lib.EPILOGUE_NONE,
                     out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """The same forward for a caller whose activations live in HOST memory (shrewq_linear_forward_host):
        x is a CPU tensor [M, in_features] of f32 or bf16; the library copies it in, runs the kernel, copies the
        result out and synchronises.  Returns a CPU tensor [M, out_features]."""
        if x.device.type != "cpu" or x.dim() != 2 or x.shape[1] != self.in_features:
            raise ShrewError(_lib.ERR_INVALID_ARG, f"forward_host: expected a CPU tensor [M,{self.in_features}], got {list(x.shape)} on {x.device}")
        if x.dtype not in _DTYPE_CODE:
            raise ShrewError(_lib.ERR_UNSUPPORTED, f"forward_host: activation dtype {x.dtype} not supported")
        x = x.contiguous()
        out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype or x.dtype)
        if out.dtype not in _DTYPE_CODE:
            raise ShrewError(_lib.ERR_UNSUPPORTED, f"forward_host: output dtype {out.dtype} not supported")
        self.device.bind_stream()
        rc = _lib.lib().shrewq_linear_forward_host(self._h, ctypes.c_void_p(x.data_ptr()), _DTYPE_CODE[x.dtype], x.shape[0],
                                                   ctypes.c_void_p(out.data_ptr()), _DTYPE_CODE[out.dtype], epilogue)
        _lib.check(rc, self.device.handle)
        return out

    def forward_gate_up_silu(self, up: "QuantizedLinear", x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """silu(self.forward(x)) * up.forward(x) in one pass over x (self is the gate)."""
        x = x.contiguous()
        M = x.shape[0]
        if out is None:
            out = torch.empty((M, self.out_features), dtype=x.dtype, device=x.device)
        ldh = out.stride(0) if M > 1 else max(out.stride(0), self.out_features)
        self.device.bind_stream()
        rc = _lib.lib().shrewq_linear_forward_gate_up_silu(self._h, up._h, _ptr(x), _DTYPE_CODE[x.dtype], M, _ptr(out),
                                                           _DTYPE_CODE[out.dtype], ldh)
        _lib.check(rc, self.device.handle)
        return out

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            try:
                _lib.lib().shrewq_linear_destroy(h)
            except Exception:
                pass
            self._h = None

    def __repr__(self) -> str:
        return (f"QuantizedLinear(in_features={self.in_features}, out_features={self.out_features}, "
                f"bits={self.weight_q.config.bits.name}, compression={self.weight_q.compression_ratio():.1f}x)")


def mlp_forward_host(gate: "QuantizedLinear", up: "QuantizedLinear", down: "QuantizedLinear", x: torch.Tensor,
                     out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
                     synchronize: bool = True) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)) for HOST activations (shrewq_mlp_forward_host): x is a CPU bf16 tensor
    [M, in_features], the result a CPU tensor [M, down.out_features].  synchronize=False returns once the work is
    enqueued (x and out pinned and left alone until Device.synchronize()); consecutive calls then overlap their
    copies with each other's kernels."""
    if x.device.type != "cpu" or x.dtype is not torch.bfloat16 or x.dim() != 2 or x.shape[1] != gate.in_features:
        raise ShrewError(_lib.ERR_INVALID_ARG, f"mlp_forward_host: expected a CPU bf16 tensor [M,{gate.in_features}]")
    x = x.contiguous()
    if out is None:
        out = torch.empty((x.shape[0], down.out_features), dtype=out_dtype or x.dtype)
    if out.device.type != "cpu" or out.dtype not in _DTYPE_CODE or not out.is_contiguous() or \
            list(out.shape) != [x.shape[0], down.out_features]:
        raise ShrewError(_lib.ERR_INVALID_ARG, "mlp_forward_host: bad output buffer")
    gate.device.bind_stream()
    rc = _lib.lib().shrewq_mlp_forward_host(gate._h, up._h, down._h, _ptr(x), x.shape[0], _ptr(out), _DTYPE_CODE[out.dtype],
                                            1 if synchronize else 0)
    _lib.check(rc, gate.device.handle)
    return out


# ---- model-level helpers (quantize.rs:500-586) ------------------------------------------------------
def quantize_named_parameters(module, config: QuantConfig, batched: bool = True) -> List[Tuple[str, QuantizedTensor]]:
    """Every parameter of rank >= 2 is quantized — including a Linear's [1,out] bias, which
    is rank 2 in Shrew (quantize.rs:507-513, :760-766).  INT8 symmetric f32 parameters go out as one
    batched call (a few launches for the whole model, the same bits); batched=False quantizes tensor by tensor."""
    params = [(name, t.detach()) for name, t in module.named_parameters() if t.dim() >= 2]
    if (batched and config._is_int8_symmetric() and params
            and all(t.dtype is torch.float32 for _, t in params)):
        return list(zip([n for n, _ in params], quantize_tensors([t for _, t in params], config)))
    return [(name, quantize_tensor(t, config)) for name, t in params]


@dataclass
class QuantStats:
    num_quantized: int
    num_fp32: int
    fp32_bytes: int
    quantized_bytes: int
    compression_ratio: float


def quantization_stats(module, config: QuantConfig) -> QuantStats:
    """quantize.rs:534-586 (pure bookkeeping, no device work)."""
    nq = nf = fp32 = qb = 0
    for _, t in module.named_parameters():
        numel = t.numel()
        fp32 += numel * 4
        if t.dim() >= 2:
            nq += 1
            size = numel if config.bits is QuantBits.Int8 else (numel + 1) // 2
            meta = 16 if config.granularity is QuantGranularity.PerTensor else (16 if t.dim() == 0 else t.shape[0] * 16)
            qb += size + meta
        else:
            nf += 1
            qb += numel * 4
    return QuantStats(nq, nf, fp32, qb, (fp32 / qb) if qb > 0 else 1.0)
