"""ctypes binding of libshrewq.so (the C ABI declared in include/shrewq.h).

The library is the product; this module only loads it and declares the signatures.  There
is no fallback: if the shared object is missing the import of any compute path fails, and
on a machine without a B200 every compute call returns SHREWQ_ERR_NO_DEVICE.
"""
from __future__ import annotations

import ctypes
import os

OK = 0
ERR_INVALID_ARG, ERR_CUDA, ERR_UNSUPPORTED, ERR_NO_DEVICE, ERR_TIMEOUT, ERR_ALLOC = -1, -2, -3, -4, -5, -6
PER_TENSOR, PER_CHANNEL = 0, 1
SYMMETRIC, ASYMMETRIC = 0, 1
F32, BF16, F16, F64 = 0, 1, 2, 3
EPILOGUE_NONE, EPILOGUE_RELU = 0, 1
EXCHANGE_FLAG_BYTES = 256

# SHREWQ_LIB points at another build of the same library (e.g. the tracing build)
LIB_PATH = os.environ.get("SHREWQ_LIB") or os.path.join(os.path.dirname(os.path.abspath(__file__)), "libshrewq.so")

# every symbol include/shrewq.h declares, with (restype, argtypes)
_vp, _sz, _ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
_pp = ctypes.POINTER(ctypes.c_void_p)
SIGNATURES = {
    "shrewq_ctx_create": (_ci, [_ci, _vp, _pp]),
    "shrewq_ctx_set_stream": (_ci, [_vp, _vp]),
    "shrewq_ctx_set_option": (_ci, [_vp, ctypes.c_char_p, _ci]),
    "shrewq_ctx_synchronize": (_ci, [_vp]),
    "shrewq_ctx_destroy": (None, [_vp]),
    "shrewq_last_error": (ctypes.c_char_p, [_vp]),
    "shrewq_version": (ctypes.c_char_p, []),
    "shrewq_quantize_f32": (_ci, [_vp, _vp, _sz, _sz, _ci, _vp, _vp]),
    "shrewq_quantize_f32_batch": (_ci, [_vp, _vp, _sz, _ci]),
    "shrewq_quantize_f32_host": (_ci, [_vp, _vp, _sz, _sz, _ci, _vp, _vp]),
    "shrewq_dequantize": (_ci, [_vp, _vp, _vp, _sz, _sz, _ci, _ci, _vp]),
    "shrewq_absmax_f32": (_ci, [_vp, _vp, _sz, _vp]),
    "shrewq_quantize_f32_given_amax": (_ci, [_vp, _vp, _sz, _vp, _vp, _vp]),
    "shrewq_quantize_f32_ex": (_ci, [_vp, _vp, _sz, _sz, _ci, _ci, _ci, _vp, _vp, _vp]),
    "shrewq_quantize_any": (_ci, [_vp, _vp, _ci, _sz, _sz, _ci, _ci, _ci, _vp, _vp, _vp]),
    "shrewq_dequantize_ex": (_ci, [_vp, _vp, _vp, _vp, _sz, _sz, _ci, _ci, _vp]),
    "shrewq_linear_create": (_ci, [_vp, _vp, _vp, _vp, _sz, _sz, _ci, _pp]),
    "shrewq_pack_int4": (_ci, [_vp, _vp, _sz, _sz, _vp]),
    "shrewq_linear_create_int4": (_ci, [_vp, _vp, _vp, _vp, _sz, _sz, _ci, _pp]),
    "shrewq_linear_create_ex": (_ci, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _ci, _pp]),
    "shrewq_linear_destroy": (None, [_vp]),
    "shrewq_linear_forward": (_ci, [_vp, _vp, _ci, _sz, _vp, _ci, _sz, _ci]),
    "shrewq_linear_forward_host": (_ci, [_vp, _vp, _ci, _sz, _vp, _ci, _ci]),
    "shrewq_mlp_forward_host": (_ci, [_vp, _vp, _vp, _vp, _sz, _vp, _ci, _ci]),
    "shrewq_linear_forward_noalloc": (_ci, [_vp, _vp, _sz, _vp, _ci, _sz, _ci]),
    "shrewq_linear_forward_peers": (_ci, [_vp, _vp, _vp, _ci, _sz, _vp, _pp, _ci, _ci, _sz, _ci]),
    "shrewq_linear_forward_gate_up_silu": (_ci, [_vp, _vp, _vp, _ci, _sz, _vp, _ci, _sz]),
    "shrewq_exchange_create": (_ci, [_vp, _ci, _ci, _pp, _pp]),
    "shrewq_exchange_barrier": (_ci, [_vp]),
    "shrewq_exchange_destroy": (None, [_vp]),
    "shrewq_linear_in_features": (_sz, [_vp]),
    "shrewq_linear_out_features": (_sz, [_vp]),
    "shrewq_linear_memory_savings_bytes": (_sz, [_vp]),
    "shrewq_linear_last_kernel": (ctypes.c_char_p, [_vp]),
    "shrewq_force_kernel": (_ci, [ctypes.c_char_p]),
    "shrewq_ctx_launch_count": (ctypes.c_uint64, [_vp]),
    "shrewq_plan_forward": (_ci, [_sz, _sz, _sz, _ci, _ci, _ci, ctypes.c_char_p, _sz, ctypes.POINTER(_ci), ctypes.POINTER(_ci),
                                 ctypes.POINTER(_ci), ctypes.POINTER(_ci), ctypes.POINTER(_ci)]),
}

class QuantItem(ctypes.Structure):
    """shrewq_quant_item: one tensor of shrewq_quantize_f32_batch."""
    _fields_ = [("w_dev", ctypes.c_void_p), ("rows", ctypes.c_size_t), ("cols", ctypes.c_size_t),
                ("q_dev", ctypes.c_void_p), ("scales_dev", ctypes.c_void_p)]


_lib = None


class ShrewError(RuntimeError):
    """Mirror of shrew_core::Error: carries the status code and the library's message."""

    def __init__(self, code: int, message: str):
        super().__init__(f"shrewq error {code}: {message}")
        self.code = code
        self.message = message


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m shrew_b200.build` "
                "(there is no CPU or PyTorch fallback for this path)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc: int, ctx=None) -> None:
    if rc != OK:
        msg = lib().shrewq_last_error(ctx)
        raise ShrewError(rc, msg.decode() if msg else "")
