"""ctypes binding of ``libsacq_b200.so`` (the C ABI declared in include/sacq_b200.h).

There is no CPU or PyTorch fallback: if the shared library is missing or does not
load, importing the bound functions raises, and every product entry point fails.
"""
from __future__ import annotations

import ctypes
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libsacq_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(HERE), "include", "sacq_b200.h")

SACQ_OK = 0
SACQ_PACKED_GUARD_BYTES = 16
ERROR_NAMES = {
    -1: "SACQ_ERR_INVALID_ARGUMENT", -2: "SACQ_ERR_UNSUPPORTED", -3: "SACQ_ERR_ALIGNMENT",
    -4: "SACQ_ERR_WORKSPACE", -5: "SACQ_ERR_CUDA", -6: "SACQ_ERR_DEVICE_TIMEOUT",
}


class SacqError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"{ERROR_NAMES.get(code, code)}: {message}")
        self.code = code


class LayerDesc(ctypes.Structure):
    _fields_ = [
        ("struct_size", ctypes.c_uint32),
        ("device", ctypes.c_int32),
        ("out_features", ctypes.c_int64),
        ("in_features", ctypes.c_int64),
        ("group_size", ctypes.c_int32),
        ("vector_dim", ctypes.c_int32),
        ("codebook_size", ctypes.c_int32),
        ("index_bits", ctypes.c_int32),
        ("packed", ctypes.c_void_p),
        ("packed_bytes", ctypes.c_int64),
        ("codebook", ctypes.c_void_p),
        ("scales", ctypes.c_void_p),
        ("bias", ctypes.c_void_p),
        ("shift_bf16", ctypes.c_uint16),
        ("reserved0", ctypes.c_uint16),
        ("reserved1", ctypes.c_uint32),
    ]


_vp, _i64, _int = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
_fp = ctypes.c_void_p  # float* passed as a raw device address

# name -> (restype, argtypes); must list every function include/sacq_b200.h declares
SIGNATURES = {
    "sacq_layer_create": (_int, [ctypes.POINTER(LayerDesc), ctypes.POINTER(_vp)]),
    "sacq_layer_destroy": (_int, [_vp]),
    "sacq_layer_resident_bytes": (_i64, [_vp]),
    "sacq_dequant_bf16": (_int, [_vp, _vp, _vp]),
    "sacq_quant_act_fp8": (_int, [_vp, _i64, _i64, _i64, _vp, _fp, _vp]),
    "sacq_quant_act_int8": (_int, [_vp, _i64, _i64, _i64, _vp, _fp, _vp]),
    "sacq_workspace_bytes_int8": (_i64, [_vp, _i64]),
    "sacq_linear_a8i": (_int, [_vp, _vp, _fp, _i64, _vp, _i64, _vp, _i64, _vp]),
    "sacq_layernorm_quant_fp8": (_int, [_vp, _i64, _vp, _vp, ctypes.c_float, _vp, _vp, _i64, _i64, _vp, _i64, _vp, _fp,
                                        _vp]),
    "sacq_modulate_quant_fp8": (_int, [_vp, _i64, _vp, _vp, _i64, _i64, _vp, _fp, _vp]),
    "sacq_act_quant_fp8": (_int, [_int, _vp, _i64, _vp, _i64, _i64, _i64, _vp, _fp, _vp]),
    "sacq_weight_row_scale": (_int, [_vp, _fp, _vp]),
    "sacq_decode_weight_fp8": (_int, [_vp, _fp, _vp, _vp]),
    "sacq_weight_row_scale_int8": (_int, [_vp, _fp, _vp]),
    "sacq_decode_weight_int8": (_int, [_vp, _fp, _vp, _vp]),
    "sacq_workspace_bytes_w8a8": (_i64, [_vp, _i64]),
    "sacq_linear_w8a8_int8": (_int, [_vp, _vp, _fp, _fp, _i64, _vp, _i64, _vp, _i64, _vp]),
    "sacq_linear_w8a8_fp8": (_int, [_vp, _vp, _fp, _fp, _i64, _vp, _i64, _vp, _i64, _vp]),
    "sacq_workspace_bytes": (_i64, [_vp, _i64]),
    "sacq_workspace_counter_bytes": (_i64, []),
    "sacq_linear_a8": (_int, [_vp, _vp, _fp, _i64, _vp, _i64, _vp, _i64, _vp]),
    "sacq_linear_a8_residual": (_int, [_vp, _vp, _fp, _i64, _vp, _i64, _vp, _i64, _vp, _i64, _vp]),
    "sacq_linear_a8_bcast": (_int, [_vp, _vp, _fp, _i64, _vp, ctypes.POINTER(_vp), _int, _i64, _vp, _i64, _vp]),
    "sacq_peer_buffer_create": (_int, [_int, _i64, ctypes.POINTER(_vp), _vp]),
    "sacq_peer_buffer_open": (_int, [_int, _vp, ctypes.POINTER(_vp)]),
    "sacq_peer_buffer_close": (_int, [_int, _vp]),
    "sacq_peer_buffer_destroy": (_int, [_int, _vp]),
    "sacq_linear_a8_multi": (_int, [ctypes.POINTER(_vp), _int, _vp, _fp, _i64, ctypes.POINTER(_vp),
                                    ctypes.POINTER(_i64), _vp, _i64, _vp]),
    "sacq_linear_bf16": (_int, [_vp, _vp, _i64, _i64, _vp, _fp, _vp, _i64, _vp, _i64, _vp]),
    "sacq_linear_bf16_host": (_int, [_vp, _vp, _i64, _vp, _vp, _i64, _vp]),
    "sacq_host_forward_scratch_bytes": (_i64, [_vp, _i64]),
    "sacq_linear_a8_static_scratch": (_int, [_vp, _vp, _fp, _i64, _vp, _i64, _vp]),
    "sacq_static_scratch_bytes": (_i64, []),
    "sacq_layer_set_kernel": (_int, [_vp, _int]),
    "sacq_layer_kernel_for": (_int, [_vp, _i64]),
    "sacq_layer_status": (_int, [_vp, ctypes.POINTER(_int)]),
    "sacq_launch_count": (_i64, []),
    "sacq_last_error": (ctypes.c_char_p, []),
    "sacq_abi_version": (_int, []),
}

_lib = None


def declared_symbols() -> list[str]:
    """Function names the public header declares (parsed from the header text)."""
    with open(HEADER_PATH) as f:
        text = f.read()
    return sorted(set(re.findall(r"SACQ_API\s+[\w\s\*]+?\b(sacq_\w+)\s*\(", text)))


def load() -> ctypes.CDLL:
    """Load the shared library (once) and attach prototypes.  Raises if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing. Build it with `python -m sacq_b200.build` (needs nvcc); "
            "sacq_b200 has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)           # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    if lib.sacq_abi_version() != 1:
        raise ImportError("libsacq_b200.so ABI version mismatch")
    _lib = lib
    return lib


def last_error() -> str:
    return load().sacq_last_error().decode("utf-8", "replace")


def check(code: int) -> None:
    if code != SACQ_OK:
        raise SacqError(code, last_error())
