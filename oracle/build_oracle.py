"""Compiles the C oracle (oracle/sacq_oracle.c) into oracle/_build/libsacq_oracle.so with
gcc and offers a small ctypes wrapper.  Test infrastructure only.

The reference is a Python package, so there is nothing of it to compile into
``oracle/_ref``; its behaviour is pinned through the fixtures in tests/golden instead.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "sacq_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "libsacq_oracle.so")


def build(force: bool = False) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["gcc", "-O3", "-fopenmp", "-fPIC", "-shared", "-fvisibility=hidden", "-o", LIB, SRC, "-lm"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("gcc failed:\n" + res.stdout + res.stderr)
    return LIB


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.sacq_oracle_threads.restype = ctypes.c_int
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def unpack(packed: np.ndarray, bits: int, count: int) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.empty(count, dtype=np.int32)
    lib().sacq_oracle_unpack(_p(packed), ctypes.c_int64(packed.size), ctypes.c_int(bits), ctypes.c_int64(count), _p(out))
    return out


def dequant(packed, bits, codebook_bits, scales_bits, shift_bits, N, K, G) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    cb = np.ascontiguousarray(codebook_bits, dtype=np.uint16)
    sc = np.ascontiguousarray(scales_bits, dtype=np.uint16)
    out = np.empty((N, K), dtype=np.uint16)
    lib().sacq_oracle_dequant(_p(packed), ctypes.c_int64(packed.size), ctypes.c_int(bits), _p(cb), _p(sc),
                              ctypes.c_uint16(int(shift_bits)), ctypes.c_int64(N), ctypes.c_int64(K),
                              ctypes.c_int(G), ctypes.c_int(cb.shape[1]), _p(out))
    return out


def quant_rows(x_bits: np.ndarray):
    x = np.ascontiguousarray(x_bits, dtype=np.uint16)
    M, K = x.shape
    q = np.empty((M, K), dtype=np.uint8)
    s = np.empty((M, 1), dtype=np.float32)
    lib().sacq_oracle_quant_rows(_p(x), ctypes.c_int64(M), ctypes.c_int64(K), _p(q), _p(s))
    return q, s


def quant_rows_int8(x_bits: np.ndarray):
    x = np.ascontiguousarray(x_bits, dtype=np.uint16)
    M, K = x.shape
    q = np.empty((M, K), dtype=np.int8)
    s = np.empty((M, 1), dtype=np.float32)
    lib().sacq_oracle_quant_rows_int8(_p(x), ctypes.c_int64(M), ctypes.c_int64(K), _p(q), _p(s))
    return q, s


def linear(packed, bits, codebook_bits, scales_bits, shift_bits, bias_bits, N, K, G, q_bits, act_scale) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    cb = np.ascontiguousarray(codebook_bits, dtype=np.uint16)
    sc = np.ascontiguousarray(scales_bits, dtype=np.uint16)
    q = np.ascontiguousarray(q_bits, dtype=np.uint8)
    s = np.ascontiguousarray(act_scale, dtype=np.float32).reshape(-1)
    M = q.shape[0]
    y = np.empty((M, N), dtype=np.float32)
    bias_ptr = _p(np.ascontiguousarray(bias_bits, dtype=np.uint16)) if bias_bits is not None else None
    lib().sacq_oracle_linear(_p(packed), ctypes.c_int64(packed.size), ctypes.c_int(bits), _p(cb), _p(sc),
                             ctypes.c_uint16(int(shift_bits)), bias_ptr, ctypes.c_int64(N), ctypes.c_int64(K),
                             ctypes.c_int(G), ctypes.c_int(cb.shape[1]), _p(q), _p(s), ctypes.c_int64(M), _p(y))
    return y


def threads() -> int:
    return int(lib().sacq_oracle_threads())


def set_threads(n: int) -> None:
    lib().sacq_oracle_set_threads(ctypes.c_int(n))


if __name__ == "__main__":
    print(build(force=True))
