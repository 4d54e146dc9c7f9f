"""ctypes binding of the C restatement (oracle/tq_oracle.c).  TEST INFRASTRUCTURE:
only tests/, __graft_entry__.smoke() and bench.py's CPU legs may import this."""

from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libtq_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the C oracle with the Makefile beside it; returns the library path."""
    src = os.path.join(_HERE, "tq_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE])
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        _lib.tqo_encode_keys.restype = C.c_int
        _lib.tqo_num_threads.restype = C.c_int
    return _lib


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t))


def encode_keys(x: np.ndarray, k_out: int):
    """x (H,S,D) float32 -> dict like tq_oracle.encode_keys."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    h, s, d = x.shape
    codes = np.empty((h, s, d), np.uint8)
    scale = np.empty((h, d), np.float32)
    mean = np.empty((h, d), np.float32)
    cap = h * s * d
    oi = np.empty(cap, np.int32)
    ov = np.empty(cap, np.uint16)
    n = lib().tqo_encode_keys(_p(x, C.c_float), h, s, d, int(k_out), _p(codes, C.c_uint8),
                              _p(scale, C.c_float), _p(mean, C.c_float), _p(oi, C.c_int32),
                              _p(ov, C.c_uint16), cap)
    assert n >= 0
    return {"codes": codes, "scale": scale, "mean": mean,
            "out_idx": oi[:n].copy() if k_out > 0 else None,
            "out_val": ov[:n].copy().view(np.float16) if k_out > 0 else None}


def encode_values(x: np.ndarray, pi_t: np.ndarray, bnd: np.ndarray):
    x = np.ascontiguousarray(x, dtype=np.float32)
    h, s, d = x.shape
    pi_t = np.ascontiguousarray(pi_t, dtype=np.float32)
    bnd = np.ascontiguousarray(bnd, dtype=np.float32)
    codes = np.empty((h, s, d), np.uint8)
    norms = np.empty((h, s), np.float32)
    lib().tqo_encode_values(_p(x, C.c_float), h, s, d, _p(pi_t, C.c_float), _p(bnd, C.c_float),
                            int(bnd.size), _p(codes, C.c_uint8), _p(norms, C.c_float))
    return {"codes": codes, "norms": norms}


def dequant_keys(codes, scale, mean, out_idx=None, out_val=None):
    h, s, d = codes.shape
    out = np.empty((h, s, d), np.float32)
    n = 0 if out_idx is None else int(out_idx.size)
    oi = np.zeros(1, np.int32) if n == 0 else np.ascontiguousarray(out_idx, np.int32)
    ov = np.zeros(1, np.uint16) if n == 0 else np.ascontiguousarray(out_val).view(np.uint16)
    lib().tqo_dequant_keys(_p(np.ascontiguousarray(codes), C.c_uint8),
                           _p(np.ascontiguousarray(scale, np.float32), C.c_float),
                           _p(np.ascontiguousarray(mean, np.float32), C.c_float), h, s, d,
                           _p(oi, C.c_int32), _p(ov, C.c_uint16), n, _p(out, C.c_float))
    return out


def dequant_values(codes, norms, cent, pi):
    h, s, d = codes.shape
    out = np.empty((h, s, d), np.float32)
    lib().tqo_dequant_values(_p(np.ascontiguousarray(codes), C.c_uint8),
                             _p(np.ascontiguousarray(norms, np.float32), C.c_float), h, s, d,
                             _p(np.ascontiguousarray(cent, np.float32), C.c_float),
                             _p(np.ascontiguousarray(pi, np.float32), C.c_float),
                             _p(out, C.c_float))
    return out


def attention(q, k, v):
    q = np.ascontiguousarray(q, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    hq, d = q.shape
    hkv, s, _ = k.shape
    out = np.empty((hq, d), np.float32)
    lib().tqo_attention(_p(q, C.c_float), _p(k, C.c_float), _p(v, C.c_float), hq, hkv, s, d,
                        _p(out, C.c_float))
    return out


def num_threads() -> int:
    return int(lib().tqo_num_threads())
