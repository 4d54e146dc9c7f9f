"""ctypes binding of libtqb200.so — the only way Python reaches the CUDA kernels.

There is deliberately no fallback: if the shared library is missing or cannot be loaded
the import of any GPU entry point raises, instead of silently running something else.
"""

from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtqb200.so")

TQ_OK = 0
TQ_F32, TQ_F16, TQ_BF16 = 0, 1, 2

ERRORS = {
    -1: "TQ_ERR_INVALID",
    -2: "TQ_ERR_UNSUPPORTED",
    -3: "TQ_ERR_CUDA",
    -4: "TQ_ERR_CAPACITY",
    -5: "TQ_ERR_EMPTY",
    -6: "TQ_ERR_NO_DEVICE",
}


class TqGeom(C.Structure):
    _fields_ = [
        ("n_layers", C.c_int32), ("n_seqs", C.c_int32), ("n_kv_heads", C.c_int32),
        ("n_q_heads", C.c_int32), ("head_dim", C.c_int32), ("key_bits", C.c_int32),
        ("value_bits", C.c_int32), ("hot_window", C.c_int32), ("kv_dtype", C.c_int32),
        ("max_tokens_per_seq", C.c_int32), ("key_mode", C.c_int32),
        ("outlier_frac", C.c_double),
        ("group", C.c_int32), ("block_tokens", C.c_int32), ("block_tokens_pad", C.c_int32),
        ("hot_cap", C.c_int32), ("max_blocks", C.c_int32), ("outlier_k", C.c_int32),
        ("k_bytes", C.c_int32), ("v_bytes", C.c_int32), ("v_off", C.c_int32),
        ("norm_off", C.c_int32), ("scale_off", C.c_int32), ("mean_off", C.c_int32),
        ("page_bytes", C.c_int32), ("pool_entries", C.c_int32), ("max_splits", C.c_int32),
        ("hdr_off", C.c_int32), ("ent_off", C.c_int32), ("reserved_", C.c_int32),
    ]


REGIONS = ("pages", "hot_k", "hot_v", "pool_dec", "pool_val", "page_meta", "state", "tables",
           "scratch")


class TqSizes(C.Structure):
    _fields_ = [(n, C.c_size_t) for n in REGIONS]


class TqBuffers(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in REGIONS]


# every exported symbol of include/tqb200.h with its signature
SIGNATURES = {
    "tq_version": (C.c_int32, []),
    "tq_last_error": (C.c_char_p, []),
    "tq_geom_finish": (C.c_int32, [C.POINTER(TqGeom)]),
    "tq_ctx_sizes": (C.c_int32, [C.POINTER(TqGeom), C.POINTER(TqSizes)]),
    "tq_ctx_create": (C.c_int32, [C.POINTER(TqGeom), C.POINTER(TqBuffers), C.c_int32,
                                  C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                  C.POINTER(C.c_void_p)]),
    "tq_ctx_destroy": (C.c_int32, [C.c_void_p]),
    "tq_append": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                              C.c_void_p, C.c_int32, C.c_int64, C.c_int64, C.c_int64,
                              C.c_void_p]),
    "tq_decode": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p,
                              C.c_void_p]),
    "tq_decode_static_scratch": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32,
                                             C.c_void_p, C.c_void_p]),
    "tq_decode_partial": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int32,
                                      C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "tq_lse_combine": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                   C.c_void_p]),
    "tq_xchg_create": (C.c_int32, [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                   C.POINTER(C.c_void_p)]),
    "tq_xchg_destroy": (C.c_int32, [C.c_void_p]),
    "tq_xchg_region_bytes": (C.c_int64, [C.c_void_p]),
    "tq_xchg_base": (C.c_void_p, [C.c_void_p]),
    "tq_xchg_ipc_handle": (C.c_int32, [C.c_void_p, C.c_void_p]),
    "tq_xchg_open_peer": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p]),
    "tq_xchg_set_peer": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p]),
    "tq_xchg_gather_merge": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                         C.c_void_p]),
    "tq_decode_exchange": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_int32, C.c_int32,
                                       C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32,
                                       C.c_void_p]),
    "tq_xchg_set_wait_limit": (C.c_int32, [C.c_void_p, C.c_int32]),
    "tq_xchg_status": (C.c_int32, [C.c_void_p, C.POINTER(C.c_int32), C.c_void_p]),
    "tq_dequant_range": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                     C.c_void_p, C.c_void_p, C.c_void_p]),
    "tq_export_block": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                    C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                    C.POINTER(C.c_int32), C.c_void_p, C.c_void_p, C.c_void_p]),
    "tq_import_block": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                    C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                    C.c_void_p, C.c_void_p, C.c_void_p]),
    "tq_restore_hot": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                   C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "tq_seq_lengths": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_int32),
                                   C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "tq_memory_stats": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_double),
                                    C.POINTER(C.c_double), C.c_void_p]),
    "tq_clear": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]),
    "tq_status": (C.c_int32, [C.c_void_p, C.POINTER(C.c_int32), C.c_void_p]),
    "tq_set_value_encoder": (C.c_int32, [C.c_int32]),
    "tq_decode_bytes": (C.c_int32, [C.c_void_p, C.c_int32, C.POINTER(C.c_double)]),
    "tq_last_launches": (C.c_int32, [C.c_void_p]),
    "tq_set_kernel": (C.c_int32, [C.c_void_p, C.c_int32]),
    "tq_last_kernel": (C.c_int32, [C.c_void_p]),
    "tq_debug_wait": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int32]),
    "tq_set_key_mean_mask": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "tq_set_key_bias_means": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "tq_debug_trace": (C.c_int32, [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "tq_profile_enable": (C.c_int32, [C.c_void_p, C.c_int32]),
    "tq_profile_read": (C.c_int32, [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_double),
                                    C.POINTER(C.c_int32)]),
}

_lib = None


def load():
    """Load libtqb200.so (once) and attach the signatures.  Raises if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python turboquant-pro_b200/build.py` "
            "(there is no CPU or pure-PyTorch fallback for the GPU path)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if lib.tq_version() != 100:
        raise RuntimeError("libtqb200.so does not match this package (version mismatch)")
    _lib = lib
    return lib


class TqError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"{ERRORS.get(code, code)}: {msg}")
        self.code = code


def check(code: int) -> None:
    """Turn a status code into the exception the reference API would raise."""
    if code == TQ_OK:
        return
    msg = load().tq_last_error().decode(errors="replace")
    if code == -1:
        raise ValueError(msg)
    if code == -2:
        raise NotImplementedError(msg)
    raise TqError(code, msg)
