"""ctypes binding of libhashattn.so: the structs and prototypes of include/hashattn.h.

There is no fallback: if the library is missing or does not export a symbol of the header,
importing the ops fails with an error that says how to build it.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_float, c_int, c_int32, c_size_t, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libhashattn.so")

HA_OK = 0
HA_ERR_BAD_ARG = 1
HA_ERR_UNSUPPORTED_DIM = 2
HA_ERR_WORKSPACE = 3
HA_ERR_LAUNCH = 4
HA_ERR_TIMEOUT = 5
HA_ERR_BAD_PAGE = 6
HA_ERR_BAD_SEQ_LEN = 7
HA_ERR_SEL_OVERFLOW = 8
HA_ERR_SCRATCH_LIMIT = 9
HA_WEIGHTS_BF16 = 0
HA_WEIGHTS_F32 = 1
HA_ABI_VERSION = 5
HA_HASH_LSH = -1  # ha_hash_weights_t.num_layers of the LSH baseline
HA_EVAL_SIMPLE = 0
HA_EVAL_DEPTH = 1
HA_OPT_CLUSTER_GATHER = 0
HA_OPT_CLUSTER_SELECT = 1
HA_OPT_PLAN_HANDOVER = 2


class HaShape(ctypes.Structure):
    _fields_ = [
        ("batch", c_int32), ("num_kv_heads", c_int32), ("gqa_group", c_int32), ("head_dim", c_int32),
        ("page_size", c_int32), ("max_pages", c_int32), ("num_pages", c_int32), ("sel_stride", c_int32),
    ]


class HaBudget(ctypes.Structure):
    _fields_ = [("init_budget", c_int32), ("recent_budget", c_int32), ("heavy_budget", c_double),
                ("eval_mode", c_int32), ("retrieve_depth", c_int32)]


class HaHashWeights(ctypes.Structure):
    _fields_ = [("wq", c_void_p), ("bq", c_void_p), ("wk", c_void_p), ("bk", c_void_p), ("dtype", c_int32),
                ("num_layers", c_int32), ("lsh_state", c_void_p)]


_P = c_void_p
_S, _B, _W = POINTER(HaShape), POINTER(HaBudget), POINTER(HaHashWeights)

# name -> (restype, argtypes); one entry per function declared in include/hashattn.h
PROTOTYPES = {
    "ha_abi_version": (c_int, []),
    "ha_status_str": (c_char_p, [c_int]),
    "ha_set_option": (c_int, [c_int, c_int]),
    "ha_get_option": (c_int, [c_int]),
    "ha_workspace_bytes": (c_size_t, [_S, _B]),
    "ha_workspace_init": (c_int, [_S, _B, _P, c_size_t, _P]),
    "ha_hash_decode": (c_int, [_S, _W, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "ha_hash_prefill": (c_int, [_S, _W, _P, _P, _P, _P, _P, _P, _P]),
    "ha_score_select": (c_int, [_S, _B, _P, _P, _P, _P, _P, _P, _P, _P, c_size_t, _P, _P]),
    "ha_static_scratch_needed": (c_size_t, [_S]),
    "ha_decode_step_launches": (c_int, [_S, _B]),
    "ha_decode_step_path": (c_char_p, [_S, _B]),
    "ha_score_plan": (c_int, [_S, _B, _P, _P, _P, _P, _P, _P, c_size_t, _P, _P]),
    "ha_select_attend": (c_int, [_S, _B, _P, _P, _P, _P, _P, _P, c_float, _P, _P, c_size_t, _P, _P]),
    "ha_score_select_static": (c_int, [_S, _B, _P, _P, _P, _P, _P, _P, _P, _P]),
    "ha_sparse_decode": (c_int, [_S, _B, _P, _P, _P, _P, _P, _P, _P, c_float, _P, _P, c_size_t, _P, _P]),
    "ha_decode_step": (c_int, [_S, _B, _W, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_float, _P, _P,
                               c_size_t, _P, _P]),
    "ha_decode_step_rows": (c_int, [_S, _B, _W, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_float, _P, _P,
                                    c_size_t, _P, _P]),
    "ha_rope_split": (c_int, [_P, _P, c_int32, c_int32, c_int32, c_float, _P, _P, _P, _P]),
    "ha_decode_step_host": (c_int, [_S, _B, _W, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
                                    _P, _P, _P, c_float, _P, c_size_t, _P, _P, c_int]),
}

_lib = None


class HashAttnLibraryError(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """Loads libhashattn.so once and attaches the prototypes. Raises if it cannot."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise HashAttnLibraryError(
            f"{LIB_PATH} is missing. Build it with `python {os.path.join(HERE, 'build.py')}` "
            "(needs nvcc; there is no CPU or PyTorch fallback for these kernels)."
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in PROTOTYPES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise HashAttnLibraryError(f"{LIB_PATH} does not export {name}; rebuild it") from e
        fn.restype = restype
        fn.argtypes = argtypes
    if lib.ha_abi_version() != HA_ABI_VERSION:
        raise HashAttnLibraryError(
            f"{LIB_PATH} has ABI version {lib.ha_abi_version()}, this package expects {HA_ABI_VERSION}"
        )
    _lib = lib
    return lib


def status_str(code: int) -> str:
    return load().ha_status_str(int(code)).decode()
