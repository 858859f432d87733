"""ctypes binding of ``libpeer_b200.so`` (the C ABI declared in
``include/peer_b200.h``).  Nothing here computes anything: a missing library
is an error, there is no other code path."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libpeer_b200.so")

ABI_VERSION = 2
OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_DEVICE_TIMEOUT, ERR_BOUNDS = range(6)
DTYPE_F32, DTYPE_BF16, DTYPE_E4M3, DTYPE_F16 = 0, 1, 2, 3
ACT_GELU, ACT_RELU = 0, 1
INDEX_REFERENCE, INDEX_PRODUCT = 0, 1


class PeerConfig(C.Structure):
    _fields_ = [
        ("abi_version", C.c_int32), ("input_dim", C.c_int32), ("output_dim", C.c_int32),
        ("num_experts", C.c_int64), ("top_k", C.c_int32), ("num_heads", C.c_int32),
        ("query_dim", C.c_int32), ("n_keys0", C.c_int32), ("n_keys1", C.c_int32),
        ("expert_hidden_size", C.c_int32), ("activation", C.c_int32), ("norm_keys", C.c_int32),
        ("norm_query", C.c_int32), ("layer_norm", C.c_int32), ("act_dtype", C.c_int32),
        ("table_dtype", C.c_int32), ("index_mode", C.c_int32), ("max_tokens", C.c_int64),
        ("num_key_dims", C.c_int32), ("n_keys2", C.c_int32), ("n_keys3", C.c_int32),
    ]


class PeerTensors(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "x", "query_w", "query_b", "ln_w", "ln_b", "keys0", "keys1", "expert_down", "expert_up",
        "down_scale", "up_scale", "out", "ids_out", "scores_out", "keys2", "keys3", "product_ids_out")]


EXPORTS = {
    "peer_abi_version": (C.c_int, []),
    "peer_create": (C.c_int, [C.POINTER(PeerConfig), C.POINTER(C.c_void_p)]),
    "peer_destroy": (C.c_int, [C.c_void_p]),
    "peer_last_error": (C.c_char_p, [C.c_void_p]),
    "peer_forward": (C.c_int, [C.c_void_p, C.POINTER(PeerTensors), C.c_int64, C.c_void_p]),
    "peer_block_forward": (C.c_int, [C.c_void_p, C.POINTER(PeerTensors), C.c_void_p, C.c_void_p, C.c_float, C.c_int64,
                                     C.c_void_p]),
    "peer_set_row_tier": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "peer_forward_host": (C.c_int, [C.c_void_p, C.POINTER(PeerTensors), C.c_int64]),
    "peer_forward_host_async": (C.c_int, [C.c_void_p, C.POINTER(PeerTensors), C.c_int64, C.POINTER(C.c_int64)]),
    "peer_forward_host_wait": (C.c_int, [C.c_void_p, C.c_int64]),
    "peer_project_queries": (C.c_int, [C.c_void_p, C.POINTER(PeerTensors), C.c_int64, C.c_void_p, C.c_void_p]),
    "peer_select": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p,
                              C.c_void_p, C.c_void_p]),
    "peer_select_tokens": (C.c_int, [C.c_void_p, C.POINTER(PeerTensors), C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "peer_route_tuples": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int64, C.c_int32, C.c_void_p,
                                    C.c_void_p]),
    "peer_gather_eval_routed": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_void_p, C.c_void_p,
                                          C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "peer_select_stats": (C.c_int, [C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.c_void_p]),
    "peer_select_nd": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p), C.c_int64, C.c_void_p, C.c_void_p,
                                 C.c_void_p]),
    "peer_select_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p), C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_int64, C.c_void_p, C.c_void_p]),
    "peer_select_noalloc": (C.c_int, [C.POINTER(PeerConfig), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p,
                                      C.c_void_p, C.c_void_p]),
    "peer_gather_eval": (C.c_int, [C.c_void_p] * 9 + [C.c_int64, C.c_void_p]),
    "peer_gather_eval_partial": (C.c_int, [C.c_void_p] * 5 + [C.c_int32] + [C.c_void_p] * 4 + [C.c_int64, C.c_void_p,
                                                                                           C.c_int64, C.c_void_p]),
    "peer_gather_eval_backward": (C.c_int, [C.c_void_p] * 11 + [C.c_int32, C.c_int64, C.c_void_p]),
    "peer_gather_eval_backward_rows": (C.c_int, [C.c_void_p] * 11 + [C.c_int32, C.c_int64, C.c_int64, C.c_void_p]),
    "peer_xchg_create": (C.c_int, [C.c_int32, C.c_int32, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                   C.POINTER(C.c_void_p)]),
    "peer_xchg_export": (C.c_int, [C.c_void_p, C.c_void_p]),
    "peer_xchg_attach": (C.c_int, [C.c_void_p, C.c_void_p]),
    "peer_xchg_push_x": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "peer_xchg_route": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "peer_xchg_wait_inputs": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_void_p]),
    "peer_xchg_combine": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "peer_xchg_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(PeerTensors), C.c_void_p, C.c_void_p, C.c_int64,
                                    C.c_void_p, C.c_void_p, C.c_void_p]),
    "peer_xchg_counts": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "peer_xchg_status": (C.c_int, [C.c_void_p, C.c_void_p]),
    "peer_xchg_destroy": (C.c_int, [C.c_void_p]),
    "peer_usage_histogram": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "peer_query_status": (C.c_int, [C.c_void_p, C.c_void_p]),
    "peer_launch_count": (C.c_int64, [C.c_void_p]),
    "peer_freeze_keys": (C.c_int, [C.c_void_p, C.c_int]),
    "peer_stage_timing": (C.c_int, [C.c_void_p, C.c_int]),
    "peer_stage_times": (C.c_int, [C.c_void_p, C.POINTER(C.c_double), C.POINTER(C.c_int64)]),
}

_lib = None


def load() -> C.CDLL:
    """Load the library once.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m llm720_b200.build` "
                "(needs nvcc; the library targets sm_100a).  There is no fallback path.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in EXPORTS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        if lib.peer_abi_version() != ABI_VERSION:
            raise RuntimeError("libpeer_b200.so was built from a different ABI version; rebuild it")
        _lib = lib
    return _lib


def last_error(handle) -> str:
    msg = load().peer_last_error(handle)
    return msg.decode() if msg else ""


def check(rc: int, handle=None) -> None:
    """Raise the Python exception matching a non-zero return code."""
    if rc == OK:
        return
    msg = last_error(handle)
    if rc in (ERR_INVALID_ARG, ERR_UNSUPPORTED):
        raise ValueError(f"peer_b200: {msg}")
    raise RuntimeError(f"peer_b200 (code {rc}): {msg}")
