"""The C-ABI library loads without a GPU and exports every symbol that
include/peer_b200.h declares; struct layouts match the header."""
import ctypes as C
import os
import re

import pytest

from llm720_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "peer_b200.h")


def declared_functions():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(peer_[a-z_]+)\s*\(", src)))


def test_header_declares_the_bound_functions():
    assert set(declared_functions()) == set(_lib.EXPORTS)


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    for name in declared_functions():
        assert hasattr(lib, name), name
    assert lib.peer_abi_version() == _lib.ABI_VERSION


def test_struct_layouts_match_header():
    # peer_config_t: int32 x3, int64, int32 x14 (with natural padding), int64, int32 x3 (+ tail padding)
    assert C.sizeof(_lib.PeerConfig) == 104
    assert _lib.PeerConfig.num_experts.offset == 16
    assert _lib.PeerConfig.max_tokens.offset == 80
    assert _lib.PeerConfig.num_key_dims.offset == 88 and _lib.PeerConfig.n_keys3.offset == 96
    assert C.sizeof(_lib.PeerTensors) == 17 * 8
    assert _lib.PeerTensors.keys2.offset == 14 * 8


def test_create_rejects_bad_arguments_without_a_device():
    lib = _lib.load()
    h = C.c_void_p()
    assert lib.peer_create(None, C.byref(h)) == _lib.ERR_INVALID_ARG
    cfg = _lib.PeerConfig(abi_version=99)
    assert lib.peer_create(C.byref(cfg), C.byref(h)) == _lib.ERR_INVALID_ARG
    assert b"abi_version" in lib.peer_last_error(None)
    cfg = _lib.PeerConfig(abi_version=_lib.ABI_VERSION, input_dim=256, output_dim=256, num_experts=16,
                          top_k=4, num_heads=2, query_dim=32, n_keys0=4, n_keys1=4, expert_hidden_size=17,
                          max_tokens=8)
    assert lib.peer_create(C.byref(cfg), C.byref(h)) == _lib.ERR_UNSUPPORTED
    assert b"expert_hidden_size" in lib.peer_last_error(None)
    cfg.expert_hidden_size = 1
    cfg.num_key_dims = 5
    assert lib.peer_create(C.byref(cfg), C.byref(h)) == _lib.ERR_UNSUPPORTED
    assert b"num_key_dims" in lib.peer_last_error(None)
    cfg.num_key_dims = 2
    cfg.n_keys1 = 5
    assert lib.peer_create(C.byref(cfg), C.byref(h)) == _lib.ERR_INVALID_ARG
    assert not h.value


def test_exchange_create_rejects_bad_arguments_without_a_device():
    lib = _lib.load()
    h = C.c_void_p()
    bf16 = _lib.DTYPE_BF16
    assert lib.peer_xchg_create(0, 0, 8, 256, 4096, 4096, bf16, C.byref(h)) == _lib.ERR_INVALID_ARG
    assert lib.peer_xchg_create(2, 2, 8, 256, 4096, 4096, bf16, C.byref(h)) == _lib.ERR_INVALID_ARG
    assert lib.peer_xchg_create(17, 0, 8, 256, 4096, 4096, bf16, C.byref(h)) == _lib.ERR_INVALID_ARG
    assert b"world" in lib.peer_last_error(None)
    assert lib.peer_xchg_create(2, 0, 8, 256, 4097, 4096, bf16, C.byref(h)) == _lib.ERR_UNSUPPORTED
    assert lib.peer_xchg_create(2, 0, 8, 256, 4096, 4096, 9, C.byref(h)) == _lib.ERR_INVALID_ARG
    assert h.value is None
    assert lib.peer_xchg_push_x(None, None, None) == _lib.ERR_INVALID_ARG
    assert lib.peer_xchg_destroy(None) == _lib.OK

