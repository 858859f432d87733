"""peer_select_noalloc — the handle-free selection entry point for callers that may not allocate
device memory (servers that gave the whole GPU to their own pool, latency-critical loops).  Its
scratch is an array inside the library, so this test checks, through the C ABI, that it returns
exactly what the handle-based peer_select returns, on two calls in a row that reuse that array,
and that an oversized call is refused instead of overrunning it.

Collected last on purpose: a failure here cannot hide another test's result under `-x`.
"""
import ctypes as C

import pytest
import torch

from llm720_b200 import _lib, synthetic as syn
from oracle import peer_oracle as orc
from _util import make_op

pytestmark = pytest.mark.gpu


def _cfg_struct(op):
    return op.cfg        # the same peer_config_t the handle was created from


def _noalloc(lib, cfg, q, k0, k1):
    T = q.shape[0]
    ids = torch.empty(T, cfg.num_heads, cfg.top_k, dtype=torch.int64, device=q.device)
    sc = torch.empty(T, cfg.num_heads, cfg.top_k, dtype=torch.float32, device=q.device)
    rc = lib.peer_select_noalloc(C.byref(cfg), C.c_void_p(q.data_ptr()), C.c_void_p(k0.data_ptr()),
                                 C.c_void_p(k1.data_ptr()), T, C.c_void_p(ids.data_ptr()),
                                 C.c_void_p(sc.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, ids, sc


@pytest.mark.parametrize("mode", ["reference", "product"])
def test_noalloc_select_equals_handle_select_twice(cuda_device, mode):
    lib = _lib.load()
    torch.manual_seed(7)
    T, H, Q, n, k = 150, 4, 128, 128, 8
    pc = syn.PeerConfig("na", 64, 64, H, Q, (n, n), k, torch.float32, torch.float32, 1, T)
    op = make_op(pc, cuda_device, mode)
    for call in range(2):                      # the second call reuses the built-in scratch array
        q = torch.randn(T - 37 * call, H, Q, device=cuda_device)
        k0 = torch.randn(n, Q // 2, device=cuda_device)
        k1 = torch.randn(n, Q // 2, device=cuda_device)
        want_ids, want_sc = op.select(q, k0, k1)
        rc, ids, sc = _noalloc(lib, _cfg_struct(op), q, k0, k1)
        assert rc == _lib.OK, _lib.last_error(None)
        torch.cuda.synchronize()
        assert torch.equal(ids, want_ids)      # same kernels, same inputs: bit-identical
        assert torch.equal(sc, want_sc)
        # and directly against the oracle's selection (experts.py:138-285 restated), near ties aside
        with torch.no_grad():
            o_ids, o_sc = orc.select(q.cpu().unsqueeze(0), [k0.cpu(), k1.cpu()], k, (n, n), index_mode=mode)
        rows, exact, near, bad = orc.compare_selection(ids.cpu(), o_ids.view(ids.shape), o_sc.view(sc.shape), sc.cpu())
        assert bad == 0 and exact >= 0.99 * rows
        assert torch.allclose(sc.cpu(), o_sc.view(sc.shape), rtol=0, atol=3e-6)


def test_noalloc_select_refuses_what_does_not_fit(cuda_device):
    lib = _lib.load()
    pc = syn.PeerConfig("na", 64, 64, 8, 256, (1024, 1024), 16, torch.float32, torch.float32, 1, 4)
    op = make_op(pc, cuda_device)
    # 2000 tokens x 8 heads x 256 floats = 16 MB > the 8 MiB array: must be refused before any launch
    q = torch.zeros(2000, 8, 256, device=cuda_device)
    k = torch.zeros(1024, 128, device=cuda_device)
    rc, _, _ = _noalloc(lib, _cfg_struct(op), q, k, k)
    assert rc == _lib.ERR_UNSUPPORTED
    msg = _lib.last_error(None)
    assert "scratch" in msg and str(8 << 20) in msg
    torch.cuda.synchronize()
