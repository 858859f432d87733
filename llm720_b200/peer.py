"""Drop-in ``PEER`` module and operator wrapper over the CUDA library.

``PEER`` has the constructor, parameter names/shapes (so state-dicts load
both ways), ``forward(hidden_states)`` signature and output shape of the
reference module (llm/models/experts.py:37-440).  The forward pass runs
entirely in the sm_100a kernels behind ``libpeer_b200.so``; there is no
PyTorch or CPU implementation behind it, and anything the kernels do not
implement raises.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import List, Optional, Tuple

import torch
import torch.nn as nn

from . import _lib

_DT = {torch.float32: _lib.DTYPE_F32, torch.bfloat16: _lib.DTYPE_BF16,
       torch.float8_e4m3fn: _lib.DTYPE_E4M3, torch.float16: _lib.DTYPE_F16}


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream(device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


class PeerOp:
    """One native operator handle (``peer_create`` ... ``peer_destroy``).

    Plays the role of ``PEEROperatorEnhanced`` in the reference
    (llm/models/kernels/peer_cutlass.h:11-57): holds the configuration and the
    device scratch, and launches the kernels on the caller's stream."""

    def __init__(self, *, input_dim: int, output_dim: int, num_heads: int, query_dim: int,
                 product_key_dim, top_k: int, act_dtype: torch.dtype, table_dtype: torch.dtype,
                 activation: str = "gelu", norm_keys: bool = True, norm_query: bool = True,
                 layer_norm: bool = True, index_mode: str = "reference", max_tokens: int = 16384,
                 expert_hidden_size: int = 1, device=None):
        if not 1 <= len(product_key_dim) <= 4:
            raise ValueError(f"product_key_dim={list(product_key_dim)}: one to four key dimensions are implemented")
        if activation not in ("gelu", "relu"):
            raise ValueError(f"Unsupported activation: {activation}")
        if index_mode not in ("reference", "product"):
            raise ValueError(f"index_mode={index_mode!r}: 'reference' or 'product'")
        if act_dtype not in (torch.float32, torch.bfloat16, torch.float16) or table_dtype not in _DT:
            raise ValueError(f"unsupported dtypes: activations {act_dtype}, tables {table_dtype}")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("peer_b200 runs on CUDA devices only (sm_100a); there is no CPU path")
        self.lib = _lib.load()
        cfg = _lib.PeerConfig(
            abi_version=_lib.ABI_VERSION, input_dim=input_dim, output_dim=output_dim,
            num_experts=math.prod(int(n) for n in product_key_dim), top_k=top_k,
            num_heads=num_heads, query_dim=query_dim, n_keys0=int(product_key_dim[0]),
            n_keys1=int(product_key_dim[1]) if len(product_key_dim) > 1 else 1,
            n_keys2=int(product_key_dim[2]) if len(product_key_dim) > 2 else 1,
            n_keys3=int(product_key_dim[3]) if len(product_key_dim) > 3 else 1,
            num_key_dims=len(product_key_dim), expert_hidden_size=expert_hidden_size,
            activation=_lib.ACT_GELU if activation == "gelu" else _lib.ACT_RELU,
            norm_keys=int(norm_keys), norm_query=int(norm_query), layer_norm=int(layer_norm),
            act_dtype=_DT[act_dtype], table_dtype=_DT[table_dtype],
            index_mode=_lib.INDEX_REFERENCE if index_mode == "reference" else _lib.INDEX_PRODUCT,
            max_tokens=int(max_tokens))
        self.cfg = cfg
        self.num_key_dims = len(product_key_dim)
        self.act_dtype, self.table_dtype = act_dtype, table_dtype
        self.handle = C.c_void_p()
        self._tier = None
        with torch.cuda.device(self.device):
            rc = self.lib.peer_create(C.byref(cfg), C.byref(self.handle))
        if rc != _lib.OK:
            self.handle = C.c_void_p()
            _lib.check(rc, None)

    # -- plumbing -----------------------------------------------------------
    def close(self):
        if getattr(self, "handle", None) is not None and self.handle.value:
            self.lib.peer_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc):
        _lib.check(rc, self.handle)

    def _dev(self, t: torch.Tensor, name: str, dtype=None, host_ok=False) -> torch.Tensor:
        if t is None:
            return None
        if not host_ok and t.device != self.device:
            raise RuntimeError(f"{name} is on {t.device}, the operator on {self.device}")
        if dtype is not None and t.dtype != dtype:
            raise TypeError(f"{name} has dtype {t.dtype}, expected {dtype}")
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
        return t

    def _tensors(self, x, w: dict, out, ids_out=None, scores_out=None, host_io=False, product_ids_out=None) -> _lib.PeerTensors:
        a, tb = self.act_dtype, self.table_dtype
        self._dev(x, "x", a, host_ok=host_io)
        self._dev(out, "out", a, host_ok=host_io)
        for k in ("query_w", "query_b", "ln_w", "ln_b", "keys0", "keys1", "keys2", "keys3"):
            self._dev(w.get(k), k, a)
        for k in ("expert_down", "expert_up"):
            tbl = w.get(k)
            if self._tier is not None and tbl is not None and tbl.device.type == "cpu":
                if not tbl.is_pinned():     # the kernels read uncached rows straight from this memory
                    raise RuntimeError(f"{k} lives in host memory that is not pinned: the GPU cannot address it")
                self._dev(tbl, k, tb, host_ok=True)
            else:
                self._dev(tbl, k, tb)
        for k in ("down_scale", "up_scale"):
            self._dev(w.get(k), k, torch.float32)
        return _lib.PeerTensors(
            x=x.data_ptr(), query_w=w["query_w"].data_ptr(),
            query_b=None if w.get("query_b") is None else w["query_b"].data_ptr(),
            ln_w=None if w.get("ln_w") is None else w["ln_w"].data_ptr(),
            ln_b=None if w.get("ln_b") is None else w["ln_b"].data_ptr(),
            keys0=w["keys0"].data_ptr(), keys1=None if w.get("keys1") is None else w["keys1"].data_ptr(),
            keys2=None if w.get("keys2") is None else w["keys2"].data_ptr(),
            keys3=None if w.get("keys3") is None else w["keys3"].data_ptr(),
            expert_down=None if w.get("expert_down") is None else w["expert_down"].data_ptr(),
            expert_up=None if w.get("expert_up") is None else w["expert_up"].data_ptr(),
            down_scale=None if w.get("down_scale") is None else w["down_scale"].data_ptr(),
            up_scale=None if w.get("up_scale") is None else w["up_scale"].data_ptr(),
            out=None if out is None else out.data_ptr(),
            ids_out=None if ids_out is None else ids_out.data_ptr(),
            scores_out=None if scores_out is None else scores_out.data_ptr(),
            product_ids_out=None if product_ids_out is None else product_ids_out.data_ptr())

    # -- entry points -------------------------------------------------------
    def forward(self, x: torch.Tensor, w: dict, out: torch.Tensor, ids_out=None, scores_out=None, product_ids_out=None):
        """x [T, D] -> out [T, D_out] on the device, asynchronously on the current stream.  ``product_ids_out``
        (int32 [T, H, k]) receives the selected experts' true positions in the key grid."""
        T = x.shape[0]
        self._dev(product_ids_out, "product_ids_out", torch.int32)
        t = self._tensors(x, w, out, ids_out, scores_out, product_ids_out=product_ids_out)
        with torch.cuda.device(self.device):
            self._check(self.lib.peer_forward(self.handle, C.byref(t), T, _stream(self.device)))

    def block_forward(self, hidden: torch.Tensor, w: dict, ln_w, ln_b, eps: float, out: torch.Tensor,
                      ids_out=None, scores_out=None):
        """out = hidden + layer(LayerNorm(hidden)); hidden, out [T, D] on the device; ln_w, ln_b fp32 [D] or None."""
        self._dev(ln_w, "ln_w", torch.float32)
        self._dev(ln_b, "ln_b", torch.float32)
        if out.data_ptr() == hidden.data_ptr():
            raise ValueError("out may not alias hidden")
        t = self._tensors(hidden, w, out, ids_out, scores_out)
        with torch.cuda.device(self.device):
            self._check(self.lib.peer_block_forward(self.handle, C.byref(t), _ptr(ln_w), _ptr(ln_b), float(eps),
                                                    hidden.shape[0], _stream(self.device)))

    def set_row_tier(self, row_map: Optional[torch.Tensor], cache_down: Optional[torch.Tensor] = None,
                     cache_up: Optional[torch.Tensor] = None):
        """Tiered table residency (``peer_set_row_tier``): from now on ``expert_down`` / ``expert_up`` passed to the
        forwards are the full tables in pinned host memory, ``row_map`` (int32 [num_experts], device) says which
        rows are slots of the HBM-resident ``cache_down`` / ``cache_up``.  ``None`` switches back."""
        if row_map is None:
            self._check(self.lib.peer_set_row_tier(self.handle, None, None, None))
            self._tier = None
            return
        self._dev(row_map, "row_map", torch.int32)
        self._dev(cache_down, "cache_down", self.table_dtype)
        self._dev(cache_up, "cache_up", self.table_dtype)
        if row_map.numel() != self.cfg.num_experts:
            raise ValueError(f"row_map has {row_map.numel()} entries for {self.cfg.num_experts} experts")
        if int(row_map.max()) >= cache_down.shape[0] or cache_down.shape[0] != cache_up.shape[0]:
            raise ValueError("row_map points past the end of the cache tables")
        self._check(self.lib.peer_set_row_tier(self.handle, _ptr(row_map), _ptr(cache_down), _ptr(cache_up)))
        self._tier = (row_map, cache_down, cache_up)          # kept alive with the handle

    def forward_host(self, x: torch.Tensor, w: dict, out: torch.Tensor, ids_out=None, scores_out=None):
        """x and out in (pinned) host memory; returns when out is complete."""
        if x.device.type != "cpu" or out.device.type != "cpu":
            raise RuntimeError("forward_host takes host tensors for x and out")
        t = self._tensors(x, w, out, ids_out, scores_out, host_io=True)
        # the library runs this call on its own streams: make earlier work of the caller's stream
        # (a weight update, for instance) visible first
        torch.cuda.current_stream(self.device).synchronize()
        with torch.cuda.device(self.device):
            self._check(self.lib.peer_forward_host(self.handle, C.byref(t), x.shape[0]))

    def forward_host_async(self, x: torch.Tensor, w: dict, out: torch.Tensor, ids_out=None, scores_out=None) -> int:
        """Submit one host-buffer batch and return its ticket; ``forward_host_wait(ticket)`` blocks until ``out``
        (and the optional id/score outputs) are complete.  x must not change and out must not be read before."""
        if x.device.type != "cpu" or out.device.type != "cpu":
            raise RuntimeError("forward_host_async takes host tensors for x and out")
        t = self._tensors(x, w, out, ids_out, scores_out, host_io=True)
        torch.cuda.current_stream(self.device).synchronize()
        ticket = C.c_int64(-1)
        with torch.cuda.device(self.device):
            self._check(self.lib.peer_forward_host_async(self.handle, C.byref(t), x.shape[0], C.byref(ticket)))
        return int(ticket.value)

    def forward_host_wait(self, ticket: int):
        with torch.cuda.device(self.device):
            self._check(self.lib.peer_forward_host_wait(self.handle, int(ticket)))

    def project_queries(self, x: torch.Tensor, w: dict) -> torch.Tensor:
        T = x.shape[0]
        q = torch.empty(T, self.cfg.num_heads, self.cfg.query_dim, dtype=torch.float32, device=self.device)
        t = self._tensors(x, w, None)
        with torch.cuda.device(self.device):
            self._check(self.lib.peer_project_queries(self.handle, C.byref(t), T, _ptr(q), _stream(self.device)))
        return q

    def select(self, queries: torch.Tensor, keys0: torch.Tensor, keys1: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """queries fp32 [T, H, Q] (after LayerNorm) -> (ids int64, raw scores fp32) [T, H, k]."""
        self._dev(queries, "queries", torch.float32)
        self._dev(keys0, "keys0", self.act_dtype)
        self._dev(keys1, "keys1", self.act_dtype)
        T = queries.shape[0]
        ids = torch.empty(T, self.cfg.num_heads, self.cfg.top_k, dtype=torch.int64, device=self.device)
        sc = torch.empty(T, self.cfg.num_heads, self.cfg.top_k, dtype=torch.float32, device=self.device)
        with torch.cuda.device(self.device):
            self._check(self.lib.peer_select(self.handle, _ptr(queries), _ptr(keys0), _ptr(keys1), T,
                                             _ptr(ids), _ptr(sc), _stream(self.device)))
        return ids, sc

    def select_tokens(self, x: torch.Tensor, w: dict) -> Tuple[torch.Tensor, torch.Tensor]:
        """Query projection + selection of x [T, D]: (flat expert ids int32, softmax weights fp32), both
        [T, num_heads*top_k] - the tuples an expert-parallel rank routes to the owners of the rows."""
        T = x.shape[0]
        HK = self.cfg.num_heads * self.cfg.top_k
        ids = torch.empty(T, HK, dtype=torch.int32, device=self.device)
        wts = torch.empty(T, HK, dtype=torch.float32, device=self.device)
        t = self._tensors(x, w, None)
        with torch.cuda.device(self.device):
            self._check(self.lib.peer_select_tokens(self.handle, C.byref(t), T, _ptr(ids), _ptr(wts), _stream(self.device)))
        return ids, wts

    def select_stats(self) -> Tuple[int, int]:
        """(candidate lists that continued in the pool, rows redone by the exact kernel) of the tensor-core
        selection since the last read; synchronises."""
        a, b = C.c_int64(0), C.c_int64(0)
        with torch.cuda.device(self.device):
            self._check(self.lib.peer_select_stats(self.handle, C.byref(a), C.byref(b), _stream(self.device)))
        return int(a.value), int(b.value)

    def select_nd(self, queries: torch.Tensor, keys) -> Tuple[torch.Tensor, torch.Tensor]:
        """Selection over a key grid of any dimensionality: queries fp32 [T, H, Q] (after LayerNorm), keys a
        sequence of num_key_dims tables -> (ids int64, raw scores fp32) [T, H, k]."""
        self._dev(queries, "queries", torch.float32)
        if len(keys) != self.num_key_dims:
            raise ValueError(f"{len(keys)} sub-key tables for {self.num_key_dims} key dimensions")
        for i, kt in enumerate(keys):
            self._dev(kt, f"keys{i}", self.act_dtype)
        T = queries.shape[0]
        ids = torch.empty(T, self.cfg.num_heads, self.cfg.top_k, dtype=torch.int64, device=self.device)
        sc = torch.empty(T, self.cfg.num_heads, self.cfg.top_k, dtype=torch.float32, device=self.device)
        ptrs = (C.c_void_p * 4)(*[kt.data_ptr() for kt in keys])
        with torch.cuda.device(self.device):
            self._check(self.lib.peer_select_nd(self.handle, _ptr(queries), ptrs, T, _ptr(ids), _ptr(sc),
                                                _stream(self.device)))
        return ids, sc

    def select_backward(self, queries, keys, product_ids, scores, grad_weights) -> torch.Tensor:
        """dL/d(queries after LayerNorm) [T, H, Q] fp32 from dL/d(softmax weights) [T, H, k]."""
        self._dev(queries, "queries", torch.float32)
        self._dev(product_ids, "product_ids", torch.int32)
        self._dev(scores, "scores", torch.float32)
        self._dev(grad_weights, "grad_weights", torch.float32)
        if len(keys) != self.num_key_dims:
            raise ValueError(f"{len(keys)} sub-key tables for {self.num_key_dims} key dimensions")
        for i, kt in enumerate(keys):
            self._dev(kt, f"keys{i}", self.act_dtype)
        T = queries.shape[0]
        gq = torch.empty_like(queries)
        ptrs = (C.c_void_p * 4)(*[kt.data_ptr() for kt in keys])
        with torch.cuda.device(self.device):
            self._check(self.lib.peer_select_backward(self.handle, _ptr(queries), ptrs, _ptr(product_ids), _ptr(scores),
                                                      _ptr(grad_weights), T, _ptr(gq), _stream(self.device)))
        return gq

    def gather_eval(self, x, ids32, weights, down, up, down_scale=None, up_scale=None, out=None):
        """out[t] = sum_j weights[t,j] * act(down[ids[t,j]] . x[t]) * up[ids[t,j]]."""
        self._dev(x, "x", self.act_dtype)
        self._dev(ids32, "ids", torch.int32)
        self._dev(weights, "weights", torch.float32)
        self._dev(down, "expert_down", self.table_dtype)
        self._dev(up, "expert_up", self.table_dtype)
        self._dev(down_scale, "down_scale", torch.float32)
        self._dev(up_scale, "up_scale", torch.float32)
        T = x.shape[0]
        if out is None:
            out = torch.empty(T, self.cfg.output_dim, dtype=self.act_dtype, device=self.device)
        with torch.cuda.device(self.device):
            self._check(self.lib.peer_gather_eval(self.handle, _ptr(x), _ptr(ids32), _ptr(weights), _ptr(down),
                                                  _ptr(up), _ptr(down_scale), _ptr(up_scale), _ptr(out), T,
                                                  _stream(self.device)))
        return out

    def gather_eval_partial(self, x, ids32, weights, counts, down, up, down_scale=None, up_scale=None):
        """Partial expert evaluation against a row shard: ids are LOCAL row numbers, token t uses its first
        counts[t] entries; returns the fp32 partial sums [T, D_out]."""
        self._dev(x, "x", self.act_dtype)
        self._dev(ids32, "ids", torch.int32)
        self._dev(weights, "weights", torch.float32)
        self._dev(counts, "counts", torch.int32)
        self._dev(down, "expert_down", self.table_dtype)
        self._dev(up, "expert_up", self.table_dtype)
        self._dev(down_scale, "down_scale", torch.float32)
        self._dev(up_scale, "up_scale", torch.float32)
        T, cap = ids32.shape
        out = torch.empty(T, self.cfg.output_dim, dtype=torch.float32, device=self.device)
        with torch.cuda.device(self.device):
            self._check(self.lib.peer_gather_eval_partial(
                self.handle, _ptr(x), _ptr(ids32), _ptr(weights), _ptr(counts), cap, _ptr(down), _ptr(up),
                _ptr(down_scale), _ptr(up_scale), down.shape[0], _ptr(out), T, _stream(self.device)))
        return out

    def gather_eval_routed(self, x_all, recv, world: int, tokens_per_rank: int, down, up, down_scale=None,
                           up_scale=None, out=None):
        """Partial expert evaluation straight from the blocks an expert-parallel rank received (int32
        [world, 2*T*E + T]: local row ids, weight bits, counts; see `sharded.route_tuples_blocks`): fp32 partial
        sums [world*T, D_out] for all tokens against this rank's row shard."""
        self._dev(x_all, "x", self.act_dtype)
        self._dev(recv, "recv", torch.int32)
        self._dev(down, "expert_down", self.table_dtype)
        self._dev(up, "expert_up", self.table_dtype)
        self._dev(down_scale, "down_scale", torch.float32)
        self._dev(up_scale, "up_scale", torch.float32)
        E = self.cfg.num_heads * self.cfg.top_k
        if recv.shape != (world, 2 * tokens_per_rank * E + tokens_per_rank):
            raise ValueError(f"recv is {tuple(recv.shape)}, expected {(world, 2 * tokens_per_rank * E + tokens_per_rank)}")
        if out is None:
            out = torch.empty(world * tokens_per_rank, self.cfg.output_dim, dtype=torch.float32, device=self.device)
        self._dev(out, "out", torch.float32)
        with torch.cuda.device(self.device):
            self._check(self.lib.peer_gather_eval_routed(
                self.handle, _ptr(x_all), _ptr(recv), int(world), int(tokens_per_rank), _ptr(down), _ptr(up),
                _ptr(down_scale), _ptr(up_scale), down.shape[0], _ptr(out), _stream(self.device)))
        return out

    def gather_eval_backward(self, x, grad_out, ids32, weights, down, up, grad_down=None, grad_up=None,
                             grad_dtype: torch.dtype = torch.float32, grad_rows: Optional[int] = None):
        """Gradients of ``gather_eval``.  Returns (grad_x [T,D] fp32, grad_weights [T,H*k] fp32, grad_down
        [N,D], grad_up [N,D_out]); the two table gradients are accumulated into the buffers passed in
        (zero-initialised ones are made when none are given), in ``grad_dtype``: fp32, or the tables' bf16.
        ``grad_rows``: the gradient tables cover rows [0, grad_rows) only (every id is known to lie below)."""
        if grad_dtype not in (torch.float32, self.table_dtype) or grad_dtype not in _DT:
            raise ValueError(f"table gradients are accumulated in fp32 or in the tables' dtype, not {grad_dtype}")
        self._dev(x, "x", self.act_dtype)
        self._dev(grad_out, "grad_out", self.act_dtype)
        self._dev(ids32, "ids", torch.int32)
        self._dev(weights, "weights", torch.float32)
        self._dev(down, "expert_down", self.table_dtype)
        self._dev(up, "expert_up", self.table_dtype)
        T = x.shape[0]
        n_rows = down.shape[0] if grad_rows is None else int(grad_rows)
        if grad_down is None:
            grad_down = torch.zeros(n_rows, down.shape[1], dtype=grad_dtype, device=self.device)
        if grad_up is None:
            grad_up = torch.zeros(n_rows, up.shape[1], dtype=grad_dtype, device=self.device)
        self._dev(grad_down, "grad_down", grad_dtype)
        self._dev(grad_up, "grad_up", grad_dtype)
        if grad_down.shape[0] != n_rows or grad_up.shape[0] != n_rows:
            raise ValueError(f"gradient tables must have {n_rows} rows")
        gx = torch.empty(T, self.cfg.input_dim, dtype=torch.float32, device=self.device)
        gw = torch.empty(T, self.cfg.num_heads * self.cfg.top_k, dtype=torch.float32, device=self.device)
        with torch.cuda.device(self.device):
            self._check(self.lib.peer_gather_eval_backward_rows(
                self.handle, _ptr(x), _ptr(grad_out), _ptr(ids32), _ptr(weights), _ptr(down), _ptr(up),
                _ptr(gx), _ptr(gw), _ptr(grad_down), _ptr(grad_up), _DT[grad_dtype], n_rows, T, _stream(self.device)))
        return gx, gw, grad_down, grad_up

    def query_status(self):
        """Synchronise and raise if a kernel recorded a timeout or an out-of-range id."""
        with torch.cuda.device(self.device):
            self._check(self.lib.peer_query_status(self.handle, _stream(self.device)))

    def freeze_keys(self, frozen: bool = True):
        """Inference with fixed sub-keys: the per-call preparation of the key tables (norms, normalised copy, error
        bounds) is done once and reused while the same key tensors come on the same stream (`peer_freeze_keys`)."""
        self._check(self.lib.peer_freeze_keys(self.handle, int(frozen)))

    def stage_timing(self, enable: bool):
        """Record CUDA events around the three stage launches of every following forward."""
        self._check(self.lib.peer_stage_timing(self.handle, int(enable)))

    def stage_times(self):
        """(ms_query, ms_select, ms_experts, n_slices) summed since the last read; synchronises."""
        ms = (C.c_double * 3)()
        n = C.c_int64()
        self._check(self.lib.peer_stage_times(self.handle, ms, C.byref(n)))
        return ms[0], ms[1], ms[2], int(n.value)

    @property
    def launch_count(self) -> int:
        return int(self.lib.peer_launch_count(self.handle))


class PEER(nn.Module):
    """Parameter Efficient Expert Retrieval layer on the B200 kernels.

    Same constructor arguments and defaults as the reference
    (llm/models/experts.py:46-61); same parameters: ``query_proj`` (Linear with
    bias), ``query_layer_norm`` (LayerNorm(query_dim) shared by all heads, or
    None), ``sub_keys`` (two ``[n_i, query_dim/2]`` tables), ``expert_down`` /
    ``expert_up`` (Embedding tables).

    Attributes that may be set after construction (keyword filtering in
    ``TransformerBlock`` passes constructor names only, foundation.py:135-147):

    * ``index_mode``: ``"reference"`` (flat id = i0 + i1, what the reference's
      PyTorch forward computes) or ``"product"`` (i0 * n1 + i1).
    * ``track_indices``: when true (default, as in the reference) every forward
      stores ``_last_expert_indices`` (int64 [B,S,H,k]) and
      ``_last_expert_scores`` (raw scores, fp32).
    * ``max_slice_tokens``: token capacity of the scratch; longer inputs run in
      slices.
    * ``table_grad_sums``: how the backward pass sums a table row's gradient.
      ``"fp32"``: in fp32, rounded once, like the reference's embedding backward.
      ``"table"`` (bf16 layers): in bf16, half the traffic, one rounding per addend.
      ``"auto"`` (default): fp32 whenever rows collect many contributions - always
      with ``index_mode="reference"`` (ids stay below n0 + n1; then only those rows
      get fp32 sums, not the whole table) and when a batch brings more than four
      selections per table row on average - else ``"table"``.
    """

    def __init__(self, input_dim: int, output_dim: int, num_experts: int, num_experts_per_tok: int = 16,
                 num_heads: int = 8, expert_hidden_size: int = 1, query_dim: int = 256,
                 product_key_dim: List[int] = [32, 32], activation: str = "gelu", dropout: float = 0.0,
                 norm_keys: bool = True, norm_query: bool = True, batch_norm_query: bool = True):
        super().__init__()
        self.input_dim = input_dim
        self.output_dim = output_dim
        self.num_experts = num_experts
        self.num_experts_per_tok = num_experts_per_tok
        self.num_heads = num_heads
        self.expert_hidden_size = expert_hidden_size
        self.query_dim = query_dim
        self.product_key_dim = list(product_key_dim)
        self.norm_keys = norm_keys
        self.norm_query = norm_query
        self.batch_norm_query = batch_norm_query
        self.activation_name = activation

        if math.prod(self.product_key_dim) != num_experts:
            raise AssertionError(f"Product of dimensions {self.product_key_dim} = {math.prod(self.product_key_dim)} "
                                 f"must equal the number of experts {num_experts}")
        if activation not in ("relu", "gelu"):
            raise ValueError(f"Unsupported activation: {activation}")
        if not 1 <= len(self.product_key_dim) <= 4:
            raise ValueError("peer_b200 implements product keys of one to four dimensions")
        if not 1 <= expert_hidden_size <= 16:
            raise ValueError("peer_b200 implements experts of 1 to 16 hidden neurons")
        if query_dim % len(self.product_key_dim):
            raise ValueError(f"query_dim {query_dim} must be divisible by the {len(self.product_key_dim)} key dimensions")

        self.query_proj = nn.Linear(input_dim, num_heads * query_dim)
        self.query_layer_norm = nn.LayerNorm(query_dim) if batch_norm_query else None
        self.sub_keys = nn.ParameterList()
        sub = query_dim // len(self.product_key_dim)
        for n in self.product_key_dim:
            self.sub_keys.append(nn.Parameter(torch.empty(n, sub).normal_(0.0, 0.02)))
        self.expert_down = nn.Embedding(num_experts, input_dim * expert_hidden_size)
        self.expert_up = nn.Embedding(num_experts, output_dim * expert_hidden_size)
        self.dropout = nn.Dropout(dropout)
        self.register_buffer("expert_down_scale", None, persistent=True)
        self.register_buffer("expert_up_scale", None, persistent=True)

        self.index_mode = "reference"
        self.track_indices = True
        self.max_slice_tokens = 16384
        self.table_grad_sums = "auto"
        self._last_expert_indices: Optional[torch.Tensor] = None
        self._last_expert_scores: Optional[torch.Tensor] = None
        self._op: Optional[PeerOp] = None
        self._op_key = None
        self._sel_op: Optional[PeerOp] = None
        self._sel_op_key = None
        self._tier = None           # (row_map, cache_down, cache_up) while the tables live in host memory

    # -- FP8 tables ---------------------------------------------------------
    @torch.no_grad()
    def quantize_tables_e4m3(self):
        """Replace both expert tables by FP8-e4m3 payloads with a per-row fp32
        scale (absmax/448)."""
        from .synthetic import quantize_rows_e4m3
        for name in ("expert_down", "expert_up"):
            emb = getattr(self, name)
            q, s = quantize_rows_e4m3(emb.weight.data)
            emb.weight = nn.Parameter(q, requires_grad=False)
            setattr(self, name + "_scale", s)
        return self

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        """A checkpoint written from a module with FP8 tables (``state_dict()`` then holds float8 payloads and the
        two per-row scale buffers; the reference saves ``model.state_dict()`` with safetensors,
        llm/training/train.py:201-246) loads into a freshly constructed module: the tables switch to FP8 storage
        before the tensors are copied."""
        names = ("expert_down", "expert_up")
        if all(prefix + n + "_scale" in state_dict for n in names):
            for n in names:
                src, scale = state_dict[prefix + n + ".weight"], state_dict[prefix + n + "_scale"]
                if src.dtype != torch.float8_e4m3fn:
                    raise TypeError(f"{prefix}{n}.weight comes with a row scale but is {src.dtype}, not float8_e4m3fn")
                emb = getattr(self, n)
                dev = emb.weight.device
                emb.weight = nn.Parameter(torch.empty(src.shape, dtype=src.dtype, device=dev), requires_grad=False)
                setattr(self, n + "_scale", torch.empty(scale.shape, dtype=scale.dtype, device=dev))
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    # -- tables larger than the GPU's memory -----------------------------------
    @torch.no_grad()
    def enable_host_tier(self, cache_rows: int, usage_counts: Optional[torch.Tensor] = None, device=None):
        """Keep the expert tables in pinned host memory and only ``cache_rows`` rows of each in HBM: the role of
        the reference's HierarchicalExpertCache (llm/models/kernels/peer_cutlass.cu:110-536,
        docs/MEMORY_HIERARCHY.md:5-11).  The cached rows are the most used ones according to ``usage_counts``
        (int64 [num_experts], e.g. ``DeviceUsageCounter`` totals; the first rows when none are given).  The
        expert stage reads a cached row through its usual HBM rings and any other row in place from host memory
        over PCIe.  Inference only; bf16 or FP8 tables, single-neuron experts.  Results are bit-identical to the
        all-HBM layer.  Call again to re-pick the cached rows."""
        if self.expert_hidden_size != 1 or self.expert_down.weight.dtype not in (torch.bfloat16, torch.float8_e4m3fn):
            raise ValueError("host tiering: bf16 or FP8 tables of single-neuron experts")
        dev = torch.device(device) if device is not None else self.query_proj.weight.device
        if dev.type != "cuda":
            raise RuntimeError("host tiering needs the small weights on a CUDA device")
        N = self.num_experts
        cache_rows = max(1, min(int(cache_rows), N))
        if usage_counts is not None:
            hot = torch.topk(usage_counts.to(dev).view(-1).float(), cache_rows).indices.sort().values
        else:
            hot = torch.arange(cache_rows, device=dev)
        row_map = torch.full((N,), -1, dtype=torch.int32, device=dev)
        row_map[hot] = torch.arange(cache_rows, dtype=torch.int32, device=dev)
        caches = []
        for name in ("expert_down", "expert_up"):
            emb = getattr(self, name)
            host = emb.weight.data
            if host.device.type != "cpu" or not host.is_pinned():
                host = host.cpu().pin_memory()
            raw = host.view(torch.uint8) if host.element_size() == 1 else host      # row gather of FP8 payloads as bytes
            caches.append(raw[hot.cpu()].view(host.dtype).to(dev).contiguous())
            emb.weight = nn.Parameter(host, requires_grad=False)
        self._tier = (row_map, caches[0], caches[1])
        self._op = None                                  # the next forward builds a handle with the tier set
        return self

    def disable_host_tier(self, device=None):
        """Move the tables back into device memory."""
        dev = torch.device(device) if device is not None else self.query_proj.weight.device
        for name in ("expert_down", "expert_up"):
            emb = getattr(self, name)
            emb.weight = nn.Parameter(emb.weight.data.to(dev), requires_grad=False)
        self._tier = None
        self._op = None
        return self

    # -- operator management -------------------------------------------------
    def _weights(self) -> dict:
        ln = self.query_layer_norm
        keys = {f"keys{i}": k for i, k in enumerate(self.sub_keys)}
        return dict(query_w=self.query_proj.weight, query_b=self.query_proj.bias,
                    ln_w=None if ln is None else ln.weight, ln_b=None if ln is None else ln.bias,
                    **keys, expert_down=self.expert_down.weight,
                    expert_up=self.expert_up.weight, down_scale=self.expert_down_scale,
                    up_scale=self.expert_up_scale)

    def _operator(self, device, act_dtype, n_tokens: int) -> PeerOp:
        cap = min(max(n_tokens, 1), self.max_slice_tokens)
        table_dtype = self.expert_down.weight.dtype
        key = (str(device), act_dtype, table_dtype, self.index_mode, self.activation_name,
               self.norm_keys, self.norm_query, self.batch_norm_query, self.expert_hidden_size)
        if self._op is None or self._op_key != key or self._op.cfg.max_tokens < cap:
            if self._op is not None:
                cap = max(cap, self._op.cfg.max_tokens) if self._op_key == key else cap
                # not closed here: an autograd graph may still hold the old handle; it is released with
                # its last reference
            self._op = PeerOp(input_dim=self.input_dim, output_dim=self.output_dim, num_heads=self.num_heads,
                              query_dim=self.query_dim, product_key_dim=self.product_key_dim,
                              top_k=self.num_experts_per_tok, act_dtype=act_dtype, table_dtype=table_dtype,
                              activation=self.activation_name, norm_keys=self.norm_keys,
                              norm_query=self.norm_query, layer_norm=self.batch_norm_query,
                              index_mode=self.index_mode, max_tokens=cap,
                              expert_hidden_size=self.expert_hidden_size, device=device)
            self._op_key = key
            if self._tier is not None:
                self._op.set_row_tier(*self._tier)
        return self._op

    def _product_operator(self, device, act_dtype, n_tokens: int) -> PeerOp:
        """A second handle whose selection returns i0 * n1 + i1 whatever ``index_mode`` is: the
        differentiable forward needs both sub-key indices of every selected expert."""
        if self.index_mode == "product":
            return self._operator(device, act_dtype, n_tokens)
        cap = min(max(n_tokens, 1), self.max_slice_tokens)
        key = (str(device), act_dtype, self.norm_keys, self.norm_query)
        if self._sel_op is None or self._sel_op_key != key or self._sel_op.cfg.max_tokens < cap:
            self._sel_op = PeerOp(input_dim=self.input_dim, output_dim=self.output_dim, num_heads=self.num_heads,
                                  query_dim=self.query_dim, product_key_dim=self.product_key_dim,
                                  top_k=self.num_experts_per_tok, act_dtype=act_dtype, table_dtype=act_dtype,
                                  activation=self.activation_name, norm_keys=self.norm_keys,
                                  norm_query=self.norm_query, layer_norm=self.batch_norm_query,
                                  index_mode="product", max_tokens=cap,
                                  expert_hidden_size=self.expert_hidden_size, device=device)
            self._sel_op_key = key
        return self._sel_op

    def _needs_grad(self, hidden_states: torch.Tensor) -> bool:
        need = torch.is_grad_enabled() and (hidden_states.requires_grad or
                                            any(p.requires_grad for p in self.parameters()))
        if need and self._tier is not None:
            raise RuntimeError("tables tiered into host memory are inference-only: call under torch.no_grad()")
        return need

    def _prepare(self, hidden_states: torch.Tensor):
        if hidden_states.dim() != 3 or hidden_states.shape[-1] != self.input_dim:
            raise ValueError(f"hidden_states must be [batch, seq, {self.input_dim}], got {tuple(hidden_states.shape)}")
        w = self._weights()
        dt = self.query_proj.weight.dtype
        if hidden_states.dtype != dt:
            raise TypeError(f"hidden_states is {hidden_states.dtype} but the module's parameters are {dt}")
        return w, dt

    # -- forward --------------------------------------------------------------
    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        """[batch, seq, input_dim] -> [batch, seq, output_dim], same dtype (experts.py:422-440).
        When gradients are being recorded the call goes through ``autograd.peer_forward_autograd``;
        dropout (training mode, experts.py:366) exists on that path only."""
        w, dt = self._prepare(hidden_states)
        grad = self._needs_grad(hidden_states)
        if not grad and self.training and self.dropout.p > 0:
            raise RuntimeError("dropout in training mode needs the differentiable path: enable gradients, "
                               "or call eval()")
        if hidden_states.device.type != "cuda":
            raise RuntimeError("peer_b200 runs on CUDA devices only (sm_100a); there is no CPU path. "
                               "Use forward_host() to feed pinned host buffers.")
        if grad:
            from .autograd import peer_forward_autograd
            return peer_forward_autograd(self, hidden_states)
        B, S, _ = hidden_states.shape
        T = B * S
        x = hidden_states.contiguous().view(T, self.input_dim)
        op = self._operator(x.device, dt, T)
        out = torch.empty(T, self.output_dim, dtype=dt, device=x.device)
        ids = sc = None
        if self.track_indices:
            ids = torch.empty(T, self.num_heads, self.num_experts_per_tok, dtype=torch.int64, device=x.device)
            sc = torch.empty(T, self.num_heads, self.num_experts_per_tok, dtype=torch.float32, device=x.device)
        op.forward(x, w, out, ids, sc)
        self._stash(ids, sc, B, S)
        return out.view(B, S, self.output_dim)

    def block_forward(self, hidden_states: torch.Tensor, ln_2: nn.LayerNorm) -> torch.Tensor:
        """``hidden_states + self(ln_2(hidden_states))``: the feed-forward half of the reference's
        TransformerBlock.forward (foundation.py:196-205) in one library call.  Inference only."""
        if self._needs_grad(hidden_states) or (torch.is_grad_enabled() and any(p.requires_grad for p in ln_2.parameters())):
            raise RuntimeError("block_forward is an inference path; call it under torch.no_grad()")
        if self.training and self.dropout.p > 0:
            raise RuntimeError("block_forward is an inference path: call eval() first (dropout is set)")
        w, dt = self._prepare(hidden_states)
        if hidden_states.device.type != "cuda":
            raise RuntimeError("peer_b200 runs on CUDA devices only (sm_100a); there is no CPU path")
        B, S, _ = hidden_states.shape
        T = B * S
        x = hidden_states.contiguous().view(T, self.input_dim)
        op = self._operator(x.device, dt, T)
        out = torch.empty(T, self.output_dim, dtype=dt, device=x.device)
        ids = sc = None
        if self.track_indices:
            ids = torch.empty(T, self.num_heads, self.num_experts_per_tok, dtype=torch.int64, device=x.device)
            sc = torch.empty(T, self.num_heads, self.num_experts_per_tok, dtype=torch.float32, device=x.device)
        f32 = lambda p: None if p is None else p.detach().float().contiguous()
        op.block_forward(x, w, f32(ln_2.weight), f32(ln_2.bias), ln_2.eps, out, ids, sc)
        self._stash(ids, sc, B, S)
        return out.view(B, S, self.output_dim)

    def forward_host(self, hidden_states: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Same layer for a HOST tensor (pinned for full speed): slices are copied to the device,
        processed and copied back on overlapping streams.  Returns a host tensor.  Inference only."""
        return self._forward_host(hidden_states, out, blocking=True)[0]

    def forward_host_wait(self, ticket) -> None:
        """Block until the batch submitted by ``forward_host_async`` has landed in its host output.  The ticket
        holds the batch's host buffers (input, output, ids, scores) until here, so none of them can be freed or
        handed out again while a copy is still queued on the library's streams; the tracker attributes
        (``_last_expert_indices`` / ``_last_expert_scores``) are set now, when their contents are complete."""
        op, tk, _x, _out, ids, sc, (B, S) = ticket
        op.forward_host_wait(tk)
        self._stash(ids, sc, B, S)

    def forward_host_async(self, hidden_states: torch.Tensor, out: Optional[torch.Tensor] = None):
        """Submit a host batch without waiting: returns ``(out, ticket)``.  The next batch may be submitted
        before this one is waited for, so that its first copy-in overlaps this one's last copy-out; give
        each batch in flight its own ``out``.  ``hidden_states`` must not change until the wait.  A batch
        submitted this way runs as one slice (its copies hide behind its neighbours' kernels); the blocking
        call slices a batch so that its own copies overlap its own kernels."""
        return self._forward_host(hidden_states, out, blocking=False)

    def _forward_host(self, hidden_states: torch.Tensor, out: Optional[torch.Tensor], blocking: bool):
        if self._needs_grad(hidden_states):
            raise RuntimeError("forward_host is an inference path; call it under torch.no_grad()")
        if self.training and self.dropout.p > 0:
            raise RuntimeError("forward_host is an inference path: call eval() first (dropout is set)")
        w, dt = self._prepare(hidden_states)
        if hidden_states.device.type != "cpu":
            raise RuntimeError("forward_host takes a host tensor")
        B, S, _ = hidden_states.shape
        T = B * S
        if not blocking and not hidden_states.is_contiguous():
            # a contiguous copy would be a temporary that dies while its copy-in is still queued
            raise ValueError("forward_host_async needs a contiguous host tensor")
        x = hidden_states.contiguous().view(T, self.input_dim)
        dev = self.query_proj.weight.device
        op = self._operator(dev, dt, T)
        if out is None:
            out = torch.empty(B, S, self.output_dim, dtype=dt, pin_memory=True)
        ids = sc = None
        if self.track_indices:
            ids = torch.empty(T, self.num_heads, self.num_experts_per_tok, dtype=torch.int64, pin_memory=True)
            sc = torch.empty(T, self.num_heads, self.num_experts_per_tok, dtype=torch.float32, pin_memory=True)
        ticket = None
        if blocking:
            op.forward_host(x, w, out.view(T, self.output_dim), ids, sc)
            self._stash(ids, sc, B, S)
        else:
            ticket = (op, op.forward_host_async(x, w, out.view(T, self.output_dim), ids, sc), x, out, ids, sc, (B, S))
        return out, ticket

    def _stash(self, ids, sc, B, S):
        if ids is not None:
            self._last_expert_indices = ids.view(B, S, self.num_heads, self.num_experts_per_tok)
            self._last_expert_scores = sc.view(B, S, self.num_heads, self.num_experts_per_tok)

    @torch.no_grad()
    def select(self, queries: torch.Tensor, top_k: Optional[int] = None):
        """Counterpart of ``_get_expert_indices_pytorch`` (experts.py:138-285):
        queries [B,S,H,Q] after LayerNorm -> (indices int64, raw scores) [B,S,H,k]."""
        if top_k is not None and top_k != self.num_experts_per_tok:
            raise ValueError("top_k must equal num_experts_per_tok")
        B, S, H, Q = queries.shape
        op = self._operator(queries.device, self.sub_keys[0].dtype, B * S)
        q = queries.float().contiguous().view(B * S, H, Q)
        if len(self.sub_keys) == 2:
            ids, sc = op.select(q, self.sub_keys[0], self.sub_keys[1])
        else:
            ids, sc = op.select_nd(q, [k.detach() for k in self.sub_keys])
        return ids.view(B, S, H, -1), sc.view(B, S, H, -1).to(queries.dtype)

    _get_expert_indices = select
    # the name the reference's own selection test calls (tests/test_peer_selection.py:123)
    _get_expert_indices_pytorch = select

    def split_queries(self, queries: torch.Tensor) -> List[torch.Tensor]:
        """One slice of the last dimension per key dimension, in order (experts.py:125-136): views of
        ``queries[..., d*w:(d+1)*w]`` with ``w = query_dim // len(product_key_dim)``.  The kernels do this split
        inside the query epilogue; the method exists for callers of the reference's API."""
        w = self.query_dim // len(self.product_key_dim)
        return [queries[..., d * w:(d + 1) * w] for d in range(len(self.product_key_dim))]
