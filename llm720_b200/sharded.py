"""Expert-parallel PEER: the expert tables are split by rows over the ranks of a process group.

The reference has no distributed PEER (its multi-GPU story is data parallelism through
Accelerate, llm/training/train.py:472-476, 638-640; expert sharding is announced in
docs/paper/paper.tex:446 and listed as future work in docs/CUTLASS_KERNEL.md:181).  This is
the layer for tables that do not fit, or should not be replicated, on every GPU:

  rank r owns rows [r*N/G, (r+1)*N/G) of expert_down / expert_up; the small weights (query
  projection, LayerNorm, sub-keys) are replicated; every rank brings its own tokens.

  1. all-gather of the activations (every owner needs x_t for the tuples it will receive);
  2. each rank selects for ITS tokens (query projection + product-key retrieval kernels);
  3. the selected (token, expert id, weight) tuples are sorted by owner and exchanged with one
     all-to-all of equal-size blocks (per destination: [local row ids T x E | weight bits T x E |
     counts T], row t = those of token t's tuples the destination owns); a token's tuples only come
     from the rank that owns the token, so the received blocks ARE the per-token lists;
  4. each rank evaluates the tuples it received against its row shard (one kernel, fp32 partial
     sums per token);
  5. reduce-scatter of the partial sums gives every rank the outputs of its own tokens.

`ShardedPEER(exchange="direct")` does steps 1, 3 and 5 without collectives: the library's `peer_xchg_*` entries
store x, the tuple blocks and the partial sums straight into the peers' memory (regions mapped through CUDA
IPC, step numbers as completion flags, bounded waits) and add the partial sums in rank order.

Result: identical to the single-device layer on the concatenated batch, up to fp32 summation
order.  The exchange logic exists twice: as plain tensor code (`route_tuples_blocks`,
`lists_from_blocks`, and the variable-length `route_tuples` / `pack_received`) that runs on any device
and is tested with CPU ranks over gloo, and in the library (`peer_route_tuples`, one kernel, wrapped by
`route_tuples_native`; `peer_gather_eval_routed`, the expert stage reading the received blocks in
place) which `ShardedPEER` uses on the GPU; a GPU test compares the two forms.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib


def rows_per_rank(num_experts: int, world: int) -> int:
    if num_experts % world:
        raise ValueError(f"{num_experts} experts do not split evenly over {world} ranks")
    return num_experts // world


def route_tuples(ids: torch.Tensor, weights: torch.Tensor, token_offset: int, rows: int, world: int):
    """ids int64/int32 [T, HK], weights fp32 [T, HK] of this rank's tokens ->
    (send int32 [n, 3] = (global token, local row, weight bits) sorted by destination rank,
     send_counts int64 [world])."""
    T, HK = ids.shape
    flat = ids.reshape(-1).to(torch.int64)
    owner = torch.div(flat, rows, rounding_mode="floor")
    order = torch.argsort(owner, stable=True)
    tok = (torch.arange(T, device=ids.device, dtype=torch.int64).repeat_interleave(HK) + token_offset)[order]
    local = (flat - owner * rows)[order]
    wbits = weights.reshape(-1).to(torch.float32).view(torch.int32)[order]
    send = torch.stack([tok.to(torch.int32), local.to(torch.int32), wbits], dim=1).contiguous()
    counts = torch.bincount(owner, minlength=world)[:world]
    return send, counts


def pack_received(recv: torch.Tensor, n_tokens: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Received tuples int32 [m, 3] (any order) -> per-token padded lists:
    (ids int32 [T, cap], weights fp32 [T, cap], counts int32 [T]); cap = the longest list (>= 1)."""
    dev = recv.device
    if recv.shape[0] == 0:
        z = torch.zeros(n_tokens, 1, dtype=torch.int32, device=dev)
        return z, torch.zeros(n_tokens, 1, dtype=torch.float32, device=dev), torch.zeros(n_tokens, dtype=torch.int32, device=dev)
    tok = recv[:, 0].to(torch.int64)
    order = torch.argsort(tok, stable=True)
    tok = tok[order]
    counts = torch.bincount(tok, minlength=n_tokens)
    cap = max(int(counts.max()), 1)
    start = torch.cumsum(counts, 0) - counts
    pos = torch.arange(tok.numel(), device=dev) - start[tok]
    ids = torch.zeros(n_tokens, cap, dtype=torch.int32, device=dev)
    w = torch.zeros(n_tokens, cap, dtype=torch.float32, device=dev)
    ids[tok, pos] = recv[order, 1]
    w[tok, pos] = recv[order, 2].contiguous().view(torch.float32)
    return ids, w, counts.to(torch.int32)


def exchange(send: torch.Tensor, send_counts: torch.Tensor, group=None) -> torch.Tensor:
    """All-to-all of variable-length tuple buckets: counts first, then the tuples."""
    world = dist.get_world_size(group)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    sc, rc = send_counts.tolist(), recv_counts.tolist()
    recv = torch.empty(sum(rc), 3, dtype=torch.int32, device=send.device)
    dist.all_to_all_single(recv, send, output_split_sizes=rc, input_split_sizes=sc, group=group)
    return recv


# ---------------------------------------------------------------------------
# Fixed-shape form of the exchange: every rank sends every peer one block of the same size,
#     [ local row ids: T x E | weight bits: T x E | counts: T ]      (int32; T tokens of the sender, E = H*k)
# row t holding, packed to the front in slot order, those of token t's tuples the peer owns.  One
# all-to-all, no counts round, no host synchronisation, shapes that never change from step to step; and
# since a token's tuples only come from the rank that owns it, block b row t of what arrives is already
# the list of global token b*T + t.
# ---------------------------------------------------------------------------
def block_words(T: int, E: int) -> int:
    return 2 * T * E + T


def route_tuples_blocks(ids: torch.Tensor, weights: torch.Tensor, rows: int, world: int) -> torch.Tensor:
    """ids [T, E] global expert ids, weights fp32 [T, E] -> int32 [world, 2*T*E + T]."""
    T, E = ids.shape
    dev = ids.device
    flat = ids.to(torch.int64)
    owner = torch.div(flat, rows, rounding_mode="floor")
    wbits = weights.to(torch.float32).contiguous().view(torch.int32)
    send = torch.zeros(world, block_words(T, E), dtype=torch.int32, device=dev)
    trow = torch.arange(T, device=dev).unsqueeze(1).expand(T, E)
    for r in range(world):
        m = owner == r
        pos = m.cumsum(1) - 1
        b_ids = send[r, :T * E].view(T, E)
        b_w = send[r, T * E:2 * T * E].view(T, E)
        b_ids[trow[m], pos[m]] = (flat[m] - r * rows).to(torch.int32)
        b_w[trow[m], pos[m]] = wbits[m]
        send[r, 2 * T * E:] = m.sum(1).to(torch.int32)
    return send


def lists_from_blocks(recv: torch.Tensor, T: int, E: int):
    """Received blocks int32 [world, 2*T*E + T] -> (ids int32 [world*T, E], weights fp32 [world*T, E],
    counts int32 [world*T]) of all tokens, global token b*T + t from block b row t."""
    world = recv.shape[0]
    ids = recv[:, :T * E].reshape(world * T, E)
    w = recv[:, T * E:2 * T * E].contiguous().view(torch.float32).reshape(world * T, E)
    cnt = recv[:, 2 * T * E:].reshape(world * T)
    return ids.contiguous(), w, cnt.contiguous()


def exchange_static(send: torch.Tensor, group=None) -> torch.Tensor:
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv


def route_tuples_native(ids32: torch.Tensor, weights: torch.Tensor, rows: int, world: int,
                        send: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`route_tuples_blocks` as one kernel of the library (CUDA tensors: int32 ids, fp32 weights)."""
    import ctypes as C
    from . import _lib
    T, E = ids32.shape
    if ids32.dtype != torch.int32 or weights.dtype != torch.float32 or not ids32.is_cuda:
        raise TypeError("route_tuples_native takes CUDA tensors: int32 ids and fp32 weights")
    if send is None:
        send = torch.empty(world, block_words(T, E), dtype=torch.int32, device=ids32.device)
    lib = _lib.load()
    with torch.cuda.device(ids32.device):
        rc = lib.peer_route_tuples(C.c_void_p(ids32.contiguous().data_ptr()), C.c_void_p(weights.contiguous().data_ptr()),
                                   T, E, int(rows), int(world), C.c_void_p(send.data_ptr()),
                                   C.c_void_p(torch.cuda.current_stream(ids32.device).cuda_stream))
    _lib.check(rc, None)
    return send


def reduce_scatter_rows(partial: torch.Tensor, group=None) -> torch.Tensor:
    """[T_total, D] fp32 partial sums -> this rank's [T_total/world, D] slice of the sum."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    t_local = partial.shape[0] // world
    if dist.get_backend(group) == "nccl":
        out = torch.empty(t_local, partial.shape[1], dtype=partial.dtype, device=partial.device)
        dist.reduce_scatter_tensor(out, partial.contiguous(), group=group)
        return out
    dist.all_reduce(partial, group=group)        # CPU test backends without reduce-scatter
    return partial[rank * t_local:(rank + 1) * t_local].clone()


def sharded_forward(x_local: torch.Tensor, select_fn: Callable, eval_fn: Callable, num_experts: int,
                    group=None, static_shapes: bool = True) -> torch.Tensor:
    """x_local [T_local, D] (same T_local on every rank) -> fp32 [T_local, D_out].

    select_fn(x_local) -> (ids [T_local, HK] global expert ids, weights fp32 [T_local, HK]);
    eval_fn(x_all [T, D], ids int32 [T, cap], weights [T, cap], counts int32 [T]) -> fp32 [T, D_out]
    evaluated against this rank's row shard (ids are local row numbers)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    rows = rows_per_rank(num_experts, world)
    t_local = x_local.shape[0]
    x_all = torch.empty(world * t_local, x_local.shape[1], dtype=x_local.dtype, device=x_local.device)
    dist.all_gather_into_tensor(x_all, x_local.contiguous(), group=group)
    ids, w = select_fn(x_local)
    if static_shapes:
        recv = exchange_static(route_tuples_blocks(ids, w, rows, world), group)
        p_ids, p_w, p_cnt = lists_from_blocks(recv, t_local, ids.shape[1])
    else:
        send, counts = route_tuples(ids, w, rank * t_local, rows, world)
        recv = exchange(send, counts, group)
        p_ids, p_w, p_cnt = pack_received(recv, world * t_local)
    partial = eval_fn(x_all, p_ids, p_w, p_cnt)
    return reduce_scatter_rows(partial, group)


class ShardedPEER:
    """The expert-parallel layer on the CUDA kernels.  `layer` is a `PEER` module whose small
    weights are replicated and whose expert tables hold only this rank's rows
    (`expert_down.weight` / `expert_up.weight` of shape [num_experts/world, D]);
    `num_experts` and `product_key_dim` describe the FULL table."""

    def __init__(self, layer, group=None, exchange: str = "nccl", freeze_keys: bool = True):
        if exchange not in ("nccl", "direct"):
            raise ValueError("exchange is 'nccl' (three collectives) or 'direct' (stores into the peers' memory)")
        self.layer, self.group, self.exchange = layer, group, exchange
        # the layer is evaluated, never trained, here: the sub-keys' derived tables are prepared once per plan
        # (pass freeze_keys=False if the sub-keys are updated in place between steps)
        self.freeze_keys = freeze_keys
        self._buf, self._buf_key, self.last_counts = None, None, None
        self._xchg = None                 # direct exchange: the library's handle of this rank's region
        self.world = dist.get_world_size(group)
        self.rows = rows_per_rank(layer.num_experts, self.world)
        if layer.expert_down.weight.shape[0] != self.rows:
            raise ValueError(f"this rank must hold {self.rows} table rows, has {layer.expert_down.weight.shape[0]}")

    @classmethod
    def build(cls, module_kwargs: dict, small_weights: dict, down_local: torch.Tensor, up_local: torch.Tensor,
              group=None, index_mode: str = "product", down_scale=None, up_scale=None, exchange: str = "nccl"):
        """Assemble the layer from replicated small weights (state-dict names of the module) and this
        rank's table rows, without ever materialising the full tables."""
        from .peer import PEER
        with torch.device("meta"):
            layer = PEER(**module_kwargs)
        layer.expert_down = torch.nn.Embedding(down_local.shape[0], down_local.shape[1], _weight=down_local)
        layer.expert_up = torch.nn.Embedding(up_local.shape[0], up_local.shape[1], _weight=up_local)
        layer.load_state_dict({k: v for k, v in small_weights.items() if not k.startswith("expert_")},
                              strict=False, assign=True)
        layer.expert_down_scale, layer.expert_up_scale = down_scale, up_scale
        layer.eval().requires_grad_(False)
        layer.index_mode = index_mode
        return cls(layer, group, exchange)

    @torch.no_grad()
    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        """[B, S, D] of THIS rank's tokens (the same B*S on every rank) -> [B, S, D_out].  Per step: three
        NCCL collectives (all-gather of x, all-to-all of the tuple buckets, reduce-scatter of the fp32
        partial sums) and the library's kernels between them: query + selection, routing, packing, partial
        expert evaluation.  Buffers are kept between calls of the same shape."""
        L = self.layer
        B, S, D = hidden_states.shape
        T = B * S
        world, rank = self.world, dist.get_rank(self.group)
        x = hidden_states.contiguous().view(T, D)
        w = L._weights()
        op = L._operator(x.device, x.dtype, T * world)
        HK = L.num_heads * L.num_experts_per_tok
        key = (T, D, x.dtype, str(x.device), id(op)) + tuple(0 if v is None else v.data_ptr() for v in w.values())
        if self._buf_key != key:
            self._plan(op, w, T, D, x.dtype, x.device)
            self._buf_key = key
        b = self._buf
        stream = C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)
        lib, h = op.lib, op.handle
        if self.exchange == "direct":
            return self._forward_direct(x, b, lib, h, stream, T, HK).view(B, S, -1)
        dist.all_gather_into_tensor(b["x_all"], x, group=self.group)
        # this rank's rows of x_all are x: the selection reads them there, so every pointer below is fixed
        _lib.check(lib.peer_select_tokens(h, b["tensors_ref"], T, b["ids_p"], b["wts_p"], stream), h)
        _lib.check(lib.peer_route_tuples(b["ids_p"], b["wts_p"], T, HK, self.rows, world, b["send_p"], stream), None)
        dist.all_to_all_single(b["recv"], b["send"], group=self.group)
        _lib.check(lib.peer_gather_eval_routed(h, b["x_all_p"], b["recv_p"], world, T, b["down_p"], b["up_p"], b["ds_p"],
                                               b["us_p"], self.rows, b["partial_p"], stream), h)
        self.last_counts = b["counts_view"]          # tuples this rank evaluated, per token (device tensor)
        out = reduce_scatter_rows(b["partial"], self.group)
        return out.to(hidden_states.dtype).view(B, S, -1)

    def _forward_direct(self, x, b, lib, h, stream, T, HK):
        """One step with the library's direct exchange (`peer_xchg_*`): x, the tuples and the partial sums go
        to the peers by stores into their memory; no collective is called.  Waits on a peer are bounded on
        the device; `check_exchange()` reports one that ran out."""
        b["tensors"].x = x.data_ptr()                 # the selection reads the caller's tensor
        out = torch.empty(T, self.layer.output_dim, dtype=x.dtype, device=x.device)
        _lib.check(lib.peer_xchg_forward(self._xchg, h, b["tensors_ref"], b["ids_p"], b["wts_p"], self.rows,
                                         b["partial_p"], C.c_void_p(out.data_ptr()), stream), None)
        self.last_counts = None                       # read on demand: received_counts()
        return out

    def received_counts(self) -> torch.Tensor:
        """int32 [world, T]: how many tuples each token brought to this rank in the last step."""
        if self._xchg is None:
            return self.last_counts
        b = self._buf
        dev = b["counts"].device
        stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        with torch.cuda.device(dev):
            _lib.check(_lib.load().peer_xchg_counts(self._xchg, C.c_void_p(b["counts"].data_ptr()), stream), None)
        return b["counts"]

    def check_exchange(self) -> None:
        """Direct exchange only: synchronises the stream and raises if a wait for a peer's data ran out."""
        if self._xchg is not None:
            dev = self.layer.expert_down.weight.device
            stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
            with torch.cuda.device(dev):
                _lib.check(_lib.load().peer_xchg_status(self._xchg, stream), None)

    def close(self) -> None:
        """Releases the direct exchange's region.  Collective: every rank calls it, after its last step."""
        if self._xchg is not None:
            torch.cuda.synchronize()
            dist.barrier(self.group)              # no peer still writes into the region
            _lib.load().peer_xchg_destroy(self._xchg)
            self._xchg = None
            self._buf_key = None

    def _plan_direct(self, T, D, dtype, dev):
        """The rank's exchange region for this step shape: created, its IPC handle exchanged over the process
        group (host side), the peers' regions mapped.  Collective; if any rank fails, every rank raises."""
        from .peer import _DT
        lib = _lib.load()
        if self._xchg is not None:
            self.close()
        L, world, rank = self.layer, self.world, dist.get_rank(self.group)
        xh, err, mine = C.c_void_p(), None, b""
        with torch.cuda.device(dev):
            try:
                _lib.check(lib.peer_xchg_create(world, rank, T, L.num_heads * L.num_experts_per_tok, D, L.output_dim,
                                                _DT[dtype], C.byref(xh)), None)
                buf = (C.c_ubyte * 64)()
                _lib.check(lib.peer_xchg_export(xh, buf), None)
                mine = bytes(buf)
            except (RuntimeError, ValueError) as e:
                err = e
            handles = [None] * world
            dist.all_gather_object(handles, mine, group=self.group)
            if err is None:
                if all(len(hb) == 64 for hb in handles):
                    try:
                        _lib.check(lib.peer_xchg_attach(xh, b"".join(handles)), None)
                    except (RuntimeError, ValueError) as e:
                        err = e
                else:
                    err = RuntimeError("a peer could not create its exchange region")
            bad = torch.tensor([0 if err is None else 1], device=dev)
            dist.all_reduce(bad, op=dist.ReduceOp.MAX, group=self.group)   # also: every region is mapped before anyone writes
            if int(bad):
                if xh.value:
                    lib.peer_xchg_destroy(xh)
                raise RuntimeError(f"direct exchange unavailable: {err if err is not None else 'a peer failed to set it up'}")
        self._xchg = xh

    def _plan(self, op, w, T, D, dtype, dev):
        """Buffers and pre-built C arguments of one step shape: a step is then three collectives and three library
        calls with no allocation and no argument marshalling in between (the host's time to enqueue a step is what
        bounds a decode-shaped batch)."""
        L, world, rank = self.layer, self.world, dist.get_rank(self.group)
        HK = L.num_heads * L.num_experts_per_tok
        op.freeze_keys(self.freeze_keys)
        x_all = torch.empty(world * T, D, dtype=dtype, device=dev)
        send = torch.empty(world, block_words(T, HK), dtype=torch.int32, device=dev)
        recv = torch.empty(world, block_words(T, HK), dtype=torch.int32, device=dev)
        partial = torch.empty(world * T, L.output_dim, dtype=torch.float32, device=dev)
        ids = torch.empty(T, HK, dtype=torch.int32, device=dev)
        wts = torch.empty(T, HK, dtype=torch.float32, device=dev)
        x_mine = x_all[rank * T:(rank + 1) * T]
        tensors = op._tensors(x_mine, w, None)
        vp = lambda t: None if t is None else C.c_void_p(t.data_ptr())
        self._buf = dict(x_all=x_all, send=send, recv=recv, partial=partial, ids=ids, wts=wts, tensors=tensors,
                         tensors_ref=C.byref(tensors), ids_p=vp(ids), wts_p=vp(wts), send_p=vp(send), recv_p=vp(recv),
                         x_all_p=vp(x_all), partial_p=vp(partial), down_p=vp(w["expert_down"]), up_p=vp(w["expert_up"]),
                         ds_p=vp(w["down_scale"]), us_p=vp(w["up_scale"]), counts_view=recv[:, 2 * T * HK:],
                         counts=torch.zeros(world, T, dtype=torch.int32, device=dev))
        if self.exchange == "direct":
            self._plan_direct(T, D, dtype, dev)

    def nvlink_bytes_per_step(self, tokens_per_rank: int) -> dict:
        """Bytes each rank SENDS per step, by collective (fixed-shape buckets: the all-to-all carries
        the padded capacity, not only the tuples in use)."""
        L, G, T = self.layer, self.world, tokens_per_rank
        HK = L.num_heads * L.num_experts_per_tok
        eb = L.query_proj.weight.element_size()
        return {"all_gather_x": (G - 1) * T * L.input_dim * eb,
                "all_to_all_blocks": (G - 1) * block_words(T, HK) * 4,
                "all_to_all_tuples_in_use": (G - 1) * T * HK * 8 // G,
                "reduce_scatter_partials_fp32": (G - 1) * T * L.output_dim * 4}

    __call__ = forward
