"""Expert-parallel PEER: the expert tables are split by rows over the ranks of a process group.

The reference has no distributed PEER (its multi-GPU story is data parallelism through
Accelerate, llm/training/train.py:472-476, 638-640; expert sharding is announced in
docs/paper/paper.tex:446 and listed as future work in docs/CUTLASS_KERNEL.md:181).  This is
the layer for tables that do not fit, or should not be replicated, on every GPU:

  rank r owns rows [r*N/G, (r+1)*N/G) of expert_down / expert_up; the small weights (query
  projection, LayerNorm, sub-keys) are replicated; every rank brings its own tokens.

  1. all-gather of the activations (every owner needs x_t for the tuples it will receive);
  2. each rank selects for ITS tokens (query projection + product-key retrieval kernels);
  3. the selected (token, expert id, weight) tuples are bucketed by owner and exchanged with one
     all-to-all (counts first, then the packed tuples);
  4. each rank evaluates the tuples it received against its row shard (one kernel, fp32 partial
     sums per token);
  5. reduce-scatter of the partial sums gives every rank the outputs of its own tokens.

Result: identical to the single-device layer on the concatenated batch, up to fp32 summation
order.  The exchange logic exists twice: as plain tensor code (`route_tuples*`, `pack_received*`)
that runs on any device and is tested with CPU ranks over gloo, and as two kernels of the library
(`peer_route_tuples`, `peer_pack_tuples`, wrapped by `route_tuples_native` / `pack_received_native`)
that `ShardedPEER` uses on the GPU: one launch each instead of some twenty-five small tensor
operations, same buckets and lists (a GPU test compares the two forms).
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


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
# Fixed-shape variant of the exchange: every rank sends every peer a bucket of the same capacity
# (T_local*HK tuples, the worst case; 24 KB per peer at 8 tokens x 256 entries), unused slots carry
# token -1.  One all-to-all, no counts to exchange, no host synchronisation, shapes that never change
# from step to step.
# ---------------------------------------------------------------------------
def route_tuples_static(ids: torch.Tensor, weights: torch.Tensor, token_offset: int, rows: int, world: int) -> torch.Tensor:
    """-> int32 [world, T*HK, 3] buckets of (global token | -1, local row, weight bits)."""
    T, HK = ids.shape
    n = T * HK
    dev = ids.device
    flat = ids.reshape(-1).to(torch.int64)
    owner = torch.div(flat, rows, rounding_mode="floor")
    order = torch.argsort(owner, stable=True)
    owner_s = owner[order]
    # fixed-size histogram (torch.bincount would read its bin count back to the host)
    counts = torch.zeros(world, dtype=torch.int64, device=dev).scatter_add_(0, owner, torch.ones_like(owner))
    start = torch.cumsum(counts, 0) - counts
    pos = torch.arange(n, device=dev) - start[owner_s]
    tok = (torch.arange(T, device=dev, dtype=torch.int64).repeat_interleave(HK) + token_offset)[order]
    send = torch.full((world, n, 3), -1, dtype=torch.int32, device=dev)
    send[owner_s, pos, 0] = tok.to(torch.int32)
    send[owner_s, pos, 1] = (flat - owner * rows)[order].to(torch.int32)
    send[owner_s, pos, 2] = weights.reshape(-1).to(torch.float32).view(torch.int32)[order]
    return send


def exchange_static(send: torch.Tensor, group=None) -> torch.Tensor:
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv


def pack_received_static(recv: torch.Tensor, n_tokens: int, cap: int):
    """Buckets int32 [world, m, 3] with -1 padding -> (ids int32 [T, cap], weights fp32 [T, cap],
    counts int32 [T]); cap must be at least the longest per-token list (HK always is)."""
    dev = recv.device
    flat = recv.reshape(-1, 3)
    tok = flat[:, 0].to(torch.int64)
    key = torch.where(tok >= 0, tok, torch.full_like(tok, n_tokens))      # padding sorts behind every token
    order = torch.argsort(key, stable=True)
    key_s = key[order]
    counts = torch.zeros(n_tokens + 1, dtype=torch.int64, device=dev).scatter_add_(0, key_s, torch.ones_like(key_s))
    start = torch.cumsum(counts, 0) - counts
    pos = torch.clamp(torch.arange(key_s.numel(), device=dev) - start[key_s], max=cap - 1)
    ids = torch.zeros(n_tokens + 1, cap, dtype=torch.int32, device=dev)    # row T collects the padding
    w = torch.zeros(n_tokens + 1, cap, dtype=torch.float32, device=dev)
    ids[key_s, pos] = flat[order, 1]
    w[key_s, pos] = flat[order, 2].contiguous().view(torch.float32)
    return ids[:n_tokens], w[:n_tokens], torch.clamp(counts[:n_tokens], max=cap).to(torch.int32)


def route_tuples_native(ids32: torch.Tensor, weights: torch.Tensor, token_offset: int, rows: int, world: int,
                        send: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`route_tuples_static` as one kernel (CUDA tensors): ids int32 [T, HK], weights fp32 [T, HK] ->
    int32 [world, T*HK, 3]; a bucket keeps (token, slot) order, padding carries token -1."""
    import ctypes as C
    from . import _lib
    T, HK = ids32.shape
    if ids32.dtype != torch.int32 or weights.dtype != torch.float32 or not ids32.is_cuda:
        raise TypeError("route_tuples_native takes CUDA tensors: int32 ids and fp32 weights")
    if send is None:
        send = torch.empty(world, T * HK, 3, dtype=torch.int32, device=ids32.device)
    lib = _lib.load()
    with torch.cuda.device(ids32.device):
        rc = lib.peer_route_tuples(C.c_void_p(ids32.contiguous().data_ptr()), C.c_void_p(weights.contiguous().data_ptr()),
                                   T, HK, int(token_offset), int(rows), int(world), T * HK, C.c_void_p(send.data_ptr()),
                                   C.c_void_p(torch.cuda.current_stream(ids32.device).cuda_stream))
    _lib.check(rc, None)
    return send


def pack_received_native(recv: torch.Tensor, n_tokens: int, cap: int, out=None):
    """`pack_received_static` as one kernel: buckets int32 [world, m, 3] -> (ids int32 [T, cap], weights fp32
    [T, cap], counts int32 [T]), lists in (source rank, position) order."""
    import ctypes as C
    from . import _lib
    if recv.dtype != torch.int32 or not recv.is_cuda or not recv.is_contiguous():
        raise TypeError("pack_received_native takes a contiguous CUDA int32 tensor")
    world, m, _ = recv.shape
    dev = recv.device
    if out is None:
        out = (torch.empty(n_tokens, cap, dtype=torch.int32, device=dev),
               torch.empty(n_tokens, cap, dtype=torch.float32, device=dev),
               torch.empty(n_tokens, dtype=torch.int32, device=dev))
    ids, w, cnt = out
    lib = _lib.load()
    with torch.cuda.device(dev):
        rc = lib.peer_pack_tuples(C.c_void_p(recv.data_ptr()), int(world), int(m), int(n_tokens), int(cap),
                                  C.c_void_p(ids.data_ptr()), C.c_void_p(w.data_ptr()), C.c_void_p(cnt.data_ptr()),
                                  C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    _lib.check(rc, None)
    return ids, w, cnt


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
        recv = exchange_static(route_tuples_static(ids, w, rank * t_local, rows, world), group)
        p_ids, p_w, p_cnt = pack_received_static(recv, world * t_local, ids.shape[1])
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

    def __init__(self, layer, group=None):
        self.layer, self.group = layer, group
        self._buf, self._buf_key, self.last_counts = None, None, None
        self.world = dist.get_world_size(group)
        self.rows = rows_per_rank(layer.num_experts, self.world)
        if layer.expert_down.weight.shape[0] != self.rows:
            raise ValueError(f"this rank must hold {self.rows} table rows, has {layer.expert_down.weight.shape[0]}")

    @classmethod
    def build(cls, module_kwargs: dict, small_weights: dict, down_local: torch.Tensor, up_local: torch.Tensor,
              group=None, index_mode: str = "product", down_scale=None, up_scale=None):
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
        return cls(layer, group)

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
        key = (T, D, x.dtype, str(x.device))
        if self._buf_key != key:
            dev = x.device
            self._buf = dict(
                x_all=torch.empty(world * T, D, dtype=x.dtype, device=dev),
                send=torch.empty(world, T * HK, 3, dtype=torch.int32, device=dev),
                recv=torch.empty(world, T * HK, 3, dtype=torch.int32, device=dev),
                lists=(torch.empty(world * T, HK, dtype=torch.int32, device=dev),
                       torch.empty(world * T, HK, dtype=torch.float32, device=dev),
                       torch.empty(world * T, dtype=torch.int32, device=dev)))
            self._buf_key = key
        b = self._buf
        dist.all_gather_into_tensor(b["x_all"], x, group=self.group)
        ids, wts = op.select_tokens(x, w)
        route_tuples_native(ids, wts, rank * T, self.rows, world, b["send"])
        dist.all_to_all_single(b["recv"], b["send"], group=self.group)
        p_ids, p_w, p_cnt = pack_received_native(b["recv"], world * T, HK, b["lists"])
        partial = op.gather_eval_partial(b["x_all"], p_ids, p_w, p_cnt, w["expert_down"], w["expert_up"],
                                         w["down_scale"], w["up_scale"])
        self.last_counts = p_cnt                  # tuples this rank evaluated, per token (device tensor)
        out = reduce_scatter_rows(partial, self.group)
        return out.to(hidden_states.dtype).view(B, S, -1)

    def nvlink_bytes_per_step(self, tokens_per_rank: int) -> dict:
        """Bytes each rank SENDS per step, by collective (fixed-shape buckets: the all-to-all carries
        the padded capacity, not only the tuples in use)."""
        L, G, T = self.layer, self.world, tokens_per_rank
        HK = L.num_heads * L.num_experts_per_tok
        eb = L.query_proj.weight.element_size()
        return {"all_gather_x": (G - 1) * T * L.input_dim * eb,
                "all_to_all_buckets": (G - 1) * T * HK * 12,
                "all_to_all_tuples_in_use": (G - 1) * T * HK * 12 // G,
                "reduce_scatter_partials_fp32": (G - 1) * T * L.output_dim * 4}

    __call__ = forward
