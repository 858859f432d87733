"""Functional entry point with the argument list of the reference's
``peer_forward_cutlass`` (llm/models/kernels/peer_cutlass.py:135-151)."""
from __future__ import annotations

import math
from typing import Optional

import torch

from .peer import PeerOp

_OPS = {}


def peer_forward(x: torch.Tensor, query_weight: torch.Tensor, query_bias: Optional[torch.Tensor],
                 key_weight_1: torch.Tensor, key_weight_2: torch.Tensor, expert_weights_u: torch.Tensor,
                 expert_weights_v: torch.Tensor, num_heads: int, num_experts: int, expert_hidden_size: int,
                 top_k: int, dropout_rate: float = 0.0, layer_norm: bool = True,
                 ln_weight: Optional[torch.Tensor] = None, ln_bias: Optional[torch.Tensor] = None, *,
                 index_mode: str = "reference", activation: str = "gelu", norm_keys: bool = True,
                 norm_query: bool = True, u_scale: Optional[torch.Tensor] = None,
                 v_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [batch, seq, input_dim] -> new tensor [batch, seq, output_dim] of x's dtype.

    query_weight is [num_heads*query_dim, input_dim] (or [num_heads, query_dim, input_dim]);
    expert tables are [num_experts, input_dim] / [num_experts, output_dim] in fp32, bf16 or
    FP8-e4m3 (then ``u_scale`` / ``v_scale`` hold the per-row fp32 scales).  Unlike the
    reference wrapper nothing is cast or copied: tensors are used where they are."""
    if dropout_rate != 0.0:
        raise RuntimeError("peer_b200 is a forward (inference) path: dropout is not implemented")
    if x.device.type != "cuda":
        raise RuntimeError("peer_b200 runs on CUDA devices only (sm_100a); there is no CPU path")
    B, S, D = x.shape
    qw = query_weight.reshape(-1, D)
    query_dim = qw.shape[0] // num_heads
    n0, n1 = key_weight_1.shape[0], key_weight_2.shape[0]
    if n0 * n1 != num_experts:
        raise ValueError(f"key tables of {n0} and {n1} rows do not address {num_experts} experts")
    h = int(expert_hidden_size)
    if h < 1:
        raise ValueError(f"expert_hidden_size={expert_hidden_size}")
    # output width as the reference takes it (peer_cutlass.py:176): dimension 1 of a [N, output_dim, h] table;
    # a flattened [N, output_dim*h] table (the module's Embedding layout, experts.py:337-352) holds h values per
    # output column
    if expert_weights_v.dim() == 3:
        out_dim = expert_weights_v.shape[1]
        if expert_weights_v.shape[2] != h:
            raise ValueError(f"expert_weights_v is {tuple(expert_weights_v.shape)}, expected [N, output_dim, {h}]")
    else:
        if expert_weights_v.shape[-1] % h:
            raise ValueError(f"expert_weights_v rows of {expert_weights_v.shape[-1]} values do not hold {h} neurons")
        out_dim = expert_weights_v.shape[-1] // h
    u = expert_weights_u.reshape(num_experts, -1)
    v = expert_weights_v.reshape(num_experts, -1)
    if u.shape[1] != D * h or v.shape[1] != out_dim * h:
        raise ValueError(f"expert tables of {u.shape[1]} / {v.shape[1]} values per row do not match input_dim {D}, "
                         f"output_dim {out_dim} and {h} neurons per expert")
    key = (str(x.device), x.dtype, u.dtype, D, out_dim, num_heads, query_dim, n0, n1, top_k, layer_norm,
           index_mode, activation, norm_keys, norm_query, expert_hidden_size)
    T = B * S
    op = _OPS.get(key)
    if op is None or op.cfg.max_tokens < min(T, 16384):
        if op is not None:
            op.close()
        op = PeerOp(input_dim=D, output_dim=out_dim, num_heads=num_heads, query_dim=query_dim,
                    product_key_dim=(n0, n1), top_k=top_k, act_dtype=x.dtype, table_dtype=u.dtype,
                    activation=activation, norm_keys=norm_keys, norm_query=norm_query, layer_norm=layer_norm,
                    index_mode=index_mode, max_tokens=min(max(T, 1), 16384),
                    expert_hidden_size=expert_hidden_size, device=x.device)
        _OPS[key] = op
    w = dict(query_w=qw, query_b=None if query_bias is None else query_bias.reshape(-1),
             ln_w=None if ln_weight is None else ln_weight.reshape(-1)[:query_dim],
             ln_b=None if ln_bias is None else ln_bias.reshape(-1)[:query_dim],
             keys0=key_weight_1, keys1=key_weight_2, expert_down=u, expert_up=v,
             down_scale=u_scale, up_scale=v_scale)
    out = torch.empty(T, out_dim, dtype=x.dtype, device=x.device)
    op.forward(x.contiguous().view(T, D), w, out)
    return out.view(B, S, out_dim)


# the name the reference module imports (llm/models/experts.py:29)
peer_forward_cutlass = peer_forward
