"""Differentiable PEER forward: the library's kernels for the values, and for
the gradients of the expert stage; torch operations for the small rest.

The reference trains through its PyTorch forward (llm/models/experts.py:
288-384; llm/training/train.py:743-768), with autograd deriving every gradient.
Without dropout the whole layer is ONE autograd node (``_FusedLayer``): its forward is the inference path
unchanged, its backward the expert-stage gradient kernel plus a torch re-derivation of the score path.  With
dropout (training mode) the stages are separate nodes:

* query projection + LayerNorm: value from the library's query kernel (fp32);
  gradient by re-running ``F.linear`` / ``F.layer_norm`` in backward
  (``_ProjectQueries``);
* product-key selection: the library's select kernel, no gradient (indices);
  the reference reads the sub-keys through ``.data`` (experts.py:154), so they
  receive no gradient there either;
* the k selected scores per head are recomputed from the queries and the 2k
  selected sub-key rows with torch operations (differentiable in the queries),
  softmax, optional dropout of the expert activations (experts.py:366; a
  per-slot factor, folded into the weights because each expert has one neuron);
* expert evaluation: ``peer_gather_eval`` forward, ``peer_gather_eval_backward``
  backward (``_ExpertEval``): dense table gradients accumulated with vector
  reductions.  Rows that collect many contributions are summed in fp32 and
  rounded once to the parameters' dtype, which is what the reference's embedding
  backward does for a bf16 layer; where a batch brings only a few selections per
  row, a bf16 layer may sum in bf16 (half the traffic, one rounding per addend).
  ``module.table_grad_sums`` ("auto", "fp32", "table") decides; see
  ``_table_grad_plan``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


class _ProjectQueries(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, ln_w, ln_b, op, wdict, num_heads, query_dim):
        ctx.save_for_backward(x, weight, bias, ln_w, ln_b)
        ctx.shape = (num_heads, query_dim)
        return op.project_queries(x, wdict)                    # [T, H, Q] fp32, after LayerNorm

    @staticmethod
    def backward(ctx, grad_q):
        saved = ctx.saved_tensors
        H, Q = ctx.shape
        leaves = [None if t is None else t.detach().requires_grad_(need)
                  for t, need in zip(saved, ctx.needs_input_grad[:5])]
        x, weight, bias, ln_w, ln_b = leaves
        with torch.enable_grad():
            q = F.linear(x, weight, bias).float().view(x.shape[0], H, Q)
            if ln_w is not None:
                q = F.layer_norm(q, (Q,), ln_w.float(), None if ln_b is None else ln_b.float(), 1e-5)
        wanted = [t for t in leaves if t is not None and t.requires_grad]
        grads = iter(torch.autograd.grad(q, wanted, grad_q.contiguous())) if wanted else iter(())
        out = [next(grads) if (t is not None and t.requires_grad) else None for t in leaves]
        return (*out, None, None, None, None)


class _ExpertEval(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weights, ids32, down, up, op, plan=(torch.float32, None)):
        ctx.save_for_backward(x, weights, ids32, down, up)
        ctx.op = op
        ctx.plan = plan
        return op.gather_eval(x, ids32, weights.contiguous(), down, up)

    @staticmethod
    def backward(ctx, grad_out):
        x, weights, ids32, down, up = ctx.saved_tensors
        gdt, rows = ctx.plan
        gx, gw, gd, gu = ctx.op.gather_eval_backward(x, grad_out.contiguous(), ids32, weights.contiguous(), down, up,
                                                     grad_dtype=gdt, grad_rows=rows)
        need = ctx.needs_input_grad
        return (gx.to(x.dtype) if need[0] else None, gw if need[1] else None, None,
                _dense_grad(gd, down) if need[3] else None, _dense_grad(gu, up) if need[4] else None, None, None)


def _reachable_rows(module) -> int:
    """Rows the layer's ids can address.  With the reference's id arithmetic the first key dimension never
    gets its multiplier (experts.py:203-204), so ids stay below 1 + (n0 - 1) + sum_{d>0} (n_d - 1) * stride_d
    (n0 + n1 - 1 for a two-dimensional grid); a one-dimensional grid returns candidate positions (< top_k)."""
    dims = list(module.product_key_dim)
    if module.index_mode != "reference":
        return module.num_experts
    if len(dims) == 1:
        return min(module.num_experts, module.num_experts_per_tok)
    strides = [1] * len(dims)
    for d in range(len(dims) - 2, -1, -1):
        strides[d] = strides[d + 1] * dims[d + 1]
    return min(module.num_experts, 1 + (dims[0] - 1) + sum((dims[d] - 1) * strides[d] for d in range(1, len(dims))))


def _table_grad_plan(module, table, n_tokens: int):
    """(dtype of the sums, rows of the gradient tables).  bf16 sums exist for single-neuron experts of a bf16
    layer with rows of at most 4 KB; a bf16 running sum loses small addends once a row collects many
    contributions, so "auto" keeps them for batches with at most four selections per reachable row on average
    and never with the reference's id arithmetic, where a few thousand rows take all of them (about a thousand
    each at the 1 M-expert layer's batch).  With fp32 sums only the reachable rows get a buffer."""
    mode = getattr(module, "table_grad_sums", "auto")
    if mode not in ("auto", "fp32", "table"):
        raise ValueError(f"table_grad_sums={mode!r}: 'auto', 'fp32' or 'table'")
    reach = _reachable_rows(module)
    eligible = (module.expert_hidden_size == 1 and table.dtype == torch.bfloat16 and
                max(module.input_dim, module.output_dim) * table.element_size() <= 4096)
    per_row = n_tokens * module.num_heads * module.num_experts_per_tok / max(reach, 1)
    in_table = eligible and (mode == "table" or (mode == "auto" and module.index_mode != "reference" and per_row <= 4.0))
    if in_table:
        return table.dtype, module.num_experts            # summed straight into what becomes .grad
    return torch.float32, reach


def _dense_grad(compact: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    """Gradient of a whole table from sums over its first rows."""
    if compact.shape[0] == like.shape[0]:
        return compact.to(like.dtype)
    g = torch.zeros(like.shape, dtype=like.dtype, device=like.device)
    g[:compact.shape[0]] = compact
    return g


def _key_grid(module):
    dims = list(module.product_key_dim)
    strides = [1] * len(dims)                               # true row-major strides of the key grid
    for d in range(len(dims) - 2, -1, -1):
        strides[d] = strides[d + 1] * dims[d + 1]
    return dims, strides


def _selected_scores(module, q, idx):
    """Scores of the selected experts from queries q [T,H,Q] (after LayerNorm) and the per-dimension indices
    idx[d] [T,H,k]: sum_d q_d . k_d[idx_d], with the normalisations of experts.py:153-163.  Differentiable in
    q; the sub-keys are read detached, as the reference reads them through ``.data``."""
    nd = len(idx)
    width = module.query_dim // nd
    scores = 0
    for d in range(nd):
        qd = q[..., d * width:(d + 1) * width]
        kd = module.sub_keys[d].detach().float()
        if module.norm_keys:
            kd = F.normalize(kd, dim=-1)
        if module.norm_query:
            qd = F.normalize(qd, dim=-1)
        scores = scores + (qd.unsqueeze(2) * kd[idx[d]]).sum(-1)
    return scores


class _FusedLayer(torch.autograd.Function):
    """The whole layer as one node: forward is the inference path (query, select and expert kernels, with the
    selected experts' grid positions as an extra output); backward runs the expert-stage gradient kernel and
    re-derives the score path (projection, LayerNorm, normalisation, the k selected scores, softmax) with torch
    operations to push the weight gradients back to x and the query parameters."""

    @staticmethod
    def forward(ctx, x, weight, bias, ln_w, ln_b, down, up, module):
        T = x.shape[0]
        H, k = module.num_heads, module.num_experts_per_tok
        op = module._operator(x.device, x.dtype, T)
        out = torch.empty(T, module.output_dim, dtype=x.dtype, device=x.device)
        ids = torch.empty(T, H, k, dtype=torch.int64, device=x.device)
        sc = torch.empty(T, H, k, dtype=torch.float32, device=x.device)
        pid = torch.empty(T, H, k, dtype=torch.int32, device=x.device)
        op.forward(x, module._weights(), out, ids, sc, pid)
        ctx.save_for_backward(x, weight, bias, ln_w, ln_b, down, up, ids, sc, pid)
        ctx.module, ctx.op = module, op
        ctx.mark_non_differentiable(ids, sc)
        return out, ids, sc

    @staticmethod
    def backward(ctx, grad_out, _gi, _gs):
        x, weight, bias, ln_w, ln_b, down, up, ids, sc, pid = ctx.saved_tensors
        module, op = ctx.module, ctx.op
        T = x.shape[0]
        H, Q, k = module.num_heads, module.query_dim, module.num_experts_per_tok
        need = ctx.needs_input_grad
        weights = torch.softmax(sc, dim=-1).view(T, H * k)
        gdt, rows = _table_grad_plan(module, down, T)
        gx, gw, gd, gu = op.gather_eval_backward(x, grad_out.contiguous(), ids.view(T, H * k).to(torch.int32), weights,
                                                 down, up, grad_dtype=gdt, grad_rows=rows)
        # score path: d(loss)/d(weights) = gw, pushed through softmax, the selected scores and the query path
        leaves = [None if t is None else t.detach().requires_grad_(n)
                  for t, n in zip((x, weight, bias, ln_w, ln_b), need[:5])]
        wanted = [t for t in leaves if t is not None and t.requires_grad]
        got = iter(())
        if wanted:
            with torch.enable_grad():                    # projection and LayerNorm again, as torch operations
                q = F.linear(leaves[0], leaves[1], leaves[2]).float().view(T, H, Q)
                if leaves[3] is not None:
                    q = F.layer_norm(q, (Q,), leaves[3].float(), None if leaves[4] is None else leaves[4].float(), 1e-5)
            gq = op.select_backward(q.detach().contiguous(), [p.detach() for p in module.sub_keys], pid.view(T, H, k),
                                    sc, gw.view(T, H, k).contiguous())
            got = iter(torch.autograd.grad(q, wanted, gq))
        grads = [next(got) if (t is not None and t.requires_grad) else None for t in leaves]
        if need[0]:
            grads[0] = (gx + grads[0].float()).to(x.dtype)
        return (*grads, _dense_grad(gd, down) if need[5] else None, _dense_grad(gu, up) if need[6] else None, None)


def peer_forward_autograd(module, hidden_states: torch.Tensor) -> torch.Tensor:
    """Forward of ``module`` (a ``llm720_b200.PEER``) that records an autograd graph."""
    w = module._weights()
    if w["down_scale"] is not None:
        raise RuntimeError("quantised (FP8) expert tables are inference-only: no backward pass")
    B, S, _ = hidden_states.shape
    T = B * S
    x = hidden_states.contiguous().view(T, module.input_dim)
    ln = module.query_layer_norm
    if not (module.training and module.dropout.p > 0):
        out, ids, sc = _FusedLayer.apply(x, module.query_proj.weight, module.query_proj.bias,
                                         None if ln is None else ln.weight, None if ln is None else ln.bias,
                                         module.expert_down.weight, module.expert_up.weight, module)
        if module.track_indices:
            module._stash(ids, sc, B, S)
        return out.view(B, S, module.output_dim)
    return _forward_with_dropout(module, x, w, B, S)


def _forward_with_dropout(module, x, w, B, S):
    """Training mode with dropout of the expert activations (experts.py:366): the stages as separate autograd
    nodes, so that the per-slot dropout factor can sit between the softmax and the expert stage."""
    if module.expert_hidden_size != 1:
        raise RuntimeError("dropout with expert_hidden_size > 1 is not implemented (it acts on every neuron)")
    T = B * S
    dt = x.dtype
    H, Q, k = module.num_heads, module.query_dim, module.num_experts_per_tok
    dims, strides = _key_grid(module)
    nd = len(dims)
    op = module._operator(x.device, dt, T)
    ln = module.query_layer_norm
    q = _ProjectQueries.apply(x, module.query_proj.weight, module.query_proj.bias,
                              None if ln is None else ln.weight, None if ln is None else ln.bias, op, w, H, Q)
    keys = [p.detach() for p in module.sub_keys]
    with torch.no_grad():
        sel = module._product_operator(x.device, dt, T)
        if nd == 2:
            pid, _ = sel.select(q.detach(), keys[0], keys[1])                  # sum_d i_d * stride_d
        else:
            pid, _ = sel.select_nd(q.detach(), keys)
        idx = [torch.div(pid, strides[d], rounding_mode="floor") % dims[d] for d in range(nd)]
        if module.index_mode == "reference" and nd > 1:      # the first dimension loses its multiplier
            flat = idx[0] + sum(idx[d] * strides[d] for d in range(1, nd))
        elif module.index_mode == "reference":               # 1-D: positions in the candidate list (experts.py:197-200)
            flat = torch.arange(k, device=pid.device).expand_as(pid).contiguous()
        else:
            flat = pid
    scores = _selected_scores(module, q, idx)
    weights = torch.softmax(scores, dim=-1)
    weights = weights * F.dropout(torch.ones_like(weights), module.dropout.p, True)
    out = _ExpertEval.apply(x, weights.view(T, H * k), flat.to(torch.int32).view(T, H * k),
                            module.expert_down.weight, module.expert_up.weight, op,
                            _table_grad_plan(module, module.expert_down.weight, T))
    if module.track_indices:
        module._stash(flat, scores.detach(), B, S)
    return out.view(B, S, module.output_dim)
