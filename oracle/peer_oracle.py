"""CPU oracle for the PEER forward path.  TEST INFRASTRUCTURE ONLY.

This file restates, with plain PyTorch CPU ops, what the reference's PyTorch
PEER forward computes (llm/models/experts.py:138-384 of wrmedford/llm720).  It
exists so the CUDA kernels can be checked against it.  Only the test-suite, the
smoke check and the CPU-baseline leg of the benchmark may import it; the
product package never does.

Parity status: PINNED.  `tests/golden/make_golden.py` imports the reference
module itself, runs it next to this restatement and requires bit-identical
indices, scores and outputs before it writes the committed golden files;
`tests/test_oracle_golden.py` re-checks the restatement against those files.

Two deliberate extensions over the reference, both off by default:
  * ``index_mode="product"``: the flat expert id is ``i0 * n1 + i1`` (true
    product-key addressing).  The reference computes ``i0 + i1`` because the
    first dimension's indices never get their multiplier
    (experts.py:203-204 initialises the running index with the raw first-dim
    indices, :230 only scales later dimensions).  ``index_mode="reference"``
    reproduces that.
  * tables may be stored in bf16 or FP8-e4m3 (+ per-row fp32 scale); gathered
    rows are widened to the compute dtype before the reference's arithmetic.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


@dataclass
class PeerWeights:
    """Parameter set of one PEER layer, named after the reference state-dict
    (experts.py:87-108): query_proj.{weight,bias}, query_layer_norm.{weight,bias},
    sub_keys.{0,1}, expert_down.weight, expert_up.weight."""

    query_w: torch.Tensor            # [H*Q, D]
    query_b: Optional[torch.Tensor]  # [H*Q]
    ln_w: Optional[torch.Tensor]     # [Q]   (None when batch_norm_query=False)
    ln_b: Optional[torch.Tensor]     # [Q]
    sub_keys: List[torch.Tensor]     # each [n_i, Q/len]
    expert_down: torch.Tensor        # [N, D]      any storage dtype
    expert_up: torch.Tensor          # [N, D_out]  any storage dtype
    down_scale: Optional[torch.Tensor] = None  # [N] fp32, FP8 tables only
    up_scale: Optional[torch.Tensor] = None    # [N] fp32, FP8 tables only


@dataclass
class PeerShape:
    """Constructor arguments of the reference module (experts.py:46-61)."""

    input_dim: int
    output_dim: int
    num_experts: int
    num_experts_per_tok: int = 16
    num_heads: int = 8
    expert_hidden_size: int = 1
    query_dim: int = 256
    product_key_dim: Sequence[int] = field(default_factory=lambda: [32, 32])
    activation: str = "gelu"
    norm_keys: bool = True
    norm_query: bool = True
    batch_norm_query: bool = True


def candidates_per_dim(top_k: int, dim_size: int, num_dims: int) -> int:
    """k' of experts.py:168-187: ceil(k^(1/dims))+2, raised to k when the
    sub-key table is at least k rows, capped by the table size, at least 1."""
    base = int(math.ceil(top_k ** (1.0 / num_dims))) + 2
    kp = min(base, dim_size)
    kp = min(max(kp, top_k if dim_size >= top_k else dim_size), dim_size)
    return max(1, kp)


def sub_key_scores(queries: torch.Tensor, sub_keys: Sequence[torch.Tensor],
                   norm_keys: bool = True, norm_query: bool = True) -> List[torch.Tensor]:
    """Per-dimension cosine scores, experts.py:149-163.  queries [B,S,H,Q]."""
    nd = len(sub_keys)
    width = queries.shape[-1] // nd
    out = []
    for i, keys in enumerate(sub_keys):
        q = queries[..., i * width:(i + 1) * width]
        k = keys.detach()
        if norm_keys:
            k = F.normalize(k, dim=-1)
        if norm_query:
            q = F.normalize(q, dim=-1)
        out.append(torch.matmul(q, k.t()))
    return out


def select(queries: torch.Tensor, sub_keys: Sequence[torch.Tensor], top_k: int,
           product_key_dim: Sequence[int], norm_keys: bool = True, norm_query: bool = True,
           index_mode: str = "reference") -> Tuple[torch.Tensor, torch.Tensor]:
    """Product-key retrieval, experts.py:138-285.

    Returns (ids int64 [B,S,H,k], raw scores [B,S,H,k]) sorted by descending
    score.  ``index_mode``: see the module docstring."""
    if index_mode not in ("reference", "product"):
        raise ValueError(index_mode)
    B, S, H, _ = queries.shape
    nd = len(product_key_dim)
    if nd == 0:
        raise ValueError("no product key dimensions")
    scores = sub_key_scores(queries, sub_keys, norm_keys, norm_query)

    top_s, top_i = [], []
    for d, sc in enumerate(scores):                       # experts.py:176-192
        kp = candidates_per_dim(top_k, product_key_dim[d], nd)
        s, i = torch.topk(sc, k=kp, dim=-1)
        top_s.append(s)
        top_i.append(i)

    if nd == 1:                                           # experts.py:197-200
        k = min(top_k, top_s[0].shape[-1])
        fs, fi = torch.topk(top_s[0], k=k, dim=-1)
        # the reference returns the positions inside its candidate list here (0..k-1), not key indices;
        # "product" mode returns the keys those positions stand for
        return (torch.gather(top_i[0], -1, fi) if index_mode == "product" else fi), fs

    mult = [1] * nd                                       # experts.py:207-210
    for d in range(nd - 2, -1, -1):
        mult[d] = mult[d + 1] * product_key_dim[d + 1]

    run_s = top_s[0]
    run_i = top_i[0] * mult[0] if index_mode == "product" else top_i[0]   # :203-204
    for d in range(1, nd):                                # experts.py:214-265
        cs = run_s.unsqueeze(-1) + top_s[d].unsqueeze(-2)
        ci = run_i.unsqueeze(-1) + top_i[d].unsqueeze(-2) * mult[d]
        fs = cs.reshape(B, S, H, -1)
        fi = ci.reshape(B, S, H, -1)
        n = fs.shape[-1]
        keep = min(top_k * 4, n) if d < nd - 1 else min(top_k, n)
        keep = max(1, keep)
        if keep == n:
            run_s, run_i = fs, fi
        else:
            run_s, pos = torch.topk(fs, k=keep, dim=-1)
            run_i = torch.gather(fi, dim=-1, index=pos)
    k = min(top_k, run_i.shape[-1])                       # experts.py:267-270
    return run_i[..., :k], run_s[..., :k]


def make_queries(x: torch.Tensor, w: PeerWeights, shape: PeerShape) -> torch.Tensor:
    """Query projection + shared LayerNorm, experts.py:302-308.  x [B,S,D]."""
    B, S, _ = x.shape
    q = F.linear(x, w.query_w, w.query_b).view(B, S, shape.num_heads, shape.query_dim)
    if shape.batch_norm_query:
        q = F.layer_norm(q, (shape.query_dim,), w.ln_w, w.ln_b, 1e-5)
    return q


def _rows(table: torch.Tensor, scale: Optional[torch.Tensor], ids: torch.Tensor,
          dtype: torch.dtype) -> torch.Tensor:
    """Embedding lookup (experts.py:332-334) widened to the compute dtype.
    FP8 rows are multiplied by their per-row scale after widening."""
    rows = F.embedding(ids, table) if table.dtype == dtype else table[ids].to(dtype)
    if scale is not None:
        rows = rows * scale[ids].to(dtype).unsqueeze(-1)
    return rows


def evaluate_experts(x: torch.Tensor, ids: torch.Tensor, scores: torch.Tensor,
                     w: PeerWeights, shape: PeerShape) -> torch.Tensor:
    """Softmax over k, gather, down-projection, activation, up-projection,
    score weighting and the two reductions: experts.py:327-382 (eval mode, so
    dropout is the identity).  x [B,S,D]; ids/scores [B,S,H,k]."""
    B, S, _ = x.shape
    H, k, h = shape.num_heads, ids.shape[-1], shape.expert_hidden_size
    p = F.softmax(scores, dim=-1)
    down = _rows(w.expert_down, w.down_scale, ids, x.dtype).view(B, S, H, k, h, shape.input_dim)
    up = _rows(w.expert_up, w.up_scale, ids, x.dtype).view(B, S, H, k, shape.output_dim, h)
    xe = x.unsqueeze(2).unsqueeze(3)
    hid = torch.matmul(down, xe.unsqueeze(-1)).squeeze(-1)
    if shape.activation == "gelu":
        hid = F.gelu(hid)
    elif shape.activation == "relu":
        hid = F.relu(hid)
    else:
        raise ValueError(shape.activation)
    y = torch.matmul(up, hid.unsqueeze(-1)).squeeze(-1)
    y = y * p.unsqueeze(-1)
    return y.sum(dim=3).sum(dim=2)


def forward(x: torch.Tensor, w: PeerWeights, shape: PeerShape, index_mode: str = "reference",
            token_chunk: Optional[int] = None):
    """Whole layer, experts.py:288-384.  Returns (out [B,S,D_out], ids, raw scores).

    ``token_chunk`` bounds the [tokens,H,k,D] intermediates the reference
    materialises (every token is independent, so chunking does not change
    which operations are applied to a token)."""
    B, S, D = x.shape
    if token_chunk is None or token_chunk >= B * S:
        q = make_queries(x, w, shape)
        ids, sc = select(q, w.sub_keys, shape.num_experts_per_tok, shape.product_key_dim,
                         shape.norm_keys, shape.norm_query, index_mode)
        return evaluate_experts(x, ids, sc, w, shape), ids, sc
    flat = x.reshape(1, B * S, D)
    outs, idss, scs = [], [], []
    for s in range(0, B * S, token_chunk):
        o, i, c = forward(flat[:, s:s + token_chunk], w, shape, index_mode, None)
        outs.append(o); idss.append(i); scs.append(c)
    H, k = shape.num_heads, idss[0].shape[-1]
    return (torch.cat(outs, 1).view(B, S, -1), torch.cat(idss, 1).view(B, S, H, k),
            torch.cat(scs, 1).view(B, S, H, k))


# ---------------------------------------------------------------------------
# FP8 (e4m3) table quantisation used by the FP8 configuration: per row,
# scale = absmax / 448 (fp32), payload = e4m3(row / scale).
# ---------------------------------------------------------------------------
def quantize_rows_e4m3(table: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    t = table.float()
    scale = t.abs().amax(dim=-1) / 448.0
    scale = torch.where(scale > 0, scale, torch.ones_like(scale))
    q = (t / scale.unsqueeze(-1)).to(torch.float8_e4m3fn)
    return q, scale


def dequantize_rows_e4m3(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return q.float() * scale.unsqueeze(-1)


# ---------------------------------------------------------------------------
# Comparison helpers shared by the parity tests.
# ---------------------------------------------------------------------------
def compare_selection(ids: torch.Tensor, ref_ids: torch.Tensor, ref_scores: torch.Tensor,
                      scores: Optional[torch.Tensor] = None, rel_gap: float = 1e-6):
    """Tie-aware comparison of ordered id lists.

    A row passes if the lists are equal, or if every position where they differ
    lies inside a run of reference scores whose neighbouring gaps are below
    ``rel_gap`` (relative to the larger magnitude).  The last position has no
    right neighbour in the reference list (the first rejected candidate is not
    returned), so a difference there is accepted only when ``scores`` (the
    checked implementation's own raw scores) is given and its last score is
    within ``rel_gap`` of the reference's last score.  Returns
    (n_rows, n_exact, n_near_tie, n_bad)."""
    k = ids.shape[-1]
    a = ids.reshape(-1, k).to(torch.int64)
    b = ref_ids.reshape(-1, k).to(torch.int64)
    s = ref_scores.reshape(-1, k).double()
    t = scores.reshape(-1, k).double() if scores is not None else None
    diff = a != b
    row_bad = diff.any(-1)
    n_rows = a.shape[0]
    n_exact = int((~row_bad).sum())
    near = bad = 0
    for r in torch.nonzero(row_bad).flatten().tolist():
        gaps = (s[r, :-1] - s[r, 1:]).abs()
        mag = torch.maximum(s[r, :-1].abs(), s[r, 1:].abs()).clamp_min(1e-30)
        tight = (gaps / mag) < rel_gap            # tight[j]: j and j+1 nearly tied
        ok = True
        for j in torch.nonzero(diff[r]).flatten().tolist():
            left = j > 0 and bool(tight[j - 1])
            right = j < k - 1 and bool(tight[j])
            last = False
            if j == k - 1 and t is not None:
                m = max(abs(float(s[r, j])), abs(float(t[r, j])), 1e-30)
                last = abs(float(s[r, j]) - float(t[r, j])) / m < rel_gap
            if not (left or right or last):
                ok = False
                break
        if ok:
            near += 1
        else:
            bad += 1
    return n_rows, n_exact, near, bad


def output_errors(out: torch.Tensor, ref: torch.Tensor):
    """(max abs error, L1-relative error) in float64."""
    a, b = out.double().flatten(), ref.double().flatten()
    return float((a - b).abs().max()), float((a - b).abs().sum() / b.abs().sum().clamp_min(1e-300))
