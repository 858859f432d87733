"""Seeded synthetic PEER layers: the shapes, dtypes and value distributions of
the benchmark configurations, generated instead of loaded.

Weights follow the reference module's parameter names (llm/models/experts.py:
87-108) so the dictionaries returned here load straight into a module's
state-dict.  Large expert tables are generated block by block, each block from
its own seed, so that any row range can be regenerated without holding the
whole table.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import Dict, Optional, Tuple

import torch

_BLOCK_ROWS = 65536


@dataclass(frozen=True)
class PeerConfig:
    name: str
    input_dim: int
    output_dim: int
    num_heads: int
    query_dim: int
    product_key_dim: Tuple[int, ...]
    top_k: int
    dtype: torch.dtype            # activations and small weights
    table_dtype: torch.dtype      # expert_down / expert_up storage
    batch: int
    seq: int
    expert_hidden_size: int = 1
    batch_norm_query: bool = True

    @property
    def num_experts(self) -> int:
        return math.prod(self.product_key_dim)

    @property
    def tokens(self) -> int:
        return self.batch * self.seq

    def module_kwargs(self) -> dict:
        return dict(input_dim=self.input_dim, output_dim=self.output_dim,
                    num_experts=self.num_experts, num_experts_per_tok=self.top_k,
                    num_heads=self.num_heads, expert_hidden_size=self.expert_hidden_size, query_dim=self.query_dim,
                    product_key_dim=list(self.product_key_dim), activation="gelu", dropout=0.0,
                    norm_keys=True, norm_query=True, batch_norm_query=self.batch_norm_query)

    def gathered_bytes_per_token(self) -> int:
        """Algorithmic bytes the expert stage must fetch for one token: one
        down row and one up row per (head, slot), plus the per-row scales of
        FP8 tables."""
        b = torch.empty(0, dtype=self.table_dtype).element_size()
        per_row_extra = 4 if self.table_dtype == torch.float8_e4m3fn else 0
        return self.num_heads * self.top_k * (
            (self.input_dim * b + self.output_dim * b) * self.expert_hidden_size + 2 * per_row_extra)


CONFIGS: Dict[str, PeerConfig] = {
    # small fp32 layer that the reference also runs on CPU
    "c1": PeerConfig("c1", 256, 256, 4, 128, (128, 128), 8, torch.float32, torch.float32, 2, 128),
    # 1M experts, bf16
    "c2": PeerConfig("c2", 2048, 2048, 8, 256, (1024, 1024), 16, torch.bfloat16, torch.bfloat16, 8, 2048),
    # 1M experts, FP8-e4m3 tables with per-row scale
    "c3": PeerConfig("c3", 2048, 2048, 8, 256, (1024, 1024), 16, torch.bfloat16, torch.float8_e4m3fn, 8, 2048),
    # decode-shaped, 4M experts
    "c4": PeerConfig("c4", 4096, 4096, 16, 256, (2048, 2048), 16, torch.bfloat16, torch.bfloat16, 64, 1),
}


def scaled(cfg: PeerConfig, **kw) -> PeerConfig:
    """A variant of a named configuration (fewer tokens, smaller key tables...)."""
    return replace(cfg, **kw)


def _gen(device, seed: int) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def _table(rows: int, width: int, std: float, dtype: torch.dtype, device, seed: int,
           tensor_id: int, row_start: int = 0) -> torch.Tensor:
    """Rows [row_start, row_start+rows) of a N(0, std^2) table, rounded to
    bf16 when the storage type is narrower than fp32."""
    if row_start % _BLOCK_ROWS:
        raise ValueError("row_start must be a multiple of the generator block")
    store = torch.bfloat16 if dtype == torch.float8_e4m3fn else dtype
    out = torch.empty(rows, width, dtype=store, device=device)
    for b0 in range(0, rows, _BLOCK_ROWS):
        n = min(_BLOCK_ROWS, rows - b0)
        blk = (row_start + b0) // _BLOCK_ROWS
        g = _gen(device, (seed * 1000003 + tensor_id * 10007 + blk) & 0x7FFFFFFF)
        out[b0:b0 + n] = (torch.randn(n, width, generator=g, device=device, dtype=torch.float32)
                          * std).to(store)
    return out


def make_weights(cfg: PeerConfig, seed: int = 0, device="cpu", table_rows: Optional[int] = None,
                 random_affine: bool = False, tables: bool = True) -> Dict[str, torch.Tensor]:
    """State-dict of a synthetic layer.  Small weights ~ N(0, 1/fan_in) in
    ``cfg.dtype``; query bias 0 and LayerNorm affine (1, 0) unless
    ``random_affine``; tables ~ N(0, 1/fan_in).  With an FP8 table type the
    tables are returned in bf16 (quantise them with ``quantize_rows_e4m3``).
    ``table_rows`` limits the tables to their first rows (enough for the
    reference's index mode, whose ids stay below n0+n1-1)."""
    D, Do, H, Q = cfg.input_dim, cfg.output_dim, cfg.num_heads, cfg.query_dim
    g = _gen(device, seed)
    rn = lambda *s: torch.randn(*s, generator=g, device=device, dtype=torch.float32)
    sd = {}
    sd["query_proj.weight"] = (rn(H * Q, D) * D ** -0.5).to(cfg.dtype)
    if random_affine:
        sd["query_proj.bias"] = (rn(H * Q) * 0.1).to(cfg.dtype)
        if cfg.batch_norm_query:
            sd["query_layer_norm.weight"] = (1.0 + 0.2 * rn(Q)).to(cfg.dtype)
            sd["query_layer_norm.bias"] = (0.1 * rn(Q)).to(cfg.dtype)
    else:
        sd["query_proj.bias"] = torch.zeros(H * Q, dtype=cfg.dtype, device=device)
        if cfg.batch_norm_query:
            sd["query_layer_norm.weight"] = torch.ones(Q, dtype=cfg.dtype, device=device)
            sd["query_layer_norm.bias"] = torch.zeros(Q, dtype=cfg.dtype, device=device)
    width = Q // len(cfg.product_key_dim)
    for i, n in enumerate(cfg.product_key_dim):
        sd[f"sub_keys.{i}"] = (rn(n, width) * width ** -0.5).to(cfg.dtype)
    if not tables:
        return sd
    rows = cfg.num_experts if table_rows is None else min(table_rows, cfg.num_experts)
    h = cfg.expert_hidden_size
    sd["expert_down.weight"] = _table(rows, D * h, D ** -0.5, cfg.table_dtype, device, seed, 1)
    sd["expert_up.weight"] = _table(rows, Do * h, (D * h) ** -0.5 if h > 1 else D ** -0.5, cfg.table_dtype, device, seed, 2)
    return sd


def make_table_shard(cfg: PeerConfig, which: str, row_start: int, rows: int, seed: int = 0, device="cpu") -> torch.Tensor:
    """Rows [row_start, row_start+rows) of `expert_down` / `expert_up` exactly as make_weights would
    generate them (row_start must be a multiple of 65,536), without building the whole table."""
    tensor_id = {"expert_down": 1, "expert_up": 2}[which]
    width = cfg.input_dim if which == "expert_down" else cfg.output_dim
    return _table(rows, width, cfg.input_dim ** -0.5, cfg.table_dtype, device, seed, tensor_id, row_start)


def make_input(cfg: PeerConfig, seed: int = 0, device="cpu") -> torch.Tensor:
    g = _gen(device, seed + 7919)
    return torch.randn(cfg.batch, cfg.seq, cfg.input_dim, generator=g, device=device,
                       dtype=torch.float32).to(cfg.dtype)


def quantize_rows_e4m3(table: torch.Tensor, block_rows: int = _BLOCK_ROWS):
    """Per-row FP8 quantisation: scale = absmax/448 (fp32), payload =
    e4m3(row/scale).  Returns (payload [N,W] float8_e4m3fn, scale [N] fp32)."""
    N, W = table.shape
    q = torch.empty(N, W, dtype=torch.float8_e4m3fn, device=table.device)
    scale = torch.empty(N, dtype=torch.float32, device=table.device)
    for b0 in range(0, N, block_rows):
        t = table[b0:b0 + block_rows].float()
        s = t.abs().amax(dim=-1) / 448.0
        s = torch.where(s > 0, s, torch.ones_like(s))
        q[b0:b0 + block_rows] = (t / s.unsqueeze(-1)).to(torch.float8_e4m3fn)
        scale[b0:b0 + block_rows] = s
    return q, scale
