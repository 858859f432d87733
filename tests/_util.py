"""Helpers shared by the tests: golden-file loading and oracle adapters."""
import hashlib
import os

import numpy as np
import torch

from llm720_b200 import synthetic as syn
from oracle import peer_oracle as orc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.detach().contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def dtype_of(name: str) -> torch.dtype:
    return {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16}[name]


def load_golden(name: str):
    """Returns (cfg, state-dict on CPU in cfg dtypes, x, record).  Weights are
    either stored in the file or regenerated from the recorded seed and
    verified against the recorded SHA-256 digests."""
    rec = np.load(os.path.join(GOLDEN, name + ".npz"))
    m = rec["meta"].tolist()
    dt = dtype_of(str(rec["dtype"]))
    cfg = syn.PeerConfig(name, m[0], m[1], m[2], m[3], (m[4], m[5]), m[6], dt, dt, m[7], m[8])
    seed, affine, rows = m[9], bool(m[10]), (None if m[11] < 0 else m[11])
    keys = ["query_proj.weight", "query_proj.bias", "query_layer_norm.weight", "query_layer_norm.bias",
            "sub_keys.0", "sub_keys.1", "expert_down.weight", "expert_up.weight"]
    if "w:x" in rec.files:
        sd = {k: torch.from_numpy(rec["w:" + k]).to(dt) for k in keys}
        x = torch.from_numpy(rec["w:x"]).to(dt)
    else:
        sd = syn.make_weights(cfg, seed, "cpu", table_rows=rows, random_affine=affine)
        x = syn.make_input(cfg, seed, "cpu")
        for k in keys:
            assert sha(sd[k]) == str(rec["sha:" + k]), f"regenerated {k} differs from the golden run"
        assert sha(x) == str(rec["sha:x"])
    return cfg, sd, x, rec


def oracle_weights(sd: dict, dtype=torch.float32, down_scale=None, up_scale=None,
                   tables_as_stored=False) -> orc.PeerWeights:
    f = lambda k: sd[k].to(dtype)
    t = (lambda k: sd[k]) if tables_as_stored else f
    return orc.PeerWeights(f("query_proj.weight"), f("query_proj.bias"), f("query_layer_norm.weight"),
                           f("query_layer_norm.bias"), [f("sub_keys.0"), f("sub_keys.1")],
                           t("expert_down.weight"), t("expert_up.weight"), down_scale, up_scale)


def oracle_shape(cfg: syn.PeerConfig) -> orc.PeerShape:
    kw = dict(cfg.module_kwargs())
    kw.pop("dropout")
    return orc.PeerShape(**kw)


def op_weights(sd: dict, device, down_scale=None, up_scale=None) -> dict:
    """State-dict -> the weight dict PeerOp takes, on the device."""
    g = lambda k: sd[k].to(device).contiguous()
    return dict(query_w=g("query_proj.weight"), query_b=g("query_proj.bias"),
                ln_w=g("query_layer_norm.weight"), ln_b=g("query_layer_norm.bias"),
                keys0=g("sub_keys.0"), keys1=g("sub_keys.1"), expert_down=g("expert_down.weight"),
                expert_up=g("expert_up.weight"),
                down_scale=None if down_scale is None else down_scale.to(device),
                up_scale=None if up_scale is None else up_scale.to(device))


def make_op(cfg: syn.PeerConfig, device, index_mode="reference", max_tokens=None, table_dtype=None, **kw):
    from llm720_b200 import PeerOp
    return PeerOp(input_dim=cfg.input_dim, output_dim=cfg.output_dim, num_heads=cfg.num_heads,
                  query_dim=cfg.query_dim, product_key_dim=cfg.product_key_dim, top_k=cfg.top_k,
                  act_dtype=cfg.dtype, table_dtype=table_dtype or cfg.table_dtype, index_mode=index_mode,
                  max_tokens=max_tokens or max(cfg.tokens, 1), device=device, **kw)


GRAD_DENSE = ("x", "query_proj.weight", "query_proj.bias", "query_layer_norm.weight", "query_layer_norm.bias")
GRAD_TABLES = ("expert_down.weight", "expert_up.weight")


def load_golden_grads(name: str):
    """Golden gradients written by tests/golden/make_golden_grads.py: (grad_out, {name: dense gradient},
    {table name: (row ids, rows)})."""
    rec = np.load(os.path.join(GOLDEN, name + "_grads.npz"))
    dense = {k: torch.from_numpy(rec["g:" + k]) for k in GRAD_DENSE}
    tables = {k: (torch.from_numpy(rec["rows:" + k].astype(np.int64)), torch.from_numpy(rec["g:" + k]))
              for k in GRAD_TABLES}
    return torch.from_numpy(rec["grad_out"]), dense, tables


def oracle_gradients(cfg, sd, x, grad_out, index_mode="reference", dtype=torch.float32):
    """Autograd through the oracle forward: {name: gradient} for x, the dense weights and both tables."""
    leaf = {k: v.to(dtype).clone().requires_grad_(True) for k, v in sd.items()}
    xl = x.to(dtype).clone().requires_grad_(True)
    out, _, _ = orc.forward(xl, oracle_weights(leaf, dtype), oracle_shape(cfg), index_mode)
    out.backward(grad_out.to(dtype))
    g = {k: v.grad for k, v in leaf.items()}
    g["x"] = xl.grad
    return g


def rel_err(a: torch.Tensor, b: torch.Tensor) -> float:
    """Largest absolute difference relative to the largest reference entry."""
    return float((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30))


GENERAL_CASES = ["h8_fp32", "k3d_h8_fp32", "k3d_pruned_fp32", "k4d_h2_fp32", "k1d_fp32"]


def load_general(name: str):
    """Golden case written by tests/golden/make_golden_general.py (constructor options beyond the benchmark
    shape): (cfg, state-dict, x, record)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden_general", os.path.join(GOLDEN, "make_golden_general.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    cfg, _ = mod.config_of(name)
    rec = np.load(os.path.join(GOLDEN, name + ".npz"))
    sd = {k[2:]: torch.from_numpy(rec[k]) for k in rec.files if k.startswith("w:")}
    return cfg, sd, torch.from_numpy(rec["x"]), rec


def general_oracle_weights(sd: dict, cfg) -> orc.PeerWeights:
    f = lambda k: sd[k].float() if k in sd else None
    return orc.PeerWeights(f("query_proj.weight"), f("query_proj.bias"), f("query_layer_norm.weight"),
                           f("query_layer_norm.bias"),
                           [sd[f"sub_keys.{i}"].float() for i in range(len(cfg.product_key_dim))],
                           f("expert_down.weight"), f("expert_up.weight"))
