"""The oracle on the constructor options beyond the benchmark shape (several neurons per expert; 1-D,
3-D, 4-D key grids), against golden outputs and gradients from the reference module
(tests/golden/make_golden_general.py).  CPU only."""
import numpy as np
import pytest
import torch

from oracle import peer_oracle as orc
from _util import GENERAL_CASES, general_oracle_weights, load_general, oracle_shape, rel_err


@pytest.mark.parametrize("name", GENERAL_CASES)
def test_oracle_forward_and_gradients(name):
    cfg, sd, x, rec = load_general(name)
    leaf = {k: v.clone().requires_grad_(True) for k, v in sd.items()}
    xl = x.clone().requires_grad_(True)
    out, ids, sc = orc.forward(xl, general_oracle_weights(leaf, cfg), oracle_shape(cfg), "reference")
    assert torch.equal(ids, torch.from_numpy(rec["ids"].astype(np.int64)))
    assert torch.allclose(sc, torch.from_numpy(rec["scores"]), rtol=0, atol=2e-6)
    assert rel_err(out.detach(), torch.from_numpy(rec["out"])) < 2e-6
    out.backward(torch.from_numpy(rec["grad_out"]))
    for k in [f[2:] for f in rec.files if f.startswith("g:")]:
        got = xl.grad if k == "x" else leaf[k].grad
        assert rel_err(got, torch.from_numpy(rec["g:" + k])) < 2e-6, k
    for i in range(len(cfg.product_key_dim)):
        assert leaf[f"sub_keys.{i}"].grad is None


def test_one_dimensional_reference_ids_are_list_positions():
    # experts.py:197-200 returns the positions inside the candidate list, not key indices
    cfg, sd, x, rec = load_general("k1d_fp32")
    assert rec["ids"].max() == cfg.top_k - 1
    w = general_oracle_weights(sd, cfg)
    with torch.no_grad():
        q = orc.make_queries(x, w, oracle_shape(cfg))
        ids_p, _ = orc.select(q, w.sub_keys, cfg.top_k, cfg.product_key_dim, index_mode="product")
    assert torch.equal(ids_p, torch.from_numpy(rec["ids_product"].astype(np.int64))) and int(ids_p.max()) > cfg.top_k
