"""Gradients of the oracle restatement (torch autograd through oracle/peer_oracle.py) against the golden
gradients produced from the reference module (tests/golden/make_golden_grads.py).  CPU only."""
import pytest
import torch

from _util import GRAD_DENSE, GRAD_TABLES, load_golden, load_golden_grads, oracle_gradients, rel_err


@pytest.mark.parametrize("name", ["tiny_fp32", "c1_affine"])
def test_oracle_gradients_match_reference_golden(name):
    cfg, sd, x, _ = load_golden(name)
    grad_out, dense, tables = load_golden_grads(name)
    g = oracle_gradients(cfg, sd, x, grad_out)
    assert g["sub_keys.0"] is None and g["sub_keys.1"] is None      # experts.py:154 reads them through .data
    for k in GRAD_DENSE:
        assert rel_err(g[k], dense[k]) < 2e-6, k
    for k in GRAD_TABLES:
        rows, vals = tables[k]
        assert rel_err(g[k][rows], vals) < 2e-6, k
        untouched = torch.ones(g[k].shape[0], dtype=torch.bool)
        untouched[rows] = False
        assert float(g[k][untouched].abs().max()) == 0.0, k
