"""The oracle restatement against the golden files produced from the
reference module (tests/golden/make_golden.py).  CPU only."""
import numpy as np
import pytest
import torch

from oracle import peer_oracle as orc
from _util import load_golden, oracle_shape, oracle_weights

CASES = ["tiny_fp32", "c1", "c1_affine", "c2_slice", "c2_slice_affine"]


@pytest.mark.parametrize("name", CASES)
def test_oracle_matches_reference_golden(name):
    cfg, sd, x, rec = load_golden(name)
    w = oracle_weights(sd)
    with torch.no_grad():
        out, ids, sc = orc.forward(x.float(), w, oracle_shape(cfg), "reference")
    ref_ids = torch.from_numpy(rec["ids"].astype(np.int64))
    ref_sc = torch.from_numpy(rec["scores"])
    ref_out = torch.from_numpy(rec["out"])
    n, exact, near, bad = orc.compare_selection(ids, ref_ids, ref_sc, sc)
    assert bad == 0 and exact >= 0.999 * n, (n, exact, near, bad)
    # same code, same torch build: normally bit-identical; allow for a host CPU
    # whose vector kernels order the sums differently
    assert torch.allclose(sc, ref_sc, rtol=0, atol=2e-6)
    assert torch.allclose(out, ref_out, rtol=0, atol=2e-6 * float(ref_out.abs().max()) + 1e-7)


@pytest.mark.parametrize("name", ["tiny_fp32", "c1"])
def test_product_mode_only_remaps_ids(name):
    cfg, sd, x, rec = load_golden(name)
    w = oracle_weights(sd)
    shape = oracle_shape(cfg)
    with torch.no_grad():
        q = orc.make_queries(x.float(), w, shape)
        ids_r, sc_r = orc.select(q, w.sub_keys, cfg.top_k, cfg.product_key_dim, index_mode="reference")
        ids_p, sc_p = orc.select(q, w.sub_keys, cfg.top_k, cfg.product_key_dim, index_mode="product")
    n1 = cfg.product_key_dim[1]
    assert torch.equal(sc_r, sc_p)
    assert torch.equal(ids_p // n1 + ids_p % n1, ids_r)
    assert torch.equal(ids_p, torch.from_numpy(rec["ids_product"].astype(np.int64)))


def test_token_chunking_is_transparent():
    cfg, sd, x, rec = load_golden("c1")
    w = oracle_weights(sd)
    with torch.no_grad():
        a = orc.forward(x.float(), w, oracle_shape(cfg))
        b = orc.forward(x.float(), w, oracle_shape(cfg), token_chunk=37)
    assert torch.equal(a[1], b[1])
    assert torch.allclose(a[0], b[0], rtol=0, atol=1e-6)


def test_candidates_per_dim_rule():
    # experts.py:168-187
    assert orc.candidates_per_dim(16, 1024, 2) == 16
    assert orc.candidates_per_dim(8, 128, 2) == 8
    assert orc.candidates_per_dim(4, 8, 2) == 4
    assert orc.candidates_per_dim(16, 8, 2) == 8      # table smaller than k
    assert orc.candidates_per_dim(1, 4, 2) == 3       # ceil(sqrt(1)) + 2
    assert orc.candidates_per_dim(4, 2, 2) == 2


def test_compare_selection_accepts_only_near_ties():
    ref_ids = torch.tensor([[5, 7, 9, 11]])
    ref_sc = torch.tensor([[0.9, 0.5, 0.5 - 1e-9, 0.1]])
    assert orc.compare_selection(torch.tensor([[5, 9, 7, 11]]), ref_ids, ref_sc)[3] == 0   # tied pair swapped
    assert orc.compare_selection(torch.tensor([[7, 5, 9, 11]]), ref_ids, ref_sc)[3] == 1   # real reorder
    assert orc.compare_selection(torch.tensor([[5, 7, 9, 12]]), ref_ids, ref_sc)[3] == 1   # last differs, no scores
    sc = torch.tensor([[0.9, 0.5, 0.5 - 1e-9, 0.1 + 1e-9]])
    assert orc.compare_selection(torch.tensor([[5, 7, 9, 12]]), ref_ids, ref_sc, sc)[3] == 0


def test_fp8_quantiser_roundtrip():
    torch.manual_seed(0)
    t = (torch.randn(64, 256) * 256 ** -0.5).bfloat16()
    q, s = orc.quantize_rows_e4m3(t)
    d = orc.dequantize_rows_e4m3(q, s)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (64,)
    assert float((d - t.float()).abs().max()) <= float(t.float().abs().max()) * 2 ** -3
    from llm720_b200.synthetic import quantize_rows_e4m3
    q2, s2 = quantize_rows_e4m3(t)
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and torch.equal(s, s2)
