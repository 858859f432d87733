"""Generate golden GRADIENTS from the reference module itself.

    python tests/golden/make_golden_grads.py --reference <reference checkout>

For every case the reference ``PEER`` (llm/models/experts.py) is built in fp32
with seeded synthetic weights, run on CPU with autograd, and ``out`` is
back-propagated with a seeded ``grad_out`` (what tests/test_peer_integration.py:
181-192 and the training step do with a loss).  The oracle restatement
(oracle/peer_oracle.py) is differentiated the same way and must agree with the
reference to 1e-6 of each gradient's largest entry, or the script aborts.
Stored: grad_out, the gradients of x, the query projection and the LayerNorm,
and the table gradients as (touched row ids, rows).  The sub-keys get no
gradient in the reference (it reads them through ``.data``, experts.py:154);
the script asserts that.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

from llm720_b200 import synthetic as syn  # noqa: E402
from oracle import peer_oracle as orc     # noqa: E402
from make_golden import build_reference   # noqa: E402

DENSE = ("x", "query_proj.weight", "query_proj.bias", "query_layer_norm.weight", "query_layer_norm.bias")
TABLES = ("expert_down.weight", "expert_up.weight")


def oracle_grads(cfg, sd, x, grad_out):
    leaf = {k: v.float().clone().requires_grad_(True) for k, v in sd.items()}
    xl = x.float().clone().requires_grad_(True)
    w = orc.PeerWeights(leaf["query_proj.weight"], leaf["query_proj.bias"], leaf["query_layer_norm.weight"],
                        leaf["query_layer_norm.bias"], [leaf["sub_keys.0"], leaf["sub_keys.1"]],
                        leaf["expert_down.weight"], leaf["expert_up.weight"])
    shape = orc.PeerShape(**{k: v for k, v in cfg.module_kwargs().items() if k != "dropout"})
    out, _, _ = orc.forward(xl, w, shape, "reference")
    out.backward(grad_out)
    g = {k: v.grad for k, v in leaf.items()}
    g["x"] = xl.grad
    return g


def run_case(PEER, name, cfg, seed, random_affine):
    sd = syn.make_weights(cfg, seed, "cpu", random_affine=random_affine)
    x = syn.make_input(cfg, seed, "cpu").float()
    gen = torch.Generator().manual_seed(seed + 4242)
    grad_out = torch.randn(cfg.batch, cfg.seq, cfg.output_dim, generator=gen)
    ref = build_reference(PEER, cfg, sd).train(False)
    xl = x.clone().requires_grad_(True)
    ref(xl).backward(grad_out)
    rg = {k: p.grad for k, p in ref.named_parameters()}
    rg["x"] = xl.grad
    assert rg["sub_keys.0"] is None and rg["sub_keys.1"] is None, "the reference gives the sub-keys no gradient"
    og = oracle_grads(cfg, sd, x, grad_out)
    assert og["sub_keys.0"] is None and og["sub_keys.1"] is None
    rec = dict(grad_out=grad_out.numpy())
    worst = 0.0
    for k in DENSE + TABLES:
        a, b = rg[k], og[k]
        err = float((a - b).abs().max() / a.abs().max().clamp_min(1e-30))
        worst = max(worst, err)
        assert err < 1e-6, (name, k, err)
        if k in TABLES:
            rows = torch.nonzero(a.abs().amax(dim=1) > 0).flatten()
            rec["rows:" + k] = rows.numpy().astype(np.int32)
            rec["g:" + k] = a[rows].numpy()
        else:
            rec["g:" + k] = a.numpy()
    path = os.path.join(HERE, name + "_grads.npz")
    np.savez_compressed(path, **rec)
    print(f"{name}: wrote {os.path.getsize(path)/1024:.0f} KiB; oracle vs reference worst relative error {worst:.2e}; "
          f"touched rows {len(rec['rows:expert_down.weight'])}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.path.join(os.path.dirname(ROOT), "reference"),
                    help="checkout of the reference project (default: a directory named reference next to this repository)")
    a = ap.parse_args()
    sys.path.insert(0, a.reference)
    from llm.models.experts import PEER  # the reference, unmodified

    torch.manual_seed(0)
    torch.set_num_threads(8)
    tiny = syn.PeerConfig("tiny", 32, 48, 2, 16, (8, 8), 4, torch.float32, torch.float32, 2, 3)
    run_case(PEER, "tiny_fp32", tiny, 3, True)
    run_case(PEER, "c1_affine", syn.CONFIGS["c1"], 1, True)


if __name__ == "__main__":
    main()
