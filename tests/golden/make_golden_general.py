"""Golden outputs AND gradients, from the reference module itself, for the constructor options beyond
the benchmark shape: several neurons per expert and key grids of one, three and four dimensions
(the layers the reference's own tests build, tests/test_peer_integration.py:24-111,
tests/test_peer_selection.py:53-72).

    python tests/golden/make_golden_general.py --reference <reference checkout>

Each case: reference ``PEER`` in fp32 on CPU with seeded synthetic weights; forward in both the
module call and ``_get_expert_indices_pytorch``; backward with a seeded grad_out.  The oracle
(oracle/peer_oracle.py) must give the same ids, scores and output bit for bit and the same gradients
to 1e-6, or the script aborts.  Weights are stored in the file (the cases are small).
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

from llm720_b200 import synthetic as syn  # noqa: E402
from oracle import peer_oracle as orc     # noqa: E402

CASES = {
    # name: (input_dim, output_dim, heads, query_dim, key grid, top_k, batch, seq, hidden, layer norm, seed)
    "h8_fp32": (128, 128, 2, 32, (8, 8), 4, 2, 5, 8, False, 21),
    "k3d_h8_fp32": (128, 128, 2, 30, (4, 4, 4), 4, 2, 5, 8, False, 22),
    "k3d_pruned_fp32": (64, 96, 3, 48, (16, 16, 4), 8, 2, 7, 1, True, 23),
    "k4d_h2_fp32": (64, 64, 2, 32, (4, 4, 4, 4), 4, 1, 9, 2, True, 24),
    "k1d_fp32": (64, 64, 2, 32, (64,), 4, 1, 9, 1, True, 25),
}


def config_of(name):
    D, Do, H, Q, grid, k, B, S, h, ln, seed = CASES[name]
    return syn.PeerConfig(name, D, Do, H, Q, tuple(grid), k, torch.float32, torch.float32, B, S,
                          expert_hidden_size=h, batch_norm_query=ln), seed


def oracle_weights(sd, cfg):
    f = lambda k: sd[k].float() if k in sd else None
    return orc.PeerWeights(f("query_proj.weight"), f("query_proj.bias"), f("query_layer_norm.weight"),
                           f("query_layer_norm.bias"), [sd[f"sub_keys.{i}"].float() for i in range(len(cfg.product_key_dim))],
                           f("expert_down.weight"), f("expert_up.weight"))


def run_case(PEER, name):
    cfg, seed = config_of(name)
    sd = syn.make_weights(cfg, seed, "cpu", random_affine=True)
    x = syn.make_input(cfg, seed, "cpu").float()
    grad_out = torch.randn(cfg.batch, cfg.seq, cfg.output_dim, generator=torch.Generator().manual_seed(seed + 4242))
    ref = PEER(**cfg.module_kwargs()).float().eval()
    ref.load_state_dict({k: v.float() for k, v in sd.items()})
    xl = x.clone().requires_grad_(True)
    ref_out = ref(xl)
    ref_ids, ref_sc = ref._last_expert_indices, ref._last_expert_scores
    ref_out.backward(grad_out)
    rg = {k: p.grad for k, p in ref.named_parameters()}
    rg["x"] = xl.grad

    shape = orc.PeerShape(**{k: v for k, v in cfg.module_kwargs().items() if k != "dropout"})
    leaf = {k: v.float().clone().requires_grad_(True) for k, v in sd.items()}
    xo = x.clone().requires_grad_(True)
    o_out, o_ids, o_sc = orc.forward(xo, oracle_weights(leaf, cfg), shape, "reference")
    o_out.backward(grad_out)
    og = {k: v.grad for k, v in leaf.items()}
    og["x"] = xo.grad
    with torch.no_grad():
        p_ids, p_sc = orc.select(orc.make_queries(x, oracle_weights(sd, cfg), shape), oracle_weights(sd, cfg).sub_keys,
                                 cfg.top_k, cfg.product_key_dim, index_mode="product")
    assert torch.equal(o_ids, ref_ids) and torch.equal(o_sc, ref_sc) and torch.equal(o_out, ref_out), name
    assert torch.equal(p_sc, ref_sc), name
    rec = dict(ids=ref_ids.numpy().astype(np.int32), scores=ref_sc.detach().numpy(), out=ref_out.detach().numpy(),
               ids_product=p_ids.numpy().astype(np.int32), grad_out=grad_out.numpy(), x=x.numpy())
    worst = 0.0
    for k, a in rg.items():
        if k.startswith("sub_keys"):
            assert a is None and og[k] is None, k
            continue
        err = float((a - og[k]).abs().max() / a.abs().max().clamp_min(1e-30))
        worst = max(worst, err)
        assert err < 1e-6, (name, k, err)
        rec["g:" + k] = a.numpy()
    for k, v in sd.items():
        rec["w:" + k] = v.float().numpy()
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **rec)
    print(f"{name}: wrote {os.path.getsize(path)/1024:.0f} KiB; max id {int(ref_ids.max())} of {cfg.num_experts}; "
          f"oracle gradient error {worst:.1e}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.path.join(os.path.dirname(ROOT), "reference"),
                    help="checkout of the reference project (default: a directory named reference next to this repository)")
    a = ap.parse_args()
    sys.path.insert(0, a.reference)
    from llm.models.experts import PEER  # the reference, unmodified
    torch.manual_seed(0)
    torch.set_num_threads(8)
    for name in CASES:
        run_case(PEER, name)


if __name__ == "__main__":
    main()
