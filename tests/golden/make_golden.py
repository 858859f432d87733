"""Generate the committed golden files from the reference module itself.

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py --reference <reference checkout>

For every case the reference ``PEER`` (llm/models/experts.py) is built, loaded
with seeded synthetic weights and run on CPU in fp32; the oracle restatement
(oracle/peer_oracle.py) is run on the same tensors and must agree BIT FOR BIT
(indices, raw scores, output) or the script aborts without writing.  The
outputs are then stored as ``.npz`` files next to this script.  Weights of the
larger cases are not stored: the tests regenerate them from the same seeds and
check a SHA-256 of every regenerated tensor against the one recorded here.
"""
from __future__ import annotations

import argparse
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from llm720_b200 import synthetic as syn  # noqa: E402
from oracle import peer_oracle as orc     # noqa: E402


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.detach().contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def build_reference(PEER, cfg: syn.PeerConfig, sd: dict, table_rows=None):
    """Reference module in fp32 holding the (bf16-representable) values of sd."""
    kw = cfg.module_kwargs()
    if table_rows is None:
        m = PEER(**kw)
    else:
        # only the first rows are ever addressed in the reference's index mode;
        # build the module with a small table and swap the lookups afterwards
        small = dict(kw, num_experts=16, product_key_dim=[4, 4])
        m = PEER(**small)
        m.num_experts = cfg.num_experts
        m.product_key_dim = list(cfg.product_key_dim)
        m.sub_keys = torch.nn.ParameterList(
            [torch.nn.Parameter(torch.empty(n, cfg.query_dim // 2)) for n in cfg.product_key_dim])
        m.expert_down = torch.nn.Embedding(table_rows, cfg.input_dim)
        m.expert_up = torch.nn.Embedding(table_rows, cfg.output_dim)
    m = m.float().eval()
    m.load_state_dict({k: v.float() for k, v in sd.items()})
    return m


def weights_of(sd: dict, dtype=torch.float32) -> orc.PeerWeights:
    f = lambda k: sd[k].to(dtype)
    return orc.PeerWeights(f("query_proj.weight"), f("query_proj.bias"), f("query_layer_norm.weight"),
                           f("query_layer_norm.bias"), [f("sub_keys.0"), f("sub_keys.1")],
                           f("expert_down.weight"), f("expert_up.weight"))


def run_case(PEER, name, cfg, seed, random_affine, table_rows, store_weights):
    sd = syn.make_weights(cfg, seed, "cpu", table_rows=table_rows, random_affine=random_affine)
    x = syn.make_input(cfg, seed, "cpu")
    ref = build_reference(PEER, cfg, sd, table_rows)
    with torch.no_grad():
        ref_out = ref(x.float())
        ref_ids, ref_sc = ref._last_expert_indices, ref._last_expert_scores
        # the selection entry point on its own, as the reference's tests call it
        q = ref.query_layer_norm(ref.query_proj(x.float()).view(cfg.batch, cfg.seq, cfg.num_heads, cfg.query_dim))
        sel_ids, sel_sc = ref._get_expert_indices_pytorch(q, cfg.top_k)
    shape = orc.PeerShape(**{k: v for k, v in cfg.module_kwargs().items() if k != "dropout"})
    with torch.no_grad():
        o_out, o_ids, o_sc = orc.forward(x.float(), weights_of(sd), shape, "reference")
        oq = orc.make_queries(x.float(), weights_of(sd), shape)
        p_ids, p_sc = orc.select(oq, weights_of(sd).sub_keys, cfg.top_k, cfg.product_key_dim,
                                 index_mode="product")
    assert torch.equal(o_ids, ref_ids) and torch.equal(sel_ids, ref_ids), name
    assert torch.equal(o_sc, ref_sc) and torch.equal(sel_sc, ref_sc), name
    assert torch.equal(o_out, ref_out), name
    assert torch.equal(oq, q), name
    # product mode only remaps integers: scores are unchanged
    assert torch.equal(p_sc, ref_sc), name
    n1 = cfg.product_key_dim[1]
    assert torch.equal(p_ids // n1 + p_ids % n1, ref_ids), name

    rec = dict(
        ids=ref_ids.numpy().astype(np.int32), scores=ref_sc.numpy(), out=ref_out.numpy(),
        ids_product=p_ids.numpy().astype(np.int32),
        meta=np.array([cfg.input_dim, cfg.output_dim, cfg.num_heads, cfg.query_dim,
                       cfg.product_key_dim[0], cfg.product_key_dim[1], cfg.top_k, cfg.batch,
                       cfg.seq, seed, int(random_affine), -1 if table_rows is None else table_rows],
                      dtype=np.int64),
        dtype=np.array(str(cfg.dtype)),
    )
    for k, v in sd.items():
        rec["sha:" + k] = np.array(sha(v))
    rec["sha:x"] = np.array(sha(x))
    if store_weights:
        for k, v in sd.items():
            rec["w:" + k] = v.float().numpy()
        rec["w:x"] = x.float().numpy()
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **rec)
    dup = sum(len(set(r)) < len(r) for r in ref_ids.reshape(-1, cfg.top_k).tolist())
    print(f"{name}: wrote {os.path.getsize(path)/1024:.0f} KiB; max id {int(ref_ids.max())}, "
          f"rows with duplicate ids {dup}/{ref_ids.numel()//cfg.top_k}; "
          f"out std {float(ref_out.std()):.4g}")


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
    run_case(PEER, "tiny_fp32", tiny, 3, True, None, True)
    c1 = syn.CONFIGS["c1"]
    run_case(PEER, "c1", c1, 0, False, None, False)
    run_case(PEER, "c1_affine", c1, 1, True, None, False)
    # the 1M-expert bf16 layer on a 48-token slice: bf16-representable values,
    # evaluated by the reference in fp32
    c2s = syn.scaled(syn.CONFIGS["c2"], name="c2_slice", batch=1, seq=48)
    run_case(PEER, "c2_slice", c2s, 0, False, 2048, False)
    run_case(PEER, "c2_slice_affine", c2s, 2, True, 2048, False)


if __name__ == "__main__":
    main()
