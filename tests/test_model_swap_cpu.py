"""The drop-in module inside the reference's own model class (BASELINE configuration 5 at a tiny size,
host side only: this library has no CPU forward, so nothing is evaluated here).

Skipped when no checkout of the reference project is present (LLM720_REFERENCE, or a `reference`
directory next to this repository).  With it, the reference's `FoundationModel` is built twice:
  * as it is, then every `block.feed_forward` replaced by `llm720_b200.PEER` the way INTEGRATION.md shows
    (constructor attributes copied, state-dict loaded with assign=True so the tables are shared);
  * with `llm.models.foundation.PEER` pointing at this library's class, so that `TransformerBlock` itself
    constructs it through its `co_varnames` filter (llm/models/foundation.py:131-147).
Checked: parameter names and shapes of the whole model are unchanged, the state-dict round-trips both
ways, `hook_expert_tracking` (llm/utils/experts/tracking.py:334-381) finds every swapped layer, and a
forward on CPU tensors is refused loudly instead of falling back to another implementation.
"""
import os
import sys

import pytest
import torch

from llm720_b200 import PEER

REFERENCE_DIR = os.environ.get("LLM720_REFERENCE") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE_DIR, "llm")),
                                reason="reference checkout not present")

PEER_ATTRS = ("input_dim", "output_dim", "num_experts", "num_experts_per_tok", "num_heads", "expert_hidden_size",
              "query_dim", "product_key_dim", "norm_keys", "norm_query", "batch_norm_query")


def _config(layers=3, start=1):
    sys.path.insert(0, REFERENCE_DIR)
    from llm.models.foundation import TransformerConfig
    return TransformerConfig(
        hidden_size=64, num_hidden_layers=layers, num_attention_heads=4, intermediate_size=128, vocab_size=1000,
        max_position_embeddings=128, use_peer=True, peer_start_layer=start,
        peer_config={"num_experts": 64, "num_experts_per_tok": 4, "num_heads": 2, "expert_hidden_size": 1,
                     "product_key_dim": [8, 8], "query_dim": 16, "batch_norm_query": True,
                     # keys the trainer's config carries and the block must filter out (foundation.py:135-143)
                     "log_expert_usage": True, "log_freq": 10, "usage_threshold": 5.0},
        mla_config={"q_lora_rank": None, "kv_lora_rank": 16, "qk_rope_head_dim": 8, "v_head_dim": 16,
                    "qk_nope_head_dim": 8})


def _swap(model):
    """INTEGRATION.md section 1, verbatim in spirit: same constructor values, tables shared."""
    n = 0
    for block in model.blocks:
        ref = block.feed_forward
        if type(ref).__name__ == "PEER":
            new = PEER(**{k: getattr(ref, k) for k in PEER_ATTRS}, activation=ref.activation_name
                       if hasattr(ref, "activation_name") else "gelu")
            new.load_state_dict(ref.state_dict(), assign=True)
            block.feed_forward = new.eval()
            n += 1
    return n


def test_swap_into_the_reference_model_keeps_its_state_dict():
    cfg = _config()
    from llm.models.foundation import FoundationModel
    torch.manual_seed(0)
    model = FoundationModel(cfg).eval()
    before = {k: (tuple(v.shape), v.dtype) for k, v in model.state_dict().items()}
    saved = {k: v.clone() for k, v in model.state_dict().items()}
    ref_table = model.blocks[1].feed_forward.expert_down.weight
    assert _swap(model) == 2                                  # layers 1 and 2; layer 0 keeps its MLP
    assert type(model.blocks[0].feed_forward).__name__ == "Sequential"
    for b in model.blocks[1:]:
        assert isinstance(b.feed_forward, PEER)
    assert model.blocks[1].feed_forward.expert_down.weight.data_ptr() == ref_table.data_ptr()    # shared, not copied
    after = {k: (tuple(v.shape), v.dtype) for k, v in model.state_dict().items()}
    assert after == before                                    # same names, shapes and dtypes, model-wide
    model.load_state_dict(saved)                              # a reference checkpoint loads into the swapped model
    fresh = FoundationModel(cfg)
    fresh.load_state_dict(model.state_dict())                 # and the swapped model's checkpoint into the reference


def test_transformer_block_constructs_this_class_through_its_kwargs_filter(monkeypatch):
    cfg = _config(layers=2, start=0)
    import llm.models.foundation as foundation
    monkeypatch.setattr(foundation, "PEER", PEER)
    model = foundation.FoundationModel(cfg)
    for b in model.blocks:
        ff = b.feed_forward
        assert isinstance(ff, PEER)
        assert (ff.input_dim, ff.output_dim, ff.num_experts, ff.num_experts_per_tok, ff.num_heads, ff.query_dim,
                ff.product_key_dim) == (64, 64, 64, 4, 2, 16, [8, 8])
    # the reference's own initialiser ran over this module's parameters (foundation.py:257-275)
    assert float(model.blocks[0].feed_forward.query_proj.bias.detach().abs().max()) == 0.0


def _stub_plotting_modules(monkeypatch):
    """The reference's tracker imports matplotlib, seaborn and wandb at module level for its plots; none of
    them is needed to register hooks.  Where they are not installed, empty stand-ins let the import pass."""
    import importlib.util
    import types
    for name in ("matplotlib", "matplotlib.pyplot", "seaborn", "wandb"):
        try:
            found = importlib.util.find_spec(name) is not None
        except (ImportError, ValueError):
            found = False
        if not found:
            monkeypatch.setitem(sys.modules, name, types.ModuleType(name))


def test_usage_tracking_hooks_find_the_swapped_layers_and_cpu_forward_is_refused(monkeypatch):
    cfg = _config()
    _stub_plotting_modules(monkeypatch)
    from llm.models.foundation import FoundationModel
    from llm.utils.experts.tracking import ExpertUsageTracker, hook_expert_tracking
    model = FoundationModel(cfg).eval()
    _swap(model)
    tracker = ExpertUsageTracker(num_experts=64, num_layers=2, wandb_enabled=False)
    hook_expert_tracking(model, tracker)
    hooked = [len(b.feed_forward._forward_hooks) for b in model.blocks]
    assert hooked == [0, 1, 1]
    ids = torch.randint(0, 1000, (2, 8))
    pos = torch.arange(8).unsqueeze(0).expand(2, -1)
    with torch.no_grad(), pytest.raises(RuntimeError, match="no CPU path"):
        model(input_ids=ids, position_ids=pos)
