"""Host-side behaviour of the drop-in module: constructor signature,
state-dict layout and error behaviour (no GPU needed).  The expected
signature and state-dict are those of the reference module
(llm/models/experts.py:46-61, 87-108)."""
import inspect
import os
import sys

import pytest
import torch

from llm720_b200 import PEER, peer_forward

REF_SIGNATURE = [
    ("input_dim", inspect.Parameter.empty), ("output_dim", inspect.Parameter.empty),
    ("num_experts", inspect.Parameter.empty), ("num_experts_per_tok", 16), ("num_heads", 8),
    ("expert_hidden_size", 1), ("query_dim", 256), ("product_key_dim", [32, 32]), ("activation", "gelu"),
    ("dropout", 0.0), ("norm_keys", True), ("norm_query", True), ("batch_norm_query", True),
]


def small():
    return PEER(32, 48, 64, num_experts_per_tok=4, num_heads=2, query_dim=16, product_key_dim=[8, 8])


def test_constructor_signature_matches_reference():
    sig = inspect.signature(PEER.__init__)
    got = [(n, p.default) for n, p in sig.parameters.items() if n != "self"]
    assert got == REF_SIGNATURE
    # TransformerBlock filters kwargs by these names (foundation.py:135-147)
    names = PEER.__init__.__code__.co_varnames[:PEER.__init__.__code__.co_argcount]
    assert list(names[1:]) == [n for n, _ in REF_SIGNATURE]


# a checkout of the reference project next to this repository (or named by LLM720_REFERENCE), when there is one
REFERENCE_DIR = os.environ.get("LLM720_REFERENCE") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE_DIR, "llm")), reason="reference checkout not present")
def test_signature_and_state_dict_against_the_reference_itself():
    sys.path.insert(0, REFERENCE_DIR)
    from llm.models.experts import PEER as RefPEER
    flat = lambda f: [(n, p.default, p.kind) for n, p in inspect.signature(f).parameters.items()]
    assert flat(RefPEER.__init__) == flat(PEER.__init__)
    kw = dict(input_dim=32, output_dim=48, num_experts=64, num_experts_per_tok=4, num_heads=2, query_dim=16,
              product_key_dim=[8, 8])
    ref, ours = RefPEER(**kw), PEER(**kw)
    rs, os_ = ref.state_dict(), ours.state_dict()
    assert list(rs.keys()) == list(os_.keys())
    assert all(rs[k].shape == os_[k].shape and rs[k].dtype == os_[k].dtype for k in rs)
    ours.load_state_dict(rs)
    ref.load_state_dict(ours.state_dict())


def test_state_dict_layout():
    m = small()
    sd = m.state_dict()
    assert {k: tuple(v.shape) for k, v in sd.items()} == {
        "query_proj.weight": (32, 32), "query_proj.bias": (32,),
        "query_layer_norm.weight": (16,), "query_layer_norm.bias": (16,),
        "sub_keys.0": (8, 8), "sub_keys.1": (8, 8),
        "expert_down.weight": (64, 32), "expert_up.weight": (64, 48)}
    assert "PEER" in type(m).__name__ and m.num_experts == 64
    assert m._last_expert_indices is None
    m2 = PEER(32, 48, 64, 4, 2, 1, 16, [8, 8], batch_norm_query=False)
    assert m2.query_layer_norm is None and "query_layer_norm.weight" not in m2.state_dict()


def test_rejects_what_the_kernels_do_not_implement():
    with pytest.raises(AssertionError):
        PEER(32, 32, 60, product_key_dim=[8, 8])
    with pytest.raises(ValueError):
        PEER(32, 32, 64, activation="swish", product_key_dim=[8, 8])
    with pytest.raises(ValueError):
        PEER(32, 32, 32, product_key_dim=[2, 2, 2, 2, 2])
    with pytest.raises(ValueError):
        PEER(32, 32, 64, expert_hidden_size=17, product_key_dim=[8, 8])
    m3 = PEER(32, 32, 64, expert_hidden_size=2, query_dim=30, product_key_dim=[4, 4, 4])
    assert len(m3.sub_keys) == 3 and m3.sub_keys[0].shape == (4, 10) and m3.expert_up.weight.shape == (64, 64)


def test_no_cpu_path():
    m = small().eval()
    x = torch.randn(2, 3, 32)
    with pytest.raises(RuntimeError, match="no CPU path"):
        m(x)                                   # parameters require grad, grad mode on: still no CPU path
    with pytest.raises(RuntimeError, match="inference path"):
        m.forward_host(x)
    with torch.no_grad():
        with pytest.raises(RuntimeError, match="no CPU path"):
            m(x)
        with pytest.raises(ValueError):
            m(torch.randn(2, 3, 31))
        with pytest.raises(TypeError):
            m(x.bfloat16())
        with pytest.raises(RuntimeError, match="no CPU path"):
            peer_forward(x, m.query_proj.weight, m.query_proj.bias, m.sub_keys[0], m.sub_keys[1],
                         m.expert_down.weight, m.expert_up.weight, 2, 64, 1, 4)
    m.train()
    m.dropout.p = 0.1
    with torch.no_grad(), pytest.raises(RuntimeError, match="dropout"):
        m(x)


def test_fp8_table_quantisation_keeps_module_consistent():
    m = small()
    m.quantize_tables_e4m3()
    assert m.expert_down.weight.dtype == torch.float8_e4m3fn
    assert m.expert_down_scale.shape == (64,) and m.expert_up_scale.dtype == torch.float32
    assert "expert_down_scale" in m.state_dict()


def test_checkpoint_round_trip_with_fp8_tables(tmp_path):
    """state_dict -> safetensors file -> fresh module (the reference's save_checkpoint / load_checkpoint,
    llm/training/train.py:201-262), with quantised tables and their scales."""
    from safetensors.torch import load_file, save_file
    torch.manual_seed(0)
    m = small().bfloat16()
    m.quantize_tables_e4m3()
    sd = m.state_dict()
    assert sd["expert_down.weight"].dtype == torch.float8_e4m3fn and "expert_up_scale" in sd
    path = str(tmp_path / "layer.safetensors")
    save_file({k: v.contiguous() for k, v in sd.items()}, path)
    fresh = small().bfloat16()
    res = fresh.load_state_dict(load_file(path))
    assert not res.missing_keys and not res.unexpected_keys
    for k, v in sd.items():
        got = fresh.state_dict()[k]
        assert got.dtype == v.dtype and torch.equal(got.view(torch.uint8), v.view(torch.uint8)), k
    assert not fresh.expert_down.weight.requires_grad
    # an unquantised checkpoint still loads into an unquantised module
    plain = small().bfloat16()
    path2 = str(tmp_path / "plain.safetensors")
    save_file(plain.state_dict(), path2)
    again = small().bfloat16()
    again.load_state_dict(load_file(path2))
    assert again.expert_down.weight.dtype == torch.bfloat16 and again.expert_down_scale is None
