"""CUDA path for the constructor options beyond the benchmark shape (several neurons per expert; 1-D, 3-D,
4-D key grids) against golden outputs and gradients from the reference module, and the general
selection kernel against the oracle and against the specialised two-dimensional kernels.

Tolerances: ids equal except inside near-tie groups (< 1e-6 relative score gap); fp32 outputs and
gradients within 2e-5 of the reference's, relative to the largest entry; bf16 against the fp32 oracle on
the same bf16-representable values: L1-relative <= 2e-2.
"""
import numpy as np
import pytest
import torch

from llm720_b200 import PEER, peer_forward_cutlass, synthetic as syn
from oracle import peer_oracle as orc
from _util import (GENERAL_CASES, general_oracle_weights, load_general, load_golden, make_op, oracle_shape,
                   oracle_weights, rel_err)

pytestmark = pytest.mark.gpu


def _module(cfg, sd, device, index_mode="reference"):
    m = PEER(**cfg.module_kwargs()).to(cfg.dtype)
    m.load_state_dict({k: v.to(cfg.dtype) for k, v in sd.items()})
    m = m.to(device).eval()
    m.index_mode = index_mode
    return m


def _check_ids(ids, ref_ids, ref_sc, sc):
    n, exact, near, bad = orc.compare_selection(ids.cpu(), ref_ids, ref_sc, sc.cpu())
    assert bad == 0 and exact >= 0.99 * n, (n, exact, near, bad)


@pytest.mark.parametrize("name", GENERAL_CASES)
def test_forward_and_backward_match_reference_golden(cuda_device, name):
    cfg, sd, x, rec = load_general(name)
    m = _module(cfg, sd, cuda_device)
    with torch.no_grad():
        out = m(x.to(cuda_device))
    m._op.query_status()
    ref_ids = torch.from_numpy(rec["ids"].astype(np.int64))
    ref_sc = torch.from_numpy(rec["scores"])
    _check_ids(m._last_expert_indices, ref_ids, ref_sc, m._last_expert_scores)
    assert torch.allclose(m._last_expert_scores.cpu(), ref_sc, rtol=0, atol=3e-6)
    assert rel_err(out.cpu(), torch.from_numpy(rec["out"])) < 2e-5
    # same through the differentiable path, and its gradients
    xl = x.to(cuda_device).requires_grad_(True)
    out2 = m(xl)
    assert rel_err(out2.detach().cpu(), torch.from_numpy(rec["out"])) < 2e-5
    out2.backward(torch.from_numpy(rec["grad_out"]).to(cuda_device))
    m._op.query_status()
    grads = {k: p.grad for k, p in m.named_parameters()}
    grads["x"] = xl.grad
    for k in [f[2:] for f in rec.files if f.startswith("g:")]:
        assert rel_err(grads[k].cpu(), torch.from_numpy(rec["g:" + k])) < 2e-5, (k, rel_err(grads[k].cpu(), torch.from_numpy(rec["g:" + k])))
    for i in range(len(cfg.product_key_dim)):
        assert grads[f"sub_keys.{i}"] is None


@pytest.mark.parametrize("name", ["k3d_pruned_fp32", "k4d_h2_fp32", "k1d_fp32"])
def test_product_index_mode(cuda_device, name):
    cfg, sd, x, rec = load_general(name)
    m = _module(cfg, sd, cuda_device, "product")
    with torch.no_grad():
        out = m(x.to(cuda_device))
        ref_out, ref_ids, ref_sc = orc.forward(x, general_oracle_weights(sd, cfg), oracle_shape(cfg), "product")
    _check_ids(m._last_expert_indices, ref_ids, ref_sc, m._last_expert_scores)
    assert torch.equal(ref_ids, torch.from_numpy(rec["ids_product"].astype(np.int64)))
    assert rel_err(out.cpu(), ref_out) < 2e-5


@pytest.mark.parametrize("grid,Q,k,H,dtype", [((16, 16, 4), 48, 8, 3, torch.float32), ((8, 6, 5, 4), 64, 16, 2, torch.float32),
                                              ((300,), 32, 16, 2, torch.bfloat16), ((32, 16, 8), 96, 16, 4, torch.bfloat16),
                                              ((40, 50), 64, 8, 2, torch.float32)])
@pytest.mark.parametrize("mode", ["reference", "product"])
def test_general_selection_against_the_oracle(cuda_device, grid, Q, k, H, dtype, mode):
    g = torch.Generator().manual_seed(len(grid) * 100 + Q)
    width = Q // len(grid)
    keys = [(torch.randn(n, width, generator=g) * width ** -0.5).to(dtype) for n in grid]
    q = torch.randn(1, 130, H, Q, generator=g)
    cfg = syn.PeerConfig("t", 64, 64, H, Q, tuple(grid), k, dtype, dtype, 1, 130)
    op = make_op(cfg, cuda_device, mode)
    ids, sc = op.select_nd(q.view(130, H, Q).to(cuda_device).contiguous(), [kt.to(cuda_device) for kt in keys])
    with torch.no_grad():
        ref_ids, ref_sc = orc.select(q, [kt.float() for kt in keys], k, grid, True, True, mode)
    _check_ids(ids.view(1, 130, H, k), ref_ids, ref_sc, sc.view(1, 130, H, k))
    assert torch.allclose(sc.cpu().view_as(ref_sc), ref_sc, rtol=0, atol=3e-6)
    if len(grid) == 2:        # the specialised kernel gives the same lists
        ids2, sc2 = op.select(q.view(130, H, Q).to(cuda_device).contiguous(), keys[0].to(cuda_device), keys[1].to(cuda_device))
        _check_ids(ids2.view(1, 130, H, k), ref_ids, ref_sc, sc2.view(1, 130, H, k))


@pytest.mark.parametrize("three_d", [False, True])
def test_functional_entry_with_several_neurons_per_expert(cuda_device, three_d):
    """peer_forward_cutlass with expert_hidden_size = 8: the output width is that of the reference wrapper
    (peer_cutlass.py:176: dimension 1 of a [N, output_dim, h] table), also when the table comes flattened as
    the module stores it ([N, output_dim*h])."""
    cfg, sd, x, rec = load_general("h8_fp32")
    g = lambda k: sd[k].to(cuda_device)
    h, N = cfg.expert_hidden_size, cfg.num_experts
    u, v = g("expert_down.weight"), g("expert_up.weight")
    if three_d:
        u, v = u.view(N, h, cfg.input_dim), v.view(N, cfg.output_dim, h)
    y = peer_forward_cutlass(x.to(cuda_device), g("query_proj.weight"), g("query_proj.bias"), g("sub_keys.0"),
                             g("sub_keys.1"), u, v, cfg.num_heads, N, h, cfg.top_k, layer_norm=False)
    assert y.shape == (cfg.batch, cfg.seq, cfg.output_dim)
    assert rel_err(y.cpu(), torch.from_numpy(rec["out"])) < 2e-5
    with pytest.raises(ValueError, match="neurons"):
        peer_forward_cutlass(x.to(cuda_device), g("query_proj.weight"), g("query_proj.bias"), g("sub_keys.0"),
                             g("sub_keys.1"), u.reshape(N, -1), v.reshape(N, -1)[:, :-1].contiguous(), cfg.num_heads, N, h,
                             cfg.top_k, layer_norm=False)


def test_reference_test_layer_in_bf16(cuda_device):
    """The bf16 layer of the reference's integration test (8 neurons per expert, 8x8 keys, no LayerNorm),
    against the fp32 oracle on the same bf16-representable values."""
    cfg = syn.PeerConfig("t", 128, 128, 2, 32, (8, 8), 4, torch.bfloat16, torch.bfloat16, 4, 16,
                         expert_hidden_size=8, batch_norm_query=False)
    sd = syn.make_weights(cfg, 31, "cpu", random_affine=True)
    x = syn.make_input(cfg, 31, "cpu")
    m = _module(cfg, sd, cuda_device)
    xl = x.to(cuda_device).requires_grad_(True)
    out = m(xl)
    assert out.dtype == torch.bfloat16 and out.shape == (4, 16, 128)
    out.sum().backward()                                   # what tests/test_peer_integration.py:181-192 does
    assert torch.isfinite(xl.grad).all()
    leaf = {k: v.float().clone().requires_grad_(True) for k, v in sd.items()}
    xo = x.float().clone().requires_grad_(True)
    ref, _, _ = orc.forward(xo, general_oracle_weights(leaf, cfg), oracle_shape(cfg), "reference")
    ref.sum().backward()
    l1 = lambda a, b: float((a - b).abs().sum() / b.abs().sum())
    assert l1(out.detach().float().cpu(), ref.detach()) <= 1e-2
    assert l1(xl.grad.float().cpu(), xo.grad) <= 2e-2
    assert l1(m.expert_up.weight.grad.float().cpu(), leaf["expert_up.weight"].grad) <= 2e-2
    assert l1(m.expert_down.weight.grad.float().cpu(), leaf["expert_down.weight"].grad) <= 2e-2


@pytest.mark.parametrize("grid,Q", [((8, 8), 32), ((4, 4, 4), 30)])
def test_reference_test_layers_in_fp16(cuda_device, grid, Q):
    """The fp16 layer of the reference's integration test (tests/test_peer_integration.py:46-67) and its 3-D
    sibling, on the CUDA-core kernels, against the fp32 oracle on the same fp16-representable values."""
    cfg = syn.PeerConfig("t", 128, 128, 2, Q, grid, 4, torch.float16, torch.float16, 4, 16,
                         expert_hidden_size=8, batch_norm_query=False)
    sd = syn.make_weights(cfg, 41, "cpu", random_affine=True)
    x = syn.make_input(cfg, 41, "cpu")
    m = _module(cfg, sd, cuda_device)
    with torch.no_grad():
        out_i = m(x.to(cuda_device))
    xl = x.to(cuda_device).requires_grad_(True)
    out = m(xl)
    assert out.dtype == torch.float16 and out.shape == (4, 16, 128) and torch.equal(out.detach(), out_i)
    out.sum().backward()
    m._op.query_status()
    leaf = {k: v.float().clone().requires_grad_(True) for k, v in sd.items()}
    xo = x.float().clone().requires_grad_(True)
    ref, ref_ids, ref_sc = orc.forward(xo, general_oracle_weights(leaf, cfg), oracle_shape(cfg), "reference")
    ref.sum().backward()
    _check_ids(m._last_expert_indices, ref_ids, ref_sc.detach(), m._last_expert_scores)
    l1 = lambda a, b: float((a - b).abs().sum() / b.abs().sum())
    assert l1(out.detach().float().cpu(), ref.detach()) <= 2e-3
    assert l1(xl.grad.float().cpu(), xo.grad) <= 5e-3
    assert l1(m.query_proj.weight.grad.float().cpu(), leaf["query_proj.weight"].grad) <= 2e-2
    assert l1(m.expert_up.weight.grad.float().cpu(), leaf["expert_up.weight"].grad) <= 5e-3
    assert l1(m.expert_down.weight.grad.float().cpu(), leaf["expert_down.weight"].grad) <= 5e-3


def test_rejected_shapes_raise(cuda_device):
    with pytest.raises(ValueError):
        PEER(32, 32, 32, product_key_dim=[2, 2, 2, 2, 2])
    with pytest.raises(ValueError):
        PEER(32, 32, 64, expert_hidden_size=17, product_key_dim=[8, 8])
    with pytest.raises(ValueError):
        PEER(32, 32, 64, query_dim=32, product_key_dim=[4, 4, 4])     # 32 is not a multiple of 3
    m = PEER(32, 32, 64, num_experts_per_tok=4, num_heads=1, query_dim=30, product_key_dim=[4, 4, 4]).to(cuda_device).eval()
    with torch.no_grad(), pytest.raises(ValueError, match="peer_select_nd"):
        m._operator(cuda_device, torch.float32, 4).select(torch.zeros(4, 1, 30, device=cuda_device),
                                                           m.sub_keys[0], m.sub_keys[1])
