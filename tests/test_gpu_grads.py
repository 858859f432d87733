"""Backward pass of the CUDA path against the golden gradients generated from the reference module
and against autograd through the oracle.

Tolerances:
  * fp32 layers: every gradient within 2e-5 of the reference's, relative to that gradient's largest
    entry (sums are accumulated with floating-point atomics, so the order of additions varies);
  * bf16 layers: against fp32 autograd through the oracle on the same bf16-representable values:
    L1-relative error <= 2e-2 for every gradient (the gradients themselves are rounded to bf16, and
    the recomputed query projection runs in bf16), largest entry error <= 5e-2 of the largest entry.
"""
import pytest
import torch

from llm720_b200 import PEER, synthetic as syn
from _util import (GRAD_DENSE, GRAD_TABLES, load_golden, load_golden_grads, make_op, oracle_gradients,
                   rel_err)

pytestmark = pytest.mark.gpu


def _module(cfg, sd, device, index_mode="reference", train=False):
    m = PEER(**cfg.module_kwargs()).to(cfg.dtype)
    m.load_state_dict({k: v.to(cfg.dtype) for k, v in sd.items()})
    m = m.to(device).train(train)
    m.index_mode = index_mode
    return m


def _module_grads(m, x, grad_out):
    xl = x.clone().requires_grad_(True)
    out = m(xl)
    out.backward(grad_out)
    g = {k: p.grad for k, p in m.named_parameters()}
    g["x"] = xl.grad
    return out, g


def _dense_reference(x, ids, w, down, up, act):
    """Plain torch fp32 statement of the expert evaluation, for autograd."""
    u = down[ids.long()]                                        # [T, HK, D]
    v = up[ids.long()]
    z = torch.einsum("tjd,td->tj", u, x)
    a = torch.nn.functional.gelu(z) if act == "gelu" else torch.relu(z)
    return torch.einsum("tj,tjd->td", w * a, v)


@pytest.mark.parametrize("dtype,D,Dout,H,k,N,T,act", [
    (torch.float32, 32, 48, 2, 4, 64, 7, "gelu"), (torch.float32, 256, 256, 4, 8, 300, 65, "relu"),
    (torch.float32, 1024, 512, 2, 4, 128, 33, "gelu"), (torch.bfloat16, 2048, 2048, 8, 16, 4096, 40, "gelu"),
    (torch.bfloat16, 512, 1024, 4, 8, 50, 129, "relu"), (torch.bfloat16, 4096, 4096, 2, 4, 64, 9, "gelu")])
def test_expert_stage_backward_from_given_selections(cuda_device, dtype, D, Dout, H, k, N, T, act):
    g = torch.Generator(device="cpu").manual_seed(D + T)
    cfg = syn.PeerConfig("t", D, Dout, H, 32, (N, 1), k, dtype, dtype, 1, T)
    op = make_op(cfg, cuda_device, activation=act)
    x = (torch.randn(T, D, generator=g)).to(dtype)
    dy = torch.randn(T, Dout, generator=g).to(dtype)
    down = (torch.randn(N, D, generator=g) * D ** -0.5).to(dtype)
    up = (torch.randn(N, Dout, generator=g) * D ** -0.5).to(dtype)
    ids = torch.randint(0, N, (T, H * k), generator=g, dtype=torch.int32)     # few rows: many collisions
    ids[:, 1] = ids[:, 0]                                                       # and repeats inside a token
    w = torch.rand(T, H * k, generator=g)
    leaves = [t.float().clone().requires_grad_(True) for t in (x, w, down, up)]
    _dense_reference(leaves[0], ids, leaves[1], leaves[2], leaves[3], act).backward(dy.float())
    dev = lambda t: t.to(cuda_device)
    gx, gw, gd, gu = op.gather_eval_backward(dev(x), dev(dy), dev(ids), dev(w), dev(down), dev(up))
    op.query_status()
    tol = 2e-5 if dtype == torch.float32 else 1e-4        # inputs are exact in both; only summation order differs
    for name, got, ref in (("x", gx, leaves[0].grad), ("weights", gw, leaves[1].grad),
                           ("down", gd, leaves[2].grad), ("up", gu, leaves[3].grad)):
        assert rel_err(got.cpu(), ref) < tol, (name, rel_err(got.cpu(), ref))
    # accumulation into given buffers: a second call doubles the table gradients
    op.gather_eval_backward(dev(x), dev(dy), dev(ids), dev(w), dev(down), dev(up), gd, gu)
    assert rel_err(gd.cpu(), 2 * leaves[2].grad) < tol and rel_err(gu.cpu(), 2 * leaves[3].grad) < tol


def test_expert_stage_backward_with_sums_in_bf16(cuda_device):
    """Table gradients accumulated in bf16 (what a bf16 training run keeps): few contributions per row, so the
    result is the fp32 sum to within a few bf16 roundings."""
    D, Dout, H, k, N, T = 2048, 2048, 8, 16, 8192, 64
    g = torch.Generator().manual_seed(7)
    cfg = syn.PeerConfig("t", D, Dout, H, 32, (N, 1), k, torch.bfloat16, torch.bfloat16, 1, T)
    op = make_op(cfg, cuda_device)
    dev = lambda t: t.to(cuda_device)
    x, dy = dev(torch.randn(T, D, generator=g).bfloat16()), dev(torch.randn(T, Dout, generator=g).bfloat16())
    down = dev((torch.randn(N, D, generator=g) * D ** -0.5).bfloat16())
    up = dev((torch.randn(N, Dout, generator=g) * D ** -0.5).bfloat16())
    ids = dev(torch.randint(0, N, (T, H * k), generator=g, dtype=torch.int32))
    w = dev(torch.rand(T, H * k, generator=g))
    gx, gw, gd, gu = op.gather_eval_backward(x, dy, ids, w, down, up)                       # fp32 sums
    gx2, gw2, gd2, gu2 = op.gather_eval_backward(x, dy, ids, w, down, up, grad_dtype=torch.bfloat16)
    op.query_status()
    assert gd2.dtype == torch.bfloat16 and gu2.dtype == torch.bfloat16
    assert torch.equal(gx, gx2) and torch.equal(gw, gw2)
    for a, b in ((gd2, gd), (gu2, gu)):
        l1 = float((a.float() - b).abs().sum() / b.abs().sum())
        assert l1 < 4e-3 and rel_err(a.float().cpu(), b.cpu()) < 1e-2, l1
    with pytest.raises(ValueError):
        op.gather_eval_backward(x, dy, ids, w, down, up, grad_dtype=torch.float16)


def test_backward_skips_out_of_range_ids(cuda_device):
    cfg = syn.PeerConfig("t", 32, 32, 1, 32, (16, 1), 2, torch.float32, torch.float32, 1, 3)
    op = make_op(cfg, cuda_device)
    dev = cuda_device
    x, dy = torch.randn(3, 32, device=dev), torch.randn(3, 32, device=dev)
    down, up = torch.randn(16, 32, device=dev), torch.randn(16, 32, device=dev)
    ids = torch.tensor([[0, 1], [99, 2], [-1, 3]], dtype=torch.int32, device=dev)
    w = torch.ones(3, 2, device=dev)
    gx, gw, gd, gu = op.gather_eval_backward(x, dy, ids, w, down, up)
    with pytest.raises(RuntimeError, match="outside"):
        op.query_status()
    assert float(gw[1, 0]) == 0.0 and float(gw[2, 0]) == 0.0
    ok = ids.clamp(0, 15)
    w2 = w.clone(); w2[1, 0] = 0; w2[2, 0] = 0                  # the skipped entries contribute nothing
    gx2, _, gd2, gu2 = op.gather_eval_backward(x, dy, ok, w2, down, up)
    op.query_status()
    assert torch.allclose(gx, gx2, atol=1e-6) and torch.allclose(gd, gd2, atol=1e-6) and torch.allclose(gu, gu2, atol=1e-6)


def test_score_path_backward_skips_positions_outside_the_key_grid(cuda_device):
    """peer_select_backward trusts nothing about the caller's product ids: a negative or too large position
    is recorded in the status word and its slot contributes ds = 0, exactly as if its weight gradient
    had been switched off; it is never turned into a key-row address."""
    cfg = syn.PeerConfig("t", 32, 32, 2, 32, (8, 8), 4, torch.float32, torch.float32, 1, 5)
    op = make_op(cfg, cuda_device, "product")
    g = torch.Generator().manual_seed(3)
    dev = cuda_device
    q = torch.randn(5, 2, 32, generator=g).to(dev)
    keys = [torch.randn(8, 16, generator=g).to(dev) for _ in range(2)]
    pid = torch.randint(0, 64, (5, 2, 4), generator=g, dtype=torch.int32).to(dev)
    sc = torch.randn(5, 2, 4, generator=g).to(dev)
    gw = torch.randn(5, 2, 4, generator=g).to(dev)
    good = op.select_backward(q, keys, pid, sc, gw)
    op.query_status()
    bad = pid.clone(); bad[1, 0, 2] = -7; bad[3, 1, 0] = 64
    got = op.select_backward(q, keys, bad, sc, gw)
    with pytest.raises(RuntimeError, match="outside"):
        op.query_status()
    assert torch.isfinite(got).all()
    untouched = [(0, 0), (0, 1), (1, 1), (2, 0), (2, 1), (3, 0), (4, 0), (4, 1)]
    for t, h in untouched:
        assert torch.equal(got[t, h], good[t, h])
    assert not torch.equal(got[1, 0], good[1, 0])


@pytest.mark.parametrize("name", ["tiny_fp32", "c1_affine"])
def test_module_gradients_match_reference_golden(cuda_device, name):
    cfg, sd, x, rec = load_golden(name)
    grad_out, dense, tables = load_golden_grads(name)
    m = _module(cfg, sd, cuda_device)
    out, g = _module_grads(m, x.to(cuda_device), grad_out.to(cuda_device))
    m._op.query_status()
    ref_out = torch.from_numpy(rec["out"])
    assert rel_err(out.detach().cpu(), ref_out) < 2e-5
    assert g["sub_keys.0"] is None and g["sub_keys.1"] is None
    for k in GRAD_DENSE:
        assert rel_err(g[k].cpu(), dense[k]) < 2e-5, (k, rel_err(g[k].cpu(), dense[k]))
    for k in GRAD_TABLES:
        rows, vals = tables[k]
        got = g[k].cpu()
        assert rel_err(got[rows], vals) < 2e-5, k
        untouched = torch.ones(got.shape[0], dtype=torch.bool)
        untouched[rows] = False
        assert float(got[untouched].abs().max()) == 0.0, k
    # the tracker attributes are filled on this path too
    assert m._last_expert_indices.shape == (cfg.batch, cfg.seq, cfg.num_heads, cfg.top_k)
    assert torch.equal(m._last_expert_indices.cpu().int(), torch.from_numpy(rec["ids"]).view(m._last_expert_indices.shape))


@pytest.mark.parametrize("mode", ["reference", "product"])
def test_bf16_layer_gradients_against_the_oracle(cuda_device, mode):
    cfg = syn.scaled(syn.CONFIGS["c2"], product_key_dim=(64, 48), batch=2, seq=96)
    sd = syn.make_weights(cfg, 11, "cpu", random_affine=True)
    x = syn.make_input(cfg, 11, "cpu")
    grad_out = (torch.randn(cfg.batch, cfg.seq, cfg.output_dim, generator=torch.Generator().manual_seed(5))
                .to(cfg.dtype))
    ref = oracle_gradients(cfg, sd, x, grad_out.float(), mode)
    m = _module(cfg, sd, cuda_device, mode)
    out, g = _module_grads(m, x.to(cuda_device), grad_out.to(cuda_device))
    m._op.query_status()
    assert out.dtype == cfg.dtype and g["x"].dtype == cfg.dtype and g["expert_up.weight"].dtype == cfg.dtype
    for k in GRAD_DENSE + GRAD_TABLES:
        a, b = g[k].float().cpu(), ref[k]
        l1 = float((a - b).abs().sum() / b.abs().sum())
        assert l1 <= 2e-2 and rel_err(a, b) <= 5e-2, (k, l1, rel_err(a, b))


def test_table_gradients_with_thousands_of_contributions_per_row(cuda_device):
    """The reference's id arithmetic (i0 + i1) sends every token to the same few rows: here 31 rows take
    about four thousand contributions each.  The default ("auto") backward sums such rows in fp32 - in a
    buffer of just the reachable rows - and rounds once (what the reference's embedding backward does), so
    the result stays at bf16 rounding of the fp32 sum; the opt-in bf16 running sums are allowed to drift and
    only have to stay finite."""
    cfg = syn.PeerConfig("coll", 256, 256, 4, 64, (16, 16), 8, torch.bfloat16, torch.bfloat16, 4, 1024)
    sd = syn.make_weights(cfg, 21, "cpu", random_affine=True)
    x = syn.make_input(cfg, 21, "cpu")
    grad_out = torch.randn(cfg.batch, cfg.seq, cfg.output_dim, generator=torch.Generator().manual_seed(9)).to(cfg.dtype)
    ref = oracle_gradients(cfg, sd, x, grad_out.float(), "reference")
    m = _module(cfg, sd, cuda_device, "reference")
    from llm720_b200.autograd import _table_grad_plan
    assert m.table_grad_sums == "auto"
    assert _table_grad_plan(m, m.expert_down.weight, cfg.tokens) == (torch.float32, 31)
    m.index_mode = "product"
    assert _table_grad_plan(m, m.expert_down.weight, 16) == (torch.bfloat16, 256)      # 2 selections per row
    assert _table_grad_plan(m, m.expert_down.weight, cfg.tokens) == (torch.float32, 256)
    m.index_mode = "reference"
    out, g = _module_grads(m, x.to(cuda_device), grad_out.to(cuda_device))
    m._op.query_status()
    per_row = torch.bincount(m._last_expert_indices.view(-1).cpu(), minlength=31)
    assert int(per_row.max()) > 2000 and int(m._last_expert_indices.max()) <= 30
    for k in GRAD_TABLES:
        a, b = g[k].float().cpu(), ref[k]
        assert g[k].dtype == cfg.dtype and g[k].shape == (256, 256)
        assert float(a[31:].abs().max()) == 0.0                       # rows the ids cannot reach
        l1 = float((a - b).abs().sum() / b.abs().sum())
        # fp32 atomics in another order + one bf16 rounding of each sum
        assert l1 <= 8e-3 and rel_err(a, b) <= 1e-2, (k, l1, rel_err(a, b))
    m2 = _module(cfg, sd, cuda_device, "reference")
    m2.table_grad_sums = "table"
    _, g2 = _module_grads(m2, x.to(cuda_device), grad_out.to(cuda_device))
    for k in GRAD_TABLES:
        assert torch.isfinite(g2[k]).all()


def test_eval_and_train_mode_agree_without_dropout_and_dropout_runs(cuda_device):
    cfg, sd, x, _ = load_golden("c1")
    grad_out, _, _ = load_golden_grads("c1_affine")
    xd, gd = x.to(cuda_device), grad_out.to(cuda_device)
    out_e, g_e = _module_grads(_module(cfg, sd, cuda_device), xd, gd)
    out_t, g_t = _module_grads(_module(cfg, sd, cuda_device, train=True), xd, gd)
    assert torch.equal(out_e, out_t)
    assert rel_err(g_t["x"].cpu(), g_e["x"].cpu()) < 1e-5
    with torch.no_grad():
        out_i = _module(cfg, sd, cuda_device)(xd)
    assert rel_err(out_e.detach().cpu(), out_i.cpu()) < 2e-6            # same values as the inference path
    m = _module(cfg, sd, cuda_device, train=True)
    m.dropout.p = 0.5
    torch.manual_seed(0)
    out_d, g_d = _module_grads(m, xd, gd)
    assert torch.isfinite(out_d).all() and torch.isfinite(g_d["x"]).all()
    assert not torch.equal(out_d, out_e)
    # frozen tables: no table gradient is requested or produced
    m2 = _module(cfg, sd, cuda_device)
    m2.expert_down.weight.requires_grad_(False)
    m2.expert_up.weight.requires_grad_(False)
    _, g2 = _module_grads(m2, xd, gd)
    assert g2["expert_down.weight"] is None and rel_err(g2["x"].cpu(), g_e["x"].cpu()) < 1e-5


def test_fp8_tables_have_no_backward(cuda_device):
    cfg = syn.scaled(syn.CONFIGS["c2"], product_key_dim=(32, 32), batch=1, seq=8)
    m = _module(cfg, syn.make_weights(cfg, 1, "cpu"), cuda_device)
    m.quantize_tables_e4m3()
    x = syn.make_input(cfg, 1, cuda_device).requires_grad_(True)
    with pytest.raises(RuntimeError, match="inference-only"):
        m(x)
