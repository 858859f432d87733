"""`hidden + PEER(LayerNorm(hidden))` in one library call (the feed-forward half of the reference's
TransformerBlock.forward, llm/models/foundation.py:196-205) against the same expression built from
torch's LayerNorm and the oracle.

Tolerances: fp32 within 2e-5 of the largest entry; bf16: the reference rounds ln_2's output to bf16 before
the layer, so the oracle is fed the bf16-rounded LayerNorm output; max-abs <= 3e-2, L1-relative <= 1e-3 of
the block output (whose magnitude is dominated by the residual)."""
import pytest
import torch

from llm720_b200 import PEER, synthetic as syn
from oracle import peer_oracle as orc
from _util import load_golden, oracle_shape, oracle_weights, rel_err

pytestmark = pytest.mark.gpu


def _module(cfg, sd, device, index_mode="reference"):
    m = PEER(**cfg.module_kwargs()).to(cfg.dtype)
    m.load_state_dict({k: v.to(cfg.dtype) for k, v in sd.items()})
    m = m.to(device).eval()
    m.index_mode = index_mode
    return m


def _ln(D, seed):
    ln = torch.nn.LayerNorm(D, eps=1e-5)                    # fp32 parameters, as the reference keeps them
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        ln.weight.copy_(1.0 + 0.2 * torch.randn(D, generator=g))
        ln.bias.copy_(0.1 * torch.randn(D, generator=g))
    return ln


def test_block_forward_fp32_against_golden_layer(cuda_device):
    cfg, sd, x, _ = load_golden("c1_affine")
    ln = _ln(cfg.input_dim, 1)
    hidden = x * 3.0 + 0.5                                   # not normalised on purpose
    with torch.no_grad():
        ref_in = ln(hidden)
        ref, ref_ids, _ = orc.forward(ref_in, oracle_weights(sd), oracle_shape(cfg), "reference")
        ref = hidden + ref
    m = _module(cfg, sd, cuda_device)
    with torch.no_grad():
        out = m.block_forward(hidden.to(cuda_device), ln.to(cuda_device))
        two_step = hidden.to(cuda_device) + m(ln(hidden.to(cuda_device)))
    m._op.query_status()
    assert rel_err(out.cpu(), ref) < 2e-5
    assert rel_err(out.cpu(), two_step.cpu()) < 2e-6
    assert torch.equal(m._last_expert_indices.cpu(), ref_ids)


def test_block_forward_bf16_sliced(cuda_device):
    cfg = syn.scaled(syn.CONFIGS["c2"], product_key_dim=(256, 128), batch=2, seq=150)
    sd = syn.make_weights(cfg, 9, cuda_device, random_affine=True)
    m = _module(cfg, sd, cuda_device, "product")
    m.max_slice_tokens = 128                                  # three slices
    ln = _ln(cfg.input_dim, 2).to(cuda_device)
    hidden = (syn.make_input(cfg, 9, cuda_device).float() * 2.0 + 0.25).to(cfg.dtype)
    with torch.no_grad():
        out = m.block_forward(hidden, ln)
        m._op.query_status()
        ln_out = ln(hidden.float()).to(torch.bfloat16)        # fp32 statistics and parameters, bf16 result: what the layer is fed
        tok = torch.arange(0, cfg.tokens, 5)
        sd_cpu = {k: v.cpu() for k, v in sd.items()}
        xs = ln_out.view(-1, cfg.input_dim)[tok.to(cuda_device)].cpu().float().unsqueeze(0)
        y, _, _ = orc.forward(xs, oracle_weights(sd_cpu, torch.float32, tables_as_stored=True), oracle_shape(cfg), "product",
                              token_chunk=64)
        ref = hidden.view(-1, cfg.input_dim)[tok.to(cuda_device)].cpu().float() + y[0]
    got = out.view(-1, cfg.output_dim)[tok.to(cuda_device)].cpu().float()
    mx = float((got - ref.to(torch.bfloat16).float()).abs().max())
    l1 = float((got - ref.to(torch.bfloat16).float()).abs().sum() / ref.abs().sum())     # both rounded to bf16 once
    assert mx <= 3e-2 and l1 <= 1e-3, (mx, l1)


@pytest.mark.parametrize("name", ["k3d_h8_fp32", "h8_fp32"])
def test_block_forward_on_the_general_kernels(cuda_device, name):
    """Several neurons per expert / a 3-D key grid: the residual is added by the general expert kernel."""
    from _util import load_general
    cfg, sd, x, _ = load_general(name)
    m = _module(cfg, sd, cuda_device)
    ln = _ln(cfg.input_dim, 3).to(cuda_device)
    hidden = (x * 2.0 - 0.3).to(cuda_device)
    with torch.no_grad():
        out = m.block_forward(hidden, ln)
        two_step = hidden + m(ln(hidden))
    m._op.query_status()
    assert rel_err(out.cpu(), two_step.cpu()) < 2e-6


def test_block_forward_argument_checks(cuda_device):
    m = PEER(64, 32, 256, num_experts_per_tok=4, num_heads=2, query_dim=32, product_key_dim=[16, 16]).to(cuda_device).eval()
    ln = torch.nn.LayerNorm(64).to(cuda_device)
    x = torch.randn(1, 4, 64, device=cuda_device)
    with torch.no_grad(), pytest.raises(ValueError, match="input_dim"):
        m.block_forward(x, ln)
    with pytest.raises(RuntimeError, match="inference path"):
        m.block_forward(x, ln)


def test_three_blocks_chained_against_the_oracle(cuda_device):
    """The twelve-layer PEER stack of the benchmark, at a size the oracle finishes in seconds: three
    blocks h + PEER(ln_2(h)) in a row, every block checked against the oracle on the block's own input
    (the same check the benchmark line reports as extra.c5_peer_stack.parity)."""
    import bench
    ok, (mx, l1) = bench._stack_parity(cuda_device)
    assert ok, (mx, l1)
