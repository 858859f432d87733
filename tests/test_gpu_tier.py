"""Tables that live in pinned host memory with an HBM cache of the most used rows (PEER.enable_host_tier /
peer_set_row_tier): the role of the reference's HierarchicalExpertCache (llm/models/kernels/
peer_cutlass.cu:110-536, docs/MEMORY_HIERARCHY.md:5-11).  A row is the same bytes wherever it is read
from, and the expert stage adds in the same order, so the tiered layer must reproduce the all-HBM layer
bit for bit - with a cache that holds some of the selected rows, none of them, or all of them."""
import pytest
import torch

from llm720_b200 import PEER, synthetic as syn
from llm720_b200.tracking import DeviceUsageCounter

pytestmark = pytest.mark.gpu


def _layer(cfg, dev, fp8=False):
    sd = syn.make_weights(cfg, 71, dev, random_affine=True)
    with torch.device("meta"):
        m = PEER(**cfg.module_kwargs())
    m.load_state_dict(sd, assign=True)
    if fp8:
        m.quantize_tables_e4m3()
    m.eval().requires_grad_(False)
    m.index_mode = "product"
    return m


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("cache_rows", [1, 700, 4096])
def test_tiered_tables_reproduce_the_resident_layer(cuda_device, cache_rows, fp8):
    cfg = syn.scaled(syn.CONFIGS["c2"], product_key_dim=(64, 64), batch=2, seq=150)
    m = _layer(cfg, cuda_device, fp8)
    x = syn.make_input(cfg, 71, cuda_device)
    with torch.no_grad():
        want = m(x).clone()
    ids = m._last_expert_indices.clone()
    counts = torch.bincount(ids.view(-1), minlength=cfg.num_experts)
    m.enable_host_tier(cache_rows, usage_counts=counts)
    assert m.expert_down.weight.device.type == "cpu" and m.expert_down.weight.is_pinned()
    row_map = m._tier[0]
    served_from_host = int((row_map[ids.view(-1)] < 0).sum())
    if cache_rows == 4096:
        assert served_from_host == 0
    else:
        assert served_from_host > 0                        # rows really come over PCIe in this run
    with torch.no_grad():
        got = m(x)
        m._op.query_status()
        assert torch.equal(got, want)
        assert torch.equal(m._last_expert_indices, ids)
        # the block form (LayerNorm + residual) runs the same expert stage
        ln = torch.nn.LayerNorm(cfg.input_dim, device=cuda_device, dtype=cfg.dtype)
        tiered_block = m.block_forward(x, ln)
    m.disable_host_tier()
    with torch.no_grad():
        assert torch.equal(m(x), want)
        assert torch.equal(m.block_forward(x, ln), tiered_block)


def test_hot_rows_come_from_the_usage_counter_and_gradients_are_refused(cuda_device):
    cfg = syn.scaled(syn.CONFIGS["c2"], product_key_dim=(32, 32), batch=1, seq=64)
    m = _layer(cfg, cuda_device)
    x = syn.make_input(cfg, 72, cuda_device)
    counter = DeviceUsageCounter(cfg.num_experts, 1, cuda_device)
    with torch.no_grad():
        want = m(x).clone()
    counter.record_usage(0, m._last_expert_indices, cfg.batch, cfg.seq)
    m.enable_host_tier(100, usage_counts=counter.counts[0])
    hot = torch.nonzero(m._tier[0] >= 0).flatten()
    assert hot.numel() == 100
    assert int(counter.counts[0][hot].min()) >= int(torch.topk(counter.counts[0], 101).values[-1])
    with torch.no_grad():
        assert torch.equal(m(x), want)
    with pytest.raises(RuntimeError, match="inference-only"):
        m.requires_grad_(False)
        m(x.clone().requires_grad_(True))
    with pytest.raises(ValueError):
        PEER(64, 64, 64, product_key_dim=[8, 8]).enable_host_tier(4)          # fp32 tables
