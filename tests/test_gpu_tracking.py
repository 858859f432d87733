"""Device-side expert-usage counting against the host loop of the reference tracker
(llm/utils/experts/tracking.py:96-100), restated here with collections.Counter."""
from collections import Counter, defaultdict

import pytest
import torch

from llm720_b200 import PEER
from llm720_b200.tracking import DeviceUsageCounter, hook_expert_tracking

pytestmark = pytest.mark.gpu


class _HostTracker:
    """The counting part of the reference's ExpertUsageTracker."""
    def __init__(self):
        self.expert_counters = defaultdict(Counter)
        self.period_tokens = 0
        self.total_tokens_processed = 0

    def record_usage(self, layer_idx, expert_indices, batch_size, seq_len):
        for e in expert_indices.detach().cpu().numpy().flatten():
            self.expert_counters[layer_idx][int(e)] += 1
        self.period_tokens += batch_size * seq_len
        self.total_tokens_processed += batch_size * seq_len


def test_histogram_equals_the_host_loop(cuda_device):
    g = torch.Generator().manual_seed(3)
    counter = DeviceUsageCounter(1000, 2, cuda_device)
    host, drained = _HostTracker(), _HostTracker()
    for step in range(3):
        for layer in range(2):
            ids = torch.randint(0, 1000, (2, 17, 4, 8), generator=g)
            ids[0, 0, 0, :] = 5                                           # repeats inside a row
            host.record_usage(layer, ids, 2, 17)
            counter.record_usage(layer, ids.to(cuda_device), 2, 17)
    counter.drain_into(drained)
    assert drained.expert_counters == host.expert_counters
    assert drained.period_tokens == host.period_tokens == 3 * 2 * 2 * 17
    assert int(counter.counts.sum()) == 0                                 # reset by the drain
    # ids outside the table are counted as dropped, never used as an address
    bad = torch.tensor([[[[-1, 1000, 7, 7]]]], device=cuda_device)
    counter.record_usage(0, bad, 1, 1)
    assert int(counter.dropped.item()) == 2 and int(counter.counts[0, 7]) == 2


def test_hook_on_a_block_structure(cuda_device):
    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.feed_forward = PEER(64, 64, 256, num_experts_per_tok=4, num_heads=2, query_dim=32, product_key_dim=[16, 16])

    class Model(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.blocks = torch.nn.ModuleList([Block(), Block()])

    model = Model().to(cuda_device).eval()
    counter = DeviceUsageCounter(256, 2, cuda_device)
    assert hook_expert_tracking(model, counter) == 2
    x = torch.randn(2, 9, 64, device=cuda_device)
    with torch.no_grad():
        for b in model.blocks:
            b.feed_forward(x)
    for layer, b in enumerate(model.blocks):
        ref = torch.bincount(b.feed_forward._last_expert_indices.flatten().cpu(), minlength=256)
        assert torch.equal(counter.counts[layer].cpu(), ref)
    assert counter.total_tokens_processed == 2 * 2 * 9
