"""Expert-usage counting on the device.

The reference's ``ExpertUsageTracker.record_usage`` (llm/utils/experts/
tracking.py:79-104) copies the ``[B,S,H,k]`` index tensor to the host after
every PEER forward and increments a Python ``Counter`` once per element
(2 M increments per layer and step at the benchmark shape).  ``DeviceUsageCounter``
keeps one int64 histogram per layer on the GPU, filled by
``peer_usage_histogram``, and hands the totals to a reference tracker only when
asked (``drain_into``), e.g. at the tracker's logging period.
"""
from __future__ import annotations

import ctypes as C
from functools import partial

import torch

from . import _lib


class DeviceUsageCounter:
    def __init__(self, num_experts: int, num_layers: int, device):
        self.num_experts, self.num_layers = num_experts, num_layers
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("DeviceUsageCounter counts on a CUDA device")
        self.lib = _lib.load()
        self.counts = torch.zeros(num_layers, num_experts, dtype=torch.int64, device=self.device)
        self.dropped = torch.zeros(1, dtype=torch.int64, device=self.device)
        self.period_tokens = 0
        self.total_tokens_processed = 0

    def record_usage(self, layer_idx: int, expert_indices: torch.Tensor, batch_size: int, seq_len: int):
        """Same signature as the reference tracker's method; asynchronous on the current stream."""
        if not 0 <= layer_idx < self.num_layers:
            raise IndexError(f"layer {layer_idx} of {self.num_layers}")
        ids = expert_indices.detach()
        if ids.device != self.device or ids.dtype != torch.int64:
            raise TypeError("expert_indices must be an int64 tensor on the counter's device")
        ids = ids.contiguous()
        with torch.cuda.device(self.device):
            rc = self.lib.peer_usage_histogram(ids.data_ptr(), ids.numel(), self.counts[layer_idx].data_ptr(),
                                               self.num_experts, self.dropped.data_ptr(),
                                               C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))
        _lib.check(rc, None)
        self.period_tokens += batch_size * seq_len
        self.total_tokens_processed += batch_size * seq_len

    def drain_into(self, tracker) -> None:
        """Add the device totals to ``tracker.expert_counters`` (a reference ``ExpertUsageTracker``) and its
        token counts, then reset.  One device-to-host copy of the non-zero entries per layer."""
        host = self.counts.cpu()
        for layer in range(self.num_layers):
            nz = torch.nonzero(host[layer]).flatten()
            for e, c in zip(nz.tolist(), host[layer][nz].tolist()):
                tracker.expert_counters[layer][e] += c
        tracker.period_tokens += self.period_tokens
        tracker.total_tokens_processed += self.period_tokens
        self.counts.zero_()
        self.period_tokens = 0


def hook_expert_tracking(module, counter: DeviceUsageCounter) -> int:
    """Register forward hooks on the PEER layers of ``module.blocks[*].feed_forward`` (the discovery rule of
    llm/utils/experts/tracking.py:358-373) that count on the device.  Returns the number of layers hooked."""
    def _hook(layer_idx, mod, args, output):
        ids = getattr(mod, "_last_expert_indices", None)
        if ids is not None:
            b, s = args[0].shape[:2]
            counter.record_usage(layer_idx, ids, b, s)

    n = 0
    for block in getattr(module, "blocks", []):
        ff = getattr(block, "feed_forward", None)
        if ff is not None and "PEER" in ff.__class__.__name__:
            ff.register_forward_hook(partial(_hook, n))
            n += 1
    return n
