"""Two-or-more-GPU check of the expert-parallel layer, run under torchrun:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29611 tests/multi_gpu_check.py

Every rank holds a row shard of the tables of a decode-shaped layer (d_model 4096, 16 heads,
query_dim 256, top-k 16, product-key ids); the result must equal the single-device layer that
rank 0 evaluates on the concatenated batch with the full tables.  Also times the sharded step.
CHECK_EXCHANGE=direct runs the layer with the library's direct exchange (stores into the peers' memory
instead of the three collectives) and also compares it with the collective form: same tuples per token,
outputs equal up to the order in which the ranks' partial sums are added.
CHECK_EXCHANGE=direct_timeout: the last rank sits one step out (it is idle between steps, nothing of its own in
flight); the others' bounded waits run out after two seconds and show as an error code, nothing hangs; the
exchange is then closed and built anew, and the next step is right again.
"""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from llm720_b200 import PEER, synthetic as syn          # noqa: E402
from llm720_b200.sharded import ShardedPEER              # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=dev)
    keys = int(os.environ.get("CHECK_KEYS", "256"))
    cfg = syn.scaled(syn.CONFIGS["c4"], product_key_dim=(keys, keys), batch=64, seq=1)
    compare = keys <= 512            # larger tables: only this rank's shard is ever built, timing only
    sd = syn.make_weights(cfg, 4, dev, random_affine=True, tables=compare)   # same seed: identical on every rank
    x = syn.make_input(cfg, 4, dev)                                 # [64, 1, 4096]
    rows = cfg.num_experts // world
    t_local = cfg.tokens // world
    if compare:
        down = sd["expert_down.weight"][rank * rows:(rank + 1) * rows].contiguous()
        up = sd["expert_up.weight"][rank * rows:(rank + 1) * rows].contiguous()
    else:
        down = syn.make_table_shard(cfg, "expert_down", rank * rows, rows, 4, dev)
        up = syn.make_table_shard(cfg, "expert_up", rank * rows, rows, 4, dev)
    mode = os.environ.get("CHECK_EXCHANGE", "nccl")
    xl = x.view(cfg.tokens, 1, -1)[rank * t_local:(rank + 1) * t_local].contiguous()
    if mode == "direct_timeout":
        return missing_rank(cfg, sd, down, up, xl, rank, world, dev)
    layer = ShardedPEER.build(cfg.module_kwargs(), sd, down, up, exchange=mode)
    out = layer(xl)
    layer.layer._op.query_status()
    layer.check_exchange()
    same = True
    if mode == "direct":
        counts = layer.received_counts().clone()
        other = ShardedPEER.build(cfg.module_kwargs(), sd, down, up, exchange="nccl")
        out_nccl = other(xl)
        same = bool(torch.equal(counts.view(-1), other.received_counts().reshape(-1).to(counts.dtype)))
        same = same and bool(torch.allclose(out.float(), out_nccl.float(), rtol=0, atol=2e-3))
        for _ in range(3):                       # both parities of the region, and a repeat: same result every step
            again = layer(xl)
            same = same and bool(torch.equal(again, out))
        layer.check_exchange()

    err = mag = 0.0
    if compare:
        with torch.device("meta"):
            full = PEER(**cfg.module_kwargs())
        full.load_state_dict(sd, assign=True)
        full.eval().requires_grad_(False)
        full.index_mode = "product"
        with torch.no_grad():
            ref = full(x)[rank * t_local:(rank + 1) * t_local]
        err = float((out.float() - ref.float()).abs().max())
        mag = float(ref.float().abs().max())
    finite = bool(torch.isfinite(out.float()).all()) and float(out.float().abs().max()) > 0
    ok = torch.tensor([1 if (err <= 2e-2 and finite and same) else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)

    # timing: per-layer latency of the sharded step (max over ranks, CUDA events)
    for _ in range(5):
        layer(xl)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier(); torch.cuda.synchronize()
    e0.record()
    steps = 20
    for _ in range(steps):
        layer(xl)
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    layer.check_exchange()
    layer.close()
    if rank == 0:
        print(f"sharded PEER x{world} ({mode} exchange): experts {cfg.num_experts}, tokens {cfg.tokens}, "
              f"{'compared with the single-device layer: ' if compare else 'timing only; '}max-abs err {err:.3g} "
              f"(|ref| max {mag:.3g}), {float(ms):.3f} ms/step, {cfg.tokens / float(ms) * 1e3:.0f} tokens/s, "
              f"{'OK' if int(ok) else 'MISMATCH'}")
    dist.destroy_process_group()
    sys.exit(0 if int(ok) else 1)


def missing_rank(cfg, sd, down, up, xl, rank, world, dev):
    layer = ShardedPEER.build(cfg.module_kwargs(), sd, down, up, exchange="direct")
    good = layer(xl)
    layer.check_exchange()
    dist.barrier()
    noticed = True
    if rank != world - 1:                      # the last rank does not take part in this step
        layer(xl)
        try:
            layer.check_exchange()
            noticed = False
        except RuntimeError as e:
            noticed = "did not arrive" in str(e)
    dist.barrier()                             # host side: every rank is between steps
    layer.close()
    fresh = ShardedPEER.build(cfg.module_kwargs(), sd, down, up, exchange="direct")
    again = fresh(xl)
    fresh.check_exchange()
    ok = torch.tensor([1 if (noticed and torch.equal(again, good)) else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    fresh.close()
    if rank == 0:
        print(f"sharded PEER x{world} (direct exchange, one rank missing a step): the others' waits ran out and were "
              f"reported, the rebuilt exchange gives the same result: {'OK' if int(ok) else 'MISMATCH'}")
    dist.destroy_process_group()
    sys.exit(0 if int(ok) else 1)


if __name__ == "__main__":
    main()
