#!/usr/bin/env python
"""PEER-layer forward benchmark.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the CPU implementation of the same layer

One step = one forward of the 1,048,576-expert bf16 PEER layer (d_model 2048,
8 heads, query dim 256, 1024x1024 sub-keys, top-k 16) over one batch of
[8, 2048, 2048] synthetic activations (seeded N(0,1); weights N(0, 1/fan_in)).
With N GPUs every rank holds a replica of the expert tables and processes its
own batch (token sharding, no collective in the layer): weak scaling.

Prints one JSON line on rank 0.  `value` is tokens/s with inputs resident in
HBM; `e2e` is the same through the host-buffer entry point (pinned host x in,
host output back, copies inside the timed region); `roofline` is the expert
(gather) stage: algorithmic gathered bytes / its CUDA-event duration over the
measured HBM copy bandwidth.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "PEER-layer tokens/sec @1M experts"
UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes moved by the expert-stage kernel per algorithmic byte, from one ncu capture of a smaller
# case of the same kernel (4096 tokens, 262,144 experts; dram__bytes_read.sum + dram__bytes_write.sum =
# 4.150 GB for 4.295 GB of algorithmic bytes; profiles/gather_eval_bf16_d2048_small_case.md).  Traffic
# grows in proportion to the tokens, so the bench scales it to its own launch size.
# FP8 tables: 2.147 GB read + 0.02 GB written for 2.152 GB algorithmic (profiles/gather_eval_fp8_d2048_small_case.md).
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = {"bfloat16": 0.966, "float8_e4m3fn": 1.007}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c2", choices=["c2", "c3"])
    ap.add_argument("--index-mode", default="product", choices=["product", "reference"])
    ap.add_argument("--tokens", type=int, default=0, help="override tokens per GPU (profiling of small cases)")
    ap.add_argument("--keys", type=int, default=0, help="override sub-keys per dimension (profiling of small cases)")
    ap.add_argument("--cpu-sample-tokens", type=int, default=256)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--backward", action="store_true",
                    help="also time forward+backward (training step of the layer) and add a 'backward' object")
    return ap.parse_args()


def hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clock/throttle samples every 50 ms while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.Q,
                                       "--format=csv,noheader,nounits", "-lms", "50"],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.f.read().splitlines():
            parts = [s.strip() for s in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        self.f.close()
        os.unlink(self.f.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def build_cfg(args):
    from llm720_b200 import synthetic as syn
    cfg = syn.CONFIGS[args.config]
    if args.tokens:
        cfg = syn.scaled(cfg, batch=1, seq=args.tokens)
    if args.keys:
        cfg = syn.scaled(cfg, product_key_dim=(args.keys, args.keys))
    return cfg


def cpu_reference_run(cfg, sd_cpu, x_cpu, index_mode, steps, warmup, sample_tokens):
    """Times the CPU implementation of the layer (the oracle restatement of the reference's
    PyTorch forward, run natively in the configuration's dtype with every host thread) on a
    token sample of the workload.  Returns (tokens/s, cores, sample description, ms/step)."""
    from oracle import peer_oracle as orc
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n = min(sample_tokens, x_cpu.shape[0] * x_cpu.shape[1])
    xs = x_cpu.reshape(1, -1, cfg.input_dim)[:, :n].contiguous()
    f = lambda k: sd_cpu[k]
    w = orc.PeerWeights(f("query_proj.weight"), f("query_proj.bias"), f("query_layer_norm.weight"),
                        f("query_layer_norm.bias"), [f("sub_keys.0"), f("sub_keys.1")],
                        f("expert_down.weight"), f("expert_up.weight"), sd_cpu.get("down_scale"),
                        sd_cpu.get("up_scale"))
    kw = dict(cfg.module_kwargs()); kw.pop("dropout")
    shape = orc.PeerShape(**kw)
    with torch.no_grad():
        for _ in range(warmup):
            orc.forward(xs, w, shape, index_mode)
        t0 = time.perf_counter()
        for _ in range(steps):
            orc.forward(xs, w, shape, index_mode)
        dt = time.perf_counter() - t0
    return n * steps / dt, cores, f"first {n} tokens of the {cfg.tokens}-token batch, {steps} passes, {x_cpu.dtype}", dt / steps * 1e3


def make_layer(cfg, args, device):
    from llm720_b200 import PEER, synthetic as syn
    sd = syn.make_weights(cfg, 0, device)
    with torch.device("meta"):          # no 2 x 8.6 GB fp32 default tables
        m = PEER(**cfg.module_kwargs())
    m.load_state_dict(sd, assign=True)
    if cfg.table_dtype == torch.float8_e4m3fn:
        m.quantize_tables_e4m3()
    m.eval().requires_grad_(False)
    m.index_mode = args.index_mode
    return m, sd


def time_backward(layer, cfg, x, steps):
    """Forward+backward of the layer (all parameters and x require gradients), and the expert-stage
    gradient kernel on its own.  Algorithmic bytes of that kernel per (token, slot): the two table rows
    read, and the two gradient rows (same dtype) read and written."""
    T, HK = cfg.tokens, cfg.num_heads * cfg.top_k
    layer.requires_grad_(True)
    xg = x.clone().requires_grad_(True)
    gen = torch.Generator(device=x.device).manual_seed(1)
    grad_out = torch.randn(x.shape[0], x.shape[1], cfg.output_dim, generator=gen, device=x.device).to(cfg.dtype)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    for i in range(2 + steps):
        if i == 2:
            torch.cuda.synchronize()
            ev[0].record()
        layer.zero_grad(set_to_none=True)
        xg.grad = None
        layer(xg).backward(grad_out)
    ev[1].record()
    torch.cuda.synchronize()
    step_ms = ev[0].elapsed_time(ev[1]) / steps
    layer.zero_grad(set_to_none=True)
    layer.requires_grad_(False)
    # the kernel alone, on the selections of the last forward
    op = layer._op
    ids = layer._last_expert_indices.view(T, HK).to(torch.int32)
    w = torch.softmax(layer._last_expert_scores.view(T, cfg.num_heads, cfg.top_k), -1).view(T, HK).contiguous()
    gdt = cfg.table_dtype                      # the sums are formed in the tables' dtype, as in the training step
    gd = torch.zeros(layer.expert_down.weight.shape, dtype=gdt, device=x.device)
    gu = torch.zeros(layer.expert_up.weight.shape, dtype=gdt, device=x.device)
    x2, g2 = x.view(T, -1), grad_out.view(T, -1)
    for i in range(1 + 3):
        if i == 1:
            ev[2].record()
        op.gather_eval_backward(x2, g2, ids, w, layer.expert_down.weight, layer.expert_up.weight, gd, gu, grad_dtype=gdt)
    ev[3].record()
    torch.cuda.synchronize()
    op.query_status()
    k_ms = ev[2].elapsed_time(ev[3]) / 3
    eb = torch.empty(0, dtype=cfg.table_dtype).element_size()
    bytes_alg = T * HK * (cfg.input_dim + cfg.output_dim) * (eb + 2 * eb)     # rows read; gradient rows read and written
    peak, kind = hbm_peak()
    return {"fwd_bwd_ms_per_step": step_ms, "fwd_bwd_tokens_per_s": T / (step_ms / 1e3), "steps": steps,
            "gather_grad_kernel_ms": k_ms, "algorithmic_bytes_per_launch": bytes_alg,
            "achieved_GBps": bytes_alg / (k_ms / 1e3) / 1e9, "frac_of_hbm_peak": bytes_alg / (k_ms / 1e3) / 1e9 / peak,
            "peak_kind": kind}


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = build_cfg(args)
    from llm720_b200 import synthetic as syn

    workload = {"workload": f"{cfg.name}: PEER forward, {cfg.num_experts} experts, d_model {cfg.input_dim}, "
                            f"{cfg.num_heads} heads, query_dim {cfg.query_dim}, top_k {cfg.top_k}, "
                            f"x [{cfg.batch},{cfg.seq},{cfg.input_dim}] per GPU",
                "tokens_per_gpu": cfg.tokens, "index_mode": args.index_mode,
                "table_dtype": str(cfg.table_dtype).replace("torch.", ""),
                "parallelism": f"token-sharded x{world}, replicated tables, no collective",
                "l2": "inputs larger than L2: each step gathers %.1f GB of table rows" %
                      (cfg.gathered_bytes_per_token() * cfg.tokens / 1e9)}

    if args.impl == "reference":
        if rank != 0:
            return
        # the CPU implementation, on this box's host cores, on a bounded sample of the same workload
        table_rows = None if args.index_mode == "product" else cfg.product_key_dim[0] + cfg.product_key_dim[1]
        gen_dev = "cuda" if torch.cuda.is_available() else "cpu"      # generation only; the timed work is on the CPU
        sd = {k: v.cpu() for k, v in syn.make_weights(cfg, 0, gen_dev, table_rows=table_rows).items()}
        if cfg.table_dtype == torch.float8_e4m3fn:
            sd["expert_down.weight"], sd["down_scale"] = syn.quantize_rows_e4m3(sd["expert_down.weight"])
            sd["expert_up.weight"], sd["up_scale"] = syn.quantize_rows_e4m3(sd["expert_up.weight"])
        x = syn.make_input(cfg, 0, "cpu")
        v, cores, sample, ms = cpu_reference_run(cfg, sd, x, args.index_mode, args.steps, max(args.warmup, 1),
                                                 args.cpu_sample_tokens)
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload,
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}))
        return

    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    layer, sd = make_layer(cfg, args, dev)
    x = syn.make_input(cfg, 1000 + rank, dev)
    T = cfg.tokens

    # ---- device-resident timing -------------------------------------------------
    with torch.no_grad():
        for _ in range(max(args.warmup, 3)):
            layer(x)
        layer._op.query_status()
        op = layer._op
        launches0 = op.launch_count
        op.stage_timing(True)
        sampler = ClockSampler(local) if rank == 0 else None
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(args.steps):
            layer(x)
        e1.record()
        barrier()
        ms_total = e0.elapsed_time(e1)
        launches = op.launch_count - launches0
        ms_q, ms_s, ms_g, n_slices = op.stage_times()
        op.stage_timing(False)
        op.query_status()
    t_ms = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
    ms_total = float(t_ms.item())
    value = world * T * args.steps / (ms_total / 1e3)

    # ---- end to end: pinned host x -> device -> host output, every step ----------
    e2e = None
    if not args.no_e2e:
        xh = x.cpu().pin_memory()
        outs = [torch.empty(cfg.batch, cfg.seq, cfg.output_dim, dtype=cfg.dtype, pin_memory=True) for _ in range(2)]
        outh = outs[0]
        layer.track_indices = False
        with torch.no_grad():
            for _ in range(3):
                layer.forward_host(xh, outh)
            # (1) one blocking call per step
            barrier()
            t0 = time.perf_counter()
            for _ in range(args.steps):
                layer.forward_host(xh, outh)     # returns when the output has landed on the host
            torch.cuda.synchronize()
            dt_serial = time.perf_counter() - t0
            # (2) the same work with step i+1 submitted before step i is waited for (two output buffers):
            #     every step still copies its input in and its whole output back inside the timed region
            barrier()
            t0 = time.perf_counter()
            prev = None
            for i in range(args.steps):
                _, tk = layer.forward_host_async(xh, outs[i & 1])
                if prev is not None:
                    layer.forward_host_wait(prev)
                prev = tk
            layer.forward_host_wait(prev)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
        layer.track_indices = True
        t_e = torch.tensor([dt, dt_serial], device=dev, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t_e, op=dist.ReduceOp.MAX)
        e2e = {"value": world * T * args.steps / float(t_e[0].item()), "unit": UNIT,
               "h2d_bytes_per_step": xh.numel() * xh.element_size() * world,
               "d2h_bytes_per_step": outh.numel() * outh.element_size() * world,
               "api": "PEER.forward_host_async/_wait -> peer_forward_host_async/_wait (C ABI), pinned host buffers, "
                      "one step in flight behind the one being waited for",
               "blocking_call_value": world * T * args.steps / float(t_e[1].item())}
    backward = None
    if args.backward and cfg.table_dtype != torch.float8_e4m3fn:
        backward = time_backward(layer, cfg, x, min(args.steps, 5))
    clocks = sampler.stop() if sampler is not None else None

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peak, peak_kind = hbm_peak()
    gathered = cfg.gathered_bytes_per_token() * T          # algorithmic bytes of one expert-stage launch
    g_ms = ms_g / max(n_slices, 1)
    achieved = gathered / (g_ms / 1e3) / 1e9
    roofline = {"bound": "hbm", "kernel": "gather_eval_kernel (expert stage)", "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                "traffic": (NCU_TRAFFIC_PER_ALGORITHMIC_BYTE.get(workload["table_dtype"]) or 0) * gathered or None,
                "traffic_note": "ncu capture of a smaller case of the same kernel, scaled by tokens",
                "ms_per_launch": g_ms,
                "algorithmic_bytes_per_launch": gathered,
                "stage_ms_per_step": {"query": ms_q / max(n_slices, 1), "select": ms_s / max(n_slices, 1),
                                      "experts": g_ms}}

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        sd_cpu = {k: v.cpu() for k, v in layer.state_dict().items()}
        sd_cpu["down_scale"] = sd_cpu.pop("expert_down_scale", None)
        sd_cpu["up_scale"] = sd_cpu.pop("expert_up_scale", None)
        v, cores, sample, _ = cpu_reference_run(cfg, sd_cpu, x.cpu(), args.index_mode, 3, 1, args.cpu_sample_tokens)
        cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}

    print(json.dumps({
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload,
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
        **({"backward": backward} if backward else {})}))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
