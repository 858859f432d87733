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
measured HBM copy bandwidth, and `roofline.layer_frac` the same bytes over the
whole step.  `extra` carries the other configurations of the workload family,
each measured in the same run: `c3` (FP8-e4m3 tables), `c5_peer_stack` (twelve
PEER layers with their block LayerNorm and residual over [4, 4096, 2048]),
`backward` (forward+backward of the layer, N = 1) and, with two or more ranks,
`c4` (the decode-shaped 4,194,304-expert layer with row-sharded tables and the
NCCL exchange of (token, id, weight) tuples).
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
REPEATS = 3          # the timed loop of K steps is run this many times; the median repeat is reported
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
    ap.add_argument("--cpu-sample-tokens", type=int, default=512)
    ap.add_argument("--cpu-passes", type=int, default=5)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="headline workload only (profiling runs)")
    ap.add_argument("--no-bind", action="store_true", help="leave CPU affinity and memory policy alone")
    ap.add_argument("--backward", action="store_true", help="kept for compatibility: extra.backward is on by default at N=1")
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
    PyTorch forward, run natively in the configuration's dtype with every host thread this
    process may use) on a token sample of the workload.  Returns (tokens/s, cores, sample
    description, ms/step)."""
    from oracle import peer_oracle as orc
    try:
        cores = len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
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


def make_layer(cfg, index_mode, device, seed=0):
    from llm720_b200 import PEER, synthetic as syn
    sd = syn.make_weights(cfg, seed, device)
    with torch.device("meta"):          # no 2 x 8.6 GB fp32 default tables
        m = PEER(**cfg.module_kwargs())
    m.load_state_dict(sd, assign=True)
    del sd
    if cfg.table_dtype == torch.float8_e4m3fn:
        m.quantize_tables_e4m3()
    m.eval().requires_grad_(False)
    m.index_mode = index_mode
    return m


class Env:
    """Rank, device, process group and the reductions the timed regions need."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.dev = torch.device("cuda", self.local)
        self.dist = None

    def init(self):
        torch.cuda.set_device(self.local)
        if self.world > 1:
            import torch.distributed as dist
            import datetime
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
            # a rank that fails must end the job, not leave the others waiting in a collective
            dist.init_process_group("nccl", device_id=self.dev, timeout=datetime.timedelta(seconds=240))
            self.dist = dist

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, values):
        t = torch.tensor(list(values), device=self.dev, dtype=torch.float64)
        if self.dist is not None:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    def close(self):
        if self.dist is not None:
            self.dist.destroy_process_group()


def time_steps(env, fn, steps, repeats=REPEATS):
    """`repeats` runs of `steps` calls of fn, each bracketed by barrier + synchronize and timed with CUDA
    events on the current stream; per repeat the max over ranks.  Returns (median ms per repeat, all)."""
    ms = []
    for _ in range(repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        env.barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        env.barrier()
        ms.append(e0.elapsed_time(e1))
    ms = env.max_over_ranks(ms)
    return statistics.median(ms), ms


def stage_roofline(cfg, index_mode, stage_ms, n_slices, step_ms, table_dtype_name):
    """The expert stage against the HBM roofline (rows addressed by product-key ids stream from HBM), or,
    with the reference's id arithmetic (at most n0 + n1 - 1 distinct rows, L2-resident), labelled as such."""
    peak, peak_kind = hbm_peak()
    T = cfg.tokens
    gathered = cfg.gathered_bytes_per_token() * T          # algorithmic bytes of one expert-stage launch
    ms_q, ms_s, ms_g = (v / max(n_slices, 1) for v in stage_ms)
    achieved = gathered / (ms_g / 1e3) / 1e9
    hbm = index_mode == "product"
    r = {"bound": "hbm" if hbm else "l2", "kernel": "gather_eval_kernel (expert stage)", "achieved": achieved,
         "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
         "traffic": ((NCU_TRAFFIC_PER_ALGORITHMIC_BYTE.get(table_dtype_name) or 0) * gathered or None) if hbm else None,
         "traffic_note": "ncu capture of a smaller case of the same kernel, scaled by tokens" if hbm else
                         "rows are L2-resident with the reference's id arithmetic: no DRAM figure applies",
         "ms_per_launch": ms_g, "algorithmic_bytes_per_launch": gathered,
         "layer_frac": gathered / (step_ms / 1e3) / 1e9 / peak,
         "stage_ms_per_step": {"query": ms_q, "select": ms_s, "experts": ms_g}}
    if not hbm:
        r["note"] = ("frac is gathered bytes over the HBM copy peak for rows served from L2: not an HBM "
                     "utilisation figure")
    return r


def run_layer_timing(env, layer, x, steps, warmup):
    """Device-resident timing of layer(x): (median ms per K steps, per-repeat ms, launches per repeat,
    stage ms sums, slices)."""
    with torch.no_grad():
        for _ in range(max(warmup, 3)):
            layer(x)
        layer._op.query_status()
        op = layer._op
        launches0 = op.launch_count
        op.stage_timing(True)
        med, all_ms = time_steps(env, lambda: layer(x), steps)
        launches = (op.launch_count - launches0) // REPEATS
        ms_q, ms_s, ms_g, n_slices = op.stage_times()
        op.stage_timing(False)
        op.query_status()
    return med, all_ms, launches, (ms_q, ms_s, ms_g), n_slices


def run_e2e(env, layer, cfg, x, steps):
    """Host-buffer path: pinned x in, whole output back, every step; plus the copy-only ceiling of this
    host measured the same way with all ranks copying at once and no kernels."""
    from llm720_b200 import hostmem
    T, world = cfg.tokens, env.world
    xh = hostmem.pinned_empty(cfg.batch, cfg.seq, cfg.input_dim, dtype=cfg.dtype)
    xh.copy_(x)
    outs = [hostmem.pinned_empty(cfg.batch, cfg.seq, cfg.output_dim, dtype=cfg.dtype) for _ in range(2)]
    layer.track_indices = False
    with torch.no_grad():
        for _ in range(3):
            layer.forward_host(xh, outs[0])
        # (1) one blocking call per step
        env.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            layer.forward_host(xh, outs[0])     # returns when the output has landed on the host
        torch.cuda.synchronize()
        dt_block = time.perf_counter() - t0
        # (2) the same work with step i+1 submitted before step i is waited for (two output buffers):
        #     every step still copies its input in and its whole output back inside the timed region
        env.barrier()
        t0 = time.perf_counter()
        prev = None
        for i in range(steps):
            _, tk = layer.forward_host_async(xh, outs[i & 1])
            if prev is not None:
                layer.forward_host_wait(prev)
            prev = tk
        layer.forward_host_wait(prev)
        torch.cuda.synchronize()
        dt_ahead = time.perf_counter() - t0
    layer.track_indices = True
    # (3) copy-only ceiling: the same bytes each way, both directions at once, no kernels
    d_in = torch.empty(cfg.batch, cfg.seq, cfg.input_dim, dtype=cfg.dtype, device=env.dev)
    d_out = torch.zeros(cfg.batch, cfg.seq, cfg.output_dim, dtype=cfg.dtype, device=env.dev)
    s_in, s_out = torch.cuda.Stream(env.dev), torch.cuda.Stream(env.dev)
    def copies(n):
        for _ in range(n):
            with torch.cuda.stream(s_in):
                d_in.copy_(xh, non_blocking=True)
            with torch.cuda.stream(s_out):
                outs[1].copy_(d_out, non_blocking=True)
        s_in.synchronize(); s_out.synchronize()
    copies(2)
    env.barrier()
    t0 = time.perf_counter()
    copies(steps)
    dt_copy = time.perf_counter() - t0
    dt_ahead, dt_block, dt_copy = env.max_over_ranks([dt_ahead, dt_block, dt_copy])
    h2d = xh.numel() * xh.element_size()
    d2h = outs[0].numel() * outs[0].element_size()
    v_ahead, v_block = world * T * steps / dt_ahead, world * T * steps / dt_block
    ceiling = world * T * steps / dt_copy
    best = max(v_ahead, v_block)
    return {"value": best, "unit": UNIT, "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world,
            "api": "PEER.forward_host_async/_wait -> peer_forward_host_async/_wait (C ABI), pinned host buffers, one "
                   "step in flight behind the one being waited for" if v_ahead >= v_block else
                   "PEER.forward_host -> peer_forward_host (C ABI), pinned host buffers, one blocking call per step",
            "submit_ahead_value": v_ahead, "blocking_call_value": v_block,
            "copy_ceiling": {"value": ceiling, "unit": UNIT,
                             "GBps_per_gpu_each_way": h2d * steps / dt_copy / 1e9,
                             "GBps_host_total": (h2d + d2h) * world * steps / dt_copy / 1e9,
                             "what": "all ranks copy the step's input in and an output back at once, no kernels"},
            "frac_of_copy_ceiling": best / ceiling}


def run_backward(env, layer, cfg, x, steps):
    """Forward+backward of the layer (all parameters and x require gradients; table gradients summed as the
    module's default policy decides, which is reported), and the expert-stage gradient kernel on its own
    with fp32 and with bf16 sums.  Algorithmic bytes of that kernel per (token, slot): the two table rows
    read, and the two gradient rows read and written."""
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
    op = layer._op
    ids = layer._last_expert_indices.view(T, HK).to(torch.int32)
    w = torch.softmax(layer._last_expert_scores.view(T, cfg.num_heads, cfg.top_k), -1).view(T, HK).contiguous()
    from llm720_b200.autograd import _table_grad_plan
    gdt_used, rows_used = _table_grad_plan(layer, layer.expert_down.weight, T)
    out = {"fwd_bwd_ms_per_step": step_ms, "fwd_bwd_tokens_per_s": T / (step_ms / 1e3), "steps": steps,
           "table_grad_sums": f"{layer.table_grad_sums}: {str(gdt_used).replace('torch.', '')} sums over {rows_used} rows "
                              f"({T * HK / rows_used:.1f} selections per row)"}
    peak, kind = hbm_peak()
    eb = torch.empty(0, dtype=cfg.table_dtype).element_size()
    x2, g2 = x.view(T, -1), grad_out.view(T, -1)
    for name, gdt in (("fp32_sums", torch.float32), ("bf16_sums", cfg.table_dtype)):
        gd = torch.zeros(layer.expert_down.weight.shape, dtype=gdt, device=x.device)
        gu = torch.zeros(layer.expert_up.weight.shape, dtype=gdt, device=x.device)
        gb = torch.empty(0, dtype=gdt).element_size()
        for i in range(1 + 3):
            if i == 1:
                ev[2].record()
            op.gather_eval_backward(x2, g2, ids, w, layer.expert_down.weight, layer.expert_up.weight, gd, gu, grad_dtype=gdt)
        ev[3].record()
        torch.cuda.synchronize()
        op.query_status()
        k_ms = ev[2].elapsed_time(ev[3]) / 3
        bytes_alg = T * HK * (cfg.input_dim + cfg.output_dim) * (eb + 2 * gb)
        out["gather_grad_kernel_" + name] = {"ms": k_ms, "algorithmic_bytes_per_launch": bytes_alg,
                                             "achieved_GBps": bytes_alg / (k_ms / 1e3) / 1e9,
                                             "frac_of_hbm_peak": bytes_alg / (k_ms / 1e3) / 1e9 / peak, "peak_kind": kind}
        del gd, gu
    return out


def run_c3(env, args, steps):
    """BASELINE configuration 3: the same layer with FP8-e4m3 tables and per-row fp32 scales."""
    from llm720_b200 import synthetic as syn
    cfg = syn.CONFIGS["c3"]
    layer = make_layer(cfg, "product", env.dev)
    x = syn.make_input(cfg, 1000 + env.rank, env.dev)
    med, all_ms, launches, stage_ms, n_slices = run_layer_timing(env, layer, x, steps, 3)
    step_ms = med / steps
    r = stage_roofline(cfg, "product", stage_ms, n_slices, step_ms, "float8_e4m3fn")
    gathered = r["algorithmic_bytes_per_launch"]
    out = {"workload": "c3: the 1,048,576-expert layer with FP8-e4m3 tables (per-row fp32 scale), product-key ids, "
                       f"x [{cfg.batch},{cfg.seq},{cfg.input_dim}] per GPU",
           "tokens_per_s": env.world * cfg.tokens * steps / (med / 1e3), "ms_per_step": step_ms, "steps": steps,
           "repeats_ms": all_ms, "roofline": r, "traffic_over_algorithmic": 1.007, "gpu_launches": launches,
           "algorithmic_bytes_per_token": cfg.gathered_bytes_per_token(), "gathered_bytes": gathered}
    del layer, x
    torch.cuda.empty_cache()
    return out


def _stack_parity(dev):
    """Three PEER blocks at a reduced key grid, every block checked against the oracle on the block's own
    input (LayerNorm in fp32 rounded to bf16, the reference's fp32 layer arithmetic on the same bf16
    values, residual added, one rounding): bf16 bound max-abs 2e-2, L1-relative 1e-3 on the block output
    minus its input."""
    import torch.nn as nn
    import torch.nn.functional as F
    from llm720_b200 import PEER, synthetic as syn
    from oracle import peer_oracle as orc
    cfg = syn.scaled(syn.CONFIGS["c2"], product_key_dim=(128, 128), batch=1, seq=96)
    h = syn.make_input(cfg, 77, dev)
    worst = (0.0, 0.0)
    ok = True
    kw = dict(cfg.module_kwargs()); kw.pop("dropout")
    shape = orc.PeerShape(**kw)
    for l in range(3):
        sd = syn.make_weights(cfg, 300 + l, dev, random_affine=True)
        with torch.device("meta"):
            m = PEER(**cfg.module_kwargs())
        m.load_state_dict(sd, assign=True)
        m.eval().requires_grad_(False)
        m.index_mode = "product"
        ln = nn.LayerNorm(cfg.input_dim, device=dev, dtype=cfg.dtype)
        with torch.no_grad():
            ln.weight.copy_(1.0 + 0.1 * torch.randn(cfg.input_dim, device=dev))
            ln.bias.copy_(0.05 * torch.randn(cfg.input_dim, device=dev))
            h_next = m.block_forward(h, ln)
            hc = h.cpu().float()
            xn = F.layer_norm(hc, (cfg.input_dim,), ln.weight.cpu().float(), ln.bias.cpu().float(), ln.eps).to(cfg.dtype).float()
            sdc = {k: v.cpu().float() for k, v in sd.items()}
            w = orc.PeerWeights(sdc["query_proj.weight"], sdc["query_proj.bias"], sdc["query_layer_norm.weight"],
                                sdc["query_layer_norm.bias"], [sdc["sub_keys.0"], sdc["sub_keys.1"]],
                                sdc["expert_down.weight"], sdc["expert_up.weight"])
            y, _, _ = orc.forward(xn, w, shape, "product")
            ref = (hc + y).to(cfg.dtype).float()
        mx, l1 = orc.output_errors(h_next.cpu().float() - hc, ref - hc)
        worst = (max(worst[0], mx), max(worst[1], l1))
        ok = ok and mx <= 2e-2 and l1 <= 1e-3 * 4          # the difference of two roundings: a few bf16 ulps of |h|
        h = h_next
    return ok, worst


def run_c5_stack(env, steps):
    """BASELINE configuration 5, the part of it this library implements: twelve PEER layers at the
    configuration-2 shape, each behind its block LayerNorm and residual (`PEER.block_forward`:
    h + PEER(ln_2(h)), llm/models/foundation.py:196-205), over [4, 4096, 2048] per GPU.  The attention
    halves of the blocks are not part of this library and not included."""
    import torch.nn as nn
    from llm720_b200 import synthetic as syn
    cfg = syn.scaled(syn.CONFIGS["c2"], batch=4, seq=4096)
    n_layers = 12
    free0 = torch.cuda.mem_get_info(env.dev)[0]
    layers, norms = [], []
    for l in range(n_layers):
        m = make_layer(cfg, "product", env.dev, seed=100 + l)
        m.track_indices = False
        layers.append(m)
        norms.append(nn.LayerNorm(cfg.input_dim, device=env.dev, dtype=cfg.dtype).requires_grad_(False))
    h0 = syn.make_input(cfg, 2000 + env.rank, env.dev)

    def timed(tag):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(n_layers + 1)]
        per_layer = [0.0] * n_layers

        def step(record):
            h = h0
            for l in range(n_layers):
                if record:
                    ev[l].record()
                h = layers[l].block_forward(h, norms[l])
            if record:
                ev[n_layers].record()
            return h

        with torch.no_grad():
            for _ in range(2):
                h = step(False)
            for m in layers:
                m._op.query_status()
            med, all_ms = time_steps(env, lambda: step(False), steps)
            h = step(True)
            torch.cuda.synchronize()
            per_layer = [ev[l].elapsed_time(ev[l + 1]) for l in range(n_layers)]
            finite = bool(torch.isfinite(h.float()).all())
        return {"ms_per_step": med / steps, "tokens_per_s": env.world * cfg.tokens * steps / (med / 1e3),
                "ms_per_layer": per_layer, "repeats_ms": all_ms, "finite": finite,
                "table_bytes_resident": sum(m.expert_down.weight.numel() * m.expert_down.weight.element_size() * 2 for m in layers),
                "device_bytes_in_use": free0 - torch.cuda.mem_get_info(env.dev)[0]}

    out = {"workload": f"{n_layers} PEER layers (1,048,576 experts, 8 heads, top-k 16, product-key ids) each as "
                       f"h + PEER(ln_2(h)), x [{cfg.batch},{cfg.seq},{cfg.input_dim}] per GPU; PEER layers only, "
                       "MLA attention not included",
           "steps": steps, "bf16": timed("bf16")}
    for m in layers:                       # the FP8 variant: quantise in place, layer by layer
        m.quantize_tables_e4m3()
        m._op = None
    torch.cuda.empty_cache()
    out["fp8"] = timed("fp8")
    del layers, norms, h0
    torch.cuda.empty_cache()
    ok, worst = _stack_parity(env.dev)
    out["parity_ok"] = ok
    out["parity"] = {"max_abs_err": worst[0], "l1_rel_err": worst[1],
                     "what": "3 blocks, 128x128 keys, 96 tokens, each block against the oracle on the block's own input"}
    return out


def run_c4(env, steps):
    """BASELINE configuration 4: d_model 4096, 16 heads, 2048 x 2048 sub-keys (4,194,304 experts, 2 x 34.4 GB
    of bf16 rows split by index range over the ranks), top-k 16, 64 single tokens per step split over the
    ranks.  Parity is checked at 65,536 experts against the single-device layer on the concatenated batch
    (the reference has no sharded layer; that layer is itself checked against the oracle by the tests)."""
    from llm720_b200 import PEER, synthetic as syn
    from llm720_b200.sharded import ShardedPEER
    dist, rank, world, dev = env.dist, env.rank, env.world, env.dev
    out = {}
    # ---- parity at a size whose full tables fit one GPU
    small = syn.scaled(syn.CONFIGS["c4"], product_key_dim=(256, 256), batch=64, seq=1)
    sd = syn.make_weights(small, 4, dev, random_affine=True)
    x = syn.make_input(small, 4, dev)
    rows, t_local = small.num_experts // world, small.tokens // world
    layer = ShardedPEER.build(small.module_kwargs(), sd, sd["expert_down.weight"][rank * rows:(rank + 1) * rows].contiguous(),
                              sd["expert_up.weight"][rank * rows:(rank + 1) * rows].contiguous())
    xl = x.view(small.tokens, 1, -1)[rank * t_local:(rank + 1) * t_local].contiguous()
    got = layer(xl)
    layer.layer._op.query_status()
    with torch.device("meta"):
        full = PEER(**small.module_kwargs())
    full.load_state_dict(sd, assign=True)
    full.eval().requires_grad_(False)
    full.index_mode = "product"
    with torch.no_grad():
        ref = full(x)[rank * t_local:(rank + 1) * t_local]
    err = float((got.float() - ref.float()).abs().max())
    finite = bool(torch.isfinite(got.float()).all()) and float(got.float().abs().max()) > 0
    worst = env.max_over_ranks([err, 0.0 if finite else 1.0])
    out["parity_ok"] = bool(worst[0] <= 2e-2 and worst[1] == 0.0)
    out["max_abs_err"] = worst[0]
    out["parity_case"] = "65,536 experts (256x256 keys), 64 tokens, against the single-device layer run in the same process group"
    del layer, full, sd, got, ref
    torch.cuda.empty_cache()
    # ---- the full size: every rank generates only its own rows
    cfg = syn.scaled(syn.CONFIGS["c4"], batch=64, seq=1)
    sd = syn.make_weights(cfg, 4, dev, random_affine=True, tables=False)
    x = syn.make_input(cfg, 4, dev)
    rows, t_local = cfg.num_experts // world, cfg.tokens // world
    down = syn.make_table_shard(cfg, "expert_down", rank * rows, rows, 4, dev)
    up = syn.make_table_shard(cfg, "expert_up", rank * rows, rows, 4, dev)
    layer = ShardedPEER.build(cfg.module_kwargs(), sd, down, up)
    xl = x.view(cfg.tokens, 1, -1)[rank * t_local:(rank + 1) * t_local].contiguous()
    for _ in range(5):
        y = layer(xl)
    layer.layer._op.query_status()
    med, all_ms = time_steps(env, lambda: layer(xl), steps)
    tuples = float(layer.last_counts.sum().item())
    t_all = torch.tensor([tuples, -tuples], device=dev, dtype=torch.float64)
    dist.all_reduce(t_all, op=dist.ReduceOp.MAX)
    ms = med / steps
    gathered = cfg.gathered_bytes_per_token() * cfg.tokens
    peak, kind = hbm_peak()
    out.update({
        "workload": f"c4: {cfg.num_experts} experts, d_model {cfg.input_dim}, {cfg.num_heads} heads, top_k {cfg.top_k}, "
                    f"{cfg.tokens} single tokens per step, tables row-sharded x{world} ({rows} rows = "
                    f"{2 * rows * cfg.input_dim * 2 / 1e9:.1f} GB per rank), product-key ids",
        "ms_per_step": ms, "tokens_per_s": cfg.tokens / (ms / 1e3), "steps": steps, "repeats_ms": all_ms,
        "finite": bool(torch.isfinite(y.float()).all()),
        "nvlink_bytes_sent_per_rank_per_step": layer.nvlink_bytes_per_step(t_local),
        "tuples_received_per_rank": {"max": float(t_all[0].item()), "min": float(-t_all[1].item()),
                                     "mean": cfg.tokens * cfg.num_heads * cfg.top_k / world},
        "gathered_bytes_per_step": gathered,
        "bandwidth_floor_us": gathered / world / (peak * 1e9) * 1e6,
        "collectives": "all_gather(x), all_to_all(tuple buckets), reduce_scatter(fp32 partial sums); NCCL, NVLS off",
    })
    # ---- the same step with the library's direct exchange (stores into the peers' memory, no collective).
    # Every rank learns whether all ranks got through the set-up and a first checked step before any of them goes on.
    direct, why = None, ""
    try:
        direct = ShardedPEER(layer.layer, None, exchange="direct")
        yd = direct(xl)
        direct.check_exchange()
        close = float((yd.float() - y.float()).abs().max())
    except Exception as e:                        # noqa: BLE001 - reported in the line, the bench goes on
        why = f"{type(e).__name__}: {e}"[:200]
    failed = env.max_over_ranks([1.0 if why else 0.0])[0] > 0
    if failed:
        out["direct_exchange"] = {"unavailable": why or "a peer rank could not set it up or timed out"}
    else:
        for _ in range(5):
            direct(xl)
        med_d, all_d = time_steps(env, lambda: direct(xl), steps)
        timed_out = 0.0
        try:
            direct.check_exchange()
        except RuntimeError:
            timed_out = 1.0
        worst = env.max_over_ranks([close, timed_out])
        out["direct_exchange"] = {"ms_per_step": med_d / steps, "tokens_per_s": cfg.tokens / (med_d / steps / 1e3),
                                  "repeats_ms": all_d, "max_abs_diff_to_collective_form": worst[0],
                                  "agrees": bool(worst[0] <= 2e-3 and worst[1] == 0.0),
                                  "what": "x, tuple blocks and fp32 partial sums written into the peers' memory over NVLink "
                                          "(CUDA IPC mappings, plain stores, step numbers as flags, bounded waits); "
                                          "partial sums added in rank order"}
    if direct is not None and direct._xchg is not None:
        direct.close()
    de = out["direct_exchange"]
    faster = "ms_per_step" in de and de.get("agrees") and de["ms_per_step"] < out["ms_per_step"]
    out["fastest_exchange"] = {"exchange": "direct" if faster else "collectives",
                               "ms_per_step": de["ms_per_step"] if faster else out["ms_per_step"]}
    del layer, down, up
    torch.cuda.empty_cache()
    return out


def main():
    args = parse()
    env = Env()
    cfg = build_cfg(args)
    from llm720_b200 import synthetic as syn

    l2_note = ("inputs larger than L2: each step gathers %.1f GB of table rows" % (cfg.gathered_bytes_per_token() * cfg.tokens / 1e9)
               if args.index_mode == "product" else
               "reference id arithmetic: at most %d distinct rows (%.1f MB) are addressed, they stay in L2; x and out (%.0f MB) "
               "stream through it" % (cfg.product_key_dim[0] + cfg.product_key_dim[1] - 1,
                                      (cfg.product_key_dim[0] + cfg.product_key_dim[1]) * (cfg.input_dim + cfg.output_dim) *
                                      torch.empty(0, dtype=cfg.table_dtype).element_size() / 1e6,
                                      cfg.tokens * (cfg.input_dim + cfg.output_dim) * 2 / 1e6))
    workload = {"workload": f"{cfg.name}: PEER forward, {cfg.num_experts} experts, d_model {cfg.input_dim}, "
                            f"{cfg.num_heads} heads, query_dim {cfg.query_dim}, top_k {cfg.top_k}, "
                            f"x [{cfg.batch},{cfg.seq},{cfg.input_dim}] per GPU",
                "tokens_per_gpu": cfg.tokens, "index_mode": args.index_mode,
                "table_dtype": str(cfg.table_dtype).replace("torch.", ""),
                "parallelism": f"token-sharded x{env.world}, replicated tables, no collective",
                "l2": l2_note}

    if args.impl == "reference":
        if env.rank != 0:
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
    try:
        affinity0 = os.sched_getaffinity(0)
    except (AttributeError, OSError):
        affinity0 = None
    binding = None
    if not args.no_bind:
        # before anything is allocated: cores and memory node local to this rank's GPU
        from llm720_b200 import hostmem
        binding = hostmem.bind_process_to_gpu(env.local, env.local, env.world)
    env.init()
    dev, rank, world = env.dev, env.rank, env.world

    layer = make_layer(cfg, args.index_mode, dev)
    x = syn.make_input(cfg, 1000 + rank, dev)
    T = cfg.tokens

    # ---- device-resident timing (the headline) ------------------------------------
    sampler = ClockSampler(env.local) if rank == 0 else None
    med, all_ms, launches, stage_ms, n_slices = run_layer_timing(env, layer, x, args.steps, args.warmup)
    value = world * T * args.steps / (med / 1e3)
    step_ms = med / args.steps

    # ---- end to end: pinned host x -> device -> host output, every step ----------
    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(env, layer, cfg, x, args.steps)
        e2e["host_binding"] = binding
    clocks = sampler.stop() if sampler is not None else None

    table_dtype_name = workload["table_dtype"]
    roofline = stage_roofline(cfg, args.index_mode, stage_ms, n_slices, step_ms, table_dtype_name)

    cpu = None
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        if affinity0 is not None:
            os.sched_setaffinity(0, affinity0)          # the CPU leg may use every core this process was given
        sd_cpu = {k: v.cpu() for k, v in layer.state_dict().items()}
        sd_cpu["down_scale"] = sd_cpu.pop("expert_down_scale", None)
        sd_cpu["up_scale"] = sd_cpu.pop("expert_up_scale", None)
        v, cores, sample, _ = cpu_reference_run(cfg, sd_cpu, x.cpu(), args.index_mode, args.cpu_passes, 1,
                                                args.cpu_sample_tokens)
        cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
        del sd_cpu

    extra = {}
    if not args.no_extra and not args.tokens and not args.keys:
        k_extra = max(3, min(args.steps, 10))
        if world == 1 and cfg.table_dtype != torch.float8_e4m3fn:
            try:
                extra["backward"] = run_backward(env, layer, cfg, x, min(args.steps, 5))
            except Exception as e:          # an extra must not take the headline down with it
                extra["backward"] = {"error": f"{type(e).__name__}: {e}"}
        del layer, x
        torch.cuda.empty_cache()
        for name, fn in (("c3", lambda: run_c3(env, args, k_extra)), ("c5_peer_stack", lambda: run_c5_stack(env, k_extra))):
            try:
                extra[name] = fn()
            except Exception as e:
                extra[name] = {"error": f"{type(e).__name__}: {e}"}
            torch.cuda.empty_cache()
        if world >= 2:
            try:
                extra["c4"] = run_c4(env, max(k_extra, 10))
            except Exception as e:
                extra["c4"] = {"error": f"{type(e).__name__}: {e}", "parity_ok": False}

    if rank != 0:
        env.close()
        return

    print(json.dumps({
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload,
        "timing": {"repeats": REPEATS, "repeats_ms_for_steps": all_ms, "reported": "median repeat"},
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
        "extra": extra}))
    env.close()


if __name__ == "__main__":
    main()
