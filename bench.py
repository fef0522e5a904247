#!/usr/bin/env python
"""MoE-layer forward benchmark: tokens/s on N B200s, with roofline and CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c3]

A step is one forward of the MoE layer over one batch of seeded synthetic
tokens (x ~ N(0,1), weights ~ N(0,0.02), random init — no dataset exists for
this metric).  ``value`` is timed with CUDA events with x resident in HBM;
``e2e`` is the same forward through the host-buffer entry point
(``omoe_forward_host``: pinned x -> H2D -> forward -> D2H y -> sync).
Prints ONE JSON line on rank 0.

Options beyond the contract: ``--tokens`` (decode sweep), ``--weak`` (weak scaling), ``--graph`` (time replays of
one captured forward), ``--block`` (the RMSNorm + residual form), ``--train`` (adds the time of a training step:
training-mode forward + backward, one GPU).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # name: T, d, dff, E, k, compute dtype, zipf bias
    "c1": dict(T=64, d=128, dff=256, E=8, k=2, dtype="f32", zipf=False,
               name="tiny fp32 layer T=64 d=128 E=8 top2 dff=256"),
    "c2": dict(T=4096, d=1024, dff=2816, E=8, k=2, dtype="bf16", zipf=False,
               name="mid-size T=4096 d=1024 E=8 top2 dff=2816"),
    "c3": dict(T=16384, d=4096, dff=14336, E=8, k=2, dtype="bf16", zipf=False,
               name="Mixtral-8x7B-shaped T=16384 d=4096 E=8 top2 dff=14336"),
    "c4": dict(T=8192, d=2048, dff=1408, E=64, k=6, dtype="bf16", zipf=True,
               name="fine-grained T=8192 d=2048 E=64 top6 dff=1408 Zipf(1.1) router bias"),
    "c5": dict(T=64, d=4096, dff=14336, E=8, k=2, dtype="bf16", zipf=False,
               name="decode-shaped d=4096 E=8 top2 dff=14336"),
}
SEED = 20240611
# dram__bytes_read.sum + dram__bytes_write.sum of one up/gate launch, from the ncu capture summarised in
# profiles/grouped_gemm_ncu_full.md (full config-3 workload on one GPU); null for every other workload.
NCU_TRAFFIC_BYTES = {("c3", 16384, 1): 5917402368 + 950249216}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            j = json.load(f)
        return dict(hbm=j["hbm_gbs"], tf_burst=j["bf16_tflops"], tf_sust=j["bf16_tflops_sustained"], src="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sust=1400.0, src="fallback")


class ClockSampler:
    """nvidia-smi clock/throttle sampling during the timed region (read-only)."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.idx = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [c.strip() for c in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # samples under load are the upper half of the clock distribution's time window; report the median
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def algorithmic(cfg, T):
    """FLOPs and bytes of one forward over T tokens (no padding, no recompute)."""
    d, dff, E, k = cfg["d"], cfg["dff"], cfg["E"], cfg["k"]
    return dict(up_gate_flops=4.0 * T * k * d * dff, down_flops=2.0 * T * k * d * dff,
                router_flops=2.0 * T * d * E, total_flops=6.0 * T * k * d * dff + 2.0 * T * d * E)


def cpu_sample(cfg, n_tokens, nthreads=0, seed=SEED):
    """Times the oracle (a restatement of the reference's host path) on n_tokens
    tokens of this configuration; returns (tokens/s, seconds, cores)."""
    import numpy as np
    from oracle import ref

    d, dff, E, k = cfg["d"], cfg["dff"], cfg["E"], cfg["k"]
    rng = np.random.Generator(np.random.Philox(key=seed))
    x = rng.standard_normal((n_tokens, d), dtype=np.float32)
    w_r = (0.02 * rng.standard_normal((E, d))).astype(np.float32)
    # one expert's matrices drawn once and repeated: values do not change the work
    one = [(0.02 * rng.standard_normal((d, dff), dtype=np.float32)) for _ in range(2)]
    one.append(0.02 * rng.standard_normal((dff, d), dtype=np.float32))
    wg, wu, wd = (np.ascontiguousarray(np.broadcast_to(m, (E,) + m.shape)) for m in one)
    bias = None
    if cfg["zipf"]:
        z = (rng.permutation(E) + 1).astype(np.float64) ** -1.1
        bias = (2.0 * z / z.max()).astype(np.float32)
    cores = ref.num_threads() if nthreads <= 0 else nthreads
    t0 = time.perf_counter()
    ref.moe_forward(x, w_r, wg, wu, wd, k, bias=bias, pretransposed=True, nthreads=nthreads)
    dt = time.perf_counter() - t0
    return n_tokens / dt, dt, cores, (x, w_r, wg, wu, wd, bias)


def run_reference(args, cfg):
    """Reference arm: the reference's CPU host path (restated in oracle/, the
    reference being Java with no JVM here) on a bounded token sample per step."""
    import numpy as np
    from oracle import ref

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    d, dff, E, k = cfg["d"], cfg["dff"], cfg["E"], cfg["k"]
    # size the sample so steps+warmup finish in about two minutes
    tps, dt, cores, data = cpu_sample(cfg, 32)
    x, w_r, wg, wu, wd, bias = data
    budget = 120.0 / max(1, args.steps + args.warmup)
    n = int(max(32, min(cfg["T"], tps * budget)))
    rng = np.random.Generator(np.random.Philox(key=SEED + 1))
    xs = rng.standard_normal((n, d), dtype=np.float32)
    times = []
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        ref.moe_forward(xs, w_r, wg, wu, wd, k, bias=bias, pretransposed=True)
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
    total = sum(times)
    value = n * len(times) / total
    line = {
        "impl": "reference", "metric": "MoE-layer forward tokens/s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / len(times), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg["name"], "sample_tokens_per_step": n},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": f"{n} tokens per step of the same layer, fp32, weights pre-laid [in,out]"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_ours(args, cfg):
    import torch
    import torch.distributed as dist

    from omega_ai_b200 import MoELayer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    T, d, dff, E, k = cfg["T"], cfg["d"], cfg["dff"], cfg["E"], cfg["k"]
    if args.tokens:
        T = args.tokens
    if args.weak:
        T *= world   # weak scaling: the per-GPU share of the tokens stays that of the one-GPU run
    cdt = torch.bfloat16 if cfg["dtype"] == "bf16" else torch.float32
    peaks = load_peaks()

    # strong scaling: T is the global batch, sharded T/world per rank; experts E/world per rank
    from omega_ai_b200.ep_layout import shard_tokens
    lo, hi = shard_tokens(T, world, rank)
    T_local = hi - lo   # ranks may hold different shares when T is not a multiple of world (0 is allowed)
    El = E // world
    g = torch.Generator(device=dev).manual_seed(SEED)
    rn = lambda *s: torch.randn(*s, generator=g, device=dev, dtype=torch.float32)
    w_r = (rn(E, d) * 0.02).to(cdt)
    bias = None
    if cfg["zipf"]:
        perm = torch.randperm(E, generator=g, device=dev).float() + 1
        z = perm ** -1.1
        bias = (2.0 * z / z.max()).to(cdt)
    # every rank draws the full stream of expert weights in the same order and keeps its slice
    def expert_w(shape):
        out = torch.empty((El,) + shape, device=dev, dtype=cdt)
        for e in range(E):
            w = rn(*shape) * 0.02
            if rank * El <= e < (rank + 1) * El:
                out[e - rank * El] = w.to(cdt)
        return out
    w_g, w_u, w_d = expert_w((dff, d)), expert_w((dff, d)), expert_w((d, dff))
    gx = torch.Generator(device=dev).manual_seed(SEED + 17 + rank)
    x = torch.randn(T_local, d, generator=gx, device=dev, dtype=torch.float32).to(cdt)
    y = torch.empty_like(x)

    t_max = max(1, -(-T // world))
    layer = MoELayer(d, dff, E, k, bias=bias is not None, t_max=t_max, compute_dtype=cdt, world=world, rank=rank)
    layer.setWeights(w_r, w_g, w_u, w_d, bias)
    if world > 1:
        layer.ep_connect()
    del w_g, w_u, w_d
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.block:
        gamma = torch.ones(d, device=dev, dtype=torch.float32)
        plain_forward = layer.forward_device
        layer.forward_device = lambda xx, yy=None: layer.forward_block(xx, gamma, yy)

    # ---- device-resident timing -------------------------------------------
    for _ in range(args.warmup):
        layer.forward_device(x, y)
    barrier()
    step = lambda: layer.forward_device(x, y)
    if args.graph:
        # the forward only enqueues kernels (the expert-parallel flags and sequence number live on the device),
        # so one capture replays as many steps as wanted: what a serving loop does for launch-bound decode steps
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            layer.forward_device(x, y)
        launches_per_step = layer.launch_count()
        step = graph.replay
        for _ in range(3):
            step()
        barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop() if rank == 0 else None
    launches = (launches_per_step if args.graph else layer.launch_count()) * args.steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    value = T / (ms_per_step * 1e-3)

    # ---- per-kernel durations (CUDA events recorded by the library on the same stream) ----
    layer.set_profiling(True)
    stage_sum = None
    n_prof = min(args.steps, 10)
    for _ in range(n_prof):
        layer.forward_device(x, y)
        st = layer.stage_ms()
        stage_sum = st if stage_sum is None else {a: stage_sum[a] + st[a] for a in st}
    layer.set_profiling(False)
    stage_ms = {a: v / n_prof for a, v in stage_sum.items()}

    # ---- optional: a training step (training-mode forward + backward), one GPU ----
    train = None
    if args.train and world == 1 and not args.block:
        layer.set_training(True)
        dy = torch.randn((T_local, d), device=dev, dtype=torch.float32).to(cdt)
        dx = torch.empty_like(x)
        t_steps = max(3, min(args.steps, 10))
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        for _ in range(2):
            layer.forward_device(x, y)
            layer.backward(x, dy, dx)
        torch.cuda.synchronize()
        f_ms = b_ms = 0.0
        for _ in range(t_steps):
            evs[0].record()
            layer.forward_device(x, y)
            evs[1].record()
            layer.backward(x, dy, dx)
            evs[2].record()
            torch.cuda.synchronize()
            f_ms += evs[0].elapsed_time(evs[1])
            b_ms += evs[1].elapsed_time(evs[2])
        f_ms, b_ms = f_ms / t_steps, b_ms / t_steps
        flops = 3 * 6.0 * T_local * k * d * dff  # forward + input gradients + weight gradients of the expert products
        train = {"forward_ms": f_ms, "backward_ms": b_ms, "tokens_per_s": T / ((f_ms + b_ms) * 1e-3),
                 "expert_tflops": flops / ((f_ms + b_ms) * 1e-3) / 1e12, "backward_launches": layer.launch_count(),
                 "steps": t_steps}
        layer.set_training(False)

    # ---- end to end through the host-buffer entry point --------------------
    xh = torch.empty((T_local, d), dtype=cdt).pin_memory()
    xh.copy_(x.cpu())
    yh = torch.empty((T_local, d), dtype=cdt).pin_memory()
    e2e_steps = max(3, min(args.steps, 20))
    for _ in range(3):
        layer.forward_host(xh, yh)
    barrier()
    ev0.record()
    for _ in range(e2e_steps):
        layer.forward_host(xh, yh)
    ev1.record()
    barrier()
    e2e_ms = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = T / (e2e_ms / e2e_steps * 1e-3)
    bpe = 2 if cdt == torch.bfloat16 else 4

    # experts that received at least one token, over all ranks (every rank takes part in the reduction)
    _, _, counts_local, _, _ = layer.routing(T_local)
    counts_all = torch.from_numpy(counts_local.astype("int64")).to(dev)
    if world > 1:
        dist.all_reduce(counts_all)
    counts_all = counts_all.cpu().numpy()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    alg = algorithmic(cfg, T_local)
    decode = T <= 256 and cfg["dtype"] == "bf16"
    if decode:
        # the bound is the rank that has the most active experts (one GPU: all active experts)
        n_active = max(int((counts_all[r * El:(r + 1) * El] > 0).sum()) for r in range(world))
        wbytes = n_active * 3.0 * d * dff * 2
        dur = (stage_ms["up_gate"] + stage_ms["down"]) * 1e-3
        # which kernels ran depends on the step: the streaming kernels for one or two tokens, the split-K cluster
        # kernels while a product's tiles fit one round of resident clusters, else the persistent kernels
        roof = {"bound": "hbm", "kernel": "expert products (up/gate + down): decode_gemv / grouped_gemm_splitk / "
                                          "grouped_gemm kernels, picked per step",
                "achieved": wbytes / dur / 1e9, "peak": peaks["hbm"], "unit": "GB/s",
                "frac": wbytes / dur / 1e9 / peaks["hbm"], "traffic": None, "peak_source": peaks["src"],
                "active_experts": n_active, "weight_bytes": wbytes,
                # the same bytes over the whole step (router, dispatch, combine and launch gaps included)
                "whole_step_frac": wbytes / (ms_per_step * 1e-3) / 1e9 / peaks["hbm"]}
    elif cfg["dtype"] == "bf16":
        dur = stage_ms["up_gate"] * 1e-3
        ach = alg["up_gate_flops"] / dur / 1e12
        timed_s = ms * 1e-3
        peak = peaks["tf_sust"] if timed_s >= 1.0 else peaks["tf_burst"]
        roof = {"bound": "tensor", "kernel": "grouped_gemm_kernel<SWIGLU> (up/gate)", "achieved": ach,
                "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                "traffic": NCU_TRAFFIC_BYTES.get((args.config, T, world)),
                "algorithmic_dram_bytes": 2.0 * (2 * El * d * dff + T_local * k * (d + dff)),
                "peak_source": peaks["src"] + (" sustained" if timed_s >= 1.0 else " burst"),
                "frac_of_burst": ach / peaks["tf_burst"], "frac_of_sustained": ach / peaks["tf_sust"],
                "down_tflops": alg["down_flops"] / (stage_ms["down"] * 1e-3) / 1e12}
    else:
        dur = (stage_ms["up_gate"] + stage_ms["down"]) * 1e-3
        ach = (alg["up_gate_flops"] + alg["down_flops"]) / dur / 1e12
        roof = {"bound": "tensor", "kernel": "grouped_sgemm_kernel (fp32 CUDA cores)", "achieved": ach,
                "peak": peaks["tf_burst"], "unit": "TFLOP/s", "frac": ach / peaks["tf_burst"], "traffic": None,
                "peak_source": peaks["src"]}

    cpu = None
    if world == 1 and not args.no_cpu:
        # a bounded sample of the workload: about 12 s of CPU work at the ~150 GFLOP/s the port reaches on 16 cores
        flops_per_token = 6.0 * k * d * dff + 2.0 * d * E
        n_cpu = args.cpu_tokens or max(256, int(12.0 * 150e9 / flops_per_token) // 64 * 64)
        n_cpu = min(n_cpu, cfg["T"])
        tps, dt, cores, _ = cpu_sample(cfg, n_cpu)
        cpu = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
               "sample": f"{n_cpu} tokens of the same layer in {dt:.1f} s, fp32, weights pre-laid [in,out]"}

    working_set = 3.0 * El * d * dff * bpe + 2.0 * T_local * d * bpe
    l2_note = ("inputs larger than L2: %.0f MB of weights and rows are streamed every step" % (working_set / 1e6)
               if working_set > 126e6 else "working set fits L2; no flush (reference-sized case)")
    line = {
        "metric": "MoE-layer forward tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak" if args.weak else "strong", "vs_baseline": None, "dtype": cfg["dtype"], "data": "synthetic",
        "config": {"workload": cfg["name"] + (" + RMSNorm + residual" if args.block else ""), "tokens_global": T, "tokens_per_gpu": T_local, "experts_per_gpu": El,
                   "parallelism": f"ep{world}", "l2": l2_note,
                   "launch": "cuda graph replay" if args.graph else "direct calls"},
        "stage_ms": stage_ms,
        "layer_tflops": alg["total_flops"] / (ms_per_step * 1e-3) / 1e12,
        "roofline": roof, "cpu_baseline": cpu, "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": T_local * d * bpe,
                "d2h_bytes_per_step": T_local * d * bpe},
        "gpu_launches": launches,
    }
    if train is not None:
        line["train"] = train
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c3", choices=sorted(CONFIGS))
    ap.add_argument("--tokens", type=int, default=0, help="override the token count (decode sweep)")
    ap.add_argument("--cpu-tokens", type=int, default=0)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--weak", action="store_true",
                    help="weak scaling: the global token count is the configuration's times the number of GPUs")
    ap.add_argument("--graph", action="store_true",
                    help="time replays of one captured forward (CUDA graph) instead of direct calls")
    ap.add_argument("--train", action="store_true",
                    help="also time a training step (training-mode forward + backward) on one GPU; adds a 'train' object")
    ap.add_argument("--block", action="store_true",
                    help="time y = x + MoE(rmsnorm(x)*gamma) (omoe_forward_block) instead of the bare layer")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    cfg = dict(CONFIGS[args.config])
    if args.impl == "reference":
        run_reference(args, cfg)
    else:
        run_ours(args, cfg)


if __name__ == "__main__":
    main()
