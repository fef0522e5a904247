#!/usr/bin/env python
"""MoE-layer forward benchmark: tokens/s on N B200s, with roofline, parity record and CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c3]

A step is one forward of the MoE layer over one batch of seeded synthetic
tokens (x ~ N(0,1), weights ~ N(0,0.02), random init — no dataset exists for
this metric).  ``value`` is timed with CUDA events with x resident in HBM;
``e2e`` is the same forward through the host-buffer entry point
(pinned x -> H2D -> forward -> D2H y, every step, inside the timed region).
Prints ONE JSON line on rank 0.

What the line carries beyond the contract:
  * the K-step timed region is repeated (``--repeats``, default 7); ``ms_per_step`` is the median region and
    ``spread`` lists every region with the SM clock sampled during it;
  * ``stage_ms`` comes from CUDA events the library records INSIDE those timed regions (no synchronisation
    between steps), so the stages add up to the step and the roofline fraction describes the same clock state;
  * ``parity``: checksums of the bit patterns of y and of the routing indices in global token order, reduced
    over the ranks (the rows are drawn from the global token index, so every GPU count must print the same
    sums), and ``oracle_ok``: rank 0 checks a few of its tokens against the CPU oracle;
  * ``decode``: the small-token sweep (T = 1, 2, 8, 64, 256 on one GPU; T = 64 expert-parallel) on the same
    weights, against the HBM roofline; ``extras``: the mid-size and the 64-expert configurations.

Options beyond the contract: ``--tokens`` (override T), ``--weak`` (weak scaling), ``--graph`` (time replays of
one captured forward), ``--block`` (the RMSNorm + residual form), ``--train`` (adds the time of a training step),
``--no-decode`` / ``--no-extras`` / ``--no-cpu`` / ``--no-oracle`` (skip those legs).
"""
from __future__ import annotations

import argparse
import datetime
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
X_BLOCK = 2048  # rows of x are drawn in blocks of this many tokens of the GLOBAL batch, one seed per block
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


def host_cores() -> int:
    """Cores this process may run on (what the launcher's OMP_NUM_THREADS says is ignored on purpose)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


class ClockSampler:
    """nvidia-smi clock/throttle sampling while the timed regions run (read-only).  Every sample carries
    nvidia-smi's own timestamp, so samples can be assigned to the region they fell into."""

    Q = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.idx = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self, windows=()):
        """windows: (t0, t1) pairs of time.time() stamps; returns the summary over all samples taken inside any
        window (all samples when none is given) and the median SM clock per window."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}, []
        time.sleep(0.12)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        samples = []  # (unix time or None, sm, max, reasons)
        for line in out.strip().splitlines():
            f = [c.strip() for c in line.split(",")]
            if len(f) < 10:
                continue
            try:
                sm, mx = float(f[2]), float(f[3])
            except ValueError:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
            except ValueError:
                ts = None
            rs = {name for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                           "sw_power_cap"), f[6:10]) if v.lower().startswith("active")}
            samples.append((ts, sm, mx, rs))
        if not samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}, []
        inside = lambda ts, w: ts is not None and w[0] - 0.03 <= ts <= w[1] + 0.03
        per_window = []
        for w in windows:
            v = [s[1] for s in samples if inside(s[0], w)]
            per_window.append(statistics.median(v) if v else None)
        used = [s for s in samples if any(inside(s[0], w) for w in windows)] if windows else samples
        if not used:
            used = samples
        reasons = set()
        for s in used:
            reasons |= s[3]
        return {"sm_mhz": statistics.median(s[1] for s in used), "sm_max_mhz": max(s[2] for s in used),
                "reasons": sorted(reasons), "samples": len(used)}, per_window


def algorithmic(cfg, T):
    """FLOPs of one forward over T tokens (no padding, no recompute)."""
    d, dff, E, k = cfg["d"], cfg["dff"], cfg["E"], cfg["k"]
    return dict(up_gate_flops=4.0 * T * k * d * dff, down_flops=2.0 * T * k * d * dff,
                router_flops=2.0 * T * d * E, total_flops=6.0 * T * k * d * dff + 2.0 * T * d * E)


def cpu_sample(cfg, n_tokens, nthreads=0, seed=SEED):
    """Times the oracle (a restatement of the reference's host path) on n_tokens
    tokens of this configuration; returns (tokens/s, seconds, cores, data)."""
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
    cores = nthreads if nthreads > 0 else host_cores()
    t0 = time.perf_counter()
    ref.moe_forward(x, w_r, wg, wu, wd, k, bias=bias, pretransposed=True, nthreads=cores)
    dt = time.perf_counter() - t0
    return n_tokens / dt, dt, cores, (x, w_r, wg, wu, wd, bias)


def reference_gpu_kernels(cfg, steps=3, warmup=1):
    """The reference's own GPU path for the expert stage on this GPU (its CUDA kernels compiled from its source
    files, cuBLAS SGEMM, fp32, null stream, the Java wrappers' launch shapes; driven from C++ because no JVM
    exists here).  Routing, permutation and combine have no reference kernel and are outside the timed region."""
    try:
        import torch

        from oracle import refk
        if not torch.cuda.is_available():
            return {"unavailable": "no GPU visible to the reference arm"}
        if not refk.available():
            return {"unavailable": "oracle/_ref cubins or librefk.so not built (needs the reference checkout at build time)"}
        local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local_rank)
        T, d, dff, E, k = cfg["T"], cfg["d"], cfg["dff"], cfg["E"], cfg["k"]
        rows = T * k // E
        g = torch.Generator(device="cuda").manual_seed(SEED)
        mk = lambda *s: torch.randn(*s, device="cuda", generator=g) * 0.02
        w1, w3, w2 = mk(E, dff, d), mk(E, dff, d), mk(E, d, dff)
        xp = torch.randn(E, rows, d, device="cuda", generator=g)
        yp = torch.empty(E, rows, d, device="cuda")
        scratch = refk.MlpScratch(rows, dff)
        refk.lib()

        def step():
            for e in range(E):
                refk.mlp(xp[e], w1[e], w3[e], w2[e], scratch, yp[e])

        for _ in range(warmup):
            step()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            step()
        t1.record()
        torch.cuda.synchronize()
        ms = t0.elapsed_time(t1) / steps
        return {"ms": ms, "tokens_per_s": T / (ms * 1e-3), "tflops": 6.0 * T * k * d * dff / (ms * 1e-3) / 1e12,
                "scope": "expert stage only (cublasSgemm x3 + silu_forward + mul_kernel per expert), fp32, one GPU, "
                         "rows pre-grouped; routing/dispatch/combine have no reference kernel", "steps": steps}
    except Exception as e:  # a reported extra: never let it take the reference line down
        return {"unavailable": f"{type(e).__name__}: {e}"[:200]}


def run_reference(args, cfg):
    """Reference arm: the reference's CPU host path (restated in oracle/, the
    reference being Java with no JVM here) on a bounded token sample per step,
    on all host cores whatever the launcher set OMP_NUM_THREADS to."""
    import numpy as np
    from oracle import ref

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    d, dff, E, k = cfg["d"], cfg["dff"], cfg["E"], cfg["k"]
    cores = host_cores()
    # size the sample so steps+warmup finish in about two minutes
    tps, dt, cores, data = cpu_sample(cfg, 32, nthreads=cores)
    x, w_r, wg, wu, wd, bias = data
    budget = 120.0 / max(1, args.steps + args.warmup)
    n = int(max(32, min(cfg["T"], tps * budget)))
    rng = np.random.Generator(np.random.Philox(key=SEED + 1))
    xs = rng.standard_normal((n, d), dtype=np.float32)
    times = []
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        ref.moe_forward(xs, w_r, wg, wu, wd, k, bias=bias, pretransposed=True, nthreads=cores)
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
    total = sum(times)
    value = n * len(times) / total
    line = {
        "impl": "reference", "metric": "MoE-layer forward tokens/s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / len(times), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg["name"], "sample_tokens_per_step": n, "cores": cores},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": f"{n} tokens per step of the same layer, fp32, weights pre-laid [in,out]"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "reference_gpu_kernels": None if args.no_refk else reference_gpu_kernels(cfg),
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------------------
def global_rows(torch, dev, lo, hi, d, cdt, seed):
    """Rows [lo, hi) of the GLOBAL batch: block b of X_BLOCK tokens is drawn from its own seed, so a token's row
    is the same however many GPUs share the batch."""
    out = torch.empty((hi - lo, d), device=dev, dtype=cdt)
    b = lo // X_BLOCK
    while b * X_BLOCK < hi:
        g = torch.Generator(device=dev).manual_seed(seed + 17 + b)
        blk = torch.randn(X_BLOCK, d, generator=g, device=dev, dtype=torch.float32)
        s0, s1 = max(lo, b * X_BLOCK), min(hi, (b + 1) * X_BLOCK)
        out[s0 - lo:s1 - lo] = blk[s0 - b * X_BLOCK:s1 - b * X_BLOCK].to(cdt)
        b += 1
    return out


def bits_checksum(torch, t, first_flat_index):
    """Sum over the elements of (bit pattern) * (16-bit weight from the element's GLOBAL flat index): an int64
    that does not depend on how the elements are split over ranks (no term exceeds 2^32, no overflow)."""
    total = 0
    flat = t.reshape(-1)
    n = flat.numel()
    step = 1 << 24
    for s0 in range(0, n, step):
        part = flat[s0:s0 + step]
        if part.dtype == torch.bfloat16:
            bits = part.view(torch.int16).to(torch.int64) & 0xFFFF
        elif part.dtype == torch.float32:
            bits = part.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
            bits = (bits ^ (bits >> 16)) & 0xFFFF
        else:
            bits = part.to(torch.int64) & 0xFFFF
        gi = torch.arange(first_flat_index + s0, first_flat_index + s0 + part.numel(), device=t.device,
                          dtype=torch.int64)
        w = (((gi * 2654435761) ^ (gi >> 11)) & 0xFFFF) | 1
        total += int((bits * w).sum().item())
    return total


def make_weights(torch, dev, cfg, cdt, world, rank, seed, keep_host=False):
    """Every rank draws the full stream of weights in the same order and keeps its experts' slice."""
    d, dff, E = cfg["d"], cfg["dff"], cfg["E"]
    El = E // world
    g = torch.Generator(device=dev).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, device=dev, dtype=torch.float32)
    w_r = (rn(E, d) * 0.02).to(cdt)
    bias = None
    if cfg["zipf"]:
        perm = torch.randperm(E, generator=g, device=dev).float() + 1
        z = perm ** -1.1
        bias = (2.0 * z / z.max()).to(cdt)
    host = {} if keep_host else None

    def expert_w(name, shape):
        out = torch.empty((El,) + shape, device=dev, dtype=cdt)
        hw = torch.empty((E,) + shape, dtype=cdt) if keep_host else None
        for e in range(E):
            w = (rn(*shape) * 0.02).to(cdt)
            if rank * El <= e < (rank + 1) * El:
                out[e - rank * El] = w
            if keep_host:
                hw[e] = w.cpu()
        if keep_host:
            host[name] = hw
        return out
    w_g, w_u, w_d = expert_w("g", (dff, d)), expert_w("u", (dff, d)), expert_w("d", (d, dff))
    return w_r, bias, w_g, w_u, w_d, host


def timed_regions(torch, dist, world, dev, step, steps, repeats, barrier, after_region=None):
    """`repeats` regions of exactly `steps` steps, each bracketed by barrier + synchronize and timed with CUDA
    events; returns per-region ms (max over ranks) and the host-clock windows of the regions.  `after_region`
    runs between regions (outside every timed region)."""
    ms_all, windows = [], []
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(repeats):
        barrier()
        w0 = time.time()
        ev0.record()
        for _ in range(steps):
            step()
        ev1.record()
        barrier()
        w1 = time.time()
        ms_all.append(ev0.elapsed_time(ev1))
        windows.append((w0, w1))
        if after_region is not None:
            after_region()
    if world > 1:
        t = torch.tensor(ms_all, device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_all = [float(v) for v in t.cpu()]
    return ms_all, windows


def mean_stage_ms(layer, n):
    """Mean per-stage device time over the last n profiled forwards (events recorded inside the timed loop)."""
    acc = None
    for back in range(n):
        st = layer.stage_ms(back)
        acc = st if acc is None else {a: acc[a] + st[a] for a in st}
    return {a: v / n for a, v in acc.items()}


def gpu_local_cpus(torch, local_rank):
    """CPUs of the NUMA node the GPU hangs off (sysfs), or None when it cannot be told."""
    try:
        p = torch.cuda.get_device_properties(local_rank)
        bdf = "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            spec = f.read().strip()
        cpus = set()
        for part in spec.split(","):
            a, _, b = part.partition("-")
            cpus.update(range(int(a), int(b or a) + 1))
        allowed = os.sched_getaffinity(0)
        cpus &= allowed
        return cpus or None
    except Exception:
        return None


def small_case(torch, dist, world, rank, dev, layer, x, steps, barrier, graph=False):
    """Times a short step (decode sweep, extras): 3 regions of `steps` steps, median; then 32 profiled forwards
    back to back for the stage times."""
    y = torch.empty_like(x)
    for _ in range(20):
        layer.forward_device(x, y)
    ms_all, _ = timed_regions(torch, dist, world, dev, lambda: layer.forward_device(x, y), steps, 3, barrier)
    ms = statistics.median(ms_all) / steps
    launches = layer.launch_count()
    layer.set_profiling(True)
    barrier()
    for _ in range(32):
        layer.forward_device(x, y)
    barrier()
    st = mean_stage_ms(layer, 32)
    layer.set_profiling(False)
    graph_ms = None
    if graph and world == 1:
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                layer.forward_device(x, y)
            for _ in range(5):
                g.replay()
            gm, _ = timed_regions(torch, dist, world, dev, g.replay, steps, 3, barrier)
            graph_ms = statistics.median(gm) / steps
        except Exception:
            graph_ms = None
    return ms, st, launches, graph_ms


def run_ours(args, cfg):
    import numpy as np
    import torch
    import torch.distributed as dist

    from omega_ai_b200 import MoELayer
    from omega_ai_b200.ep_layout import shard_tokens

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
    bpe = 2 if cdt == torch.bfloat16 else 4
    peaks = load_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # strong scaling: T is the global batch, sharded T/world per rank; experts E/world per rank
    lo, hi = shard_tokens(T, world, rank)
    T_local = hi - lo   # ranks may hold different shares when T is not a multiple of world (0 is allowed)
    El = E // world
    want_oracle = (not args.no_oracle) and rank == 0 and cfg["dtype"] == "bf16"
    w_r, bias, w_g, w_u, w_d, host_w = make_weights(torch, dev, cfg, cdt, world, rank, SEED, keep_host=want_oracle)
    x = global_rows(torch, dev, lo, hi, d, cdt, SEED)
    y = torch.empty_like(x)

    t_max = max(1, -(-T // world))
    layer = MoELayer(d, dff, E, k, bias=bias is not None, t_max=t_max, compute_dtype=cdt, world=world, rank=rank)
    layer.setWeights(w_r, w_g, w_u, w_d, bias)
    if world > 1:
        layer.ep_connect()
    # the decode sweep runs on the SAME weights through a second handle sized for decode steps
    decode_layer = None
    decode_shape = cfg["dtype"] == "bf16" and not args.no_decode and not args.tokens and not args.weak and \
        (d, dff, E, k) == (4096, 14336, 8, 2)
    if decode_shape:
        dt_max = 256 if world == 1 else max(1, 64 // world)
        decode_layer = MoELayer(d, dff, E, k, t_max=dt_max, compute_dtype=cdt, world=world, rank=rank)
        decode_layer.setWeights(w_r, w_g, w_u, w_d, bias)
        if world > 1:
            decode_layer.ep_connect()
    w_r_host = w_r.float().cpu().numpy() if want_oracle else None
    bias_host = bias.float().cpu().numpy() if (want_oracle and bias is not None) else None
    del w_g, w_u, w_d
    torch.cuda.synchronize()

    if args.block:
        gamma = torch.ones(d, device=dev, dtype=torch.float32)
        layer.forward_device = lambda xx, yy=None: layer.forward_block(xx, gamma, yy)

    # ---- device-resident timing: `repeats` regions of exactly `steps` steps ------------------------------
    for _ in range(args.warmup):
        layer.forward_device(x, y)
    barrier()
    step = lambda: layer.forward_device(x, y)
    launches_per_step = None
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
    else:
        layer.set_profiling(True)   # stage events are recorded inside the timed regions (no host sync between steps)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.1)
    n_prof = min(args.steps, 32)
    region_stages = []   # per region: mean stage times of its last n_prof steps
    collect = None if args.graph else (lambda: region_stages.append(mean_stage_ms(layer, n_prof)))
    ms_all, windows = timed_regions(torch, dist, world, dev, step, args.steps, args.repeats, barrier, collect)
    clocks, mhz_per_region = sampler.stop(windows) if rank == 0 else (None, [])
    order = sorted(range(len(ms_all)), key=lambda i: ms_all[i])
    med_i = order[len(order) // 2]
    ms = ms_all[med_i]
    ms_per_step = ms / args.steps
    value = T / (ms_per_step * 1e-3)
    if args.graph:
        # a replayed graph records no stage events: time the stages in a back-to-back run of direct calls
        layer.set_profiling(True)
        barrier()
        for _ in range(n_prof):
            layer.forward_device(x, y)
        barrier()
        stage_ms = mean_stage_ms(layer, n_prof)
    else:
        stage_ms = region_stages[med_i]   # the stages of the region that is reported
    layer.set_profiling(False)
    if launches_per_step is None:
        launches_per_step = layer.launch_count()
    stage_sum = sum(stage_ms.values())

    # ---- parity record: checksums in global token order, reduced over the ranks ---------------------------
    layer.forward_device(x, y)
    torch.cuda.synchronize()
    idx_l, gw_l, counts_local, _, _ = layer.routing(T_local)
    y_sum = bits_checksum(torch, y, lo * d) if T_local else 0
    idx_sum = bits_checksum(torch, torch.from_numpy(idx_l.astype(np.int64)).to(dev), lo * k) if T_local else 0
    sums = torch.tensor([y_sum, idx_sum, T_local], device=dev, dtype=torch.int64)
    counts_all = torch.from_numpy(counts_local.astype("int64")).to(dev)
    if world > 1:
        dist.all_reduce(sums)
        dist.all_reduce(counts_all)
    counts_all = counts_all.cpu().numpy()
    parity = {"y_sum": "%016x" % (int(sums[0].item()) & (2 ** 64 - 1)),
              "idx_sum": "%016x" % (int(sums[1].item()) & (2 ** 64 - 1)), "tokens": int(sums[2].item()),
              "what": "sum of bit pattern x index weight over y [T,d] and topk_idx [T,k] in global token order; "
                      "equal at every GPU count when no bit of the layer depends on the sharding"}
    oracle_ok = None
    if want_oracle and T_local and not args.block:
        # rank 0 holds its own slice of the tokens against the CPU oracle: routing of every one, outputs of a few
        from oracle import ref
        n_sel = min(8, T_local)
        sel = np.sort(np.random.default_rng(5).choice(T_local, n_sel, replace=False)).astype(np.int32)
        f = lambda t: t.float().numpy()
        r = ref.moe_forward(x.float().cpu().numpy(), w_r_host, f(host_w["g"]), f(host_w["u"]), f(host_w["d"]), k,
                            bias=bias_host, bf16=True, sel=sel, nthreads=host_cores())
        routing_exact = bool(np.array_equal(idx_l, r.topk_idx))
        got = y[torch.from_numpy(sel.astype(np.int64)).to(dev)].float().cpu().numpy().astype(np.float64)
        want = r.y.astype(np.float64)
        rms = float(np.sqrt(np.mean(want ** 2)))
        # the parity tests' bf16 bound: rel 2e-2 per element plus 2e-2 of the output's RMS for elements near zero
        worst = float((np.abs(got - want) / (2e-2 * np.abs(want) + 2e-2 * rms)).max())
        oracle_ok = {"ok": routing_exact and worst <= 1.0, "routing_bit_exact_tokens": int(T_local) if routing_exact else 0,
                     "output_tokens": int(n_sel), "worst_err_over_bound": worst}
        del r
    host_w = None

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

    # ---- end to end through the host-buffer entry points ----------------------------------------------------
    # Every step copies its rows from pinned host memory and its result back, inside the timed region; the steps
    # are enqueued with omoe_forward_host_async and awaited once with omoe_wait, so the copies of a step overlap
    # the kernels of its neighbours.  `sync_value` is the same loop with a host wait after every step.
    layer.forward_device(x, y)   # y of an inference forward (a training step above may have rounded differently)
    # Several GPUs copying at once load the host's memory fabric: each rank runs on the CPUs of its GPU's NUMA
    # node while it allocates and fills its pinned buffers and drives the copies, as a host process feeding one GPU
    # of a multi-socket box would (the affinity is put back afterwards; nothing on the GPU is set).
    saved_affinity, numa_bound = None, False
    if world > 1:
        cpus = gpu_local_cpus(torch, local_rank)
        if cpus:
            try:
                saved_affinity = os.sched_getaffinity(0)
                os.sched_setaffinity(0, cpus)
                numa_bound = True
            except OSError:
                saved_affinity = None
    xh = torch.empty((T_local, d), dtype=cdt).pin_memory()
    xh.copy_(x.cpu())
    yh = torch.empty((T_local, d), dtype=cdt).pin_memory()
    e2e_steps = max(3, min(args.steps, 20))
    for _ in range(3):
        layer.forward_host(xh, yh)
    e2e_ok = bool(torch.equal(yh, y.cpu())) if not args.block else None

    def e2e_region(pipelined):
        evs0, evs1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        evs0.record()
        for _ in range(e2e_steps):
            if pipelined:
                layer.forward_host_async(xh, yh)
            else:
                layer.forward_host(xh, yh)
        if pipelined:
            layer.wait()
        evs1.record()
        barrier()
        m = evs0.elapsed_time(evs1)
        if world > 1:
            t = torch.tensor([m], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            m = float(t.item())
        return m
    e2e_sync_ms = statistics.median(e2e_region(False) for _ in range(3))
    e2e_ms = statistics.median(e2e_region(True) for _ in range(3)) if not args.block else e2e_sync_ms
    e2e_value = T / (e2e_ms / e2e_steps * 1e-3)
    # What the box's host<->device copies alone cost per step (all ranks copying at once, both directions, no
    # kernels): the end-to-end step cannot be shorter than this, whatever the library does.
    copy_floor_ms = None
    try:
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        x_tmp = torch.empty_like(x)
        def copies():
            with torch.cuda.stream(s_in):
                x_tmp.copy_(xh, non_blocking=True)
            with torch.cuda.stream(s_out):
                yh.copy_(y, non_blocking=True)
        for _ in range(2):
            copies()
        barrier()
        t0c = time.perf_counter()
        for _ in range(10):
            copies()
        torch.cuda.synchronize()
        dtc = (time.perf_counter() - t0c) * 1e3 / 10
        if world > 1:
            t = torch.tensor([dtc], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dtc = float(t.item())
        copy_floor_ms = dtc
        del x_tmp
    except Exception:
        copy_floor_ms = None
    if saved_affinity is not None:
        os.sched_setaffinity(0, saved_affinity)

    # ---- decode sweep (config 5) on the same weights -------------------------------------------------------
    decode = None
    if decode_layer is not None:
        decode = []
        for Td in ((1, 2, 8, 64, 256) if world == 1 else (64,)):
            dlo, dhi = shard_tokens(Td, world, rank)
            xd = global_rows(torch, dev, dlo, dhi, d, cdt, SEED + 1000 + Td)
            ms_d, st, n_launch, graph_ms = small_case(torch, dist, world, rank, dev, decode_layer, xd, 200, barrier,
                                                      graph=True)
            _, _, c_loc, _, _ = decode_layer.routing(dhi - dlo)
            c_all = torch.from_numpy(c_loc.astype("int64")).to(dev)
            if world > 1:
                dist.all_reduce(c_all)
            c_all = c_all.cpu().numpy()
            # the bound is the rank that has the most active experts (one GPU: all active experts)
            n_active = max(int((c_all[r * El:(r + 1) * El] > 0).sum()) for r in range(world))
            wbytes = n_active * 3.0 * d * dff * 2
            kern_s = (st["up_gate"] + st["down"]) * 1e-3
            # A decode step is a handful of short launches, so a serving loop replays it from a CUDA graph: that
            # is the step time reported (one GPU); the same step issued as direct calls is given beside it.
            step_ms = graph_ms if graph_ms is not None else ms_d
            ent = {"tokens": Td, "ms_per_step": step_ms,
                   "launch": "cuda graph replay" if graph_ms is not None else "direct calls",
                   "direct_ms_per_step": ms_d, "n_active": n_active, "weight_bytes": wbytes,
                   "expert_kernels_ms": kern_s * 1e3, "expert_kernels_gbs": wbytes / kern_s / 1e9,
                   "frac": wbytes / kern_s / 1e9 / peaks["hbm"],
                   "whole_step_frac": wbytes / (step_ms * 1e-3) / 1e9 / peaks["hbm"],
                   "direct_whole_step_frac": wbytes / (ms_d * 1e-3) / 1e9 / peaks["hbm"], "launches": n_launch,
                   "stage_ms": st}
            decode.append(ent)
        decode_layer.close()
        decode = {"workload": CONFIGS["c5"]["name"], "bound": "hbm", "peak_gbs": peaks["hbm"],
                  "peak_source": peaks["src"], "steps": 200, "regions": 3,
                  "l2": "the active experts' weights (352 MB each) are streamed every step; no flush",
                  "sweep": decode}
    layer.close()
    del layer
    torch.cuda.empty_cache()

    # ---- extras: the mid-size and the 64-expert configurations as one-line records -------------------------
    extras = None
    if not args.no_extras and args.config == "c3" and not args.tokens and not args.weak and not args.block:
        extras = {}
        for name in ("c2", "c4"):
            c = CONFIGS[name]
            if name == "c2" and world > 1:
                continue   # stated for one GPU
            if c["E"] % world:
                continue
            Te = c["T"]
            elo, ehi = shard_tokens(Te, world, rank)
            wr2, b2, wg2, wu2, wd2, _ = make_weights(torch, dev, c, torch.bfloat16, world, rank, SEED + 7)
            lay = MoELayer(c["d"], c["dff"], c["E"], c["k"], bias=b2 is not None, t_max=max(1, -(-Te // world)),
                           compute_dtype=torch.bfloat16, world=world, rank=rank)
            lay.setWeights(wr2, wg2, wu2, wd2, b2)
            if world > 1:
                lay.ep_connect()
            del wg2, wu2, wd2
            xe = global_rows(torch, dev, elo, ehi, c["d"], torch.bfloat16, SEED + 2000)
            ms_e, st, n_launch, _ = small_case(torch, dist, world, rank, dev, lay, xe, 200, barrier)
            _, _, c_loc, _, _ = lay.routing(ehi - elo)
            lay.close()
            a = algorithmic(c, Te)
            extras[name] = {"workload": c["name"], "ms_per_step": ms_e, "tokens_per_s": Te / (ms_e * 1e-3),
                            "stage_ms": st, "launches": n_launch,
                            "layer_tflops_per_gpu": a["total_flops"] / world / (ms_e * 1e-3) / 1e12}
            if world == 1:   # per-kernel rates need the rows of the GPU; with skewed loads they differ per rank
                ug = a["up_gate_flops"] / (st["up_gate"] * 1e-3) / 1e12
                extras[name].update({"up_gate_tflops": ug, "up_gate_frac_of_burst": ug / peaks["tf_burst"],
                                     "down_tflops": a["down_flops"] / (st["down"] * 1e-3) / 1e12,
                                     "load_max_over_mean": float(c_loc.max() / max(1e-9, c_loc.mean()))})
            torch.cuda.empty_cache()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    alg = algorithmic(cfg, T_local)
    small = T <= 256 and cfg["dtype"] == "bf16"
    if small:
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
                "down_tflops": alg["down_flops"] / (stage_ms["down"] * 1e-3) / 1e12,
                "down_frac_of_burst": alg["down_flops"] / (stage_ms["down"] * 1e-3) / 1e12 / peaks["tf_burst"],
                "duration_from": "CUDA events recorded inside the timed regions (mean of the last %d steps)" % n_prof}
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
    layer_tf = alg["total_flops"] / (ms_per_step * 1e-3) / 1e12
    line = {
        "metric": "MoE-layer forward tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak" if args.weak else "strong", "vs_baseline": None, "dtype": cfg["dtype"], "data": "synthetic",
        "config": {"workload": cfg["name"] + (" + RMSNorm + residual" if args.block else ""), "tokens_global": T,
                   "tokens_per_gpu": T_local, "experts_per_gpu": El, "parallelism": f"ep{world}", "l2": l2_note,
                   "launch": "cuda graph replay" if args.graph else "direct calls",
                   "x": "row t of the global batch is drawn from the seed of its 2048-token block (same rows at every GPU count)"},
        "spread": {"regions": len(ms_all), "ms_per_step_median": ms_per_step,
                   "ms_per_step_min": min(ms_all) / args.steps, "ms_per_step_max": max(ms_all) / args.steps,
                   "ms_per_step_all": [m / args.steps for m in ms_all], "sm_mhz_median_per_region": mhz_per_region,
                   "reported": "median region; every region is exactly `steps` steps between barrier + synchronize"},
        "stage_ms": stage_ms, "stage_sum_ms": stage_sum, "stage_sum_over_step": stage_sum / ms_per_step,
        "layer_tflops": layer_tf,
        "layer_frac_of_burst": layer_tf / peaks["tf_burst"] if cfg["dtype"] == "bf16" else None,
        "roofline": roof, "cpu_baseline": cpu, "clocks": clocks,
        "parity": parity, "oracle_ok": oracle_ok,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": T_local * d * bpe,
                "d2h_bytes_per_step": T_local * d * bpe, "steps": e2e_steps,
                "how": "omoe_forward_host_async per step + one omoe_wait: each step's H2D and D2H are inside the "
                       "timed region and overlap neighbouring steps' kernels",
                "sync_value": T / (e2e_sync_ms / e2e_steps * 1e-3), "matches_device_path": e2e_ok,
                "host_threads_on_gpu_numa_node": numa_bound, "ms_per_step": e2e_ms / e2e_steps,
                "copies_alone_ms_per_step": copy_floor_ms,
                "copies_alone": "the same H2D + D2H per step on all ranks at once with no kernels running: a floor "
                                "the host's copy fabric sets for the end-to-end step"},
        "gpu_launches": launches_per_step * args.steps, "timed_regions": len(ms_all),
    }
    if decode is not None:
        line["decode"] = decode
    if extras:
        line["extras"] = extras
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
    ap.add_argument("--repeats", type=int, default=7, help="timed regions of `steps` steps; the median is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c3", choices=sorted(CONFIGS))
    ap.add_argument("--tokens", type=int, default=0, help="override the token count (decode sweep)")
    ap.add_argument("--cpu-tokens", type=int, default=0)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="skip the decode sweep")
    ap.add_argument("--no-extras", action="store_true", help="skip the config-2 / config-4 records")
    ap.add_argument("--no-oracle", action="store_true", help="skip rank 0's check of sampled tokens against the oracle")
    ap.add_argument("--no-refk", action="store_true", help="reference arm: skip the reference's GPU kernels")
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
    args.repeats = max(1, args.repeats)
    cfg = dict(CONFIGS[args.config])
    if args.impl == "reference":
        run_reference(args, cfg)
    else:
        run_ours(args, cfg)


if __name__ == "__main__":
    main()
