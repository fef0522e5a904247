"""Times the reference's own GPU path for the expert stage on this GPU: per expert, cuBLAS SGEMM (gate),
`silu_forward`, SGEMM (up), `mul_kernel`, SGEMM (down), fp32 on the null stream, launch shapes as in the
reference's Java wrappers (oracle/refk_driver.cu) — what LlamaMLPLayer.output() would run for each expert's
rows if a JVM with JCuda were here.  Routing, permutation and combine have no reference kernel and are
not in the timed region: rows arrive already grouped, T*k/E per expert.  A reported baseline, not a target.

    python oracle/refk_bench.py --config c3 [--steps 3 --warmup 1]

Prints one JSON line.  Test infrastructure: nothing in the product or in bench.py imports this file.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import refk  # noqa: E402

CONFIGS = {  # the benchmark's configurations (tokens, d_model, d_ff, experts, top-k)
    "c1": (64, 128, 256, 8, 2),
    "c2": (4096, 1024, 2816, 8, 2),
    "c3": (16384, 4096, 14336, 8, 2),
    "c4": (8192, 2048, 1408, 64, 6),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="c3", choices=sorted(CONFIGS))
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    a = ap.parse_args()
    T, d, dff, E, k = CONFIGS[a.config]
    rows = T * k // E
    g = torch.Generator(device="cuda").manual_seed(20240611)
    mk = lambda *s: torch.randn(*s, device="cuda", generator=g) * 0.02
    w1, w3, w2 = mk(E, dff, d), mk(E, dff, d), mk(E, d, dff)
    xp = torch.randn(E, rows, d, device="cuda", generator=g)
    yp = torch.empty(E, rows, d, device="cuda")
    scratch = refk.MlpScratch(rows, dff)
    refk.lib()

    def step():
        for e in range(E):
            refk.mlp(xp[e], w1[e], w3[e], w2[e], scratch, yp[e])

    for _ in range(a.warmup):
        step()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(a.steps):
        step()
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / a.steps
    flops = 6.0 * T * k * d * dff
    print(json.dumps({"impl": "reference kernels, C++-driven (no JVM)", "config": a.config, "dtype": "f32",
                      "stage": "expert products only (rows pre-grouped, T*k/E per expert)",
                      "ms_per_step": ms, "tokens_per_s": T / (ms * 1e-3), "tflops": flops / (ms * 1e-3) / 1e12,
                      "steps": a.steps, "warmup": a.warmup}))


if __name__ == "__main__":
    main()
