"""Regenerates tests/golden/moe_small.npz from the CPU oracle.

The reference ships no fixtures for this path (it has no MoE layer), so these
vectors pin the ORACLE: a later change to its arithmetic or to the routing
rules shows up as a diff against this file.  Run from the repository root:
    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from helpers import make_layer  # noqa: E402
from oracle import ref  # noqa: E402


def main():
    out = {}
    # fp32, the reference-sized configuration scaled down: T=24, d=64, d_ff=96, E=8, top-2
    x, w_r, w_g, w_u, w_d, _ = make_layer(24, 64, 96, 8, 2, seed=101)
    r = ref.moe_forward(x, w_r, w_g, w_u, w_d, 2)
    out.update(f32_logits=r.logits, f32_idx=r.topk_idx, f32_w=r.topk_w, f32_counts=r.counts, f32_perm=r.perm, f32_y=r.y)
    # bf16 rounding points, skewed router bias, top-3 of 16
    x, w_r, w_g, w_u, w_d, bias = make_layer(40, 64, 64, 16, 3, seed=102, zipf=True)
    xb, w_rb, bb = ref.bf16_round(x), ref.bf16_round(w_r), ref.bf16_round(bias)
    r = ref.moe_forward(xb, w_rb, w_g, w_u, w_d, 3, bias=bb, bf16=True)
    out.update(bf16_logits=r.logits, bf16_idx=r.topk_idx, bf16_w=r.topk_w, bf16_counts=r.counts, bf16_perm=r.perm,
               bf16_y=r.y)
    # backward of the fp32 case (with the auxiliary-loss term), for a fixed dy
    x, w_r, w_g, w_u, w_d, _ = make_layer(24, 64, 96, 8, 2, seed=101)
    dy = np.random.default_rng(103).standard_normal(x.shape).astype(np.float32)
    g = ref.moe_backward(x, w_r * 10, w_g * 3, w_u * 3, w_d * 3, 2, dy, aux_coef=0.25)
    out.update(bw_dx=g.dx, bw_d_w_r=g.d_w_r, bw_d_w_gate=g.d_w_gate, bw_d_w_up=g.d_w_up, bw_d_w_down=g.d_w_down)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "moe_small.npz"), **out)


if __name__ == "__main__":
    main()
