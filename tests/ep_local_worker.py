"""Worker of the single-process expert-parallel test: ONE process drives two GPUs (the reference's
threads-per-device mode).  Run with CUDA_MODULE_LOADING=EAGER: with lazy loading, the first use of a kernel on
one device can wait for the other device's running kernel, which here is waiting for that very kernel."""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from helpers import assert_close_bf16, make_layer  # noqa: E402
from omega_ai_b200 import MoELayer  # noqa: E402
from oracle import ref  # noqa: E402


def main():
    world, d, dff, E, k, T = 2, 256, 384, 8, 2, 200
    El = E // world
    _, w_r, w_g, w_u, w_d, _ = make_layer(1, d, dff, E, k, seed=80)
    w_r = ref.bf16_round(w_r)
    layers, xs = [], []
    for r in range(world):
        torch.cuda.set_device(r)
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(f"cuda:{r}").to(torch.bfloat16).contiguous()
        layer = MoELayer(d, dff, E, k, t_max=T, compute_dtype=torch.bfloat16, world=world, rank=r)
        sl = slice(r * El, (r + 1) * El)
        layer.setWeights(dev(w_r), dev(w_g[sl]), dev(w_u[sl]), dev(w_d[sl]))
        layers.append(layer)
        xs.append(ref.bf16_round(
            np.random.Generator(np.random.Philox(key=900 + r)).standard_normal((T, d), dtype=np.float32)))
    for r in range(world):
        torch.cuda.synchronize(r)
    MoELayer.ep_connect_local(layers)
    xd = [torch.from_numpy(xs[r]).to(f"cuda:{r}").to(torch.bfloat16) for r in range(world)]
    for r in range(world):
        torch.cuda.synchronize(r)
    for step in range(2):
        outs = []
        for r in range(world):           # issue every rank's forward before waiting for any
            torch.cuda.set_device(r)
            outs.append(layers[r].forward_device(xd[r]))
        for r in range(world):
            torch.cuda.synchronize(r)
        for r in range(world):
            torch.cuda.set_device(r)
            want = ref.moe_forward(xs[r], w_r, w_g, w_u, w_d, k, bf16=True)
            assert np.array_equal(layers[r].routing(T)[0], want.topk_idx)
            assert_close_bf16(outs[r].float().cpu().numpy(), want.y)
    for r in range(world):
        torch.cuda.set_device(r)
        layers[r].close()
    print("single-process ep ok")


if __name__ == "__main__":
    main()
