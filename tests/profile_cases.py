"""Small programs that put one kernel (or one step) on the GPU for a profiler capture; the summaries under profiles/
name the case they were taken from.  Usage: python tests/profile_cases.py <case> [args]

  train <c2|c3|c4> [steps]   training steps (training-mode forward + backward) of a benchmark configuration
  splitk                     the per-GPU share of an 8-GPU config-5 decode step: 1 expert, 16 rows, L2 flushed
  router                     config-4 forwards (64 experts): the router kernel with many experts
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from omega_ai_b200 import MoELayer  # noqa: E402

CONFIGS = {"c2": (4096, 1024, 2816, 8, 2), "c3": (16384, 4096, 14336, 8, 2), "c4": (8192, 2048, 1408, 64, 6)}


def _layer(T, d, dff, E, k, seed=1):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda *s: (torch.randn(*s, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    layer = MoELayer(d, dff, E, k, t_max=T, compute_dtype=torch.bfloat16)
    layer.setWeights(mk(E, d), mk(E, dff, d), mk(E, dff, d), mk(E, d, dff))
    return layer, g


def train(cfg="c3", steps=2):
    T, d, dff, E, k = CONFIGS[cfg]
    layer, g = _layer(T, d, dff, E, k)
    x = torch.randn(T, d, device="cuda", generator=g).to(torch.bfloat16)
    dy = torch.randn(T, d, device="cuda", generator=g).to(torch.bfloat16)
    layer.set_training(True)
    for _ in range(int(steps)):
        layer.forward_device(x)
        dx = layer.backward(x, dy)
    torch.cuda.synchronize()
    print("ok", float(dx.float().abs().mean()))


def splitk():
    d, dff, E, k, T = 4096, 14336, 1, 1, 16
    layer, g = _layer(T, d, dff, E, k)
    x = (torch.randn(T, d, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(4):
        flush.zero_()
        layer.forward_device(x)
    torch.cuda.synchronize()
    print("ok")


def router():
    T, d, dff, E, k = CONFIGS["c4"]
    layer, g = _layer(T, d, dff, E, k)
    x = torch.randn(T, d, device="cuda", generator=g).to(torch.bfloat16)
    for _ in range(4):
        layer.forward_device(x)
    torch.cuda.synchronize()
    print("ok")


if __name__ == "__main__":
    {"train": train, "splitk": splitk, "router": router}[sys.argv[1]](*sys.argv[2:])
