"""Expert-parallel parity on 2+ GPUs: spawns one process per GPU (torchrun)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(n):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", OMOE_EP_WAIT_MS="5000")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29517", os.path.join(ROOT, "tests", "ep_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert "ep parity ok" in p.stdout


def test_expert_parallel_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    _run(2)


def test_expert_parallel_all_gpus():
    n = torch.cuda.device_count()
    if n < 4:
        pytest.skip("needs 4 or more GPUs")
    _run(8 if n >= 8 else 4)


def test_expert_parallel_in_one_process():
    """One process drives two GPUs (the reference's threads-per-device mode): handles connected with
    omoe_ep_connect_local, each rank's forward issued in turn from this thread, then both awaited."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from helpers import assert_close_bf16, make_layer
    from omega_ai_b200 import MoELayer
    from oracle import ref
    world, d, dff, E, k, T = 2, 256, 384, 8, 2, 200
    El = E // world
    _, w_r, w_g, w_u, w_d, _ = make_layer(1, d, dff, E, k, seed=80)
    w_r = ref.bf16_round(w_r)
    layers, xs, ys = [], [], []
    for r in range(world):
        torch.cuda.set_device(r)
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(f"cuda:{r}").to(torch.bfloat16).contiguous()
        layer = MoELayer(d, dff, E, k, t_max=T, compute_dtype=torch.bfloat16, world=world, rank=r)
        sl = slice(r * El, (r + 1) * El)
        layer.setWeights(dev(w_r), dev(w_g[sl]), dev(w_u[sl]), dev(w_d[sl]))
        layers.append(layer)
        x = ref.bf16_round(np.random.Generator(np.random.Philox(key=900 + r)).standard_normal((T, d), dtype=np.float32))
        xs.append(x)
    for r in range(world):
        torch.cuda.synchronize(r)
    MoELayer.ep_connect_local(layers)
    for step in range(2):
        outs = []
        for r in range(world):           # issue every rank's forward before waiting for any
            torch.cuda.set_device(r)
            xd = torch.from_numpy(xs[r]).to(f"cuda:{r}").to(torch.bfloat16)
            outs.append(layers[r].forward_device(xd))
        for r in range(world):
            torch.cuda.synchronize(r)
        for r in range(world):
            torch.cuda.set_device(r)
            want = ref.moe_forward(xs[r], w_r, w_g, w_u, w_d, k, bf16=True)
            idx = layers[r].routing(T)[0]
            assert np.array_equal(idx, want.topk_idx)
            assert_close_bf16(outs[r].float().cpu().numpy(), want.y)
    for r in range(world):
        torch.cuda.set_device(r)
        layers[r].close()
    torch.cuda.set_device(0)
