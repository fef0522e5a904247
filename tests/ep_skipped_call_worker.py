"""Worker of the failure-detection test on 2 GPUs: a rank that skips one collective call.

No GPU faults, traps or hangs: rank 1 simply does not make one ``forward`` call between two steps (it is alive,
idle, with nothing in flight).  Rank 0's step then waits for rank 1's count row; the wait is bounded
(``OMOE_EP_WAIT_MS``, a few hundred ms here), runs out, the kernels of the step finish without touching a row, and
the next synchronising call on rank 0 reports ``OMOE_ERR_DEVICE``.  The CUDA context stays usable: rank 0 then runs
a single-GPU layer on the same device and checks it against the oracle.  Both ranks meet at a host barrier before
they tear anything down.
"""
import os
import sys
import time

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from helpers import assert_close_bf16, make_layer  # noqa: E402
from omega_ai_b200 import MoELayer, OmoeError  # noqa: E402
from oracle import ref  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    assert world == 2
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    # host-side barriers only (gloo): no collective kernel is in flight while a rank sits a step out
    dist.init_process_group("gloo")
    d, dff, E, k, T = 128, 256, 8, 2, 64
    El = E // world
    _, w_r, w_g, w_u, w_d, _ = make_layer(1, d, dff, E, k, seed=91)
    w_r = ref.bf16_round(w_r)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda().to(torch.bfloat16).contiguous()
    layer = MoELayer(d, dff, E, k, t_max=T, compute_dtype=torch.bfloat16, world=world, rank=rank)
    sl = slice(rank * El, (rank + 1) * El)
    layer.setWeights(dev(w_r), dev(w_g[sl]), dev(w_u[sl]), dev(w_d[sl]))
    layer.ep_connect()
    rng = np.random.Generator(np.random.Philox(key=6000 + rank))
    x = ref.bf16_round(rng.standard_normal((T, d), dtype=np.float32))
    xd = dev(x)
    # step 1: both ranks take part; correct
    y = layer.forward_device(xd).float().cpu().numpy()
    assert_close_bf16(y, ref.moe_forward(x, w_r, w_g, w_u, w_d, k, bf16=True).y)
    torch.cuda.synchronize()
    dist.barrier()
    # step 2: rank 1 sits it out (between steps, nothing of its own in flight)
    if rank == 0:
        t0 = time.time()
        layer.forward_device(xd)
        try:
            layer.routing(T)   # synchronises and reads the device error word
            raise AssertionError("the wait for the absent rank should have run out")
        except OmoeError as e:
            assert e.code == -6 and "bounded wait ran out" in str(e), str(e)
        waited = time.time() - t0
        assert waited < 5.0, f"the bounded waits took {waited:.1f} s"
        # the context is intact: a fresh single-GPU layer on the same device computes correctly
        solo = MoELayer(d, dff, E, k, t_max=T, compute_dtype=torch.bfloat16)
        solo.setWeights(dev(w_r), dev(w_g), dev(w_u), dev(w_d))
        ys = solo.forward_device(xd).float().cpu().numpy()
        assert_close_bf16(ys, ref.moe_forward(x, w_r, w_g, w_u, w_d, k, bf16=True).y)
        solo.close()
        print(f"rank 0: wait ran out after {waited:.2f} s, OMOE_ERR_DEVICE reported, context intact")
    else:
        time.sleep(0.2)
    torch.cuda.synchronize()
    dist.barrier()
    layer.close()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("skipped-call detection ok")


if __name__ == "__main__":
    main()
