"""Worker of the expert-parallel parity test: one process per GPU (torchrun).

Every rank holds E/world experts and its own tokens; the layer's output and
routing on each rank are compared with the CPU oracle run on that rank's tokens
with ALL experts.  Exits non-zero on any mismatch.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from helpers import assert_close_bf16, assert_close_bf16_grad, assert_close_f32, make_layer  # noqa: E402
from omega_ai_b200 import MoELayer  # noqa: E402
from oracle import ref  # noqa: E402


def run_case(rank, world, tokens, d, dff, E, k, compute, zipf, steps=2):
    El = E // world
    t_max = max(max(tokens), 1)
    _, w_r, w_g, w_u, w_d, bias = make_layer(1, d, dff, E, k, seed=77, zipf=zipf)
    bf = compute == torch.bfloat16
    if bf:
        w_r = ref.bf16_round(w_r)
        bias = None if bias is None else ref.bf16_round(bias)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda().to(compute).contiguous()
    layer = MoELayer(d, dff, E, k, bias=bias is not None, t_max=t_max, compute_dtype=compute, world=world, rank=rank)
    sl = slice(rank * El, (rank + 1) * El)
    layer.setWeights(dev(w_r), dev(w_g[sl]), dev(w_u[sl]), dev(w_d[sl]), None if bias is None else dev(bias))
    layer.ep_connect()
    for step in range(steps):
        T = tokens[(rank + step) % len(tokens)]
        rng = np.random.Generator(np.random.Philox(key=1000 + 10 * step + rank))
        x = rng.standard_normal((T, d), dtype=np.float32)
        if bf:
            x = ref.bf16_round(x)
        xd = dev(x) if T > 0 else torch.empty(0, d, device="cuda", dtype=compute)
        y = layer.forward_device(xd).float().cpu().numpy()
        idx, w, counts, offsets, perm = layer.routing(T)
        if T == 0:
            assert counts.sum() == 0
            layer.forward_block(xd, torch.ones(d, device="cuda"))  # every rank makes the same number of calls
            continue
        r = ref.moe_forward(x, w_r, w_g, w_u, w_d, k, bias=bias, bf16=bf)
        np.testing.assert_array_equal(idx, r.topk_idx)
        np.testing.assert_array_equal(counts, r.counts)
        np.testing.assert_array_equal(offsets, r.offsets)
        np.testing.assert_array_equal(perm, r.perm)
        np.testing.assert_allclose(w, r.topk_w, rtol=1e-5, atol=1e-7)
        (assert_close_bf16 if bf else assert_close_f32)(y, r.y)
        # the block form (RMSNorm in front, residual add in the combine) through the same transport
        gamma = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32)
        yb = layer.forward_block(xd, torch.from_numpy(gamma).cuda()).float().cpu().numpy()
        rb_ = ref.moe_block(x, gamma, w_r, w_g, w_u, w_d, k, bias=bias, bf16=bf)
        np.testing.assert_array_equal(layer.routing(T)[0], rb_.topk_idx)
        (assert_close_bf16 if bf else assert_close_f32)(yb, rb_.y)
    torch.cuda.synchronize()
    dist.barrier()
    layer.close()


def run_backward_case(rank, world, compute):
    """Expert-parallel training step: each rank's dx against the oracle run on ALL ranks' tokens (rank-major), the
    local experts' weight gradients against the oracle's for those experts, the router's gradients summed over
    the ranks.  Two steps with different rows; one rank has fewer tokens, and in the second step none."""
    d, dff, E, k = 128, 256, 8, 2
    El = E // world
    bf = compute == torch.bfloat16
    _, w_r, w_g, w_u, w_d, _ = make_layer(1, d, dff, E, k, seed=79)
    w_r, w_g, w_u, w_d = (w_r * 10), (w_g * 3), (w_u * 3), (w_d * 3)
    if bf:
        w_r, w_g, w_u, w_d = (ref.bf16_round(a) for a in (w_r, w_g, w_u, w_d))
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda().to(compute).contiguous()
    t_cap = 96
    layer = MoELayer(d, dff, E, k, t_max=t_cap, compute_dtype=compute, world=world, rank=rank)
    sl = slice(rank * El, (rank + 1) * El)
    layer.setWeights(dev(w_r), dev(w_g[sl]), dev(w_u[sl]), dev(w_d[sl]))
    layer.ep_connect()
    layer.set_training(True)
    for step in range(2):
        counts_t = [t_cap if q != world - 1 else (40 if step == 0 else 0) for q in range(world)]
        xs, dys = [], []
        for q in range(world):  # every rank can regenerate every rank's rows: nothing to exchange in the test
            rng = np.random.Generator(np.random.Philox(key=2000 + 10 * step + q))
            xq = rng.standard_normal((counts_t[q], d), dtype=np.float32)
            dq = rng.standard_normal((counts_t[q], d), dtype=np.float32)
            if bf:
                xq, dq = ref.bf16_round(xq), ref.bf16_round(dq)
            xs.append(xq)
            dys.append(dq)
        T = counts_t[rank]
        xd = dev(xs[rank]) if T else torch.empty(0, d, device="cuda", dtype=compute)
        dyd = dev(dys[rank]) if T else torch.empty(0, d, device="cuda", dtype=compute)
        layer.forward_device(xd)
        dx = layer.backward(xd, dyd).float().cpu().numpy()
        g = layer.weight_grads()
        d_router = g["d_router"].clone()
        dist.all_reduce(d_router)
        want = ref.moe_backward(np.concatenate(xs), w_r, w_g, w_u, w_d, k, np.concatenate(dys), bf16=bf)
        lo = sum(counts_t[:rank])
        close = (lambda a, b_, n: assert_close_bf16_grad(a, b_)) if bf else (
            lambda a, b_, n: np.testing.assert_allclose(a, b_, rtol=0, atol=2e-4 * (np.abs(b_).max() + 1e-30), err_msg=n))
        if T:
            close(dx, want.dx[lo:lo + T], "dx")
        close(g["d_gate"].cpu().numpy(), want.d_w_gate[sl], "d_w_gate")
        close(g["d_up"].cpu().numpy(), want.d_w_up[sl], "d_w_up")
        close(g["d_down"].cpu().numpy(), want.d_w_down[sl], "d_w_down")
        close(d_router.cpu().numpy(), want.d_w_r, "d_w_r")
    # The auxiliary loss and the block form under expert parallelism: what they add depends on the rank's own
    # tokens only (router side, RMSNorm, residual), so the oracle run on this rank's rows alone must agree.
    T = t_cap
    rng = np.random.Generator(np.random.Philox(key=3000 + rank))
    x = rng.standard_normal((T, d), dtype=np.float32)
    dy = (0.05 * rng.standard_normal((T, d))).astype(np.float32)
    gamma = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    if bf:
        x, dy = ref.bf16_round(x), ref.bf16_round(dy)
    close = (lambda a, b_, n: assert_close_bf16_grad(a, b_)) if bf else (
        lambda a, b_, n: np.testing.assert_allclose(a, b_, rtol=0, atol=2e-4 * (np.abs(b_).max() + 1e-30), err_msg=n))
    layer.set_aux_loss(0.5)
    xd, dyd = dev(x), dev(dy)
    layer.forward_device(xd)
    dx = layer.backward(xd, dyd).float().cpu().numpy()
    g = layer.weight_grads()
    want = ref.moe_backward(x, w_r, w_g, w_u, w_d, k, dy, bf16=bf, aux_coef=0.5)
    close(dx, want.dx, "dx with aux loss")
    close(g["d_router"].cpu().numpy(), want.d_w_r, "d_w_r with aux loss")
    layer.set_aux_loss(0.0)
    gd = torch.from_numpy(gamma).cuda()
    layer.forward_block(xd, gd)
    dxb, dgamma = layer.backward_block(xd, gd, dyd)
    dx_ref, dgamma_ref, _ = ref.moe_block_backward(x, gamma, w_r, w_g, w_u, w_d, k, dy, bf16=bf)
    close(dxb.float().cpu().numpy(), dx_ref, "block dx")
    close(dgamma.cpu().numpy(), dgamma_ref, "dgamma")
    torch.cuda.synchronize()
    dist.barrier()
    layer.close()


def run_graph_case(rank, world):
    """A captured expert-parallel forward replays: flags and the step's sequence number live on the device, so
    nothing in the kernels' arguments changes between steps.  Replays with fresh rows in the captured input
    buffer must equal direct calls on the same rows."""
    d, dff, E, k, T = 256, 384, 8, 2, 16
    El = E // world
    _, w_r, w_g, w_u, w_d, _ = make_layer(1, d, dff, E, k, seed=78)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda().to(torch.bfloat16).contiguous()
    layer = MoELayer(d, dff, E, k, t_max=T, compute_dtype=torch.bfloat16, world=world, rank=rank)
    sl = slice(rank * El, (rank + 1) * El)
    layer.setWeights(dev(ref.bf16_round(w_r)), dev(w_g[sl]), dev(w_u[sl]), dev(w_d[sl]))
    layer.ep_connect()
    rows = lambda i: dev(np.random.Generator(np.random.Philox(key=500 + 10 * i + rank)).standard_normal(
        (T, d), dtype=np.float32))
    x_static, y_static = rows(0), torch.empty(T, d, device="cuda", dtype=torch.bfloat16)
    for _ in range(2):
        layer.forward_device(x_static, y_static)
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        layer.forward_device(x_static, y_static)
    replayed = []
    for i in range(1, 4):
        x_static.copy_(rows(i))
        g.replay()
        torch.cuda.synchronize()
        replayed.append(y_static.clone())
    for i in range(1, 4):
        y = layer.forward_device(rows(i))
        torch.cuda.synchronize()
        assert torch.equal(y, replayed[i - 1]), f"graph replay {i} differs from the direct call on rank {rank}"
    dist.barrier()
    layer.close()


def run_refused_case(rank, world):
    """A step that does not fit an owner's buffer (recv_rows_max far below what the picks need) is refused by every
    rank alike: no row moves (nothing outside any buffer is touched), the output is zeros, the next synchronising
    call reports the device error, and the step after it -- one that fits -- is correct again."""
    from omega_ai_b200 import OmoeError
    d, dff, E, k, T = 128, 256, 8, 2, 512
    El = E // world
    _, w_r, w_g, w_u, w_d, _ = make_layer(1, d, dff, E, k, seed=81)
    w_r = ref.bf16_round(w_r)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda().to(torch.bfloat16).contiguous()
    # capacity: (ceil(64/128) + El) * 128 rows per owner; every expert receives world * 128 rows on average,
    # which padded to 128 per expert is more than that for every world size
    layer = MoELayer(d, dff, E, k, t_max=T, compute_dtype=torch.bfloat16, world=world, rank=rank, recv_rows_max=64)
    sl = slice(rank * El, (rank + 1) * El)
    layer.setWeights(dev(w_r), dev(w_g[sl]), dev(w_u[sl]), dev(w_d[sl]))
    layer.ep_connect()
    rng = np.random.Generator(np.random.Philox(key=4000 + rank))
    x = ref.bf16_round(rng.standard_normal((T, d), dtype=np.float32))
    y = torch.full((T, d), 7.0, device="cuda", dtype=torch.bfloat16)
    layer.forward_device(dev(x), y)
    torch.cuda.synchronize()
    try:
        layer.routing(T)
        raise AssertionError("a refused step must report OMOE_ERR_DEVICE")
    except OmoeError as e:
        assert e.code == -6 and "index check" in str(e), str(e)
    assert float(y.float().abs().max()) == 0.0, "a refused step combines nothing"
    dist.barrier()
    # a step small enough to fit: few tokens, so every owner receives at most 2 * 8 * world rows
    Ts = 8
    xs = ref.bf16_round(rng.standard_normal((Ts, d), dtype=np.float32))
    ys = layer.forward_device(dev(xs)).float().cpu().numpy()
    idx = layer.routing(Ts)[0]
    r = ref.moe_forward(xs, w_r, w_g, w_u, w_d, k, bf16=True)
    np.testing.assert_array_equal(idx, r.topk_idx)
    assert_close_bf16(ys, r.y)
    torch.cuda.synchronize()
    dist.barrier()
    layer.close()


def run_host_chunks_case(rank, world):
    """Host-buffer forwards under expert parallelism are cut into the same number of chunks on every rank (from
    t_max), also when the ranks hold different numbers of tokens; rows are bit-identical to the device path, and
    calls enqueued back to back with omoe_forward_host_async give the same rows after one omoe_wait."""
    d, dff, E, k = 256, 384, 8, 2
    El = E // world
    t_max = 2048   # four chunks of at least 512 tokens
    _, w_r, w_g, w_u, w_d, _ = make_layer(1, d, dff, E, k, seed=83)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda().to(torch.bfloat16).contiguous()
    layer = MoELayer(d, dff, E, k, t_max=t_max, compute_dtype=torch.bfloat16, world=world, rank=rank)
    sl = slice(rank * El, (rank + 1) * El)
    layer.setWeights(dev(ref.bf16_round(w_r)), dev(w_g[sl]), dev(w_u[sl]), dev(w_d[sl]))
    layer.ep_connect()
    for step, T in enumerate([2048 if rank % 2 == 0 else 700, 1500, 0 if rank == world - 1 else 2048]):
        rng = np.random.Generator(np.random.Philox(key=5000 + 10 * step + rank))
        x = torch.from_numpy(rng.standard_normal((T, d), dtype=np.float32)).to(torch.bfloat16)
        xd = x.cuda()
        want = layer.forward_device(xd).cpu()
        xh, yh = x.pin_memory(), torch.empty(T, d, dtype=torch.bfloat16).pin_memory()
        layer.forward_host(xh, yh)
        assert torch.equal(yh, want), f"host chunks differ from the device path (step {step}, rank {rank})"
        yh2 = [torch.empty(T, d, dtype=torch.bfloat16).pin_memory() for _ in range(3)]
        for i in range(3):
            layer.forward_host_async(xh, yh2[i])
        layer.wait()
        for i in range(3):
            assert torch.equal(yh2[i], want), f"pipelined host call {i} differs (step {step}, rank {rank})"
        dist.barrier()
    layer.close()


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    # uneven token counts per rank, one rank with no tokens in some steps
    run_case(rank, world, [300, 171, 0, 64], 256, 384, 8, 2, torch.bfloat16, False, steps=3)
    run_case(rank, world, [256, 128], 256, 256, 64, 6, torch.bfloat16, True, steps=2)
    run_case(rank, world, [64, 40], 128, 256, 8, 2, torch.float32, False, steps=2)
    run_graph_case(rank, world)
    run_host_chunks_case(rank, world)
    run_refused_case(rank, world)
    run_backward_case(rank, world, torch.float32)
    run_backward_case(rank, world, torch.bfloat16)
    dist.destroy_process_group()
    if rank == 0:
        print("ep parity ok")


if __name__ == "__main__":
    main()
