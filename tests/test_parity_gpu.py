"""GPU parity: the CUDA path through the C ABI against the CPU oracle."""
import numpy as np
import pytest
import torch

from helpers import assert_close_bf16, assert_close_f32, make_layer

pytestmark = pytest.mark.gpu


def run_gpu(x, w_r, w_g, w_u, w_d, bias, k, compute_dtype, io_dtype, renorm=True, t_max=None):
    from omega_ai_b200 import MoELayer, Tensor

    T, d = x.shape
    E, dff, _ = w_g.shape
    layer = MoELayer(d, dff, E, k, bias=bias is not None, t_max=t_max or max(T, 1),
                     compute_dtype=compute_dtype, renormalize=renorm)
    dev = lambda a: torch.from_numpy(a).cuda().to(compute_dtype).contiguous()
    layer.setWeights(dev(w_r), dev(w_g), dev(w_u), dev(w_d), None if bias is None else dev(bias))
    xin = Tensor(T, 1, 1, d, data=x, dtype=io_dtype)
    out = layer.forward(xin)
    y = out.syncHost().reshape(T, d)
    routing = layer.routing(T)
    logits = layer.logits(T)
    n_launch = layer.launch_count()
    layer.close()
    return y, routing, logits, n_launch


def check_routing(routing, logits, r):
    idx, w, counts, offsets, perm = routing
    np.testing.assert_array_equal(logits.view(np.uint32), r.logits.view(np.uint32))  # bit-exact logits
    np.testing.assert_array_equal(idx, r.topk_idx)
    np.testing.assert_array_equal(counts, r.counts)
    np.testing.assert_array_equal(offsets, r.offsets)
    np.testing.assert_array_equal(perm, r.perm)
    np.testing.assert_allclose(w, r.topk_w, rtol=1e-5, atol=1e-7)


def test_config1_fp32(oracle):
    """Tiny fp32 layer: T=64, d=128, E=8, top-2, d_ff=256."""
    x, w_r, w_g, w_u, w_d, bias = make_layer(64, 128, 256, 8, 2)
    r = oracle.moe_forward(x, w_r, w_g, w_u, w_d, 2)
    y, routing, logits, n = run_gpu(x, w_r, w_g, w_u, w_d, None, 2, torch.float32, torch.float32)
    check_routing(routing, logits, r)
    assert_close_f32(y, r.y)
    assert n >= 5


@pytest.mark.parametrize("T,d,dff,E,k", [(64, 128, 256, 8, 2), (300, 256, 384, 8, 2), (129, 192, 320, 16, 4)])
def test_small_bf16(oracle, T, d, dff, E, k):
    x, w_r, w_g, w_u, w_d, _ = make_layer(T, d, dff, E, k, seed=7)
    rb = oracle.bf16_round
    xb, w_rb = rb(x), rb(w_r)
    r = oracle.moe_forward(xb, w_rb, w_g, w_u, w_d, k, bf16=True)
    y, routing, logits, n = run_gpu(xb, w_rb, rb(w_g), rb(w_u), rb(w_d), None, k, torch.bfloat16, torch.bfloat16)
    check_routing(routing, logits, r)
    assert_close_bf16(y, r.y)
