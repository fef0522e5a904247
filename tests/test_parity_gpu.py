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


def test_config2_bf16_full(oracle):
    """Mid-size layer in full: T=4096, d=1024, E=8, top-2, d_ff=2816."""
    x, w_r, w_g, w_u, w_d, _ = make_layer(4096, 1024, 2816, 8, 2)
    rb = oracle.bf16_round
    xb, w_rb = rb(x), rb(w_r)
    rng = np.random.default_rng(0)
    sel = np.sort(rng.choice(4096, 256, replace=False)).astype(np.int32)
    r = oracle.moe_forward(xb, w_rb, w_g, w_u, w_d, 2, bf16=True, sel=sel)
    y, routing, logits, n = run_gpu(xb, w_rb, rb(w_g), rb(w_u), rb(w_d), None, 2, torch.bfloat16, torch.bfloat16)
    check_routing(routing, logits, r)
    assert_close_bf16(y[sel], r.y)


def test_config4_skewed_bf16(oracle):
    """Many experts with a Zipf router bias (skewed load), scaled down in T and d_ff."""
    x, w_r, w_g, w_u, w_d, bias = make_layer(2048, 512, 256, 64, 6, zipf=True)
    rb = oracle.bf16_round
    xb, w_rb, bb = rb(x), rb(w_r), rb(bias)
    r = oracle.moe_forward(xb, w_rb, w_g, w_u, w_d, 6, bias=bb, bf16=True)
    assert r.counts.max() > 4 * r.counts.mean() or r.counts.min() < 0.25 * r.counts.mean()
    y, routing, logits, n = run_gpu(xb, w_rb, rb(w_g), rb(w_u), rb(w_d), bb, 6, torch.bfloat16, torch.bfloat16)
    check_routing(routing, logits, r)
    assert_close_bf16(y, r.y)


@pytest.mark.parametrize("T", [1, 8, 64, 256])
def test_decode_shapes_bf16(oracle, T):
    """Small token counts (decode): some experts get no rows at all."""
    x, w_r, w_g, w_u, w_d, _ = make_layer(T, 512, 1024, 8, 2, seed=11)
    rb = oracle.bf16_round
    xb, w_rb = rb(x), rb(w_r)
    r = oracle.moe_forward(xb, w_rb, w_g, w_u, w_d, 2, bf16=True)
    y, routing, logits, n = run_gpu(xb, w_rb, rb(w_g), rb(w_u), rb(w_d), None, 2, torch.bfloat16, torch.bfloat16,
                                    t_max=256)
    check_routing(routing, logits, r)
    assert_close_bf16(y, r.y)


def test_fp32_io_on_bf16_layer(oracle):
    """fp32 Tensor buffers in and out of a bf16 layer (the engine's Tensor is fp32 only)."""
    x, w_r, w_g, w_u, w_d, _ = make_layer(200, 256, 384, 8, 2, seed=5)
    r = oracle.moe_forward(x, w_r, w_g, w_u, w_d, 2, bf16=True, out_bf16=False)
    from omega_ai_b200 import MoELayer, Tensor
    layer = MoELayer(256, 384, 8, 2, t_max=200, compute_dtype=torch.bfloat16)
    dev = lambda a: torch.from_numpy(a).cuda().contiguous()
    layer.setWeights(dev(w_r), dev(w_g), dev(w_u), dev(w_d))  # fp32 sources, converted by the library
    y = layer.forward(Tensor(200, 1, 1, 256, data=x)).syncHost().reshape(200, 256)
    check_routing(layer.routing(200), layer.logits(200), r)
    assert_close_bf16(y, r.y)
    layer.close()


def test_forward_host_matches_device(oracle):
    x, w_r, w_g, w_u, w_d, _ = make_layer(300, 256, 384, 8, 2, seed=9)
    from omega_ai_b200 import MoELayer
    layer = MoELayer(256, 384, 8, 2, t_max=300, compute_dtype=torch.bfloat16)
    dev = lambda a: torch.from_numpy(a).cuda().to(torch.bfloat16).contiguous()
    layer.setWeights(dev(w_r), dev(w_g), dev(w_u), dev(w_d))
    xd = dev(x)
    yd = layer.forward_device(xd)
    xh = xd.cpu().pin_memory()
    yh = torch.empty_like(xh).pin_memory()
    layer.forward_host(xh, yh)
    assert torch.equal(yd.cpu(), yh)
    layer.close()


def test_errors_are_reported_not_fatal():
    from omega_ai_b200 import MoELayer, OmoeError
    layer = MoELayer(128, 256, 8, 2, t_max=16, compute_dtype=torch.bfloat16)
    x = torch.zeros(32, 128, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(OmoeError) as e:  # forward before weights
        layer.forward_device(x[:8])
    assert e.value.code == -4
    layer.initParam()
    with pytest.raises(OmoeError) as e:  # T beyond t_max: refused, no hidden realloc
        layer.forward_device(x)
    assert e.value.code == -3
    y = layer.forward_device(x[:0].contiguous())  # empty batch is a no-op
    assert y.shape[0] == 0
    layer.close()
    with pytest.raises(OmoeError):
        MoELayer(130, 256, 8, 2)  # d_model not a multiple of 8
    with pytest.raises(OmoeError):
        MoELayer(128, 256, 8, 9)  # top_k > experts


@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (2, 8, 2), (5, 8, 2), (8, 8, 2), (7, 64, 6)])
def test_decode_streaming_path_bf16(oracle, T, E, k):
    """T <= 8 takes the weight-streaming expert kernels; odd sizes exercise the K split and row passes."""
    x, w_r, w_g, w_u, w_d, _ = make_layer(T, 520, 1096, E, k, seed=13)
    rb = oracle.bf16_round
    xb, w_rb = rb(x), rb(w_r)
    r = oracle.moe_forward(xb, w_rb, w_g, w_u, w_d, k, bf16=True)
    y, routing, logits, n = run_gpu(xb, w_rb, rb(w_g), rb(w_u), rb(w_d), None, k, torch.bfloat16, torch.bfloat16,
                                    t_max=64)
    check_routing(routing, logits, r)
    assert_close_bf16(y, r.y)
