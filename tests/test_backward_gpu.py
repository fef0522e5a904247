"""Backward pass through the C ABI against the oracle's backward (same rules, CPU)."""
import numpy as np
import pytest
import torch

from helpers import assert_close_bf16, assert_close_bf16_grad, assert_close_f32, make_layer

pytestmark = pytest.mark.gpu

NAMES = ("dx", "d_w_r", "d_w_gate", "d_w_up", "d_w_down")


def dev(a, dt=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda().to(dt).contiguous()


def run_layer(T, d, dff, E, k, compute, io, x, w_r, w_g, w_u, w_d, dy, bias=None, renorm=True):
    from omega_ai_b200 import MoELayer
    layer = MoELayer(d, dff, E, k, t_max=max(T, 1), compute_dtype=compute, bias=bias is not None, renormalize=renorm)
    layer.setWeights(dev(w_r, compute), dev(w_g, compute), dev(w_u, compute), dev(w_d, compute),
                     router_bias=None if bias is None else dev(bias, compute))
    layer.set_training(True)
    xd = dev(x, io)
    y = layer.forward_device(xd)
    dx = layer.backward(xd, dev(dy, io))
    g = layer.weight_grads()
    out = dict(y=y.float().cpu().numpy(), dx=dx.float().cpu().numpy(), d_w_r=g["d_router"].cpu().numpy(),
               d_bias=g["d_bias"].cpu().numpy(), d_w_gate=g["d_gate"].cpu().numpy(), d_w_up=g["d_up"].cpu().numpy(),
               d_w_down=g["d_down"].cpu().numpy())
    routing = layer.routing(T)
    layer.close()
    return out, routing


def close_scaled(got, ref, name, rtol):
    scale = np.abs(ref).max() + 1e-30
    err = np.abs(got - ref).max()
    assert err <= rtol * scale, f"{name}: max err {err:.3e} against scale {scale:.3e}"


@pytest.mark.parametrize("T,d,dff,E,k,renorm,with_bias", [
    (64, 128, 256, 8, 2, True, False),      # the reference-sized configuration
    (300, 256, 384, 8, 2, True, True),
    (130, 64, 136, 16, 4, False, True),     # d_ff not a multiple of 64, no renormalisation
    (5, 128, 128, 8, 2, True, False),       # experts without rows: zero weight gradients
])
def test_fp32_backward_matches_oracle(oracle, T, d, dff, E, k, renorm, with_bias):
    x, w_r, w_g, w_u, w_d, _ = make_layer(T, d, dff, E, k, seed=21)
    w_r = (w_r * 10).astype(np.float32)
    w_g, w_u, w_d = (w_g * 3).astype(np.float32), (w_u * 3).astype(np.float32), (w_d * 3).astype(np.float32)
    bias = (0.3 * np.random.default_rng(2).standard_normal(E)).astype(np.float32) if with_bias else None
    dy = np.random.default_rng(3).standard_normal((T, d)).astype(np.float32)
    got, routing = run_layer(T, d, dff, E, k, torch.float32, torch.float32, x, w_r, w_g, w_u, w_d, dy, bias, renorm)
    r = oracle.moe_forward(x, w_r, w_g, w_u, w_d, k, bias=bias, renorm=renorm)
    assert np.array_equal(routing[0], r.topk_idx)
    assert_close_f32(got["y"], r.y)  # the training-mode forward is still the layer
    ref = oracle.moe_backward(x, w_r, w_g, w_u, w_d, k, dy, bias=bias, renorm=renorm)
    for name in NAMES:
        close_scaled(got[name], getattr(ref, name), name, 2e-4)
    if with_bias:
        close_scaled(got["d_bias"], ref.d_bias, "d_bias", 2e-4)
    for e in np.nonzero(r.counts == 0)[0]:
        assert not got["d_w_gate"][e].any() and not got["d_w_up"][e].any() and not got["d_w_down"][e].any()


@pytest.mark.parametrize("T,d,dff,E,k,io", [
    (512, 256, 512, 8, 2, torch.bfloat16),
    (300, 320, 448, 8, 2, torch.float32),    # odd tile counts, fp32 rows in and out
    (700, 128, 256, 16, 4, torch.bfloat16),
    (9, 256, 256, 8, 2, torch.bfloat16),     # experts without rows
])
def test_bf16_backward_matches_oracle(oracle, T, d, dff, E, k, io):
    x, w_r, w_g, w_u, w_d, _ = make_layer(T, d, dff, E, k, seed=22)
    rb = oracle.bf16_round
    x, w_r = rb(x), rb(w_r * 10)
    w_g, w_u, w_d = rb(w_g * 3), rb(w_u * 3), rb(w_d * 3)
    dy = rb(np.random.default_rng(4).standard_normal((T, d)).astype(np.float32))
    got, routing = run_layer(T, d, dff, E, k, torch.bfloat16, io, x, w_r, w_g, w_u, w_d, dy)
    out_bf16 = io == torch.bfloat16
    r = oracle.moe_forward(x, w_r, w_g, w_u, w_d, k, bf16=True, out_bf16=out_bf16)
    assert np.array_equal(routing[0], r.topk_idx)
    # a training-mode forward rounds g and u to bf16 before SiLU (they are kept for the backward), one rounding
    # more than the inference forward the oracle's moe_forward states: held to the two-rounding bound
    assert_close_bf16_grad(got["y"], r.y)
    ref = oracle.moe_backward(x, w_r, w_g, w_u, w_d, k, dy, bf16=True, out_bf16=out_bf16)
    for name in NAMES:
        try:
            assert_close_bf16_grad(got[name], getattr(ref, name))
        except AssertionError as e:
            raise AssertionError(f"{name}: {e}") from None
    for e in np.nonzero(r.counts == 0)[0]:
        assert not got["d_w_gate"][e].any() and not got["d_w_up"][e].any() and not got["d_w_down"][e].any()


@pytest.mark.parametrize("compute", [torch.float32, torch.bfloat16])
def test_aux_loss_value_and_gradient(oracle, compute):
    from omega_ai_b200 import MoELayer
    T, d, dff, E, k = 200, 128, 256, 16, 2
    x, w_r, w_g, w_u, w_d, _ = make_layer(T, d, dff, E, k, seed=24)
    rb = oracle.bf16_round
    x, w_r = rb(x), rb(w_r * 10)
    dy = rb((0.01 * np.random.default_rng(7).standard_normal((T, d))).astype(np.float32))
    bf = compute == torch.bfloat16
    layer = MoELayer(d, dff, E, k, t_max=T, compute_dtype=compute)
    layer.setWeights(dev(w_r, compute), dev(w_g, compute), dev(w_u, compute), dev(w_d, compute))
    layer.set_training(True)
    layer.set_aux_loss(0.5)
    xd = dev(x, compute)
    layer.forward_device(xd)
    _, _, counts, _, _ = layer.routing(T)
    want = oracle.aux_loss(layer.logits(T), counts, k)
    assert abs(layer.aux_loss() - want) <= 1e-5 * want
    dx = layer.backward(xd, dev(dy, compute)).float().cpu().numpy()
    g = layer.weight_grads()
    ref = oracle.moe_backward(x, w_r, w_g, w_u, w_d, k, dy, bf16=bf, aux_coef=0.5)
    ref0 = oracle.moe_backward(x, w_r, w_g, w_u, w_d, k, dy, bf16=bf)
    assert np.abs(ref.d_w_r - ref0.d_w_r).max() > 10 * np.abs(ref0.d_w_r).max() * 1e-3   # the term matters here
    if bf:
        assert_close_bf16_grad(g["d_router"].cpu().numpy(), ref.d_w_r)
        assert_close_bf16_grad(dx, ref.dx)
    else:
        close_scaled(g["d_router"].cpu().numpy(), ref.d_w_r, "d_w_r", 2e-4)
        close_scaled(dx, ref.dx, "dx", 2e-4)
    layer.close()


@pytest.mark.parametrize("compute,io", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                        (torch.bfloat16, torch.float32)])
def test_block_backward_matches_oracle(oracle, compute, io):
    """y = x + MoE(rmsnorm(x) * gamma): dx, d gamma and the weight gradients of omoe_backward_block."""
    from omega_ai_b200 import MoELayer
    T, d, dff, E, k = 300, 256, 384, 8, 2
    x, w_r, w_g, w_u, w_d, _ = make_layer(T, d, dff, E, k, seed=25)
    bf = compute == torch.bfloat16
    rb = oracle.bf16_round
    x = (2.0 * x).astype(np.float32)
    w_r, w_g, w_u, w_d = w_r * 10, w_g * 3, w_u * 3, w_d * 3
    gamma = (1.0 + 0.2 * np.random.default_rng(3).standard_normal(d)).astype(np.float32)
    dy = np.random.default_rng(4).standard_normal((T, d)).astype(np.float32)
    if io == torch.bfloat16:
        x, dy = rb(x), rb(dy)
    if bf:
        w_r, w_g, w_u, w_d = rb(w_r), rb(w_g), rb(w_u), rb(w_d)
    out_bf16 = io == torch.bfloat16
    dx_ref, dgamma_ref, g_ref = oracle.moe_block_backward(x, gamma, w_r, w_g, w_u, w_d, k, dy, bf16=bf, out_bf16=out_bf16)
    layer = MoELayer(d, dff, E, k, t_max=T, compute_dtype=compute)
    layer.setWeights(dev(w_r, compute), dev(w_g, compute), dev(w_u, compute), dev(w_d, compute))
    layer.set_training(True)
    xd, gd = dev(x, io), dev(gamma)
    layer.forward_block(xd, gd)
    dx, dgamma = layer.backward_block(xd, gd, dev(dy, io))
    g = layer.weight_grads()
    got = dict(dx=dx.float().cpu().numpy(), dgamma=dgamma.cpu().numpy(), d_w_r=g["d_router"].cpu().numpy(),
               d_w_gate=g["d_gate"].cpu().numpy(), d_w_down=g["d_down"].cpu().numpy())
    want = dict(dx=dx_ref, dgamma=dgamma_ref, d_w_r=g_ref.d_w_r, d_w_gate=g_ref.d_w_gate, d_w_down=g_ref.d_w_down)
    for name in got:
        if bf:
            try:
                assert_close_bf16_grad(got[name], want[name])
            except AssertionError as e:
                raise AssertionError(f"{name}: {e}") from None
        else:
            close_scaled(got[name], want[name], name, 2e-4)
    layer.close()


def test_backward_call_order_and_modes(oracle):
    from omega_ai_b200 import MoELayer
    from omega_ai_b200.native import OmoeError
    T, d, dff, E, k = 64, 128, 256, 8, 2
    x, w_r, w_g, w_u, w_d, _ = make_layer(T, d, dff, E, k, seed=23)
    layer = MoELayer(d, dff, E, k, t_max=T, compute_dtype=torch.bfloat16)
    b = lambda a: dev(a, torch.bfloat16)
    layer.setWeights(b(w_r), b(w_g), b(w_u), b(w_d))
    xd, dy = b(x), b(np.ones((T, d), np.float32))
    y_inf = layer.forward_device(xd).float().cpu().numpy()
    with pytest.raises(OmoeError):   # not in training mode
        layer.backward(xd, dy)
    layer.set_training(True)
    with pytest.raises(OmoeError):   # no training-mode forward yet
        layer.backward(xd, dy)
    y_tr = layer.forward_device(xd).float().cpu().numpy()
    assert_close_bf16(y_tr, y_inf)
    dx1 = layer.backward(xd, dy).float().cpu().numpy()
    g1 = {n: v.cpu().numpy() for n, v in layer.weight_grads().items()}
    layer.forward_device(xd)
    dx2 = layer.backward(xd, dy).float().cpu().numpy()
    g2 = {n: v.cpu().numpy() for n, v in layer.weight_grads().items()}
    assert np.array_equal(dx1, dx2) and all(np.array_equal(g1[n], g2[n]) for n in g1)   # reproducible, overwritten
    layer.forward_block(xd, torch.ones(d, device="cuda"))
    with pytest.raises(OmoeError):   # the block form's RMSNorm and residual are not differentiated
        layer.backward(xd, dy)
    layer.set_training(False)
    layer.forward_device(xd)
    with pytest.raises(OmoeError):   # the inference forward overwrote what the backward reads
        layer.backward(xd, dy)
    layer.close()


def test_weight_gradients_on_transposed_copies_in_a_subprocess():
    """The weight-gradient products read the activations in place (MN-major tensor-core operands) by default;
    OMOE_WGRAD_TRANSPOSED=1, read when training mode is switched on, selects the older path through explicit
    transposed copies.  Both must give the oracle's gradients."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, OMOE_WGRAD_TRANSPOSED="1")
    cmd = [sys.executable, "-m", "pytest", os.path.join(root, "tests", "test_backward_gpu.py"), "-x", "-q", "-m", "gpu",
           "-k", "bf16_backward"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=root)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]


def test_full_size_backward_properties():
    """Config 3 at full size (16384 tokens, d=4096, d_ff=14336, 8 experts, top-2), where the CPU oracle would take
    minutes: properties that need no oracle.  Doubling dy is exact in floating point, so every gradient must double
    bit for bit; a second run must reproduce the first bit for bit; the rows of d logits sum to zero (softmax_back),
    so d router_bias sums to (nearly) zero; nothing is NaN or infinite."""
    from omega_ai_b200 import MoELayer
    T, d, dff, E, k = 16384, 4096, 14336, 8, 2
    g = torch.Generator(device="cuda").manual_seed(5)
    mk = lambda *s, sc=0.02: (torch.randn(*s, device="cuda", generator=g) * sc).to(torch.bfloat16)
    layer = MoELayer(d, dff, E, k, bias=True, t_max=T, compute_dtype=torch.bfloat16)
    layer.setWeights(mk(E, d), mk(E, dff, d), mk(E, dff, d), mk(E, d, dff), router_bias=mk(E, sc=0.1))
    x, dy = mk(T, d, sc=1.0), mk(T, d, sc=1.0)
    layer.set_training(True)

    def step(grad):
        layer.forward_device(x)
        dx = layer.backward(x, grad).clone()
        return dx, {n: v.clone() for n, v in layer.weight_grads().items()}

    dx1, g1 = step(dy)
    dx1b, g1b = step(dy)
    assert torch.equal(dx1, dx1b) and all(torch.equal(g1[n], g1b[n]) for n in g1)
    del dx1b, g1b
    dx2, g2 = step(dy * 2)
    assert torch.equal(dx2.float(), dx1.float() * 2)
    for n in g1:
        assert torch.isfinite(g1[n]).all(), n
        assert torch.equal(g2[n], g1[n] * 2), n
    assert g1["d_bias"].abs().max() > 0
    assert abs(float(g1["d_bias"].sum())) <= 1e-3 * float(g1["d_bias"].abs().sum())
    _, _, counts, _, _ = layer.routing(T)
    assert counts.sum() == T * k
    layer.close()
