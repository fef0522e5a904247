"""The oracle's backward against an independent formulation: PyTorch autograd in float64 over the same
routing (the picks are constants), CPU only."""
import numpy as np
import pytest
import torch

from helpers import make_layer


def autograd_grads(x, w_r, w_g, w_u, w_d, k, dy, bias=None, renorm=True):
    t = lambda a: torch.tensor(a, dtype=torch.float64, requires_grad=True)
    X, Wr, Wg, Wu, Wd = t(x), t(w_r), t(w_g), t(w_u), t(w_d)
    B = None if bias is None else t(bias)
    logits = X @ Wr.T + (0 if B is None else B)
    # the picks come from the fp32 oracle (ties and rounding are its business); here they are constants
    return (X, Wr, B, Wg, Wu, Wd), logits


def run_autograd(oracle, x, w_r, w_g, w_u, w_d, k, dy, bias=None, renorm=True, aux_coef=0.0):
    (X, Wr, B, Wg, Wu, Wd), logits = autograd_grads(x, w_r, w_g, w_u, w_d, k, dy, bias, renorm)
    r = oracle.moe_forward(x, w_r, w_g, w_u, w_d, k, bias=bias, renorm=renorm)
    idx = torch.tensor(r.topk_idx.astype(np.int64))
    p = torch.softmax(logits, dim=1)
    pk = torch.gather(p, 1, idx)
    w = pk / pk.sum(dim=1, keepdim=True) if renorm else pk
    y = torch.zeros_like(X)
    for j in range(k):
        e = idx[:, j]
        g = torch.einsum("td,tfd->tf", X, Wg[e])
        u = torch.einsum("td,tfd->tf", X, Wu[e])
        h = torch.nn.functional.silu(g) * u
        y = y + w[:, j:j + 1] * torch.einsum("tf,tdf->td", h, Wd[e])
    objective = (y * torch.tensor(dy, dtype=torch.float64)).sum()
    if aux_coef:
        T, E = p.shape
        f = torch.tensor(r.counts.astype(np.float64)) / (T * k)
        objective = objective + aux_coef * E * (f * p.mean(dim=0)).sum()
    objective.backward()
    out = dict(dx=X.grad, d_w_r=Wr.grad, d_w_gate=Wg.grad, d_w_up=Wu.grad, d_w_down=Wd.grad)
    if B is not None:
        out["d_bias"] = B.grad
    return {n: v.numpy() for n, v in out.items()}, r


def close(got, ref, name, rtol=2e-4):
    scale = np.abs(ref).max() + 1e-30
    err = np.abs(got - ref).max()
    assert err <= rtol * scale, f"{name}: max err {err:.3e} against scale {scale:.3e}"


@pytest.mark.parametrize("T,d,dff,E,k,renorm,with_bias", [
    (16, 32, 48, 4, 2, True, False),
    (40, 64, 96, 8, 2, True, True),
    (33, 48, 80, 8, 3, False, True),
    (24, 32, 64, 16, 6, True, False),
    (5, 32, 48, 8, 2, True, False),   # most experts get no row: their weight gradients are zero
])
def test_backward_matches_autograd(oracle, T, d, dff, E, k, renorm, with_bias):
    x, w_r, w_g, w_u, w_d, _ = make_layer(T, d, dff, E, k, seed=11)
    w_r = (w_r * 20).astype(np.float32)  # spread the probabilities so the router's gradient is not negligible
    w_g, w_u, w_d = (w_g * 5).astype(np.float32), (w_u * 5).astype(np.float32), (w_d * 5).astype(np.float32)
    bias = (0.3 * np.random.default_rng(2).standard_normal(E)).astype(np.float32) if with_bias else None
    dy = np.random.default_rng(3).standard_normal((T, d)).astype(np.float32)
    ref, r = run_autograd(oracle, x, w_r, w_g, w_u, w_d, k, dy, bias, renorm)
    g = oracle.moe_backward(x, w_r, w_g, w_u, w_d, k, dy, bias=bias, renorm=renorm)
    for name in ("dx", "d_w_r", "d_w_gate", "d_w_up", "d_w_down"):
        close(getattr(g, name), ref[name], name)
    if with_bias:
        close(g.d_bias, ref["d_bias"], "d_bias")
    empty = np.nonzero(r.counts == 0)[0]
    for e in empty:
        assert not g.d_w_gate[e].any() and not g.d_w_up[e].any() and not g.d_w_down[e].any()


def test_backward_bf16_mode_stays_near_fp32(oracle):
    T, d, dff, E, k = 64, 64, 128, 8, 2
    x, w_r, w_g, w_u, w_d, _ = make_layer(T, d, dff, E, k, seed=12)
    rb = oracle.bf16_round
    x, w_r, w_g, w_u, w_d = rb(x), rb(w_r), rb(w_g * 5), rb(w_u * 5), rb(w_d * 5)
    dy = rb(np.random.default_rng(4).standard_normal((T, d)).astype(np.float32))
    a = oracle.moe_backward(x, w_r, w_g, w_u, w_d, k, dy)
    b = oracle.moe_backward(x, w_r, w_g, w_u, w_d, k, dy, bf16=True)
    for name in ("dx", "d_w_r", "d_w_gate", "d_w_up", "d_w_down"):
        close(getattr(b, name), getattr(a, name), name, rtol=3e-2)


def test_elementwise_backward_rules(oracle):
    rng = np.random.default_rng(5)
    x = (3 * rng.standard_normal(1000)).astype(np.float32)
    dl = rng.standard_normal(1000).astype(np.float32)
    xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    torch.nn.functional.silu(xt).backward(torch.tensor(dl, dtype=torch.float64))
    np.testing.assert_allclose(oracle.silu_backward(x, dl), xt.grad.numpy(), rtol=1e-5, atol=1e-6)
    lg = torch.tensor(rng.standard_normal((7, 16)), dtype=torch.float64, requires_grad=True)
    p = torch.softmax(lg, dim=1)
    dp = rng.standard_normal((7, 16))
    p.backward(torch.tensor(dp))
    got = oracle.softmax_back_rows(p.detach().numpy().astype(np.float32), dp.astype(np.float32))
    np.testing.assert_allclose(got, lg.grad.numpy(), rtol=1e-4, atol=1e-6)


def test_aux_loss_value_and_gradient(oracle):
    T, d, dff, E, k = 48, 32, 48, 8, 2
    x, w_r, w_g, w_u, w_d, _ = make_layer(T, d, dff, E, k, seed=13)
    w_r = (w_r * 20).astype(np.float32)
    dy = (0.01 * np.random.default_rng(6).standard_normal((T, d))).astype(np.float32)
    r = oracle.moe_forward(x, w_r, w_g, w_u, w_d, k)
    p = torch.softmax(torch.tensor(r.logits, dtype=torch.float64), dim=1).numpy()
    want = E * ((r.counts / (T * k)) * p.mean(axis=0)).sum()
    assert abs(oracle.aux_loss(r.logits, r.counts, k) - want) < 1e-5
    ref, _ = run_autograd(oracle, x, w_r, w_g, w_u, w_d, k, dy, aux_coef=0.5)
    g = oracle.moe_backward(x, w_r, w_g, w_u, w_d, k, dy, aux_coef=0.5)
    g0 = oracle.moe_backward(x, w_r, w_g, w_u, w_d, k, dy)
    for name in ("dx", "d_w_r", "d_w_gate", "d_w_up", "d_w_down"):
        close(getattr(g, name), ref[name], name)
    assert np.abs(g.d_w_r - g0.d_w_r).max() > 1e-4          # the term is there
    assert np.array_equal(g.d_w_down, g0.d_w_down)           # and touches the router's side only


def test_rmsnorm_backward_matches_autograd(oracle):
    rng = np.random.default_rng(8)
    x = (2 * rng.standard_normal((9, 96))).astype(np.float32)
    gamma = (1 + 0.2 * rng.standard_normal(96)).astype(np.float32)
    dout = rng.standard_normal((9, 96)).astype(np.float32)
    X = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    G = torch.tensor(gamma, dtype=torch.float64, requires_grad=True)
    out = X / torch.sqrt((X * X).mean(dim=1, keepdim=True) + 1e-5) * G
    out.backward(torch.tensor(dout, dtype=torch.float64))
    dinp, dgamma = oracle.rmsnorm_backward(x, gamma, dout)
    close(dinp, X.grad.numpy(), "dinp", rtol=1e-5)
    close(dgamma, G.grad.numpy(), "dgamma", rtol=1e-5)
