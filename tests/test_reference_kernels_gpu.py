"""The oracle and the CUDA path against the REFERENCE's own kernels, run on this GPU.

The reference has no MoE layer, but it has the pieces the layer is specified from: the `softmax` kernel,
`silu_forward`, `mul_kernel`, the RMSNorm forward kernel and FullyLayer's cublasSgemm call, strung together
by LlamaMLPLayer.output().  oracle/_ref holds those kernels compiled from the reference's own source
files; oracle/refk_driver.cu starts them as the reference's Java wrappers do.  Here the CPU oracle's
restatement of each stage is held against them, and so is the product: with the routing the library
reports, every expert's rows go through the reference's dense MLP, the gate-weighted sum is formed on the
host, and the result must match what `omoe_forward` returned within the fp32 tolerance (1e-4 abs, 1e-3 rel).
"""
import numpy as np
import pytest
import torch

from helpers import assert_close_f32, make_layer

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def refk():
    from oracle import refk as m
    if not m.available():
        pytest.skip("oracle/_ref (the reference's kernels, built where the reference checkout is) is not here")
    m.lib()
    return m


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def test_softmax_kernel_pins_the_oracle(oracle, refk):
    rng = np.random.default_rng(5)
    for rows, n in [(64, 8), (1000, 64), (3, 128), (1, 8)]:
        x = (3.0 * rng.standard_normal((rows, n))).astype(np.float32)
        x[0, : min(n, 3)] = x[0, 0]  # equal logits
        got = refk.softmax(dev(x)).cpu().numpy()
        ref = oracle.softmax_rows(x)
        # same three passes in the same order; the device's expf may differ from the host's in the last place
        np.testing.assert_allclose(ref, got, rtol=2e-6, atol=1e-9)
        assert (np.argmax(ref, axis=1) == np.argmax(got, axis=1)).all()


def test_silu_kernel_pins_the_oracle(oracle, refk):
    demo = np.array([1, 2, 3, 4, -5, 6, -7, -8, 9, 10, 11, -12, 13, 14, 15, -16], np.float32)  # SiLUKernel.java:33
    x = np.concatenate([demo, np.random.default_rng(6).standard_normal(5000).astype(np.float32) * 4])
    got = refk.silu(dev(x)).cpu().numpy()
    np.testing.assert_allclose(oracle.silu(x), got, rtol=2e-6, atol=1e-9)


def test_backward_kernels_pin_the_oracle(oracle, refk):
    rng = np.random.default_rng(10)
    x = (3 * rng.standard_normal(5000)).astype(np.float32)
    dl = rng.standard_normal(5000).astype(np.float32)
    got = refk.silu_backward(dev(x), dev(dl)).cpu().numpy()
    np.testing.assert_allclose(oracle.silu_backward(x, dl), got, rtol=3e-6, atol=1e-7)
    p = oracle.softmax_rows((2 * rng.standard_normal((300, 64))).astype(np.float32))
    dp = rng.standard_normal((300, 64)).astype(np.float32)
    got = refk.softmax_back(dev(p), dev(dp)).cpu().numpy()
    np.testing.assert_allclose(oracle.softmax_back_rows(p, dp), got, rtol=1e-5, atol=1e-7)


def test_mul_kernel_is_a_plain_product(refk):
    rng = np.random.default_rng(7)
    a, b = rng.standard_normal(4097).astype(np.float32), rng.standard_normal(4097).astype(np.float32)
    assert np.array_equal(refk.mul(dev(a), dev(b)).cpu().numpy(), a * b)


def test_rmsnorm_kernel_pins_the_oracle(oracle, refk):
    rng = np.random.default_rng(8)
    for rows, width in [(7, 256), (300, 1024), (33, 4096)]:
        x = (2.0 * rng.standard_normal((rows, width))).astype(np.float32)
        gamma = (1.0 + 0.2 * rng.standard_normal(width)).astype(np.float32)
        got = refk.rmsnorm(dev(x), dev(gamma)).cpu().numpy()
        # the kernel sums the squares in its own warp order: equal up to the rounding of that sum
        np.testing.assert_allclose(oracle.rmsnorm(x, gamma), got, rtol=1e-5, atol=1e-6)


def test_linear_is_x_times_w_transposed(oracle, refk):
    rng = np.random.default_rng(9)
    x = rng.standard_normal((37, 192)).astype(np.float32)
    w = (0.05 * rng.standard_normal((80, 192))).astype(np.float32)
    got = refk.linear(dev(x), dev(w)).cpu().numpy()
    assert_close_f32(got, oracle.linear_nt(x, w))
    ones = refk.linear(dev(np.ones((4, 64))), dev(np.ones((5, 64)))).cpu().numpy()
    assert np.array_equal(ones, np.full((4, 5), 64.0, np.float32))  # all-ones product = K


def _reference_moe(refk, x, idx, w, w_g, w_u, w_d):
    """The layer as the reference would compute it given the routing: each expert's rows through its own
    dense MLP kernels, then y[t] = ((w0*y0) + w1*y1) + ... in pick order."""
    T, k = idx.shape
    E = w_g.shape[0]
    xd = dev(x)
    outs = {}
    for e in range(E):
        rows = np.nonzero((idx == e).any(axis=1))[0]
        if rows.size == 0:
            continue
        ye = refk.mlp(xd[torch.from_numpy(rows).cuda()].contiguous(), dev(w_g[e]), dev(w_u[e]), dev(w_d[e]))
        outs[e] = (rows, ye.cpu().numpy())
    y = np.zeros_like(x)
    row_of = {e: {int(t): i for i, t in enumerate(rows)} for e, (rows, _) in outs.items()}
    for t in range(T):
        acc = None
        for j in range(k):
            e = int(idx[t, j])
            term = np.float32(w[t, j]) * outs[e][1][row_of[e][t]]
            acc = term if acc is None else (acc + term).astype(np.float32)
        y[t] = acc
    return y


@pytest.mark.parametrize("T,d,dff,E,k", [(64, 128, 256, 8, 2), (300, 256, 384, 8, 2), (200, 256, 128, 16, 4)])
def test_fp32_layer_against_reference_kernels(oracle, refk, T, d, dff, E, k):
    from omega_ai_b200 import MoELayer
    x, w_r, w_g, w_u, w_d, _ = make_layer(T, d, dff, E, k, seed=77)
    layer = MoELayer(d, dff, E, k, t_max=T, compute_dtype=torch.float32)
    layer.setWeights(dev(w_r), dev(w_g), dev(w_u), dev(w_d))
    y = layer.forward_device(dev(x)).cpu().numpy()
    idx, w, counts, _, _ = layer.routing(T)
    logits = layer.logits(T)
    # gate weights: the reference's softmax kernel on the library's logits, read at the picks and renormalised
    p = refk.softmax(dev(logits)).cpu().numpy()
    picked = np.take_along_axis(p, idx.astype(np.int64), axis=1)
    w_ref = picked / picked.sum(axis=1, keepdims=True, dtype=np.float32)
    np.testing.assert_allclose(w, w_ref, rtol=1e-5, atol=1e-7)
    y_ref = _reference_moe(refk, x, idx, w, w_g, w_u, w_d)
    assert_close_f32(y, y_ref)
    # and the oracle's whole layer against the same
    r = oracle.moe_forward(x, w_r, w_g, w_u, w_d, k)
    assert np.array_equal(r.topk_idx, idx)
    assert_close_f32(r.y, y_ref)
    layer.close()


def test_bf16_layer_against_reference_kernels(oracle, refk):
    """bf16 operands on tensor cores against the reference's fp32 kernels fed the same bf16-rounded values:
    what is left is the rounding of h and of the output (rel 2e-2)."""
    from helpers import assert_close_bf16
    from omega_ai_b200 import MoELayer
    T, d, dff, E, k = 512, 256, 512, 8, 2
    x, w_r, w_g, w_u, w_d, _ = make_layer(T, d, dff, E, k, seed=78)
    rb = oracle.bf16_round
    x, w_r, w_g, w_u, w_d = rb(x), rb(w_r), rb(w_g), rb(w_u), rb(w_d)
    layer = MoELayer(d, dff, E, k, t_max=T, compute_dtype=torch.bfloat16)
    b = lambda a: dev(a).to(torch.bfloat16)
    layer.setWeights(b(w_r), b(w_g), b(w_u), b(w_d))
    y = layer.forward_device(b(x)).float().cpu().numpy()
    idx, w, _, _, _ = layer.routing(T)
    y_ref = _reference_moe(refk, x, idx, w, w_g, w_u, w_d)
    assert_close_bf16(y, y_ref)
    layer.close()
