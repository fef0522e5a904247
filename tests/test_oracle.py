"""CPU tests of the oracle: known answers, an independent restatement, golden vectors."""
import os

import numpy as np
import torch

from helpers import make_layer

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "moe_small.npz")


def test_silu_known_answers(oracle):
    # the inputs of the reference's SiLU demo (SiLUKernel.java:33)
    x = np.array([1, 2, 3, 4, -5, 6, -7, -8, 9, 10, 11, -12, 13, 14, 15, -16], np.float32)
    got = oracle.silu(x)
    want = x.astype(np.float64) / (1.0 + np.exp(-x.astype(np.float64)))
    np.testing.assert_allclose(got, want, rtol=2e-7)
    np.testing.assert_allclose(got[:4], [0.7310586, 1.7615942, 2.8577224, 3.9280552], rtol=1e-6)


def test_all_ones_gemm_equals_k(oracle):
    # the check of the engine's host SGEMM demo: all-ones 64^3 gives 64 everywhere
    one = np.ones((64, 64), np.float32)
    assert (oracle.linear_nt(one, one) == 64.0).all()


def test_linear_is_x_times_w_transposed(oracle):
    rng = np.random.default_rng(1)
    X, W = rng.standard_normal((5, 37), dtype=np.float32), rng.standard_normal((11, 37), dtype=np.float32)
    np.testing.assert_allclose(oracle.linear_nt(X, W), X.astype(np.float64) @ W.astype(np.float64).T, rtol=1e-5, atol=1e-5)


def test_softmax_three_pass(oracle):
    rng = np.random.default_rng(2)
    x = (5 * rng.standard_normal((9, 13))).astype(np.float32)
    p = oracle.softmax_rows(x)
    np.testing.assert_allclose(p.sum(1), 1.0, rtol=1e-6)
    np.testing.assert_allclose(p, torch.softmax(torch.from_numpy(x).double(), -1).numpy(), rtol=1e-5, atol=1e-8)
    big = np.array([[1e4, 1e4 - 1, -1e4]], np.float32)  # max subtraction keeps it finite
    assert np.isfinite(oracle.softmax_rows(big)).all()


def test_bf16_rounding_matches_torch(oracle):
    rng = np.random.default_rng(3)
    v = np.concatenate([rng.standard_normal(4096).astype(np.float32) * 10.0 ** rng.integers(-20, 20, 4096),
                        np.array([0.0, -0.0, 1.0, 1.00390625, 1.005859375, np.inf, -np.inf], np.float32)])
    got = oracle.bf16_round(v)
    want = torch.from_numpy(v).to(torch.bfloat16).float().numpy()
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))


def _lane_tree_logit(x, w):
    """Independent restatement of the router's reduction order, float32 step by step."""
    even = [np.float32(0.0)] * 32
    odd = [np.float32(0.0)] * 32
    for i in range(x.size):
        l = (i // 8) % 32
        # fused multiply-add: exact product and sum in float64, one rounding to float32
        if i % 2:
            odd[l] = np.float32(np.float64(x[i]) * np.float64(w[i]) + np.float64(odd[l]))
        else:
            even[l] = np.float32(np.float64(x[i]) * np.float64(w[i]) + np.float64(even[l]))
    lanes = [np.float32(a + b) for a, b in zip(even, odd)]
    for m in (16, 8, 4, 2, 1):
        lanes = [np.float32(lanes[l] + lanes[l ^ m]) for l in range(32)]
    return lanes[0]


def test_router_reduction_tree_bit_exact(oracle):
    rng = np.random.default_rng(4)
    # bf16-valued operands: their product is exact in float64, so the float64 emulation of fmaf is exact
    x = oracle.bf16_round(rng.standard_normal((3, 520), dtype=np.float32))
    w = oracle.bf16_round((0.02 * rng.standard_normal((4, 520))).astype(np.float32))
    bias = rng.standard_normal(4).astype(np.float32)
    got = oracle.router_logits(x, w, bias)
    for t in range(3):
        for e in range(4):
            want = np.float32(_lane_tree_logit(x[t], w[e]) + bias[e])
            assert got[t, e].view(np.uint32) == want.view(np.uint32)


def test_topk_ties_and_renormalisation(oracle):
    logits = np.array([[1.0, 3.0, 3.0, 2.0], [0.5, 0.5, 0.5, 0.5], [-1.0, -2.0, -3.0, 4.0]], np.float32)
    idx, w = oracle.topk_gate(logits, 2, renorm=True)
    np.testing.assert_array_equal(idx, [[1, 2], [0, 1], [3, 0]])  # ties go to the lower expert
    np.testing.assert_allclose(w.sum(1), 1.0, rtol=1e-6)
    _, w_raw = oracle.topk_gate(logits, 2, renorm=False)
    p = oracle.softmax_rows(logits)
    np.testing.assert_allclose(w_raw, np.take_along_axis(p, idx, 1), rtol=1e-7)


def test_permutation_is_stable_bijection(oracle):
    rng = np.random.default_rng(5)
    T, E, k = 200, 8, 3
    idx = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    counts, offsets, perm, pos = oracle.histogram_permute(idx, E)
    assert counts.sum() == T * k and offsets[-1] == T * k
    assert sorted(perm.tolist()) == list(range(T * k))
    flat = idx.reshape(-1)
    for e in range(E):
        seg = perm[offsets[e]:offsets[e + 1]]
        assert (flat[seg] == e).all() and (np.diff(seg) > 0).all()  # grouped by expert, ascending flat index
    np.testing.assert_array_equal(perm[pos], np.arange(T * k))


def test_whole_layer_against_float64_torch(oracle):
    x, w_r, w_g, w_u, w_d, _ = make_layer(48, 64, 96, 8, 2, seed=6)
    r = oracle.moe_forward(x, w_r, w_g, w_u, w_d, 2)
    X = torch.from_numpy(x).double()
    lg = X @ torch.from_numpy(w_r).double().T
    p = torch.softmax(lg, -1)
    _, ti = torch.topk(lg, 2, dim=-1)
    np.testing.assert_array_equal(ti.numpy(), r.topk_idx)
    w = torch.gather(p, 1, ti)
    w = w / w.sum(-1, keepdim=True)
    y = torch.zeros(48, 64, dtype=torch.double)
    for t in range(48):
        for j in range(2):
            e = int(ti[t, j])
            g, u = torch.from_numpy(w_g[e]).double() @ X[t], torch.from_numpy(w_u[e]).double() @ X[t]
            y[t] += w[t, j] * (torch.from_numpy(w_d[e]).double() @ (torch.nn.functional.silu(g) * u))
    np.testing.assert_allclose(r.y, y.numpy(), rtol=1e-4, atol=1e-6)
    np.testing.assert_allclose(r.topk_w, w.numpy(), rtol=1e-5)


def test_token_subset_and_pretransposed_agree(oracle):
    x, w_r, w_g, w_u, w_d, _ = make_layer(40, 64, 96, 4, 2, seed=8)
    full = oracle.moe_forward(x, w_r, w_g, w_u, w_d, 2)
    sel = np.array([3, 17, 5, 39], np.int32)
    sub = oracle.moe_forward(x, w_r, w_g, w_u, w_d, 2, sel=sel)
    np.testing.assert_array_equal(sub.y, full.y[sel])
    tr = lambda a: np.ascontiguousarray(a.transpose(0, 2, 1))
    pre = oracle.moe_forward(x, w_r, tr(w_g), tr(w_u), tr(w_d), 2, pretransposed=True)
    np.testing.assert_array_equal(pre.y, full.y)


def test_golden_vectors(oracle):
    g = np.load(GOLDEN)
    x, w_r, w_g, w_u, w_d, _ = make_layer(24, 64, 96, 8, 2, seed=101)
    r = oracle.moe_forward(x, w_r, w_g, w_u, w_d, 2)
    np.testing.assert_array_equal(r.logits, g["f32_logits"])
    np.testing.assert_array_equal(r.topk_idx, g["f32_idx"])
    np.testing.assert_array_equal(r.counts, g["f32_counts"])
    np.testing.assert_array_equal(r.perm, g["f32_perm"])
    np.testing.assert_allclose(r.topk_w, g["f32_w"], rtol=1e-6)
    np.testing.assert_allclose(r.y, g["f32_y"], rtol=1e-5, atol=1e-8)
    x, w_r, w_g, w_u, w_d, bias = make_layer(40, 64, 64, 16, 3, seed=102, zipf=True)
    xb, w_rb, bb = oracle.bf16_round(x), oracle.bf16_round(w_r), oracle.bf16_round(bias)
    r = oracle.moe_forward(xb, w_rb, w_g, w_u, w_d, 3, bias=bb, bf16=True)
    np.testing.assert_array_equal(r.logits, g["bf16_logits"])
    np.testing.assert_array_equal(r.topk_idx, g["bf16_idx"])
    np.testing.assert_array_equal(r.counts, g["bf16_counts"])
    np.testing.assert_array_equal(r.perm, g["bf16_perm"])
    np.testing.assert_allclose(r.y, g["bf16_y"], rtol=1e-2, atol=1e-6)  # one bf16 ulp of slack for libm's expf
    # backward of the fp32 case with the auxiliary-loss term
    x, w_r, w_g, w_u, w_d, _ = make_layer(24, 64, 96, 8, 2, seed=101)
    dy = np.random.default_rng(103).standard_normal(x.shape).astype(np.float32)
    b = oracle.moe_backward(x, w_r * 10, w_g * 3, w_u * 3, w_d * 3, 2, dy, aux_coef=0.25)
    for name in ("dx", "d_w_r", "d_w_gate", "d_w_up", "d_w_down"):
        want = g["bw_" + name]
        np.testing.assert_allclose(getattr(b, name), want, rtol=1e-5, atol=1e-6 * np.abs(want).max())


def test_rmsnorm_matches_the_reference_formula(oracle):
    rng = np.random.default_rng(9)
    x = (3 * rng.standard_normal((7, 200))).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(200)).astype(np.float32)
    got = oracle.rmsnorm(x, g, 1e-5)
    X = x.astype(np.float64)
    want = X / np.sqrt((X * X).mean(1, keepdims=True) + 1e-5) * g
    np.testing.assert_allclose(got, want, rtol=3e-6)
    gb = oracle.rmsnorm(x, g, 1e-5, bf16=True)
    np.testing.assert_array_equal(gb.view(np.uint32), oracle.bf16_round(got).view(np.uint32))
