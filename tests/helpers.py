"""Shared helpers for the parity tests: seeded synthetic layers and tolerances."""
import numpy as np


def make_layer(T, d, dff, E, k, seed=20240611, bias_scale=0.0, zipf=False):
    """x ~ N(0,1), weights ~ N(0,0.02) (the benchmark configurations' distributions).

    With ``zipf`` the router bias is 2.0 * z/max(z), z[e] = rank(e)^-1.1 over a
    seeded permutation of the experts, which skews the expert load."""
    rng = np.random.Generator(np.random.Philox(key=seed))
    x = rng.standard_normal((T, d), dtype=np.float32)
    w_r = (0.02 * rng.standard_normal((E, d))).astype(np.float32)
    w_g = (0.02 * rng.standard_normal((E, dff, d))).astype(np.float32)
    w_u = (0.02 * rng.standard_normal((E, dff, d))).astype(np.float32)
    w_d = (0.02 * rng.standard_normal((E, d, dff))).astype(np.float32)
    bias = None
    if zipf:
        ranks = rng.permutation(E) + 1
        z = ranks.astype(np.float64) ** -1.1
        bias = (2.0 * z / z.max()).astype(np.float32)
    elif bias_scale:
        bias = (bias_scale * rng.standard_normal(E)).astype(np.float32)
    return x, w_r, w_g, w_u, w_d, bias


# tolerances stated by the task: fp32 max-abs 1e-4 / rel 1e-3; bf16 rel 2e-2
F32_ATOL, F32_RTOL = 1e-4, 1e-3
BF16_RTOL = 2e-2


def assert_close_f32(got, ref):
    err = np.abs(got - ref)
    bound = F32_ATOL + F32_RTOL * np.abs(ref)
    assert (err <= bound).all(), f"fp32 parity: max err {err.max():.3e} (max |ref| {np.abs(ref).max():.3e})"


def assert_close_bf16(got, ref):
    """rel 2e-2 per element, with an absolute floor of 2e-2 of the output's RMS
    so elements near zero are judged against the scale of the row."""
    err = np.abs(got - ref)
    floor = BF16_RTOL * float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    bound = BF16_RTOL * np.abs(ref) + floor
    assert (err <= bound).all(), (
        f"bf16 parity: max err {err.max():.3e}, worst ratio {(err / bound).max():.2f}, rms {floor / BF16_RTOL:.3e}")
