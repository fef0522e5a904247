"""Worker of the self-checking-build test: runs with OMOE_LIB pointing at libomoe_check.so.

In that build every one-GPU forward first fills the dispatch, hidden and expert-output buffers with NaN patterns,
validates all routing indices on the device after the dispatch and checks that no row outside the rows in use was
written (csrc/check.cu); any violation comes back as OMOE_ERR_DEVICE from the next synchronising call.  Here the
small configurations run under it, their outputs must be finite and match the oracle, and every intermediate
(dispatched rows, hidden rows, expert outputs) is read back and held against the oracle's primitives.
"""
import ctypes as C
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from helpers import assert_close_bf16, assert_close_f32, make_layer  # noqa: E402
from omega_ai_b200 import MoELayer, native  # noqa: E402
from oracle import ref  # noqa: E402


def read_rows(layer, which, rows, width, bf16):
    L = native.lib()
    L.omoe_check_read_rows.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_long, C.c_long]
    L.omoe_check_read_rows.restype = C.c_int
    buf = np.empty((rows, width), np.uint16 if bf16 else np.float32)
    rc = L.omoe_check_read_rows(layer._h, which, buf.ctypes.data_as(C.c_void_p), 0, rows)
    assert rc == 0
    if bf16:
        return (buf.astype(np.uint32) << 16).view(np.float32)
    return buf


def case(T, d, dff, E, k, compute, zipf=False, seed=5):
    bf = compute == torch.bfloat16
    x, w_r, w_g, w_u, w_d, bias = make_layer(T, d, dff, E, k, seed=seed, zipf=zipf)
    rb = ref.bf16_round
    if bf:
        x, w_r, w_g, w_u, w_d = rb(x), rb(w_r), rb(w_g), rb(w_u), rb(w_d)
        bias = None if bias is None else rb(bias)
    r = ref.moe_forward(x, w_r, w_g, w_u, w_d, k, bias=bias, bf16=bf)
    dev = lambda a: torch.from_numpy(a).cuda().to(compute).contiguous()
    layer = MoELayer(d, dff, E, k, bias=bias is not None, t_max=T, compute_dtype=compute)
    layer.setWeights(dev(w_r), dev(w_g), dev(w_u), dev(w_d), None if bias is None else dev(bias))
    y = layer.forward_device(dev(x)).float().cpu().numpy()
    idx, w, counts, offsets, perm = layer.routing(T)   # synchronises: a failed device check raises here
    assert np.isfinite(y).all(), "a row the step never wrote reached the output"
    np.testing.assert_array_equal(idx, r.topk_idx)
    np.testing.assert_array_equal(perm, r.perm)
    (assert_close_bf16 if bf else assert_close_f32)(y, r.y)
    # intermediates, expert by expert (rows of expert e start at a multiple of 128)
    rows_cap = ((T * k + 127) // 128 + E) * 128
    xp = read_rows(layer, 0, rows_cap, d, bf)
    hb = read_rows(layer, 1, rows_cap, dff, bf)
    yp = read_rows(layer, 2, rows_cap, d, bf)
    poff = 0
    for e in range(E):
        c = int(counts[e])
        tok = perm[offsets[e]:offsets[e] + c] // k
        np.testing.assert_array_equal(xp[poff:poff + c], x[tok])             # dispatch is a copy: bit-exact
        if c:
            g, u = ref.linear_nt(x[tok], w_g[e]), ref.linear_nt(x[tok], w_u[e])
            hh = ref.silu(g) * u
            if bf:
                hh = rb(hh)
            yy = ref.linear_nt(hh, w_d[e])
            if bf:
                yy = rb(yy)
            (assert_close_bf16 if bf else assert_close_f32)(hb[poff:poff + c], hh)
            (assert_close_bf16 if bf else assert_close_f32)(yp[poff:poff + c], yy)
        pad = (c + 127) // 128 * 128
        assert np.isnan(xp[poff + c:poff + pad]).all(), "padding rows of the dispatch buffer were written"
        poff += pad
    assert np.isnan(xp[poff:]).all()
    layer.close()


def main():
    assert os.environ.get("OMOE_LIB", "").endswith("libomoe_check.so")
    assert hasattr(native.lib(), "omoe_check_read_rows"), "not the self-checking build"
    torch.cuda.set_device(0)
    case(64, 128, 256, 8, 2, torch.float32)                   # the reference-sized configuration
    case(512, 256, 512, 8, 2, torch.bfloat16, seed=3)         # tensor-core path
    case(300, 256, 384, 64, 6, torch.bfloat16, zipf=True)     # skewed load, empty experts
    case(5, 512, 1024, 8, 2, torch.bfloat16, seed=13)         # one-launch routing + few-row products
    case(1, 512, 1024, 8, 2, torch.bfloat16, seed=14)         # weight-streaming products
    case(200, 328, 200, 8, 2, torch.bfloat16, seed=31)        # K and N tails
    print("self-check ok")


if __name__ == "__main__":
    main()
