"""The allocation-free routing entry point against the regular one.

``omoe_route_noalloc`` is for callers that may not allocate device memory where
they need a routing decision (for example a serving loop whose own pool holds
all free memory and which forbids cudaMalloc on the request path).  It must
give the same indices, gate weights and per-expert counts as ``omoe_forward``
followed by ``omoe_get_routing``, on consecutive calls that share the library's
fixed scratch array.  This file sorts last on purpose, so a failure here cannot
hide the result of any other test in a run that stops at the first failure.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import make_layer

pytestmark = pytest.mark.gpu


def _route_noalloc(x, w_r, bias, k, renorm=True):
    from omega_ai_b200 import native

    L = native.lib()
    T, d = x.shape
    E = w_r.shape[0]
    idx = torch.full((T, k), -7, dtype=torch.int32, device="cuda")
    w = torch.full((T, k), -1.0, dtype=torch.float32, device="cuda")
    counts = torch.full((E,), -7, dtype=torch.int32, device="cuda")
    io = native.OMOE_BF16 if x.dtype == torch.bfloat16 else native.OMOE_F32
    rc = L.omoe_route_noalloc(x.data_ptr(), w_r.data_ptr(), None if bias is None else bias.data_ptr(), T, d, E, k,
                              int(renorm), io, idx.data_ptr(), w.data_ptr(), counts.data_ptr(),
                              torch.cuda.current_stream().cuda_stream)
    assert rc == 0, L.omoe_route_noalloc_error().decode()
    torch.cuda.synchronize()
    return idx.cpu().numpy(), w.cpu().numpy(), counts.cpu().numpy()


def _route_regular(x, w_r, w_g, w_u, w_d, bias, k):
    from omega_ai_b200 import MoELayer

    T, d = x.shape
    E, dff, _ = w_g.shape
    layer = MoELayer(d, dff, E, k, bias=bias is not None, t_max=T, compute_dtype=torch.bfloat16)
    layer.setWeights(w_r, w_g, w_u, w_d, bias)
    layer.forward_device(x)
    idx, w, counts, _, _ = layer.routing(T)
    layer.close()
    return idx, w, counts


@pytest.mark.parametrize("E,k,zipf", [(8, 2, False), (64, 6, True)])
def test_noalloc_matches_regular_twice(E, k, zipf):
    d, dff = 256, 128
    dev = lambda a, dt=torch.float32: torch.from_numpy(a).cuda().to(dt).contiguous()
    # two calls in a row; the second is smaller, so the shared scratch still holds
    # rows of the first call beyond what the second one writes
    for T, seed in ((700, 21), (131, 22)):
        x, w_r, w_g, w_u, w_d, bias = make_layer(T, d, dff, E, k, seed=seed, zipf=zipf)
        xb = dev(x, torch.bfloat16)
        w_rb = dev(w_r, torch.bfloat16)
        bb = None if bias is None else dev(bias, torch.bfloat16)
        ref_idx, ref_w, ref_counts = _route_regular(xb, w_rb, dev(w_g, torch.bfloat16), dev(w_u, torch.bfloat16),
                                                    dev(w_d, torch.bfloat16), bb, k)
        # the allocation-free call takes the router weights in fp32 (the values the regular path keeps)
        idx, w, counts = _route_noalloc(xb, w_rb.float().contiguous(), None if bb is None else bb.float().contiguous(), k)
        np.testing.assert_array_equal(idx, ref_idx)
        np.testing.assert_array_equal(counts, ref_counts)
        np.testing.assert_allclose(w, ref_w, rtol=1e-6, atol=0)
        assert counts.sum() == T * k


@pytest.mark.parametrize("T,d,E,k,xdt,zipf", [
    (700, 256, 8, 2, torch.bfloat16, False),
    (4096, 512, 128, 16, torch.float32, False),   # the largest footprint the fixed array allows, fp32 rows
    (4096, 256, 64, 6, torch.bfloat16, True),
])
def test_noalloc_matches_oracle_and_allocates_nothing(oracle, T, d, E, k, xdt, zipf):
    """Against the CPU oracle (logits -> top-k and gate weights -> counts), not only against the library itself;
    and the device's free memory is the same before and after a call once the first call in the context (which
    may make the driver load the library's module, the array included) has been made."""
    x, w_r, _, _, _, bias = make_layer(T, d, 8, E, k, seed=31, zipf=zipf)
    if xdt == torch.bfloat16:
        x = oracle.bf16_round(x)
    w_r = oracle.bf16_round(w_r)
    bias = None if bias is None else oracle.bf16_round(bias)
    xd = torch.from_numpy(x).cuda().to(xdt).contiguous()
    wd = torch.from_numpy(w_r).cuda().contiguous()
    bd = None if bias is None else torch.from_numpy(bias).cuda().contiguous()
    _route_noalloc(xd, wd, bd, k)           # first call in this context: set-up
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    idx, w, counts = _route_noalloc(xd, wd, bd, k)
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, f"device free memory changed across the call: {free0} -> {free1}"
    logits = oracle.router_logits(x, w_r, bias)
    ref_idx, ref_w = oracle.topk_gate(logits, k)
    np.testing.assert_array_equal(idx, ref_idx)
    np.testing.assert_allclose(w, ref_w, rtol=1e-5, atol=1e-7)
    np.testing.assert_array_equal(counts, np.bincount(ref_idx.reshape(-1), minlength=E))


def test_noalloc_rejects_misaligned_buffers():
    from omega_ai_b200 import native

    L = native.lib()
    x = torch.zeros(8 * 64 + 8, device="cuda")
    w = torch.zeros(8 * 64 + 8, device="cuda")
    out_i = torch.zeros(8, 2, dtype=torch.int32, device="cuda")
    out_w = torch.zeros(8, 2, device="cuda")
    counts = torch.zeros(8, dtype=torch.int32, device="cuda")
    for xo, wo in ((4, 0), (0, 4)):   # a view that starts 4 bytes into an allocation
        rc = L.omoe_route_noalloc(x.data_ptr() + xo, w.data_ptr() + wo, None, 8, 64, 8, 2, 1, native.OMOE_F32,
                                  out_i.data_ptr(), out_w.data_ptr(), counts.data_ptr(), None)
        assert rc == -1 and b"16-byte aligned" in L.omoe_route_noalloc_error()


def test_noalloc_rejects_sizes_beyond_its_scratch():
    from omega_ai_b200 import native

    L = native.lib()
    T = native.NOALLOC_MAX_TOKENS + 1
    x = torch.zeros(8, 64, device="cuda")
    w = torch.zeros(8, 64, device="cuda")
    out_i = torch.zeros(8, 2, dtype=torch.int32, device="cuda")
    out_w = torch.zeros(8, 2, device="cuda")
    counts = torch.zeros(8, dtype=torch.int32, device="cuda")
    rc = L.omoe_route_noalloc(x.data_ptr(), w.data_ptr(), None, T, 64, 8, 2, 1, native.OMOE_F32, out_i.data_ptr(),
                              out_w.data_ptr(), counts.data_ptr(), None)
    assert rc == -3  # OMOE_ERR_TOO_LARGE
    assert b"too small" in L.omoe_route_noalloc_error()
    rc = L.omoe_route_noalloc(x.data_ptr(), w.data_ptr(), None, 8, 64, 200, 2, 1, native.OMOE_F32, out_i.data_ptr(),
                              out_w.data_ptr(), counts.data_ptr(), None)
    assert rc == -3
