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


@pytest.mark.parametrize("T", [8192 + 24, 16384 + 37, 40000])
def test_forward_host_in_chunks_matches_device(T):
    """Large host batches are cut into 2, 4 or 8 chunks whose copies overlap the kernels of their neighbours.
    Tokens are independent: every output row keeps its bits."""
    from omega_ai_b200 import MoELayer
    d, dff, E, k = 128, 128, 8, 2
    _, w_r, w_g, w_u, w_d, _ = make_layer(1, d, dff, E, k, seed=10)
    layer = MoELayer(d, dff, E, k, t_max=T, compute_dtype=torch.bfloat16)
    dev = lambda a: torch.from_numpy(a).cuda().to(torch.bfloat16).contiguous()
    layer.setWeights(dev(w_r), dev(w_g), dev(w_u), dev(w_d))
    g = torch.Generator(device="cuda").manual_seed(3)
    xd = torch.randn(T, d, device="cuda", generator=g).to(torch.bfloat16)
    yd = layer.forward_device(xd).clone()
    xh = xd.cpu().pin_memory()
    yh = torch.empty_like(xh).pin_memory()
    layer.forward_host(xh, yh)
    assert torch.equal(yd.cpu(), yh)
    layer.close()


def test_forward_host_async_pipelines_calls():
    """Calls enqueued with omoe_forward_host_async before one omoe_wait run in order with their copies overlapped;
    batches of different sizes (different chunking) in a row keep every row's bits."""
    from omega_ai_b200 import MoELayer
    d, dff, E, k = 128, 128, 8, 2
    _, w_r, w_g, w_u, w_d, _ = make_layer(1, d, dff, E, k, seed=11)
    layer = MoELayer(d, dff, E, k, t_max=20000, compute_dtype=torch.bfloat16)
    dev = lambda a: torch.from_numpy(a).cuda().to(torch.bfloat16).contiguous()
    layer.setWeights(dev(w_r), dev(w_g), dev(w_u), dev(w_d))
    g = torch.Generator(device="cuda").manual_seed(4)
    cases = []
    for T in (20000, 300, 9000, 9000, 17000, 0, 20000):
        xd = torch.randn(T, d, device="cuda", generator=g).to(torch.bfloat16)
        want = layer.forward_device(xd).cpu()
        cases.append((xd.cpu().pin_memory(), torch.full((T, d), 3.0, dtype=torch.bfloat16).pin_memory(), want))
    for xh, yh, _ in cases:
        layer.forward_host_async(xh, yh)
    layer.wait()
    for i, (_, yh, want) in enumerate(cases):
        assert torch.equal(yh, want), f"call {i} differs"
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
    # a view that starts 4 bytes into an allocation: refused before any launch (rows move as 16-byte vectors)
    import ctypes as C
    from omega_ai_b200 import native
    L = native.lib()
    flat = torch.zeros(8 * 128 + 8, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(8 * 128 + 8, device="cuda", dtype=torch.bfloat16)
    for xo, yo in ((4, 0), (0, 4)):
        rc = L.omoe_forward(layer._h, flat.data_ptr() + xo, out.data_ptr() + yo, 8, native.OMOE_BF16, None)
        assert rc == -1 and b"16-byte aligned" in L.omoe_last_error(layer._h)
    layer.forward_device(x[:8].contiguous())  # and the handle still works
    torch.cuda.synchronize()
    layer.close()
    with pytest.raises(OmoeError):
        MoELayer(130, 256, 8, 2)  # d_model not a multiple of 8
    with pytest.raises(OmoeError):
        MoELayer(128, 256, 8, 9)  # top_k > experts


@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (2, 8, 2), (3, 8, 2), (4, 8, 2), (5, 8, 2), (8, 8, 2), (7, 64, 6), (4, 64, 6)])
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


@pytest.mark.parametrize("T,d,dff", [
    (2, 36864, 64),    # two token rows of this width leave room for two ring stages per warp, not three
    (1, 36864, 64),
    (2, 45056, 64),    # and of this width for none: the register-streaming kernel serves the step
    (2, 64, 36864),    # the wide side is the down product's K
])
def test_decode_wide_layers_bf16(oracle, T, d, dff):
    """Streaming products on very wide layers: fewer ring stages, or the other kernel; K of 64 is one short piece."""
    x, w_r, w_g, w_u, w_d, _ = make_layer(T, d, dff, 4, 2, seed=17)
    rb = oracle.bf16_round
    xb, w_rb = rb(x), rb(w_r)
    r = oracle.moe_forward(xb, w_rb, w_g, w_u, w_d, 2, bf16=True)
    y, routing, logits, n = run_gpu(xb, w_rb, rb(w_g), rb(w_u), rb(w_d), None, 2, torch.bfloat16, torch.bfloat16,
                                    t_max=8)
    check_routing(routing, logits, r)
    assert_close_bf16(y, r.y)


@pytest.mark.parametrize("T,d,dff,E,k", [
    (200, 328, 200, 8, 2),     # K and N not multiples of the 64/128/256 tile sizes (tails come from TMA bounds)
    (77, 64, 64, 4, 1),        # smallest bf16 shapes, top-1
    (300, 256, 128, 128, 8),   # 128 experts, top-8
    (150, 192, 256, 24, 3),    # expert count that is not a power of two
    (513, 128, 384, 12, 12),   # every expert picked (k = E)
])
def test_odd_shapes_bf16(oracle, T, d, dff, E, k):
    x, w_r, w_g, w_u, w_d, _ = make_layer(T, d, dff, E, k, seed=31)
    rb = oracle.bf16_round
    xb, w_rb = rb(x), rb(w_r)
    r = oracle.moe_forward(xb, w_rb, w_g, w_u, w_d, k, bf16=True)
    y, routing, logits, n = run_gpu(xb, w_rb, rb(w_g), rb(w_u), rb(w_d), None, k, torch.bfloat16, torch.bfloat16)
    check_routing(routing, logits, r)
    assert_close_bf16(y, r.y)


@pytest.mark.parametrize("T", [5, 16, 40])
def test_single_expert_layer_bf16(oracle, T):
    """One expert, top-1: what a GPU of an 8-way expert-parallel Mixtral-shaped layer holds.  Few rows, so the
    products run with K split over a cluster."""
    d, dff = 512, 1024
    x, w_r, w_g, w_u, w_d, _ = make_layer(T, d, dff, 1, 1, seed=44)
    rb = oracle.bf16_round
    xb, w_rb = rb(x), rb(w_r)
    r = oracle.moe_forward(xb, w_rb, w_g, w_u, w_d, 1, bf16=True)
    y, routing, logits, n = run_gpu(xb, w_rb, rb(w_g), rb(w_u), rb(w_d), None, 1, torch.bfloat16, torch.bfloat16)
    check_routing(routing, logits, r)
    assert_close_bf16(y, r.y)


def test_router_bias_and_raw_gate_weights(oracle):
    """A router bias and renormalize=0 (gate weights are the softmax values themselves)."""
    x, w_r, w_g, w_u, w_d, bias = make_layer(260, 256, 256, 16, 4, seed=32, bias_scale=0.5)
    rb = oracle.bf16_round
    xb, w_rb, bb = rb(x), rb(w_r), rb(bias)
    r = oracle.moe_forward(xb, w_rb, w_g, w_u, w_d, 4, bias=bb, bf16=True, renorm=False)
    y, routing, logits, n = run_gpu(xb, w_rb, rb(w_g), rb(w_u), rb(w_d), bb, 4, torch.bfloat16, torch.bfloat16,
                                    renorm=False)
    check_routing(routing, logits, r)
    assert_close_bf16(y, r.y)
    assert (routing[1].sum(1) < 1.0).all()


@pytest.mark.parametrize("T,d,dff,E,k", [(257, 72, 40, 16, 4), (33, 128, 256, 8, 2), (1, 64, 64, 8, 2)])
def test_fp32_layer_shapes(oracle, T, d, dff, E, k):
    x, w_r, w_g, w_u, w_d, _ = make_layer(T, d, dff, E, k, seed=33)
    r = oracle.moe_forward(x, w_r, w_g, w_u, w_d, k)
    y, routing, logits, n = run_gpu(x, w_r, w_g, w_u, w_d, None, k, torch.float32, torch.float32)
    check_routing(routing, logits, r)
    assert_close_f32(y, r.y)


def test_ties_go_to_the_lower_expert():
    """Identical router rows give identical logits: the picks must be experts 0..k-1, bit for bit."""
    from omega_ai_b200 import MoELayer
    T, d, dff, E, k = 40, 128, 128, 8, 3
    g = torch.Generator(device="cuda").manual_seed(1)
    w_r = torch.randn(1, d, generator=g, device="cuda").repeat(E, 1).to(torch.bfloat16).contiguous()
    w = lambda *s: (0.02 * torch.randn(*s, generator=g, device="cuda")).to(torch.bfloat16)
    layer = MoELayer(d, dff, E, k, t_max=T, compute_dtype=torch.bfloat16)
    layer.setWeights(w_r, w(E, dff, d), w(E, dff, d), w(E, d, dff))
    layer.forward_device(torch.randn(T, d, generator=g, device="cuda").to(torch.bfloat16))
    idx, wts, counts, _, _ = layer.routing(T)
    assert (idx == np.arange(k)[None, :]).all()
    np.testing.assert_allclose(wts, 1.0 / k, rtol=1e-6)
    assert counts[:k].tolist() == [T] * k and counts[k:].sum() == 0
    layer.close()


def test_repeated_forwards_are_deterministic():
    from omega_ai_b200 import MoELayer
    layer = MoELayer(512, 768, 8, 2, t_max=1000, compute_dtype=torch.bfloat16)
    layer.initParam(seed=3)
    x = torch.randn(1000, 512, device="cuda").to(torch.bfloat16)
    y0 = layer.forward_device(x).clone()
    for T in (1000, 7, 1000, 300):
        y = layer.forward_device(x[:T].contiguous())
        assert torch.equal(y, y0[:T])  # same bits whatever ran before, and rows do not depend on the batch
    layer.close()


@pytest.mark.slow
def test_config3_full_size_properties(oracle):
    """Mixtral-shaped layer at full size (T=16384): routing bit-exact on all tokens, outputs on a token sample."""
    from omega_ai_b200 import MoELayer
    T, d, dff, E, k = 16384, 4096, 14336, 8, 2
    g = torch.Generator(device="cuda").manual_seed(20240611)
    rn = lambda *s: (0.02 * torch.randn(*s, generator=g, device="cuda", dtype=torch.float32)).to(torch.bfloat16)
    w_r, w_g, w_u, w_d = rn(E, d), rn(E, dff, d), rn(E, dff, d), rn(E, d, dff)
    x = torch.randn(T, d, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    layer = MoELayer(d, dff, E, k, t_max=T, compute_dtype=torch.bfloat16)
    layer.setWeights(w_r, w_g, w_u, w_d)
    y = layer.forward_device(x).float().cpu().numpy()
    idx, w, counts, offsets, perm = layer.routing(T)
    logits = layer.logits(T)
    layer.close()
    # size-independent properties
    assert counts.sum() == T * k and offsets[-1] == T * k
    assert np.array_equal(np.sort(perm), np.arange(T * k))
    flat = idx.reshape(-1)
    assert (np.diff(flat[perm]) >= 0).all()                       # grouped by expert
    same = flat[perm][1:] == flat[perm][:-1]
    assert (np.diff(perm)[same] > 0).all()                        # stable inside an expert
    np.testing.assert_allclose(w.sum(1), 1.0, rtol=1e-5)
    # oracle: routing for every token, outputs for 12 of them
    sel = np.sort(np.random.default_rng(1).choice(T, 12, replace=False)).astype(np.int32)
    f = lambda t: t.float().cpu().numpy()
    r = oracle.moe_forward(f(x), f(w_r), f(w_g), f(w_u), f(w_d), k, bf16=True, sel=sel)
    np.testing.assert_array_equal(logits.view(np.uint32), r.logits.view(np.uint32))
    np.testing.assert_array_equal(idx, r.topk_idx)
    np.testing.assert_array_equal(counts, r.counts)
    np.testing.assert_array_equal(perm, r.perm)
    assert_close_bf16(y[sel], r.y)


@pytest.mark.slow
def test_config4_full_size_skewed(oracle):
    """Fine-grained layer at full size: T=8192, d=2048, E=64, top-6, d_ff=1408, Zipf(1.1) router bias scaled to 2."""
    from omega_ai_b200 import MoELayer
    T, d, dff, E, k = 8192, 2048, 1408, 64, 6
    g = torch.Generator(device="cuda").manual_seed(20240611)
    rn = lambda *s: (0.02 * torch.randn(*s, generator=g, device="cuda", dtype=torch.float32)).to(torch.bfloat16)
    w_r, w_g, w_u, w_d = rn(E, d), rn(E, dff, d), rn(E, dff, d), rn(E, d, dff)
    z = (torch.randperm(E, generator=g, device="cuda").float() + 1) ** -1.1
    bias = (2.0 * z / z.max()).to(torch.bfloat16)
    x = torch.randn(T, d, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    layer = MoELayer(d, dff, E, k, bias=True, t_max=T, compute_dtype=torch.bfloat16)
    layer.setWeights(w_r, w_g, w_u, w_d, bias)
    y = layer.forward_device(x).float().cpu().numpy()
    idx, w, counts, offsets, perm = layer.routing(T)
    logits = layer.logits(T)
    layer.close()
    assert counts.sum() == T * k and np.array_equal(np.sort(perm), np.arange(T * k))
    assert counts.max() > 4 * counts.mean() and counts.min() < counts.mean()  # the load really is skewed
    sel = np.sort(np.random.default_rng(2).choice(T, 48, replace=False)).astype(np.int32)
    f = lambda t: t.float().cpu().numpy()
    r = oracle.moe_forward(f(x), f(w_r), f(w_g), f(w_u), f(w_d), k, bias=f(bias), bf16=True, sel=sel)
    np.testing.assert_array_equal(logits.view(np.uint32), r.logits.view(np.uint32))
    np.testing.assert_array_equal(idx, r.topk_idx)
    np.testing.assert_array_equal(counts, r.counts)
    np.testing.assert_array_equal(perm, r.perm)
    assert_close_bf16(y[sel], r.y)


@pytest.fixture(scope="module")
def decode_layer():
    """Decode-shaped layer at full size (d=4096, E=8, top-2, d_ff=14336), shared by the token-count sweep."""
    from omega_ai_b200 import MoELayer
    d, dff, E, k = 4096, 14336, 8, 2
    g = torch.Generator(device="cuda").manual_seed(20240611)
    rn = lambda *s: (0.02 * torch.randn(*s, generator=g, device="cuda", dtype=torch.float32)).to(torch.bfloat16)
    w = (rn(E, d), rn(E, dff, d), rn(E, dff, d), rn(E, d, dff))
    layer = MoELayer(d, dff, E, k, t_max=256, compute_dtype=torch.bfloat16)
    layer.setWeights(*w)
    host = tuple(t.float().cpu().numpy() for t in w)
    yield layer, host
    layer.close()


@pytest.mark.slow
@pytest.mark.parametrize("T", [1, 2, 8, 64, 256])
def test_config5_full_size_decode(oracle, decode_layer, T):
    layer, (w_r, w_g, w_u, w_d) = decode_layer
    g = torch.Generator(device="cuda").manual_seed(100 + T)
    x = torch.randn(T, 4096, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    y = layer.forward_device(x).float().cpu().numpy()
    routing, logits = layer.routing(T), layer.logits(T)
    sel = np.arange(min(T, 8), dtype=np.int32)
    r = oracle.moe_forward(x.float().cpu().numpy(), w_r, w_g, w_u, w_d, 2, bf16=True, sel=sel)
    check_routing(routing, logits, r)
    assert_close_bf16(y[sel], r.y)


@pytest.mark.parametrize("knob", ["OMOE_SPLITK=0", "OMOE_SPLITK=1", "OMOE_SPLITK=2", "OMOE_SPLITK=4", "OMOE_SPLITK=8"])
def test_few_row_variants_forced_in_a_subprocess(knob):
    """Steps with few row tiles run the expert products with K split over a cluster of 1, 2, 4 or 8 CTAs (picked
    from the host's bound on the step's rows).  The knob, read once per process, forces one choice for every
    step: small, skewed and odd-shaped cases must pass with each, and with the split switched off."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    name, value = knob.split("=")
    env = dict(os.environ, **{name: value})
    cmd = [sys.executable, "-m", "pytest", os.path.join(root, "tests", "test_parity_gpu.py"), "-x", "-q", "-m", "gpu",
           "-k", "small_bf16 or config4_skewed or odd_shapes or block_forward"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=root)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]


@pytest.mark.parametrize("knobs", ["OMOE_DECODE_MMA=0", "OMOE_DECODE_MAX_T=8", "OMOE_DECODE_MAX_T=8 OMOE_DECODE_MMA=0"])
def test_decode_kernel_variants_forced_in_a_subprocess(knobs):
    """The weight-streaming products exist twice: staged through per-warp rings of bulk copies (the default) and
    loaded straight into registers.  By default they serve steps of one or two tokens; raised to 8 tokens, experts
    hold more rows than one pass folds, so the weights are streamed in several passes.  Every combination must
    pass the decode cases (odd K: the last chunk of a weight row is short)."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, **dict(kv.split("=") for kv in knobs.split()))
    cmd = [sys.executable, "-m", "pytest", os.path.join(root, "tests", "test_parity_gpu.py"), "-x", "-q", "-m", "gpu",
           "-k", "decode_streaming_path or decode_shapes"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=root)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]


@pytest.mark.parametrize("compute,io", [(torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32),
                                        (torch.float32, torch.float32)])
@pytest.mark.parametrize("T", [3, 300])
def test_block_forward_rmsnorm_and_residual(oracle, compute, io, T):
    """y = x + MoE(rmsnorm(x) * gamma) in one call; logits stay bit-exact because the norm's reduction is fixed."""
    from omega_ai_b200 import MoELayer
    d, dff, E, k = 256, 384, 8, 2
    x, w_r, w_g, w_u, w_d, _ = make_layer(T, d, dff, E, k, seed=41)
    x = (2.0 * x).astype(np.float32)
    gamma = (1.0 + 0.2 * np.random.default_rng(3).standard_normal(d)).astype(np.float32)
    bf = compute == torch.bfloat16
    rb = oracle.bf16_round
    if io == torch.bfloat16:
        x = rb(x)
    if bf:
        w_r = rb(w_r)
    r = oracle.moe_block(x, gamma, w_r, w_g, w_u, w_d, k, bf16=bf, out_bf16=(io == torch.bfloat16))
    layer = MoELayer(d, dff, E, k, t_max=T, compute_dtype=compute)
    dev = lambda a, dt: torch.from_numpy(a).cuda().to(dt).contiguous()
    layer.setWeights(dev(w_r, compute), dev(w_g, compute), dev(w_u, compute), dev(w_d, compute))
    y = layer.forward_block(dev(x, io), dev(gamma, torch.float32)).float().cpu().numpy()
    check_routing(layer.routing(T), layer.logits(T), r)
    (assert_close_bf16 if bf else assert_close_f32)(y, r.y)
    layer.close()
