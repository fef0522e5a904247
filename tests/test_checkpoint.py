"""Checkpoint convention: headerless little-endian float32, router then per-expert gate/up/down."""
import io
import struct

import numpy as np
import pytest
import torch

from omega_ai_b200 import checkpoint


def test_stream_layout_and_byte_order():
    E, d, dff = 2, 3, 4
    rng = np.random.default_rng(0)
    w_r, b = rng.standard_normal((E, d), dtype=np.float32), rng.standard_normal(E, dtype=np.float32)
    g, u = rng.standard_normal((E, dff, d), dtype=np.float32), rng.standard_normal((E, dff, d), dtype=np.float32)
    dn = rng.standard_normal((E, d, dff), dtype=np.float32)
    f = io.BytesIO()
    checkpoint.write_moe(f, w_r, b, g, u, dn)
    raw = f.getvalue()
    order = [w_r, b, g[0], u[0], dn[0], g[1], u[1], dn[1]]
    want = b"".join(struct.pack("<f", float(v)) for a in order for v in a.reshape(-1))
    assert raw == want  # no header, low byte first, tensors in the stated order
    f.seek(0)
    got = checkpoint.read_moe(f, E, d, dff, has_bias=True)
    for a, bb in zip(got, (w_r, b, g, u, dn)):
        np.testing.assert_array_equal(a, bb)
    with pytest.raises(EOFError):
        checkpoint.read_moe(io.BytesIO(raw[:-4]), E, d, dff, has_bias=True)


def test_upcycling_from_a_dense_mlp_file():
    d, dff, E = 4, 6, 3
    rng = np.random.default_rng(1)
    mats = [rng.standard_normal(s, dtype=np.float32) for s in ((dff, d), (dff, d), (d, dff))]
    f = io.BytesIO(b"".join(m.astype("<f4").tobytes() for m in mats))  # linear1, linear3, linear2
    g, u, dn = checkpoint.read_dense_mlp(f, d, dff)
    G, U, D = checkpoint.upcycle_dense(g, u, dn, E)
    assert G.shape == (E, dff, d) and D.shape == (E, d, dff)
    for e in range(E):
        np.testing.assert_array_equal(G[e], mats[0])
        np.testing.assert_array_equal(U[e], mats[1])
        np.testing.assert_array_equal(D[e], mats[2])


@pytest.mark.gpu
def test_save_load_round_trip_on_gpu():
    from omega_ai_b200 import MoELayer
    a = MoELayer(128, 256, 8, 2, bias=True, t_max=64, compute_dtype=torch.bfloat16, keep_weights=True)
    a.initParam(seed=5)
    x = torch.randn(64, 128, device="cuda").to(torch.bfloat16)
    ya = a.forward_device(x).clone()
    f = io.BytesIO()
    a.saveModel(f)
    assert len(f.getvalue()) == 4 * (8 * 128 + 8 + 8 * 3 * 128 * 256)
    f.seek(0)
    b = MoELayer(128, 256, 8, 2, bias=True, t_max=64, compute_dtype=torch.bfloat16)
    b.loadModel(f)
    assert torch.equal(b.forward_device(x), ya)
    a.close()
    b.close()
