"""A few steps of plain gradient descent through the C ABI: training-mode forward, backward, weight update by the
host (as the engine's updaters would do on the FullyLayers' diffW), weights handed back with setWeights.  The loss
of a small regression problem has to fall: signs and scales of every gradient are right together."""
import numpy as np
import pytest
import torch

from helpers import make_layer

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("compute", [torch.float32, torch.bfloat16])
def test_gradient_descent_lowers_the_loss(compute):
    from omega_ai_b200 import MoELayer
    T, d, dff, E, k = 256, 64, 128, 8, 2
    x, w_r, w_g, w_u, w_d, _ = make_layer(T, d, dff, E, k, seed=41)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()
    # master weights in fp32 on the host side of the boundary; the library gets (rounded) copies every step
    W = dict(r=dev(w_r * 5), g=dev(w_g * 5), u=dev(w_u * 5), dn=dev(w_d * 5))
    xd = dev(x).to(compute)
    gen = torch.Generator(device="cuda").manual_seed(7)
    target = (xd.float() @ (torch.randn(d, d, device="cuda", generator=gen) * 0.2)).contiguous()
    layer = MoELayer(d, dff, E, k, t_max=T, compute_dtype=compute)
    layer.set_training(True)
    lr, losses = 0.05, []
    for step in range(40):
        layer.setWeights(*(W[n].to(compute).contiguous() for n in ("r", "g", "u", "dn")))
        y = layer.forward_device(xd).float()
        diff = y - target
        losses.append(float((diff * diff).mean()))
        dy = (2.0 / diff.numel() * diff).to(compute).contiguous()
        layer.backward(xd, dy)
        g = layer.weight_grads()
        for n, gn in (("r", "d_router"), ("g", "d_gate"), ("u", "d_up"), ("dn", "d_down")):
            W[n] -= lr * T * g[gn]   # the mean over T*d elements makes the raw gradients tiny; scale the step
    assert all(np.isfinite(losses))
    assert losses[-1] < 0.7 * losses[0], losses[::8]
    layer.close()
