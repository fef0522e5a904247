"""Weight files in the engine's checkpoint convention.

The reference stores parameters as a headerless stream of little-endian
float32 values, tensors in a fixed order (network/utils/ModelUtils.java:237-278:
``writeFloatArray`` emits the four bytes of ``Float.floatToIntBits`` low byte
first).  A ``FullyLayer`` writes its weight ``[out, in]`` and then its bias if
it has one (FullyLayer.java:854-866); ``LlamaMLPLayer`` writes linear1 (gate),
linear3 (up), linear2 (down) (LlamaMLPLayer.java:273-277).

The MoE layer keeps that convention: router (weight, then bias if present),
then for every expert gate, up, down.
"""
from __future__ import annotations

import numpy as np

LE_F32 = np.dtype("<f4")


def _write(f, a):
    f.write(np.ascontiguousarray(a, dtype=np.float32).astype(LE_F32, copy=False).tobytes())


def _read(f, shape):
    n = int(np.prod(shape))
    buf = f.read(4 * n)
    if len(buf) != 4 * n:
        raise EOFError(f"checkpoint ends early: wanted {4 * n} bytes, got {len(buf)}")
    return np.frombuffer(buf, dtype=LE_F32).astype(np.float32).reshape(shape)


def write_moe(f, w_router, router_bias, w_gate, w_up, w_down):
    """router [E,d] (+ bias [E]), then per expert gate [dff,d], up [dff,d], down [d,dff]."""
    _write(f, w_router)
    if router_bias is not None:
        _write(f, router_bias)
    for e in range(w_gate.shape[0]):
        _write(f, w_gate[e])
        _write(f, w_up[e])
        _write(f, w_down[e])


def read_moe(f, n_experts, d_model, d_ff, has_bias=False):
    w_router = _read(f, (n_experts, d_model))
    bias = _read(f, (n_experts,)) if has_bias else None
    w_gate = np.empty((n_experts, d_ff, d_model), np.float32)
    w_up = np.empty((n_experts, d_ff, d_model), np.float32)
    w_down = np.empty((n_experts, d_model, d_ff), np.float32)
    for e in range(n_experts):
        w_gate[e] = _read(f, (d_ff, d_model))
        w_up[e] = _read(f, (d_ff, d_model))
        w_down[e] = _read(f, (d_model, d_ff))
    return w_router, bias, w_gate, w_up, w_down


def read_dense_mlp(f, d_model, d_ff):
    """One dense ``LlamaMLPLayer`` (no biases): linear1 = gate, linear3 = up, linear2 = down."""
    return _read(f, (d_ff, d_model)), _read(f, (d_ff, d_model)), _read(f, (d_model, d_ff))


def upcycle_dense(gate, up, down, n_experts):
    """Every expert starts as a copy of a dense SwiGLU MLP (sparse upcycling)."""
    rep = lambda a: np.ascontiguousarray(np.broadcast_to(a, (n_experts,) + a.shape))
    return rep(gate), rep(up), rep(down)
