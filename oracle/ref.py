"""ctypes front end of the CPU oracle (``oracle/moe_ref.c``).

TEST INFRASTRUCTURE ONLY: imported by the tests, by the smoke check and by the
benchmark's CPU-baseline leg, never by the product package.  Parity: the stages
the reference has (softmax, SiLU, product, RMSNorm, X*W^T, the dense SwiGLU
sequence) are pinned to the reference's own kernels (``oracle/refk.py``); PARITY
UNPINNED for the routing rules the reference lacks — see the header of ``moe_ref.h``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libmoe_ref.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file."""
    src = [os.path.join(_HERE, f) for f in ("moe_ref.c", "moe_ref.h", "Makefile")]
    stale = (not os.path.exists(_LIB_PATH)) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in src
    )
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-s"] + (["-B"] if force else []))
    return _LIB_PATH


class _Shape(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("T", "d", "dff", "E", "k", "renorm", "bf16", "out_bf16", "pretransposed")]


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        fp, ip = C.POINTER(C.c_float), C.POINTER(C.c_int32)
        i64 = C.c_int64
        _lib.ref_bf16_round.restype = C.c_float
        _lib.ref_bf16_round.argtypes = [C.c_float]
        _lib.ref_bf16_round_array.argtypes = [fp, i64]
        _lib.ref_silu.argtypes = [fp, fp, i64]
        _lib.ref_linear_nt.argtypes = [fp, fp, fp, i64, i64, i64]
        _lib.ref_softmax_rows.argtypes = [fp, fp, i64, i64]
        _lib.ref_rmsnorm_rows.argtypes = [fp, fp, C.c_float, i64, i64, C.c_int, fp]
        _lib.ref_router_logits.argtypes = [fp, fp, fp, i64, i64, i64, fp]
        _lib.ref_topk_gate.argtypes = [fp, i64, i64, i64, C.c_int, ip, fp]
        _lib.ref_histogram_permute.argtypes = [ip, i64, i64, i64, ip, ip, ip, ip]
        _lib.ref_moe_forward.argtypes = [
            C.POINTER(_Shape), fp, fp, fp, fp, fp, fp, fp, ip, fp, ip, ip, ip, ip, i64, fp, C.c_int,
        ]
        _lib.ref_rmsnorm_backward_rows.argtypes = [fp, fp, C.c_float, fp, i64, i64, fp, fp]
        _lib.ref_silu_backward.argtypes = [fp, fp, fp, i64]
        _lib.ref_softmax_back_rows.argtypes = [fp, fp, fp, i64, i64]
        _lib.ref_moe_backward.argtypes = [C.POINTER(_Shape)] + [fp] * 7 + [C.c_float] + [fp] * 6 + [C.c_int]
        _lib.ref_aux_loss.argtypes = [fp, ip, i64, i64, i64]
        _lib.ref_aux_loss.restype = C.c_float
        _lib.ref_num_threads.restype = C.c_int
    return _lib


def _f(a):
    return None if a is None else a.ctypes.data_as(C.POINTER(C.c_float))


def _i(a):
    return None if a is None else a.ctypes.data_as(C.POINTER(C.c_int32))


def _cf(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def num_threads() -> int:
    return int(lib().ref_num_threads())


def bf16_round(a: np.ndarray) -> np.ndarray:
    out = _cf(a).copy()
    lib().ref_bf16_round_array(_f(out), out.size)
    return out


def silu(x: np.ndarray) -> np.ndarray:
    x = _cf(x)
    out = np.empty_like(x)
    lib().ref_silu(_f(x), _f(out), x.size)
    return out


def linear_nt(X: np.ndarray, W: np.ndarray) -> np.ndarray:
    X, W = _cf(X), _cf(W)
    m, k = X.shape
    n = W.shape[0]
    Y = np.empty((m, n), np.float32)
    lib().ref_linear_nt(_f(X), _f(W), _f(Y), m, n, k)
    return Y


def softmax_rows(x: np.ndarray) -> np.ndarray:
    x = _cf(x)
    out = np.empty_like(x)
    lib().ref_softmax_rows(_f(x), _f(out), x.shape[0], x.shape[1])
    return out


def rmsnorm(x, gamma, eps: float = 1e-5, bf16: bool = False) -> np.ndarray:
    x, gamma = _cf(x), _cf(gamma)
    out = np.empty_like(x)
    lib().ref_rmsnorm_rows(_f(x), _f(gamma), eps, x.shape[0], x.shape[1], int(bf16), _f(out))
    return out


def moe_block(x, gamma, w_r, w_gate, w_up, w_down, k: int, *, eps=1e-5, bias=None, renorm=True, bf16=False,
              out_bf16=None, sel=None) -> "MoEResult":
    """y = x + MoE(rmsnorm(x) * gamma): norm2 -> mlp -> residual add of the transformer block
    (LlamaTransformerBlock.java:134-136).  The sum x + (combined rows) is formed in fp32 and rounded once."""
    x = _cf(x)
    if out_bf16 is None:
        out_bf16 = bf16
    xn = rmsnorm(x, gamma, eps, bf16)
    r = moe_forward(xn, w_r, w_gate, w_up, w_down, k, bias=bias, renorm=renorm, bf16=bf16, out_bf16=False, sel=sel)
    rows = x if sel is None else x[np.asarray(sel)]
    y = rows + r.y
    r.y = bf16_round(y) if out_bf16 else y
    return r


def router_logits(x, w_r, bias=None) -> np.ndarray:
    x, w_r = _cf(x), _cf(w_r)
    bias = None if bias is None else _cf(bias)
    T, d = x.shape
    E = w_r.shape[0]
    out = np.empty((T, E), np.float32)
    lib().ref_router_logits(_f(x), _f(w_r), _f(bias), T, d, E, _f(out))
    return out


def topk_gate(logits, k: int, renorm: bool = True):
    logits = _cf(logits)
    T, E = logits.shape
    idx = np.empty((T, k), np.int32)
    w = np.empty((T, k), np.float32)
    lib().ref_topk_gate(_f(logits), T, E, k, int(renorm), _i(idx), _f(w))
    return idx, w


def histogram_permute(topk_idx, E: int):
    topk_idx = np.ascontiguousarray(topk_idx, dtype=np.int32)
    T, k = topk_idx.shape
    counts = np.empty(E, np.int32)
    offsets = np.empty(E + 1, np.int32)
    perm = np.empty(T * k, np.int32)
    pos = np.empty(T * k, np.int32)
    lib().ref_histogram_permute(_i(topk_idx), T, E, k, _i(counts), _i(offsets), _i(perm), _i(pos))
    return counts, offsets, perm, pos


@dataclass
class MoEResult:
    logits: np.ndarray
    topk_idx: np.ndarray
    topk_w: np.ndarray
    counts: np.ndarray
    offsets: np.ndarray
    perm: np.ndarray
    y: np.ndarray | None
    sel: np.ndarray | None


def moe_forward(x, w_r, w_gate, w_up, w_down, k: int, *, bias=None, renorm=True, bf16=False,
                out_bf16=None, sel=None, compute_y=True, nthreads: int = 0,
                pretransposed=False) -> MoEResult:
    """Whole layer on the CPU.

    ``w_r`` [E,d]; ``w_gate``/``w_up`` [E,dff,d]; ``w_down`` [E,d,dff] — all
    [out,in] row-major as the reference's FullyLayer stores weights.  With
    ``bf16`` the expert weights are rounded to bf16 here (the router keeps the
    values it is given) and the bf16 rounding points of the tensor-core path
    apply.  ``sel`` restricts the expert products to those token indices.
    """
    x, w_r = _cf(x), _cf(w_r)
    w_gate, w_up, w_down = _cf(w_gate), _cf(w_up), _cf(w_down)
    if bf16:
        w_gate, w_up, w_down = bf16_round(w_gate), bf16_round(w_up), bf16_round(w_down)
    bias = None if bias is None else _cf(bias)
    T, d = x.shape
    if pretransposed:  # [in,out] layouts: gate/up [E,d,dff], down [E,dff,d]
        E, _, dff = w_gate.shape
        assert w_r.shape == (E, d) and w_up.shape == (E, d, dff) and w_down.shape == (E, dff, d)
    else:
        E, dff, _ = w_gate.shape
        assert w_r.shape == (E, d) and w_up.shape == (E, dff, d) and w_down.shape == (E, d, dff)
    if out_bf16 is None:
        out_bf16 = bf16
    shp = _Shape(T, d, dff, E, k, int(renorm), int(bf16), int(out_bf16), int(pretransposed))
    logits = np.empty((T, E), np.float32)
    idx = np.empty((T, k), np.int32)
    w = np.empty((T, k), np.float32)
    counts = np.empty(E, np.int32)
    offsets = np.empty(E + 1, np.int32)
    perm = np.empty(T * k, np.int32)
    sel_a = None if sel is None else np.ascontiguousarray(sel, dtype=np.int32)
    n_sel = T if sel_a is None else sel_a.size
    y = np.empty((n_sel, d), np.float32) if compute_y else None
    lib().ref_moe_forward(C.byref(shp), _f(x), _f(w_r), _f(bias), _f(w_gate), _f(w_up), _f(w_down),
                          _f(logits), _i(idx), _f(w), _i(counts), _i(offsets), _i(perm),
                          _i(sel_a), n_sel, _f(y), nthreads)
    return MoEResult(logits, idx, w, counts, offsets, perm, y, sel_a)


def silu_backward(x: np.ndarray, delta: np.ndarray) -> np.ndarray:
    x, delta = _cf(x), _cf(delta)
    out = np.empty_like(x)
    lib().ref_silu_backward(_f(x), _f(delta), _f(out), x.size)
    return out


def softmax_back_rows(out: np.ndarray, delta: np.ndarray) -> np.ndarray:
    out, delta = _cf(out), _cf(delta)
    diff = np.empty_like(out)
    lib().ref_softmax_back_rows(_f(out), _f(delta), _f(diff), out.shape[0], out.shape[1])
    return diff


@dataclass
class MoEGrads:
    dx: np.ndarray
    d_w_r: np.ndarray
    d_bias: np.ndarray
    d_w_gate: np.ndarray
    d_w_up: np.ndarray
    d_w_down: np.ndarray


def aux_loss(logits: np.ndarray, counts: np.ndarray, k: int) -> float:
    """E * sum_e (counts[e]/(T*k)) * mean_t softmax(logits)[t,e]."""
    logits = _cf(logits)
    counts = np.ascontiguousarray(counts, dtype=np.int32)
    return float(lib().ref_aux_loss(_f(logits), _i(counts), logits.shape[0], logits.shape[1], k))


def moe_backward(x, w_r, w_gate, w_up, w_down, k: int, dy, *, bias=None, renorm=True, bf16=False,
                 out_bf16=None, aux_coef: float = 0.0, nthreads: int = 0) -> MoEGrads:
    """Gradients of the whole layer for ``dy`` [T,d]; same conventions as :func:`moe_forward`."""
    x, w_r, dy = _cf(x), _cf(w_r), _cf(dy)
    w_gate, w_up, w_down = _cf(w_gate), _cf(w_up), _cf(w_down)
    if bf16:
        w_gate, w_up, w_down = bf16_round(w_gate), bf16_round(w_up), bf16_round(w_down)
    bias = None if bias is None else _cf(bias)
    T, d = x.shape
    E, dff, _ = w_gate.shape
    assert dy.shape == (T, d) and w_r.shape == (E, d) and w_up.shape == (E, dff, d) and w_down.shape == (E, d, dff)
    if out_bf16 is None:
        out_bf16 = bf16
    shp = _Shape(T, d, dff, E, k, int(renorm), int(bf16), int(out_bf16), 0)
    g = MoEGrads(np.empty((T, d), np.float32), np.empty((E, d), np.float32), np.empty(E, np.float32),
                 np.empty((E, dff, d), np.float32), np.empty((E, dff, d), np.float32),
                 np.empty((E, d, dff), np.float32))
    lib().ref_moe_backward(C.byref(shp), _f(x), _f(w_r), _f(bias), _f(w_gate), _f(w_up), _f(w_down), _f(dy), float(aux_coef),
                           _f(g.dx), _f(g.d_w_r), _f(g.d_bias), _f(g.d_w_gate), _f(g.d_w_up), _f(g.d_w_down),
                           nthreads)
    return g


def rmsnorm_backward(x, gamma, dout, eps: float = 1e-5):
    """(dinp [T,d], dgamma [d]) of out = (x / rms(x)) * gamma for a given dout."""
    x, gamma, dout = _cf(x), _cf(gamma), _cf(dout)
    dinp, dgamma = np.empty_like(x), np.empty_like(gamma)
    lib().ref_rmsnorm_backward_rows(_f(x), _f(gamma), eps, _f(dout), x.shape[0], x.shape[1], _f(dinp), _f(dgamma))
    return dinp, dgamma


def moe_block_backward(x, gamma, w_r, w_gate, w_up, w_down, k: int, dy, *, eps=1e-5, bias=None, renorm=True,
                       bf16=False, out_bf16=None):
    """Backward of y = x + MoE(rmsnorm(x) * gamma): (dx, dgamma, MoEGrads of the layer on the normalised rows).
    bf16 mode rounds where the GPU path stores bf16: the normalised rows, and (with out_bf16) the gradient of
    the normalised rows and dx."""
    if out_bf16 is None:
        out_bf16 = bf16
    xn = rmsnorm(x, gamma, eps, bf16=bf16)
    g = moe_backward(xn, w_r, w_gate, w_up, w_down, k, dy, bias=bias, renorm=renorm, bf16=bf16, out_bf16=out_bf16)
    dinp, dgamma = rmsnorm_backward(x, gamma, g.dx, eps)
    dx = (_cf(dy) + dinp).astype(np.float32)
    if out_bf16:
        dx = bf16_round(dx)
    return dx, dgamma, g
