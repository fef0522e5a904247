"""ctypes front end of ``oracle/refk_driver.cu``: the REFERENCE's own CUDA kernels (softmax, SiLU,
element-wise product, RMSNorm — compiled from the reference's source files into ``oracle/_ref/*.cubin``)
plus cuBLAS SGEMM, started the way the reference's Java wrappers start them.

TEST INFRASTRUCTURE ONLY.  It pins the CPU oracle (and through it the product) to what the reference
itself computes for the stages it has, and gives the "reference kernels on this GPU" baseline.  The
cubins are built where the reference checkout is present (``make -C oracle ref_kernels``) and travel
with the tree; a machine without them reports ``available() == False`` and the tests skip.

All tensors are contiguous float32 CUDA tensors; every call runs on the null stream, as the reference does.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_REF_DIR = os.path.join(_HERE, "_ref")
_LIB_PATH = os.path.join(_HERE, "librefk.so")
_CUBINS = ("SoftmaxKernel.cubin", "activeFunction.cubin", "OPKernel.cubin", "RMSKernel.cubin")
_lib = None


def available() -> bool:
    return os.path.exists(_LIB_PATH) and all(os.path.exists(os.path.join(_REF_DIR, f)) for f in _CUBINS)


def _check(rc):
    if rc != 0:
        raise RuntimeError("reference-kernel driver: " + _lib.refk_error().decode())


def lib():
    global _lib
    if _lib is None:
        if not available():
            raise RuntimeError("oracle/_ref cubins or librefk.so missing: run `make -C oracle ref_kernels` "
                               "where the reference checkout is present")
        torch.cuda.init()
        _lib = C.CDLL(_LIB_PATH)
        _lib.refk_error.restype = C.c_char_p
        _check(_lib.refk_init(_REF_DIR.encode()))
    return _lib


def _p(t: torch.Tensor):
    assert t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()
    return C.c_void_p(t.data_ptr())


def softmax(x: torch.Tensor) -> torch.Tensor:
    """Rows of ``x`` [rows, n] through the reference's `softmax` kernel (SoftmaxKernel.cu:5)."""
    out = torch.empty_like(x)
    _check(lib().refk_softmax(_p(x), _p(out), x.shape[0], x.shape[1]))
    return out


def silu(x: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(x)
    _check(lib().refk_silu(_p(x), _p(out), x.numel()))
    return out


def silu_backward(x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    diff = torch.empty_like(x)
    _check(lib().refk_silu_backward(_p(x), _p(x), _p(delta), _p(diff), x.numel()))
    return diff


def softmax_back(out: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    diff = torch.empty_like(out)
    _check(lib().refk_softmax_back(_p(out), _p(delta), _p(diff), out.shape[0], out.shape[1]))
    return diff


def mul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(a)
    _check(lib().refk_mul(_p(a), _p(b), _p(out), a.numel()))
    return out


def rmsnorm(x: torch.Tensor, gamma: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(x)
    _check(lib().refk_rmsnorm(_p(out), _p(x), _p(gamma), x.shape[0], x.shape[1]))
    return out


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x`` [rows, in] times ``w`` [out, in] transposed: FullyLayer.output()'s cublasSgemm call."""
    y = torch.empty(x.shape[0], w.shape[0], dtype=torch.float32, device=x.device)
    _check(lib().refk_linear(_p(x), _p(w), _p(y), x.shape[0], x.shape[1], w.shape[0]))
    return y


class MlpScratch:
    """linear1 output, SiLU output, linear3 output and product, kept as the reference keeps them."""

    def __init__(self, rows: int, dff: int, device="cuda"):
        self.g, self.a, self.u, self.tmp = (torch.empty(rows, dff, dtype=torch.float32, device=device)
                                            for _ in range(4))


def mlp(x, w1, w3, w2, scratch: MlpScratch | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """LlamaMLPLayer.output(): linear1 -> SiLU -> linear3 -> product -> linear2 on ``x`` [rows, d]."""
    rows, d = x.shape
    dff = w1.shape[0]
    s = scratch or MlpScratch(rows, dff, x.device)
    y = out if out is not None else torch.empty(rows, d, dtype=torch.float32, device=x.device)
    _check(lib().refk_mlp(_p(x), _p(w1), _p(w3), _p(w2), _p(s.g), _p(s.a), _p(s.u), _p(s.tmp), _p(y), rows, d, dff))
    return y
