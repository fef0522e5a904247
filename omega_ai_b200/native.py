"""ctypes binding of ``libomoe.so`` — the C ABI declared in ``include/omoe.h``.

This is the same binding a Java host would make through JNI or the FFM API:
plain integers, raw device addresses and a config struct.  There is no CPU
fallback: if the shared library is missing the import of :func:`lib` raises.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

_PKG = os.path.dirname(os.path.abspath(__file__))
# OMOE_LIB selects another build of the same ABI, e.g. the self-checking one (libomoe_check.so, csrc/check.cu)
LIB_PATH = os.environ.get("OMOE_LIB") or os.path.join(_PKG, "libomoe.so")
CHECK_LIB_PATH = os.path.join(_PKG, "libomoe_check.so")
CSRC = os.path.join(_PKG, "csrc")

OMOE_F32 = 0
OMOE_BF16 = 1
N_STAGES = 8
STAGE_NAMES = ("router", "scan", "permute", "dispatch", "up_gate", "down", "return", "combine")
EP_BLOB_BYTES = 320

ERRORS = {
    0: "OMOE_OK", -1: "OMOE_ERR_INVALID", -2: "OMOE_ERR_CUDA", -3: "OMOE_ERR_TOO_LARGE",
    -4: "OMOE_ERR_STATE", -5: "OMOE_ERR_UNSUPPORTED", -6: "OMOE_ERR_DEVICE", -7: "OMOE_ERR_COMM",
    -8: "OMOE_ERR_NOMEM",
}

# every symbol include/omoe.h declares
SYMBOLS = (
    "omoe_create", "omoe_destroy", "omoe_last_error", "omoe_set_weights", "omoe_forward",
    "omoe_forward_host", "omoe_forward_host_async", "omoe_wait", "omoe_forward_block", "omoe_get_routing", "omoe_get_logits", "omoe_last_launch_count",
    "omoe_set_profiling", "omoe_get_stage_ms", "omoe_get_stage_ms_at", "omoe_ep_export", "omoe_ep_import",
    "omoe_route_noalloc", "omoe_route_noalloc_error",
    "omoe_ep_connect_local", "omoe_set_training", "omoe_backward", "omoe_backward_block", "omoe_get_weight_grads", "omoe_set_aux_loss", "omoe_get_aux_loss",
)
NOALLOC_MAX_TOKENS = 4096


class OmoeError(RuntimeError):
    """Raised for any non-zero status; mirrors the RuntimeException thrown by
    CUDAManager.checkCUDA in the reference (CUDAManager.java:118-123)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"{ERRORS.get(code, code)}: {message}")
        self.code = code


class Config(C.Structure):
    _fields_ = [
        ("t_max", C.c_int32), ("d_model", C.c_int32), ("d_ff", C.c_int32), ("n_experts", C.c_int32),
        ("top_k", C.c_int32), ("compute_dtype", C.c_int32), ("renormalize", C.c_int32),
        ("has_router_bias", C.c_int32), ("world", C.c_int32), ("rank", C.c_int32),
        ("recv_rows_max", C.c_int32), ("reserved", C.c_int32 * 5),
    ]


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".sh"))) + [
        os.path.join(os.path.dirname(_PKG), "include", "omoe.h")
    ]


def build(force: bool = False, check: bool = False) -> str:
    """Compile ``libomoe.so`` for sm_100a with nvcc (cross-compiles without a GPU); with ``check`` the
    self-checking variant ``libomoe_check.so`` (-DOMOE_BOUNDS_CHECK)."""
    path = CHECK_LIB_PATH if check else os.path.join(_PKG, "libomoe.so")
    stale = (not os.path.exists(path)) or any(os.path.getmtime(s) > os.path.getmtime(path) for s in sources())
    if force or stale:
        subprocess.check_call(["sh", os.path.join(CSRC, "build.sh")] + (["check"] if check else []))
    return path


_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with omega_ai_b200.native.build() "
            "(nvcc, sm_100a).  There is no CPU fallback for this layer."
        )
    L = C.CDLL(LIB_PATH)
    vp, i32 = C.c_void_p, C.c_int32
    L.omoe_create.argtypes = [C.POINTER(Config), C.POINTER(vp)]
    L.omoe_destroy.argtypes = [vp]
    L.omoe_last_error.argtypes = [vp]
    L.omoe_last_error.restype = C.c_char_p
    L.omoe_set_weights.argtypes = [vp, vp, vp, vp, vp, vp, i32, vp]
    L.omoe_forward.argtypes = [vp, vp, vp, i32, i32, vp]
    L.omoe_forward_host.argtypes = [vp, vp, vp, i32, i32, vp]
    L.omoe_forward_host_async.argtypes = [vp, vp, vp, i32, i32, vp]
    L.omoe_wait.argtypes = [vp]
    L.omoe_forward_block.argtypes = [vp, vp, vp, C.c_float, vp, i32, i32, vp]
    L.omoe_get_routing.argtypes = [vp, vp, vp, vp, vp, vp]
    L.omoe_get_logits.argtypes = [vp, vp]
    L.omoe_last_launch_count.argtypes = [vp]
    L.omoe_set_profiling.argtypes = [vp, i32]
    L.omoe_get_stage_ms.argtypes = [vp, vp]
    L.omoe_get_stage_ms_at.argtypes = [vp, i32, vp]
    L.omoe_ep_export.argtypes = [vp, vp]
    L.omoe_ep_import.argtypes = [vp, vp]
    L.omoe_route_noalloc.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp]
    L.omoe_ep_connect_local.argtypes = [C.POINTER(vp), i32]
    L.omoe_set_training.argtypes = [vp, i32]
    L.omoe_backward.argtypes = [vp, vp, vp, vp, i32, i32, vp]
    L.omoe_backward_block.argtypes = [vp, vp, vp, C.c_float, vp, vp, vp, i32, i32, vp]
    L.omoe_get_weight_grads.argtypes = [vp, vp, vp, vp, vp, vp, vp]
    L.omoe_set_aux_loss.argtypes = [vp, C.c_float]
    L.omoe_get_aux_loss.argtypes = [vp, C.POINTER(C.c_float)]
    L.omoe_route_noalloc_error.argtypes = []
    L.omoe_route_noalloc_error.restype = C.c_char_p
    for name in SYMBOLS:
        if name not in ("omoe_last_error", "omoe_route_noalloc_error"):
            getattr(L, name).restype = C.c_int
    _lib = L
    return L


def check(handle, rc: int):
    if rc != 0:
        msg = lib().omoe_last_error(handle)
        raise OmoeError(rc, msg.decode() if msg else "")
