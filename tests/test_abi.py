"""CPU tests of the boundary: the library loads, exports what the header declares, and fails loudly."""
import ctypes as C
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "omoe.h")


@pytest.fixture(scope="module")
def native():
    from omega_ai_b200 import native as n

    n.build()
    return n


def header_symbols():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"OMOE_API\s+[\w\s\*]*?\b(omoe_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(native):
    lib = C.CDLL(native.LIB_PATH)
    declared = header_symbols()
    assert len(declared) >= 13
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in omoe.h but not exported"
    assert sorted(native.SYMBOLS) == declared  # the ctypes binding covers the whole header


def test_library_has_no_link_time_gpu_driver_dependency(native):
    out = subprocess.run(["ldd", native.LIB_PATH], capture_output=True, text=True).stdout
    assert "libcuda.so" not in out and "libnccl" not in out and "libtorch" not in out


def test_config_struct_layout_matches_c(native, tmp_path):
    src = tmp_path / "sz.c"
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "omoe.h"\n'
                   'int main(){printf("%zu %zu %zu", sizeof(omoe_config), offsetof(omoe_config, world), '
                   'offsetof(omoe_config, reserved));return 0;}')
    exe = tmp_path / "sz"
    subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    size, off_world, off_res = map(int, subprocess.check_output([str(exe)]).split())
    assert size == C.sizeof(native.Config)
    assert off_world == native.Config.world.offset and off_res == native.Config.reserved.offset


def test_bad_arguments_return_codes_without_a_gpu(native):
    lib = native.lib()
    h = C.c_void_p()
    assert lib.omoe_create(None, C.byref(h)) == -1
    cfg = native.Config(t_max=16, d_model=130, d_ff=256, n_experts=8, top_k=2, compute_dtype=1, renormalize=1,
                        world=1, rank=0)
    assert lib.omoe_create(C.byref(cfg), C.byref(h)) == -1 and b"multiples of 8" in lib.omoe_last_error(None)
    cfg.d_model = 128
    cfg.top_k = 9
    assert lib.omoe_create(C.byref(cfg), C.byref(h)) == -1
    cfg.top_k = 2
    cfg.world, cfg.rank = 3, 0  # 8 experts do not split over 3 ranks
    assert lib.omoe_create(C.byref(cfg), C.byref(h)) == -1
    assert lib.omoe_forward(None, None, None, 1, 0, None) == -1
    # the training and multi-GPU entries refuse a null handle the same way
    assert lib.omoe_set_training(None, 1) == -1
    assert lib.omoe_backward(None, None, None, None, 1, 0, None) == -1
    assert lib.omoe_backward_block(None, None, None, 1e-5, None, None, None, 1, 0, None) == -1
    assert lib.omoe_get_weight_grads(None, None, None, None, None, None, None) == -1
    assert lib.omoe_set_aux_loss(None, 0.5) == -1
    assert lib.omoe_get_aux_loss(None, None) == -1
    assert lib.omoe_ep_connect_local(None, 2) == -1
    two = (C.c_void_p * 2)(None, None)
    assert lib.omoe_ep_connect_local(two, 2) == -1 and lib.omoe_ep_connect_local(two, 9) == -1
    assert lib.omoe_destroy(None) == 0


def test_create_fails_loudly_without_a_b200(native):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = native.lib()
    h = C.c_void_p()
    cfg = native.Config(t_max=16, d_model=128, d_ff=256, n_experts=8, top_k=2, compute_dtype=1, renormalize=1,
                        world=1, rank=0)
    rc = lib.omoe_create(C.byref(cfg), C.byref(h))
    assert rc < 0 and not h.value  # no silent CPU path
    assert lib.omoe_last_error(None)


def test_host_mirror_refuses_to_run_without_the_library(native, monkeypatch):
    monkeypatch.setattr(native, "LIB_PATH", os.path.join(ROOT, "does_not_exist.so"))
    monkeypatch.setattr(native, "_lib", None)
    with pytest.raises(ImportError):
        native.lib()


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "omega_ai_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text and "moe_ref" not in text, f"{f} mentions the oracle"
