"""The small configurations under the self-checking build (libomoe_check.so, -DOMOE_BOUNDS_CHECK): NaN-filled
workspaces, device-side validation of every routing index and of the untouched padding rows, and every
intermediate compared with the oracle.  Stands in for a memory checker.  Runs in a child process because the
library build is chosen when the package is first imported."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_small_configs_under_the_self_checking_build():
    from omega_ai_b200 import native
    if not os.path.exists(native.CHECK_LIB_PATH):
        native.build(check=True)
    env = dict(os.environ, OMOE_LIB=native.CHECK_LIB_PATH)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "self_check_worker.py")], capture_output=True,
                       text=True, timeout=900, env=env, cwd=ROOT)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert "self-check ok" in p.stdout
