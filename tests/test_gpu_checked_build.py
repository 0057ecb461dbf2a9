"""The index-checked build of the library (-DRWKV7_CHECKED -DRWKV7_NVTX): device code verifies tile rows, output
rows and workspace slots before using them and reports a bad one through the status word instead of performing
the access.  A child process loads that build, runs small parity cases of every WKV7 path with all outputs
and the workspace between canary pads, and checks results, canaries and the status word."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CHECKED = os.path.join(ROOT, "rwkv-rs-stable_b200", "librwkv7_b200_checked.so")


@pytest.mark.gpu
def test_parity_cases_on_the_checked_build_with_canaries():
    assert os.path.exists(CHECKED), "build it with __graft_entry__.build()"
    env = dict(os.environ, RWKV7_B200_LIB=CHECKED)
    res = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "checked_child.py")], env=env,
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "CHECKED_BUILD_OK" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]


def test_build_features_flag():
    """The product build carries neither instrumentation; the checked variant carries both."""
    import ctypes
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    assert entry.load_package().lib().rwkv7_build_features() == 0
    if os.path.exists(CHECKED):
        assert ctypes.CDLL(CHECKED).rwkv7_build_features() == 3
