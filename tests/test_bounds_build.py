"""The bounds-checked debug build (libhearth_b200_bounds.so, -DHB200_BOUNDS): the streaming kernels compare every
global-memory index they compute with the extent of its buffer, skip an access outside it and count it, and
hb200_check_status reports the count.  It stands in for compute-sanitizer's memcheck, which is not available here.

CPU part: the library builds, loads and says what it is.  GPU part: the parity tests with ragged shapes, cut panels and
every K-quant token count run again in a child process on that library; any counted access fails the run (the `hb`
fixture ends with hb200_check_status), and so does any result that differs from the oracle."""
import ctypes as C
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def bounds_lib():
    from hearth_b200 import build
    return build.build_bounds()


def test_bounds_library_builds_and_identifies_itself():
    from hearth_b200 import build
    path = bounds_lib()
    assert os.path.exists(path)
    dbg = C.CDLL(path)
    dbg.hb200_bounds_checked.restype = C.c_int
    assert dbg.hb200_bounds_checked() == 1
    normal = C.CDLL(build.build())
    normal.hb200_bounds_checked.restype = C.c_int
    assert normal.hb200_bounds_checked() == 0
    # the same C ABI: every symbol the Python binding declares is exported by the debug build too
    from hearth_b200 import lib as L
    for name in L.SIGNATURES:
        assert hasattr(dbg, name), name


@pytest.mark.gpu
def test_parity_tests_pass_on_the_bounds_checked_build():
    env = dict(os.environ, HB200_LIB=bounds_lib())
    cmd = [sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu", "-p", "no:cacheprovider",
           os.path.join(ROOT, "tests", "test_gpu_parity.py"), os.path.join(ROOT, "tests", "test_gpu_batch_paths.py"),
           os.path.join(ROOT, "tests", "test_gpu_producers.py"),
           "-k", "kquant or cut_panels or quantize or dot_rows or row_split or batch or producers or rms or silu or hadamard"]
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=1200)
    tail = (p.stdout + p.stderr)[-3000:]
    assert p.returncode == 0, tail
    assert " passed" in p.stdout and "error" not in p.stdout.lower().split("passed")[-1], tail


@pytest.mark.gpu
def test_bounds_checks_count_and_skip_an_out_of_range_index():
    """The mechanism itself: a launch whose pitch is too small on purpose (the buffers are not) must report exactly the
    accesses beyond it; the normal build refuses the self-test."""
    code = ("from hearth_b200 import api, lib; api.init(0); l = lib.load(); "
            "assert l.hb200_bounds_checked() == 1; rc = l.hb200_bounds_selftest(); "
            "assert rc == 0, (rc, lib.last_error()); api.check_status(); print('selftest ok')")
    p = subprocess.run([sys.executable, "-c", code], cwd=ROOT, env=dict(os.environ, HB200_LIB=bounds_lib()),
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and "selftest ok" in p.stdout, (p.stdout + p.stderr)[-2000:]
    from hearth_b200 import lib
    assert lib.load().hb200_bounds_selftest() == -7  # HB200_ERR_UNSUPPORTED in the normal build
