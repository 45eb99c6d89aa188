"""The bounds-check build (`python vearo_b200/build.py --bounds-check`, -DVB200_BOUNDS_CHECK) on the small-shape op tests.

On pools where no memory checker may run, this build is the stand-in: kernels that compute gather / scatter indices verify
them (VB_BC in csrc/common.h); an index outside its tensor sets a bit of the device error word -- it never traps or faults --
and `vb_check_errors`, which every parity test calls, turns it into a failure.  The child process runs the convolution,
pooling, reduction, embedding and attention tests against that library through VB200_LIB.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_small_shape_ops_under_the_bounds_check_build():
    lib = os.path.join(ROOT, "vearo_b200", "libvearo_b200_bc.so")
    if not os.path.exists(lib):
        from vearo_b200 import build as vb_build
        vb_build.build(bounds_check=True)
    env = dict(os.environ, VB200_LIB=lib)
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_gpu_ops.py"), "-m", "gpu", "-x", "-q",
                        "-k", "conv2d or pools or reduce_to or sum_mean or embedding or fused_attention or bn_relu or binary"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert " passed" in r.stdout
