"""The C++ host layer (include/xnq.hpp) over the C ABI: built with g++ against libxnq.so."""
import os
import subprocess

import numpy as np
import pytest

from conftest import assert_close_ref
from xn_b200 import synth
from xn_b200.dtypes import GgmlDType as D

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "host_mirror_test.cpp")


@pytest.fixture(scope="module")
def exe(tmp_path_factory):
    from xn_b200 import _lib
    _lib.lib()
    out = str(tmp_path_factory.mktemp("cpp") / "host_mirror_test")
    libdir = os.path.join(ROOT, "xn_b200")
    cmd = ["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), SRC, "-o", out, "-L", libdir, "-l:libxnq.so",
           f"-Wl,-rpath,{libdir}", "-ldl", "-lpthread", "-lrt"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return out


def test_cpp_mirror_shape_and_dtype_errors(exe):
    r = subprocess.run([exe, "cpu"], capture_output=True, text=True)
    assert r.returncode == 0 and "cpu ok" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("dt,m", [(D.Q4K, 6), (D.Q8_0, 40)])
def test_cpp_mirror_forward_on_gpu(exe, O, tmp_path, dt, m):
    n, k = 96, 1024
    w = synth.make_weight(dt, n, k, seed=400)
    x = synth.make_activation(m, k, seed=401)
    bias = synth.make_activation(1, n, seed=402)[0]
    paths = [str(tmp_path / f) for f in ("w.bin", "x.bin", "b.bin", "y.bin")]
    w.tofile(paths[0]); x.tofile(paths[1]); bias.tofile(paths[2])
    r = subprocess.run([exe, "gpu", str(int(dt)), str(n), str(k), str(m), *paths], capture_output=True, text=True)
    assert r.returncode == 0 and "gpu ok" in r.stdout, r.stdout + r.stderr
    y = np.fromfile(paths[3], np.float32).reshape(m, n)
    want = O.matmul(int(dt), x, w, n) + bias
    if m <= 16:
        assert_close_ref(y, want, 2e-3, f"c++ {dt.name}")
    else:
        rms = float(np.sqrt((want.astype(np.float64) ** 2).mean()))
        assert np.abs(y - want).max() <= 5e-3 * rms
