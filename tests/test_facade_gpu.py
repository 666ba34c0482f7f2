"""Builds and runs the C++ facade test program (tests/facade_test.cu) against the shared library."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_facade_program(built_lib, tmp_path):
    exe = str(tmp_path / "facade_test")
    libdir = os.path.join(ROOT, "clusternet_b200")
    subprocess.check_call(["/usr/local/cuda/bin/nvcc", "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a",
                           os.path.join(ROOT, "tests", "facade_test.cu"), "-o", exe, f"-L{libdir}", "-lclusternet_b200",
                           "-Xlinker", f"-rpath={libdir}"])
    r = subprocess.run([exe, os.path.join(ROOT, "tests", "golden", "codebook_126.f32"), str(tmp_path),
                        os.path.join(ROOT, "tests", "golden", "numpy_arange_as_h5py.hdf5")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "All tests passed" in r.stdout, r.stdout + r.stderr
