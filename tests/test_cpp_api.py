"""The reference-shaped C++ API (include/cake.h): compile a caller against the
header, link it to libcake_b200.so, run it on the GPU."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "api_test.cpp")


def _build(cake, tmp_path):
    exe = str(tmp_path / "api_test")
    libdir = os.path.dirname(cake.library_path())
    cmd = ["g++", "-O1", "-std=c++17", "-I", os.path.join(ROOT, "include"), SRC, "-o", exe,
           "-L", libdir, "-l:libcake_b200.so", "-Wl,-rpath," + libdir]
    env = dict(os.environ)
    env.pop("CXX", None)
    subprocess.run(cmd, check=True, capture_output=True, text=True, env=env)
    return exe


def test_caller_compiles_and_links(cake, tmp_path):
    assert os.path.exists(_build(cake, tmp_path))


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(777, 515, 1030), (111, 96, 211), (1500, 1024, 1280)])
def test_cpp_api_end_to_end(cake, tmp_path, shape):
    exe = _build(cake, tmp_path)
    r = subprocess.run([exe] + [str(v) for v in shape], capture_output=True, text=True, timeout=600)
    print(r.stdout[-2000:], r.stderr[-2000:])
    assert r.returncode == 0
    assert "ALL CORRECT" in r.stdout
