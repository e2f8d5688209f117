"""Builds cake_on_cpu_b200/libcake_b200.so in-tree with nvcc for sm_100a.

    python -m cake_on_cpu_b200.build [--verbose]

The shared library holds the CUDA kernels, the C ABI (include/cake_b200.h) and
the C++ API of the reference (include/cake.h).  nvcc cross-compiles without a
GPU, so this also serves as the "does it build" check.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libcake_b200.so")

SOURCES = ["abi.cu", "sgemm_ffma.cu", "sgemm_tf32x3.cu", "sgemm_small_tf32x3.cu", "conv_tf32x3.cu", "gemv.cu", "kshard.cu", "peak_tf32.cu", "pack.cu", "sparse.cu", "conv.cu", "tiling.cpp", "tune.cpp", "host_api.cpp"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", *(["-DCAKEB200_ROLE_TIMERS"] if os.environ.get("CAKEB200_ROLE_TIMERS") else []),
    "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def needs_build():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps += [os.path.join(ROOT, "include", f) for f in os.listdir(os.path.join(ROOT, "include"))]
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose=False, force=False):
    """Compile every source for sm_100a and link the shared library."""
    if not force and not needs_build():
        return LIB
    nvcc = _nvcc()
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    objs, procs = [], []
    extra = ["-Xptxas", "-v"] if verbose else []
    for src in SOURCES:
        obj = os.path.join(objdir, src.rsplit(".", 1)[0] + ".o")
        objs.append(obj)
        cmd = [nvcc] + NVCC_FLAGS + extra + ["-x", "cu", "-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write("== %s ==\n%s\n" % (src, out))
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    link = [nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart_static", "-lpthread", "-ldl", "-lrt"]
    subprocess.run(link, check=True)
    return LIB


LINEAR_EXT = os.path.join(HERE, "linear_cpp.so")


def build_linear_ext(force=False):
    """Compile csrc/linear.cpp, the PyTorch extension `linear_cpp` of the reference's binding
    (reference src/linear.cpp, python/setup.py), against include/cake.h and link it to
    libcake_b200.so.  g++ only (the file holds no kernels); the module lands next to the library."""
    src = os.path.join(CSRC, "linear.cpp")
    if not force and os.path.exists(LINEAR_EXT) and os.path.getmtime(LINEAR_EXT) >= max(os.path.getmtime(src), os.path.getmtime(LIB)):
        return LINEAR_EXT
    import sysconfig
    import torch
    from torch.utils import cpp_extension
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(_nvcc())), "include")
    cmd = [os.environ.get("CXX_FOR_EXT", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=linear_cpp",
           "-DTORCH_API_INCLUDE_EXTENSION_H", "-I", os.path.join(ROOT, "include"), "-I", cuda_inc,
           "-I", sysconfig.get_paths()["include"]]
    for inc in cpp_extension.include_paths():
        cmd += ["-isystem", inc]
    cmd += [src, "-o", LINEAR_EXT, "-L", libdir, "-lc10", "-lc10_cuda", "-ltorch", "-ltorch_cpu", "-ltorch_python",
            "-L", HERE, "-l:libcake_b200.so", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + libdir]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError("compiling linear.cpp failed")
    return LINEAR_EXT


if __name__ == "__main__":
    build(verbose="--verbose" in sys.argv, force=True)
    print(LIB)
    if "--linear" in sys.argv:
        print(build_linear_ext(force=True))
