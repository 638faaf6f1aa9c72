#!/usr/bin/env python3
"""Builds the unmodified reference project with its CUDA backend for sm_100 into baseline/_ref, and the small
driver baseline/reference_bench.cpp against its static libraries.

    python baseline/build_reference.py [/path/to/reference]

The reference is a CMake C++ project (no Python package): `cmake -DMINILLM_ENABLE_CUDA=ON
-DCMAKE_CUDA_ARCHITECTURES=100` configures it, ninja builds its libraries.  nvcc cross-compiles, so this works
on a machine without a GPU; the build folder then travels to the GPU machine with the repository."""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
BINARY = os.path.join(OUT, "reference_bench")


DEFAULT_REFERENCE = os.environ.get("LLME_REFERENCE", os.path.join(os.path.expanduser("~"), "reference"))


def build(reference: str = DEFAULT_REFERENCE) -> str:
    if not os.path.exists(os.path.join(reference, "CMakeLists.txt")):
        raise RuntimeError(f"the reference's sources are not at {reference}")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    build_dir = os.path.join(OUT, "build")
    os.makedirs(build_dir, exist_ok=True)
    env = dict(os.environ, CUDACXX=nvcc)
    run = lambda cmd: subprocess.run(cmd, check=True, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    try:
        run(["cmake", "-S", reference, "-B", build_dir, "-G", "Ninja", "-DCMAKE_BUILD_TYPE=Release",
             "-DMINILLM_ENABLE_CUDA=ON", "-DCMAKE_CUDA_ARCHITECTURES=100", "-DBUILD_TESTING=OFF",
             # built on one machine, run on another: a fixed instruction set (AVX2 + FMA) instead of the builder's own
             "-DMINILLM_ENABLE_NATIVE_ARCH=OFF", "-DCMAKE_CXX_FLAGS=-march=x86-64-v3"])
        run(["ninja", "-C", build_dir, "minillm_model"])
        libs = [os.path.join(build_dir, f"libminillm_{n}.a") for n in ("model", "runtime", "graph", "core")]
        cuda_home = os.path.dirname(os.path.dirname(nvcc))
        run(["g++", "-std=c++23", "-O2", "-march=x86-64-v3", "-fopenmp", "-DMINILLM_ENABLE_CUDA=1",
             "-I", os.path.join(reference, "include"), "-I", os.path.join(cuda_home, "include"),
             os.path.join(HERE, "reference_bench.cpp"), *libs, "-L", os.path.join(cuda_home, "lib64"),
             "-lcudart", "-lcublas", "-Wl,-rpath," + os.path.join(cuda_home, "lib64"), "-o", BINARY])
    except subprocess.CalledProcessError as e:
        raise RuntimeError(f"{' '.join(e.cmd[:3])} ... failed:\n{e.stdout[-3000:]}") from None
    return BINARY


if __name__ == "__main__":
    print(build(*sys.argv[1:2]))
