#!/usr/bin/env python
"""Builds the UNMODIFIED reference operator for sm_100a into ``baseline/_ref`` (git-ignored).

    python baseline/build_reference.py [/path/to/reference/checkout]

The reference's own ``setup.py`` cannot be used offline (it runs ``git submodule update`` for its
CUTLASS submodule, which is not vendored in the checkout, and asks for a visible GPU to pick the
architecture), so this script compiles the reference's two translation units where they lie
(``csrc/smxx/fwd_launch.cu``, ``csrc/flash_kda.cpp``) with the flags of its ``setup.py:68-84`` and
the CUTLASS headers that ship inside the installed ``flashinfer`` wheel.  Nothing of the reference
is copied into tracked files: the outputs land in ``baseline/_ref``:

    baseline/_ref/flash_kda_C.so            the reference's extension module (sm_100a)
    baseline/_ref/flash_kda/__init__.py     its Python wrapper, as ``pip install --target`` would place it
    baseline/_ref/tests/torch_ref.py        its torch oracle (needs a GPU: JIT kernel + cuBLAS)

The binary serves as the "reference beside ours" timing row and as a bit-level parity target; the
oracle file serves the GPU-side golden generator (``tests/golden/make_golden_gpu.py``).  Neither is
imported by the ``flashkda_b200`` package.
"""
import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def cutlass_root():
    import flashinfer
    root = os.path.join(os.path.dirname(flashinfer.__file__), "data", "cutlass")
    if not os.path.isdir(os.path.join(root, "include", "cute")):
        raise SystemExit("no CUTLASS headers found under " + root)
    return root


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else None
    if ref is None or not os.path.isdir(os.path.join(ref, "csrc")):
        raise SystemExit("usage: build_reference.py /path/to/reference/checkout")
    import torch
    from torch.utils import cpp_extension
    os.makedirs(OUT, exist_ok=True)
    cut = cutlass_root()
    obj = os.path.join(OUT, "_obj")
    os.makedirs(obj, exist_ok=True)
    inc = ["-I" + os.path.join(cut, "include"), "-I" + os.path.join(cut, "tools", "util", "include"),
           "-I" + os.path.join(ref, "csrc")]
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    threads = str(max(1, min(8, os.cpu_count() or 1)))
    subprocess.check_call(
        [nvcc, "-c", os.path.join(ref, "csrc", "smxx", "fwd_launch.cu"), "-o", os.path.join(obj, "fwd_launch.o"),
         "-std=c++17", "-O3", *inc,
         "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
         "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "--expt-relaxed-constexpr", "--expt-extended-lambda",
         "--use_fast_math", "-lineinfo", "--threads", threads,
         "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"])
    tinc = ["-I" + p for p in cpp_extension.include_paths()]
    pyinc = "-I" + sysconfig.get_paths()["include"]
    abi = "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)
    subprocess.check_call(
        ["g++", "-c", os.path.join(ref, "csrc", "flash_kda.cpp"), "-o", os.path.join(obj, "flash_kda.o"),
         "-std=c++17", "-O3", "-fPIC", "-Wno-psabi", abi, "-DTORCH_EXTENSION_NAME=flash_kda_C",
         "-DTORCH_API_INCLUDE_EXTENSION_H", *tinc, pyinc, *inc, "-I/usr/local/cuda/include"])
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    subprocess.check_call(
        ["g++", "-shared", "-o", os.path.join(OUT, "flash_kda_C.so"), os.path.join(obj, "flash_kda.o"),
         os.path.join(obj, "fwd_launch.o"), "-L" + tlib, "-Wl,-rpath," + tlib, "-ltorch", "-ltorch_python", "-lc10",
         "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-L/usr/local/cuda/lib64", "-lcudart"])
    os.makedirs(os.path.join(OUT, "flash_kda"), exist_ok=True)
    shutil.copyfile(os.path.join(ref, "flash_kda", "__init__.py"), os.path.join(OUT, "flash_kda", "__init__.py"))
    os.makedirs(os.path.join(OUT, "tests"), exist_ok=True)
    shutil.copyfile(os.path.join(ref, "tests", "torch_ref.py"), os.path.join(OUT, "tests", "torch_ref.py"))
    shutil.rmtree(obj)
    print("built", os.path.join(OUT, "flash_kda_C.so"))


if __name__ == "__main__":
    main()
