#!/usr/bin/env python3
"""Builds the benchmark's reference arm: kishida/questwend itself, unmodified, with its CUDA backend.

    python baseline/build_reference.py --reference DIR [--build-dir DIR] [--arch 100]

The reference is a CMake C++ project (no Python package: ``pip install`` of it fails with "Neither 'setup.py' nor
'pyproject.toml' found"), so it is built the way its README builds it, with its own switch for CUDA
(CMakeLists.txt:13, 17-23: QW_CUDA -> GGML_CUDA and GGML_CUDA_GRAPHS), from the read-only checkout into a build folder
outside it.  Then ``ref_bench.cpp`` (beside this file), which calls the reference's public classes only, is linked against
the reference's static libraries, and the one program is put under ``baseline/_ref/bin/``, which is not tracked by git
but travels to the GPU box.  ``bench.py --impl reference`` runs that program.  No GPU is needed to build.
"""
import argparse
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("QW_REFERENCE_DIR"), required="QW_REFERENCE_DIR" not in os.environ,
                    help="the checkout of kishida/questwend (read only; or the environment variable QW_REFERENCE_DIR)")
    ap.add_argument("--build-dir", default=os.path.join(tempfile.gettempdir(), "qw_ref_cuda_build"))
    ap.add_argument("--arch", default="100", help="CMAKE_CUDA_ARCHITECTURES (100: sm_100 machine code and compute_100 PTX)")
    ap.add_argument("--jobs", type=int, default=os.cpu_count() or 4)
    args = ap.parse_args()
    ref, bd = args.reference, args.build_dir
    subprocess.check_call(["cmake", "-S", ref, "-B", bd, "-G", "Ninja", "-DQW_CUDA=ON", f"-DCMAKE_CUDA_ARCHITECTURES={args.arch}",
                           "-DGGML_NATIVE=OFF", "-DGGML_OPENMP=OFF", "-DCMAKE_BUILD_TYPE=Release", "-DBUILD_SHARED_LIBS=OFF"])
    subprocess.check_call(["cmake", "--build", bd, "--target", "questwend_core", "qw-cli", "-j", str(args.jobs)])
    libs = []
    for root, _, files in os.walk(bd):
        libs += [os.path.join(root, f) for f in files if f.endswith(".a")]
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    out_dir = os.path.join(HERE, "_ref", "bin")
    os.makedirs(out_dir, exist_ok=True)
    out = os.path.join(out_dir, "qw_ref_bench")
    # the CUDA runtime and cuBLAS are linked as shared libraries: the GPU box has the same toolkit image.  ggml's CUDA
    # backend links NCCL when CMake finds it (for its two-GPU split, which the reference never uses): link what it found.
    nccl = []
    with open(os.path.join(bd, "build.ninja")) as f:
        if "libnccl" in f.read():
            nccl = ["-lnccl"]
    subprocess.check_call(["g++", "-O2", "-std=c++17", os.path.join(HERE, "ref_bench.cpp"), "-I", os.path.join(ref, "core"),
                           "-I", os.path.join(ref, "third_party/ggml/include"), "-o", out, "-Wl,--start-group"] + libs +
                          ["-Wl,--end-group", f"-L{cuda}/lib64", f"-L{cuda}/lib64/stubs", "-lcudart", "-lcublas", "-lcublasLt",
                           "-lcuda", *nccl, f"-Wl,-rpath,{cuda}/lib64", "-lpthread", "-ldl", "-lm"])
    print(out)
    return 0


if __name__ == "__main__":
    sys.exit(main())
