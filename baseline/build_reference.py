"""Builds the UNMODIFIED reference (a CMake C++ project, CPU only) under ``baseline/_ref`` and the
small driver that times its stock ``Trainer::train_step`` on the tiny byte-level configuration.

    python baseline/build_reference.py [--source /path/to/reference]

The reference tree is copied to a temporary directory first (its own tree may be read-only and
CMake writes a generated header next to the build), CUDA detection is switched off (its
``cuda_add_library`` call does not configure with a modern CMake, and nothing on Linux links those
kernels), and only the libraries the driver needs are built. Outputs: ``baseline/_ref/build/*.a``,
``baseline/_ref/include`` (headers), ``baseline/_ref/ref_config1`` (the driver binary).
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
LIBS = ["oil_trainer", "oil_tokenizer", "oil_model", "oil_inference", "oil_kernel", "oil_format", "oil_math", "oil_core"]


def main() -> int:
    ap = argparse.ArgumentParser()
    # default: $MYTHOS_REFERENCE, else a checkout named "reference" beside this repository
    sibling = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    ap.add_argument("--source", default=os.environ.get("MYTHOS_REFERENCE", sibling))
    a = ap.parse_args()
    if not os.path.exists(os.path.join(a.source, "CMakeLists.txt")):
        print(f"no reference checkout at {a.source}", file=sys.stderr)
        return 1
    os.makedirs(OUT, exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "src")
        shutil.copytree(a.source, src)
        build = os.path.join(OUT, "build")
        subprocess.run(["cmake", "-S", src, "-B", build, "-DCMAKE_DISABLE_FIND_PACKAGE_CUDAToolkit=ON",
                        "-DCMAKE_BUILD_TYPE=Release", "-DOIL_BUILD_TESTS=OFF", "-DOIL_BUILD_BENCHMARKS=OFF"], check=True)
        subprocess.run(["make", "-C", build, f"-j{os.cpu_count() or 4}", *LIBS], check=True)
        inc = os.path.join(OUT, "include")
        shutil.rmtree(inc, ignore_errors=True)
        shutil.copytree(os.path.join(src, "include"), inc)
    libs = [os.path.join(OUT, "build", f"lib{n}.a") for n in LIBS]
    subprocess.run(["g++", "-O2", "-std=c++20", "-I", os.path.join(OUT, "include"), "-I", os.path.join(OUT, "build"),
                    os.path.join(HERE, "ref_config1_driver.cpp"), "-o", os.path.join(OUT, "ref_config1"),
                    "-Wl,--start-group", *libs, "-Wl,--end-group", "-lpthread"], check=True)
    print("built", os.path.join(OUT, "ref_config1"))
    return 0


if __name__ == "__main__":
    sys.exit(main())
