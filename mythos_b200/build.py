"""In-tree build of the native code.

Three artefacts are produced next to the Python sources (never in a user cache directory, so
they travel with a checkout):

* ``mythos_b200/_C*.so``      kernels (``csrc/kernels/*.cu``, sm_100a only) + torch binding
* ``mythos_b200/libmythos_kernels.so``  the same kernels with a plain C ABI, no torch
* ``mythos_b200/liboil_host.so``        host runtime: ``.oil`` container, SHA-256, BPE, RNG,
                                         page allocator, C API (``csrc/host/*.cpp``)

``nvcc`` cross-compiles for ``sm_100a`` without a GPU. Objects are rebuilt only when their
source (or a header) is newer. Run ``python -m mythos_b200.build`` or call :func:`build_all`.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "csrc" / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--use_fast_math", "-Xptxas", "-v",
]
# --use_fast_math would change expf/sincosf accuracy; the kernels pick fast intrinsics explicitly.
NVCC_FLAGS.remove("--use_fast_math")


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def _run(cmd, log: Path | None = None) -> None:
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        log.write_text(res.stdout)
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError("build step failed: " + " ".join(map(str, cmd)))


def _torch_paths():
    import torch
    from torch.utils import cpp_extension as ce

    inc = ce.include_paths()
    lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    return inc, lib


def build_kernels(verbose: bool = False) -> list[Path]:
    OBJ.mkdir(parents=True, exist_ok=True)
    kdir = CSRC / "kernels"
    headers = list(kdir.glob("*.h")) + list(kdir.glob("*.cuh"))
    jobs = []
    objs = []
    for src in sorted(kdir.glob("*.cu")):
        obj = OBJ / (src.stem + ".o")
        objs.append(obj)
        if _newer(obj, [src] + headers):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        _run([_nvcc(), *NVCC_FLAGS, "-I", str(kdir), "-c", str(src), "-o", str(obj)], OBJ / (src.stem + ".ptxas.log"))
        if verbose:
            print("nvcc", src.name)

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(compile_one, jobs))
    return objs


def build_binding(objs, verbose: bool = False) -> Path:
    inc, torch_lib = _torch_paths()
    ext = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    target = PKG / ("_C" + ext)
    bsrc = CSRC / "bindings.cpp"
    bobj = OBJ / "bindings.o"
    headers = list((CSRC / "kernels").glob("*.h"))
    if _newer(bobj, [bsrc] + headers):
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
               "-D_GLIBCXX_USE_CXX11_ABI=1", "-I", str(CSRC), "-I", "/usr/local/cuda/include",
               "-I", sysconfig.get_paths()["include"]]
        for p in inc:
            cmd += ["-isystem", p]
        cmd += ["-c", str(bsrc), "-o", str(bobj)]
        _run(cmd)
        if verbose:
            print("g++ bindings.cpp")
    if _newer(target, list(objs) + [bobj]):
        cmd = ["g++", "-shared", "-o", str(target), str(bobj), *map(str, objs), "-L", torch_lib,
               "-L", "/usr/local/cuda/lib64", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
               "-ltorch_python", "-lcudart", "-Wl,-rpath," + torch_lib, "-Wl,-rpath,/usr/local/cuda/lib64"]
        _run(cmd)
    return target


def build_kernel_clib(objs) -> Path:
    """Kernels behind a plain C ABI (csrc/c_abi.cu), for callers without torch."""
    target = PKG / "libmythos_kernels.so"
    src = CSRC / "c_abi.cu"
    if not src.exists():
        return target
    obj = OBJ / "c_abi.o"
    headers = list((CSRC / "kernels").glob("*.h")) + list(CSRC.glob("*.h"))
    if _newer(obj, [src] + headers):
        _run([_nvcc(), *NVCC_FLAGS, "-I", str(CSRC / "kernels"), "-I", str(CSRC), "-c", str(src), "-o", str(obj)],
             OBJ / "c_abi.ptxas.log")
    if _newer(target, list(objs) + [obj]):
        _run([_nvcc(), "-shared", "-o", str(target), str(obj), *map(str, objs), "-lcudart"])
    return target


def build_host(verbose: bool = False) -> Path:
    hdir = CSRC / "host"
    target = PKG / "liboil_host.so"
    srcs = sorted(hdir.glob("*.cpp")) if hdir.exists() else []
    if not srcs:
        return target
    headers = list(hdir.glob("*.h"))
    OBJ.mkdir(parents=True, exist_ok=True)
    objs = []
    for src in srcs:
        obj = OBJ / ("host_" + src.stem + ".o")
        objs.append(obj)
        if _newer(obj, [src] + headers):
            _run(["g++", "-O2", "-std=c++17", "-fPIC", "-Wall", "-I", str(hdir), "-c", str(src), "-o", str(obj)])
            if verbose:
                print("g++", src.name)
    if _newer(target, objs):
        _run(["g++", "-shared", "-o", str(target), *map(str, objs), "-lpthread", "-ldl"])
    return target


def build_host_sanitized(out_dir) -> Path:
    """The host runtime with AddressSanitizer and UndefinedBehaviorSanitizer (the reference's
    ``-DOIL_SANITIZE=ON``, cmake/compiler.cmake:8-11). Load it through ``MYTHOS_HOST_LIB`` in a
    process started with ``LD_PRELOAD=$(gcc -print-file-name=libasan.so)``."""
    hdir = CSRC / "host"
    target = Path(out_dir) / "liboil_host_asan.so"
    srcs = sorted(hdir.glob("*.cpp"))
    _run(["g++", "-O1", "-g", "-std=c++17", "-fPIC", "-fno-omit-frame-pointer", "-fsanitize=address,undefined",
          "-fno-sanitize-recover=undefined", "-I", str(hdir), "-shared", "-o", str(target), *map(str, srcs), "-lpthread",
          "-ldl"])
    return target


def build_capi(verbose: bool = False) -> Path:
    """C API (oil_model_load / oil_generate): a bridge library that embeds or joins CPython."""
    target = PKG / "liboil_capi.so"
    src = CSRC / "capi" / "oil_c_api.cpp"
    if not src.exists():
        return target
    if _newer(target, [src, CSRC / "capi" / "oil_c_api.h"]):
        libdir = sysconfig.get_config_var("LIBDIR") or "/usr/lib"
        ver = sysconfig.get_config_var("LDVERSION") or sysconfig.get_python_version()
        _run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-I", sysconfig.get_paths()["include"], "-I",
              str(CSRC / "capi"), str(src), "-o", str(target), "-L", libdir, f"-lpython{ver}", "-ldl", "-lm",
              "-Wl,-rpath," + libdir])
        if verbose:
            print("g++ oil_c_api.cpp")
    return target


def build_all(verbose: bool = False) -> dict:
    objs = build_kernels(verbose)
    out = {"binding": build_binding(objs, verbose), "kernels_c": build_kernel_clib(objs), "host": build_host(verbose),
           "capi": build_capi(verbose)}
    return out


if __name__ == "__main__":
    res = build_all(verbose=True)
    for k, v in res.items():
        print(k, v, "ok" if Path(v).exists() else "absent")
