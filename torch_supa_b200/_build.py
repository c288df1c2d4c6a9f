"""In-tree build of the native parts: explicit nvcc / g++ command lines, no JIT cache.

Three artefacts, all written next to the sources so that they ship with the working tree:

* ``torch_supa_b200/lib/libsupa_b200_kernels.so`` -- the sm_100a kernel library behind the C ABI of
  ``include/supa_b200_kernels.h`` (CUDA only, no torch).
* ``torch_supa_b200/lib/libtorch_supa_b200.so`` -- the C++ host layer: PrivateUse1 ("supa") device guard,
  stream pool, cudaMallocAsync allocator, ATen operator registrations, NCCL loss reducer.
* ``oracle/_build/liboracle.so`` -- the plain-C CPU restatement used by the tests as the checker.

Objects are rebuilt when a source or any header is newer than the object.  Run as
``python -m torch_supa_b200._build [--force] [--verbose]``.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
LIB_DIR = PKG / "lib"
OBJ_DIR = ROOT / "build"
KERNEL_DIR = PKG / "csrc" / "kernels"
HOST_DIRS = [PKG / "csrc" / "runtime", PKG / "csrc" / "aten", PKG / "csrc" / "dist"]
INCLUDE_DIR = ROOT / "include"
ORACLE_DIR = ROOT / "oracle"

KERNEL_LIB = LIB_DIR / "libsupa_b200_kernels.so"
HOST_LIB = LIB_DIR / "libtorch_supa_b200.so"
ORACLE_LIB = ORACLE_DIR / "_build" / "liboracle.so"

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")
    return exe


def _cuda_home() -> Path:
    return Path(_nvcc()).resolve().parent.parent


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    proc = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build command failed:\n" + " ".join(str(c) for c in cmd) + "\n" + proc.stdout + proc.stderr)
    if verbose and (proc.stdout or proc.stderr):
        print(proc.stdout + proc.stderr, flush=True)


def _newest(paths) -> float:
    return max((p.stat().st_mtime for p in paths), default=0.0)


def _stale(target: Path, deps) -> bool:
    return (not target.exists()) or target.stat().st_mtime < _newest(deps)


def _compile_all(jobs, verbose):
    """jobs: list of (cmd, object). Runs them in parallel."""
    if not jobs:
        return
    workers = min(len(jobs), max(1, (os.cpu_count() or 2)))
    with concurrent.futures.ThreadPoolExecutor(workers) as ex:
        for fut in [ex.submit(_run, cmd, verbose) for cmd, _ in jobs]:
            fut.result()


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/kernels/*.cu`` for sm_100a and link the C-ABI shared library."""
    srcs = sorted(KERNEL_DIR.glob("*.cu"))
    hdrs = sorted(KERNEL_DIR.glob("*.cuh")) + sorted(INCLUDE_DIR.glob("*.h"))
    obj_dir = OBJ_DIR / "kernels"
    obj_dir.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    jobs, objs = [], []
    for src in srcs:
        obj = obj_dir / (src.stem + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + hdrs):
            cmd = [_nvcc(), *NVCC_ARCH, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
                   "-Xcompiler", "-fvisibility=hidden", "-I", INCLUDE_DIR, "-I", KERNEL_DIR, "-c", src, "-o", obj]
            jobs.append((cmd, obj))
    _compile_all(jobs, verbose)
    if force or jobs or _stale(KERNEL_LIB, objs):
        cmd = [_nvcc(), *NVCC_ARCH, "-shared", "-cudart", "shared", "-o", KERNEL_LIB, *objs,
               "-Xlinker", "-rpath," + str(_cuda_home() / "lib64")]
        _run(cmd, verbose)
    return KERNEL_LIB


def _torch_flags():
    import torch
    from torch.utils import cpp_extension

    inc = []
    for p in cpp_extension.include_paths():
        inc += ["-isystem", p]
    torch_lib = Path(torch.__file__).resolve().parent / "lib"
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    return inc, torch_lib, abi


def build_host(force: bool = False, verbose: bool = False) -> Path:
    """Compile the C++ host layer against the installed torch and link it with the kernel library."""
    import sysconfig

    srcs = [s for d in HOST_DIRS for s in sorted(d.glob("*.cpp"))]
    hdrs = [h for d in HOST_DIRS for h in sorted(d.glob("*.h"))] + sorted(INCLUDE_DIR.glob("*.h"))
    if not srcs:
        raise RuntimeError("no host sources found")
    build_kernels(force=False, verbose=verbose)
    inc, torch_lib, abi = _torch_flags()
    obj_dir = OBJ_DIR / "host"
    obj_dir.mkdir(parents=True, exist_ok=True)
    jobs, objs = [], []
    for src in srcs:
        obj = obj_dir / (src.parent.name + "_" + src.stem + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + hdrs):
            cmd = ["g++", "-O2", "-g1", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-unused-function",
                   f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_SUPA_B200_BUILD",
                   "-I", INCLUDE_DIR, "-I", PKG / "csrc", "-isystem", _cuda_home() / "include",
                   "-isystem", sysconfig.get_paths()["include"], *inc, "-c", src, "-o", obj]
            jobs.append((cmd, obj))
    _compile_all(jobs, verbose)
    if force or jobs or _stale(HOST_LIB, objs + [KERNEL_LIB]):
        cmd = ["g++", "-shared", "-o", HOST_LIB, *objs, "-L", LIB_DIR, "-lsupa_b200_kernels",
               "-L", torch_lib, "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_python",
               "-L", _cuda_home() / "lib64", "-lcudart", "-ldl", "-lpthread",
               "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}", f"-Wl,-rpath,{_cuda_home() / 'lib64'}",
               "-Wl,--no-undefined-version"]
        _run(cmd, verbose)
    return HOST_LIB


def build_oracle(force: bool = False, verbose: bool = False) -> Path:
    """Compile the plain-C CPU restatement (test infrastructure, never loaded by the product path)."""
    srcs = sorted(ORACLE_DIR.glob("*.c"))
    hdrs = sorted(ORACLE_DIR.glob("*.h"))
    ORACLE_LIB.parent.mkdir(parents=True, exist_ok=True)
    if force or _stale(ORACLE_LIB, srcs + hdrs):
        cmd = ["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-fopenmp", "-o", ORACLE_LIB, *srcs, "-lm"]
        _run(cmd, verbose)
    return ORACLE_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force, verbose)
    if any(list(d.glob("*.cpp")) for d in HOST_DIRS):
        build_host(force, verbose)
    if ORACLE_DIR.exists() and list(ORACLE_DIR.glob("*.c")):
        build_oracle(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="--verbose" in sys.argv or "-v" in sys.argv)
    print("built:", KERNEL_LIB, HOST_LIB, ORACLE_LIB if ORACLE_LIB.exists() else "")
