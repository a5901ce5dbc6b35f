"""Build libb200wmma.so in-tree with nvcc for sm_100a.

The shared library is the product: every Python entry point in this package goes through it by
ctypes and raises if it is missing.  nvcc cross-compiles without a GPU, so this runs anywhere the
CUDA toolkit is installed.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
BUILD_DIR = PKG_DIR / "build"
LIB_PATH = PKG_DIR / "libb200wmma.so"

SOURCES = ["api.cu", "gemm_sm100.cu", "gemm_simple.cu", "wmma_unit.cu", "noalloc.cu", "sharded.cu"]
HEADERS = ["ptx_sm100.cuh", "gemm_sm100.cuh", "internal.h", "rng.cuh", "wmma_frag.cuh"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA toolkit is needed to build libb200wmma.so")
    return nvcc


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu under csrc/ and link libb200wmma.so next to this file."""
    nvcc = find_nvcc()
    BUILD_DIR.mkdir(exist_ok=True)
    header_deps = [CSRC / h for h in HEADERS] + [INCLUDE / "b200wmma.h"]
    jobs = []
    for src in SOURCES:
        obj = BUILD_DIR / (src + ".o")
        if force or _stale(obj, [CSRC / src] + header_deps):
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(INCLUDE), "-c", str(CSRC / src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stdout + r.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 1)) as ex:
            for out in ex.map(run, jobs):
                if verbose and out:
                    print(out)
    objs = [BUILD_DIR / (s + ".o") for s in SOURCES]
    if force or jobs or _stale(LIB_PATH, objs):
        # link beside the target and rename: a reader (a loader, a copy of the tree) never sees half a library
        tmp = LIB_PATH.with_suffix(".so.tmp")
        run([nvcc, "-Wno-deprecated-gpu-targets", "-shared", "-o", str(tmp), *map(str, objs), "-lcudart"])
        os.replace(tmp, LIB_PATH)
    return LIB_PATH


DEVICE_LIB_SRC = CSRC / "wmma_device_lib.cu"
DEVICE_LIB_OBJ = PKG_DIR / "libb200wmma_device.o"
DEVICE_LIB_PTX = PKG_DIR / "b200wmma_device.ptx"
HARNESS_SRC = PKG_DIR.parent / "tests" / "device_lib_harness.cu"
HARNESS_LIB = PKG_DIR.parent / "tests" / "libdevice_harness.so"


def build_device_lib(force: bool = False) -> Path:
    """The linkable device-side fragment library: a relocatable sm_100a object (for `nvcc -rdc` /
    nvlink users) and its PTX (for CUDAdrv's CuLink `add_data!`), plus the test harness that links
    against it the way a foreign kernel would."""
    nvcc = find_nvcc()
    deps = [DEVICE_LIB_SRC, CSRC / "wmma_frag.cuh", INCLUDE / "b200wmma.h"]
    common = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "-rdc=true",
              "-Xcompiler", "-fPIC", "-I", str(INCLUDE)]

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)

    if force or _stale(DEVICE_LIB_OBJ, deps):
        run([nvcc, *common, "-c", str(DEVICE_LIB_SRC), "-o", str(DEVICE_LIB_OBJ)])
    if force or _stale(DEVICE_LIB_PTX, deps):
        run([nvcc, "-arch=compute_100a", "-O3", "-std=c++17", "-rdc=true", "-I", str(INCLUDE), "-ptx", str(DEVICE_LIB_SRC),
             "-o", str(DEVICE_LIB_PTX)])
    if force or _stale(HARNESS_LIB, [HARNESS_SRC, DEVICE_LIB_OBJ]):
        run([nvcc, "-Wno-deprecated-gpu-targets", *common, "-shared", str(HARNESS_SRC), str(DEVICE_LIB_OBJ), "-o", str(HARNESS_LIB),
             "-lcudart"])
    return DEVICE_LIB_OBJ


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
    print(build_device_lib(force="--force" in sys.argv))
