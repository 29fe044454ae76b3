"""Builds the CUDA library in-tree: muzero_b200/lib/libmuzero_b200.so (sm_100a only).

    python -m muzero_b200.build [--force] [--verbose] [--bounds]

nvcc cross-compiles without a GPU; the shared object is git-ignored but ships with the tree.
--bounds builds a second library, lib/libmuzero_b200_bounds.so, with -DMZ_BOUNDS: guarded global stores
compare their index with the extent the host passed, skip and count an access outside it, and
mz_bounds_violations() reports the count.  Select it with MUZERO_B200_LIB=<path>.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libmuzero_b200.so")
BOUNDS_LIB_PATH = os.path.join(LIB_DIR, "libmuzero_b200_bounds.so")
SOURCES = ["mz_tables.cu", "mz_rows.cu", "mz_flush.cu", "mz_decode.cu", "mz_decode_generic.cu", "mz_decode_tiles.cu", "mz_decode_mma.cu", "mz_decode_umma.cu", "mz_qkav.cu", "mz_decode_static.cu", "mz_step.cu", "mz_manage.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "--fmad=true", "-Xptxas", "-v",
]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _newest_source_mtime() -> float:
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    paths.append(os.path.join(os.path.dirname(HERE), "include", "muzero_b200.h"))
    return max(os.path.getmtime(p) for p in paths)


def needs_build(path: str = LIB_PATH) -> bool:
    return not os.path.exists(path) or os.path.getmtime(path) < _newest_source_mtime()


def build(force: bool = False, verbose: bool = False, bounds: bool = False) -> str:
    lib_path = BOUNDS_LIB_PATH if bounds else LIB_PATH
    if not force and not needs_build(lib_path):
        return lib_path
    os.makedirs(LIB_DIR, exist_ok=True)
    obj_dir = os.path.join(LIB_DIR, "obj_bounds" if bounds else "obj")
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = _nvcc()
    # the checked build shares one device-side record between translation units: relocatable device code
    extra = ["-DMZ_BOUNDS", "-rdc=true"] if bounds else []

    def compile_one(src: str) -> str:
        obj = os.path.join(obj_dir, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        log = res.stdout + res.stderr
        with open(obj + ".log", "w") as f:
            f.write(" ".join(cmd) + "\n" + log)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{log}")
        if verbose:
            print(log)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    link_arch = ["-gencode", "arch=compute_100a,code=sm_100a"] if bounds else []   # device link of the rdc objects
    cmd = [nvcc, "-shared", *link_arch, "-o", lib_path, *objs, "-lcudart", "-ldl"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + res.stdout + res.stderr)
    return lib_path


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, bounds="--bounds" in sys.argv)
    print(path)
