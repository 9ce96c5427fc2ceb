"""Builds ``libcandle_b200.so`` (the C-ABI library) in-tree with nvcc for sm_100a."""
from __future__ import annotations

import os
import shutil
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
LIB_DIR = os.path.join(_HERE, "_lib")
LIB_PATH = os.path.join(LIB_DIR, "libcandle_b200.so")
NCCL_LIB_PATH = os.path.join(LIB_DIR, "libcandle_b200_nccl.so")

CORE_SOURCES = ["capi.cu", "launch_cache.cu", "rms_rowreg.cu", "kqrms.cu", "norm_lanerow.cu", "norm_slow.cu", "neighbours.cu", "embedding.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--use_fast_math=false",
]


def _nvcc() -> str:
    for cand in (os.environ.get("CB200_NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA extension cannot be built")


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    deps = list(sources) + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    inc = os.path.join(os.path.dirname(_HERE), "include")
    deps += [os.path.join(inc, f) for f in os.listdir(inc) if f.endswith(".h")]
    return any(os.path.getmtime(d) > t for d in deps)


def _source_stale(obj: str, src: str) -> bool:
    return _stale(obj, [src])


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles every source into its own object (in parallel, only the stale ones) and links."""
    from concurrent.futures import ThreadPoolExecutor

    obj_dir = os.path.join(LIB_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    srcs = [os.path.join(CSRC, s) for s in CORE_SOURCES]
    objs = [os.path.join(obj_dir, os.path.splitext(s)[0] + ".o") for s in CORE_SOURCES]
    flags = [f for f in NVCC_FLAGS if f != "--use_fast_math=false"]
    if verbose:
        flags = ["-Xptxas=-v", *flags]

    def compile_one(pair):
        src, obj = pair
        if force or _source_stale(obj, src):
            subprocess.run([_nvcc(), *flags, "-ccbin", "/usr/bin/g++", "-c", "-o", obj, src], check=True)
            return True
        return False

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        rebuilt = list(pool.map(compile_one, zip(srcs, objs)))
    if any(rebuilt) or not os.path.exists(LIB_PATH):
        subprocess.run([_nvcc(), *flags, "-ccbin", "/usr/bin/g++", "-shared", "-o", LIB_PATH, *objs, "-ldl"], check=True)
    return LIB_PATH


def build_nccl(force: bool = False) -> str | None:
    """The vocab-sharded entry points live in their own library so that the core one has no NCCL
    dependency.  It links the NCCL that is already in the process (torch's) or the system one."""
    src = os.path.join(CSRC, "sharded.cu")
    if not os.path.exists(src):
        return None
    if force or _stale(NCCL_LIB_PATH, [src]):
        flags = [f for f in NVCC_FLAGS if f != "--use_fast_math=false"]
        cmd = [_nvcc(), *flags, "-ccbin", "/usr/bin/g++", "-shared", "-o", NCCL_LIB_PATH, src,
               "-L" + LIB_DIR, "-l:libcandle_b200.so", "-Xlinker", "-rpath=$ORIGIN", "-lnccl"]
        subprocess.run(cmd, check=True)
    return NCCL_LIB_PATH


if __name__ == "__main__":
    import sys

    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_nccl(force="--force" in sys.argv))
