"""Build libspaurora_sm100.so (the C-ABI CUDA library) in-tree with nvcc.

    python -m sp_aurora_b200.build [--force]

Every translation unit is compiled for sm_100a only (`-gencode
arch=compute_100a,code=sm_100a -lineinfo`); nvcc cross-compiles without a GPU.
The CUDA runtime is linked statically so the library loads in a process that
has no CUDA libraries on its path; the driver entry point for TMA descriptor
encoding is looked up at run time.
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
LIB_PATH = PKG_DIR / "libspaurora_sm100.so"
SOURCES = ["spa_abi.cu", "attn_fwd_sm100.cu", "attn_bwd_dq_sm100.cu", "attn_bwd_dkv_sm100.cu",
           "attn_simt.cu", "wait_selftest.cu"]
HEADERS = [CSRC / "tc05.cuh", CSRC / "spa_internal.h", PKG_DIR.parent / "include" / "spa.h"]

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "--use_fast_math=false", "-cudart", "static",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; cannot build libspaurora_sm100.so")
    return exe


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile (if stale) and return the path of the shared library. Safe to call from several
    processes at once (one rank per GPU importing the package): an exclusive file lock lets one
    of them build while the others wait and then find the library fresh; the library itself is
    replaced atomically."""
    import fcntl
    obj_dir = PKG_DIR / "build"
    obj_dir.mkdir(exist_ok=True)
    with open(obj_dir / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            return _build_locked(force, verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(force: bool, verbose: bool) -> Path:
    nvcc = _nvcc()
    flags = [f for f in NVCC_FLAGS if not f.startswith("--use_fast_math")]
    obj_dir = PKG_DIR / "build"
    obj_dir.mkdir(exist_ok=True)
    jobs = []
    for src in SOURCES:
        s = CSRC / src
        o = obj_dir / (src + ".o")
        if force or _stale(o, [s, *HEADERS]):
            jobs.append((s, o))

    def compile_one(job):
        s, o = job
        cmd = [nvcc, *flags, "-c", str(s), "-o", str(o)]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {s.name}:\n{r.stdout}\n{r.stderr}")
        return o

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 1)) as ex:
            list(ex.map(compile_one, jobs))
    objs = [obj_dir / (src + ".o") for src in SOURCES]
    if force or jobs or _stale(LIB_PATH, objs):
        tmp = LIB_PATH.with_name(f"{LIB_PATH.name}.{os.getpid()}.tmp")
        cmd = [nvcc, "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a",
               "-o", str(tmp), *map(str, objs)]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose=True)
    print(p)
