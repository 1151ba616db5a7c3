"""In-tree build of the native library.

Every ``csrc/**/*.cu`` is compiled by ``nvcc`` for ``sm_100a`` only (``-gencode
arch=compute_100a,code=sm_100a``; no multi-architecture fat binary, no JIT fallback) and every
``csrc/**/*.cpp`` by ``g++``; the objects are linked into ``context_parallelism_b200/lib/libcpb.so``.
The library exposes a plain ``extern "C"`` ABI consumed through ``ctypes`` (see ``_native.py``), so
the build needs neither the PyTorch headers nor pybind11 and finishes in seconds.  Objects are
rebuilt only when their source (or any header) is newer.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path
from typing import List

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
PKG = Path(__file__).resolve().parent
LIB_DIR = PKG / "lib"
OBJ_DIR = CSRC / "build"
LIB_PATH = LIB_DIR / "libcpb.so"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
              "--expt-relaxed-constexpr"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread"]


def _cuda_home() -> str:
    for c in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if c and Path(c, "bin", "nvcc").exists():
            return c
    nv = shutil.which("nvcc")
    if nv:
        return str(Path(nv).resolve().parent.parent)
    raise RuntimeError("nvcc not found")


def _nccl_paths():
    """NCCL header and library shipped inside the PyTorch wheel's ``nvidia/nccl`` package."""
    for p in sys.path:
        inc = Path(p) / "nvidia" / "nccl" / "include" / "nccl.h"
        if inc.exists():
            libdir = Path(p) / "nvidia" / "nccl" / "lib"
            return str(inc.parent), str(libdir)
    for inc in ("/usr/include", "/usr/local/cuda/include"):
        if Path(inc, "nccl.h").exists():
            return inc, "/usr/lib/x86_64-linux-gnu"
    return None, None


def _newest_header_mtime() -> float:
    return max((p.stat().st_mtime for p in CSRC.rglob("*") if p.suffix in (".h", ".cuh", ".hpp")), default=0.0)


def _compile_one(src: Path, verbose: bool, ptxas_v: bool) -> Path:
    cuda = _cuda_home()
    tag = hashlib.sha1(str(src.relative_to(CSRC)).encode()).hexdigest()[:8]
    obj = OBJ_DIR / f"{src.stem}_{tag}.o"
    hdr_m = _newest_header_mtime()
    if obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, hdr_m):
        return obj
    nccl_inc, _ = _nccl_paths()
    incs = ["-I", str(CSRC), "-I", str(CSRC / "kernels"), "-I", str(CSRC / "runtime"), "-I", f"{cuda}/include"]
    if nccl_inc:
        incs += ["-I", nccl_inc]
    if src.suffix == ".cu":
        cmd = [f"{cuda}/bin/nvcc", *NVCC_FLAGS, *os.environ.get("CPB_NVCC_EXTRA", "").split(),
               *(["-Xptxas", "-v"] if ptxas_v else []), *incs, "-c", str(src), "-o", str(obj)]
    else:
        cmd = ["g++", *CXX_FLAGS, *incs, "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose or ptxas_v:
        sys.stderr.write(r.stderr)
    return obj


def sources() -> List[Path]:
    return sorted(p for p in CSRC.rglob("*") if p.suffix in (".cu", ".cpp") and "build" not in p.parts)


def build(verbose: bool = False, ptxas_v: bool = False, force: bool = False) -> Path:
    """Compile what is stale and link ``libcpb.so``; returns its path."""
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    if force:
        for o in OBJ_DIR.glob("*.o"):
            o.unlink()
    srcs = sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, verbose, ptxas_v), srcs))
    if LIB_PATH.exists() and all(LIB_PATH.stat().st_mtime > o.stat().st_mtime for o in objs):
        return LIB_PATH
    cuda = _cuda_home()
    _, nccl_lib = _nccl_paths()
    link = [f"{cuda}/bin/nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB_PATH),
            *map(str, objs), "-lcudart", "-lpthread", "-ldl"]
    if nccl_lib:
        # the native process group (csrc/runtime/process_group.cpp) calls NCCL: link the copy shipped inside the
        # PyTorch wheel (the one torch itself loads) and record its directory as rpath
        link += ["-L", nccl_lib, "-l:libnccl.so.2", "-Xlinker", f"-rpath={nccl_lib}"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed: {' '.join(link)}\n{r.stdout}\n{r.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    p = build(verbose="-v" in sys.argv, ptxas_v="--ptxas" in sys.argv, force="--force" in sys.argv)
    print(p)
