"""Build recipe of the native library: nvcc, sm_100a only, in-tree output.

`python -m flux_b200.build` (or `build_library()`) compiles every `.cu` file of
`flux_b200/csrc/` into `flux_b200/libfluxb.so`. The library links the CUDA
runtime statically and resolves the one driver entry point it needs at run
time, so it loads on hosts without a GPU driver (build hosts, symbol checks).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libfluxb.so"
INCLUDE_DIR = PKG_DIR.parent / "include"

NVCC_FLAGS = [
    "-std=c++17",
    "-O3",
    "-lineinfo",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
    "-cudart",
    "static",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; the library has no prebuilt or CPU form")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [INCLUDE_DIR / "fluxb.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build_library(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile the library if it is missing or older than its sources."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = _nvcc()
    objs = []
    build_dir = PKG_DIR / "build"
    build_dir.mkdir(exist_ok=True)
    procs = []
    for src in sources():
        obj = build_dir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(INCLUDE_DIR), "-c", str(src), "-o", str(obj)]
        if ptxas_info:
            cmd += ["-Xptxas", "-v"]
        if verbose:
            print(" ".join(cmd), file=sys.stderr)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = []
    for src, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0:
            failed.append((src, out))
        elif verbose or ptxas_info:
            print(out, file=sys.stderr)
    if failed:
        msg = "\n".join(f"--- {s} ---\n{o}" for s, o in failed)
        raise RuntimeError(f"nvcc failed:\n{msg}")
    tmp = LIB_PATH.with_suffix(".so.tmp")
    cmd = [nvcc, "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a",
           "-o", str(tmp), *map(str, objs)]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    p = build_library(force="--force" in sys.argv, verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(p)
