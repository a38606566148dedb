"""Build libs24.so (the C-ABI CUDA library) in-tree for sm_100a.

    python gpu-compression-kernel_b200/build.py [--force] [--verbose] [--define NAME=VALUE ...] [--out PATH]

nvcc cross-compiles without a GPU.  The shared object lands next to the Python loader
(``s24/libs24.so``) so that it travels with the source tree; it links the CUDA runtime
statically and resolves the one driver entry point it needs (cuTensorMapEncodeTiled) at
run time, so loading it does not require a driver to be installed.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OUT = HERE / "s24" / "libs24.so"
SOURCES = ["api.cu", "prune_compress.cu", "spmm_tcgen05.cu", "spmm_prune_in.cu", "peer.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (Path(cand).exists() or cand == "nvcc"):
            return cand
    raise RuntimeError("nvcc not found")


def _stale() -> bool:
    if not OUT.exists():
        return True
    t = OUT.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "s24.h", Path(__file__)]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, defines=(), dest: Path = OUT) -> Path:
    """`defines` (NAME=VALUE strings) and `dest` build a variant library somewhere else, e.g. the
    timing experiments of csrc/spmm_tcgen05.cu; load it with S24_LIBRARY=<path>."""
    variant = bool(defines) or Path(dest) != OUT
    if not variant and not force and not _stale():
        return OUT
    objs = []
    objdir = (HERE / "build") if not variant else Path(dest).with_suffix(".objs")
    objdir.mkdir(parents=True, exist_ok=True)
    srcs = [CSRC / s for s in SOURCES if (CSRC / s).exists()]
    procs = []
    for src in srcs:
        obj = objdir / (src.stem + ".o")
        cmd = [nvcc(), *NVCC_FLAGS, *[f"-D{d}" for d in defines], "-Xptxas", "-v" if verbose else "-O3", "-c", str(src),
               "-o", str(obj)]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            print(out, file=sys.stderr)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}")
    link = [nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
            "-o", str(dest), *map(str, objs)]
    subprocess.run(link, check=True)
    return Path(dest)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--define", action="append", default=[], metavar="NAME=VALUE", help="extra -D for a variant build")
    ap.add_argument("--out", default=str(OUT), help="where to put the shared object (default: next to the loader)")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose, defines=a.define, dest=Path(a.out)))
