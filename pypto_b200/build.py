"""In-tree build of the CUDA library: nvcc -> pypto_b200/libpypto_b200.so (sm_100a only).

The shared object links the CUDA runtime statically and resolves the one driver symbol it needs
(cuTensorMapEncodeTiled) at run time, so it loads on a machine without a GPU driver.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libpypto_b200.so"
SOURCES = ["capi.cu", "li_score.cu", "topk_select.cu", "sfa_decode.cu", "sfa_pair.cu", "prolog.cu", "prolog_gemm.cu",
           "prolog_sgemm.cu"]
HEADERS = [CSRC / "common.cuh", CSRC / "sfa_common.cuh", PKG.parent / "include" / "pypto_b200.h"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set $NVCC)")


def needs_build() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + HEADERS
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB
    objs = []
    bdir = PKG / "build"
    bdir.mkdir(exist_ok=True)
    common = [nvcc_path(), "-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v" if verbose else "-warn-spills"]
    procs = []
    for s in SOURCES:
        obj = bdir / (Path(s).stem + ".o")
        objs.append(str(obj))
        procs.append((s, subprocess.Popen(common + ["-c", str(CSRC / s), "-o", str(obj)], stdout=subprocess.PIPE,
                                          stderr=subprocess.STDOUT, text=True)))
    failed = False
    for s, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0 or verbose:
            sys.stderr.write(f"--- {s}\n{out}\n")
        failed |= pr.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    link = [nvcc_path(), "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB)] + objs + ["-ldl"]
    subprocess.run(link, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
