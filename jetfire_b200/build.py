"""Build ``libjetfire_b200.so`` in-tree with nvcc for sm_100a.

    python -m jetfire_b200.build [--force]

The library is plain C ABI (``include/jetfire_b200.h``); Python loads it with ctypes
(``jetfire_b200._lib``).  The build is skipped when the library is newer than every
source file.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libjetfire_b200.so"
SOURCES = ["pack_append.cu", "decode_scan.cu", "decode_scan_k4v4.cu", "topk_select.cu", "decode_finish.cu", "decode_static.cu",
           "jf_misc.cu", "mirror_append.cu", "mirror_correct.cu", "cpu_correction.cpp", "numa_place.cpp"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-O3", "-Xcompiler", "-pthread"]


def nvcc_path() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def up_to_date() -> bool:
    if not LIB.exists():
        return False
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.cpp")) + list(CSRC.glob("*.h")) + \
        [PKG.parent / "include" / "jetfire_b200.h"]
    return all(d.stat().st_mtime <= t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and up_to_date():
        return LIB
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    nvcc = nvcc_path()
    objs = []
    procs = []
    for src in SOURCES:
        obj = objdir / (src.rsplit(".", 1)[0] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *os.environ.get("JF_NVCC_EXTRA", "").split(), "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
        if verbose and out.strip():
            print(out)
    link = [nvcc, "-shared", "-o", str(LIB), *objs, "-lpthread",
            "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
