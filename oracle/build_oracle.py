"""Build the oracle's native pieces (test infrastructure, never the product).

* ``oracle/_build/libjf_oracle_c.so`` -- the C restatement in ``oracle/jf_oracle_c.c``.
* ``oracle/_ref/jetfire_cpu_topk_attn_ref_<isa>.so`` -- the reference's own host
  correction, ``jetfire_vllm/csrc/cpu_topk_attn.cpp``, compiled UNMODIFIED from where it
  lies in the read-only reference checkout with the flags of its loader
  (``jetfire_vllm/kernels/cpu_topk_attn.py:41-52``) except ``-march=native``, which is
  replaced by explicit ISA sets so that the binary can run on another host: ``avx512bf16``
  (the reference's SIMD path) and ``avx2`` (its scalar template, auto-vectorised).
  Built only where the checkout exists; outputs are git-ignored and travel with the tree.
* ``oracle/_ref/jetfire_<kernel>_ref.so`` -- the reference's own GPU kernels for the two paper
  modes, compiled UNMODIFIED from the same checkout for sm_100: Stage A ``int3_qk_scores.cu`` and
  ``int8tc_qk_scores.cu``, Stage B ``int2_softmax_v.cu``, ``int4_softmax_v.cu`` and
  ``int8tc_softmax_v_fused.cu``, and ``blend.cu``.  The first, third, fourth and last carry no
  architecture flag in their loaders (``jetfire_vllm/kernels/int3_split.py:40-46``,
  ``int2_split.py:60-66``, ``int4_split.py:60-66``, ``blend.py:45-46``), so this is what the
  reference's own JIT build produces on a B200.  The two ``int8tc_*`` loaders pin sm_90 / sm_90a
  (``kernels/int8tc_qk_scores.py:43-48``, ``int8tc_softmax_v_fused.py:49-54``); their sources are
  compiled as they are with only that flag changed to sm_100 (and ``--use_fast_math`` kept for the
  second) -- labelled "flag edit" wherever their numbers are shown.  They pin the restated scan /
  top-k / Stage B arithmetic on the GPU box and give a same-box GPU baseline.

    python -m oracle.build_oracle [reference_root]

The reference checkout is found from the argument, else the ``JETFIRE_REFERENCE_ROOT``
environment variable, else a directory named ``reference`` next to this repository.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
BUILD = HERE / "_build"
REF_OUT = HERE / "_ref"
C_LIB = BUILD / "libjf_oracle_c.so"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))

ISA_FLAGS = {
    "avx512bf16": ["-mavx512f", "-mavx512bw", "-mavx512vl", "-mavx512dq", "-mavx512bf16", "-mavx2", "-mfma",
                   "-mf16c", "-mbmi2"],
    "avx2": ["-mavx2", "-mfma", "-mf16c"],
}


def _run(cmd):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(map(str, cmd)) + "\n" + r.stdout[-4000:])


def build_c(force: bool = False) -> Path:
    src = HERE / "jf_oracle_c.c"
    if not force and C_LIB.exists() and C_LIB.stat().st_mtime >= src.stat().st_mtime:
        return C_LIB
    BUILD.mkdir(exist_ok=True)
    _run(["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-fPIC", "-shared", str(src), "-o", str(C_LIB), "-lm"])
    return C_LIB


def ref_module_path(isa: str) -> Path:
    return REF_OUT / f"jetfire_cpu_topk_attn_ref_{isa}.so"


def reference_root(arg: str | Path | None = None) -> Path:
    if arg:
        return Path(arg)
    env = os.environ.get("JETFIRE_REFERENCE_ROOT")
    return Path(env) if env else HERE.parent.parent / "reference"


def build_ref(ref_root: str | Path | None = None, force: bool = False) -> list[Path]:
    src = reference_root(ref_root) / "jetfire_vllm" / "csrc" / "cpu_topk_attn.cpp"
    if not src.exists():
        return [ref_module_path(i) for i in ISA_FLAGS if ref_module_path(i).exists()]
    from torch.utils.cpp_extension import include_paths, library_paths
    import torch
    REF_OUT.mkdir(exist_ok=True)
    incs = [f"-I{p}" for p in include_paths()] + [f"-I{sysconfig.get_paths()['include']}", f"-I{CUDA_HOME}/include"]
    libdirs = library_paths() + [str(CUDA_HOME / "lib64"), str(CUDA_HOME / "lib64" / "stubs")]
    outs, procs = [], []
    for isa, flags in ISA_FLAGS.items():
        out = ref_module_path(isa)
        outs.append(out)
        if not force and out.exists():
            continue
        name = out.name[:-3]
        cmd = ["g++", "-O3", "-std=c++17", "-fopenmp", "-ffast-math", "-fPIC", "-shared", *flags,
               f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H",
               f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
               *incs, str(src), "-o", str(out),
               *[f"-L{d}" for d in libdirs], *[f"-Wl,-rpath,{d}" for d in libdirs[:-1]],
               "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
               "-lcudart", "-lcuda", "-fopenmp"]
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        out_text, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError("reference build failed: " + " ".join(cmd) + "\n" + out_text[-4000:])
    return outs


# name -> (source under jetfire_vllm/csrc, extra nvcc flags, label)
REF_GPU = {
    "int3_qk_scores": ("int3_qk_scores.cu", [], "unmodified"),
    "int2_softmax_v": ("int2_softmax_v.cu", [], "unmodified"),
    "int4_softmax_v": ("int4_softmax_v.cu", [], "unmodified"),
    "blend": ("blend.cu", [], "unmodified"),
    "int8tc_qk_scores": ("int8tc_qk_scores.cu", [], "flag edit: sm_90 -> sm_100"),
    "int8tc_softmax_v_fused": ("int8tc_softmax_v_fused.cu", ["--use_fast_math"], "flag edit: sm_90a -> sm_100"),
}


def ref_gpu_path(name: str) -> Path:
    return REF_OUT / f"jetfire_{name}_ref.so"


def build_ref_gpu(ref_root: str | Path | None = None, force: bool = False, jobs: int = 0) -> list[Path]:
    """The reference's GPU kernels as torch extension modules for sm_100 (a few minutes each; run
    ``jobs`` at a time, default: one per two host cores)."""
    csrc = reference_root(ref_root) / "jetfire_vllm" / "csrc"
    outs = [ref_gpu_path(n) for n in REF_GPU]
    if not csrc.exists():
        return [o for o in outs if o.exists()]
    from torch.utils.cpp_extension import include_paths, library_paths
    import torch
    REF_OUT.mkdir(exist_ok=True)
    incs = [f"-I{p}" for p in include_paths()] + [f"-I{sysconfig.get_paths()['include']}"]
    libdirs = library_paths() + [str(CUDA_HOME / "lib64")]
    todo = []
    for name, (src, extra, _label) in REF_GPU.items():
        out = ref_gpu_path(name)
        if not force and out.exists():
            continue
        mod = out.name[:-3]
        todo.append([str(CUDA_HOME / "bin" / "nvcc"), "-O3", "-std=c++17", "-gencode", "arch=compute_100,code=sm_100",
                     *extra, "-Xcompiler", "-fPIC", "-Xcompiler", "-O3", "-shared", f"-DTORCH_EXTENSION_NAME={mod}",
                     "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
                     "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
                     "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__", "--expt-relaxed-constexpr",
                     *incs, str(csrc / src), "-o", str(out), *[f"-L{d}" for d in libdirs],
                     "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"])
    jobs = jobs or max(1, (os.cpu_count() or 2) // 2)
    running = []
    while todo or running:
        while todo and len(running) < jobs:
            cmd = todo.pop(0)
            running.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        cmd, p = running.pop(0)
        out_text, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError("reference GPU kernel build failed: " + " ".join(cmd) + "\n" + out_text[-4000:])
    return outs


def build_all() -> None:
    build_c()
    build_ref()
    build_ref_gpu()


if __name__ == "__main__":
    build_c(force=True)
    print(C_LIB)
    for p in build_ref(sys.argv[1] if len(sys.argv) > 1 else None, force=True):
        print(p)
    for p in build_ref_gpu(sys.argv[1] if len(sys.argv) > 1 else None, force=True):
        print(p)
