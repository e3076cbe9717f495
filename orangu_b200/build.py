"""Builds the native libraries in-tree.

  orangu_b200/_lib/liborangu_b200.so   CUDA kernels + C ABI, sm_100a only (nvcc)
  orangu_b200/_lib/libob_synth.so      synthetic weight builder (host, g++)

Run as ``python -m orangu_b200.build``.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "_lib")
OBJDIR = os.path.join(LIBDIR, "obj")
LIB = os.path.join(LIBDIR, "liborangu_b200.so")
SYNTH_LIB = os.path.join(LIBDIR, "libob_synth.so")

CU_SOURCES = ["formats.cu", "act_quant.cu", "gemv.cu", "glue.cu", "attention.cu", "api.cu", "model.cu", "tp.cu", "noalloc.cu", "stream_gemv.cu", "layer_stream.cu", "gemm_mma.cu", "gemm_tc5.cu", "gguf.cu", "sched.cu", "q5k.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    # The reproduced arithmetic never fuses a*b+c; FMAs are written out where wanted.
    "-fmad=false",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _host_cxx() -> str:
    # the environment's CXX may be a g++ without libgomp
    return "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else (shutil.which("g++") or "g++")


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _headers() -> list[str]:
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    hs.append(os.path.join(os.path.dirname(HERE), "include", "orangu_b200.h"))
    return hs


def build_cuda(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJDIR, exist_ok=True)
    nvcc = _nvcc()
    hdrs = _headers()
    jobs = []
    for src in CU_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJDIR, src.replace(".cu", ".o"))
        if force or _newer(o, [s] + hdrs):
            jobs.append((s, o))

    def compile_one(job):
        s, o = job
        cmd = [nvcc, *NVCC_FLAGS, "-c", s, "-o", o]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {s}:\n{r.stdout}\n{r.stderr}")
        return r.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for log in ex.map(compile_one, jobs):
                if verbose and log:
                    print(log, file=sys.stderr)
    objs = [os.path.join(OBJDIR, s.replace(".cu", ".o")) for s in CU_SOURCES]
    if force or jobs or _newer(LIB, objs):
        cmd = [nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


def build_synth(force: bool = False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    src = os.path.join(HERE, "synth", "synth.cpp")
    if force or _newer(SYNTH_LIB, [src]):
        # x86-64-v3, not -march=native: the library travels to other hosts
        cmd = [_host_cxx(), "-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-std=c++17", "-shared", "-o", SYNTH_LIB, src]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"g++ failed on synth.cpp:\n{r.stdout}\n{r.stderr}")
    return SYNTH_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cuda(force, verbose)
    build_synth(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
    print(SYNTH_LIB)
