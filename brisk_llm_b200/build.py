"""Builds libbrisk_cuda.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m brisk_llm_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OUT = os.path.join(PKG, "libbrisk_cuda.so")
OBJ = os.path.join(PKG, "build")
SOURCES = ["repack.cu", "activations.cu", "matvec.cu", "gemm.cu", "gemm_tc.cu", "gemm_k.cu", "misc.cu", "gemma.cu", "decode.cu", "step.cu", "token.cu", "topk.cu", "attn_chain.cu", "smallbatch.cu", "tp_peer.cu", "session.cu", "hooks.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
# development aid: BRISK_TOK_TRACE=1 compiles cycle stamps into the one-launch token kernel (slower; never the default)
EXTRA = ["-DBK_TOK_TRACE"] if os.environ.get("BRISK_TOK_TRACE") else []
FLAGS = ["-std=c++20", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-fmad=false",
         "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _deps():
    hdr = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    hdr.append(os.path.join(os.path.dirname(PKG), "include", "brisk_cuda.h"))
    return hdr


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    hdr = _deps()
    jobs = []
    for src in SOURCES:
        path = os.path.join(CSRC, src)
        obj = os.path.join(OBJ, src.replace(".cu", ".o"))
        if force or _stale(obj, [path] + hdr):
            jobs.append((path, obj))

    def compile_one(job):
        path, obj = job
        r = subprocess.run([NVCC, *FLAGS, *EXTRA, "-c", path, "-o", obj], capture_output=True, text=True)
        with open(obj + ".log", "w") as f:
            f.write(r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {path}:\n{r.stderr[-4000:]}")
        return r.stderr

    with ThreadPoolExecutor(max_workers=8) as ex:
        logs = list(ex.map(compile_one, jobs))
    if verbose:
        for log in logs:
            print(log)
    objs = [os.path.join(OBJ, s.replace(".cu", ".o")) for s in SOURCES]
    if force or jobs or _stale(OUT, objs):
        r = subprocess.run([NVCC, "-shared", "-o", OUT, *objs], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stderr[-4000:]}")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
