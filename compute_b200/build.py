"""Builds libcudabackend.so (sm_100a) in-tree with nvcc.  Run: python -m compute_b200.build"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libcudabackend.so")
OBJ = os.path.join(HERE, "build")

SOURCES = ["runtime.cu", "qdense.cu", "qdense_prefill.cu", "qdense_decode_tc.cu", "dot.cu", "dot_generic.cu", "gemm_tcgen05.cu",
           "sdpa.cu", "sdpa_generic.cu", "sdpa_flash.cu", "sdpa_decode.cu", "qdense_ggml.cu", "qdense_ggml_mma.cu", "qdense_w4.cu", "helper_ops.cu", "fused_small.cu", "elementwise.cu", "graph.cu", "comm.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
              "-DCB_BUILDING"]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(HERE, "..", "include", "cudabackend.h"))
    headers.append(os.path.join(HERE, "..", "include", "cudabackend_graph.h"))
    headers.append(os.path.abspath(__file__))
    cc = nvcc()
    # gcc 13 from the system; an unrelated CC in the environment must not leak into nvcc
    host = shutil.which("g++") or "g++"
    objs, jobs = [], []
    for src in SOURCES:
        sp = os.path.join(CSRC, src)
        op = os.path.join(OBJ, src.replace(".cu", ".o"))
        objs.append(op)
        if force or not _newer(op, [sp] + headers):
            cmd = [cc, "-ccbin", host] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-c", sp, "-o", op]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or ptxas_info or r.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for " + cmd[-3])
        return r

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(run, jobs))
    if jobs or force or not os.path.exists(OUT):
        run([cc, "-ccbin", host, "-shared", "-o", OUT] + objs + ["-cudart", "static", "-ldl", "-Xlinker", "--no-undefined"])
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv))
