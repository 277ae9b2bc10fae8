"""Builds librx_b200.so (sm_100a) in-tree with nvcc.

Run as `python reactant.jl_b200/build.py`; `__graft_entry__.build()` calls
`build()` below.  Objects are rebuilt only when a source or header is newer.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "librx_b200.so")
OBJ = os.path.join(HERE, "build")

SOURCES = [
    "rx_parser.cpp", "rx_plan.cpp", "rx_kernels.cu", "rx_gemm.cu", "rx_gemm_tc.cu",
    "rx_stencil.cu", "rx_stencil_tma.cu", "rx_collective.cu", "rx_runtime.cu", "rx_noalloc.cu",
]

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function,-fvisibility=default",
    "-gencode", "arch=compute_100a,code=sm_100a", "-I", os.path.join(HERE, "..", "include"), "-I", CSRC,
    "--expt-relaxed-constexpr",
]


def _stale(obj: str, deps: list[str]) -> bool:
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False, ptxas_info: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    headers.append(os.path.join(HERE, "..", "include", "rx_b200.h"))
    srcs = [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    objs, jobs = [], []
    for s in srcs:
        src = os.path.join(CSRC, s)
        obj = os.path.join(OBJ, s + ".o")
        objs.append(obj)
        if _stale(obj, [src] + headers):
            cmd = [NVCC, *FLAGS, "-x", "cu", "-c", src, "-o", obj]
            if ptxas_info:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
        return r.stderr

    with ThreadPoolExecutor(max_workers=8) as ex:
        logs = list(ex.map(run, jobs))
    if jobs or not os.path.exists(OUT):
        link = [NVCC, "-shared", "-o", OUT, *objs, "-cudart", "static", "-ldl", "-lpthread",
                "-gencode", "arch=compute_100a,code=sm_100a"]
        run(link)
    if ptxas_info:
        sys.stderr.write("\n".join(logs))
    return OUT


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv))
