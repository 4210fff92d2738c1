"""Ahead-of-time build of libb200q.so (sm_100a only) with nvcc.

The kernels are compiled here, in the source tree, not JIT-compiled at first use:
`python -m tilus_b200.build` (or `__graft_entry__.build()`) leaves
tilus_b200/libb200q.so next to the package.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "_build")
LIB = os.path.join(HERE, "libb200q.so")
NPARTS = 8

# Extra -D definitions for experiments (e.g. B200Q_EXTRA_DEFS="-DB200Q_GPW=2") and an
# alternative output name (B200Q_LIB_NAME) so that several builds can sit side by side.
EXTRA_DEFS = os.environ.get("B200Q_EXTRA_DEFS", "").split()
if os.environ.get("B200Q_LIB_NAME"):
    LIB = os.path.join(HERE, os.environ["B200Q_LIB_NAME"])
    OBJ = OBJ + "_" + os.environ["B200Q_LIB_NAME"].replace(".", "_")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else "nvcc"


def _jobs():
    jobs = []
    for part in range(NPARTS):
        jobs.append(("stream_kernel.cu", f"stream_part{part}.o", [f"-DB200Q_NPARTS={NPARTS}", f"-DB200Q_PART={part}"]))
    for part in range(NPARTS):
        jobs.append(("wide_kernel.cu", f"wide_part{part}.o", [f"-DB200Q_NPARTS={NPARTS}", f"-DB200Q_PART={part}"]))
    for part in range(NPARTS):
        jobs.append(("umma_kernel.cu", f"umma_part{part}.o", [f"-DB200Q_NPARTS={NPARTS}", f"-DB200Q_PART={part}"]))
    jobs.append(("dequant_kernel.cu", "dequant.o", []))
    jobs.append(("quantize_kernel.cu", "quantize.o", []))
    jobs.append(("cast_kernel.cu", "cast.o", []))
    jobs.append(("gather_kernel.cu", "gather.o", []))
    jobs.append(("fetch_kernel.cu", "fetch.o", []))
    jobs.append(("api.cu", "api.o", [f"-DB200Q_NPARTS={NPARTS}"]))
    return jobs


def _sources_mtime() -> float:
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".h"))]
    paths.append(os.path.join(os.path.dirname(HERE), "include", "b200q.h"))
    paths.append(os.path.abspath(__file__))
    return max(os.path.getmtime(p) for p in paths)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    newest = _sources_mtime()
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= newest:
        return LIB
    nvcc = _nvcc()

    def compile_one(job):
        src, obj, defs = job
        out = os.path.join(OBJ, obj)
        if not force and os.path.exists(out) and os.path.getmtime(out) >= newest:
            return (obj, "")
        cmd = [nvcc, *NVCC_FLAGS, *EXTRA_DEFS, *defs, "-c", os.path.join(CSRC, src), "-o", out]
        if ptxas_info:
            cmd[1:1] = ["-Xptxas", "-v"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src} ({' '.join(defs)}):\n{r.stdout}\n{r.stderr}")
        return (obj, r.stderr)

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        results = list(ex.map(compile_one, _jobs()))
    if verbose or ptxas_info:
        for obj, log in results:
            if log.strip():
                print(f"--- {obj}\n{log}", file=sys.stderr)
    objs = [os.path.join(OBJ, j[1]) for j in _jobs()]
    cmd = [nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv))
