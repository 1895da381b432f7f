"""Builds libfe2o3_b200.so in-tree with nvcc for sm_100a.

Usage: python fe2o3_b200/build.py [--force] [--verbose] [--trace]

--trace builds a second library, libfe2o3_b200_trace.so, whose kernels record device time stamps
(-DFE2O3_EP_TRACE -DFE2O3_ATTN_TRACE); FE2O3_B200_LIB selects it, fe2o3_b200/trace.py reads the stamps.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libfe2o3_b200.so")
OBJ = os.path.join(HERE, "build")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC,-fopenmp,-fno-fast-math", "-Xptxas", "-v"]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False, trace=False):
    if trace:
        return _build(force, verbose, os.path.join(HERE, "build_trace"), os.path.join(HERE, "libfe2o3_b200_trace.so"),
                      ["-DFE2O3_EP_TRACE", "-DFE2O3_ATTN_TRACE"])
    return _build(force, verbose, OBJ, OUT, [])


def _build(force, verbose, OBJ, OUT, extra):
    os.makedirs(OBJ, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(HERE, "..", "include", "fe2o3_b200.h"))
    jobs = []
    for src in sources():
        obj = os.path.join(OBJ, src[:-3] + ".o")
        if force or _stale(obj, [os.path.join(CSRC, src)] + headers):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [NVCC] + FLAGS + extra + ["-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        return src, r.stderr

    with ThreadPoolExecutor(max_workers=8) as ex:
        for src, log in ex.map(compile_one, jobs):
            if verbose:
                print(f"== {src}\n{log}")
            with open(os.path.join(OBJ, src[:-3] + ".ptxas.log"), "w") as f:
                f.write(log)
    objs = [os.path.join(OBJ, s[:-3] + ".o") for s in sources()]
    if force or jobs or _stale(OUT, objs):
        cmd = [NVCC, "-shared", "-o", OUT] + objs + ["-Xcompiler", "-fopenmp", "-lgomp", "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, trace="--trace" in sys.argv))
