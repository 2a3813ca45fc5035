"""Builds libqw_gpu_cuda.so (all CUDA kernels + the C-ABI backend + the host engine) for sm_100a, in-tree.

    python -m qwental_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The IQ3_S codebook include is generated first from the installed `gguf`
package (qwental_b200/csrc/gen_tables.py).  Objects and the library go to qwental_b200/_build/ (git-ignored).
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "_build")
LIB = os.path.join(OUT, "libqw_gpu_cuda.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "-ccbin", "/usr/bin/g++", "-I", os.path.join(ROOT, "include")]


def _newer(src: str, dst: str, deps) -> bool:
    if not os.path.exists(dst):
        return True
    t = os.path.getmtime(dst)
    return any(os.path.getmtime(d) > t for d in [src] + deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OUT, exist_ok=True)
    gen = os.path.join(CSRC, "_gen", "iq3s_grid.inc")
    if force or not os.path.exists(gen):
        subprocess.run([sys.executable, os.path.join(CSRC, "gen_tables.py"), gen], check=True)
    srcs = sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    hdrs += [os.path.join(ROOT, "include", f) for f in os.listdir(os.path.join(ROOT, "include"))] + [gen]
    objs, jobs = [], []
    for f in srcs:
        src, obj = os.path.join(CSRC, f), os.path.join(OUT, f.rsplit(".", 1)[0] + ".o")
        objs.append(obj)
        if force or _newer(src, obj, hdrs):
            cmd = [NVCC] + FLAGS + (["-x", "cu"] if f.endswith(".cpp") else []) + ["-Xptxas", "-v", "-c", src, "-o", obj]
            jobs.append((f, cmd))

    def run(job):
        f, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        return f, r

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for f, r in ex.map(run, jobs):
                log = os.path.join(OUT, f + ".ptxas.log")
                with open(log, "w") as fh:
                    fh.write(r.stdout + r.stderr)
                if verbose:
                    sys.stderr.write(r.stderr)
                if r.returncode != 0:
                    raise RuntimeError("nvcc failed on %s:\n%s" % (f, r.stderr[-4000:]))
    if jobs or not os.path.exists(LIB):
        cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-ccbin", "/usr/bin/g++", "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stderr[-4000:])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
