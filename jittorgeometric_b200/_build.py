"""In-tree build of ``libjgb200.so`` (all CUDA sources under ``csrc/``) for sm_100a.

``python -m jittorgeometric_b200._build`` or ``build()`` compiles each ``.cu`` to
an object with nvcc (cross-compiles without a GPU) and links one shared library
next to this file.  Objects are rebuilt only when their source or a header is
newer.
"""
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OBJDIR = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libjgb200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libjgb200.so cannot be built")
    return exe


def _newest_header():
    t = 0.0
    for d in (CSRC, INCLUDE):
        for name in os.listdir(d):
            if name.endswith((".h", ".cuh")):
                t = max(t, os.path.getmtime(os.path.join(d, name)))
    return t


def build(force=False, verbose=False, ptxas_info=False):
    """Compile and link the library; returns its path."""
    nvcc = _nvcc()
    os.makedirs(OBJDIR, exist_ok=True)
    sources = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    hdr_t = _newest_header()
    jobs, objs = [], []
    for src in sources:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJDIR, src[:-3] + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_t):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-I", INCLUDE, "-c", s, "-o", o]
            jobs.append((src, cmd))

    def run(job):
        name, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        return name, r

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for name, r in ex.map(run, jobs):
            if verbose or ptxas_info or r.returncode != 0:
                sys.stderr.write(f"[nvcc {name}]\n{r.stdout}{r.stderr}")
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {name}")
    if jobs or not os.path.exists(LIB) or force:
        cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link of libjgb200.so failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv))
