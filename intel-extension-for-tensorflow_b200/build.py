"""Builds libitexb200.so (CUDA kernels + C-ABI + op layer) for sm_100a with nvcc.

    python intel-extension-for-tensorflow_b200/build.py [--force]

nvcc cross-compiles without a GPU.  The library links the CUDA runtime statically and
reaches the driver only through cudaGetDriverEntryPoint, so it loads (and exports every
symbol of include/itexb200.h) on a machine that has no GPU or driver.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OUT_DIR = os.path.join(PKG, "lib")
LIB = os.path.join(OUT_DIR, "libitexb200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-fmad=false",  # separate fp32 multiply and add, like the CPU reference path
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Wno-unused-function,-ffp-contract=off",
    "-I" + os.path.join(ROOT, "include"), "-I" + CSRC,
]


def sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cc")))


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    os.makedirs(OUT_DIR, exist_ok=True)
    obj_dir = os.path.join(PKG, "build")
    os.makedirs(obj_dir, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".h")]
    headers.append(os.path.join(ROOT, "include", "itexb200.h"))
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    jobs, objs = [], []
    for src in sources():
        obj = os.path.join(obj_dir, os.path.splitext(src)[0] + ".o")
        objs.append(obj)
        path = os.path.join(CSRC, src)
        if force or _stale(obj, [path] + headers):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-x", "cu", "-c", path, "-o", obj]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
        return r.stderr

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        logs = list(ex.map(run, jobs))
    if verbose:
        for log in logs:
            sys.stderr.write(log)
    if jobs or force or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-cudart", "static", "-o", LIB] + objs + ["-Xlinker", "--no-undefined", "-lpthread", "-ldl", "-lrt"]
        run(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
