"""Builds libdpb.so (the C-ABI library) in-tree with nvcc for sm_100a.

Run as a script or call build(). Object files go to deep-prove_b200/build/,
the library next to this file.  Nothing is built at import time.
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libdpb.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function",
    "--expt-relaxed-constexpr",
    "-I", os.path.join(HERE, "..", "include"),
]


def sources():
    out = []
    for root, _, files in os.walk(CSRC):
        for f in sorted(files):
            if f.endswith((".cu", ".cpp")):
                out.append(os.path.join(root, f))
    return sorted(out)


def headers_mtime():
    newest = 0.0
    for root, _, files in os.walk(os.path.join(HERE, "..", "include")):
        for f in files:
            newest = max(newest, os.path.getmtime(os.path.join(root, f)))
    for root, _, files in os.walk(CSRC):
        for f in files:
            if f.endswith((".cuh", ".h", ".hpp")):
                newest = max(newest, os.path.getmtime(os.path.join(root, f)))
    return newest


def _compile(src, obj, verbose):
    cmd = [NVCC, *FLAGS, "-x", "cu", "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    return src, r.returncode, r.stdout + r.stderr


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    hdr = headers_mtime()
    jobs, objs = [], []
    for src in sources():
        obj = os.path.join(OBJ, os.path.relpath(src, CSRC).replace(os.sep, "_") + ".o")
        objs.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr)
        if stale:
            jobs.append((src, obj))
    log = []
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for src, rc, out in ex.map(lambda j: _compile(j[0], j[1], verbose), jobs):
                log.append(f"== {os.path.relpath(src, HERE)}\n{out}")
                if rc != 0:
                    raise RuntimeError(f"nvcc failed for {src}:\n{out}")
    if jobs or not os.path.exists(LIB):
        cmd = [NVCC, "-shared", "-o", LIB, *objs, "-lcudart", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}{r.stderr}")
    return "\n".join(log)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print("built", LIB)
