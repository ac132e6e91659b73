"""Builds libdnn_b200.so (sm_100a) in-tree with nvcc.

    python dnn.c_b200/build.py [--force] [--verbose]

Every .cu under csrc/ is compiled to an object (only when its source or a
header is newer) and linked into dnn.c_b200/libdnn_b200.so.  The arch is
passed as -gencode so the tcgen05 PTX is accepted; there is no other target.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libdnn_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr", "-I" + os.path.join(ROOT, "include"), "-I" + CSRC,
]


def _newest_header():
    t = 0.0
    for d in (CSRC, os.path.join(ROOT, "include")):
        for f in os.listdir(d):
            if f.endswith((".h", ".cuh")):
                t = max(t, os.path.getmtime(os.path.join(d, f)))
    return t


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    hdr_t = _newest_header()
    srcs = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    jobs = []
    for s in srcs:
        src = os.path.join(CSRC, s)
        obj = os.path.join(OBJ, s[:-3] + ".o")
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_t):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            jobs.append((s, cmd))

    def run(job):
        name, cmd = job
        r = subprocess.run(cmd, capture_output=True, text=True)
        return name, r

    failed = False
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        for name, r in ex.map(run, jobs):
            if r.returncode != 0:
                failed = True
                sys.stderr.write("nvcc failed on %s:\n%s\n" % (name, r.stderr))
            elif verbose or r.stderr.strip():
                sys.stderr.write("[%s]\n%s\n" % (name, r.stderr))
    if failed:
        raise RuntimeError("libdnn_b200 build failed")
    objs = [os.path.join(OBJ, s[:-3] + ".o") for s in srcs]
    if jobs or not os.path.exists(LIB):
        cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-Xlinker", "-Bsymbolic", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
