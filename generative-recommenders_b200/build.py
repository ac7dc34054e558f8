"""Build libb200_hstu.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python generative-recommenders_b200/build.py [--force] [--verbose]

Each csrc/*.cu becomes build/<name>.o; the objects are linked into
generative-recommenders_b200/libb200_hstu.so.  Files are rebuilt when they or any header
in csrc/ or include/ are newer than their object.
"""

import argparse
import concurrent.futures
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libb200_hstu.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]
# B200_HSTU_TRACE_BUILD=1 compiles the in-kernel timeline marks in (a profiling aid; the marks sit in
# the hot loops, so the default build leaves them out); rebuild with force after changing it
if os.environ.get("B200_HSTU_TRACE_BUILD"):
    NVCC_FLAGS.append("-DB200_HSTU_TRACE_BUILD")


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _newest_header():
    hdrs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    return max(os.path.getmtime(h) for h in hdrs)


def _compile(src, obj, verbose):
    cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    return src, r.returncode, r.stdout + r.stderr


def build(force=False, verbose=False):
    os.makedirs(BUILD, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdr_time = _newest_header()
    jobs, objs = [], []
    for s in srcs:
        o = os.path.join(BUILD, os.path.splitext(os.path.basename(s))[0] + ".o")
        objs.append(o)
        stale = force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_time)
        if stale:
            jobs.append((s, o))
    failed = False
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for src, rc, out in ex.map(lambda j: _compile(j[0], j[1], verbose), jobs):
            if rc != 0 or verbose:
                sys.stderr.write("== %s (exit %d)\n%s\n" % (os.path.basename(src), rc, out))
            failed = failed or rc != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if jobs or not os.path.exists(LIB):
        cmd = [_nvcc(), "-shared", "-o", LIB] + objs + ["-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
