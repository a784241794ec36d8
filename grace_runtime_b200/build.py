"""Builds grace_runtime_b200/libgrace_b200.so from csrc/ with nvcc for sm_100a (cross-compiles without a GPU).

    python -m grace_runtime_b200.build [--force] [-j N]

Objects go to csrc/build/; a source is recompiled when it or a header is newer than its object.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libgrace_b200.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", "-DGRACE_B200_BUILD"]


def nvcc():
    p = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(p):
        raise RuntimeError("nvcc not found: the library is CUDA only")
    return p


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))


def _compile(src, obj, verbose):
    extra = os.environ.get("GRACE_B200_NVCC_FLAGS", "").split()    # e.g. -D switches of a diagnostic build
    cmd = [nvcc()] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-x", "cu", "-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    return src, r.returncode, r.stdout + r.stderr


def build(force=False, jobs=None, verbose=False):
    bdir = os.path.join(CSRC, "build")
    os.makedirs(bdir, exist_ok=True)
    headers = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + \
        [os.path.join(HERE, "..", "include", "grace_b200.h")]
    newest_h = max(os.path.getmtime(h) for h in headers)
    todo, objs = [], []
    for s in sources():
        o = os.path.join(bdir, os.path.basename(s) + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), newest_h):
            todo.append((s, o))
    logs = []
    if todo:
        with cf.ThreadPoolExecutor(max_workers=jobs or min(8, os.cpu_count() or 2)) as ex:
            for src, rc, log in ex.map(lambda so: _compile(so[0], so[1], verbose), todo):
                logs.append((src, log))
                if rc != 0:
                    raise RuntimeError(f"nvcc failed on {src}:\n{log}")
    if todo or not os.path.exists(OUT):
        cmd = [nvcc(), "-shared", "-o", OUT] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    return OUT, logs


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-j", type=int, default=None)
    ap.add_argument("-v", action="store_true", help="print ptxas register / shared-memory usage")
    a = ap.parse_args()
    out, logs = build(a.force, a.j, a.v)
    if a.v:
        for src, log in logs:
            print("==", src)
            print(log)
    print(out)
    sys.exit(0)
