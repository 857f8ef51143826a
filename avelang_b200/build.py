"""Ahead-of-time build of libave_gdn_b200.so with nvcc for sm_100a (no JIT, no torch headers).

The reference builds its device helpers at first use with the host compiler
(python/avelang/runtime/build.py:16-89); here everything is compiled once, in-tree, so the shared
object travels with the source tree."""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB = os.path.join(HERE, "libave_gdn_b200.so")
SOURCES = ["api.cu", "decode.cu", "decode_layer.cu", "backward.cu", "rmsnorm.cu", "prefill_simt.cu", "elementwise.cu", "gemm.cu", "tmap.cu", "prefill_tc.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-I" + INCLUDE,
              "-I" + CSRC]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _digest() -> str:
    hsh = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    names = sorted(os.listdir(CSRC)) + [os.path.join(INCLUDE, "ave_gdn.h")]
    for name in names:
        path = name if os.path.isabs(name) else os.path.join(CSRC, name)
        if os.path.isfile(path):
            hsh.update(open(path, "rb").read())
    return hsh.hexdigest()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu into objects and link the shared library; skipped when sources are unchanged."""
    stamp = LIB + ".stamp"
    digest = _digest()
    if not force and os.path.exists(LIB) and os.path.exists(stamp) and open(stamp).read() == digest:
        return LIB
    objdir = os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    nvcc = _nvcc()
    procs = []
    for src in SOURCES:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objs = []
    for src, obj, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
        objs.append(obj)
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", *objs, "-o", LIB, "-lcuda"]
    subprocess.run(link, check=True)
    with open(stamp, "w") as f:
        f.write(digest)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
