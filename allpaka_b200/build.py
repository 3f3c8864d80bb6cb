"""Compile libapk_b200.so for sm_100a with nvcc (cross-compiles without a GPU).

The matvec kernel's instantiations live in one translation unit per weight format
(csrc/mv_*.cu); the units are compiled side by side and linked into one shared library."""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libapk_b200.so")
SOURCES = ["apk_b200.cu", "mv_q8_0.cu", "mv_q5_0.cu", "mv_q2_k.cu", "mv_q4_k.cu", "mv_q5_k.cu", "mv_q6_k.cu"]
DEPS = SOURCES + ["decode.inl", "noalloc.inl", "gguf.inl", "kernels.cuh", "mv_pick.h",
                  os.path.join("..", "..", "include", "allpaka_b200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--fmad=true",           # explicit __fmul_rn/__fadd_rn guard the few spots that must not fuse
    "-Xptxas", "-v",
]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(os.path.join(CSRC, d)) > t for d in DEPS)


def _compile(src: str):
    obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
    cmd = [nvcc()] + NVCC_FLAGS + ["-c", "-o", obj, os.path.join(CSRC, src)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    return obj, cmd, proc


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not stale():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    log_path = os.path.join(HERE, "build.log")
    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as pool:
        results = list(pool.map(_compile, SOURCES))
    text, failed = "", False
    for obj, cmd, proc in results:
        text += " ".join(cmd) + "\n" + proc.stdout + proc.stderr
        failed = failed or proc.returncode != 0
    if not failed:
        link = [nvcc(), "-shared", "-o", LIB] + [r[0] for r in results] + ["-ldl"]
        proc = subprocess.run(link, capture_output=True, text=True)
        text += " ".join(link) + "\n" + proc.stdout + proc.stderr
        failed = proc.returncode != 0
    for obj, _, _ in results:  # the objects are only a step towards the library: do not leave them in the tree
        if os.path.exists(obj):
            os.remove(obj)
    if os.path.isdir(OBJ) and not os.listdir(OBJ):
        os.rmdir(OBJ)
    with open(log_path, "w") as f:
        f.write(text)
    if verbose or failed:
        sys.stderr.write(text)
    if failed:
        raise RuntimeError(f"nvcc failed; see {log_path}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
