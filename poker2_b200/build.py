"""Builds libpoker2_b200.so (the sm_100a kernels behind the C ABI) in-tree with nvcc."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libpoker2_b200.so")
SOURCES = ["common.cu", "rank7.cu", "showdown.cu", "cfr.cu", "cfr_wide.cu", "cfr_iter.cu", "stepops.cu", "chance.cu", "treebuild.cu", "selftest.cu", "api.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    # The fp32 arithmetic of the CFR path must round like the separate multiply/add/divide
    # ops of the upstream PyTorch code: no fused multiply-add contraction.
    "-fmad=false",
    "-Xcompiler", "-fPIC",
]


def nvcc_path() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build poker2_b200")
    return cand


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    lib_m = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(PKG_DIR, "..", "include", "poker2_b200.h"))
    return any(os.path.getmtime(d) > lib_m for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB_PATH
    objs = []
    build_dir = os.path.join(PKG_DIR, "build")
    os.makedirs(build_dir, exist_ok=True)
    nvcc = nvcc_path()
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(PKG_DIR, "..", "include", "poker2_b200.h"))
    newest_header = max(os.path.getmtime(h) for h in headers)
    procs = []
    for src in SOURCES:
        obj = os.path.join(build_dir, src.replace(".cu", ".o"))
        objs.append(obj)
        src_path = os.path.join(CSRC, src)
        # an object is reused when it is newer than its source (cfr_wide.cu is cfr.cu compiled a second time)
        # and than every header
        newest_source = os.path.getmtime(src_path)
        if src == "cfr_wide.cu":
            newest_source = max(newest_source, os.path.getmtime(os.path.join(CSRC, "cfr.cu")))
        if not force and os.path.exists(obj) and os.path.getmtime(obj) > max(newest_source, newest_header):
            continue
        cmd = [nvcc, *NVCC_FLAGS, "-c", src_path, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    cmd = [nvcc, "-shared", "-Wno-deprecated-gpu-targets", "-o", LIB_PATH, *objs]
    subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
