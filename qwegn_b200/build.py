"""Builds libqwcuda.so in place with nvcc for sm_100a (cross-compiles without a GPU).

    python -m qwegn_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libqwcuda.so")
SOURCES = ["qwc_api.cu", "qwc_dequant.cu", "qwc_gemv.cu"]
OPTIONAL_SOURCES = ["qwc_gemm_tc.cu", "qwc_moe.cu", "qwc_noalloc.cu", "qwc_norm.cu", "qwc_f32.cu", "qwc_ep.cu"]
HEADERS = ["qwc_common.cuh", os.path.join("..", "..", "include", "qwc.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; libqwcuda.so cannot be built")


def sources() -> list[str]:
    out = [os.path.join(CSRC, s) for s in SOURCES]
    out += [os.path.join(CSRC, s) for s in OPTIONAL_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    return out


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = sources() + [os.path.join(CSRC, h) for h in HEADERS] + [
        os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return LIB_PATH
    objs = []
    obj_dir = os.path.join(PKG_DIR, "build")
    os.makedirs(obj_dir, exist_ok=True)
    procs = []
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src).replace(".cu", ".o"))
        # QWC_NVCC_EXTRA (build time only): extra compiler flags, e.g. -DQWC_TUNING for a build whose launch code reads
        # its tuning knobs from the environment
        cmd = [_nvcc(), *NVCC_FLAGS, *os.environ.get("QWC_NVCC_EXTRA", "").split(), "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for cmd, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + out)
        if verbose or "warning" in out:
            sys.stderr.write(out)
    link = [_nvcc(), "-shared", "-o", LIB_PATH, *objs, "-Xcompiler", "-fPIC", "-lcudart"]
    subprocess.check_call(link)
    return LIB_PATH


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(LIB_PATH)
