"""Builds the C-ABI shared library (hand-written sm_100a CUDA) in-tree with nvcc.

    python skyrl-tx-rocm_b200/build.py [--force]

Output: skyrl-tx-rocm_b200/lib/libskyrl_w8a8_sm100.so
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
LIB_PATH = LIB_DIR / "libskyrl_w8a8_sm100.so"
SOURCES = ["api.cu", "quant_route_sm100.cu", "lora_a_proj_sm100.cu", "lora_rows_sm100.cu",
           "w8a8_gemm_sm100.cu", "tp_exchange_sm100.cu", "grad_quant_sm100.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return exe


def _digest() -> str:
    h = hashlib.sha256()
    for path in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.c")) +
                       list((PKG.parent / "include").glob("*.h"))):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build_library(force: bool = False, verbose: bool = False) -> Path:
    LIB_DIR.mkdir(exist_ok=True)
    stamp = LIB_DIR / "build.sha256"
    digest = _digest()
    if not force and LIB_PATH.exists() and stamp.exists() and stamp.read_text().strip() == digest:
        return LIB_PATH
    nvcc = _nvcc()
    objs = []
    procs = []
    for src in SOURCES:
        obj = LIB_DIR / (src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    for src, proc in procs:
        out, _ = proc.communicate()
        if verbose or proc.returncode:
            print(out)
        if proc.returncode:
            raise RuntimeError(f"nvcc failed on {src}")
    link = [nvcc, "-shared", "-o", str(LIB_PATH), *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    subprocess.run(link, check=True)
    build_abi_check()
    stamp.write_text(digest + "\n")
    return LIB_PATH


def build_abi_check() -> Path:
    """Plain-C consumer of the public header (csrc/abi_check.c), linked against the library."""
    gcc = shutil.which("gcc")
    if gcc is None:
        raise RuntimeError("gcc not found; the C-ABI check cannot be built")
    exe = LIB_DIR / "abi_check"
    subprocess.run([gcc, "-std=c11", "-Wall", "-Wextra", "-Werror", "-pedantic", str(CSRC / "abi_check.c"), "-o", str(exe),
                    f"-L{LIB_DIR}", "-lskyrl_w8a8_sm100", f"-Wl,-rpath,{LIB_DIR}", "-Wl,-rpath,$ORIGIN"], check=True)
    return exe


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
