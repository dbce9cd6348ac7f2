"""Compiles the CUDA sources under csrc/ into libpaged_decode_b200.so next to this file.

The library is a plain C-ABI shared object (include/paged_decode.h) built with nvcc for
sm_100a only; it does not link against torch.  ``python -m paged_decode_attention_b200.build``
rebuilds it; importing the package never compiles anything.
"""

from __future__ import annotations

import os
import pathlib
import shutil
import subprocess
import sys
import time

PKG = pathlib.Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libpaged_decode_b200.so"
SOURCES = ("pd_api.cu", "pd_stream.cu", "pd_stream_f16.cu", "pd_stream_bf16.cu", "pd_stream_e5m2.cu",
           "pd_stream_e5m2_scaled.cu", "pd_stream_i8.cu")
NVCC_FLAGS = (
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
)


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and pathlib.Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def needs_build() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(CSRC.iterdir()) + [PKG.parent / "include" / "paged_decode.h"])
    return LIB.stat().st_mtime < newest


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    if not force and not needs_build():
        return LIB
    started = time.time()
    objs = []
    tmp = PKG / "build"
    tmp.mkdir(exist_ok=True)
    procs = []
    for src in SOURCES:
        obj = tmp / (src + ".o")
        cmd = [_nvcc(), *NVCC_FLAGS, "-Xptxas", "-v" if verbose else "-warn-spills",
               "-c", str(CSRC / src), "-o", str(obj)]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    for src, proc in procs:
        out, _ = proc.communicate()
        if verbose or proc.returncode:
            sys.stderr.write(out)
        if proc.returncode:
            raise RuntimeError(f"nvcc failed on {src}")
    # link beside the target and rename: a reader never sees a half-written library
    fresh = LIB.with_suffix(".so.new")
    link = [_nvcc(), "-shared", "-o", str(fresh), *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    subprocess.run(link, check=True)
    # date the library at the start of the build: a source edited while the compiler ran is then
    # newer than the library, and the next call rebuilds instead of trusting a stale file
    os.utime(fresh, (started, started))
    os.replace(fresh, LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
