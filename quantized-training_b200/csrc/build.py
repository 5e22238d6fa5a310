"""Builds libqt_b200.so (sm_100a only) next to the Python package that loads it.

    python quantized-training_b200/csrc/build.py [--force]

nvcc cross-compiles without a GPU. The library has no dependency on torch or libcuda at link
time (the driver entry point it needs is resolved at run time through the CUDA runtime).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
SOURCES = ["lib.cu", "quantize.cu", "producers.cu", "gemm_sm100.cu", "gemm_tile_sm100.cu", "optim.cu", "bitnet.cu"]
HEADERS = ["common.cuh", "tcgen05.cuh", "../../include/qt_b200.h"]
OUT = CSRC.parent / "gn_kernels" / "libqt_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return exe


def _stale() -> bool:
    if not OUT.exists():
        return True
    t = OUT.stat().st_mtime
    deps = [CSRC / s for s in SOURCES if (CSRC / s).exists()] + [CSRC / h for h in HEADERS] + [Path(__file__)]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu into one shared library; returns its path."""
    if not force and not _stale():
        return OUT
    nvcc = _nvcc()
    objdir = CSRC / "build"
    objdir.mkdir(exist_ok=True)
    objs = []
    procs = []
    for src in SOURCES:
        if not (CSRC / src).exists():
            continue
        obj = objdir / (src + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    for src, proc in procs:
        out, _ = proc.communicate()
        if verbose and out:
            print(out)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
    link = [nvcc, "-shared", "-o", str(OUT), *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}")
    return OUT


CHECK_OUT = CSRC.parent / "gn_kernels" / "libqt_b200_check.so"
CHECKED_SOURCES = ["quantize.cu"]   # the translation units that carry store guards


def build_checked(force: bool = False) -> Path:
    """The debug library: the same code with -DQT_BOUNDS_CHECK on the sources that carry store guards (every
    global store of the quantize kernels checks its address against the ranges its entry point declared and
    reports through the device status word instead of writing outside them). The other objects are the
    release ones, so build() runs first."""
    build(force=False)
    deps = [CSRC / s for s in CHECKED_SOURCES] + [CSRC / h for h in HEADERS] + [Path(__file__), OUT]
    if not force and CHECK_OUT.exists() and all(d.stat().st_mtime <= CHECK_OUT.stat().st_mtime for d in deps):
        return CHECK_OUT
    nvcc = _nvcc()
    objdir = CSRC / "build"
    objs = []
    for src in SOURCES:
        if src in CHECKED_SOURCES:
            obj = objdir / (src + ".check.o")
            res = subprocess.run([nvcc, *NVCC_FLAGS, "-DQT_BOUNDS_CHECK", "-c", str(CSRC / src), "-o", str(obj)],
                                 stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src} (checked build):\n{res.stdout}")
        else:
            obj = objdir / (src + ".o")
        objs.append(str(obj))
    res = subprocess.run([nvcc, "-shared", "-o", str(CHECK_OUT), *objs, "-gencode", "arch=compute_100a,code=sm_100a"],
                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed (checked build):\n{res.stdout}")
    return CHECK_OUT


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
    if "--checked" in sys.argv:
        print(build_checked(force="--force" in sys.argv))
