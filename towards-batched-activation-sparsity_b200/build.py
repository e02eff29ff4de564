"""Build libbas.so in-tree with nvcc for sm_100a (no JIT cache, no pip install).

    python towards-batched-activation-sparsity_b200/build.py [--force] [--verbose]

The shared library lands next to this file so that it travels with the source tree.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libbas.so"
SOURCES = ["bas_api.cu", "bas_gemv.cu", "bas_umma.cu", "bas_misc.cu", "bas_list.cu"]
HEADERS = [CSRC / "bas_common.cuh", CSRC / "bas_kernels.cuh", CSRC / "bas_trace.cuh", HERE.parent / "include" / "bas.h"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found; libbas needs the CUDA toolkit to build")
    return exe


def needs_build() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + HEADERS + [Path(__file__)]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, extra_flags=(), out: Path = LIB) -> Path:
    if not force and not needs_build() and out == LIB:
        return LIB
    objs = []
    build_dir = HERE / ("build" if out == LIB else "build_" + out.stem)
    build_dir.mkdir(exist_ok=True)
    common = [
        _nvcc(), "-std=c++17", "-O3", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    ]
    common += list(extra_flags)
    if verbose:
        common += ["-Xptxas", "-v"]
    procs = []
    for src in SOURCES:
        obj = build_dir / (Path(src).stem + ".o")
        objs.append(str(obj))
        procs.append((src, subprocess.Popen(common + ["-c", str(CSRC / src), "-o", str(obj)],
                                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        log, _ = p.communicate()
        if log.strip() and (verbose or p.returncode != 0):
            print(f"--- {src}\n{log}", file=sys.stderr)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed; see the messages above")
    subprocess.check_call([_nvcc(), "-shared", "-o", str(out)] + objs)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register / shared-memory usage")
    ap.add_argument("--define", action="append", default=[], help="extra -D macro (diagnostic builds)")
    ap.add_argument("--out", default=str(LIB), help="output path (diagnostic builds)")
    a = ap.parse_args()
    print(build(a.force or bool(a.define), a.verbose, ["-D" + d for d in a.define], Path(a.out)))
