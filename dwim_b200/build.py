"""Builds ``libdwim_b200.so`` in place with nvcc, for sm_100a only.

    python -m dwim_b200.build [--verbose]

The library is kept in the package directory so that it travels with the
source tree; nothing is installed into site-packages.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libdwim_b200.so"
SOURCES = ["abi.cu", "codec.cu", "prologue.cu", "gemv.cu", "gemm.cu", "static_scratch.cu", "peer.cu", "neighbours.cu"]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "dwim_b200.h"]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIB
    obj_dir = PKG / "build"
    obj_dir.mkdir(exist_ok=True)
    host_cc = "/usr/bin/g++" if Path("/usr/bin/g++").exists() else "g++"
    common = [nvcc(), "-ccbin", host_cc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr"]
    if verbose:
        common += ["-Xptxas", "-v"]
    objs = []
    procs = []
    for src in SOURCES:
        obj = obj_dir / (src + ".o")
        objs.append(str(obj))
        procs.append((src, subprocess.Popen(common + ["-c", str(CSRC / src), "-o", str(obj)],
                                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(f"--- {src}\n{out}\n")
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    subprocess.run([nvcc(), "-ccbin", host_cc, "-shared", "-o", str(LIB)] + objs + ["-cudart", "static"], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True, verbose="--verbose" in sys.argv))
