"""Builds the native parts in-tree: `libvteb200.so` (the C-ABI shim with the
kernels linked in) and the cubin the dispatcher loads through the driver API.

    python -m vte_b200.build [--force] [--verbose]

Everything is compiled for sm_100a only
(`nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`).
"""
from __future__ import annotations

import argparse
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libvteb200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
ARCH = "sm_100a"


def _nvcc() -> str:
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _newer(target: Path, sources) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(s.stat().st_mtime <= t for s in sources)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    sources = [CSRC / "vteb200_shim.cu", *sorted((CSRC / "kernels").glob("*.cu*")),
               PKG.parent / "include" / "vteb200.h"]
    if not force and _newer(LIB, sources):
        return LIB
    cmd = [_nvcc(), *ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
           "-diag-suppress", "550", "-o", str(LIB), str(CSRC / "vteb200_shim.cu"), "-ldl"]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd))
    subprocess.run(cmd, check=True, capture_output=not verbose, text=True)
    return LIB


def build_cubins(force: bool = False) -> list[str]:
    """Ahead-of-time cubins for the default (split-count) build, in the content-hash
    cache the codegen engine reads."""
    from .compiler.codegen import CodegenEngine
    eng = CodegenEngine()
    return [eng.compile_kernel("decode_attention", ARCH, force_recompile=force)]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args(argv)
    lib = build_library(a.force, a.verbose)
    cubins = build_cubins(a.force)
    print(f"built {lib}")
    for c in cubins:
        print(f"built {c}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
