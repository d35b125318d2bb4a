"""Builds the reference's own decode-attention kernels for the CPU.  TEST INFRASTRUCTURE ONLY.

    python -m oracle.build_ref [--reference /path/to/VTE] [--chunk-size 32]

The reference's kernels are HIP templates (vte/compiler/templates/rdna/*.hip.template).  The five
that make up the decode-attention path use nothing beyond the launch-geometry variables, shared
memory, __syncthreads, __expf and the half conversions, so they compile as host C++ against the
small stand-in headers in oracle/hip_cpu/hip/ and run with one CPU thread per GPU thread
(oracle/hip_cpu/harness.cpp).  This recipe

  1. reads the templates from where they lie in the reference checkout (nothing is copied into this
     repository: the instantiated sources live in oracle/_ref/ only while the compiler runs, the library
     stays there, and git ignores that directory),
  2. instantiates them the way the reference's CodegenEngine does (vte/compiler/codegen.py:12-22,
     `{{ split_kv_chunk_size }}` -> the number) and rewrites the two shared-memory declaration forms
     (`extern __shared__` -> `extern`, `__shared__` -> `static`: one block runs at a time, so a
     process-wide object is the block's shared memory),
  3. compiles them with g++ -O2 -ffp-contract=off (no fused multiply-add, as in the reference's numpy
     checks) together with the harness into oracle/_ref/libvte_ref_kernels_c<chunk>.so.

`oracle/ref_kernels.py` loads the library; tests/test_reference_kernels_cpu.py checks the numpy oracle
against it, and tests/golden/make_golden.py stores outputs of these kernels as fixtures that travel
to machines without the reference checkout.
"""
from __future__ import annotations

import argparse
import re
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
TEMPLATES = ("kv_cache_append", "flash_attention_split_kv_partial", "flash_attention_split_kv_reduce",
             "flash_attention", "rope")
DEFAULT_REFERENCE = Path("/root/reference")


def library_path(chunk_size: int) -> Path:
    return OUT / f"libvte_ref_kernels_c{int(chunk_size)}.so"


def instantiate(text: str, chunk_size: int) -> str:
    text = re.sub(r"\{\{\s*split_kv_chunk_size\s*\}\}", str(int(chunk_size)), text)
    if "{{" in text or "{%" in text:
        raise RuntimeError("template placeholder left uninstantiated")
    text = text.replace("extern __shared__", "extern")
    return re.sub(r"(?<![A-Za-z_])__shared__(?![A-Za-z_])", "static", text)


def build(reference: Path = DEFAULT_REFERENCE, chunk_size: int = 32, force: bool = False) -> Path:
    """Returns the library's path; raises FileNotFoundError when the reference checkout is absent."""
    tdir = Path(reference) / "vte" / "compiler" / "templates" / "rdna"
    lib = library_path(chunk_size)
    if lib.exists() and not force:
        return lib
    if not tdir.is_dir():
        raise FileNotFoundError(f"no reference templates under {tdir}")
    gxx = shutil.which("g++")
    if gxx is None:
        raise FileNotFoundError("g++ not found")
    gen = OUT / f"gen_c{int(chunk_size)}"
    gen.mkdir(parents=True, exist_ok=True)
    sources = []
    for name in TEMPLATES:
        dst = gen / f"{name}.cpp"
        dst.write_text(instantiate((tdir / f"{name}.hip.template").read_text(encoding="utf-8"), chunk_size), encoding="utf-8")
        sources.append(str(dst))
    cmd = [gxx, "-std=c++17", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-pthread",
           f"-DVTE_REF_SPLIT_KV_CHUNK_SIZE={int(chunk_size)}", f"-I{HERE / 'hip_cpu'}",
           "-o", str(lib), str(HERE / "hip_cpu" / "harness.cpp"), *sources]
    try:
        subprocess.run(cmd, check=True, capture_output=True, text=True)
    finally:
        shutil.rmtree(gen, ignore_errors=True)          # the instantiated reference sources are not kept
    return lib


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", type=Path, default=DEFAULT_REFERENCE)
    ap.add_argument("--chunk-size", type=int, action="append")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args(argv)
    for c in a.chunk_size or [32, 8]:
        try:
            print(build(a.reference, c, a.force))
        except subprocess.CalledProcessError as e:
            sys.stderr.write(e.stderr)
            return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
