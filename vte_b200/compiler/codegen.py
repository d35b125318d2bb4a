"""Kernel "compiler": hand-written .cu -> cubin with nvcc, cached by content hash.

Stands in for vte/compiler/codegen.py:52-311.  The reference renders a HIP
template, hashes the rendered text, and calls `hipcc --genco`; here the source
is a fixed `.cu` file, the template parameters become `-D` macros (sanitised
the same way, codegen.py:12-22), the cache key is the sha256 of the sources
plus the macro list (codegen.py:47-50), and the compiler is
`nvcc -gencode arch=compute_100a,code=sm_100a -cubin`.  `load_kernel_safe`
keeps the reference's contract (codegen.py:283-311): compile or reuse, load,
and on a load failure recompile once and try again.
"""
from __future__ import annotations

import hashlib
import logging
import os
import re
import shutil
import subprocess
from pathlib import Path

from ..bridge.errors import CudaSafetyError
from .signatures import TEMPLATE_SOURCES

logger = logging.getLogger(__name__)

KERNEL_DIR = Path(__file__).resolve().parent.parent / "csrc" / "kernels"
CACHE_DIR = Path(__file__).resolve().parent / "cache"


def _sanitize_var(value) -> str:
    """Only numbers and [A-Za-z0-9_] strings may reach the compiler command line."""
    if isinstance(value, bool):
        return "1" if value else "0"
    if isinstance(value, (int, float)):
        return str(value)
    if isinstance(value, str):
        if not re.fullmatch(r"[A-Za-z0-9_]+", value):
            raise CudaSafetyError(f"unsafe template variable blocked: {value!r}")
        return value
    raise CudaSafetyError(f"unsupported template variable type: {type(value)}")


def _arch_flags(arch: str) -> list[str]:
    m = re.fullmatch(r"sm_(\d+a?)", arch)
    if not m:
        raise CudaSafetyError(f"unsupported architecture string {arch!r}")
    if m.group(1) != "100a":
        raise CudaSafetyError(f"these kernels are written for sm_100a only, not {arch}")
    return ["-gencode", "arch=compute_100a,code=sm_100a"]


class CodegenEngine:
    def __init__(self, cache_dir: Path | None = None, nvcc: str | None = None):
        self.kernel_dir = KERNEL_DIR
        self.cache_dir = Path(cache_dir) if cache_dir else CACHE_DIR
        self.cache_dir.mkdir(parents=True, exist_ok=True)
        self.nvcc = nvcc or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"

    def _source_for(self, template_name: str) -> Path:
        fname = TEMPLATE_SOURCES.get(template_name)
        if fname is None:
            raise CudaSafetyError(f"unknown kernel template {template_name!r}")
        return self.kernel_dir / fname

    @staticmethod
    def _defines(params: dict) -> list[str]:
        """-D macros from the template parameters, plus (development switch) those named in the
        environment variable VTEB_KERNEL_DEFINES as `name=value,name=value`; both are sanitised and
        both enter the cache key."""
        merged = dict(params)
        for item in filter(None, os.environ.get("VTEB_KERNEL_DEFINES", "").split(",")):
            k, _, v = item.partition("=")
            merged[k.strip()] = int(v) if v.strip().lstrip("-").isdigit() else v.strip()
        return [f"-D{_sanitize_var(k).upper()}={_sanitize_var(v)}" for k, v in sorted(merged.items())]

    def cache_path(self, template_name: str, arch: str, **params) -> Path:
        """cache/<arch>/kernel_<sha256[:16]>.cubin, keyed by every source the
        translation unit includes and by the macro values."""
        src = self._source_for(template_name)
        h = hashlib.sha256()
        for f in sorted(self.kernel_dir.glob("*.cu*")):
            h.update(f.name.encode())
            h.update(f.read_bytes())
        h.update(src.name.encode())
        h.update(" ".join(self._defines(params)).encode())
        return self.cache_dir / arch / f"kernel_{h.hexdigest()[:16]}.cubin"

    def compile_kernel(self, template_name: str, arch: str, force_recompile: bool = False, **params) -> str:
        out = self.cache_path(template_name, arch, **params)
        if out.exists() and not force_recompile:
            return str(out)
        out.parent.mkdir(parents=True, exist_ok=True)
        src = self._source_for(template_name)
        cmd = [self.nvcc, *_arch_flags(arch), "-O3", "-std=c++17", "-lineinfo", "-cubin",
               *self._defines(params), "-o", str(out), str(src)]
        logger.info("compiling %s: %s", template_name, " ".join(cmd))
        try:
            subprocess.run(cmd, check=True, capture_output=True, text=True)
        except FileNotFoundError as e:
            raise CudaSafetyError(f"nvcc not found ({self.nvcc}); cannot build {src.name}") from e
        except subprocess.CalledProcessError as e:
            raise CudaSafetyError(f"nvcc failed for {src.name} ({arch}):\n{e.stderr}") from e
        return str(out)

    def load_kernel_safe(self, hip, template_name: str, arch: str, kernel_name: str, **kwargs):
        path = self.compile_kernel(template_name, arch, **kwargs)
        try:
            return hip.load_kernel(path, kernel_name)
        except Exception as e:
            logger.warning("loading %s failed (%s); recompiling once", path, e)
            path = self.compile_kernel(template_name, arch, force_recompile=True, **kwargs)
            return hip.load_kernel(path, kernel_name)
