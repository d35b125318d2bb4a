"""`CudaRuntime`: the Python face of libvteb200.so.

It keeps the method names, argument order and error behaviour of the wrapper
it replaces, `HIPRuntime` (vte/bridge/hip_runtime.py:155-1089), so dispatcher
and executor code written against that class runs unchanged: tracked
allocations with bounds-checked copies (:586-762), `load_kernel` (:793),
`launch_kernel` with its argument-count check (:805-867),
`launch_kernel_recorded` with its different argument order (:869-907), stream
capture and graph calls (:991-1038), events (:319-340), `synchronize` under a
host watchdog (:909-929), `cleanup` and the context-manager protocol
(:1040-1089).  Differences, all forced by CUDA: dynamic shared memory above
48 KB needs an opt-in on the function, which `launch_*` applies on demand, and
launches can carry the programmatic-dependent-launch attribute.

There is no CPU fallback.  Without the shared library or without a CUDA
device, construction or `initialize()` raises.
"""
from __future__ import annotations

import ctypes
import logging
import os
import threading
from pathlib import Path
from typing import Optional

from ..config import (MAX_ALLOCATION_SIZE, MAX_GRID_DIMENSIONS, VRAM_USAGE_LIMIT, DEFAULT_SYNC_TIMEOUT_S,
                      ENV_DEVICE_INDEX)
from .errors import CudaRuntimeError, CudaSafetyError, MemoryGuardianOOMError

logger = logging.getLogger(__name__)

_LIB_NAME = "libvteb200.so"

ATTR_SM_COUNT = 0
ATTR_MAX_THREADS_PER_BLOCK = 1
ATTR_MAX_SMEM_PER_BLOCK = 2
ATTR_MAX_SMEM_PER_BLOCK_OPTIN = 3
ATTR_CC_MAJOR = 4
ATTR_CC_MINOR = 5
ATTR_L2_BYTES = 6
ATTR_CLOCK_KHZ = 7

LAUNCH_PROGRAMMATIC = 1

ATTN_COMPAT = 1
ATTN_WRITE_EMPTY_O = 2
ATTN_PROGRAMMATIC = 4
ATTN_COMPACT = 16
ATTN_NO_TENSOR_MAPS = 32
ATTN_BALANCED = 64
ATTN_SHORT_SPLITS = 128

ERR_DEVICE_STATUS = -6


class FastPlan(ctypes.Structure):
    """Mirror of `vteb_fast_plan` (include/vteb200.h)."""
    _fields_ = [("ok", ctypes.c_int), ("hg", ctypes.c_int), ("n_hgroups", ctypes.c_int),
                ("tile", ctypes.c_int), ("nstages", ctypes.c_int), ("smem_bytes", ctypes.c_int),
                ("threads", ctypes.c_int), ("combine_dsplit", ctypes.c_int),
                ("combine_smem_bytes", ctypes.c_int)]


class KvTensorMap(ctypes.Structure):
    """The 128-byte tensor map of a K or V cache, passed to the fast split kernels by value."""
    _fields_ = [("opaque", ctypes.c_uint64 * 16)]


def default_library_path() -> Path:
    return Path(__file__).resolve().parent.parent / _LIB_NAME


def _declare(lib):
    """Argument and result types of every entry point of include/vteb200.h."""
    vp, vpp = ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)
    i, ip, u = ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.c_uint
    sz, szp = ctypes.c_size_t, ctypes.POINTER(ctypes.c_size_t)
    f, ll, ull = ctypes.c_float, ctypes.c_longlong, ctypes.c_ulonglong
    sigs = {
        "vteb_last_error_string": (ctypes.c_char_p, []),
        "vteb_version": (i, []),
        "vteb_device_count": (i, [ip]),
        "vteb_init": (i, [i]),
        "vteb_current_device": (i, [ip]),
        "vteb_device_attr": (i, [i, i, ip]),
        "vteb_device_name": (i, [i, ctypes.c_char_p, i]),
        "vteb_mem_info": (i, [szp, szp]),
        "vteb_device_synchronize": (i, []),
        "vteb_malloc": (i, [vpp, sz]),
        "vteb_free": (i, [vp]),
        "vteb_memcpy_h2d": (i, [vp, vp, sz]),
        "vteb_memcpy_d2h": (i, [vp, vp, sz]),
        "vteb_memcpy_d2d": (i, [vp, vp, sz]),
        "vteb_memcpy_h2d_async": (i, [vp, vp, sz, vp]),
        "vteb_memcpy_d2h_async": (i, [vp, vp, sz, vp]),
        "vteb_memset": (i, [vp, i, sz]),
        "vteb_memset_async": (i, [vp, i, sz, vp]),
        "vteb_host_alloc": (i, [vpp, sz]),
        "vteb_host_free": (i, [vp]),
        "vteb_module_load": (i, [vpp, ctypes.c_char_p]),
        "vteb_module_get_function": (i, [vpp, vp, ctypes.c_char_p]),
        "vteb_module_unload": (i, [vp]),
        "vteb_func_set_max_dynamic_smem": (i, [vp, i]),
        "vteb_func_set_shared_carveout": (i, [vp, i]),
        "vteb_launch": (i, [vp, u, u, u, u, u, u, u, vp, vpp, u]),
        "vteb_stream_create": (i, [vpp]),
        "vteb_stream_destroy": (i, [vp]),
        "vteb_stream_synchronize": (i, [vp]),
        "vteb_stream_begin_capture": (i, [vp, i]),
        "vteb_stream_end_capture": (i, [vp, vpp]),
        "vteb_graph_instantiate": (i, [vpp, vp]),
        "vteb_graph_launch": (i, [vp, vp]),
        "vteb_graph_destroy": (i, [vp]),
        "vteb_graph_exec_destroy": (i, [vp]),
        "vteb_graph_node_count": (i, [vp, szp]),
        "vteb_event_create": (i, [vpp]),
        "vteb_event_record": (i, [vp, vp]),
        "vteb_event_synchronize": (i, [vp]),
        "vteb_event_elapsed_ms": (i, [ctypes.POINTER(f), vp, vp]),
        "vteb_event_destroy": (i, [vp]),
        "vteb_nccl_unique_id": (i, [vp]),
        "vteb_nccl_comm_init_rank": (i, [vpp, i, vp, i]),
        "vteb_nccl_all_gather_f32": (i, [vp, vp, vp, sz, vp]),
        "vteb_nccl_all_reduce_max_f32": (i, [vp, vp, vp, sz, vp]),
        "vteb_nccl_comm_destroy": (i, [vp]),
        "vteb_ipc_get_handle": (i, [vp, vp]),
        "vteb_ipc_open_handle": (i, [vp, vpp]),
        "vteb_ipc_close_handle": (i, [vp]),
        "vteb_split_kv_plan": (i, [i, i, i, ctypes.POINTER(FastPlan)]),
        "vteb_split_kv_plan_compact": (i, [i, i, i, ctypes.POINTER(FastPlan)]),
        "vteb_kv_tensor_map": (i, [vp, vp, ctypes.c_longlong, i, i]),
        "vteb_combine_rows_epl": (i, [i, i]),
        "vteb_split_kv_decode": (i, [vp, vp, vp, vp, vp, i, vp, vp, vp, vp, i, i, i, i, f, ll, i, i, u, i, vp]),
        "vteb_split_kv_decode_noalloc": (i, [vp, vp, vp, vp, vp, i, i, i, i, i, f, ll, i, i, u, i, vp]),
        "vteb_kv_cache_append": (i, [vp, vp, vp, vp, vp, i, i, i, ll, vp]),
        "vteb_check_status": (i, [vp, vp]),
        "vteb_noalloc_check_status": (i, [vp]),
        "vteb_fill_normal_f16": (i, [vp, sz, ull, f, f, f, vp]),
        "vteb_read_bandwidth_probe": (i, [vp, sz, vp, i, vp]),
    }
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return sorted(sigs)


EXPORTED_SYMBOLS: list[str] = []


def load_library(path: Optional[str] = None):
    """dlopen the shim and declare its prototypes.  Raises CudaRuntimeError if the
    file is missing: the product has no other way to reach the device."""
    lib_path = Path(path) if path else default_library_path()
    if not lib_path.exists():
        raise CudaRuntimeError(
            f"{lib_path} not found. Build it with `python -m vte_b200.build` "
            f"(nvcc -gencode arch=compute_100a,code=sm_100a); there is no CPU fallback.")
    lib = ctypes.CDLL(str(lib_path))
    names = _declare(lib)
    if not EXPORTED_SYMBOLS:
        EXPORTED_SYMBOLS.extend(names)
    return lib


def _ptr_value(p) -> int:
    if isinstance(p, ctypes.c_void_p):
        return p.value or 0
    if hasattr(p, "ptr"):
        return int(p.ptr)
    return int(p or 0)


class CudaRuntime:
    """One device, one stream, tracked allocations.  Not thread-safe (like the
    wrapper it mirrors): launches are made from one thread."""

    _process_wide_allocated_bytes = 0
    _live_instance_count = 0
    # Device-to-host copies are refused unless the tag names one of these
    # (hip_runtime.py:732-736: only results may leave the device).
    D2H_ALLOWED_TAGS = ("logits", "output", "sampler")

    def __init__(self, library_path: Optional[str] = None, device_index: Optional[int] = None,
                 sync_timeout_s: float = DEFAULT_SYNC_TIMEOUT_S):
        self._lib = load_library(library_path)
        self._initialized = False
        self._in_cleanup_mode = False
        self._counted_as_live = False
        self._active_allocations: dict[int, tuple[int, str]] = {}
        self._host_allocations: dict[int, int] = {}
        self._modules: list[int] = []
        self._stream = ctypes.c_void_p()
        self._device_index = device_index
        self._vram_total = 0
        self._props: dict = {}
        self._smem_optin_set: dict[int, int] = {}
        self._signatures: dict[int, tuple[str, int]] = {}
        self._panic = False
        self._sync_timeout_s = sync_timeout_s
        self.programmatic_launch = False   # when True, recorded launches carry the PDL attribute

    # ------------------------------------------------------------------ errors
    def _last_error(self) -> str:
        msg = self._lib.vteb_last_error_string()
        return msg.decode("utf-8", "replace") if msg else ""

    def _check_error(self, err: int, context: str):
        if err != 0:
            raise CudaRuntimeError(f"{context} returned code {err}: {self._last_error()}", code=err)

    def _require_init(self):
        if not self._initialized:
            raise CudaSafetyError("CUDA operation requires initialisation (call initialize()).")

    # ------------------------------------------------------------------ device
    def _select_device_index(self) -> int:
        """Explicit argument, then VTE_DEVICE_INDEX, then LOCAL_RANK, then 0
        (hip_runtime.py:346-434 chooses one device; multi-GPU runs use one
        process per device)."""
        if self._device_index is not None:
            return int(self._device_index)
        for key in (ENV_DEVICE_INDEX, "LOCAL_RANK"):
            v = os.environ.get(key)
            if v not in (None, ""):
                try:
                    return int(v)
                except ValueError:
                    raise CudaSafetyError(f"{key}={v!r} is not a device index")
        return 0

    def initialize(self) -> bool:
        if self._initialized:
            return True
        count = ctypes.c_int(0)
        self._check_error(self._lib.vteb_device_count(ctypes.byref(count)), "cudaGetDeviceCount")
        if count.value <= 0:
            raise CudaRuntimeError("no CUDA device is visible; this path has no CPU fallback")
        idx = self._select_device_index()
        if not (0 <= idx < count.value):
            raise CudaSafetyError(f"device index {idx} out of range (0..{count.value - 1})")
        self._check_error(self._lib.vteb_init(idx), "vteb_init")
        self._device_index = idx
        self._check_error(self._lib.vteb_stream_create(ctypes.byref(self._stream)), "cudaStreamCreate")
        self._initialized = True
        self._props = self._query_properties(idx)
        free_b, total_b = self.get_real_mem_info()
        self._vram_total = total_b
        CudaRuntime._live_instance_count += 1
        self._counted_as_live = True
        logger.info("CUDA device %d: %s, %d SMs, %.1f GB", idx, self._props["name"],
                    self._props["multi_processor_count"], total_b / 2 ** 30)
        return True

    def _attr(self, attr_id: int, device: Optional[int] = None) -> int:
        v = ctypes.c_int(0)
        dev = self._device_index if device is None else device
        self._check_error(self._lib.vteb_device_attr(dev, attr_id, ctypes.byref(v)), "cudaDeviceGetAttribute")
        return v.value

    def _query_properties(self, device: int) -> dict:
        name = ctypes.create_string_buffer(256)
        self._check_error(self._lib.vteb_device_name(device, name, 256), "cudaGetDeviceProperties")
        return {
            "name": name.value.decode("utf-8", "replace"),
            "multi_processor_count": self._attr(ATTR_SM_COUNT, device),
            "max_threads_per_block": self._attr(ATTR_MAX_THREADS_PER_BLOCK, device),
            "shared_mem_per_block": self._attr(ATTR_MAX_SMEM_PER_BLOCK, device),
            "shared_mem_per_block_optin": self._attr(ATTR_MAX_SMEM_PER_BLOCK_OPTIN, device),
            "compute_capability": (self._attr(ATTR_CC_MAJOR, device), self._attr(ATTR_CC_MINOR, device)),
            "l2_bytes": self._attr(ATTR_L2_BYTES, device),
            "clock_khz": self._attr(ATTR_CLOCK_KHZ, device),
        }

    def get_device_properties(self, device_id: Optional[int] = None) -> dict:
        self._require_init()
        if device_id is None or device_id == self._device_index:
            return dict(self._props)
        return self._query_properties(device_id)

    def get_num_cus(self) -> int:
        """Streaming-multiprocessor count (hip_runtime.py:538-547 returns the
        compute-unit count; there it feeds the chunk-size rule)."""
        self._require_init()
        return int(self._props["multi_processor_count"])

    def get_gpu_architecture(self) -> str:
        """`sm_<major><minor>a`, the string handed to nvcc (hip_runtime.py:549-563
        returns the gfx name handed to hipcc)."""
        self._require_init()
        major, minor = self._props["compute_capability"]
        return f"sm_{major}{minor}a"

    def get_real_mem_info(self) -> tuple[int, int]:
        self._require_init()
        free_b, total_b = ctypes.c_size_t(0), ctypes.c_size_t(0)
        self._check_error(self._lib.vteb_mem_info(ctypes.byref(free_b), ctypes.byref(total_b)), "cudaMemGetInfo")
        return free_b.value, total_b.value

    @property
    def stream(self) -> ctypes.c_void_p:
        return self._stream

    @property
    def device_index(self) -> int:
        return int(self._device_index or 0)

    # ------------------------------------------------------------------ memory
    def safe_malloc(self, size_bytes: int, tag: str = "unnamed") -> ctypes.c_void_p:
        self._require_init()
        if size_bytes <= 0:
            raise CudaSafetyError(f"invalid allocation size: {size_bytes} bytes")
        if size_bytes > MAX_ALLOCATION_SIZE:
            raise CudaSafetyError(f"allocation above the maximum: {size_bytes} > {MAX_ALLOCATION_SIZE}")
        reserved = CudaRuntime._process_wide_allocated_bytes
        if reserved + size_bytes > self._vram_total * VRAM_USAGE_LIMIT:
            raise MemoryGuardianOOMError(
                f"allocating {size_bytes} bytes [{tag}] would exceed {VRAM_USAGE_LIMIT:.0%} of device memory "
                f"({self._vram_total} bytes); already reserved by this process: {reserved} bytes")
        try:
            real_free, real_total = self.get_real_mem_info()
            if size_bytes > real_free - int(real_total * (1.0 - VRAM_USAGE_LIMIT)):
                raise MemoryGuardianOOMError(
                    f"allocating {size_bytes} bytes [{tag}] would pass {VRAM_USAGE_LIMIT:.0%} real usage of the "
                    f"device (free now: {real_free} of {real_total} bytes)")
        except CudaRuntimeError as e:   # best effort, as in the reference
            logger.warning("cudaMemGetInfo failed, skipping the real-usage check: %s", e)
        ptr = ctypes.c_void_p()
        err = self._lib.vteb_malloc(ctypes.byref(ptr), size_bytes)
        if err == 2:   # cudaErrorMemoryAllocation
            raise MemoryGuardianOOMError(f"cudaMalloc ran out of memory ({size_bytes} bytes, [{tag}])")
        self._check_error(err, "cudaMalloc")
        if not ptr.value:
            raise CudaSafetyError("cudaMalloc returned a null pointer with status 0")
        self._active_allocations[ptr.value] = (size_bytes, tag)
        CudaRuntime._process_wide_allocated_bytes += size_bytes
        return ptr

    def safe_free(self, ptr, tag: str = "unnamed") -> bool:
        val = _ptr_value(ptr)
        if val not in self._active_allocations:
            if self._in_cleanup_mode:
                logger.warning("untracked pointer 0x%016X during cleanup [%s]", val, tag)
                return False
            raise CudaSafetyError(f"attempt to free an untracked pointer 0x{val:016X} [{tag}] "
                                  f"(use after free or corruption)")
        size_bytes, _ = self._active_allocations[val]
        self._check_error(self._lib.vteb_free(ctypes.c_void_p(val)), "cudaFree")
        del self._active_allocations[val]
        CudaRuntime._process_wide_allocated_bytes = max(0, CudaRuntime._process_wide_allocated_bytes - size_bytes)
        return True

    def _containing_allocation(self, addr: int, nbytes: int, what: str, tag: str) -> None:
        for base, (size, _) in self._active_allocations.items():
            if base <= addr < base + size:
                if addr + nbytes > base + size:
                    raise CudaSafetyError(f"{what} overflow: {nbytes} bytes at 0x{addr:016X} cross the end of "
                                          f"the allocation [{tag}]")
                return
        raise CudaSafetyError(f"{what}: untracked device pointer 0x{addr:016X} [{tag}]")

    @staticmethod
    def _host_view(buf, writable: bool):
        """(address, nbytes, keepalive) of a bytes-like or numpy host buffer."""
        if hasattr(buf, "__array_interface__"):
            import numpy as np
            arr = np.ascontiguousarray(buf) if not writable else buf
            if writable and not arr.flags["C_CONTIGUOUS"]:
                raise CudaSafetyError("destination host array must be C-contiguous")
            return arr.ctypes.data, arr.nbytes, arr
        if isinstance(buf, (bytes, bytearray, memoryview)):
            n = len(buf)
            if writable:
                if isinstance(buf, bytes):
                    raise CudaSafetyError("destination host buffer must be writable (bytearray)")
                c = (ctypes.c_char * n).from_buffer(buf)
            else:
                c = (ctypes.c_char * n).from_buffer_copy(buf) if n else (ctypes.c_char * 1)()
            return ctypes.addressof(c), n, c
        raise CudaSafetyError(f"unsupported host buffer type {type(buf)}")

    def safe_memcpy_host_to_device(self, dst, src, tag: str = "unnamed") -> bool:
        """`src` is bytes-like (as in the reference) or a numpy array."""
        self._require_init()
        addr, n, keep = self._host_view(src, writable=False)
        if n == 0:
            return True
        dval = _ptr_value(dst)
        self._containing_allocation(dval, n, "memcpy_h2d", tag)
        self._check_error(self._lib.vteb_memcpy_h2d(ctypes.c_void_p(dval), ctypes.c_void_p(addr), n), "cudaMemcpy (H2D)")
        return True

    def safe_memset(self, dst, size_bytes: int, tag: str = "unnamed", value: int = 0) -> bool:
        self._require_init()
        if size_bytes <= 0:
            raise CudaSafetyError(f"memset of {size_bytes} bytes [{tag}]")
        dval = _ptr_value(dst)
        self._containing_allocation(dval, size_bytes, "memset", tag)
        self._check_error(self._lib.vteb_memset(ctypes.c_void_p(dval), int(value) & 0xFF, size_bytes), "cudaMemset")
        return True

    def safe_memcpy_device_to_host(self, dst, src, tag: str = "unnamed") -> bool:
        """`dst` is a bytearray (as in the reference) or a writable numpy array."""
        self._require_init()
        if not any(word in tag for word in self.D2H_ALLOWED_TAGS):
            raise CudaSafetyError(f"device-to-host copy refused for tag [{tag}]: only results "
                                  f"({', '.join(self.D2H_ALLOWED_TAGS)}) may leave the device")
        addr, n, keep = self._host_view(dst, writable=True)
        if n == 0:
            return True
        sval = _ptr_value(src)
        self._containing_allocation(sval, n, "memcpy_d2h", tag)
        self._check_error(self._lib.vteb_memcpy_d2h(ctypes.c_void_p(addr), ctypes.c_void_p(sval), n), "cudaMemcpy (D2H)")
        return True

    # Pinned staging buffers and asynchronous copies: used by the decode-step
    # driver, which must not synchronise between the copy and the graph launch.
    def host_alloc(self, size_bytes: int) -> ctypes.c_void_p:
        self._require_init()
        if size_bytes <= 0:
            raise CudaSafetyError(f"invalid pinned allocation size: {size_bytes}")
        p = ctypes.c_void_p()
        self._check_error(self._lib.vteb_host_alloc(ctypes.byref(p), size_bytes), "cudaHostAlloc")
        self._host_allocations[p.value] = size_bytes
        return p

    def host_free(self, ptr) -> None:
        val = _ptr_value(ptr)
        if val not in self._host_allocations:
            raise CudaSafetyError(f"untracked pinned pointer 0x{val:016X}")
        self._check_error(self._lib.vteb_host_free(ctypes.c_void_p(val)), "cudaFreeHost")
        del self._host_allocations[val]

    def memcpy_h2d_async(self, dst, src_host_ptr, nbytes: int, tag: str = "unnamed") -> None:
        self._require_init()
        dval = _ptr_value(dst)
        self._containing_allocation(dval, nbytes, "memcpy_h2d_async", tag)
        self._check_error(self._lib.vteb_memcpy_h2d_async(ctypes.c_void_p(dval), ctypes.c_void_p(_ptr_value(src_host_ptr)),
                                                          nbytes, self._stream), "cudaMemcpyAsync (H2D)")

    def memcpy_d2h_async(self, dst_host_ptr, src, nbytes: int, tag: str = "output") -> None:
        self._require_init()
        sval = _ptr_value(src)
        self._containing_allocation(sval, nbytes, "memcpy_d2h_async", tag)
        self._check_error(self._lib.vteb_memcpy_d2h_async(ctypes.c_void_p(_ptr_value(dst_host_ptr)), ctypes.c_void_p(sval),
                                                          nbytes, self._stream), "cudaMemcpyAsync (D2H)")

    def memset_async(self, dst, size_bytes: int, value: int = 0, tag: str = "unnamed") -> None:
        self._require_init()
        dval = _ptr_value(dst)
        self._containing_allocation(dval, size_bytes, "memset_async", tag)
        self._check_error(self._lib.vteb_memset_async(ctypes.c_void_p(dval), int(value) & 0xFF, size_bytes, self._stream),
                          "cudaMemsetAsync")

    # ------------------------------------------------------------------ kernels
    def load_kernel(self, cubin_path: str, kernel_name: str):
        """Load a cubin and return (module, function) as c_void_p."""
        self._require_init()
        module, function = ctypes.c_void_p(), ctypes.c_void_p()
        self._check_error(self._lib.vteb_module_load(ctypes.byref(module), str(cubin_path).encode("utf-8")), "cuModuleLoad")
        self._modules.append(module.value)
        self._check_error(self._lib.vteb_module_get_function(ctypes.byref(function), module, kernel_name.encode("utf-8")),
                          "cuModuleGetFunction")
        from ..compiler.signatures import KERNEL_SIGNATURES
        if kernel_name in KERNEL_SIGNATURES:
            self._signatures[function.value] = (kernel_name, len(KERNEL_SIGNATURES[kernel_name]))
            # Every kernel of the attention path asks for the same (maximum) shared-memory
            # carve-out: the SMs then never have to drain to re-split L1 / shared memory
            # between the split launch and the small launches around it.
            self._check_error(self._lib.vteb_func_set_shared_carveout(function, 100), "cuFuncSetAttribute")
        return module, function

    def register_kernel_signature(self, function, name: str, n_args: int) -> None:
        self._signatures[_ptr_value(function)] = (name, n_args)

    def _validate_launch(self, function, grid, block, shared_mem: int, n_args: int):
        self._require_init()
        if self._panic:
            raise CudaSafetyError("runtime is in panic state (a synchronize timed out); new launches are blocked")
        if len(grid) != 3 or any(int(g) <= 0 for g in grid):
            raise CudaSafetyError(f"invalid grid dims: {grid}")
        if len(block) != 3 or any(int(b) <= 0 for b in block):
            raise CudaSafetyError(f"invalid block dims: {block}")
        total_grid = int(grid[0]) * int(grid[1]) * int(grid[2])
        if total_grid > MAX_GRID_DIMENSIONS:
            raise CudaSafetyError(f"grid of {total_grid} blocks exceeds the limit {MAX_GRID_DIMENSIONS}")
        total_block = int(block[0]) * int(block[1]) * int(block[2])
        if total_block > self._props["max_threads_per_block"]:
            raise CudaSafetyError(f"block size {total_block} exceeds max_threads_per_block "
                                  f"{self._props['max_threads_per_block']}")
        if shared_mem < 0 or shared_mem > self._props["shared_mem_per_block_optin"]:
            raise CudaSafetyError(f"shared memory {shared_mem} exceeds the device maximum "
                                  f"{self._props['shared_mem_per_block_optin']}")
        fval = _ptr_value(function)
        if not fval:
            raise CudaSafetyError("null kernel function")
        sig = self._signatures.get(fval)
        if sig is not None and sig[1] != n_args:
            raise CudaSafetyError(f"ABI mismatch: kernel {sig[0]} takes {sig[1]} arguments, got {n_args}")
        if shared_mem > self._props["shared_mem_per_block"] and self._smem_optin_set.get(fval, 0) < shared_mem:
            self._check_error(self._lib.vteb_func_set_max_dynamic_smem(ctypes.c_void_p(fval), int(shared_mem)),
                              "cuFuncSetAttribute")
            self._smem_optin_set[fval] = int(shared_mem)

    @staticmethod
    def _marshal(args: list):
        """void*[] of pointers to the argument values.  ctypes scalars are passed
        by reference; a bare Python int is taken as a 64-bit value, as
        launch_kernel_recorded does in the reference (hip_runtime.py:886-895)."""
        keep = []
        arr = (ctypes.c_void_p * max(1, len(args)))()
        for i, a in enumerate(args):
            if isinstance(a, int) and not isinstance(a, bool):
                a = ctypes.c_uint64(a)
            elif not isinstance(a, ctypes._SimpleCData) and not isinstance(a, ctypes.Structure):
                raise CudaSafetyError(f"kernel argument {i} has unsupported type {type(a)}")
            keep.append(a)
            arr[i] = ctypes.cast(ctypes.byref(a), ctypes.c_void_p)
        return arr, keep

    def _launch(self, function, grid, block, args, shared_mem: int, flags: int):
        arr, keep = self._marshal(args)
        err = self._lib.vteb_launch(ctypes.c_void_p(_ptr_value(function)), int(grid[0]), int(grid[1]), int(grid[2]),
                                    int(block[0]), int(block[1]), int(block[2]), int(shared_mem), self._stream,
                                    arr, flags)
        self._check_error(err, "cuLaunchKernel")

    def launch_kernel(self, function, grid: tuple, block: tuple, args: list, shared_mem: int = 0,
                      expected_args: Optional[int] = None) -> bool:
        if expected_args is not None and len(args) != expected_args:
            raise CudaSafetyError(f"ABI mismatch: kernel expects {expected_args} args, got {len(args)}")
        self._validate_launch(function, grid, block, shared_mem, len(args))
        self._launch(function, grid, block, args, shared_mem, 0)
        return True

    def launch_kernel_recorded(self, function, args: list, grid: tuple, block: tuple, shared_mem: int = 0) -> bool:
        """Launch on the runtime's stream; while the stream is capturing, the
        driver records the launch into the graph instead of running it."""
        self._validate_launch(function, grid, block, shared_mem, len(args))
        self._launch(function, grid, block, args, shared_mem, LAUNCH_PROGRAMMATIC if self.programmatic_launch else 0)
        return True

    # ------------------------------------------------------------------ sync, graphs, events
    def synchronize(self) -> bool:
        self._require_init()
        if self._panic:
            raise CudaSafetyError("runtime is in panic state (a synchronize timed out); refusing to wait again")
        timed_out = threading.Event()
        done = threading.Event()

        def watch():
            if not done.wait(self._sync_timeout_s):
                timed_out.set()
                self._panic = True
                logger.error("cudaDeviceSynchronize exceeded %.1f s; entering panic state", self._sync_timeout_s)

        watcher = threading.Thread(target=watch, daemon=True)
        watcher.start()
        try:
            err = self._lib.vteb_device_synchronize()
        finally:
            done.set()
        self._check_error(err, "cudaDeviceSynchronize")
        if timed_out.is_set():
            raise CudaRuntimeError(f"cudaDeviceSynchronize took longer than {self._sync_timeout_s} s")
        return True

    def is_panic_state(self) -> bool:
        return self._panic

    def stream_begin_capture(self):
        self._require_init()
        self._check_error(self._lib.vteb_stream_begin_capture(self._stream, 0), "cudaStreamBeginCapture")

    def stream_end_capture(self) -> ctypes.c_void_p:
        graph = ctypes.c_void_p()
        self._check_error(self._lib.vteb_stream_end_capture(self._stream, ctypes.byref(graph)), "cudaStreamEndCapture")
        return graph

    def graph_instantiate(self, graph) -> ctypes.c_void_p:
        graph_exec = ctypes.c_void_p()
        self._check_error(self._lib.vteb_graph_instantiate(ctypes.byref(graph_exec), graph), "cudaGraphInstantiate")
        return graph_exec

    def graph_launch(self, graph_exec):
        if self._panic:
            raise CudaSafetyError("runtime is in panic state; graph launch blocked")
        self._check_error(self._lib.vteb_graph_launch(graph_exec, self._stream), "cudaGraphLaunch")

    def graph_node_count(self, graph) -> int:
        n = ctypes.c_size_t(0)
        self._check_error(self._lib.vteb_graph_node_count(graph, ctypes.byref(n)), "cudaGraphGetNodes")
        return n.value

    def graph_destroy(self, graph):
        self._check_error(self._lib.vteb_graph_destroy(graph), "cudaGraphDestroy")

    def graph_exec_destroy(self, graph_exec):
        self._check_error(self._lib.vteb_graph_exec_destroy(graph_exec), "cudaGraphExecDestroy")

    def event_create(self) -> ctypes.c_void_p:
        self._require_init()
        ev = ctypes.c_void_p()
        self._check_error(self._lib.vteb_event_create(ctypes.byref(ev)), "cudaEventCreate")
        return ev

    def event_record(self, event):
        self._check_error(self._lib.vteb_event_record(event, self._stream), "cudaEventRecord")

    def event_synchronize(self, event):
        self._check_error(self._lib.vteb_event_synchronize(event), "cudaEventSynchronize")

    def event_elapsed_ms(self, start, stop) -> float:
        self._check_error(self._lib.vteb_event_synchronize(stop), "cudaEventSynchronize")
        ms = ctypes.c_float(0.0)
        self._check_error(self._lib.vteb_event_elapsed_ms(ctypes.byref(ms), start, stop), "cudaEventElapsedTime")
        return ms.value

    def event_destroy(self, event):
        self._check_error(self._lib.vteb_event_destroy(event), "cudaEventDestroy")

    def stream_synchronize(self):
        self._require_init()
        self._check_error(self._lib.vteb_stream_synchronize(self._stream), "cudaStreamSynchronize")

    # ------------------------------------------------------------------ peer memory
    def ipc_export(self, ptr) -> bytes:
        """64-byte handle of the cudaMalloc allocation that starts at `ptr`."""
        self._require_init()
        val = _ptr_value(ptr)
        if val not in self._active_allocations:
            raise CudaSafetyError("only the base of a tracked allocation can be exported to peers")
        buf = ctypes.create_string_buffer(64)
        self._check_error(self._lib.vteb_ipc_get_handle(ctypes.c_void_p(val), buf), "cudaIpcGetMemHandle")
        return buf.raw

    def ipc_open(self, handle: bytes) -> int:
        """Map a peer rank's exported allocation; returns its address in this process."""
        self._require_init()
        if len(handle) != 64:
            raise CudaSafetyError(f"ipc handle has {len(handle)} bytes, expected 64")
        p = ctypes.c_void_p()
        self._check_error(self._lib.vteb_ipc_open_handle(ctypes.create_string_buffer(handle, 64), ctypes.byref(p)),
                          "cudaIpcOpenMemHandle")
        return p.value

    def ipc_close(self, ptr) -> None:
        self._check_error(self._lib.vteb_ipc_close_handle(ctypes.c_void_p(_ptr_value(ptr))), "cudaIpcCloseMemHandle")

    # ------------------------------------------------------------------ attention entry points
    def split_kv_plan(self, num_q_heads: int, num_kv_heads: int, head_dim: int, compact: bool = False) -> FastPlan:
        plan = FastPlan()
        fn = self._lib.vteb_split_kv_plan_compact if compact else self._lib.vteb_split_kv_plan
        self._check_error(fn(num_q_heads, num_kv_heads, head_dim, ctypes.byref(plan)), "vteb_split_kv_plan")
        return plan

    def kv_tensor_map(self, cache_ptr: int, n_rows: int, row_halves: int, box_rows: int) -> KvTensorMap:
        """Tensor map over a cache of `n_rows` position rows of `row_halves` fp16 values (boxes of
        64 values x `box_rows` rows, 128-byte swizzle) for the fast split kernels."""
        tm = KvTensorMap()
        self._check_error(self._lib.vteb_kv_tensor_map(ctypes.byref(tm), ctypes.c_void_p(int(cache_ptr)), int(n_rows),
                                                       int(row_halves), int(box_rows)), "vteb_kv_tensor_map")
        return tm

    def combine_rows_epl(self, rows: int, head_dim: int) -> int:
        return int(self._lib.vteb_combine_rows_epl(int(rows), int(head_dim)))

    def split_kv_decode(self, q, k_cache, v_cache, kv_offsets, output, out_is_f32: bool, partial_m, partial_l,
                        partial_o, work, batch: int, num_q_heads: int, num_kv_heads: int, head_dim: int,
                        scale: float, kv_batch_stride: int, max_chunks: int, min_chunk: int = 0, flags: int = 0,
                        n_ctas: int = 0) -> None:
        """Direct C-ABI launch of one layer's split + combine on the runtime's stream."""
        self._require_init()
        v = lambda p: ctypes.c_void_p(_ptr_value(p))
        err = self._lib.vteb_split_kv_decode(v(q), v(k_cache), v(v_cache), v(kv_offsets), v(output), int(bool(out_is_f32)),
                                             v(partial_m), v(partial_l), v(partial_o), v(work), batch, num_q_heads,
                                             num_kv_heads, head_dim, float(scale), int(kv_batch_stride), max_chunks,
                                             min_chunk, flags, n_ctas, self._stream)
        if err < 0:
            raise CudaSafetyError(f"vteb_split_kv_decode refused the call ({err}): {self._last_error()}")
        self._check_error(err, "vteb_split_kv_decode")

    def split_kv_decode_noalloc(self, q, k_cache, v_cache, kv_offsets, output, out_is_f32: bool, batch: int,
                                num_q_heads: int, num_kv_heads: int, head_dim: int, scale: float, kv_batch_stride: int,
                                max_chunks: int, min_chunk: int = 0, flags: int = 0, n_ctas: int = 0) -> None:
        """One layer's split + combine with the library's built-in scratch: for
        callers that must not allocate (inside a stream capture, a plugin without
        an allocator).  Requests beyond the 16 MiB array raise CudaSafetyError.
        The first call on a device does one-time set-up, so make it before any
        capture; calls share the scratch and must not overlap on the GPU."""
        self._require_init()
        v = lambda p: ctypes.c_void_p(_ptr_value(p))
        err = self._lib.vteb_split_kv_decode_noalloc(v(q), v(k_cache), v(v_cache), v(kv_offsets), v(output),
                                                     int(bool(out_is_f32)), batch, num_q_heads, num_kv_heads, head_dim,
                                                     float(scale), int(kv_batch_stride), max_chunks, min_chunk, flags,
                                                     n_ctas, self._stream)
        if err < 0:
            raise CudaSafetyError(f"vteb_split_kv_decode_noalloc refused the call ({err}): {self._last_error()}")
        self._check_error(err, "vteb_split_kv_decode_noalloc")

    def kv_cache_append(self, k, v, k_cache, v_cache, kv_offsets, batch: int, num_kv_heads: int, head_dim: int,
                        kv_batch_stride: int) -> None:
        self._require_init()
        p = lambda x: ctypes.c_void_p(_ptr_value(x))
        err = self._lib.vteb_kv_cache_append(p(k), p(v), p(k_cache), p(v_cache), p(kv_offsets), batch, num_kv_heads,
                                             head_dim, int(kv_batch_stride), self._stream)
        if err < 0:
            raise CudaSafetyError(f"vteb_kv_cache_append refused the call ({err}): {self._last_error()}")
        self._check_error(err, "vteb_kv_cache_append")

    def check_status(self, work) -> None:
        """Raise if a split kernel recorded a timed-out wait in work[1]."""
        err = self._lib.vteb_check_status(ctypes.c_void_p(_ptr_value(work)), self._stream)
        if err == ERR_DEVICE_STATUS:
            raise CudaRuntimeError(self._last_error(), code=err)
        self._check_error(err, "vteb_check_status")

    def noalloc_check_status(self) -> None:
        """`check_status` for the work words inside the library's own scratch array: raises if a
        bounded wait of any `split_kv_decode_noalloc` call since the last check gave up."""
        err = self._lib.vteb_noalloc_check_status(self._stream)
        if err == ERR_DEVICE_STATUS:
            raise CudaRuntimeError(self._last_error(), code=err)
        self._check_error(err, "vteb_noalloc_check_status")

    def fill_normal_f16(self, dst, n: int, seed: int, sigma: float = 1.0, outlier_prob: float = 0.0,
                        outlier_scale: float = 1.0) -> None:
        self._require_init()
        self._containing_allocation(_ptr_value(dst), 2 * n, "fill", "fill")
        self._check_error(self._lib.vteb_fill_normal_f16(ctypes.c_void_p(_ptr_value(dst)), n, seed, sigma, outlier_prob,
                                                         outlier_scale, self._stream), "vteb_fill_normal_f16")

    def read_bandwidth_probe(self, src, nbytes: int, sink, n_ctas: int) -> None:
        self._require_init()
        self._containing_allocation(_ptr_value(src), nbytes, "probe", "probe")
        self._check_error(self._lib.vteb_read_bandwidth_probe(ctypes.c_void_p(_ptr_value(src)), nbytes,
                                                              ctypes.c_void_p(_ptr_value(sink)), n_ctas, self._stream),
                          "vteb_read_bandwidth_probe")

    # ------------------------------------------------------------------ teardown
    def cleanup(self):
        """Free every tracked allocation and unload modules.  Never resets the
        device: other runtimes of the process may still own memory on it
        (the reference resets only when the last instance goes, :1053-1077;
        the CUDA context dies with the process here)."""
        self._in_cleanup_mode = True
        if self._initialized:
            try:
                self._lib.vteb_device_synchronize()
            except Exception:   # pragma: no cover
                pass
        for val, (size, tag) in list(self._active_allocations.items()):
            try:
                self.safe_free(ctypes.c_void_p(val), f"{tag}_cleanup")
            except Exception as e:   # keep going: cleanup is fail-safe
                logger.error("error freeing 0x%016X: %s", val, e)
        for val in list(self._host_allocations):
            try:
                self.host_free(ctypes.c_void_p(val))
            except Exception as e:
                logger.error("error freeing pinned 0x%016X: %s", val, e)
        for m in self._modules:
            self._lib.vteb_module_unload(ctypes.c_void_p(m))
        self._modules.clear()
        self._signatures.clear()
        self._smem_optin_set.clear()
        if self._initialized and self._stream:
            self._lib.vteb_stream_destroy(self._stream)
            self._stream = ctypes.c_void_p()
        if self._counted_as_live:
            CudaRuntime._live_instance_count = max(0, CudaRuntime._live_instance_count - 1)
            self._counted_as_live = False
        self._in_cleanup_mode = False
        self._initialized = False

    def __enter__(self):
        self.initialize()
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        self.cleanup()
        return False
