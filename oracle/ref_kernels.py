"""The reference's own kernels, compiled for the CPU by oracle/build_ref.py, behind numpy.
TEST INFRASTRUCTURE ONLY: nothing in the product imports this module.

Each function allocates the buffers the kernel's argument list names (vte/core/kernel_arg_builder.py:
57-71, 388-431; vte/core/split_kv_attention.py:166-214), launches the kernel with the grid and block
the reference's executor and dispatcher use (hip_graph_executor.py:352-367, split_kv_attention.py:
190-229) and returns the outputs.  `available()` is False where the library has not been built (a
machine without the reference checkout).
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import build_ref

_LIBS: dict[int, ctypes.CDLL] = {}


def available(chunk_size: int = 32) -> bool:
    return build_ref.library_path(chunk_size).exists()


def _lib(chunk_size: int) -> ctypes.CDLL:
    lib = _LIBS.get(chunk_size)
    if lib is None:
        lib = ctypes.CDLL(str(build_ref.library_path(chunk_size)))
        if lib.vte_ref_split_kv_chunk_size() != chunk_size:
            raise RuntimeError("reference kernel library built for another chunk size")
        _LIBS[chunk_size] = lib
    return lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _fp(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _ip(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_int))


def _f16(a):
    return np.ascontiguousarray(a, dtype=np.float16)


def kv_cache_append(k_new, v_new, k_cache, v_cache, kv_offsets, chunk_size: int = 32):
    """In place on k_cache / v_cache [B, max_seq, Hkv, D] fp16, like the kernel."""
    B, _, Hkv, D = k_cache.shape
    off = np.ascontiguousarray(kv_offsets, dtype=np.int32)
    k_new, v_new = _f16(k_new), _f16(v_new)
    assert k_cache.flags.c_contiguous and v_cache.flags.c_contiguous and k_cache.dtype == np.float16
    _lib(chunk_size).vte_ref_kv_cache_append(_p(k_new), _p(v_new), _p(k_cache), _p(v_cache), B, Hkv, D, _ip(off),
                                             k_cache.shape[1] * Hkv * D)


def split_kv_partial(q, k_cache, v_cache, kv_offsets, scale, max_chunks, chunk_size: int = 32):
    """(partial_m, partial_l [B,Hq,C], partial_o [B,Hq,C,D]) of flash_attention_split_kv_partial_kernel."""
    q, k_cache, v_cache = _f16(q), _f16(k_cache), _f16(v_cache)
    B, Hq, D = q.shape
    Hkv = k_cache.shape[2]
    off = np.ascontiguousarray(kv_offsets, dtype=np.int32)
    pm = np.full((B, Hq, max_chunks), np.nan, dtype=np.float32)
    pl = np.full((B, Hq, max_chunks), np.nan, dtype=np.float32)
    po = np.full((B, Hq, max_chunks, D), np.nan, dtype=np.float32)
    _lib(chunk_size).vte_ref_split_kv_partial(_p(q), _p(k_cache), _p(v_cache), _fp(pm), _fp(pl), _fp(po), B, Hq, Hkv, D,
                                              ctypes.c_float(scale), _ip(off), k_cache.shape[1] * Hkv * D, max_chunks)
    return pm, pl, po


def split_kv_reduce(partial_m, partial_l, partial_o, chunk_size: int = 32):
    """fp16 output [B,Hq,D] of flash_attention_split_kv_reduce_kernel."""
    pm = np.ascontiguousarray(partial_m, dtype=np.float32)
    pl = np.ascontiguousarray(partial_l, dtype=np.float32)
    po = np.ascontiguousarray(partial_o, dtype=np.float32)
    B, Hq, C, D = po.shape
    out = np.zeros((B, Hq, D), dtype=np.float16)
    _lib(chunk_size).vte_ref_split_kv_reduce(_fp(pm), _fp(pl), _fp(po), _p(out), B, Hq, D, C)
    return out


def flash_attention(q, k_new, v_new, k_cache, v_cache, kv_offsets, scale, chunk_size: int = 32):
    """The unsplit kernel: appends k_new / v_new in place, returns the fp16 output [B,Hq,D]."""
    q, k_new, v_new = _f16(q), _f16(k_new), _f16(v_new)
    B, Hq, D = q.shape
    Hkv = k_cache.shape[2]
    off = np.ascontiguousarray(kv_offsets, dtype=np.int32)
    out = np.zeros((B, Hq, D), dtype=np.float16)
    assert k_cache.flags.c_contiguous and v_cache.flags.c_contiguous and k_cache.dtype == np.float16
    _lib(chunk_size).vte_ref_flash_attention(_p(q), _p(k_new), _p(v_new), _p(k_cache), _p(v_cache), _p(out), B, 1, Hq, Hkv, D,
                                             ctypes.c_float(scale), _ip(off), k_cache.shape[1] * Hkv * D)
    return out


def rope(q, k, cos_table, sin_table, kv_offsets, rope_type: int = 0, rotary_dim: int | None = None, chunk_size: int = 32):
    """rope_kernel on copies of q [B,Hq,D] and k [B,Hkv,D] (one token per sequence); returns (q', k')."""
    q, k = _f16(q).copy(), _f16(k).copy()
    cos_table, sin_table = _f16(cos_table), _f16(sin_table)
    B, Hq, D = q.shape
    Hkv = k.shape[1]
    off = np.ascontiguousarray(kv_offsets, dtype=np.int32)
    block = 256
    grid_x = max(1, (Hq * D + block - 1) // block)          # seq_len * shape of the Q node, hip_graph_executor.py:359-367
    _lib(chunk_size).vte_ref_rope(_p(q), _p(k), _p(cos_table), _p(sin_table), grid_x, B, block, 1, Hq, Hkv, D, _ip(off),
                                  int(rope_type), int(D if rotary_dim is None else rotary_dim))
    return q, k
