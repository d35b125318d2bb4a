"""The allocation-free entry point, vteb_split_kv_decode_noalloc.

Some callers cannot allocate device memory: code inside a CUDA stream capture
(cudaMalloc is illegal there), a plugin that is handed tensors but no allocator,
a serving loop that must not risk the device-wide synchronisation an allocation
can cause.  For them the library keeps the split partials in a 16 MiB array of
its own.  This test calls it through the C ABI twice in a row and compares each
result with the ordinary entry point, which takes caller-provided scratch; the
second call finds the first call's leftovers in the array and must not care.
This file sorts last so a run that stops at the first failure has already run
every other test.
"""
import ctypes

import numpy as np
import pytest

from oracle import attention_oracle as orc
from vte_b200.bridge.errors import CudaSafetyError
from vte_b200.workloads import DecodeConfig, make_layer_inputs

pytestmark = pytest.mark.gpu

MAX_ABS, REL_L2 = 2e-3, 1e-2      # the tolerance every parity test here uses


def test_noalloc_entry_matches_scratch_entry_twice(cuda_runtime):
    rt = cuda_runtime
    lib = rt._lib
    bufs = []

    def dev(arr=None, nbytes=None):
        n = arr.nbytes if arr is not None else nbytes
        p = rt.safe_malloc(n, "noalloc test output")
        bufs.append(p)
        if arr is not None:
            rt.safe_memcpy_host_to_device(p, arr, "noalloc test output")
        else:
            rt.safe_memset(p, n, "noalloc test output")
        return p

    try:
        # two different problems back to back: the second one sees the first one's partials
        cases = [(DecodeConfig("na1", 41, 3, 12, 2, 128, 40, 700, 1), 8),
                 (DecodeConfig("na2", 42, 2, 32, 8, 64, 10, 300, 1), 5)]
        for cfg, C in cases:
            q, k, v, off = make_layer_inputs(cfg, 0)
            B, Hq, Hkv, D = cfg.batch, cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim
            dq, dk, dv, doff = dev(q), dev(k), dev(v), dev(off)
            out_a, out_b = dev(nbytes=B * Hq * D * 4), dev(nbytes=B * Hq * D * 4)
            pm, pl = dev(nbytes=B * Hq * C * 4), dev(nbytes=B * Hq * C * 4)
            po, work = dev(nbytes=B * Hq * C * D * 4), dev(nbytes=16)
            vp = lambda p: ctypes.c_void_p(p.value)
            rc = lib.vteb_split_kv_decode(vp(dq), vp(dk), vp(dv), vp(doff), vp(out_a), 1, vp(pm), vp(pl), vp(po), vp(work),
                                          B, Hq, Hkv, D, cfg.scale, cfg.kv_batch_stride, C, 0, 0, 0, rt.stream)
            assert rc == 0, lib.vteb_last_error_string()
            ref = np.zeros((B, Hq, D), np.float32)
            rt.stream_synchronize()
            rt.safe_memcpy_device_to_host(ref, out_a, "noalloc test output")
            for call in range(2):
                rc = lib.vteb_split_kv_decode_noalloc(vp(dq), vp(dk), vp(dv), vp(doff), vp(out_b), 1, B, Hq, Hkv, D,
                                                      cfg.scale, cfg.kv_batch_stride, C, 0, 0, 0, rt.stream)
                assert rc == 0, lib.vteb_last_error_string()
                rt.stream_synchronize()
                rt.noalloc_check_status()        # the status word inside the library's array: no wait gave up
                got = np.zeros_like(ref)
                rt.safe_memcpy_device_to_host(got, out_b, "noalloc test output")
                max_abs, rel = orc.parity_metrics(got, ref)
                assert max_abs <= MAX_ABS and rel <= REL_L2, (cfg.name, call, max_abs, rel)
                # both entry points launch the same kernels on the same inputs: identical bits
                assert np.array_equal(got, ref), (cfg.name, call)
                rt.safe_memset(out_b, B * Hq * D * 4, "noalloc test output")
            # and both agree with the CPU oracle
            max_abs, rel = orc.parity_metrics(ref, orc.decode_attention(q, k, v, off))
            assert max_abs <= MAX_ABS and rel <= REL_L2

        # beyond the built-in array: a clear refusal, nothing launched
        cfg, _ = cases[0]
        with pytest.raises(CudaSafetyError, match="needs .* bytes of scratch"):
            rt.split_kv_decode_noalloc(dq, dk, dv, doff, out_b, True, 64, 32, 8, 128, 0.1, cfg.kv_batch_stride, 256)
    finally:
        for p in bufs:
            rt.safe_free(p, "noalloc test cleanup")
