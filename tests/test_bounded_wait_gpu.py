"""A device-side wait that runs out: the kernel returns, the status word says why,
the host turns it into an exception and clears it.  Nothing faults, traps or hangs.

Every wait in the kernels is bounded by VTEB_WAIT_LIMIT_CYCLES (about two seconds
by default).  A build with a limit of 200,000 cycles (~0.1 ms) lets this test watch one
expire: the shard-merge kernel of the KV-range path polls its own board for the
tagged words of two ranks, but nobody ever stores them (the board is zeroed, the
expected tag is 1).  The behaviour mirrors the reference's watchdog
(vte/bridge/watchdog.py:111-134: raise a panic flag, never reset the device).
"""
import ctypes
import time

import numpy as np
import pytest

from vte_b200.bridge.errors import CudaRuntimeError

pytestmark = pytest.mark.gpu


def test_a_wait_that_nothing_satisfies_times_out_and_is_reported(cuda_runtime, codegen):
    rt = cuda_runtime
    _, merge_fn = codegen.load_kernel_safe(rt, 'decode_attention', rt.get_gpu_architecture(),
                                           'vteb_merge_shard_states_ll_kernel', vteb_wait_limit_cycles=200000)
    world, rows, D, layers = 2, 12, 128, 1
    board_bytes = 2 * layers * world * rows * (D + 2) * 8
    bufs = []

    def zeroed(nbytes):
        p = rt.safe_malloc(nbytes, "bounded wait test output")
        rt.safe_memset(p, nbytes, "bounded wait test output")
        bufs.append(p)
        return p

    try:
        board, out, step, work = zeroed(board_bytes), zeroed(rows * D * 4), zeroed(64), zeroed(16)
        vp, ci = ctypes.c_void_p, ctypes.c_int
        args = [vp(board.value), vp(out.value), ci(world), ci(rows), ci(D), ci(0), ci(layers), vp(step.value),
                vp(work.value + 4)]
        t0 = time.perf_counter()
        rt.launch_kernel(merge_fn, (rows, 1, 1), (D, 1, 1), args)
        rt.synchronize()
        assert time.perf_counter() - t0 < 5.0          # ~0.1 ms of polling, not the two-second default
        status = np.zeros(4, dtype=np.int32)
        rt.safe_memcpy_device_to_host(status, work, "status word output")
        assert status[1] == 4                          # kStatusGridTimeout: a rank never arrived
        with pytest.raises(CudaRuntimeError, match="never arrived"):
            rt.check_status(work)
        rt.check_status(work)                          # the word was cleared: a second check passes
        # the context is intact: an ordinary launch still works
        rt.safe_memset(out, rows * D * 4, "bounded wait test output")
        rt.synchronize()
    finally:
        for p in bufs:
            rt.safe_free(p, "bounded wait test cleanup")
