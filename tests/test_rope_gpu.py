"""Rotary embedding beside the decode-attention path: the standalone rotation launch
(`rope_kernel`, the reference's argument list) and the rotation folded into the cache
append (K) and into the split kernel's Q load.

Integer-exact where the arithmetic allows it: rotated rows are compared bit for bit with
the oracle, and the fused step must return exactly the bits of the separate one; the
attention output is held to the path's tolerance (max-abs <= 2e-3, relative L2 <= 1e-2).
"""
import ctypes

import numpy as np
import pytest

from oracle import attention_oracle as orc
from vte_b200.core.decode_executor import DecodeAttentionExecutor
from vte_b200.workloads import DecodeConfig, make_layer_inputs

pytestmark = pytest.mark.gpu

MAX_ABS, REL_L2 = 2e-3, 1e-2
THETA = 1e4
N_LAYERS = 2

CASES = {
    # name: (head_dim, Hq, Hkv, rope_type, rotary_dim)
    "split_half_d128": (128, 12, 2, 0, 128),
    "split_half_d64": (64, 8, 4, 0, 64),
    "interleaved_d128": (128, 8, 2, 1, 128),
    "interleaved_d64": (64, 4, 4, 1, 64),
    "partial64_d256": (256, 8, 2, 2, 64),
    "partial128_d256": (256, 4, 1, 2, 128),
    "partial32_d64": (64, 8, 2, 2, 32),
    "full_width_partial_d256": (256, 8, 2, 2, 256),
}


def run_steps(rt, codegen, cfg, meta, mode, layers, news, offsets_per_step, splits, variant):
    """Runs the decode steps in `mode` and returns, per step, (outputs [L,B,Hq,D], last cache rows of
    layer 0 per sequence, the Q buffer after the step)."""
    ex = DecodeAttentionExecutor(rt, codegen, meta, cfg.batch, cfg.max_seq, N_LAYERS, rope=mode, rope_theta=THETA,
                                 num_splits=splits, min_chunk=0, variant=variant)
    results = []
    try:
        for l, (q, k, v, _) in enumerate(layers):
            ex.upload_layer(l, q, k, v)
        q_host = np.stack([q for q, _, _, _ in layers])
        for step, off in enumerate(offsets_per_step):
            for l in range(N_LAYERS):
                ex.upload_new_kv(l, news[step][l][0], news[step][l][1])
            out = ex.execute_decode_batch(off, q_host=q_host)
            rows = [ex.download_cache_rows(0, b, int(off[b]) + 1) for b in range(cfg.batch)]
            q_after = np.empty_like(q_host[0])
            rt.safe_memcpy_device_to_host(q_after, ctypes.c_void_p(ex.q_all.ptr), "q buffer for output check")
            results.append((out, rows, q_after))
    finally:
        ex.cleanup()
    return results


@pytest.mark.parametrize("name", sorted(CASES))
def test_rotation_modes_match_oracle_and_each_other(cuda_runtime, codegen, name):
    D, Hq, Hkv, rope_type, rot = CASES[name]
    cfg = DecodeConfig(name, 31, 3, Hq, Hkv, D, 260, 260, N_LAYERS)
    meta = {'attention.head_count': Hq, 'attention.head_count_kv': Hkv, 'attention.key_length': D,
            'rope_type': rope_type, 'rotary_dim': rot}
    width = rot if rope_type == 2 else D
    cos_t, sin_t = orc.rope_tables(cfg.max_seq, width, THETA)
    layers = [make_layer_inputs(cfg, l) for l in range(N_LAYERS)]
    rng = np.random.default_rng(5)
    offsets_per_step = [np.array([40, 131, 7], dtype=np.int32), np.array([41, 259, 8], dtype=np.int32)]
    news = [[(rng.standard_normal((cfg.batch, Hkv, D), dtype=np.float32).astype(np.float16),
              rng.standard_normal((cfg.batch, Hkv, D), dtype=np.float32).astype(np.float16))
             for _ in range(N_LAYERS)] for _ in offsets_per_step]

    for splits, variant in ((1, "full"), (4, "full"), (3, "compact")):
        got = {mode: run_steps(cuda_runtime, codegen, cfg, meta, mode, layers, news, offsets_per_step, splits, variant)
               for mode in ("separate", "fused", "fused-append")}
        caches = [(k.copy(), v.copy()) for _, k, v, _ in layers]
        for step, off in enumerate(offsets_per_step):
            for l, (q, _, _, _) in enumerate(layers):
                k_new, v_new = news[step][l]
                q_rot, k_rot = orc.rope_step(q, k_new, cos_t, sin_t, off, rope_type, rot)
                k, v = caches[l]
                orc.kv_cache_append(k_rot, v_new, k, v, off)
                ref = orc.decode_attention(q_rot, k, v, off)
                for mode in ("separate", "fused", "fused-append"):
                    out, rows, q_after = got[mode][step]
                    max_abs, rel = orc.parity_metrics(out[l], ref)
                    assert max_abs <= MAX_ABS and rel <= REL_L2, (mode, step, l, max_abs, rel)
                    assert max_abs <= 1e-4, (mode, step, l, max_abs)
                    if l == 0:
                        for b in range(cfg.batch):
                            kr, vr = rows[b]
                            # the appended row is the oracle's rotated row, bit for bit
                            assert np.array_equal(kr[off[b]], k_rot[b]), (mode, step, b)
                            assert np.array_equal(vr[off[b]], v_new[b])
                            assert np.array_equal(kr[:off[b]], k[b, :off[b]])
                        if mode == "separate":
                            assert np.array_equal(q_after, q_rot)          # rotated in place
                        else:
                            assert np.array_equal(q_after, q)              # left as it was
            # the two routes round at the same points: identical output bits
            assert np.array_equal(got["separate"][step][0], got["fused"][step][0]), (splits, variant, step)
            # ... and so does the route whose split kernel also does the append (no append launch)
            assert np.array_equal(got["separate"][step][0], got["fused-append"][step][0]), (splits, variant, step)


def test_rotation_kernel_handles_several_tokens_and_any_grid(cuda_runtime, codegen):
    """`rope_kernel` with seq_len > 1 (the reference launches it for prefill too): token i of sequence b
    sits at position offset[b] + i; a grid smaller than the pair count still covers every pair."""
    rt = cuda_runtime
    B, T, Hq, Hkv, D = 2, 5, 4, 2, 128
    cos_t, sin_t = orc.rope_tables(64, D, THETA)
    rng = np.random.default_rng(9)
    q = rng.standard_normal((B, T, Hq, D), dtype=np.float32).astype(np.float16)
    k = rng.standard_normal((B, T, Hkv, D), dtype=np.float32).astype(np.float16)
    off = np.array([3, 50], dtype=np.int32)
    arch = rt.get_gpu_architecture()
    _, fn = codegen.load_kernel_safe(rt, "rope", arch, "rope_kernel")
    bufs = {}
    try:
        for nm, arr in (("q", q), ("k", k), ("cos", cos_t), ("sin", sin_t), ("off", off)):
            bufs[nm] = rt.safe_malloc(arr.nbytes, f"rope test {nm} output")
            rt.safe_memcpy_host_to_device(bufs[nm], arr, f"rope test {nm} output")
        for rope_type, grid_x in ((0, 1), (1, 40)):
            rt.safe_memcpy_host_to_device(bufs["q"], q, "rope test q output")
            rt.safe_memcpy_host_to_device(bufs["k"], k, "rope test k output")
            vp, ci = ctypes.c_void_p, ctypes.c_int
            args = [vp(bufs["q"].value), vp(bufs["k"].value), vp(bufs["cos"].value), vp(bufs["sin"].value),
                    ci(T), ci(Hq), ci(Hkv), ci(D), vp(bufs["off"].value), ci(rope_type), ci(D)]
            rt.launch_kernel(fn, (grid_x, B, 1), (64, 1, 1), args)
            rt.synchronize()
            q2, k2 = np.empty_like(q), np.empty_like(k)
            rt.safe_memcpy_device_to_host(q2, bufs["q"], "rope test q output")
            rt.safe_memcpy_device_to_host(k2, bufs["k"], "rope test k output")
            for b in range(B):
                for t in range(T):
                    pos = int(off[b]) + t
                    assert np.array_equal(q2[b, t], orc.rope_apply(q[b, t], cos_t[pos], sin_t[pos], rope_type))
                    assert np.array_equal(k2[b, t], orc.rope_apply(k[b, t], cos_t[pos], sin_t[pos], rope_type))
    finally:
        for p in bufs.values():
            rt.safe_free(p, "rope test")


@pytest.mark.parametrize("name", ["neox_d128", "interleaved_d64", "partial_d256"])
def test_rotation_kernel_equals_the_reference_kernel_vectors(cuda_runtime, codegen, name):
    """tests/golden/refkernel_rope.npz holds the output of the reference's own rope_kernel (its template
    compiled for CPU threads, oracle/build_ref.py) for the three rotation types; the kernel here must give
    the same fp16 bits.  The interleaved type has no other pin: the reference has no Python rotation for it."""
    import importlib.util
    from pathlib import Path
    gold = Path(__file__).resolve().parent / "golden"
    spec = importlib.util.spec_from_file_location("make_refkernel_golden", gold / "make_refkernel_golden.py")
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    g = np.load(gold / "refkernel_rope.npz")
    q, k, cos_t, sin_t, off, rope_type, rot = gen.rope_case_inputs(name)
    B, Hq, D = q.shape
    Hkv = k.shape[1]
    rt = cuda_runtime
    _, fn = codegen.load_kernel_safe(rt, "rope", rt.get_gpu_architecture(), "rope_kernel")
    bufs = {}
    try:
        for nm, arr in (("q", q), ("k", k), ("cos", cos_t), ("sin", sin_t), ("off", off)):
            bufs[nm] = rt.safe_malloc(arr.nbytes, f"rope test {nm} output")
            rt.safe_memcpy_host_to_device(bufs[nm], arr, f"rope test {nm} output")
        vp, ci = ctypes.c_void_p, ctypes.c_int
        args = [vp(bufs["q"].value), vp(bufs["k"].value), vp(bufs["cos"].value), vp(bufs["sin"].value),
                ci(1), ci(Hq), ci(Hkv), ci(D), vp(bufs["off"].value), ci(rope_type), ci(rot)]
        rt.launch_kernel(fn, (max(1, (Hq * D + 255) // 256), B, 1), (256, 1, 1), args)     # the reference's grid rule
        rt.synchronize()
        q2, k2 = np.empty_like(q), np.empty_like(k)
        rt.safe_memcpy_device_to_host(q2, bufs["q"], "rope test q output")
        rt.safe_memcpy_device_to_host(k2, bufs["k"], "rope test k output")
        assert np.array_equal(q2, g[f"{name}.q"]) and np.array_equal(k2, g[f"{name}.k"])
    finally:
        for p_ in bufs.values():
            rt.safe_free(p_, "rope test")
