"""Generates tests/golden/refkernel_*.npz by running the REFERENCE's own kernels on the CPU.

    python -m oracle.build_ref                      # compiles the reference's templates (needs the checkout)
    python tests/golden/make_refkernel_golden.py

The kernels are the reference's HIP templates, built unmodified for host threads by oracle/build_ref.py
(oracle/ref_kernels.py launches them with the reference's grids).  Inputs are seeded here and stored in
the files where they are small, so the fixtures can be checked on machines without the reference checkout:
`refkernel_split_kv.npz` holds the append, the partial kernel's (m, l, o), the reduce kernel's fp16 output
and the unsplit kernel's fp16 output; `refkernel_rope.npz` holds rope_kernel's output for the three
rotation types.
"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from oracle import ref_kernels as rk          # noqa: E402
from oracle import attention_oracle as orc    # noqa: E402

SPLIT_CASES = {
    # name: (B, Hq, Hkv, D, max_seq, offsets, chunk_size)
    "gqa3_d64_c32": (3, 6, 2, 64, 140, [0, 57, 139], 32),
    "gqa6_d128_c8": (2, 12, 2, 128, 70, [69, 12], 8),
}
ROPE_CASES = {
    # name: (B, Hq, Hkv, D, rope_type, rotary_dim, theta, offsets)
    "neox_d128": (3, 12, 2, 128, 0, 128, 1e6, [0, 5, 300]),
    "interleaved_d64": (3, 8, 2, 64, 1, 64, 1e4, [0, 7, 301]),
    "partial_d256": (2, 8, 2, 256, 2, 64, 1e7, [1, 255]),
}


def split_case_inputs(name):
    B, Hq, Hkv, D, max_seq, offsets, chunk = SPLIT_CASES[name]
    rng = np.random.default_rng([91, len(name), B, D])
    q = rng.standard_normal((B, Hq, D), dtype=np.float32).astype(np.float16)
    k = rng.standard_normal((B, max_seq, Hkv, D), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((B, max_seq, Hkv, D), dtype=np.float32).astype(np.float16)
    k_new = rng.standard_normal((B, Hkv, D), dtype=np.float32).astype(np.float16)
    v_new = rng.standard_normal((B, Hkv, D), dtype=np.float32).astype(np.float16)
    return q, k, v, k_new, v_new, np.array(offsets, dtype=np.int32), chunk, float(1.0 / np.sqrt(D))


def rope_case_inputs(name):
    B, Hq, Hkv, D, rope_type, rot, theta, offsets = ROPE_CASES[name]
    rng = np.random.default_rng([92, len(name), B, D])
    q = rng.standard_normal((B, Hq, D), dtype=np.float32).astype(np.float16)
    k = rng.standard_normal((B, Hkv, D), dtype=np.float32).astype(np.float16)
    width = rot if rope_type == 2 else D
    cos_t, sin_t = orc.rope_tables(max(offsets) + 1, width, theta)      # pinned to the reference's builder elsewhere
    return q, k, cos_t, sin_t, np.array(offsets, dtype=np.int32), rope_type, rot


def main():
    out = {}
    for name in SPLIT_CASES:
        q, k, v, k_new, v_new, off, chunk, scale = split_case_inputs(name)
        max_chunks = -(-k.shape[1] // chunk)
        k1, v1 = k.copy(), v.copy()
        rk.kv_cache_append(k_new, v_new, k1, v1, off, chunk)
        pm, pl, po = rk.split_kv_partial(q, k1, v1, off, scale, max_chunks, chunk)
        red = rk.split_kv_reduce(pm, pl, po, chunk)
        k2, v2 = k.copy(), v.copy()
        unsplit = rk.flash_attention(q, k_new, v_new, k2, v2, off, scale, chunk)
        assert np.array_equal(k1, k2) and np.array_equal(v1, v2)
        rows = np.stack([k1[b, off[b]] for b in range(len(off))]), np.stack([v1[b, off[b]] for b in range(len(off))])
        out.update({f"{name}.pm": pm, f"{name}.pl": pl, f"{name}.po": po, f"{name}.reduce": red, f"{name}.unsplit": unsplit,
                    f"{name}.k_rows": rows[0], f"{name}.v_rows": rows[1]})
        print(name, "max_chunks", max_chunks, float(np.abs(red.astype(np.float32)).max()))
    np.savez_compressed(HERE / "refkernel_split_kv.npz", **out)
    out = {}
    for name in ROPE_CASES:
        q, k, cos_t, sin_t, off, rope_type, rot = rope_case_inputs(name)
        q2, k2 = rk.rope(q, k, cos_t, sin_t, off, rope_type, rot)
        out.update({f"{name}.q": q2, f"{name}.k": k2})
        print(name, int((q2 != q).sum()), "q elements changed")
    np.savez_compressed(HERE / "refkernel_rope.npz", **out)


if __name__ == "__main__":
    main()
