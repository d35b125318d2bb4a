"""The numpy oracle against the reference's own kernels run on the CPU.

`tests/golden/refkernel_*.npz` hold what the reference's HIP templates produce when they are compiled for
host threads (oracle/build_ref.py) and launched with the reference's grids (oracle/ref_kernels.py); the
generator is tests/golden/make_refkernel_golden.py.  The first tests need only the fixtures; the last ones
run the kernels themselves and are skipped where the library was not built (no reference checkout)."""
import importlib.util
from pathlib import Path

import numpy as np
import pytest

from oracle import attention_oracle as orc
from oracle import ref_kernels as rk

GOLD = Path(__file__).resolve().parent / "golden"
_spec = importlib.util.spec_from_file_location("make_refkernel_golden", GOLD / "make_refkernel_golden.py")
gen = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(gen)


@pytest.mark.parametrize("name", sorted(gen.SPLIT_CASES))
def test_oracle_reproduces_the_reference_kernels_split_path(name):
    """append -> partial -> reduce and the unsplit kernel: the oracle's restatements against the reference
    kernels' outputs.  The append is a copy (bit-exact).  The partial kernel sums q*k with a shared-memory
    tree and the oracle with numpy, so (m, l, o) agree to fp32 reassociation; empty chunks are exactly the
    neutral state.  The two fp16 outputs are compared at fp16 resolution."""
    g = np.load(GOLD / "refkernel_split_kv.npz")
    q, k, v, k_new, v_new, off, chunk, scale = gen.split_case_inputs(name)
    B, max_seq = k.shape[0], k.shape[1]
    max_chunks = -(-max_seq // chunk)
    k1, v1 = k.copy(), v.copy()
    orc.kv_cache_append(k_new, v_new, k1, v1, off)
    for b in range(B):
        assert np.array_equal(k1[b, off[b]], g[f"{name}.k_rows"][b]) and np.array_equal(v1[b, off[b]], g[f"{name}.v_rows"][b])
    pm, pl, po = orc.split_kv_partial(q, k1, v1, off, scale, max_chunks, chunk_size=chunk)
    rm, rl, ro = g[f"{name}.pm"], g[f"{name}.pl"], g[f"{name}.po"]
    live = rl > 0
    for b in range(B):
        n_live = -(-(int(off[b]) + 1) // chunk)
        assert np.all(live[b, :, :n_live]) and not np.any(live[b, :, n_live:])
    assert np.all(rm[~live] == np.float32(-1e30)) and np.all(ro[~live] == 0)
    assert np.array_equal(pm[~live], rm[~live]) and np.all(pl[~live] == 0) and np.all(po[~live] == 0)
    assert np.allclose(pm[live], rm[live], rtol=0, atol=2e-6)
    assert np.allclose(pl[live], rl[live], rtol=2e-6, atol=0)
    assert np.allclose(po[live], ro[live], rtol=1e-5, atol=2e-6)
    # the oracle's reduce on the REFERENCE's partials against the reference's reduce (fp16 store)
    red = orc.split_kv_reduce(rm, rl, ro)
    assert np.max(np.abs(red - g[f"{name}.reduce"].astype(np.float32))) <= 1e-3
    assert np.mean(red.astype(np.float16) == g[f"{name}.reduce"]) > 0.97     # same fp16 value except at rounding ties
    # the unsplit kernel equals the one-call oracle and the split route
    ref = orc.decode_attention(q, k1, v1, off, scale=scale)
    assert np.max(np.abs(ref - g[f"{name}.unsplit"].astype(np.float32))) <= 1e-3
    assert np.max(np.abs(g[f"{name}.unsplit"].astype(np.float32) - g[f"{name}.reduce"].astype(np.float32))) <= 2e-3


@pytest.mark.parametrize("name", sorted(gen.ROPE_CASES))
def test_oracle_rotation_equals_the_reference_kernel_bit_for_bit(name):
    """rope_kernel for the three rotation types (split-half, interleaved, partial split-half): the oracle
    rounds at the same points, so every fp16 value must be identical.  This is the pin for the interleaved
    type, which has no Python counterpart in the reference."""
    g = np.load(GOLD / "refkernel_rope.npz")
    q, k, cos_t, sin_t, off, rope_type, rot = gen.rope_case_inputs(name)
    q2, k2 = orc.rope_step(q, k, cos_t, sin_t, off, rope_type, rot)
    assert np.array_equal(q2, g[f"{name}.q"]) and np.array_equal(k2, g[f"{name}.k"])
    assert not np.array_equal(q2, q)


needs_kernels = pytest.mark.skipif(not (rk.available(32) and rk.available(8)),
                                   reason="reference kernels not built here (no reference checkout)")


@needs_kernels
def test_fixtures_are_what_the_reference_kernels_produce_now():
    """Guards the generator: rerunning the kernels gives the committed bytes."""
    g = np.load(GOLD / "refkernel_split_kv.npz")
    for name in gen.SPLIT_CASES:
        q, k, v, k_new, v_new, off, chunk, scale = gen.split_case_inputs(name)
        k1, v1 = k.copy(), v.copy()
        rk.kv_cache_append(k_new, v_new, k1, v1, off, chunk)
        pm, pl, po = rk.split_kv_partial(q, k1, v1, off, scale, -(-k.shape[1] // chunk), chunk)
        assert np.array_equal(pm, g[f"{name}.pm"]) and np.array_equal(pl, g[f"{name}.pl"]) and np.array_equal(po, g[f"{name}.po"])
        assert np.array_equal(rk.split_kv_reduce(pm, pl, po, chunk), g[f"{name}.reduce"])
    g = np.load(GOLD / "refkernel_rope.npz")
    for name in gen.ROPE_CASES:
        q, k, cos_t, sin_t, off, rope_type, rot = gen.rope_case_inputs(name)
        q2, k2 = rk.rope(q, k, cos_t, sin_t, off, rope_type, rot)
        assert np.array_equal(q2, g[f"{name}.q"]) and np.array_equal(k2, g[f"{name}.k"])


@needs_kernels
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_oracle_against_live_reference_kernels_on_random_shapes(seed):
    rng = np.random.default_rng(seed)
    B = int(rng.integers(1, 4))
    Hkv = int(rng.choice([1, 2, 4]))
    group = int(rng.choice([1, 2, 4, 6]))
    D = int(rng.choice([64, 128]))
    max_seq = int(rng.integers(20, 90))
    chunk = int(rng.choice([8, 32]))
    Hq = Hkv * group
    q = rng.standard_normal((B, Hq, D), dtype=np.float32).astype(np.float16)
    k = rng.standard_normal((B, max_seq, Hkv, D), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((B, max_seq, Hkv, D), dtype=np.float32).astype(np.float16)
    off = rng.integers(0, max_seq, size=B).astype(np.int32)
    scale = float(1.0 / np.sqrt(D))
    C = -(-max_seq // chunk)
    rm, rl, ro = rk.split_kv_partial(q, k, v, off, scale, C, chunk)
    pm, pl, po = orc.split_kv_partial(q, k, v, off, scale, C, chunk_size=chunk)
    assert np.allclose(pm, rm, rtol=0, atol=2e-6) and np.allclose(pl, rl, rtol=2e-6) and np.allclose(po, ro, rtol=1e-5, atol=2e-6)
    out = rk.split_kv_reduce(rm, rl, ro, chunk).astype(np.float32)
    assert np.max(np.abs(out - orc.decode_attention(q, k, v, off, scale=scale))) <= 1.5e-3
