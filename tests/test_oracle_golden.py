"""The CPU oracle against vectors produced by the reference's own functions
(tests/golden/make_golden.py), plus the oracle's internal consistency."""
from pathlib import Path

import numpy as np
import pytest

from oracle import attention_oracle as orc
from vte_b200.workloads import CONFIGS, make_layer_inputs, rope_rotate_neox
from tests.golden.make_golden import SMALL_CASES, digest

GOLD = Path(__file__).resolve().parent / "golden"
ATOL, RTOL = 2e-3, 1e-2   # tolerance the CUDA path is held to; the oracle itself must be far inside


def _case(name):
    if name in SMALL_CASES:
        return SMALL_CASES[name]
    return {"c1": (CONFIGS["c1"], None), "c2_layer0": (CONFIGS["c2"], None)}[name]


@pytest.mark.parametrize("name", ["ragged_d64", "outlier_d256", "mha_d128", "group8_d128", "c1", "c2_layer0"])
def test_decode_attention_matches_reference_vectors(name):
    cfg, lens = _case(name)
    gold = np.load(GOLD / f"attn_{name}.npz")
    q, k, v, off = make_layer_inputs(cfg, 0, lengths=lens)
    sha = digest(q, off, *[k[b, :off[b] + 1] for b in range(cfg.batch)], *[v[b, :off[b] + 1] for b in range(cfg.batch)])
    assert sha == str(gold["input_sha256"]), "the seeded input generator no longer reproduces the golden inputs"
    assert np.array_equal(off, gold["offsets"])
    out = orc.decode_attention(q, k, v, off)
    # same arithmetic, same numpy: the restatement reproduces the reference's numbers
    np.testing.assert_allclose(out, gold["out"], rtol=0, atol=1e-6)
    max_abs, rel = orc.parity_metrics(out, gold["out"])
    assert max_abs <= 1e-6 and rel <= 1e-6


@pytest.mark.parametrize("name", ["ragged_d64", "outlier_d256", "group8_d128", "c1"])
def test_oracle_is_accurate_against_float64(name):
    cfg, lens = _case(name)
    q, k, v, off = make_layer_inputs(cfg, 0, lengths=lens)
    o32 = orc.decode_attention(q, k, v, off)
    o64 = orc.decode_attention(q, k, v, off, dtype=np.float64)
    max_abs, rel = orc.parity_metrics(o32, o64)
    assert max_abs < 5e-6 and rel < 5e-6


@pytest.mark.parametrize("name,chunks,fixed", [("ragged_d64", 4, None), ("ragged_d64", 9, 16), ("outlier_d256", 8, None),
                                               ("group8_d128", 3, None), ("c1", 16, 32), ("c1", 148, None)])
def test_split_then_reduce_equals_unsplit(name, chunks, fixed):
    cfg, lens = _case(name)
    q, k, v, off = make_layer_inputs(cfg, 0, lengths=lens)
    if fixed:
        chunks = max(chunks, -(-int(off.max() + 1) // fixed))
    pm, pl, po = orc.split_kv_partial(q, k, v, off, cfg.scale, chunks, chunk_size=fixed)
    out = orc.split_kv_reduce(pm, pl, po)
    ref = orc.decode_attention(q, k, v, off)
    max_abs, rel = orc.parity_metrics(out, ref)
    assert max_abs < 1e-5 and rel < 1e-5
    # empty splits carry the neutral state
    total = off + 1
    for b in range(cfg.batch):
        for c, (s, e) in enumerate(orc.split_ranges(int(total[b]), chunks, fixed)):
            if e <= s:
                assert np.all(pm[b, :, c] == np.float32(-1e30)) and np.all(pl[b, :, c] == 0) and np.all(po[b, :, c] == 0)


def test_split_ranges_cover_every_position_once():
    for total in [1, 2, 15, 16, 17, 31, 32, 33, 100, 511, 512, 513, 4097]:
        for chunks in [1, 2, 3, 7, 8, 64, 148, 256]:
            for fixed in [None, 8, 32]:
                if fixed and chunks * fixed < total:
                    continue
                seen = np.zeros(total, dtype=int)
                for s, e in orc.split_ranges(total, chunks, fixed):
                    seen[s:e] += 1
                assert np.all(seen == 1), (total, chunks, fixed)


def test_rope_matches_reference_tables_and_rotation():
    gold = np.load(GOLD / "rope.npz")
    theta, pos = float(gold["theta"]), int(gold["position"])
    for r, cos_row, sin_row in zip(gold["rows"], gold["cos_rows"], gold["sin_rows"]):
        c, s = orc.rope_row(int(r), 128, theta)
        assert np.array_equal(c, cos_row) and np.array_equal(s, sin_row)
    cos_t, sin_t = orc.rope_tables(64, 128, theta)
    c2, s2 = orc.rope_row(2, 128, theta)
    assert np.array_equal(cos_t[2], c2) and np.array_equal(sin_t[2], s2)
    c, s = orc.rope_row(pos, 128, theta)
    y = orc.rope_neox(gold["x"], c, s)
    assert np.array_equal(y, gold["x_rotated"])
    # the workload generator's rotation is the same function
    assert np.array_equal(rope_rotate_neox(gold["x"], pos, theta), gold["x_rotated"])


def test_rope_types_match_reference_rotation():
    # type 0 through the general entry point equals the pinned split-half rotation
    gold = np.load(GOLD / "rope.npz")
    c, s = orc.rope_row(int(gold["position"]), 128, float(gold["theta"]))
    assert np.array_equal(orc.rope_apply(gold["x"], c, s, 0), gold["x_rotated"])
    # type 2 (partial split-half): the reference's numpy rotation of the first rotary_dim channels
    part = np.load(GOLD / "rope_partial.npz")
    rot, theta = int(part["rotary_dim"]), float(part["theta"])
    for pi, pos in enumerate(part["positions"]):
        c, s = orc.rope_row(int(pos), rot, theta)
        assert np.array_equal(c, part["cos_rows"][pi]) and np.array_equal(s, part["sin_rows"][pi])
        y = orc.rope_apply(part["x"], c, s, 2, rot)
        assert np.array_equal(y, part["x_rotated"][pi])
        assert np.array_equal(y[:, rot:], part["x"][:, rot:])          # untouched channels
    # type 2 with rotary_dim == D is type 0
    c, s = orc.rope_row(5, 128, 1e4)
    assert np.array_equal(orc.rope_apply(gold["x"], c, s, 2, 128), orc.rope_apply(gold["x"], c, s, 0))
    # type 1 (interleaved; no Python counterpart in the reference): a rotation of adjacent pairs,
    # so pair norms survive up to fp16 rounding and position 0 is the identity
    x = gold["x"]
    y = orc.rope_apply(x, c, s, 1)
    n_in = np.hypot(x[:, 0::2].astype(np.float64), x[:, 1::2].astype(np.float64))
    n_out = np.hypot(y[:, 0::2].astype(np.float64), y[:, 1::2].astype(np.float64))
    assert np.max(np.abs(n_in - n_out)) < 4e-3
    c0, s0 = orc.rope_row(0, 128, 1e4)
    assert np.array_equal(orc.rope_apply(x, c0, s0, 1), x)
    # rope_step rotates every sequence at its own position
    cos_t, sin_t = orc.rope_tables(16, 128, 1e4)
    q = np.stack([x, x]); k = q[:, :2]
    q2, k2 = orc.rope_step(q, k, cos_t, sin_t, np.array([3, 9]), 0)
    assert np.array_equal(q2[1], orc.rope_apply(x, cos_t[9], sin_t[9], 0))
    assert np.array_equal(k2[0], orc.rope_apply(x[:2], cos_t[3], sin_t[3], 0))


def test_chunk_rule_matches_reference():
    gold = np.load(GOLD / "chunk_rule.npz")
    from vte_b200.core.split_kv_attention import _chunk_size_for_cus
    for cus, chunk in zip(gold["cus"], gold["chunk"]):
        assert orc.chunk_size_for_cus(int(cus)) == int(chunk)
        assert _chunk_size_for_cus(int(cus)) == int(chunk)


def test_kv_cache_append_writes_one_row():
    cfg, lens = SMALL_CASES["ragged_d64"]
    q, k, v, off = make_layer_inputs(cfg, 0, lengths=lens)
    k0, v0 = k.copy(), v.copy()
    rng = np.random.default_rng(5)
    kn = rng.standard_normal((cfg.batch, cfg.num_kv_heads, cfg.head_dim), dtype=np.float32).astype(np.float16)
    vn = rng.standard_normal((cfg.batch, cfg.num_kv_heads, cfg.head_dim), dtype=np.float32).astype(np.float16)
    orc.kv_cache_append(kn, vn, k, v, off)
    for b in range(cfg.batch):
        assert np.array_equal(k[b, off[b]], kn[b]) and np.array_equal(v[b, off[b]], vn[b])
        mask = np.ones(cfg.max_seq, dtype=bool)
        mask[off[b]] = False
        assert np.array_equal(k[b, mask], k0[b, mask]) and np.array_equal(v[b, mask], v0[b, mask])


def test_shard_merge_equals_single_pass():
    """KV-range sharding: per-shard unnormalised (m, l, o) merged with the reduce
    arithmetic equals attention over the whole range."""
    cfg, lens = _case("c1")
    q, k, v, off = make_layer_inputs(cfg, 0, lengths=lens)
    ref = orc.decode_attention(q, k, v, off)[0]
    S = int(off[0]) + 1
    for n in (2, 4, 8):
        states = []
        for r in range(n):
            lo, hi = r * S // n, (r + 1) * S // n
            pm, pl, po = orc.split_kv_partial(q, k[:, lo:hi], v[:, lo:hi], np.array([hi - lo - 1], dtype=np.int32),
                                              cfg.scale, 1)
            states.append((pm[0, :, 0], pl[0, :, 0], po[0, :, 0]))
        out = orc.merge_shard_states(states)
        max_abs, rel = orc.parity_metrics(out[None], ref[None])
        assert max_abs < 1e-5 and rel < 1e-5
