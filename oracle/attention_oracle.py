"""CPU oracle for VTE's split-KV decode-attention path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this module.  It exists so the CUDA path
can be checked against the arithmetic the reference itself trusts, and so the
benchmark can time that arithmetic on host cores as a reported baseline.

Parity pin: `tests/golden/make_golden.py` imports the reference's own
`tools/validate_attention.py::ref_gqa_attention` and
`vte/compiler/rope_cache_builder.py::RoPECacheBuilder` in a container that has
the reference checkout, runs them on seeded inputs, and commits the outputs
under `tests/golden/`.  `tests/test_oracle_golden.py` checks every function in
this file against those vectors.

What each function restates (paths are relative to the reference project):

* `ref_gqa_attention`            tools/validate_attention.py:11-66
* `decode_attention`             the per-sequence decode call of the above
                                 (tools/validate_attention.py:84-86 casts fp16
                                 inputs to fp32 first; one query, all cached
                                 positions visible, so `causal=False`)
* `split_kv_partial`             vte/compiler/templates/rdna/
                                 flash_attention_split_kv_partial.hip.template:47-119
* `split_kv_reduce`              vte/compiler/templates/rdna/
                                 flash_attention_split_kv_reduce.hip.template:24-66
* `kv_cache_append`              vte/compiler/templates/rdna/kv_cache_append.hip.template:23-38
* `rope_tables`, `rope_neox`     vte/compiler/rope_cache_builder.py:42-97 and
                                 vte/compiler/templates/rdna/rope.hip.template:82-97
* `rope_apply`                   vte/compiler/templates/rdna/rope.hip.template:55-97
                                 (the three rotation types; type 0 and type 2
                                 are pinned through the reference's own numpy
                                 rotation; type 1, which has no Python
                                 counterpart in the reference, is pinned like
                                 the other two through the reference's
                                 rope_kernel itself, see below)

Second pin: `oracle/build_ref.py` compiles the reference's own kernel templates
(append, partial, reduce, unsplit, rope) for CPU threads, and
`tests/golden/make_refkernel_golden.py` stores their outputs as
`tests/golden/refkernel_*.npz`; `tests/test_reference_kernels_cpu.py` checks
`kv_cache_append`, `split_kv_partial`, `split_kv_reduce`, `decode_attention` and
`rope_step` against them (rotation and append bit for bit).
* `chunk_size_for_cus`           vte/core/split_kv_attention.py:40-49
"""
from __future__ import annotations

import numpy as np

NEUTRAL_M = np.float32(-1e30)


def ref_gqa_attention(Q, K, V, head_dim=128, causal=False):
    """fp32 grouped-query attention on [batch, seq, heads, dim] arrays.

    Restates tools/validate_attention.py:11-66.  Scores are
    `einsum(Q_group, K_head) / sqrt(head_dim)`, softmax is the max-subtracted
    form, the output is `einsum(weights, V_head)`; all in the dtype of the
    inputs (the reference's callers pass fp32).  `causal=True` reproduces the
    reference's upper-triangular -1e9 fill, which only broadcasts when the
    query and key lengths are equal; decode never uses it.
    """
    n_batch, q_len, n_q, _ = Q.shape
    k_len, n_kv = K.shape[1], K.shape[2]
    group = n_q // n_kv
    inv_sqrt_d = 1.0 / np.sqrt(head_dim)
    out = np.zeros_like(Q)
    for kv in range(n_kv):
        heads = slice(kv * group, (kv + 1) * group)
        s = np.einsum('bqhd,bkd->bhqk', Q[:, :, heads, :], K[:, :, kv, :]) * inv_sqrt_d
        if causal:
            blocked = np.triu(np.ones((q_len, k_len)), k=1).astype(bool)
            s[:, :, blocked] = -1e9
        e = np.exp(s - np.max(s, axis=-1, keepdims=True))
        w = e / np.sum(e, axis=-1, keepdims=True)
        out[:, :, heads, :] = np.einsum('bhqk,bkd->bqhd', w, V[:, :, kv, :])
    return out


def decode_attention(q, k_cache, v_cache, kv_offsets, scale=None, dtype=np.float32):
    """One decode step for a ragged batch, the way the reference's tool would
    be called once per sequence.

    q        [B, Hq, D]            fp16
    k_cache  [B, max_seq, Hkv, D]  fp16 (v_cache alike)
    kv_offsets int32[B]; sequence b attends to positions 0..kv_offsets[b]
             inclusive (flash_attention_split_kv_partial.hip.template:52-53).
    scale    None -> 1/sqrt(D) (validate_attention.py:22).  Another value is
             applied by rescaling q, which is how `attention_scale` metadata
             replaces the default (vte/core/split_kv_attention.py:163-164).
    Returns [B, Hq, D] in `dtype` (fp32 is the reference's; fp64 is used by
    the tests to bound the oracle's own error).
    """
    B, Hq, D = q.shape
    out = np.zeros((B, Hq, D), dtype=dtype)
    for b in range(B):
        n = int(kv_offsets[b]) + 1
        qb = q[b].astype(dtype)[None, None, :, :]
        if scale is not None:
            qb = qb * dtype(scale * np.sqrt(D))
        kb = k_cache[b, :n].astype(dtype)[None]
        vb = v_cache[b, :n].astype(dtype)[None]
        out[b] = ref_gqa_attention(qb, kb, vb, head_dim=D, causal=False)[0, 0]
    return out


def chunk_size_for_cus(num_cus: int) -> int:
    """Fixed chunk length the reference derives from the compute-unit count
    (vte/core/split_kv_attention.py:40-49): 1024/num_cus rounded, kept in
    [8, 64]; 32 when the count is unknown."""
    if num_cus <= 0:
        return 32
    return max(8, min(64, round(1024 / num_cus)))


def split_ranges(total: int, max_chunks: int, chunk_size: int | None, align: int = 16):
    """Position range [start, end) of every split of one sequence.

    chunk_size given  -> the reference's fixed-size mode: split c covers
                         [c*chunk, min((c+1)*chunk, total)).
    chunk_size None   -> split-count mode: chunk = ceil(total / max_chunks)
                         rounded up to `align`; same formula afterwards.
    Splits that start at or beyond `total` are empty (start == end).
    """
    if chunk_size is None:
        chunk = -(-total // max_chunks)
        chunk = -(-chunk // align) * align
    else:
        chunk = chunk_size
    ranges = []
    for c in range(max_chunks):
        s = c * chunk
        ranges.append((s, min(s + chunk, total)) if s < total else (total, total))
    return ranges


def split_kv_partial(q, k_cache, v_cache, kv_offsets, scale, max_chunks,
                     chunk_size=None, align=16):
    """Unnormalised per-split online-softmax state.

    Restates flash_attention_split_kv_partial.hip.template:47-119: for query
    head h of sequence b and split c, over the split's positions j:
    score_j = scale * <q_h, K[j, h // G]>; m = max score; l = sum exp(score-m);
    o[d] = sum exp(score-m) * V[j, h // G, d].  An empty split stores
    m = -1e30, l = 0, o = 0 (template lines 59-69).  The template builds m, l, o
    by a running rescale; the closed form here is the same quantity and is
    compared with a tolerance, never bit-for-bit.

    Returns partial_m, partial_l [B, Hq, C] and partial_o [B, Hq, C, D], fp32.
    """
    B, Hq, D = q.shape
    Hkv = k_cache.shape[2]
    G = Hq // Hkv
    pm = np.full((B, Hq, max_chunks), NEUTRAL_M, dtype=np.float32)
    pl = np.zeros((B, Hq, max_chunks), dtype=np.float32)
    po = np.zeros((B, Hq, max_chunks, D), dtype=np.float32)
    for b in range(B):
        total = int(kv_offsets[b]) + 1
        qf = q[b].astype(np.float32)
        for c, (s, e) in enumerate(split_ranges(total, max_chunks, chunk_size, align)):
            if e <= s:
                continue
            for kv in range(Hkv):
                kf = k_cache[b, s:e, kv].astype(np.float32)
                vf = v_cache[b, s:e, kv].astype(np.float32)
                hs = slice(kv * G, (kv + 1) * G)
                sc = (qf[hs] @ kf.T) * np.float32(scale)
                m = sc.max(axis=1)
                p = np.exp(sc - m[:, None])
                pm[b, hs, c] = m
                pl[b, hs, c] = p.sum(axis=1)
                po[b, hs, c] = p @ vf
    return pm, pl, po


def split_kv_reduce(partial_m, partial_l, partial_o):
    """Log-sum-exp merge of the split states into the attention output.

    Restates flash_attention_split_kv_reduce.hip.template:24-66:
    M = max_c m_c (starting from -1e30); w_c = exp(m_c - M);
    L = max(sum_c l_c * w_c, 1e-20); out[d] = (sum_c o_c[d] * w_c) / L.
    Returns fp32 [B, Hq, D] (the template rounds this to fp16 on store).
    """
    M = np.maximum(partial_m.max(axis=2), NEUTRAL_M)
    w = np.exp(partial_m - M[..., None]).astype(np.float32)
    L = np.maximum((partial_l * w).sum(axis=2), np.float32(1e-20))
    num = (partial_o * w[..., None]).sum(axis=2)
    return (num / L[..., None]).astype(np.float32)


def kv_cache_append(k_new, v_new, k_cache, v_cache, kv_offsets):
    """Writes the current token's K/V rows at position kv_offsets[b] of each
    sequence, in place (kv_cache_append.hip.template:23-38).
    k_new, v_new: [B, Hkv, D] fp16."""
    for b in range(k_new.shape[0]):
        pos = int(kv_offsets[b])
        k_cache[b, pos] = k_new[b]
        v_cache[b, pos] = v_new[b]


def rope_tables(max_seq_len: int, head_dim: int, rope_theta: float):
    """fp16 cos/sin tables of shape [max_seq_len, head_dim] with both halves
    equal (vte/compiler/rope_cache_builder.py:58-90).  Angles are formed in
    fp32 exactly as the reference does: fp32 positions times fp32 inverse
    frequencies theta^-(i / (D/2))."""
    half = head_dim // 2
    inv_freq = 1.0 / (rope_theta ** (np.arange(0, half, dtype=np.float32) / half))
    ang = np.outer(np.arange(max_seq_len, dtype=np.float32), inv_freq)
    cos_h = np.cos(ang).astype(np.float16)
    sin_h = np.sin(ang).astype(np.float16)
    return np.concatenate([cos_h, cos_h], axis=1), np.concatenate([sin_h, sin_h], axis=1)


def rope_row(position: int, head_dim: int, rope_theta: float):
    """One row of `rope_tables` without building the whole table."""
    half = head_dim // 2
    inv_freq = 1.0 / (rope_theta ** (np.arange(0, half, dtype=np.float32) / half))
    ang = np.float32(position) * inv_freq
    cos_h = np.cos(ang).astype(np.float16)
    sin_h = np.sin(ang).astype(np.float16)
    return np.concatenate([cos_h, cos_h]), np.concatenate([sin_h, sin_h])


def rope_neox(x, cos_row, sin_row):
    """Split-half ("NEOX") rotation of [..., D] fp16 vectors at one position,
    computed in fp32 and rounded to fp16 on store
    (rope.hip.template:82-97): x'[j] = x[j]*cos - x[j+D/2]*sin,
    x'[j+D/2] = x[j]*sin + x[j+D/2]*cos for j < D/2."""
    half = x.shape[-1] // 2
    xf = x.astype(np.float32)
    c = cos_row[:half].astype(np.float32)
    s = sin_row[:half].astype(np.float32)
    lo, hi = xf[..., :half], xf[..., half:]
    return np.concatenate([lo * c - hi * s, lo * s + hi * c], axis=-1).astype(np.float16)


def rope_apply(x, cos_row, sin_row, rope_type=0, rotary_dim=None):
    """Rotation of [..., D] fp16 vectors at one position for the reference's
    three `rope_type`s (rope.hip.template:55-97), fp32 arithmetic with each
    product rounded separately, fp16 on store.

    0  split-half over the whole head: row length D, pair (j, j + D/2).
    1  interleaved: pair (2i, 2i+1) uses entry i of a row of length D
       (template lines 57-66).
    2  split-half inside the first `rotary_dim` channels only: row length
       `rotary_dim`, pair (j, j + rotary_dim/2); the remaining channels pass
       through untouched (template lines 67-81)."""
    D = x.shape[-1]
    xf = x.astype(np.float32)
    cos_row = np.asarray(cos_row).astype(np.float32)
    sin_row = np.asarray(sin_row).astype(np.float32)
    if rope_type == 1:
        c, s = cos_row[:D // 2], sin_row[:D // 2]
        x0, x1 = xf[..., 0::2], xf[..., 1::2]
        out = np.empty_like(xf)
        out[..., 0::2] = x0 * c - x1 * s
        out[..., 1::2] = x0 * s + x1 * c
        return out.astype(np.float16)
    rot = D if rope_type == 0 else int(rotary_dim)
    half = rot // 2
    c, s = cos_row[:half], sin_row[:half]
    lo, hi = xf[..., :half], xf[..., half:rot]
    out = xf.copy()
    out[..., :half] = lo * c - hi * s
    out[..., half:rot] = lo * s + hi * c
    return out.astype(np.float16)


def rope_step(q, k, cos_table, sin_table, kv_offsets, rope_type=0, rotary_dim=None):
    """What `rope_kernel` does in one decode step (seq_len 1): rotates
    q [B, Hq, D] and k [B, Hkv, D] of sequence b at position kv_offsets[b]
    (rope.hip.template:41-55).  Tables are [max_seq, D] (types 0, 1) or
    [max_seq, rotary_dim] (type 2).  Returns new arrays."""
    q2, k2 = q.copy(), k.copy()
    for b in range(q.shape[0]):
        pos = int(kv_offsets[b])
        q2[b] = rope_apply(q[b], cos_table[pos], sin_table[pos], rope_type, rotary_dim)
        k2[b] = rope_apply(k[b], cos_table[pos], sin_table[pos], rope_type, rotary_dim)
    return q2, k2


def merge_shard_states(states):
    """Merge per-shard unnormalised (m, l, o) states of one query head set:
    the KV-range sharded path runs `split_kv_reduce`'s arithmetic over the
    shard axis.  `states` is a list of (m [Hq], l [Hq], o [Hq, D])."""
    m = np.stack([s[0] for s in states], axis=-1)[None]
    l = np.stack([s[1] for s in states], axis=-1)[None]
    o = np.stack([s[2] for s in states], axis=-2)[None]
    return split_kv_reduce(m, l, o)[0]


def parity_metrics(out, ref):
    """(max-abs error, worst per-sequence relative L2 error) between two
    [B, Hq, D] arrays: the two figures the tolerance is stated in."""
    out = np.asarray(out, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    max_abs = float(np.max(np.abs(out - ref))) if out.size else 0.0
    rel = 0.0
    for b in range(out.shape[0]):
        den = float(np.linalg.norm(ref[b]))
        num = float(np.linalg.norm(out[b] - ref[b]))
        rel = max(rel, num / den if den > 0 else num)
    return max_abs, rel
