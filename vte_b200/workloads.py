"""Seeded synthetic inputs for the five decode-attention configurations.

No public dataset is involved: shapes follow the layer shapes of the models the
reference runs (Qwen2.5-1.5B: 12 query / 2 KV heads of 128; a Granite-like
32 / 8 heads of 64; a Qwen3.5-like 8 / 2 heads of 256), values are i.i.d.
normal, drawn in fp32 and rounded to fp16.

Draw order per layer, from `numpy.random.default_rng([base_seed, layer])`:
context lengths, Q, K, V, outlier masks.  `base_seed = 42 + config index`
(42 is the seed the reference's own tests use,
tests/integration/test_kernels_numerical.py:43).  The lengths of a config are
those of layer 0 and are the same for every layer.
"""
from __future__ import annotations

from dataclasses import dataclass, replace

import numpy as np


@dataclass(frozen=True)
class DecodeConfig:
    name: str
    index: int
    batch: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    ctx_min: int
    ctx_max: int              # also max_seq of the cache
    layers: int
    sigma_kv: float = 1.0
    outlier_frac: float = 0.0
    outlier_scale: float = 1.0
    rope_theta: float | None = None     # Q rotated (NEOX split-half) at its own position

    @property
    def group(self) -> int:
        return self.num_q_heads // self.num_kv_heads

    @property
    def scale(self) -> float:
        return 1.0 / float(np.sqrt(self.head_dim))

    @property
    def max_seq(self) -> int:
        return self.ctx_max

    @property
    def kv_batch_stride(self) -> int:
        """Elements between consecutive sequences in a K or V cache
        (Hkv * D * context_length, vte/compiler/qwen_mapper.py:321-351)."""
        return self.max_seq * self.num_kv_heads * self.head_dim

    @property
    def base_seed(self) -> int:
        return 42 + self.index

    def shard(self, rank: int, world: int) -> "DecodeConfig":
        """Contiguous block of sequences owned by `rank` (no collective needed)."""
        if self.batch % world:
            raise ValueError(f"batch {self.batch} does not divide over {world} ranks")
        return replace(self, batch=self.batch // world)


CONFIGS = {
    "c1": DecodeConfig("c1", 1, 1, 12, 2, 128, 512, 512, 1),
    "c2": DecodeConfig("c2", 2, 1, 12, 2, 128, 32768, 32768, 28, rope_theta=1e6),
    "c3": DecodeConfig("c3", 3, 64, 32, 8, 64, 1024, 16384, 40),
    "c4": DecodeConfig("c4", 4, 16, 8, 2, 256, 2048, 65536, 1, sigma_kv=0.5, outlier_frac=0.01,
                       outlier_scale=20.0),
    "c5": DecodeConfig("c5", 5, 1, 12, 2, 128, 1048576, 1048576, 1),
}


def draw_context_lengths(cfg: DecodeConfig) -> np.ndarray:
    """int32[batch] context lengths S_b, uniform integers in [ctx_min, ctx_max]."""
    rng = np.random.default_rng([cfg.base_seed, 0])
    return _draw_lengths(cfg, rng)


def _draw_lengths(cfg, rng):
    if cfg.ctx_min == cfg.ctx_max:
        return np.full(cfg.batch, cfg.ctx_max, dtype=np.int32)
    return rng.integers(cfg.ctx_min, cfg.ctx_max + 1, size=cfg.batch).astype(np.int32)


def _normal_f16(rng, shape, sigma):
    x = rng.standard_normal(size=shape, dtype=np.float32)
    if sigma != 1.0:
        x *= np.float32(sigma)
    return x


def rope_rotate_neox(x: np.ndarray, position: int, theta: float) -> np.ndarray:
    """Split-half rotation of fp16 [..., D] vectors at `position`, with the fp16
    cos/sin table the reference builds (fp32 angle = fp32 position * fp32 inverse
    frequency; vte/compiler/rope_cache_builder.py:58-90) and fp32 arithmetic
    rounded to fp16 (vte/compiler/templates/rdna/rope.hip.template:82-97)."""
    d = x.shape[-1]
    half = d // 2
    inv_freq = 1.0 / (theta ** (np.arange(0, half, dtype=np.float32) / half))
    ang = np.float32(position) * inv_freq
    cos = np.cos(ang).astype(np.float16).astype(np.float32)
    sin = np.sin(ang).astype(np.float16).astype(np.float32)
    xf = x.astype(np.float32)
    lo, hi = xf[..., :half], xf[..., half:]
    return np.concatenate([lo * cos - hi * sin, lo * sin + hi * cos], axis=-1).astype(np.float16)


def build_rope_cache(max_seq_len: int, width: int, theta: float):
    """fp16 cos and sin tables [max_seq_len, width], both halves of a row equal, with the
    reference's arithmetic (fp32 positions times fp32 inverse frequencies
    theta^-(i / (width/2)); vte/compiler/rope_cache_builder.py:58-90).  `width` is head_dim,
    or rotary_dim for the partial rotation (vte/compiler/qwen3_5_mapper.py:292-298)."""
    half = width // 2
    inv_freq = 1.0 / (theta ** (np.arange(0, half, dtype=np.float32) / half))
    ang = np.outer(np.arange(max_seq_len, dtype=np.float32), inv_freq)
    cos_h, sin_h = np.cos(ang).astype(np.float16), np.sin(ang).astype(np.float16)
    return np.concatenate([cos_h, cos_h], axis=1), np.concatenate([sin_h, sin_h], axis=1)


def make_layer_inputs(cfg: DecodeConfig, layer: int = 0, lengths: np.ndarray | None = None,
                      seq_slice: slice | None = None):
    """(q [B,Hq,D] f16, k_cache [B,max_seq,Hkv,D] f16, v_cache, kv_offsets int32[B]).

    Only positions below S_b are filled; the rest of the cache is zero and is
    never read.  `lengths` overrides the drawn context lengths (they are still
    drawn, to keep the stream position).  `seq_slice` returns only those
    sequences (every sequence is still drawn so the values do not depend on the
    slice).
    """
    rng = np.random.default_rng([cfg.base_seed, layer])
    drawn = _draw_lengths(cfg, rng)
    lens = drawn if lengths is None else np.asarray(lengths, dtype=np.int32)
    B, Hq, Hkv, D = cfg.batch, cfg.num_q_heads, cfg.num_kv_heads, cfg.head_dim
    q = _normal_f16(rng, (B, Hq, D), 1.0).astype(np.float16)
    if cfg.rope_theta:
        for b in range(B):
            q[b] = rope_rotate_neox(q[b], int(lens[b]) - 1, cfg.rope_theta)
    sel = range(B)[seq_slice] if seq_slice is not None else range(B)
    k_cache = np.zeros((len(sel), cfg.max_seq, Hkv, D), dtype=np.float16)
    v_cache = np.zeros((len(sel), cfg.max_seq, Hkv, D), dtype=np.float16)
    kvs = []
    for which in range(2):            # all K first, then all V
        rows = []
        for b in range(B):
            x = _normal_f16(rng, (int(lens[b]), Hkv, D), cfg.sigma_kv)
            rows.append(x if b in sel else None)
        kvs.append(rows)
    if cfg.outlier_frac > 0:
        for which in range(2):
            for b in range(B):
                mask = rng.random(size=(int(lens[b]), Hkv, D), dtype=np.float32) < cfg.outlier_frac
                if kvs[which][b] is not None:
                    kvs[which][b][mask] *= np.float32(cfg.outlier_scale)
    for i, b in enumerate(sel):
        k_cache[i, :int(lens[b])] = kvs[0][b].astype(np.float16)
        v_cache[i, :int(lens[b])] = kvs[1][b].astype(np.float16)
    offsets = (lens - 1).astype(np.int32)
    if seq_slice is not None:
        return q[seq_slice], k_cache, v_cache, offsets[seq_slice]
    return q, k_cache, v_cache, offsets


def algorithmic_bytes(cfg: DecodeConfig, lengths: np.ndarray) -> int:
    """Bytes one layer's decode step has to move: K and V once per KV head, Q in,
    fp32 output out, one int32 offset per sequence.  Partial buffers are overhead
    and are not counted."""
    kv = int(np.sum(lengths.astype(np.int64))) * 2 * cfg.num_kv_heads * cfg.head_dim * 2
    B = len(lengths)
    return kv + B * cfg.num_q_heads * cfg.head_dim * (2 + 4) + 4 * B
