"""Generates tests/golden/*.npz by running the REFERENCE's own numpy functions.

Run in a container that has the reference checkout (it is not needed afterwards):

    python tests/golden/make_golden.py /path/to/reference

Imported from the reference, unmodified:
  tools/validate_attention.py::ref_gqa_attention          (the attention oracle)
  tools/validate_rope.py::apply_rope_reference            (NEOX rotation)
  vte/compiler/rope_cache_builder.py::RoPECacheBuilder    (fp16 cos/sin tables)
  vte/core/split_kv_attention.py::_chunk_size_for_cus     (chunk-size rule)

Inputs come from vte_b200.workloads (seeded); each file stores the reference's
outputs plus a sha256 of the input bytes so a test can tell "generator changed"
from "arithmetic changed".
"""
import hashlib
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from vte_b200.workloads import CONFIGS, DecodeConfig, make_layer_inputs  # noqa: E402

SMALL_CASES = {
    # name: (config, explicit lengths)
    "ragged_d64": (DecodeConfig("ragged_d64", 11, 3, 8, 2, 64, 1, 130, 1), [1, 17, 130]),
    "outlier_d256": (DecodeConfig("outlier_d256", 12, 2, 8, 2, 256, 1, 300, 1, sigma_kv=0.5,
                                  outlier_frac=0.01, outlier_scale=20.0), [33, 300]),
    "mha_d128": (DecodeConfig("mha_d128", 13, 2, 4, 4, 128, 1, 96, 1), [96, 31]),
    "group8_d128": (DecodeConfig("group8_d128", 14, 1, 16, 2, 128, 1, 257, 1), [257]),
}


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def reference_decode(ref_fn, cfg, q, k, v, offsets):
    out = np.zeros((cfg.batch, cfg.num_q_heads, cfg.head_dim), dtype=np.float32)
    for b in range(cfg.batch):
        n = int(offsets[b]) + 1
        Q = q[b].astype(np.float32)[None, None]
        K = k[b, :n].astype(np.float32)[None]
        V = v[b, :n].astype(np.float32)[None]
        out[b] = ref_fn(Q, K, V, head_dim=cfg.head_dim, causal=False)[0, 0]
    return out


def make_rope_partial(vr, RoPECacheBuilder):
    """Partial split-half rotation (rope_type 2): the reference builds the table with
    head_dim = rotary_dim (vte/compiler/qwen3_5_mapper.py:292-298) and rotates only
    those channels, so its own numpy rotation applied to the first `rotary_dim`
    channels is the pin."""
    D, rot, theta, max_seq = 256, 64, 1e7, 4096
    cos, sin = RoPECacheBuilder(max_seq_len=max_seq, head_dim=rot, rope_theta=theta).build_cache()
    rng = np.random.default_rng(11)
    x = rng.standard_normal((8, D), dtype=np.float32).astype(np.float16)
    positions = np.array([0, 1, 77, 4095])
    rotated = np.zeros((len(positions),) + x.shape, dtype=np.float16)
    for pi, pos in enumerate(positions):
        xin = np.zeros((1, pos + 1, x.shape[0], rot), dtype=np.float32)
        xin[0, pos] = x[:, :rot].astype(np.float32)
        y = vr.apply_rope_reference(xin, cos.astype(np.float32), sin.astype(np.float32), pos + 1, x.shape[0], rot)
        rotated[pi] = x
        rotated[pi, :, :rot] = y[0, pos].astype(np.float16)
    np.savez_compressed(HERE / "rope_partial.npz", x=x, positions=positions, cos_rows=cos[positions],
                        sin_rows=sin[positions], x_rotated=rotated, rotary_dim=np.array(rot), theta=np.array(theta))


def main(ref_root: str):
    sys.path.insert(0, ref_root)
    sys.path.insert(0, str(Path(ref_root) / "tools"))
    import validate_attention as va          # reference module
    import validate_rope as vr               # reference module
    from vte.compiler.rope_cache_builder import RoPECacheBuilder
    from vte.core.split_kv_attention import _chunk_size_for_cus

    # --- attention outputs
    cases = {name: (cfg, lens) for name, (cfg, lens) in SMALL_CASES.items()}
    cases["c1"] = (CONFIGS["c1"], None)
    cases["c2_layer0"] = (CONFIGS["c2"], None)
    for name, (cfg, lens) in cases.items():
        q, k, v, off = make_layer_inputs(cfg, 0, lengths=lens)
        out = reference_decode(va.ref_gqa_attention, cfg, q, k, v, off)
        np.savez_compressed(HERE / f"attn_{name}.npz", out=out, offsets=off, q=q if q.size < 1 << 16 else q[:1],
                            input_sha256=np.array(digest(q, off, *[k[b, :off[b] + 1] for b in range(cfg.batch)],
                                                         *[v[b, :off[b] + 1] for b in range(cfg.batch)])))
        print(name, out.shape, float(np.abs(out).max()))

    # --- RoPE: table rows and a rotated Q, from the reference's builder and tool
    D, theta, max_seq = 128, 1e6, 32768
    cos, sin = RoPECacheBuilder(max_seq_len=max_seq, head_dim=D, rope_theta=theta).build_cache()
    rows = np.array([0, 1, 2, 1000, 32767])
    rng = np.random.default_rng(7)
    x = rng.standard_normal((12, D), dtype=np.float32).astype(np.float16)
    # the tool rotates [batch, seq, heads, dim] for positions 0..seq-1; place x at the last row
    pos = 32767
    xin = np.zeros((1, pos + 1, 1, D), dtype=np.float32)
    rotated = []
    for h in range(x.shape[0]):
        xin[0, pos, 0] = x[h].astype(np.float32)
        y = vr.apply_rope_reference(xin, cos.astype(np.float32), sin.astype(np.float32), pos + 1, 1, D)
        rotated.append(y[0, pos, 0].astype(np.float16))
    np.savez_compressed(HERE / "rope.npz", rows=rows, cos_rows=cos[rows], sin_rows=sin[rows], x=x,
                        x_rotated=np.stack(rotated), position=np.array(pos), theta=np.array(theta))

    make_rope_partial(vr, RoPECacheBuilder)

    # --- chunk-size rule
    cus = np.array([0, -1, 1, 8, 16, 20, 32, 48, 64, 96, 128, 148, 296, 1024])
    np.savez_compressed(HERE / "chunk_rule.npz", cus=cus, chunk=np.array([_chunk_size_for_cus(int(c)) for c in cus]))
    print("done")


def main_rope_partial_only(ref_root: str):
    sys.path.insert(0, ref_root)
    sys.path.insert(0, str(Path(ref_root) / "tools"))
    import validate_rope as vr               # reference module
    from vte.compiler.rope_cache_builder import RoPECacheBuilder
    make_rope_partial(vr, RoPECacheBuilder)


if __name__ == "__main__":
    # `--only-rope-partial` writes that one fixture and leaves the others' bytes alone
    argv = [a for a in sys.argv[1:] if not a.startswith("--")]
    if not argv:
        sys.exit("usage: make_golden.py <path of the reference checkout> [--only-rope-partial]")
    root = argv[0]
    (main_rope_partial_only if "--only-rope-partial" in sys.argv else main)(root)
