"""Argument lists of every kernel the cubin exports, as ctypes types.

The runtime checks the argument count of each launch against this table: the
reference paid for a missing check of this kind with a GPU hang
(docs/BUGS.md:35) and only validates counts when the caller passes
`expected_args` (vte/bridge/hip_runtime.py:814-818).  The three reference-named
kernels list exactly the arguments of
kv_cache_append.hip.template:13-22,
flash_attention_split_kv_partial.hip.template:31-45 and
flash_attention_split_kv_reduce.hip.template:14-22; `rope_kernel` lists those of
rope.hip.template:17-37 (vte/core/kernel_arg_builder.py:44-56); `flash_attention_kernel` those of
flash_attention.hip.template:29-43 (vte/core/kernel_arg_builder.py:57-71).
"""
import ctypes

P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float

_REFERENCE_PARTIAL = [P, P, P, P, P, P, I, I, I, F, P, I, I]
_FAST_PARTIAL = _REFERENCE_PARTIAL + [I, I, I, P, P, P, P, P, P, I, ctypes.Structure, ctypes.Structure]
# ... batch, min_chunk, flags, seq_order, ticket, status, next K, next V, output, out_kind,
#     tensor map of the K cache, tensor map of the V cache (128 bytes each, by value)
_ROPE_TAIL = [P, P, I, I]                                 # cos table, sin table, rope_type, rotary_dim
_REDUCE = [P, P, P, P, I, I, I]
_FAST_COMBINE = _REDUCE + [I, P]                          # dsplit, ticket

KERNEL_SIGNATURES = {
    "kv_cache_append_kernel": [P, P, P, P, I, I, P, I],
    "kv_cache_append_rope_kernel": [P, P, P, P, I, I, P, I] + _ROPE_TAIL,
    "rope_kernel": [P, P, P, P, I, I, I, I, P, I, I],
    "flash_attention_kernel": [P, P, P, P, P, P, I, I, I, I, F, P, I],     # flash_attention.hip.template:29-43
    "flash_attention_split_kv_partial_kernel": _REFERENCE_PARTIAL,
    "flash_attention_split_kv_reduce_kernel": _REDUCE,
    "flash_attention_split_kv_reduce_f32_kernel": _REDUCE,
    "vteb_split_kv_partial_d64_kernel": _FAST_PARTIAL,
    "vteb_split_kv_partial_d128_kernel": _FAST_PARTIAL,
    "vteb_split_kv_partial_d256_kernel": _FAST_PARTIAL,
    "vteb_split_kv_partial_rope_d64_kernel": _FAST_PARTIAL + _ROPE_TAIL + [P, P],     # + new K row, new V row (fused append)
    "vteb_split_kv_partial_rope_d128_kernel": _FAST_PARTIAL + _ROPE_TAIL + [P, P],
    "vteb_split_kv_partial_rope_d256_kernel": _FAST_PARTIAL + _ROPE_TAIL + [P, P],
    "vteb_split_kv_partial_compact_rope_d64_kernel": _FAST_PARTIAL + _ROPE_TAIL + [P, P],
    "vteb_split_kv_partial_compact_rope_d128_kernel": _FAST_PARTIAL + _ROPE_TAIL + [P, P],
    "vteb_split_kv_partial_compact_rope_d256_kernel": _FAST_PARTIAL + _ROPE_TAIL + [P, P],
    "vteb_split_kv_partial_compact_d64_kernel": _FAST_PARTIAL,
    "vteb_split_kv_partial_compact_d128_kernel": _FAST_PARTIAL,
    "vteb_split_kv_partial_compact_cs_d128_kernel": _FAST_PARTIAL,   # the head's warps split the output columns (short splits)
    "vteb_split_kv_partial_compact_d256_kernel": _FAST_PARTIAL,
    "vteb_split_kv_combine_f16_kernel": _FAST_COMBINE,
    "vteb_split_kv_combine_f32_kernel": _FAST_COMBINE,
    "vteb_split_kv_combine_state_kernel": _FAST_COMBINE,
    "vteb_split_kv_combine_rows_kernel": [P, P, P, P, I, I, I, I, P, I, I],
    "vteb_split_kv_combine_small_kernel": [P, P, P, P, I, I, I, I, P, I, I],
    "vteb_merge_shard_states_kernel": [P, P, I, I, I],
    "vteb_push_shard_state_kernel": [P, ctypes.Structure, I, I, I, I, I, P],
    "vteb_merge_shard_states_p2p_kernel": [P, P, P, I, I, I, I, I, P, P],
    "vteb_split_kv_combine_push_kernel": [P, P, P, P, ctypes.Structure, I, I, I, I, P, I, I, I, I, I, P, P, P, P],
    "vteb_merge_shard_states_ll_kernel": [P, P, I, I, I, I, I, P, P],
    "vteb_advance_step_kernel": [P],
}

# template name (what the reference passes to load_kernel_safe) -> source file
TEMPLATE_SOURCES = {
    "kv_cache_append": "decode_attention.cu",
    "rope": "decode_attention.cu",
    "flash_attention": "decode_attention.cu",
    "flash_attention_split_kv_partial": "decode_attention.cu",
    "flash_attention_split_kv_reduce": "decode_attention.cu",
    "decode_attention": "decode_attention.cu",
}
