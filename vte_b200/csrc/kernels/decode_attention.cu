// Split-KV flash-decoding GQA attention over an fp16 KV cache, for sm_100a.
//
// Two families of kernels share the same buffers:
//
//   * the reference-named kernels (`kv_cache_append_kernel`,
//     `flash_attention_split_kv_partial_kernel`,
//     `flash_attention_split_kv_reduce_kernel`, and the unsplit `flash_attention_kernel`)
//     keep VTE's argument lists AND
//     its launch geometry (grid (B, Hq, C) / (B, Hq, 1) / (B, Hkv, 1), block
//     (head_dim, 1, 1)), so a dispatcher written for the reference can launch
//     them unchanged;
//   * the `vteb_*` kernels are what the B200 dispatcher launches: a persistent
//     split kernel that streams K/V tiles through shared memory with bulk
//     asynchronous copies and serves every query head of a KV head from one
//     read, and a combine kernel that skips empty splits.
//
// Buffer layout (all as in VTE): q [B, Hq, D] fp16; k_cache, v_cache
// [B, max_seq, Hkv, D] fp16, sequence b at element offset b * kv_batch_stride;
// kv_cache_offset_ptr int32[B], sequence b attends to positions
// 0..offset[b] inclusive; partial_m, partial_l [B, Hq, C] fp32; partial_o
// [B, Hq, C, D] fp32.  partial_m is the maximum scaled score of the split in
// natural-log units, partial_l the sum of exp(score - m), partial_o the
// exp-weighted sum of V rows; an empty split holds (-1e30, 0, 0).
#include "vteb_common.cuh"
#include "consumer_block.cuh"

using namespace vteb;

#ifndef SPLIT_KV_CHUNK_SIZE
#define SPLIT_KV_CHUNK_SIZE 0   // > 0 reproduces the reference's fixed chunk length
#endif

// ---------------------------------------------------------------------------
// kv_cache_append_kernel: grid (B, Hkv, 1), block (D, 1, 1).
// Replaces vte/compiler/templates/rdna/kv_cache_append.hip.template:13-39.
// ---------------------------------------------------------------------------
extern "C" __global__ void kv_cache_append_kernel(
    const __half* __restrict__ k, const __half* __restrict__ v,
    __half* __restrict__ k_cache, __half* __restrict__ v_cache,
    int num_kv_heads, int head_dim,
    const int* __restrict__ kv_cache_offset_ptr, int kv_batch_stride)
{
    grid_launch_dependents();
    grid_dependency_wait();
    const int b = blockIdx.x, head = blockIdx.y;
    const long long row = (long long)kv_cache_offset_ptr[b] * num_kv_heads + head;
    const long long dst = (long long)b * kv_batch_stride + row * head_dim;
    const long long src = ((long long)b * num_kv_heads + head) * head_dim;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        k_cache[dst + d] = k[src + d];
        v_cache[dst + d] = v[src + d];
    }
}

// ---------------------------------------------------------------------------
// kv_cache_append_rope_kernel: the append with the K rotation folded in, so the
// row is rotated exactly once, where it enters the cache (rotating K on the
// attention read would rotate history again every step).  Same grid and block;
// `k` is the un-rotated projection and is left as it is.  The reference tried
// this fusion together with the Q-side one of the split kernel and removed it
// again; its standalone counterpart is rope_kernel below.
// ---------------------------------------------------------------------------
extern "C" __global__ void kv_cache_append_rope_kernel(
    const __half* __restrict__ k, const __half* __restrict__ v,
    __half* __restrict__ k_cache, __half* __restrict__ v_cache,
    int num_kv_heads, int head_dim,
    const int* __restrict__ kv_cache_offset_ptr, int kv_batch_stride,
    const __half* __restrict__ cos_cache, const __half* __restrict__ sin_cache,
    int rope_type, int rotary_dim)
{
    grid_launch_dependents();
    grid_dependency_wait();
    const int b = blockIdx.x, head = blockIdx.y;
    const int pos = kv_cache_offset_ptr[b];
    const long long row = (long long)pos * num_kv_heads + head;
    const long long dst = (long long)b * kv_batch_stride + row * head_dim;
    const long long src = ((long long)b * num_kv_heads + head) * head_dim;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        k_cache[dst + d] = rope_channel(k + src, d, head_dim, cos_cache, sin_cache, pos, rope_type, rotary_dim);
        v_cache[dst + d] = v[src + d];
    }
}

// ---------------------------------------------------------------------------
// rope_kernel: in-place rotation of Q and K, any grid (gx, B, 1) and block.
// Replaces vte/compiler/templates/rdna/rope.hip.template:17-140 with its
// argument list: q [B, seq_len, Hq, D], k [B, seq_len, Hkv, D], token i of
// sequence b sits at position kv_cache_offset_ptr[b] + i.  One thread per
// rotated pair (grid-stride over the pairs of Q, then of K).
// ---------------------------------------------------------------------------
__device__ __forceinline__ void rope_rows_inplace(__half* x, int seq_len, int heads, int D, int pos0,
                                                  const __half* cos_cache, const __half* sin_cache,
                                                  int rope_type, int rotary_dim)
{
    const int rot = (rope_type == 1 || rope_type == 0) ? D : rotary_dim;
    const int pairs_per_row = rot >> 1;
    const long long n_pairs = (long long)seq_len * heads * pairs_per_row;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x; p < n_pairs; p += stride) {
        const long long rowi = p / pairs_per_row;
        const int j = (int)(p - rowi * pairs_per_row);
        const int pos = pos0 + (int)(rowi / heads);
        __half* row = x + rowi * D;
        const int i1 = (rope_type == 1) ? 2 * j : j;
        const int i2 = (rope_type == 1) ? 2 * j + 1 : j + pairs_per_row;
        const long long tab = (long long)pos * rot + j;
        float y1, y2;
        rope_pair(__half2float(row[i1]), __half2float(row[i2]),
                  __half2float(cos_cache[tab]), __half2float(sin_cache[tab]), y1, y2);
        row[i1] = __float2half(y1);
        row[i2] = __float2half(y2);
    }
}

extern "C" __global__ void rope_kernel(
    __half* __restrict__ q, __half* __restrict__ k,
    const __half* __restrict__ cos_cache, const __half* __restrict__ sin_cache,
    int seq_len, int num_q_heads, int num_kv_heads, int head_dim,
    const int* __restrict__ kv_cache_offset_ptr, int rope_type, int rotary_dim)
{
    grid_launch_dependents();
    grid_dependency_wait();
    const int b = blockIdx.y;
    const int pos0 = kv_cache_offset_ptr[b];
    rope_rows_inplace(q + (long long)b * seq_len * num_q_heads * head_dim, seq_len, num_q_heads, head_dim, pos0,
                      cos_cache, sin_cache, rope_type, rotary_dim);
    rope_rows_inplace(k + (long long)b * seq_len * num_kv_heads * head_dim, seq_len, num_kv_heads, head_dim, pos0,
                      cos_cache, sin_cache, rope_type, rotary_dim);
}

// ---------------------------------------------------------------------------
// flash_attention_split_kv_partial_kernel, reference geometry:
// grid (B, Hq, C), block (D, 1, 1) with D a multiple of 32 and at most 256.
// Replaces flash_attention_split_kv_partial.hip.template:31-120.  Each warp
// walks every (D/32)-th position of the split with vector loads and a shuffle
// reduction, keeps its own running (m, l, o), and the warps are merged at the
// end.  This is the compatibility kernel; the fast path is further down.
// ---------------------------------------------------------------------------
// kUnsplit: the same walk with ONE split covering every position, preceded by the cache append and
// followed by the normalisation: flash_attention_kernel below.
template <int EPL, bool kUnsplit>   // EPL = elements per lane = head_dim / 32
__device__ __forceinline__ void compat_partial_body(
    const __half* __restrict__ q, const __half* k_cache, const __half* v_cache,
    float* __restrict__ partial_m, float* __restrict__ partial_l, float* __restrict__ partial_o,
    int num_q_heads, int num_kv_heads, float scale,
    const int* __restrict__ kv_cache_offset_ptr, int kv_batch_stride, int max_chunks,
    const __half* __restrict__ k_new = nullptr, const __half* __restrict__ v_new = nullptr,
    __half* __restrict__ output = nullptr)
{
    constexpr int D = EPL * 32;
    __shared__ float sh_m[8], sh_l[8];
    __shared__ float sh_o[8][D];

    const int b = blockIdx.x, h = blockIdx.y, c = kUnsplit ? 0 : blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int total = kv_cache_offset_ptr[b] + 1;
    const int kv_head = h / (num_q_heads / num_kv_heads);
    if constexpr (kUnsplit) {
        // every block writes its KV head's new row (the blocks of a group write identical bytes) and
        // reads it back only after its own barrier
        __half* kc = const_cast<__half*>(k_cache) + (long long)b * kv_batch_stride + ((long long)(total - 1) * num_kv_heads + kv_head) * D;
        __half* vc = const_cast<__half*>(v_cache) + (long long)b * kv_batch_stride + ((long long)(total - 1) * num_kv_heads + kv_head) * D;
        const long long src = ((long long)b * num_kv_heads + kv_head) * D;
        for (int d = threadIdx.x; d < D; d += blockDim.x) { kc[d] = k_new[src + d]; vc[d] = v_new[src + d]; }
        __syncthreads();
    }
    const int chunk = kUnsplit ? total : split_chunk_len(total, max_chunks, SPLIT_KV_CHUNK_SIZE, 0);
    const long long stat = ((long long)b * num_q_heads + h) * max_chunks + c;
    const int start = c * chunk;
    if (!kUnsplit && start >= total) {
        if (threadIdx.x == 0) { partial_m[stat] = kNeutralM; partial_l[stat] = 0.f; }
        for (int d = threadIdx.x; d < D; d += blockDim.x) partial_o[stat * D + d] = 0.f;
        return;
    }
    const int end = min(start + chunk, total);

    float qf[EPL];
    {
        const __half* qp = q + ((long long)b * num_q_heads + h) * D + lane * EPL;
#pragma unroll
        for (int i = 0; i < EPL; ++i) qf[i] = __half2float(qp[i]) * (scale * kLog2e);
    }
    float m = kNeutralM, l = 0.f, o[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) o[i] = 0.f;

    const long long row_stride = (long long)num_kv_heads * D;
    const __half* kbase = k_cache + (long long)b * kv_batch_stride + (long long)kv_head * D + lane * EPL;
    const __half* vbase = v_cache + (long long)b * kv_batch_stride + (long long)kv_head * D + lane * EPL;
    for (int j = start + warp; j < end; j += nwarps) {
        __half kr[EPL], vr[EPL];
        const __half* kp = kbase + (long long)j * row_stride;
        const __half* vp = vbase + (long long)j * row_stride;
        if constexpr (EPL == 8) {
            *reinterpret_cast<uint4*>(kr) = *reinterpret_cast<const uint4*>(kp);
            *reinterpret_cast<uint4*>(vr) = *reinterpret_cast<const uint4*>(vp);
        } else if constexpr (EPL == 4) {
            *reinterpret_cast<uint2*>(kr) = *reinterpret_cast<const uint2*>(kp);
            *reinterpret_cast<uint2*>(vr) = *reinterpret_cast<const uint2*>(vp);
        } else {
            *reinterpret_cast<uint32_t*>(kr) = *reinterpret_cast<const uint32_t*>(kp);
            *reinterpret_cast<uint32_t*>(vr) = *reinterpret_cast<const uint32_t*>(vp);
        }
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) s = fmaf(qf[i], __half2float(kr[i]), s);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        const float m_new = fmaxf(m, s);
        const float corr = fast_exp2(m - m_new);
        const float p = fast_exp2(s - m_new);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < EPL; ++i) o[i] = fmaf(p, __half2float(vr[i]), o[i] * corr);
        m = m_new;
    }
    if (lane == 0) { sh_m[warp] = m; sh_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < EPL; ++i) sh_o[warp][lane * EPL + i] = o[i];
    __syncthreads();
    float mm = kNeutralM;
    for (int w = 0; w < nwarps; ++w) mm = fmaxf(mm, sh_m[w]);
    float ll = 0.f;
    for (int w = 0; w < nwarps; ++w) ll += sh_l[w] * fast_exp2(sh_m[w] - mm);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.f;
        for (int w = 0; w < nwarps; ++w) acc += sh_o[w][d] * fast_exp2(sh_m[w] - mm);
        if constexpr (kUnsplit) output[((long long)b * num_q_heads + h) * D + d] = __float2half(acc / fmaxf(ll, 1e-20f));
        else partial_o[stat * D + d] = acc;
    }
    if (!kUnsplit && threadIdx.x == 0) {
        partial_m[stat] = mm * kLn2;
        partial_l[stat] = ll;
    }
}

extern "C" __global__ void flash_attention_split_kv_partial_kernel(
    const __half* __restrict__ q, const __half* __restrict__ k_cache, const __half* __restrict__ v_cache,
    float* __restrict__ partial_m, float* __restrict__ partial_l, float* __restrict__ partial_o,
    int num_q_heads, int num_kv_heads, int head_dim, float scale,
    const int* __restrict__ kv_cache_offset_ptr, int kv_batch_stride, int max_chunks)
{
    grid_launch_dependents();
    grid_dependency_wait();
    switch (head_dim) {
    case 64:
        compat_partial_body<2, false>(q, k_cache, v_cache, partial_m, partial_l, partial_o, num_q_heads,
                                      num_kv_heads, scale, kv_cache_offset_ptr, kv_batch_stride, max_chunks);
        break;
    case 128:
        compat_partial_body<4, false>(q, k_cache, v_cache, partial_m, partial_l, partial_o, num_q_heads,
                                      num_kv_heads, scale, kv_cache_offset_ptr, kv_batch_stride, max_chunks);
        break;
    case 256:
        compat_partial_body<8, false>(q, k_cache, v_cache, partial_m, partial_l, partial_o, num_q_heads,
                                      num_kv_heads, scale, kv_cache_offset_ptr, kv_batch_stride, max_chunks);
        break;
    default:
        break;   // the host refuses other head sizes before launching
    }
}

// ---------------------------------------------------------------------------
// flash_attention_kernel, the reference's unsplit decode attention with its 13 arguments
// (vte/compiler/templates/rdna/flash_attention.hip.template:29-113, argument table
// vte/core/kernel_arg_builder.py:57-71) and its launch geometry: grid (B, Hq, 1), block
// (head_dim, 1, 1) (dynamic shared memory is accepted and not used).  It is what the reference's
// batched executor records (vte/core/batched_hip_graph_executor.py:231-247): append this step's
// K/V rows at position kv_offset, attend to positions 0..kv_offset, store the normalised fp16
// output.  `seq_len` must be 1, as in the reference.  One block serves one query head, so K and V
// are read once per query head (through L2); the dispatcher's own one-launch path for short
// contexts is the split kernel with one split, which reads them once per KV head.
// ---------------------------------------------------------------------------
extern "C" __global__ void flash_attention_kernel(
    const __half* __restrict__ q, const __half* __restrict__ k, const __half* __restrict__ v,
    __half* __restrict__ k_cache, __half* __restrict__ v_cache, __half* __restrict__ output,
    int seq_len, int num_q_heads, int num_kv_heads, int head_dim, float scale,
    const int* __restrict__ kv_cache_offset_ptr, int kv_batch_stride)
{
    grid_launch_dependents();
    grid_dependency_wait();
    (void)seq_len;
    switch (head_dim) {
    case 64:
        compat_partial_body<2, true>(q, k_cache, v_cache, nullptr, nullptr, nullptr, num_q_heads, num_kv_heads, scale,
                                     kv_cache_offset_ptr, kv_batch_stride, 1, k, v, output);
        break;
    case 128:
        compat_partial_body<4, true>(q, k_cache, v_cache, nullptr, nullptr, nullptr, num_q_heads, num_kv_heads, scale,
                                     kv_cache_offset_ptr, kv_batch_stride, 1, k, v, output);
        break;
    case 256:
        compat_partial_body<8, true>(q, k_cache, v_cache, nullptr, nullptr, nullptr, num_q_heads, num_kv_heads, scale,
                                     kv_cache_offset_ptr, kv_batch_stride, 1, k, v, output);
        break;
    default:
        break;   // the host refuses other head sizes before launching
    }
}

// ---------------------------------------------------------------------------
// Log-sum-exp merge of the split states.  grid (B, Hq, 1); any block size that
// is a multiple of 32 (the reference launches head_dim threads); dynamic
// shared memory max_chunks * 4 bytes.
// Replaces flash_attention_split_kv_reduce.hip.template:14-67.
//   M = max_c m_c;  w_c = exp(m_c - M);  L = max(sum_c l_c w_c, 1e-20);
//   out[d] = sum_c o_c[d] w_c / L.
// kSkipNeutral: splits whose m is the neutral -1e30 get weight 0 and their
// partial_o is never read (the fast split kernel does not write it for them).
// ---------------------------------------------------------------------------
template <typename OutT> __device__ __forceinline__ OutT to_out(float x);
template <> __device__ __forceinline__ float to_out<float>(float x) { return x; }
template <> __device__ __forceinline__ __half to_out<__half>(float x) { return __float2half(x); }

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, v, off);
        v = is_max ? fmaxf(v, other) : v + other;
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = scratch[0];
    for (int w = 1; w < nwarps; ++w) r = is_max ? fmaxf(r, scratch[w]) : r + scratch[w];
    return r;
}

template <typename OutT, bool kSkipNeutral>
__device__ __forceinline__ void reduce_body(
    const float* __restrict__ partial_m, const float* __restrict__ partial_l,
    const float* __restrict__ partial_o, OutT* __restrict__ output,
    int num_q_heads, int head_dim, int max_chunks)
{
    extern __shared__ float weight_sh[];   // max_chunks floats
    __shared__ float scratch[32];
    const int b = blockIdx.x, h = blockIdx.y;
    const long long base = ((long long)b * num_q_heads + h) * max_chunks;

    float mx = kNeutralM;
    for (int c = threadIdx.x; c < max_chunks; c += blockDim.x) mx = fmaxf(mx, partial_m[base + c]);
    const float M = block_reduce(mx, true, scratch);

    float lsum = 0.f;
    for (int c = threadIdx.x; c < max_chunks; c += blockDim.x) {
        const float mc = partial_m[base + c];
        float w = __expf(mc - M);
        if (kSkipNeutral && mc <= -1e29f) w = 0.f;
        weight_sh[c] = w;
        lsum += partial_l[base + c] * w;
    }
    const float L = fmaxf(block_reduce(lsum, false, scratch), 1e-20f);
    const float inv = 1.f / L;
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        const float* op = partial_o + base * head_dim + d;
        float a0 = 0.f, a1 = 0.f;
        int c = 0;
        for (; c + 1 < max_chunks; c += 2) {
            const float w0 = weight_sh[c], w1 = weight_sh[c + 1];
            if (!kSkipNeutral || w0 != 0.f) a0 = fmaf(op[(long long)c * head_dim], w0, a0);
            if (!kSkipNeutral || w1 != 0.f) a1 = fmaf(op[(long long)(c + 1) * head_dim], w1, a1);
        }
        if (c < max_chunks) {
            const float w0 = weight_sh[c];
            if (!kSkipNeutral || w0 != 0.f) a0 = fmaf(op[(long long)c * head_dim], w0, a0);
        }
        output[((long long)b * num_q_heads + h) * head_dim + d] = to_out<OutT>((a0 + a1) * inv);
    }
}

extern "C" __global__ void flash_attention_split_kv_reduce_kernel(
    const float* __restrict__ partial_m, const float* __restrict__ partial_l,
    const float* __restrict__ partial_o, __half* __restrict__ output,
    int num_q_heads, int head_dim, int max_chunks)
{
    grid_launch_dependents();
    grid_dependency_wait();
    reduce_body<__half, false>(partial_m, partial_l, partial_o, output, num_q_heads, head_dim, max_chunks);
}

// Same arguments, fp32 output: the variant the parity tolerance is stated on.
extern "C" __global__ void flash_attention_split_kv_reduce_f32_kernel(
    const float* __restrict__ partial_m, const float* __restrict__ partial_l,
    const float* __restrict__ partial_o, float* __restrict__ output,
    int num_q_heads, int head_dim, int max_chunks)
{
    grid_launch_dependents();
    grid_dependency_wait();
    reduce_body<float, false>(partial_m, partial_l, partial_o, output, num_q_heads, head_dim, max_chunks);
}

// ---------------------------------------------------------------------------
// Fast combine: grid (B * Hq * D/32, 1, 1), block 256, dynamic shared memory
// max_chunks * 4 bytes.  One CTA merges the splits of one (sequence, query
// head) for 32 output columns.  Thread (r = tid / 8, q = tid % 8) owns the
// float4 columns 4q..4q+3 of splits r, r+32, r+64, ...; every global load of a
// pass (m, l and up to eight partial_o rows per thread) is issued before any of
// them is used, so a CTA pays one L2 round trip, not one per split.  Neutral
// splits get weight 0 and their partial_o is never used.  CTA 0 also clears the
// work-queue ticket so the next split launch starts from zero.
// ---------------------------------------------------------------------------
// kFused: called from inside the split kernel by its 256 consumer threads after a
// grid-wide barrier; CTA-wide synchronisation then uses named barrier 1 (the loader
// warps have left) and partials are read with L2-only loads.
template <bool kFused>
__device__ __forceinline__ void combine_sync() {
    if constexpr (kFused) asm volatile("bar.sync 1, 256;" ::: "memory");
    else __syncthreads();
}

template <bool kFused>
__device__ __forceinline__ float combine_ld(const float* p) { return kFused ? __ldcg(p) : *p; }
template <bool kFused>
__device__ __forceinline__ float4 combine_ld4(const float* p) {
    return kFused ? __ldcg(reinterpret_cast<const float4*>(p)) : *reinterpret_cast<const float4*>(p);
}

// out_kind: 1 = fp16 output, 2 = fp32 output, 3 = unnormalised shard state [D + 2] per row
template <bool kFused>
__device__ __forceinline__ void combine_slice(
    const float* __restrict__ partial_m, const float* __restrict__ partial_l,
    const float* __restrict__ partial_o, void* __restrict__ output, int out_kind,
    int head_dim, int max_chunks, int dsplit, int slice, float* weight_sh)
{
    __shared__ float red_max[8], red_sum[8];
    __shared__ float4 acc_sh[8][8];                // [warp][q]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int bh = slice / dsplit, dpart = slice - bh * dsplit;
    const long long base = (long long)bh * max_chunks;
    const int r = tid >> 3, q = tid & 7;
    const float* o_base = partial_o + base * head_dim + dpart * 32 + q * 4;

    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float M = kNeutralM, lsum = 0.f;
    // max_chunks <= 256 takes one pass; longer split lists are folded pass by pass
    // with the usual running-maximum rescale.
    for (int c0 = 0; c0 < max_chunks; c0 += 256) {
        const int cm = c0 + tid;
        const float my_m = (cm < max_chunks) ? combine_ld<kFused>(partial_m + base + cm) : kNeutralM;
        const float my_l = (cm < max_chunks) ? combine_ld<kFused>(partial_l + base + cm) : 0.f;
        float4 o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int c = c0 + r + 32 * k;
            o[k] = (c < max_chunks) ? combine_ld4<kFused>(o_base + (long long)c * head_dim) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        // ---- maximum of this pass
        float mx = my_m;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        combine_sync<kFused>();                     // previous pass / slice is done with red_* and weight_sh
        if (lane == 0) red_max[warp] = mx;
        combine_sync<kFused>();
        float pass_max = red_max[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) pass_max = fmaxf(pass_max, red_max[w]);
        const float M_new = fmaxf(M, pass_max);
        const float rescale = __expf(M - M_new);    // 1 on the first pass (both neutral) or exp(-big) = 0
        M = M_new;
        // ---- weights and the sum of l
        const float wgt = (my_m <= -1e29f) ? 0.f : __expf(my_m - M);
        if (cm < max_chunks) weight_sh[cm - c0] = wgt;
        float ls = my_l * wgt;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ls += __shfl_xor_sync(0xffffffffu, ls, off);
        if (lane == 0) red_sum[warp] = ls;
        combine_sync<kFused>();
        float pass_l = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) pass_l += red_sum[w];
        lsum = lsum * rescale + pass_l;
        acc.x *= rescale; acc.y *= rescale; acc.z *= rescale; acc.w *= rescale;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int c = c0 + r + 32 * k;
            if (c < max_chunks) {
                const float w = weight_sh[c - c0];
                if (w != 0.f) {
                    acc.x = fmaf(o[k].x, w, acc.x); acc.y = fmaf(o[k].y, w, acc.y);
                    acc.z = fmaf(o[k].z, w, acc.z); acc.w = fmaf(o[k].w, w, acc.w);
                }
            }
        }
    }
    // ---- sum over the 32 row groups: lanes with equal q inside a warp, then the 8 warps
#pragma unroll
    for (int off = 8; off <= 16; off <<= 1) {
        acc.x += __shfl_xor_sync(0xffffffffu, acc.x, off); acc.y += __shfl_xor_sync(0xffffffffu, acc.y, off);
        acc.z += __shfl_xor_sync(0xffffffffu, acc.z, off); acc.w += __shfl_xor_sync(0xffffffffu, acc.w, off);
    }
    if (lane < 8) acc_sh[warp][lane] = acc;
    combine_sync<kFused>();
    if (tid < 32) {
        const float* flat = reinterpret_cast<const float*>(acc_sh);
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) s += flat[w * 32 + tid];
        if (out_kind == 3) {
            // unnormalised state of this shard: o[D], then m (natural-log units), then l
            float* st = reinterpret_cast<float*>(output) + (long long)bh * (head_dim + 2);
            st[dpart * 32 + tid] = s;
            if (dpart == 0 && tid == 0) { st[head_dim] = M; st[head_dim + 1] = lsum; }
        } else {
            const float v = s / fmaxf(lsum, 1e-20f);
            const long long idx = (long long)bh * head_dim + dpart * 32 + tid;
            if (out_kind == 2) reinterpret_cast<float*>(output)[idx] = v;
            else reinterpret_cast<__half*>(output)[idx] = __float2half(v);
        }
    }
}

__device__ __forceinline__ void fast_combine_kernel_body(
    const float* __restrict__ partial_m, const float* __restrict__ partial_l,
    const float* __restrict__ partial_o, void* __restrict__ output, int out_kind,
    int head_dim, int max_chunks, int dsplit, int* __restrict__ ticket)
{
    extern __shared__ float combine_weight_sh[];   // [min(max_chunks, 256)]
#ifdef VTEB_TRACE
    // timeline trace (see split_kv_fast.cuh): first and last CTA stamp %globaltimer at entry, after the
    // dependency wait and at the end, into [launch][2][4] 64-bit words at byte 256 + 64 * 3 * 10 * 32 * 8
    unsigned long long* ctr = nullptr;
    if (threadIdx.x == 0 && ticket != nullptr && (blockIdx.x == 0 || blockIdx.x + 1 == gridDim.x)) {
        const int sel = blockIdx.x == 0 ? 0 : 1;
        const int launch = atomicAdd(ticket + 1 + 18 + sel, 1);
        if (launch < 64) ctr = reinterpret_cast<unsigned long long*>(ticket) + 32 + 64 * 3 * 10 * 32 + (launch * 2 + sel) * 4;
        if (ctr) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ctr[0]));
    }
#endif
    grid_launch_dependents();
    grid_dependency_wait();
#ifdef VTEB_TRACE
    if (ctr) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ctr[1]));
#endif
    if (blockIdx.x == 0 && threadIdx.x == 0 && ticket != nullptr) *ticket = 0;
    combine_slice<false>(partial_m, partial_l, partial_o, output, out_kind, head_dim, max_chunks, dsplit,
                         blockIdx.x, combine_weight_sh);
#ifdef VTEB_TRACE
    if (ctr) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ctr[2]));
#endif
}

extern "C" __global__ void __launch_bounds__(256) vteb_split_kv_combine_f16_kernel(
    const float* __restrict__ partial_m, const float* __restrict__ partial_l,
    const float* __restrict__ partial_o, __half* __restrict__ output,
    int num_q_heads, int head_dim, int max_chunks, int dsplit, int* __restrict__ ticket)
{
    fast_combine_kernel_body(partial_m, partial_l, partial_o, output, 1, head_dim, max_chunks, dsplit, ticket);
}

extern "C" __global__ void __launch_bounds__(256) vteb_split_kv_combine_f32_kernel(
    const float* __restrict__ partial_m, const float* __restrict__ partial_l,
    const float* __restrict__ partial_o, float* __restrict__ output,
    int num_q_heads, int head_dim, int max_chunks, int dsplit, int* __restrict__ ticket)
{
    fast_combine_kernel_body(partial_m, partial_l, partial_o, output, 2, head_dim, max_chunks, dsplit, ticket);
}

// ---------------------------------------------------------------------------
// Combine for short split lists (max_chunks <= 64), as batched decode produces:
// one warp per (sequence, query head) row, eight rows per CTA, no shared memory
// and no CTA-wide barrier.  Lane c holds the m and l of splits c and c + 32; the
// lane owns head_dim / 32 consecutive output columns and walks the splits eight
// at a time with all loads of a group in flight.  A warp covers 32 * epl columns
// of a row (epl in {1, 2, 4, 8}, chosen by the host so that a few thousand warps
// exist); grid (ceil(B * Hq * head_dim / (32 * epl) / 8), 1, 1), block 256.
// out_kind: 1 fp16, 2 fp32, 3 shard state.
// ---------------------------------------------------------------------------
template <int EPL>
__device__ __forceinline__ void combine_rows_body(
    const float* __restrict__ partial_m, const float* __restrict__ partial_l,
    const float* __restrict__ partial_o, void* __restrict__ output, int out_kind,
    int rows, int max_chunks, int D)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int groups = D / (32 * EPL);                 // column groups per row
    const int unit = blockIdx.x * 8 + warp;
    const int row = unit / groups, col0 = (unit - row * groups) * 32 * EPL;
    if (row >= rows) return;
    const long long base = (long long)row * max_chunks;
    const float m0 = (lane < max_chunks) ? partial_m[base + lane] : kNeutralM;
    const float m1 = (lane + 32 < max_chunks) ? partial_m[base + lane + 32] : kNeutralM;
    const float l0 = (lane < max_chunks) ? partial_l[base + lane] : 0.f;
    const float l1 = (lane + 32 < max_chunks) ? partial_l[base + lane + 32] : 0.f;
    float M = fmaxf(m0, m1);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
    const float w0 = (m0 <= -1e29f) ? 0.f : __expf(m0 - M);
    const float w1 = (m1 <= -1e29f) ? 0.f : __expf(m1 - M);
    float L = l0 * w0 + l1 * w1;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) L += __shfl_xor_sync(0xffffffffu, L, off);

    // Live splits come first (a split is empty only past the sequence's end), so the
    // walk stops at the last split that holds anything.
    const unsigned live0 = __ballot_sync(0xffffffffu, m0 > -1e29f), live1 = __ballot_sync(0xffffffffu, m1 > -1e29f);
    const int n_live = live1 ? 64 - __clz(live1) : 32 - __clz(live0);

    float acc[EPL];
#pragma unroll
    for (int i = 0; i < EPL; ++i) acc[i] = 0.f;
    const float* op = partial_o + base * D + col0 + lane * EPL;
    for (int c0 = 0; c0 < n_live; c0 += 8) {
        float x[8][EPL];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int c = c0 + k;
            if (c < n_live) {
                const float* src = op + (long long)c * D;
                if constexpr (EPL == 1) {
                    x[k][0] = *src;
                } else if constexpr (EPL == 2) {
                    const float2 v = *reinterpret_cast<const float2*>(src);
                    x[k][0] = v.x; x[k][1] = v.y;
                } else {
#pragma unroll
                    for (int i = 0; i < EPL; i += 4) {
                        const float4 v = *reinterpret_cast<const float4*>(src + i);
                        x[k][i] = v.x; x[k][i + 1] = v.y; x[k][i + 2] = v.z; x[k][i + 3] = v.w;
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < EPL; ++i) x[k][i] = 0.f;
            }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int c = c0 + k;                                  // warp-uniform
            const float w = __shfl_sync(0xffffffffu, (c < 32) ? w0 : w1, c & 31);
            if (c < n_live && w != 0.f) {
#pragma unroll
                for (int i = 0; i < EPL; ++i) acc[i] = fmaf(x[k][i], w, acc[i]);
            }
        }
    }
    if (out_kind == 3) {
        float* st = reinterpret_cast<float*>(output) + (long long)row * (D + 2);
#pragma unroll
        for (int i = 0; i < EPL; ++i) st[col0 + lane * EPL + i] = acc[i];
        if (lane == 0 && col0 == 0) { st[D] = M; st[D + 1] = L; }
    } else {
        const float inv = 1.f / fmaxf(L, 1e-20f);
        if (out_kind == 2) {
            float* o = reinterpret_cast<float*>(output) + (long long)row * D + col0 + lane * EPL;
#pragma unroll
            for (int i = 0; i < EPL; ++i) o[i] = acc[i] * inv;
        } else {
            __half* o = reinterpret_cast<__half*>(output) + (long long)row * D + col0 + lane * EPL;
#pragma unroll
            for (int i = 0; i < EPL; ++i) o[i] = __float2half(acc[i] * inv);
        }
    }
}

extern "C" __global__ void __launch_bounds__(256) vteb_split_kv_combine_rows_kernel(
    const float* __restrict__ partial_m, const float* __restrict__ partial_l,
    const float* __restrict__ partial_o, void* __restrict__ output,
    int num_q_heads, int head_dim, int max_chunks, int out_kind, int* __restrict__ ticket, int rows, int epl)
{
    grid_launch_dependents();
    grid_dependency_wait();
    if (blockIdx.x == 0 && threadIdx.x == 0 && ticket != nullptr) *ticket = 0;
    (void)num_q_heads;
    // epl = columns per lane; a warp covers 32 * epl columns of one row
    if (epl == 1) combine_rows_body<1>(partial_m, partial_l, partial_o, output, out_kind, rows, max_chunks, head_dim);
    else if (epl == 2) combine_rows_body<2>(partial_m, partial_l, partial_o, output, out_kind, rows, max_chunks, head_dim);
    else if (epl == 4) combine_rows_body<4>(partial_m, partial_l, partial_o, output, out_kind, rows, max_chunks, head_dim);
    else combine_rows_body<8>(partial_m, partial_l, partial_o, output, out_kind, rows, max_chunks, head_dim);
}

// Combine for one short sequence (compact split kernel; chosen up to 32 splits, correct up to 64): one warp per
// (query head, 32 output columns), lane = column, no shared memory, no barrier, and every load of the
// first 32 splits (m, l and the lane's column of every split's partial_o) is issued before the first use:
// one L2 round trip.  Capped at 80 registers so that its CTAs sit beside a compact split CTA like the wide
// combine's (the row kernel above needs 111 and starts only when the split CTA has left).  Same argument
// list as the row kernel (`epl` is 1); grid (ceil(rows * head_dim / 32 / 8), 1, 1), block 256.
extern "C" __global__ void __maxnreg__(80) vteb_split_kv_combine_small_kernel(
    const float* __restrict__ partial_m, const float* __restrict__ partial_l,
    const float* __restrict__ partial_o, void* __restrict__ output,
    int num_q_heads, int head_dim, int max_chunks, int out_kind, int* __restrict__ ticket, int rows, int epl)
{
    grid_launch_dependents();
    grid_dependency_wait();
    if (blockIdx.x == 0 && threadIdx.x == 0 && ticket != nullptr) *ticket = 0;
    (void)num_q_heads; (void)epl;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int D = head_dim, groups = D / 32;
    const int unit = blockIdx.x * 8 + warp;
    const int row = unit / groups, col = (unit - row * groups) * 32 + lane;
    if (row >= rows) return;
    const long long base = (long long)row * max_chunks;
    const float m0 = (lane < max_chunks) ? partial_m[base + lane] : kNeutralM;
    const float m1 = (lane + 32 < max_chunks) ? partial_m[base + lane + 32] : kNeutralM;
    const float l0 = (lane < max_chunks) ? partial_l[base + lane] : 0.f;
    const float l1 = (lane + 32 < max_chunks) ? partial_l[base + lane + 32] : 0.f;
    const float* op = partial_o + base * D + col;
    float x[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) x[k] = (k < max_chunks) ? op[(long long)k * D] : 0.f;
    float M = fmaxf(m0, m1);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
    const float w0 = (m0 <= -1e29f) ? 0.f : __expf(m0 - M);      // an empty split's partial_o may hold anything
    const float w1 = (m1 <= -1e29f) ? 0.f : __expf(m1 - M);
    float L = l0 * w0 + l1 * w1;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) L += __shfl_xor_sync(0xffffffffu, L, off);
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) {
        const float w = __shfl_sync(0xffffffffu, w0, k);
        if (w != 0.f) acc = fmaf(x[k], w, acc);
    }
    if (max_chunks > 32) {
#pragma unroll
        for (int k = 0; k < 32; ++k) x[k] = (k + 32 < max_chunks) ? op[(long long)(k + 32) * D] : 0.f;
#pragma unroll
        for (int k = 0; k < 32; ++k) {
            const float w = __shfl_sync(0xffffffffu, w1, k);
            if (w != 0.f) acc = fmaf(x[k], w, acc);
        }
    }
    if (out_kind == 3) {
        float* st = reinterpret_cast<float*>(output) + (long long)row * (D + 2);
        st[col] = acc;
        if (col == 0) { st[D] = M; st[D + 1] = L; }
    } else {
        const float v = acc / fmaxf(L, 1e-20f);
        if (out_kind == 2) reinterpret_cast<float*>(output)[(long long)row * D + col] = v;
        else reinterpret_cast<__half*>(output)[(long long)row * D + col] = __float2half(v);
    }
}

// ---------------------------------------------------------------------------
// KV-range sharding across GPUs (one very long sequence): every GPU reduces its
// own splits to ONE unnormalised state per query head, laid out as
// [B * Hq][D + 2] floats = o[D], m, l (6,240 bytes for 12 heads of 128), the
// states are all-gathered, and vteb_merge_shard_states_kernel applies the same
// log-sum-exp merge over the shard axis.  No counterpart in the reference, which
// is single-GPU; the arithmetic is that of
// flash_attention_split_kv_reduce.hip.template:24-66.
// ---------------------------------------------------------------------------
extern "C" __global__ void __launch_bounds__(256) vteb_split_kv_combine_state_kernel(
    const float* __restrict__ partial_m, const float* __restrict__ partial_l,
    const float* __restrict__ partial_o, float* __restrict__ state,
    int num_q_heads, int head_dim, int max_chunks, int dsplit, int* __restrict__ ticket)
{
    fast_combine_kernel_body(partial_m, partial_l, partial_o, state, 3, head_dim, max_chunks, dsplit, ticket);
}

// Merges up to eight shard states of one query row: `st0` points at shard 0's row
// ([head_dim] o, m, l), consecutive shards are `shard_stride` floats apart.  Every load of a
// column is issued before any is used (one L2 round trip instead of one per shard).
template <bool kBypassL1>
__device__ __forceinline__ void merge_row_states(const float* __restrict__ st0, long long shard_stride, int n_shards,
                                                 int head_dim, float* __restrict__ out_row)
{
    float mr[8], lr[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        const float* st = st0 + r * shard_stride;
        mr[r] = (r < n_shards) ? (kBypassL1 ? __ldcg(st + head_dim) : st[head_dim]) : kNeutralM;
        lr[r] = (r < n_shards) ? (kBypassL1 ? __ldcg(st + head_dim + 1) : st[head_dim + 1]) : 0.f;
    }
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float ov[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const float* st = st0 + r * shard_stride;
            ov[r] = (r < n_shards) ? (kBypassL1 ? __ldcg(st + d) : st[d]) : 0.f;
        }
        float M = kNeutralM;
#pragma unroll
        for (int r = 0; r < 8; ++r) M = fmaxf(M, mr[r]);
        float acc = 0.f, L = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const float w = (mr[r] <= -1e29f) ? 0.f : __expf(mr[r] - M);
            acc = fmaf(ov[r], w, acc);
            L = fmaf(lr[r], w, L);
        }
        out_row[d] = acc / fmaxf(L, 1e-20f);
    }
}

// gathered: [n_shards][rows][D + 2]; out: [rows][D] fp32.  grid (rows, 1, 1), block (D, 1, 1).
extern "C" __global__ void vteb_merge_shard_states_kernel(
    const float* __restrict__ gathered, float* __restrict__ out, int n_shards, int rows, int head_dim)
{
    grid_launch_dependents();
    grid_dependency_wait();
    const int row = blockIdx.x, pitch = head_dim + 2;
    if (n_shards <= 8) {
        merge_row_states<false>(gathered + (long long)row * pitch, (long long)rows * pitch, n_shards, head_dim,
                                out + (long long)row * head_dim);
        return;
    }
    float M = kNeutralM;
    for (int r = 0; r < n_shards; ++r) M = fmaxf(M, gathered[((long long)r * rows + row) * pitch + head_dim]);
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float acc = 0.f, L = 0.f;
        for (int r = 0; r < n_shards; ++r) {
            const float* st = gathered + ((long long)r * rows + row) * pitch;
            const float m = st[head_dim];
            const float w = (m <= -1e29f) ? 0.f : __expf(m - M);
            if (w != 0.f) { acc = fmaf(st[d], w, acc); L = fmaf(st[head_dim + 1], w, L); }
        }
        out[(long long)row * head_dim + d] = acc / fmaxf(L, 1e-20f);
    }
}

// ---------------------------------------------------------------------------
// The same exchange without a collective library: every rank stores its state
// row block straight into each peer's "board" over NVLink (plain peer stores into
// memory the peer exported), then raises a flag there; the merge kernel waits,
// bounded, for the flags of all ranks.  Boards are double-buffered by step parity
// (a rank can run at most one step ahead of the slowest: its next merge needs that
// rank's push), flags hold step + 1, and the step word is advanced by the last
// kernel of the step.
//   board: [2 parities][n_layers][world][state_floats] floats
//   flags: [2 parities][n_layers][world] ints
// ---------------------------------------------------------------------------
struct VtebPeerTable {
    float* board[8];
    int* flags[8];
};

// grid (world, 1, 1), block 256: CTA p copies this rank's state into peer p's board.
extern "C" __global__ void __launch_bounds__(256) vteb_push_shard_state_kernel(
    const float* __restrict__ state, VtebPeerTable peers, int world, int rank, int layer, int n_layers,
    int state_floats, const int* __restrict__ step_word)
{
    grid_launch_dependents();
    grid_dependency_wait();
    const int p = blockIdx.x;
    if (p >= world) return;
    const int step = *step_word;
    const long long slot = ((long long)(step & 1) * n_layers + layer) * world + rank;
    float* dst = peers.board[p] + slot * state_floats;
    for (int i = threadIdx.x; i < state_floats; i += blockDim.x) dst[i] = state[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        volatile int* flag = peers.flags[p] + slot;
        *flag = step + 1;
        __threadfence_system();
    }
}

// grid (rows, 1, 1), block (D, 1, 1): waits for every rank's flag, then merges.
extern "C" __global__ void vteb_merge_shard_states_p2p_kernel(
    const float* __restrict__ board, const int* __restrict__ flags, float* __restrict__ out, int world, int rows,
    int head_dim, int layer, int n_layers, const int* __restrict__ step_word, int* __restrict__ status)
{
    __shared__ int ok_sh;
    grid_launch_dependents();
    grid_dependency_wait();
    const int step = *step_word;
    const long long slot0 = ((long long)(step & 1) * n_layers + layer) * world;
    if (threadIdx.x == 0) {
        int ok = 1;
        const long long t0 = clock64();
        for (int r = 0; r < world && ok; ++r) {
            const volatile int* flag = flags + slot0 + r;
            while (*flag != step + 1) {
                if (clock64() - t0 > kWaitLimitCycles) { ok = 0; break; }   // give up, report, return
            }
        }
        __threadfence_system();
        if (!ok) atomicCAS(status, 0, kStatusGridTimeout);
        ok_sh = ok;
    }
    __syncthreads();
    if (!ok_sh) return;
    const int row = blockIdx.x, pitch = head_dim + 2;
    const long long state_floats = (long long)rows * pitch;
    const float* base = board + slot0 * state_floats;
    float M = kNeutralM;
    for (int r = 0; r < world; ++r) M = fmaxf(M, __ldcg(base + r * state_floats + (long long)row * pitch + head_dim));
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float acc = 0.f, L = 0.f;
        for (int r = 0; r < world; ++r) {
            const float* st = base + r * state_floats + (long long)row * pitch;
            const float m = __ldcg(st + head_dim);
            const float w = (m <= -1e29f) ? 0.f : __expf(m - M);
            if (w != 0.f) { acc = fmaf(__ldcg(st + d), w, acc); L = fmaf(__ldcg(st + head_dim + 1), w, L); }
        }
        out[(long long)row * head_dim + d] = acc / fmaxf(L, 1e-20f);
    }
}

// ---------------------------------------------------------------------------
// The exchange fused into the state combine ("LL" form): every value travels as an
// 8-byte word (fp32 bits, tag = step + 1) written with one 64-bit store, so a word is
// valid exactly when its tag matches and neither a fence nor a separate flag is needed.
//   pairs: [2 parities][n_layers][world][state_floats] 64-bit words per rank's board
// vteb_split_kv_combine_push_kernel = vteb_split_kv_combine_state_kernel (same grid, block
// and shared memory) + peer stores of the slice each CTA produced, into every rank's board
// (its own included) + that slice of the merge: the CTA's first warp polls (bounded) the same
// 32 columns and the row's m, l of every rank on the local board and stores the merged,
// normalised output.  With `merged_out` null the merge is left to
// vteb_merge_shard_states_ll_kernel.  Plain peer stores and local loads only.
// ---------------------------------------------------------------------------
struct VtebPairBoards {
    unsigned long long* board[8];
};

__device__ __forceinline__ void store_tagged(unsigned long long* p, float v, int tag) {
    const unsigned long long w = ((unsigned long long)(unsigned)tag << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long load_tagged(const unsigned long long* p) {
    unsigned long long w;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}

// (capped at 80 registers so that its CTAs still fit beside a compact split CTA)
extern "C" __global__ void __maxnreg__(80) vteb_split_kv_combine_push_kernel(
    const float* __restrict__ partial_m, const float* __restrict__ partial_l,
    const float* __restrict__ partial_o, float* __restrict__ state, VtebPairBoards peers,
    int num_q_heads, int head_dim, int max_chunks, int dsplit, int* __restrict__ ticket,
    int world, int rank, int layer, int n_layers, int rows, const int* __restrict__ step_word,
    const unsigned long long* __restrict__ local_board, float* __restrict__ merged_out, int* __restrict__ status)
{
    extern __shared__ float combine_weight_sh[];   // [min(max_chunks, 256)]
    grid_launch_dependents();
    grid_dependency_wait();
    if (blockIdx.x == 0 && threadIdx.x == 0 && ticket != nullptr) *ticket = 0;
    combine_slice<false>(partial_m, partial_l, partial_o, state, 3, head_dim, max_chunks, dsplit, blockIdx.x,
                         combine_weight_sh);
    if (threadIdx.x >= 32) return;
    // the first warp wrote this CTA's 32 columns (and m, l for column part 0) of the local state
    __syncwarp();
    const int bh = blockIdx.x / dsplit, dpart = blockIdx.x - bh * dsplit, pitch = head_dim + 2;
    const int step = *step_word, tag = step + 1;
    const long long state_floats = (long long)rows * pitch;
    const long long layer_slot = ((long long)(step & 1) * n_layers + layer) * world * state_floats;
    const long long slot = layer_slot + (long long)rank * state_floats;
    const long long e = (long long)bh * pitch + dpart * 32 + threadIdx.x;
    const long long em = (long long)bh * pitch + head_dim;
    const float v = state[e];
    const bool extra = dpart == 0 && threadIdx.x < 2;                       // m and l of the row
    const float v2 = extra ? state[em + threadIdx.x] : 0.f;
#pragma unroll
    for (int p = 0; p < 8; ++p) {
        if (p < world) {
            store_tagged(peers.board[p] + slot + e, v, tag);
            if (extra) store_tagged(peers.board[p] + slot + em + threadIdx.x, v2, tag);
        }
    }
    if (merged_out == nullptr) return;             // the merge runs as a launch of its own
    // ---- this CTA's slice of the merge: the same 32 columns (and the row's m, l) of every rank,
    // read from the local board as they arrive
    unsigned long long wo[8], wm[8], wl[8];
    const long long t0 = clock64();
    bool ok = true;
    for (;;) {
        bool all = true;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (r < world) {
                const unsigned long long* st = local_board + layer_slot + r * state_floats;
                wo[r] = load_tagged(st + e);
                wm[r] = load_tagged(st + em);
                wl[r] = load_tagged(st + em + 1);
                all = all && (unsigned)(wo[r] >> 32) == (unsigned)tag && (unsigned)(wm[r] >> 32) == (unsigned)tag &&
                      (unsigned)(wl[r] >> 32) == (unsigned)tag;
            }
        }
        if (all) break;
        if (clock64() - t0 > kWaitLimitCycles) { ok = false; break; }          // give up, report, return
    }
    if (!ok) { atomicCAS(status, 0, kStatusGridTimeout); return; }
    float M = kNeutralM;
#pragma unroll
    for (int r = 0; r < 8; ++r) if (r < world) M = fmaxf(M, __uint_as_float((unsigned)wm[r]));
    float acc = 0.f, L = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        if (r < world) {
            const float m = __uint_as_float((unsigned)wm[r]);
            const float w = (m <= -1e29f) ? 0.f : __expf(m - M);
            acc = fmaf(__uint_as_float((unsigned)wo[r]), w, acc);
            L = fmaf(__uint_as_float((unsigned)wl[r]), w, L);
        }
    }
    merged_out[(long long)bh * head_dim + dpart * 32 + threadIdx.x] = acc / fmaxf(L, 1e-20f);
}

// grid (rows, 1, 1), block (D, 1, 1) with D <= 256.
extern "C" __global__ void vteb_merge_shard_states_ll_kernel(
    const unsigned long long* __restrict__ board, float* __restrict__ out, int world, int rows, int head_dim,
    int layer, int n_layers, const int* __restrict__ step_word, int* __restrict__ status)
{
    grid_launch_dependents();
    grid_dependency_wait();
    const int step = *step_word;
    const unsigned tag = (unsigned)(step + 1);
    const int row = blockIdx.x, pitch = head_dim + 2, d = threadIdx.x;
    const long long state_floats = (long long)rows * pitch;
    const unsigned long long* base = board + (((long long)(step & 1) * n_layers + layer) * world) * state_floats +
                                     (long long)row * pitch;
    unsigned long long wo[8], wm[8], wl[8];
    const long long t0 = clock64();
    bool ok = true;
    for (;;) {
        bool all = true;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (r < world) {
                const unsigned long long* st = base + r * state_floats;
                wo[r] = (d < head_dim) ? load_tagged(st + d) : ((unsigned long long)tag << 32);
                wm[r] = load_tagged(st + head_dim);
                wl[r] = load_tagged(st + head_dim + 1);
                all = all && (unsigned)(wo[r] >> 32) == tag && (unsigned)(wm[r] >> 32) == tag && (unsigned)(wl[r] >> 32) == tag;
            }
        }
        if (all) break;
        if (clock64() - t0 > kWaitLimitCycles) { ok = false; break; }          // give up, report, return
    }
    if (!ok) { atomicCAS(status, 0, kStatusGridTimeout); return; }
    if (d >= head_dim) return;
    float M = kNeutralM;
#pragma unroll
    for (int r = 0; r < 8; ++r) if (r < world) M = fmaxf(M, __uint_as_float((unsigned)wm[r]));
    float acc = 0.f, L = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        if (r < world) {
            const float m = __uint_as_float((unsigned)wm[r]);
            const float w = (m <= -1e29f) ? 0.f : __expf(m - M);
            acc = fmaf(__uint_as_float((unsigned)wo[r]), w, acc);
            L = fmaf(__uint_as_float((unsigned)wl[r]), w, L);
        }
    }
    out[(long long)row * head_dim + d] = acc / fmaxf(L, 1e-20f);
}

// One thread: the decode step is over, the next one uses the other board parity.
extern "C" __global__ void vteb_advance_step_kernel(int* __restrict__ step_word)
{
    grid_launch_dependents();
    grid_dependency_wait();
    if (blockIdx.x == 0 && threadIdx.x == 0) *step_word = *step_word + 1;
}

#include "split_kv_fast.cuh"
