// Split-KV flash-decoding GQA attention over an fp16 KV cache, for sm_100a.
//
// Two families of kernels share the same buffers:
//
//   * the reference-named kernels (`kv_cache_append_kernel`,
//     `flash_attention_split_kv_partial_kernel`,
//     `flash_attention_split_kv_reduce_kernel`) keep VTE's argument lists AND
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
// flash_attention_split_kv_partial_kernel, reference geometry:
// grid (B, Hq, C), block (D, 1, 1) with D a multiple of 32 and at most 256.
// Replaces flash_attention_split_kv_partial.hip.template:31-120.  Each warp
// walks every (D/32)-th position of the split with vector loads and a shuffle
// reduction, keeps its own running (m, l, o), and the warps are merged at the
// end.  This is the compatibility kernel; the fast path is further down.
// ---------------------------------------------------------------------------
template <int EPL>   // elements per lane = head_dim / 32
__device__ __forceinline__ void compat_partial_body(
    const __half* __restrict__ q, const __half* __restrict__ k_cache, const __half* __restrict__ v_cache,
    float* __restrict__ partial_m, float* __restrict__ partial_l, float* __restrict__ partial_o,
    int num_q_heads, int num_kv_heads, float scale,
    const int* __restrict__ kv_cache_offset_ptr, int kv_batch_stride, int max_chunks)
{
    constexpr int D = EPL * 32;
    __shared__ float sh_m[8], sh_l[8];
    __shared__ float sh_o[8][D];

    const int b = blockIdx.x, h = blockIdx.y, c = blockIdx.z;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int total = kv_cache_offset_ptr[b] + 1;
    const int chunk = split_chunk_len(total, max_chunks, SPLIT_KV_CHUNK_SIZE, 0);
    const long long stat = ((long long)b * num_q_heads + h) * max_chunks + c;
    const int start = c * chunk;
    if (start >= total) {
        if (threadIdx.x == 0) { partial_m[stat] = kNeutralM; partial_l[stat] = 0.f; }
        for (int d = threadIdx.x; d < D; d += blockDim.x) partial_o[stat * D + d] = 0.f;
        return;
    }
    const int end = min(start + chunk, total);
    const int kv_head = h / (num_q_heads / num_kv_heads);

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
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.f;
        for (int w = 0; w < nwarps; ++w) acc += sh_o[w][d] * fast_exp2(sh_m[w] - mm);
        partial_o[stat * D + d] = acc;
    }
    if (threadIdx.x == 0) {
        float ll = 0.f;
        for (int w = 0; w < nwarps; ++w) ll += sh_l[w] * fast_exp2(sh_m[w] - mm);
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
        compat_partial_body<2>(q, k_cache, v_cache, partial_m, partial_l, partial_o, num_q_heads,
                               num_kv_heads, scale, kv_cache_offset_ptr, kv_batch_stride, max_chunks);
        break;
    case 128:
        compat_partial_body<4>(q, k_cache, v_cache, partial_m, partial_l, partial_o, num_q_heads,
                               num_kv_heads, scale, kv_cache_offset_ptr, kv_batch_stride, max_chunks);
        break;
    case 256:
        compat_partial_body<8>(q, k_cache, v_cache, partial_m, partial_l, partial_o, num_q_heads,
                               num_kv_heads, scale, kv_cache_offset_ptr, kv_batch_stride, max_chunks);
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
// Fast combine: grid (B * Hq * dsplit, 1, 1), block 256, dynamic shared memory
// max_chunks * 4 + 8 * dchunk * 4 bytes, where dchunk = head_dim / dsplit.
// Warp w accumulates splits w, w+8, ... for the CTA's slice of head_dim, the
// eight warp sums are added through shared memory.  Neutral splits are
// skipped.  The CTA with index 0 also clears the work-queue ticket so the next
// split launch starts from zero.
// ---------------------------------------------------------------------------
template <typename OutT>
__device__ __forceinline__ void fast_combine_body(
    const float* __restrict__ partial_m, const float* __restrict__ partial_l,
    const float* __restrict__ partial_o, OutT* __restrict__ output,
    int num_q_heads, int head_dim, int max_chunks, int dsplit, int* __restrict__ ticket)
{
    extern __shared__ float csh[];
    float* weight_sh = csh;                  // [max_chunks]
    float* acc_sh = csh + max_chunks;        // [8][dchunk]
    __shared__ float scratch[32];
    grid_launch_dependents();
    grid_dependency_wait();
    if (blockIdx.x == 0 && threadIdx.x == 0 && ticket != nullptr) *ticket = 0;

    const int dchunk = head_dim / dsplit;
    const int bh = blockIdx.x / dsplit, dpart = blockIdx.x % dsplit;
    const long long base = (long long)bh * max_chunks;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    float mx = kNeutralM;
    for (int c = threadIdx.x; c < max_chunks; c += blockDim.x) mx = fmaxf(mx, partial_m[base + c]);
    const float M = block_reduce(mx, true, scratch);
    float lsum = 0.f;
    for (int c = threadIdx.x; c < max_chunks; c += blockDim.x) {
        const float mc = partial_m[base + c];
        const float w = (mc <= -1e29f) ? 0.f : __expf(mc - M);
        weight_sh[c] = w;
        lsum += partial_l[base + c] * w;
    }
    const float L = fmaxf(block_reduce(lsum, false, scratch), 1e-20f);

    // dchunk is 32, 64, 128 or 256: each lane owns dchunk / 32 consecutive floats.
    const int epl = dchunk >> 5;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    const float* op = partial_o + base * head_dim + dpart * dchunk + lane * epl;
    for (int c = warp; c < max_chunks; c += 8) {
        const float w = weight_sh[c];
        if (w == 0.f) continue;
        const float* row = op + (long long)c * head_dim;
        if (epl == 4) {
            const float4 x = *reinterpret_cast<const float4*>(row);
            acc[0] = fmaf(x.x, w, acc[0]); acc[1] = fmaf(x.y, w, acc[1]);
            acc[2] = fmaf(x.z, w, acc[2]); acc[3] = fmaf(x.w, w, acc[3]);
        } else if (epl == 8) {
            const float4 x = *reinterpret_cast<const float4*>(row);
            const float4 y = *reinterpret_cast<const float4*>(row + 4);
            acc[0] = fmaf(x.x, w, acc[0]); acc[1] = fmaf(x.y, w, acc[1]);
            acc[2] = fmaf(x.z, w, acc[2]); acc[3] = fmaf(x.w, w, acc[3]);
            acc[4] = fmaf(y.x, w, acc[4]); acc[5] = fmaf(y.y, w, acc[5]);
            acc[6] = fmaf(y.z, w, acc[6]); acc[7] = fmaf(y.w, w, acc[7]);
        } else if (epl == 2) {
            const float2 x = *reinterpret_cast<const float2*>(row);
            acc[0] = fmaf(x.x, w, acc[0]); acc[1] = fmaf(x.y, w, acc[1]);
        } else {
            acc[0] = fmaf(row[0], w, acc[0]);
        }
    }
    for (int i = 0; i < epl; ++i) acc_sh[warp * dchunk + lane * epl + i] = acc[i];
    __syncthreads();
    const float inv = 1.f / L;
    for (int d = threadIdx.x; d < dchunk; d += blockDim.x) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) s += acc_sh[w * dchunk + d];
        output[(long long)bh * head_dim + dpart * dchunk + d] = to_out<OutT>(s * inv);
    }
}

extern "C" __global__ void __launch_bounds__(256) vteb_split_kv_combine_f16_kernel(
    const float* __restrict__ partial_m, const float* __restrict__ partial_l,
    const float* __restrict__ partial_o, __half* __restrict__ output,
    int num_q_heads, int head_dim, int max_chunks, int dsplit, int* __restrict__ ticket)
{
    fast_combine_body<__half>(partial_m, partial_l, partial_o, output, num_q_heads, head_dim, max_chunks, dsplit, ticket);
}

extern "C" __global__ void __launch_bounds__(256) vteb_split_kv_combine_f32_kernel(
    const float* __restrict__ partial_m, const float* __restrict__ partial_l,
    const float* __restrict__ partial_o, float* __restrict__ output,
    int num_q_heads, int head_dim, int max_chunks, int dsplit, int* __restrict__ ticket)
{
    fast_combine_body<float>(partial_m, partial_l, partial_o, output, num_q_heads, head_dim, max_chunks, dsplit, ticket);
}

// ---------------------------------------------------------------------------
// Fast split kernel.
//
// grid (n_ctas, 1, 1) persistent, block 288 = eight consumer warps + one loader
// warp, dynamic shared memory from make_fast_plan().  A work item is one split
// of one sequence for one group of `hg` KV heads; item t maps to
// (sequence rank t / (n_hgroups * C), head group, split).  CTA i starts with
// item i and draws the following ones from `*ticket` (gridDim.x + atomicAdd).
//
// Loader warp: for every tile of `tile` positions, waits for a free stage,
// writes the tile header, announces the byte count on the stage's "full"
// mbarrier and issues one bulk asynchronous copy per position row of K and of
// V (row_bytes contiguous bytes covering the group's heads) into rows padded by
// 16 bytes.  Rows past the end of the item are filled from the item's last row
// so that every row a consumer touches holds finite numbers.
//
// Consumer warp w: KV head (w % hg) of the group, every wph-th 16-position
// block.  Per block: S = Q K^T with mma.sync m16n8k16 (Q rows are the query
// heads of the KV head, K fragments via ldmatrix), online softmax in the log2
// domain on the accumulator fragment, P split into an fp16 high and low part,
// O += P V with V fragments via ldmatrix.trans.  At the end of an item the
// warps of a KV head exchange (m, l, o) through shared memory and the merged
// state is stored to partial_m / partial_l / partial_o.
//
// Every wait is bounded; a wait that gives up stores a code in `*status`,
// raises the CTA's abort word, and the CTA drains its outstanding copies
// (again bounded) and returns.
// ---------------------------------------------------------------------------
struct FastArgs {
    const __half* q; const __half* k_cache; const __half* v_cache;
    float* partial_m; float* partial_l; float* partial_o;
    int num_q_heads, num_kv_heads; float scale;
    const int* kv_offsets; long long kv_batch_stride; int max_chunks;
    int batch, min_chunk, flags; const int* seq_order; int* ticket; int* status;
};

constexpr int kFlagWriteEmptyO = 1;   // also zero partial_o of empty splits (reference semantics)

template <int D>
__device__ __forceinline__ void fast_partial_body(const FastArgs& a)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const FastPlan plan = make_fast_plan(a.num_q_heads, a.num_kv_heads, D);
    const int group = a.num_q_heads / a.num_kv_heads;

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw);          // full[8], empty[8], merge[2]
    volatile int* abort_word = reinterpret_cast<volatile int*>(smem_raw + 256);
    TileHeader* headers = reinterpret_cast<TileHeader*>(smem_raw + 512);   // 8 * 32 B
    float* merge = reinterpret_cast<float*>(smem_raw + kCtrlBytes);
    uint32_t* q_store = reinterpret_cast<uint32_t*>(smem_raw + kCtrlBytes + plan.merge_bytes);
    unsigned char* stages = smem_raw + kCtrlBytes + plan.merge_bytes + plan.q_bytes;

    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kMaxStages);
    const uint32_t merge_bar0 = smem_u32(bars + 2 * kMaxStages);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, plan.active_warps);
        }
        mbar_init(merge_bar0, plan.active_warps);
        mbar_init(merge_bar0 + 8, plan.active_warps);
        *abort_word = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    grid_launch_dependents();

    const int items_per_seq = plan.n_hgroups * a.max_chunks;
    const int total_items = a.batch * items_per_seq;
    const int nstages = plan.nstages;

    if (warp == kProducerWarp) {
        // ------------------------------ loader ------------------------------
        int stage = 0;
        uint32_t empty_parity = 0;      // bit s: parity to wait for on empty[s]
        int filled = 0;                 // stages handed out so far
        bool dep_done = false;
        bool alive = true;
        int item = blockIdx.x;
        auto acquire = [&]() -> bool {
            if (filled >= nstages) {
                if (!mbar_wait_bounded(empty0 + 8 * stage, (empty_parity >> stage) & 1u, abort_word)) {
                    if (lane == 0) { if (*abort_word == 0) atomicCAS(a.status, 0, kStatusEmptyTimeout); *abort_word = 1; }
                    return false;
                }
                empty_parity ^= (1u << stage);
            }
            return true;
        };
        auto publish_header_only = [&](int b, int hgi, int c, int flags) {
            if (lane == 0) {
                TileHeader h; h.b = b; h.hgroup = hgi; h.c = c; h.blk0 = 0; h.nvalid = 0; h.flags = flags; h.pos0 = 0; h.pad = 0;
                headers[stage] = h;
                mbar_arrive(full0 + 8 * stage);
            }
            __syncwarp();
            ++filled;
            stage = (stage + 1 == nstages) ? 0 : stage + 1;
        };
        while (alive && item < total_items) {
            const int rank = item / items_per_seq;
            const int rem = item - rank * items_per_seq;
            const int hgi = rem / a.max_chunks, c = rem - hgi * a.max_chunks;
            const int b = a.seq_order ? a.seq_order[rank] : rank;
            const int total = a.kv_offsets[b] + 1;
            const int chunk = split_chunk_len(total, a.max_chunks, SPLIT_KV_CHUNK_SIZE, a.min_chunk);
            const long long start_ll = (long long)c * chunk;
            if (start_ll >= total) {
                if (!acquire()) { alive = false; break; }
                publish_header_only(b, hgi, c, kTileFirst | kTileLast | kTileEmpty);
            } else {
                const int start = (int)start_ll;
                const int end = min(start + chunk, total);
                const unsigned char* kseq = reinterpret_cast<const unsigned char*>(a.k_cache) +
                    2ll * ((long long)b * a.kv_batch_stride + (long long)hgi * plan.hg * D);
                const unsigned char* vseq = reinterpret_cast<const unsigned char*>(a.v_cache) +
                    2ll * ((long long)b * a.kv_batch_stride + (long long)hgi * plan.hg * D);
                const long long pos_stride = 2ll * a.num_kv_heads * D;
                for (int pos0 = start; pos0 < end; pos0 += plan.tile) {
                    if (!acquire()) { alive = false; break; }
                    const int nvalid = min(plan.tile, end - pos0);
                    const int nrows = vteb_round_up(nvalid, kBlockPos);
                    // The newest cache row may be written by the kernel launched just
                    // before this one: wait for it before touching the final position.
                    if (!dep_done && pos0 + nvalid >= total) { grid_dependency_wait(); dep_done = true; }
                    const uint32_t bar = full0 + 8 * stage;
                    if (lane == 0) {
                        TileHeader h; h.b = b; h.hgroup = hgi; h.c = c; h.blk0 = (pos0 - start) / kBlockPos;
                        h.nvalid = nvalid; h.pos0 = pos0; h.pad = 0;
                        h.flags = (pos0 == start ? kTileFirst : 0) | (pos0 + plan.tile >= end ? kTileLast : 0);
                        headers[stage] = h;
                        mbar_arrive_expect_tx(bar, 2u * nrows * plan.row_bytes);
                    }
                    __syncwarp();
                    const uint32_t kdst = smem_u32(stages + (size_t)stage * plan.stage_bytes);
                    const uint32_t vdst = kdst + plan.tile * plan.row_pitch;
                    for (int r = lane; r < nrows; r += 32) {
                        const long long src_pos = min(pos0 + r, end - 1);
                        bulk_load_row(kdst + r * plan.row_pitch, kseq + src_pos * pos_stride, plan.row_bytes, bar);
                        bulk_load_row(vdst + r * plan.row_pitch, vseq + src_pos * pos_stride, plan.row_bytes, bar);
                    }
                    ++filled;
                    stage = (stage + 1 == nstages) ? 0 : stage + 1;
                }
            }
            if (!alive) break;
            // Later items come from the shared ticket, which the previous combine
            // launch reset: it may only be touched once that launch has completed.
            if (!dep_done) { grid_dependency_wait(); dep_done = true; }
            int next = 0;
            if (lane == 0) next = gridDim.x + atomicAdd(a.ticket, 1);
            item = __shfl_sync(0xffffffffu, next, 0);
        }
        if (alive && acquire()) publish_header_only(0, 0, 0, kTileStop);
        if (!dep_done) grid_dependency_wait();
        // Do not leave while copies may still be landing in this CTA's shared
        // memory: wait (bounded, 100 ms per stage) for the latest "full" phase of
        // every stage that was handed out.  Stages are used round-robin from 0.
        for (int s = 0; s < nstages; ++s) {
            const int fills = filled / nstages + (s < filled % nstages ? 1 : 0);
            if (fills > 0) mbar_wait_bounded(full0 + 8 * s, (uint32_t)(fills - 1) & 1u, nullptr, 100000000ull);
        }
        return;
    }

    if (warp >= plan.active_warps) return;

    // -------------------------------- consumers --------------------------------
    const int hh = warp % plan.hg;        // KV head within the group
    const int sub = warp / plan.hg;       // which of the wph interleaved block streams
    const int g = lane >> 2, t = lane & 3;
    const float scale2 = a.scale * kLog2e;
    constexpr int KS = D / 16;            // k-steps of the QK^T product
    constexpr int NT = D / 8;             // 8-wide output column tiles

    // Q fragments live in a per-thread column of shared memory: word i of this
    // thread is q_frag[i * 32]; a thread only ever reads what it wrote itself.
    uint32_t* q_frag = q_store + warp * (KS * 2 * 32) + lane;
    float o_acc[NT][2];
    float m_run = kNeutralM, l_run = 0.f;
    int stage = 0;
    uint32_t full_parity = 0;
    uint32_t merge_parity = 0;
    bool merge_pending = false;           // previous item's readers may still use the exchange area
    bool q_ready = false;

    // Lane-constant parts of the ldmatrix addresses.
    const int k_row = (lane & 7) + ((lane >> 4) << 3);
    const int k_col = ((lane >> 3) & 1) * 8;
    const int v_row = (lane & 7) + (((lane >> 3) & 1) << 3);
    const int v_col = (lane >> 4) * 8;

    for (;;) {
        if (!mbar_wait_bounded(full0 + 8 * stage, (full_parity >> stage) & 1u, abort_word)) {
            if (lane == 0) { if (*abort_word == 0) atomicCAS(a.status, 0, kStatusFullTimeout); *abort_word = 1; }
            return;
        }
        full_parity ^= (1u << stage);
        const TileHeader hd = headers[stage];
        if (hd.flags & kTileStop) break;

        if (hd.flags & kTileFirst) {
            m_run = kNeutralM; l_run = 0.f;
#pragma unroll
            for (int n = 0; n < NT; ++n) { o_acc[n][0] = 0.f; o_acc[n][1] = 0.f; }
            if (!q_ready) { grid_dependency_wait(); q_ready = true; }
            // Row g of the A operand is query head (kv_head * group + g); rows >= group are zero.
            const int kv_head = hd.hgroup * plan.hg + hh;
            const uint32_t* qrow = reinterpret_cast<const uint32_t*>(
                a.q + ((long long)hd.b * a.num_q_heads + (long long)kv_head * group + g) * D);
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                q_frag[(2 * ks) * 32] = (g < group) ? qrow[ks * 8 + t] : 0u;
                q_frag[(2 * ks + 1) * 32] = (g < group) ? qrow[ks * 8 + 4 + t] : 0u;
            }
        }

        if (!(hd.flags & kTileEmpty)) {
            const uint32_t kt = smem_u32(stages + (size_t)stage * plan.stage_bytes) + hh * D * 2;
            const uint32_t vt = kt + plan.tile * plan.row_pitch;
            const int nblk = (hd.nvalid + kBlockPos - 1) / kBlockPos;
            for (int blk = 0; blk < nblk; ++blk) {
                if ((hd.blk0 + blk) % plan.wph != sub) continue;
                const int r0 = blk * kBlockPos;
                // ---- S = Q K^T for 16 positions: s[0] positions 0..7, s[1] positions 8..15
                float s[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
                const uint32_t kaddr = kt + (r0 + k_row) * plan.row_pitch + k_col * 2;
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4(kaddr + ks * 32, b0, b1, b2, b3);
                    const uint32_t qa0 = q_frag[(2 * ks) * 32], qa1 = q_frag[(2 * ks + 1) * 32];
                    mma_rows0to7(s[0][0], s[0][1], qa0, qa1, b0, b1);
                    mma_rows0to7(s[1][0], s[1][1], qa0, qa1, b2, b3);
                }
                // ---- online softmax (log2 domain); positions past the item's end are masked
                const int left = hd.nvalid - r0;        // valid positions in this block (may exceed 16)
                float mx = kNeutralM;
#pragma unroll
                for (int n = 0; n < 2; ++n)
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const bool valid = (n * 8 + 2 * t + j) < left;
                        s[n][j] = valid ? s[n][j] * scale2 : kNeutralM;
                        mx = fmaxf(mx, s[n][j]);
                    }
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m_run, mx);
                const float corr = fast_exp2(m_run - m_new);
                if (__any_sync(0xffffffffu, corr != 1.f)) {
                    l_run *= corr;
#pragma unroll
                    for (int n = 0; n < NT; ++n) { o_acc[n][0] *= corr; o_acc[n][1] *= corr; }
                }
                m_run = m_new;
                float p[2][2];
#pragma unroll
                for (int n = 0; n < 2; ++n)
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        const bool valid = (n * 8 + 2 * t + j) < left;
                        p[n][j] = valid ? fast_exp2(s[n][j] - m_new) : 0.f;
                    }
                l_run += (p[0][0] + p[0][1]) + (p[1][0] + p[1][1]);
                // P = P_hi + P_lo, both fp16: keeps ~22 bits of each probability.
                uint32_t ph[2], pl[2];
#pragma unroll
                for (int n = 0; n < 2; ++n) {
                    const __half2 hi = __floats2half2_rn(p[n][0], p[n][1]);
                    const float2 hif = __half22float2(hi);
                    ph[n] = *reinterpret_cast<const uint32_t*>(&hi);
                    pl[n] = pack_half2(p[n][0] - hif.x, p[n][1] - hif.y);
                }
                // ---- O += P V
                const uint32_t vaddr = vt + (r0 + v_row) * plan.row_pitch + v_col * 2;
#pragma unroll
                for (int np = 0; np < NT / 2; ++np) {
                    uint32_t v0, v1, v2, v3;
                    ldmatrix_x4_trans(vaddr + np * 32, v0, v1, v2, v3);
                    mma_rows0to7(o_acc[2 * np][0], o_acc[2 * np][1], ph[0], ph[1], v0, v1);
                    mma_rows0to7(o_acc[2 * np + 1][0], o_acc[2 * np + 1][1], ph[0], ph[1], v2, v3);
                    mma_rows0to7(o_acc[2 * np][0], o_acc[2 * np][1], pl[0], pl[1], v0, v1);
                    mma_rows0to7(o_acc[2 * np + 1][0], o_acc[2 * np + 1][1], pl[0], pl[1], v2, v3);
                }
            }
        }

        // Hand the stage back to the loader.
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * stage);
        stage = (stage + 1 == nstages) ? 0 : stage + 1;

        if (hd.flags & kTileLast) {
            // ---- exchange (m, l, o) between the warps of each KV head and store the item
            const int pitch = D + kMergePad;           // floats per (warp, row): o[D], 4 unused, m, l, 2 unused
            if (merge_pending) {
                // everyone must have finished reading the previous item's exchange area
                if (!mbar_wait_bounded(merge_bar0 + 8, (merge_parity >> 1) & 1u, abort_word)) {
                    if (lane == 0) { if (*abort_word == 0) atomicCAS(a.status, 0, kStatusMergeTimeout); *abort_word = 1; }
                    return;
                }
                merge_parity ^= 2u;
            }
            float l_quad = l_run;
            l_quad += __shfl_xor_sync(0xffffffffu, l_quad, 1);
            l_quad += __shfl_xor_sync(0xffffffffu, l_quad, 2);
            if (g < group) {
                float* dst = merge + ((size_t)warp * group + g) * pitch;
#pragma unroll
                for (int n = 0; n < NT; ++n)
                    *reinterpret_cast<float2*>(dst + n * 8 + 2 * t) = make_float2(o_acc[n][0], o_acc[n][1]);
                if (t == 0) { dst[D + 4] = m_run; dst[D + 5] = l_quad; }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(merge_bar0);
            if (!mbar_wait_bounded(merge_bar0, merge_parity & 1u, abort_word)) {
                if (lane == 0) { if (*abort_word == 0) atomicCAS(a.status, 0, kStatusMergeTimeout); *abort_word = 1; }
                return;
            }
            merge_parity ^= 1u;

            const bool empty = (hd.flags & kTileEmpty) != 0;
            const int nthreads = plan.active_warps * 32;
            const int heads_item = plan.hg * group;                    // query heads of this item
            const int q_head0 = hd.hgroup * heads_item;
            const long long stat0 = ((long long)hd.b * a.num_q_heads + q_head0) * a.max_chunks + hd.c;
            if (!empty || (a.flags & kFlagWriteEmptyO)) {
                for (int idx = threadIdx.x; idx < heads_item * (D / 4); idx += nthreads) {
                    const int hq = idx / (D / 4), d4 = idx - hq * (D / 4);
                    const int kvh = hq / group, row = hq - kvh * group;
                    float mm = kNeutralM;
                    for (int w = 0; w < plan.wph; ++w)
                        mm = fmaxf(mm, merge[((size_t)(w * plan.hg + kvh) * group + row) * pitch + D + 4]);
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int w = 0; w < plan.wph; ++w) {
                        const float* src = merge + ((size_t)(w * plan.hg + kvh) * group + row) * pitch;
                        const float wt = fast_exp2(src[D + 4] - mm);
                        const float4 x = *reinterpret_cast<const float4*>(src + d4 * 4);
                        acc.x = fmaf(x.x, wt, acc.x); acc.y = fmaf(x.y, wt, acc.y);
                        acc.z = fmaf(x.z, wt, acc.z); acc.w = fmaf(x.w, wt, acc.w);
                    }
                    float* out = a.partial_o + (stat0 + (long long)hq * a.max_chunks) * D + d4 * 4;
                    *reinterpret_cast<float4*>(out) = acc;
                }
            }
            for (int hq = threadIdx.x; hq < heads_item; hq += nthreads) {
                const int kvh = hq / group, row = hq - kvh * group;
                float mm = kNeutralM, ll = 0.f;
                for (int w = 0; w < plan.wph; ++w)
                    mm = fmaxf(mm, merge[((size_t)(w * plan.hg + kvh) * group + row) * pitch + D + 4]);
                for (int w = 0; w < plan.wph; ++w) {
                    const float* src = merge + ((size_t)(w * plan.hg + kvh) * group + row) * pitch;
                    ll += src[D + 5] * fast_exp2(src[D + 4] - mm);
                }
                a.partial_m[stat0 + (long long)hq * a.max_chunks] = empty ? kNeutralM : mm * kLn2;
                a.partial_l[stat0 + (long long)hq * a.max_chunks] = empty ? 0.f : ll;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(merge_bar0 + 8);
            merge_pending = true;
        }
    }
}

#define VTEB_FAST_PARTIAL(NAME, DIM)                                                                  \
    extern "C" __global__ void __launch_bounds__(kFastThreads, 1) NAME(                               \
        const __half* __restrict__ q, const __half* __restrict__ k_cache,                             \
        const __half* __restrict__ v_cache, float* __restrict__ partial_m,                            \
        float* __restrict__ partial_l, float* __restrict__ partial_o, int num_q_heads,                \
        int num_kv_heads, int head_dim, float scale, const int* __restrict__ kv_cache_offset_ptr,     \
        int kv_batch_stride, int max_chunks, int batch, int min_chunk, int flags,                     \
        const int* __restrict__ seq_order, int* __restrict__ ticket, int* __restrict__ status)        \
    {                                                                                                 \
        FastArgs a;                                                                                   \
        a.q = q; a.k_cache = k_cache; a.v_cache = v_cache;                                            \
        a.partial_m = partial_m; a.partial_l = partial_l; a.partial_o = partial_o;                    \
        a.num_q_heads = num_q_heads; a.num_kv_heads = num_kv_heads; a.scale = scale;                  \
        a.kv_offsets = kv_cache_offset_ptr; a.kv_batch_stride = kv_batch_stride;                      \
        a.max_chunks = max_chunks; a.batch = batch; a.min_chunk = min_chunk; a.flags = flags;         \
        a.seq_order = seq_order; a.ticket = ticket; a.status = status;                                \
        (void)head_dim;                                                                               \
        fast_partial_body<DIM>(a);                                                                    \
    }

VTEB_FAST_PARTIAL(vteb_split_kv_partial_d64_kernel, 64)
VTEB_FAST_PARTIAL(vteb_split_kv_partial_d128_kernel, 128)
VTEB_FAST_PARTIAL(vteb_split_kv_partial_d256_kernel, 256)
