// Shared device helpers for the sm_100a decode-attention kernels: mbarrier and
// bulk-copy wrappers with bounded waits, ldmatrix / mma.sync wrappers, and the
// shared-memory plan that host and device code both derive from the head
// geometry.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace vteb {

// Two shapes of the split kernel's CTA, both one CTA per SM with the whole shared memory
// as K/V stages and two loader warps (K rows / V rows):
//   full:    8 consumer warps, for work that keeps an SM busy for tens of microseconds;
//   compact: 6 consumer warps, at most 160 registers.  Ten warps of 168 registers fill two of
//            the SM's four register-file partitions, so no CTA of the combine kernel launched
//            behind can become resident until a split CTA leaves, and the launch after that
//            cannot even start until every combine CTA has.  Eight warps of 160 registers
//            (two per partition) leave 6 K registers free in every partition: the combine
//            CTAs sit at their dependency wait while the split runs and the next layer's
//            split is launched on time.  Measured at 32k context, one sequence: 10.6 us per
//            layer against 12.5 us (4 consumer warps at 168 registers: 10.9 us; 6 at 168: 11.1 us).
constexpr int kFullConsumerWarps = 8;
constexpr int kCompactConsumerWarps = 6;
constexpr int kFullThreads = (kFullConsumerWarps + 2) * 32;         // 320
constexpr int kCompactThreads = (kCompactConsumerWarps + 2) * 32;   // 256
constexpr int kMaxStages = 8;
constexpr int kBlockPos = 16;                            // positions per mma step
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kNeutralM = -1e30f;                      // reference's "empty split" maximum
#ifndef VTEB_SMEM_BUDGET_KB
#define VTEB_SMEM_BUDGET_KB 225   /* 227 KB per CTA minus the split kernel's static shared memory */
#endif
constexpr int kSmemBudget = VTEB_SMEM_BUDGET_KB * 1024;  // dynamic shared memory the split kernel may use

// Every device-side wait gives up after this many SM clock cycles (about two seconds at 2 GHz),
// records a status code and returns.  A build with a smaller value (-DVTEB_WAIT_LIMIT_CYCLES=n)
// lets a test watch a wait run out without anything hanging.
#ifndef VTEB_WAIT_LIMIT_CYCLES
#define VTEB_WAIT_LIMIT_CYCLES 4000000000
#endif
constexpr long long kWaitLimitCycles = VTEB_WAIT_LIMIT_CYCLES;

// Status word written by a kernel that gave up on a wait.  The host reads it
// after synchronising; zero means every wait completed.
constexpr int kStatusOk = 0;
constexpr int kStatusFullTimeout = 1;    // consumer never saw a tile arrive
constexpr int kStatusEmptyTimeout = 2;   // loader never got a stage back
constexpr int kStatusMergeTimeout = 3;   // cross-warp merge barrier never completed
constexpr int kStatusGridTimeout = 4;    // another CTA never reached the grid-wide barrier

// Tile flags carried in the per-stage header.
constexpr int kTileFirst = 1;   // first tile of a work item: reset state, fetch Q
constexpr int kTileLast = 2;    // last tile of a work item: merge warps, store partials
constexpr int kTileEmpty = 4;   // item has no positions: store the neutral state
constexpr int kTileStop = 8;    // no more work for this CTA

struct TileHeader {
    int b;        // sequence index
    int hgroup;   // KV-head group index
    int c;        // split index
    int blk0;     // index, within the item, of the first 16-position block of this tile
    int nvalid;   // positions of this tile that belong to the item
    int flags;
    int pos0;     // absolute position of the tile's first row
    int last_pos; // last position of the item (rows past it are filled from this one)
};

// Everything the launch geometry depends on.  Computed identically on the host
// (to size the launch) and on the device (to carve shared memory).
struct FastPlan {
    int hg;            // KV heads staged together per work item
    int n_hgroups;     // ceil(num_kv_heads / hg)
    int wph;           // consumer warps per KV head
    int active_warps;  // wph * hg
    int tile;          // positions per stage
    int row_bytes;     // bytes of one position's K (or V) row for the head group
    int blk_bytes;     // one 128-byte-wide column block of a tile: tile * 128
    int stage_bytes;   // K tile + V tile
    int merge_bytes;   // per-warp (m, l, o) exchange area
    int q_bytes;       // Q operand fragments in shared memory (keeps them out of registers)
    int consumer_warps;
    int loader_warps;
    int threads;
    int nstages;
    int smem_bytes;    // total dynamic shared memory
    int ok;            // 0 when the geometry is outside what the fast kernel covers
};

constexpr int kCtrlBytes = 1024;   // barriers, abort word, tile headers
constexpr int kStageAlign = 1024;  // stages start on a 1024-byte shared-memory address (the 128-byte swizzle repeats every 8 rows)
constexpr int kMergePad = 8;       // floats after o[D] in an exchange row: 4 unused, m, l, true maximum, 1 unused

__host__ __device__ inline int vteb_round_up(int x, int m) { return (x + m - 1) / m * m; }

// 1: 128-wide heads, and 256-wide heads in the full CTA shape, take the transposed form of the block
// arithmetic (consumer_block.cuh, second half): positions are the M dimension of both products.  A warp
// then holds all 256 output columns of a head in 64 accumulator registers, so 256-wide heads need no
// second warp per (head, block).
#ifndef VTEB_TRANSPOSED
#define VTEB_TRANSPOSED 1
#endif

__host__ __device__ inline FastPlan make_fast_plan(int num_q_heads, int num_kv_heads, int head_dim, int compact = 0) {
    FastPlan p;
    p.ok = 0;
    p.hg = p.n_hgroups = p.wph = p.active_warps = p.tile = p.row_bytes = p.blk_bytes = 0;
    p.stage_bytes = p.merge_bytes = p.q_bytes = p.nstages = p.smem_bytes = 0;
    const int cw = compact ? kCompactConsumerWarps : kFullConsumerWarps;
    p.consumer_warps = cw;
    p.loader_warps = 2;
    p.threads = (cw + p.loader_warps) * 32;
    if (num_kv_heads <= 0 || num_q_heads <= 0 || num_q_heads % num_kv_heads != 0) return p;
    int group = num_q_heads / num_kv_heads;
    if (group > 8) return p;
    if (head_dim != 64 && head_dim != 128 && head_dim != 256) return p;
    // largest divisor of num_kv_heads with hg * head_dim <= 512 halves and a consumer warp left
    // for every head; 256-wide heads go one per item: a 16-position block of such a head keeps
    // a warp for ~1,500 cycles, and four blocks in flight per head instead of two took the
    // 16-sequence ragged batch from 5.6 to 5.9 TB/s
    int cap = (head_dim == 256) ? 1 : 512 / head_dim;
    if (cap > cw) cap = cw;
    int hg = 1;
    for (int d = 1; d <= cap; ++d) if (num_kv_heads % d == 0) hg = d;
    // 256-wide heads in the untransposed form: two warps share a (head, block), each owning half of the
    // output columns (both compute the scores); halves the accumulator registers per warp.
    const int dsplit = (head_dim == 256 && (compact || !VTEB_TRANSPOSED)) ? 2 : 1;
    p.hg = hg;
    p.n_hgroups = num_kv_heads / hg;
    p.wph = cw / (hg * dsplit);
    if (p.wph < 1) return p;
    p.active_warps = p.wph * hg * dsplit;
    p.row_bytes = hg * head_dim * 2;
    // 16 KB of K (and of V) per stage; 32 KB for 1024-byte rows, whose tensor-map boxes would
    // otherwise be 2 KB each (measured on 64 ragged sequences of 8 x 64-wide heads: 6.5 against 5.7 TB/s)
    int tile = ((p.row_bytes >= 1024 ? 32768 : 16384) / p.row_bytes) / kBlockPos * kBlockPos;
    if (tile < kBlockPos) tile = kBlockPos;
    if (tile > 64) tile = 64;
    p.tile = tile;
    p.blk_bytes = tile * 128;
    p.stage_bytes = 2 * tile * p.row_bytes;
    p.merge_bytes = vteb_round_up(p.active_warps * group * (head_dim + kMergePad) * 4, 128);
    p.q_bytes = hg * (head_dim / 8) * 32 * 4;   // one fragment image per KV head, shared by its warps
    int left = kSmemBudget - kCtrlBytes - p.merge_bytes - p.q_bytes - kStageAlign;
    int n = left / p.stage_bytes;
    if (n > kMaxStages) n = kMaxStages;
    if (n < 2) return p;
    p.nstages = n;
    p.smem_bytes = kCtrlBytes + p.merge_bytes + p.q_bytes + kStageAlign + n * p.stage_bytes;
    p.ok = 1;
    return p;
}

// Positions covered by one split of a sequence with `total` cached positions.
// `fixed_chunk > 0` is the reference's compile-time chunk length; otherwise the
// chunk is ceil(total / max_chunks) rounded up to 16 and not below `min_chunk`.
__host__ __device__ inline int split_chunk_len(int total, int max_chunks, int fixed_chunk, int min_chunk) {
    if (fixed_chunk > 0) return fixed_chunk;
    int chunk = (total + max_chunks - 1) / max_chunks;
    chunk = vteb_round_up(chunk < 1 ? 1 : chunk, kBlockPos);
    if (chunk < min_chunk) chunk = vteb_round_up(min_chunk, kBlockPos);
    return chunk;
}

#if defined(__CUDACC__)

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        "  .reg .pred p;\n"
        "  mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "  selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Waits for a barrier phase for at most `limit_cycles` SM clock cycles
// (the default is about two seconds), also giving up as soon as another warp of the
// CTA has raised `*abort_word` (pass nullptr to ignore it).  Returns false when
// it gave up; the caller then records a status code and leaves.  The SM-local
// cycle counter is used because reading %globaltimer costs microseconds.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_word,
                                                  long long limit_cycles = kWaitLimitCycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t spin = 1; spin < (1u << 30); ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 0x3F) == 0) {
            if (abort_word != nullptr && *abort_word != 0) return false;
            if (clock64() - t0 > limit_cycles) return false;
        }
    }
    return false;
}

// 16 bytes global -> shared through the asynchronous copy path (L2 only, no
// register staging); the source must be 16-byte aligned.  Used for ragged tiles
// (the end of a split) and for caches a tensor map cannot describe; whole tiles
// travel as tensor-map boxes (tma_load_box_2d), which cost the loader a handful
// of instructions per tile instead of ~1,200 cycles.
__device__ __forceinline__ void async_copy_16(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}

// ---- tensor-map (TMA) tile copies -------------------------------------------
// A 128-byte tensor map as the driver encodes it (CUtensorMap); kernels take it as a
// `__grid_constant__` parameter and hand its address to the copy instruction.
struct alignas(64) KvTensorMap { unsigned long long opaque[16]; };

// Counts the calling thread's arrival on `bar` and announces `bytes` of asynchronous
// writes that will complete on it.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// One box of a 2-D tiled tensor map (x = element index inside a row, a multiple of 8 halves;
// y = row) from global to shared memory; the bytes complete on `bar`.  With a 64-half-wide
// box and the map's 128-byte swizzle the box lands in the tile layout described in
// split_kv_fast.cuh.  This CTA's own shared memory only: no cluster, no multi-CTA delivery.
__device__ __forceinline__ void tma_load_box_2d(uint32_t dst_smem, const void* tensor_map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst_smem), "l"(tensor_map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// Makes the calling thread's earlier async_copy_16 operations count as one
// arrival on the barrier once they have all landed.
__device__ __forceinline__ void async_copy_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void grid_dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void grid_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

// D(16x8, f32) += A(16x16, f16) * B(16x8, f16) where rows 8..15 of A are zero:
// only the two accumulators of row (lane / 4) are kept.
__device__ __forceinline__ void mma_rows0to7(float& d0, float& d1, uint32_t a_lo, uint32_t a_hi, uint32_t b0, uint32_t b1) {
    float u0, u1;
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%10,%11};"
        : "+f"(d0), "+f"(d1), "=f"(u0), "=f"(u1)
        : "r"(a_lo), "r"(0u), "r"(a_hi), "r"(0u), "r"(b0), "r"(b1), "f"(0.f), "f"(0.f));
}

// D(16x8) = A(16x16) * B(16x8) + C with rows 0..7 of A = (hi_lo, hi_hi) and rows
// 8..15 of A = (lo_lo, lo_hi): one instruction multiplies both fp16 halves of a
// split-precision operand by the same B.  d0, d1 accumulate the rows 0..7
// product; e0, e1 return the rows 8..15 product (started from zero).
__device__ __forceinline__ void mma_hi_lo(float& d0, float& d1, float& e0, float& e1, uint32_t hi_lo, uint32_t lo_lo,
                                          uint32_t hi_hi, uint32_t lo_hi, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%10,%11};"
        : "+f"(d0), "+f"(d1), "=f"(e0), "=f"(e1)
        : "r"(hi_lo), "r"(lo_lo), "r"(hi_hi), "r"(lo_hi), "r"(b0), "r"(b1), "f"(0.f), "f"(0.f));
}

__device__ __forceinline__ uint32_t pack_half2(float x, float y) {
    __half2 h = __floats2half2_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- rotary position embedding --------------------------------------------
// One rotated pair, as vte/compiler/templates/rdna/rope.hip.template:62-63,76-77,94-95
// writes it: y1 = x1*c - x2*s, y2 = x1*s + x2*c in fp32.  Every product is rounded on
// its own (no fused multiply-add), so the standalone kernel, the rotation fused into
// the cache append and the one fused into the split kernel's Q load give identical bits.
__device__ __forceinline__ void rope_pair(float x1, float x2, float c, float s, float& y1, float& y2) {
    y1 = __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s));
    y2 = __fadd_rn(__fmul_rn(x1, s), __fmul_rn(x2, c));
}

__device__ __forceinline__ float2 unpack_half2(uint32_t w) {
    return __half22float2(*reinterpret_cast<const __half2*>(&w));
}

// Split-half rotation of a lane's Q operand words when the rotated width is HK * 32
// channels: word q[2*ks + e] (k-step ks, e = 0/1) holds channels ks*16 + e*8 + 2t, +1 and
// pairs with the same word HK k-steps later.  `c32`/`s32` point at the position's table row.
template <int KS, int HK>
__device__ __forceinline__ void rope_rotate_words_split_half(uint32_t (&q)[KS * 2], const uint32_t* c32,
                                                             const uint32_t* s32, int t) {
#pragma unroll
    for (int ks = 0; ks < HK; ++ks) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int w = ks * 8 + e * 4 + t;
            const float2 c = unpack_half2(c32[w]), s = unpack_half2(s32[w]);
            const float2 lo = unpack_half2(q[2 * ks + e]), hi = unpack_half2(q[2 * (ks + HK) + e]);
            float a0, b0, a1, b1;
            rope_pair(lo.x, hi.x, c.x, s.x, a0, b0);
            rope_pair(lo.y, hi.y, c.y, s.y, a1, b1);
            q[2 * ks + e] = pack_half2(a0, a1);
            q[2 * (ks + HK) + e] = pack_half2(b0, b1);
        }
    }
}

// Rotates a lane's Q operand words (layout above) at position `pos`.
// rope_type 0: split-half over the head, table rows of KS*16 entries; 1: adjacent pairs,
// entry i of a KS*16-entry row for pair (2i, 2i+1); 2: split-half over the first
// `rotary_dim` channels (32, 64, 128 or 256), table rows of rotary_dim entries.
template <int KS>
__device__ __forceinline__ void rope_rotate_q_words(uint32_t (&q)[KS * 2], const __half* cos_table,
                                                    const __half* sin_table, int pos, int rope_type,
                                                    int rotary_dim, int t) {
    constexpr int D = KS * 16;
    if (rope_type < 0) return;                                      // no rotation asked for
    if (rope_type == 1) {
        const __half* c = cos_table + (long long)pos * D;
        const __half* s = sin_table + (long long)pos * D;
#pragma unroll
        for (int i = 0; i < KS * 2; ++i) {
            const int w = (i >> 1) * 8 + (i & 1) * 4 + t;          // word index = pair index
            const float2 x = unpack_half2(q[i]);
            float y0, y1;
            rope_pair(x.x, x.y, __half2float(c[w]), __half2float(s[w]), y0, y1);
            q[i] = pack_half2(y0, y1);
        }
        return;
    }
    const int rot = (rope_type == 2) ? rotary_dim : D;
    const uint32_t* c32 = reinterpret_cast<const uint32_t*>(cos_table + (long long)pos * rot);
    const uint32_t* s32 = reinterpret_cast<const uint32_t*>(sin_table + (long long)pos * rot);
    const int hk = rot >> 5;                                        // k-steps per rotated half
    if (hk == 1) rope_rotate_words_split_half<KS, 1>(q, c32, s32, t);
    if constexpr (KS >= 4) { if (hk == 2) rope_rotate_words_split_half<KS, 2>(q, c32, s32, t); }
    if constexpr (KS >= 8) { if (hk == 4) rope_rotate_words_split_half<KS, 4>(q, c32, s32, t); }
    if constexpr (KS >= 16) { if (hk == 8) rope_rotate_words_split_half<KS, 8>(q, c32, s32, t); }
}

// One channel of a rotated row: what channel `d` of the D-wide row `x` becomes.
__device__ __forceinline__ __half rope_channel(const __half* x, int d, int D, const __half* cos_table,
                                               const __half* sin_table, int pos, int rope_type, int rotary_dim) {
    float y1, y2;
    if (rope_type < 0) return x[d];                                 // no rotation asked for
    if (rope_type == 1) {
        const int i = d >> 1;
        rope_pair(__half2float(x[2 * i]), __half2float(x[2 * i + 1]),
                  __half2float(cos_table[(long long)pos * D + i]), __half2float(sin_table[(long long)pos * D + i]), y1, y2);
        return __float2half((d & 1) ? y2 : y1);
    }
    const int rot = (rope_type == 2) ? rotary_dim : D;
    if (d >= rot) return x[d];
    const int half = rot >> 1, j = (d < half) ? d : d - half;
    rope_pair(__half2float(x[j]), __half2float(x[j + half]),
              __half2float(cos_table[(long long)pos * rot + j]), __half2float(sin_table[(long long)pos * rot + j]), y1, y2);
    return __float2half((d < half) ? y1 : y2);
}

#endif  // __CUDACC__

}  // namespace vteb
