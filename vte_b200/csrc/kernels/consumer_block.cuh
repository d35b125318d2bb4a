// The arithmetic of one 16-position block of the split kernel's consumer warps, in two forms.
//
// First half of the file, query heads as the M dimension (64-wide heads; 256-wide heads in the
// compact shape): S = Q K^T (mma.sync m16n8k16, K fragments via ldmatrix), online softmax in the
// log2 domain on the accumulator fragment, O += P V (V fragments via ldmatrix.trans) with P carried
// as an fp16 high part in rows 0..7 of the A operand and an fp16 low part in rows 8..15.
// Second half, positions as the M dimension (128-wide heads; 256-wide heads in the full shape):
// S^T = K Q^T, movmatrix transposes of the P fragments, O^T += V^T P^T.
// Both keep a reference maximum per row that moves only when a score exceeds it by VTEB_LAZY_MAX.
//
// Replaces the per-position loop of
// vte/compiler/templates/rdna/flash_attention_split_kv_partial.hip.template:92-113
// (one position per iteration, one shared-memory tree reduction per position).
//
// Tile layout expected in shared memory: see split_kv_fast.cuh (128-byte column blocks,
// 128-byte swizzle).  `kaddr` / `vaddr` are the lane's ldmatrix base addresses for the block.
#pragma once

#include "vteb_common.cuh"

#ifndef VTEB_LAZY_MAX
#define VTEB_LAZY_MAX 8   // 0: the reference maximum follows every block's maximum
#endif

namespace vteb {

// Where a warp's exchange row keeps the row's true maximum: a slot of its own under the lazy
// maximum, the reference maximum's slot (D + 4) otherwise.
constexpr int kMergeTrueMax = (VTEB_LAZY_MAX > 0) ? 6 : 4;

// Scores of one block: sn[0] positions 0..7, sn[1] positions 8..15 (raw dot products, unscaled),
// thread (g = lane / 4, t = lane % 4) holds query row g, positions 2t, 2t+1 of each half.
// QKC independent accumulation chains per position half: on this part a dependent mma.sync waits
// for the previous one's full latency, so KS k-steps in one chain cost KS latencies.
template <int D, int QKC>
__device__ __forceinline__ void qk_block(const uint32_t* __restrict__ q_frag, uint32_t kaddr, int blk_bytes,
                                         float (&sn)[2][2]) {
    constexpr int KS = D / 16;
    static_assert(KS % QKC == 0, "chains must divide the k-steps");
    float s[QKC][2][2];
#pragma unroll
    for (int c = 0; c < QKC; ++c) { s[c][0][0] = s[c][0][1] = s[c][1][0] = s[c][1][1] = 0.f; }
    constexpr int KC = KS < 8 ? KS : 8;          // k-steps whose K fragments are fetched together
#pragma unroll
    for (int kc = 0; kc < KS; kc += KC) {
        uint32_t kf[KC][4];
#pragma unroll
        for (int i = 0; i < KC; ++i)
            ldmatrix_x4((kaddr ^ (((kc + i) & 3) << 5)) + ((kc + i) >> 2) * blk_bytes, kf[i][0], kf[i][1], kf[i][2], kf[i][3]);
#pragma unroll
        for (int i = 0; i < KC; ++i) {
            const int ks = kc + i;
            const uint32_t qa0 = q_frag[(2 * ks) * 32], qa1 = q_frag[(2 * ks + 1) * 32];
            mma_rows0to7(s[ks % QKC][0][0], s[ks % QKC][0][1], qa0, qa1, kf[i][0], kf[i][1]);
            mma_rows0to7(s[ks % QKC][1][0], s[ks % QKC][1][1], qa0, qa1, kf[i][2], kf[i][3]);
        }
    }
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            float acc = s[0][n][j];
#pragma unroll
            for (int c = 1; c < QKC; ++c) acc += s[c][n][j];
            sn[n][j] = acc;
        }
}

// Online-softmax state of a consumer warp for NT 8-wide output column tiles.  With LOACC the
// products of the low parts of P accumulate in registers of their own (`o_lo`) and are added once
// per item (fold_lo) instead of once per block.
template <int NT, bool LOACC>
struct ConsumerState {
    float o[NT][2];
    float o_lo[LOACC ? NT : 1][2];
    float m, l;
    float mt;   // lazy maximum only: this thread's largest score so far (m then lags behind the row's true maximum)
    __device__ __forceinline__ void reset() {
        m = kNeutralM; l = 0.f; mt = kNeutralM;
#pragma unroll
        for (int n = 0; n < NT; ++n) { o[n][0] = 0.f; o[n][1] = 0.f; }
        if constexpr (LOACC) {
#pragma unroll
            for (int n = 0; n < NT; ++n) { o_lo[n][0] = 0.f; o_lo[n][1] = 0.f; }
        }
    }
    // The row's true maximum (quad-wide); equals m unless the maximum is lazy.
    __device__ __forceinline__ float true_max() const {
#if VTEB_LAZY_MAX > 0
        float v = mt;
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
        return v;
#else
        return m;
#endif
    }
    __device__ __forceinline__ void fold_lo() {
        if constexpr (LOACC) {
#pragma unroll
            for (int n = 0; n < NT; ++n) { o[n][0] += o_lo[n][0]; o[n][1] += o_lo[n][1]; o_lo[n][0] = 0.f; o_lo[n][1] = 0.f; }
        }
    }
};

// D(16x8) += A(16x16) * B(16x8), all four accumulators kept: rows 0..7 in (d0, d1), rows 8..15 in (e0, e1).
__device__ __forceinline__ void mma_hi_lo_acc(float& d0, float& d1, float& e0, float& e1, uint32_t hi_lo, uint32_t lo_lo,
                                              uint32_t hi_hi, uint32_t lo_hi, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d0), "+f"(d1), "+f"(e0), "+f"(e1)
        : "r"(hi_lo), "r"(lo_lo), "r"(hi_hi), "r"(lo_hi), "r"(b0), "r"(b1));
}

// Online softmax (log2 domain) of a block's raw scores and O += P V.  `left` = positions of the
// block that belong to the item (may exceed 16); the rest are masked.  `scale2` = scale * log2(e).
template <int NT, bool LOACC>
__device__ __forceinline__ void softmax_pv(ConsumerState<NT, LOACC>& st, const float (&sraw)[2][2], uint32_t vaddr,
                                           int blk_bytes, int left, float scale2, int t) {
    // V fragments do not depend on the softmax: fetch the first 64 columns now
    constexpr int VC = (NT >= 8) ? 4 : NT / 2;   // ldmatrix.x4.trans per chunk (4 = 64 output columns)
    constexpr int NVC = NT / (2 * VC);           // chunks
    uint32_t vf[2][VC][4];
#pragma unroll
    for (int i = 0; i < VC; ++i) ldmatrix_x4_trans(vaddr ^ (i << 5), vf[0][i][0], vf[0][i][1], vf[0][i][2], vf[0][i][3]);
    float s[2][2];
    float mx = kNeutralM;
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const bool valid = (n * 8 + 2 * t + j) < left;
            s[n][j] = valid ? sraw[n][j] * scale2 : kNeutralM;
            mx = fmaxf(mx, s[n][j]);
        }
#if VTEB_LAZY_MAX > 0
    // The reference maximum m moves only when some score of the warp exceeds it by more than
    // VTEB_LAZY_MAX (log2 units): probabilities then reach 2^VTEB_LAZY_MAX at most, and the two
    // shuffles, the correction factor and the rescaling leave the chain of nearly every block.
    st.mt = fmaxf(st.mt, mx);
    if (__any_sync(0xffffffffu, mx > st.m + (float)VTEB_LAZY_MAX)) {
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_up = fmaxf(st.m, mx);
        const float corr = fast_exp2(st.m - m_up);
        st.l *= corr;
#pragma unroll
        for (int n = 0; n < NT; ++n) { st.o[n][0] *= corr; st.o[n][1] *= corr; }
        if constexpr (LOACC) {
#pragma unroll
            for (int n = 0; n < NT; ++n) { st.o_lo[n][0] *= corr; st.o_lo[n][1] *= corr; }
        }
        st.m = m_up;
    }
    const float m_new = st.m;
#else
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(st.m, mx);
    const float corr = fast_exp2(st.m - m_new);
    if (__any_sync(0xffffffffu, corr != 1.f)) {
        st.l *= corr;
#pragma unroll
        for (int n = 0; n < NT; ++n) { st.o[n][0] *= corr; st.o[n][1] *= corr; }
        if constexpr (LOACC) {
#pragma unroll
            for (int n = 0; n < NT; ++n) { st.o_lo[n][0] *= corr; st.o_lo[n][1] *= corr; }
        }
    }
    st.m = m_new;
#endif
    float p[2][2];
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const bool valid = (n * 8 + 2 * t + j) < left;
            p[n][j] = valid ? fast_exp2(s[n][j] - m_new) : 0.f;
        }
    st.l += (p[0][0] + p[0][1]) + (p[1][0] + p[1][1]);
    // P = P_hi + P_lo, both fp16: keeps ~22 bits of each probability.
    uint32_t ph[2], pl[2];
#pragma unroll
    for (int n = 0; n < 2; ++n) {
        const __half2 hi = __floats2half2_rn(p[n][0], p[n][1]);
        const float2 hif = __half22float2(hi);
        ph[n] = *reinterpret_cast<const uint32_t*>(&hi);
        pl[n] = pack_half2(p[n][0] - hif.x, p[n][1] - hif.y);
    }
    // O += P V, 64 columns per chunk; the next chunk's fragments load meanwhile
#pragma unroll
    for (int ch = 0; ch < NVC; ++ch) {
        if (ch + 1 < NVC) {
#pragma unroll
            for (int i = 0; i < VC; ++i)
                ldmatrix_x4_trans((vaddr ^ (i << 5)) + (ch + 1) * blk_bytes, vf[(ch + 1) & 1][i][0], vf[(ch + 1) & 1][i][1],
                                  vf[(ch + 1) & 1][i][2], vf[(ch + 1) & 1][i][3]);
        }
#pragma unroll
        for (int i = 0; i < VC; ++i) {
            const int n = 2 * (ch * VC + i);
            if constexpr (LOACC) {
                mma_hi_lo_acc(st.o[n][0], st.o[n][1], st.o_lo[n][0], st.o_lo[n][1], ph[0], pl[0], ph[1], pl[1],
                              vf[ch & 1][i][0], vf[ch & 1][i][1]);
                mma_hi_lo_acc(st.o[n + 1][0], st.o[n + 1][1], st.o_lo[n + 1][0], st.o_lo[n + 1][1], ph[0], pl[0], ph[1], pl[1],
                              vf[ch & 1][i][2], vf[ch & 1][i][3]);
            } else {
                float e0, e1, f0, f1;
                mma_hi_lo(st.o[n][0], st.o[n][1], e0, e1, ph[0], pl[0], ph[1], pl[1], vf[ch & 1][i][0], vf[ch & 1][i][1]);
                mma_hi_lo(st.o[n + 1][0], st.o[n + 1][1], f0, f1, ph[0], pl[0], ph[1], pl[1], vf[ch & 1][i][2], vf[ch & 1][i][3]);
                // rows 8..15 of A carried P_lo; their product belongs to this thread's row too
                st.o[n][0] += e0; st.o[n][1] += e1; st.o[n + 1][0] += f0; st.o[n + 1][1] += f1;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Transposed form of the same block: positions are the M dimension of both products.
//   S^T (16 positions x 8 heads) = K (A operand, all 16 rows used) * Q^T (B operand),
//   O^T (16 columns x 8 heads)  += V^T (A operand) * P^T (B operand, fp16 high part, then low part).
// Against the form above: 8 + 16 instead of 16 + 16 mma.sync per block, no additions of a
// low-part product, and four movmatrix transposes that turn the S^T accumulator fragment into
// the B fragments of P^T.  The ldmatrix loads are the same ones, taken in another register order.
// Thread (g = lane / 4, t = lane % 4) holds heads 2t and 2t+1: scores of positions g and g+8,
// output columns 16*mt + g and + 8 of every 16-column tile mt.

__device__ __forceinline__ void mma_full(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 8x8 transpose of 16-bit elements across the warp: lane (g, t) gives row g, columns 2t, 2t+1
// and receives row g, columns 2t, 2t+1 of the transposed matrix.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
    uint32_t y;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}

template <int MT>
struct ConsumerStateT {
    float o[MT][4];       // tile mt: (column 16mt+g, head 2t), (same, head 2t+1), (column 16mt+g+8, head 2t), (same, head 2t+1)
    float m[2], l[2];     // reference maximum (log2 domain) and this thread's part of the sum, heads 2t and 2t+1
    float mt[2];          // this thread's largest score per head (lazy maximum only)
    __device__ __forceinline__ void reset() {
        m[0] = m[1] = kNeutralM; l[0] = l[1] = 0.f; mt[0] = mt[1] = kNeutralM;
#pragma unroll
        for (int i = 0; i < MT; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    }
};

// Maximum / sum over the eight lanes that share t (the positions of a head).
__device__ __forceinline__ float max_over_g(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
}
__device__ __forceinline__ float sum_over_g(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    v += __shfl_xor_sync(0xffffffffu, v, 8);
    return v + __shfl_xor_sync(0xffffffffu, v, 16);
}

// Raw scores of one block: s[0] (position g, head 2t), s[1] (g, 2t+1), s[2] (g+8, 2t), s[3] (g+8, 2t+1).
template <int D>
__device__ __forceinline__ void qk_block_t(const uint32_t* __restrict__ q_frag, uint32_t kaddr, int blk_bytes, float (&s)[4]) {
    constexpr int KS = D / 16;
    float acc[2][4];
#pragma unroll
    for (int c = 0; c < 2; ++c) { acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0.f; }
    constexpr int KC = KS < 8 ? KS : 8;
#pragma unroll
    for (int kc = 0; kc < KS; kc += KC) {
        uint32_t kf[KC][4];
#pragma unroll
        for (int i = 0; i < KC; ++i)
            ldmatrix_x4((kaddr ^ (((kc + i) & 3) << 5)) + ((kc + i) >> 2) * blk_bytes, kf[i][0], kf[i][1], kf[i][2], kf[i][3]);
#pragma unroll
        for (int i = 0; i < KC; ++i) {
            const int ks = kc + i;
            // kf: (positions 0-7, k 0-7), (0-7, 8-15), (8-15, 0-7), (8-15, 8-15); the A operand wants rows before columns
            mma_full(acc[ks & 1], kf[i][0], kf[i][2], kf[i][1], kf[i][3], q_frag[(2 * ks) * 32], q_frag[(2 * ks + 1) * 32]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) s[i] = acc[0][i] + acc[1][i];
}

template <int MT>
__device__ __forceinline__ void softmax_pv_t(ConsumerStateT<MT>& st, const float (&sraw)[4], uint32_t vaddr, int blk_bytes,
                                             int left, float scale2, int g) {
    constexpr int VC = (MT >= 4) ? 4 : MT;       // ldmatrix.x4.trans per chunk (4 = 64 output columns)
    constexpr int NVC = MT / VC;
    uint32_t vf[2][VC][4];
#pragma unroll
    for (int i = 0; i < VC; ++i) ldmatrix_x4_trans(vaddr ^ (i << 5), vf[0][i][0], vf[0][i][1], vf[0][i][2], vf[0][i][3]);
    const bool valid[2] = {g < left, g + 8 < left};
    float s[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) s[i] = valid[i >> 1] ? sraw[i] * scale2 : kNeutralM;
    float mx[2] = {fmaxf(s[0], s[2]), fmaxf(s[1], s[3])};
#if VTEB_LAZY_MAX > 0
    st.mt[0] = fmaxf(st.mt[0], mx[0]);
    st.mt[1] = fmaxf(st.mt[1], mx[1]);
    const bool move = __any_sync(0xffffffffu, (mx[0] > st.m[0] + (float)VTEB_LAZY_MAX) | (mx[1] > st.m[1] + (float)VTEB_LAZY_MAX));
#else
    const bool move = true;
#endif
    if (move) {
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float m_up = fmaxf(st.m[h], max_over_g(mx[h]));
            corr[h] = fast_exp2(st.m[h] - m_up);
            st.l[h] *= corr[h];
            st.m[h] = m_up;
        }
#pragma unroll
        for (int i = 0; i < MT; ++i) { st.o[i][0] *= corr[0]; st.o[i][1] *= corr[1]; st.o[i][2] *= corr[0]; st.o[i][3] *= corr[1]; }
    }
    float p[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = valid[i >> 1] ? fast_exp2(s[i] - st.m[i & 1]) : 0.f;
    st.l[0] += p[0] + p[2];
    st.l[1] += p[1] + p[3];
    // P = P_hi + P_lo, both fp16; rows of the 8x8 matrices are positions, columns heads: transpose into B fragments
    uint32_t bh[2], bl[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const __half2 hi = __floats2half2_rn(p[2 * r], p[2 * r + 1]);
        const float2 hif = __half22float2(hi);
        bh[r] = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&hi));
        bl[r] = movmatrix_trans(pack_half2(p[2 * r] - hif.x, p[2 * r + 1] - hif.y));
    }
#pragma unroll
    for (int ch = 0; ch < NVC; ++ch) {
        if (ch + 1 < NVC) {
#pragma unroll
            for (int i = 0; i < VC; ++i)
                ldmatrix_x4_trans((vaddr ^ (i << 5)) + (ch + 1) * blk_bytes, vf[(ch + 1) & 1][i][0], vf[(ch + 1) & 1][i][1],
                                  vf[(ch + 1) & 1][i][2], vf[(ch + 1) & 1][i][3]);
        }
        // vf: (positions 0-7, columns 0-7)^T, (8-15, 0-7)^T, (0-7, 8-15)^T, (8-15, 8-15)^T
#pragma unroll
        for (int i = 0; i < VC; ++i)
            mma_full(st.o[ch * VC + i], vf[ch & 1][i][0], vf[ch & 1][i][2], vf[ch & 1][i][1], vf[ch & 1][i][3], bh[0], bh[1]);
#pragma unroll
        for (int i = 0; i < VC; ++i)
            mma_full(st.o[ch * VC + i], vf[ch & 1][i][0], vf[ch & 1][i][2], vf[ch & 1][i][1], vf[ch & 1][i][3], bl[0], bl[1]);
    }
}

// Column-split variant of the transposed form: the warps of a KV head all compute the scores of every
// block of the item (the same S^T, the same maximum and sum) and each accumulates only its own run of
// 16-column output tiles [mt0, mt0 + nmt), nmt <= NMT.  No warp holds a partial sum over positions, so
// nothing has to be merged across warps at the end of an item.
// The state may have more tiles than NMT (the kernel lends the full-width state); tiles 0..NMT-1 are used.
template <int NMT, int MT>
__device__ __forceinline__ void softmax_pv_t_cols(ConsumerStateT<MT>& st, const float (&sraw)[4], uint32_t vaddr, int blk_bytes,
                                                  int left, float scale2, int g, int mt0, int nmt) {
    static_assert(NMT <= MT, "state too narrow");
    uint32_t vf[NMT][4];
#pragma unroll
    for (int i = 0; i < NMT; ++i)
        if (i < nmt) {
            const int mt = mt0 + i;
            ldmatrix_x4_trans((vaddr ^ ((mt & 3) << 5)) + (mt >> 2) * blk_bytes, vf[i][0], vf[i][1], vf[i][2], vf[i][3]);
        }
    const bool valid[2] = {g < left, g + 8 < left};
    float s[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) s[i] = valid[i >> 1] ? sraw[i] * scale2 : kNeutralM;
    float mx[2] = {fmaxf(s[0], s[2]), fmaxf(s[1], s[3])};
#if VTEB_LAZY_MAX > 0
    st.mt[0] = fmaxf(st.mt[0], mx[0]);
    st.mt[1] = fmaxf(st.mt[1], mx[1]);
    const bool move = __any_sync(0xffffffffu, (mx[0] > st.m[0] + (float)VTEB_LAZY_MAX) | (mx[1] > st.m[1] + (float)VTEB_LAZY_MAX));
#else
    const bool move = true;
#endif
    if (move) {
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float m_up = fmaxf(st.m[h], max_over_g(mx[h]));
            corr[h] = fast_exp2(st.m[h] - m_up);
            st.l[h] *= corr[h];
            st.m[h] = m_up;
        }
#pragma unroll
        for (int i = 0; i < NMT; ++i) { st.o[i][0] *= corr[0]; st.o[i][1] *= corr[1]; st.o[i][2] *= corr[0]; st.o[i][3] *= corr[1]; }
    }
    float p[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = valid[i >> 1] ? fast_exp2(s[i] - st.m[i & 1]) : 0.f;
    st.l[0] += p[0] + p[2];
    st.l[1] += p[1] + p[3];
    uint32_t bh[2], bl[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const __half2 hi = __floats2half2_rn(p[2 * r], p[2 * r + 1]);
        const float2 hif = __half22float2(hi);
        bh[r] = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&hi));
        bl[r] = movmatrix_trans(pack_half2(p[2 * r] - hif.x, p[2 * r + 1] - hif.y));
    }
#pragma unroll
    for (int i = 0; i < NMT; ++i)
        if (i < nmt) mma_full(st.o[i], vf[i][0], vf[i][2], vf[i][1], vf[i][3], bh[0], bh[1]);
#pragma unroll
    for (int i = 0; i < NMT; ++i)
        if (i < nmt) mma_full(st.o[i], vf[i][0], vf[i][2], vf[i][1], vf[i][3], bl[0], bl[1]);
}

}  // namespace vteb
