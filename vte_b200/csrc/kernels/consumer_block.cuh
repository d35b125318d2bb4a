// The arithmetic of one 16-position block of the split kernel's consumer warps:
// S = Q K^T (mma.sync m16n8k16, K fragments via ldmatrix), online softmax in the log2 domain on
// the accumulator fragment, O += P V (V fragments via ldmatrix.trans) with P carried as an fp16
// high part in rows 0..7 of the A operand and an fp16 low part in rows 8..15.
//
// Replaces the per-position loop of
// vte/compiler/templates/rdna/flash_attention_split_kv_partial.hip.template:92-113
// (one position per iteration, one shared-memory tree reduction per position).
//
// Tile layout expected in shared memory: see split_kv_fast.cuh (128-byte column blocks,
// 128-byte swizzle).  `kaddr` / `vaddr` are the lane's ldmatrix base addresses for the block.
#pragma once

#include "vteb_common.cuh"

namespace vteb {

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
    __device__ __forceinline__ void reset() {
        m = kNeutralM; l = 0.f;
#pragma unroll
        for (int n = 0; n < NT; ++n) { o[n][0] = 0.f; o[n][1] = 0.f; }
        if constexpr (LOACC) {
#pragma unroll
            for (int n = 0; n < NT; ++n) { o_lo[n][0] = 0.f; o_lo[n][1] = 0.f; }
        }
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

}  // namespace vteb
