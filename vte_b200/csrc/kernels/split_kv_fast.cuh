// Fast split kernel of the decode-attention path (included by decode_attention.cu).
//
// grid (n_ctas, 1, 1) persistent, block 320 = eight consumer warps + two loader
// warps (256 = six + two in the compact shape), dynamic shared memory from
// make_fast_plan().  A work item is a range of positions of one sequence for one group of `hg`
// KV heads, stored as one split of that (sequence, head group).  Two ways to hand them out:
//   work queue: item t is (sequence rank t / (n_hgroups * C), head group, split) with equal
//     splits; CTA i starts with item i and draws the following ones from `*ticket`
//     (gridDim.x + atomicAdd);
//   balanced partition (kFlagBalanced, full shape): every CTA takes an equal share of all
//     cached positions and its items are the pieces of sequences inside it (BalancedShare below).
//
// Loader warp K (the first warp after the consumers): for every tile of `tile` positions it
// waits for a free stage, writes the tile header, and fetches the K rows (row_bytes contiguous
// bytes covering the group's heads): a whole tile as tensor-map box copies (one box of `tile`
// rows x 64 halves per 128-byte column block; issued by as many lanes at once in the full
// shape, by one lane in turn in the compact shape), a ragged tile with 16-byte
// asynchronous copies, one 512-byte piece per warp instruction; both write the
// 128-byte-swizzled tile layout.  Loader warp V (the next warp) follows the headers and
// fetches the V rows.  Completion is counted on the stage's "full" mbarrier (transaction
// bytes for the boxes, deferred arrivals for the 16-byte copies).  Rows past the end of the
// item are filled from the item's last row so that every row a consumer touches holds finite
// numbers.
//
// Consumer warp w: KV head (w % hg) of the group, every wph-th 16-position
// block.  Per block (consumer_block.cuh, which has both forms): Q K^T and P V with mma.sync
// m16n8k16, K fragments via ldmatrix, V fragments via ldmatrix.trans, online softmax in the
// log2 domain on the accumulator fragment with a reference maximum that moves only when a
// score exceeds it by VTEB_LAZY_MAX, P split into an fp16 high and low part.  128-wide heads
// (and 256-wide heads in the full shape) take the transposed form, positions as the M
// dimension of both products; the others the form with the query heads as M and the two
// parts of P in rows 0..7 and 8..15 of one A operand.  At the end of an item the
// warps of a KV head exchange (m, l, o) and the row's true maximum through shared memory and
// the merged state is stored to partial_m / partial_l / partial_o.
//
// Under programmatic dependent launch everything that does not depend on the previous launch runs
// before griddepcontrol.wait: barrier set-up, the first item's geometry (kv offsets, sequence order),
// the K/V tiles of positions older than the newest one, and an L2 prefetch of the first item's Q rows.
//
// The rotating variants (`..._rope_...`) rotate Q while loading it and, when handed this step's K
// and V projections, also do the cache append: the loader warps of the CTA whose tile ends with a
// sequence's newest position write that row into the cache and into the tile.
//
// Every wait is bounded; a wait that gives up stores a code in `*status`,
// raises the CTA's abort word, and the CTA's warps return (the loader warps
// first wait for their own outstanding copies).
#pragma once

#ifndef VTEB_QK_CHAINS
#define VTEB_QK_CHAINS 2         // independent accumulation chains of the Q K^T product per position half
#endif
#ifndef VTEB_PV_LO_ACC
#define VTEB_PV_LO_ACC 0         // 1: the low parts of P accumulate in registers of their own
#endif
// (KV head, query row) pairs a warp merges per pass at the end of an item, for heads up to 128 wide
// (256-wide heads always take one): 2 = one pair per half-warp.  Measured with 12 query heads on six
// warps (one pass instead of two): the 32k-context layer 10.13 against 10.40 us, its split kernel alone
// 9.34 against 9.80 us per launch.
#ifndef VTEB_TMA_LANES
#define VTEB_TMA_LANES 1   // 1: full shape, the boxes of a tile are issued by as many lanes at once; 0: by one lane in turn
#endif
#ifndef VTEB_MERGE_PAIRS
#define VTEB_MERGE_PAIRS 2
#endif
constexpr int kQkChains = VTEB_QK_CHAINS;
constexpr bool kLoAcc = VTEB_PV_LO_ACC != 0;

struct FastArgs {
    const __half* q; const __half* k_cache; const __half* v_cache;
    float* partial_m; float* partial_l; float* partial_o;
    int num_q_heads, num_kv_heads; float scale;
    const int* kv_offsets; long long kv_batch_stride; int max_chunks;
    int batch, min_chunk, flags; const int* seq_order; int* ticket; int* status;
    const __half* next_k_cache; const __half* next_v_cache;   // optional: the next layer's caches, for L2 prefetch
    void* output; int out_kind;   // out_kind != 0: combine inside this launch (1 fp16, 2 fp32, 3 shard state)
    // rotary tables for the kernels that rotate Q while loading it (null otherwise)
    const __half* rope_cos; const __half* rope_sin; int rope_type, rotary_dim;
    // tensor maps over the K and V caches (rows = positions of all sequences, 64-half boxes of
    // `tile` rows, 128-byte swizzle); used for whole tiles when kFlagTensorMaps is set
    const KvTensorMap* tmap_k; const KvTensorMap* tmap_v;
    // fused append (rotating kernels only): this step's K and V projections [B, Hkv, D], 16-byte aligned
    // (the masked rows of the sequence's last tile are filled from them with 16-byte asynchronous copies);
    // the CTA whose tile holds a sequence's newest position writes the row into the cache and into its tile
    const __half* k_new; const __half* v_new;
};

constexpr int kFlagWriteEmptyO = 1;   // also zero partial_o of empty splits (reference semantics)
constexpr int kFlagDirectOutput = 2;  // max_chunks == 1: normalise and store the attention output here, no partials
constexpr int kFlagTensorMaps = 4;    // tmap_k / tmap_v are valid: whole tiles are fetched with tensor-map copies
constexpr int kFlagBalanced = 16;     // several sequences: every CTA takes an equal share of all cached positions (see BalancedShare), no work queue
constexpr int kFlagPrefetchQ = 8;     // ask L2 for an item's Q rows ahead of their use (the first item's before the dependency wait); a hint, no data is read

// ---- optional timeline trace (compiled in with -DVTEB_TRACE=1, used by vte_b200/trace_timeline.py) ----
// The status word's allocation is then a trace buffer: 64-bit words from byte 256 on,
// [launch 0..63][traced CTA 0..2][warp 0..9][32 stamps]; per-CTA launch counters sit at byte 64.
// Lane 0 of every warp of three CTAs (first, middle, last but two) stamps the SM cycle counter at fixed
// points, plus %globaltimer at entry and exit so that CTAs and launches can be laid on one axis.
#ifdef VTEB_TRACE
struct TraceCtx { unsigned long long* base; };
__device__ __forceinline__ unsigned long long trace_globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define VTEB_TR(ctx, slot) do { if ((ctx).base != nullptr && (threadIdx.x & 31) == 0) (ctx).base[slot] = (unsigned long long)clock64(); } while (0)
#define VTEB_TR_GT(ctx, slot) do { if ((ctx).base != nullptr && (threadIdx.x & 31) == 0) (ctx).base[slot] = trace_globaltimer(); } while (0)
#else
#define VTEB_TR(ctx, slot) do { } while (0)
#define VTEB_TR_GT(ctx, slot) do { } while (0)
#endif

// Stores four (or two) normalised output values; out_kind 1 = fp16, 2 = fp32.
__device__ __forceinline__ void store_out4(void* output, int out_kind, long long idx, float4 v) {
    if (out_kind == 2) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(output) + idx) = v;
    } else {
        __half2* o = reinterpret_cast<__half2*>(reinterpret_cast<__half*>(output) + idx);
        o[0] = __floats2half2_rn(v.x, v.y);
        o[1] = __floats2half2_rn(v.z, v.w);
    }
}
__device__ __forceinline__ void store_out2(void* output, int out_kind, long long idx, float2 v) {
    if (out_kind == 2) *reinterpret_cast<float2*>(reinterpret_cast<float*>(output) + idx) = v;
    else *reinterpret_cast<__half2*>(reinterpret_cast<__half*>(output) + idx) = __floats2half2_rn(v.x, v.y);
}

// Shared-memory control block (first kCtrlBytes of dynamic shared memory).
constexpr int kBarFull = 0;                        // 8 barriers
constexpr int kBarEmpty = 8 * kMaxStages;          // 8 barriers
constexpr int kBarHeader = 16 * kMaxStages;        // 8 barriers: header published (K loader -> V loader)
constexpr int kBarMerge = 24 * kMaxStages;         // 2 barriers
constexpr int kBarFinal = 24 * kMaxStages + 16;    // 2 barriers: CTA's partials stored / grid barrier passed
constexpr int kGridOkOffset = 260;                 // int: result of the grid barrier
constexpr int kAbortOffset = 256;
constexpr int kHeaderOffset = 512;

__device__ __forceinline__ void raise_abort(volatile int* abort_word, int* status, int code) {
    if ((threadIdx.x & 31) == 0) {
        if (*abort_word == 0) atomicCAS(status, 0, code);
        *abort_word = 1;
    }
}

// Shared-memory layout of a K (or V) tile: column blocks of 128 bytes (64 halves).  Block cb
// starts at cb * blk_bytes (blk_bytes = tile * 128); inside it position row r is at r * 128 and
// its 16-byte chunk c sits at ((c ^ (r & 7)) << 4).  This is the 128-byte swizzle a tensor-map
// copy with a 128-byte-wide box produces, and it keeps the eight row addresses of an ldmatrix
// on distinct banks without padding.  Tiles start on 1024-byte shared addresses.
//
// Copies `nrows` (a multiple of 16) position rows of `row_bytes` <= 1024 bytes each from
// global into that layout with 16-byte asynchronous copies; rows at or past `nvalid`
// are taken from `src_last` (the item's last row).  A warp instruction moves 512 bytes:
// one piece of a long row, or several whole short rows (256-byte rows: two per
// instruction).  Eight instructions' addresses are formed first and their copies issued
// back to back: an asynchronous copy holds its address registers until the load/store
// unit has picked it up, so a loop that bumps one pointer per copy stalls for that
// latency on every row (measured: ~230 cycles per row instead of ~16).
__device__ __forceinline__ void copy_rows_async(const unsigned char* src, const unsigned char* src_last,
                                                uint32_t dst, int nrows, int nvalid, int row_bytes,
                                                int blk_bytes, long long pos_stride, int lane) {
    if (row_bytes >= 512) {
        const bool piece0 = lane * 16 < row_bytes;                    // bytes [0, 512) of the row
        const bool piece1 = 512 + lane * 16 < row_bytes;              // bytes [512, 1024)
        src += lane * 16; src_last += lane * 16;
        dst += (lane >> 3) * blk_bytes;                               // this lane's column block
        const uint32_t chunk = (lane & 7) << 4;
        for (int r0 = 0; r0 < nrows; r0 += 8) {                       // r0 & 7 == 0: row i of the group has r & 7 == i
            const unsigned char* s[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) s[i] = (r0 + i < nvalid) ? src + (long long)i * pos_stride : src_last;
            if (piece0) {
#pragma unroll
                for (int i = 0; i < 8; ++i) async_copy_16(dst + i * 128 + (chunk ^ (i << 4)), s[i]);
            }
            if (piece1) {
#pragma unroll
                for (int i = 0; i < 8; ++i) async_copy_16(dst + 4 * blk_bytes + i * 128 + (chunk ^ (i << 4)), s[i] + 512);
            }
            src += 8 * pos_stride;
            dst += 8 * 128;
        }
    } else {
        const int lanes_per_row = row_bytes >> 4;                     // 16 for 256-byte rows, 8 for 128
        const int rows_per_instr = 32 / lanes_per_row;
        const int my_row = lane / lanes_per_row, my_chunk = lane - my_row * lanes_per_row;
        src += my_chunk * 16; src_last += my_chunk * 16;
        dst += (my_chunk >> 3) * blk_bytes;
        for (int r0 = 0; r0 < nrows; r0 += 8 * rows_per_instr) {
            const unsigned char* s[8];
            uint32_t d[8];
            bool on[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int r = r0 + i * rows_per_instr + my_row;
                on[i] = r < nrows && my_row < rows_per_instr;
                s[i] = (r < nvalid) ? src + (long long)r * pos_stride : src_last;
                d[i] = dst + r * 128 + (((my_chunk ^ r) & 7) << 4);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) if (on[i]) async_copy_16(d[i], s[i]);
        }
    }
}

// When a CTA owns exactly one item (one sequence, splits <= CTAs) and the
// dispatcher passed the next layer's cache, a loader warp that has issued its last
// copy asks L2 to fetch the byte range the same CTA will stream in the next
// layer's launch.  HBM then stays busy while this launch drains its tail and the
// combine runs, and the next launch starts from L2.  Every byte is still read
// from HBM once per step.  Requests are 8 KB each, spread over the lanes.
// Its place matters: issued right after the loader's last tile and its (fruitless) ticket
// draw it is worth 0.35 us per 32k-context layer (1.2 us per launch when split launches run back to
// back); issued one atomic round trip earlier it is worth 0.07 us less, and held back until the
// consumers have released the last tile it costs 1.2 us.
// The prefetch only pays while a whole layer's K and V stay in L2 until the next launch reads
// them: above this many bytes per tensor (the grid's total) it is skipped.  Measured at one
// million positions (0.5 GB per tensor): prefetching cost 15 % of the throughput.
constexpr long long kL2PrefetchMaxBytes = 24ll << 20;

__device__ __forceinline__ void prefetch_range_l2(const unsigned char* base, long long bytes, int lane) {
    constexpr long long kPiece = 8192;
    for (long long off = (long long)lane * kPiece; off < bytes; off += 32 * kPiece) {
        const unsigned n = (unsigned)((bytes - off < kPiece) ? (bytes - off) : kPiece) & ~15u;
        if (n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + off), "r"(n) : "memory");
    }
}

// Grid-wide barrier for a grid whose CTAs are all resident (grid <= SM count, one CTA
// per SM).  words[0] counts arrivals and is cleared by the last arriver, words[1] is a
// generation number; one thread per CTA calls this.  The wait is bounded (kWaitLimitCycles).
__device__ __forceinline__ bool grid_barrier_bounded(int* words, int n_ctas) {
    volatile int* gen = words + 1;
    const int my_gen = *gen;
    __threadfence();
    const int old = atomicAdd(words, 1);
    if (old == n_ctas - 1) {
        words[0] = 0;
        __threadfence();
        atomicAdd(words + 1, 1);
        return true;
    }
    const long long t0 = clock64();
    while (*gen == my_gen) {
        if (clock64() - t0 > kWaitLimitCycles) return false;
    }
    __threadfence();
    return true;
}

struct ItemGeometry {
    int b, hgroup, c, start, end;   // end <= start: empty item
};

__device__ __forceinline__ ItemGeometry decode_item(const FastArgs& a, const FastPlan& plan, int item) {
    ItemGeometry g;
    const int items_per_seq = plan.n_hgroups * a.max_chunks;
    const int rank = item / items_per_seq;
    const int rem = item - rank * items_per_seq;
    g.hgroup = rem / a.max_chunks;
    g.c = rem - g.hgroup * a.max_chunks;
    g.b = a.seq_order ? a.seq_order[rank] : rank;
    const int total = a.kv_offsets[g.b] + 1;
    const int chunk = split_chunk_len(total, a.max_chunks, SPLIT_KV_CHUNK_SIZE, a.min_chunk);
    const long long start = (long long)g.c * chunk;
    if (start >= total) { g.start = total; g.end = total; }
    else { g.start = (int)start; g.end = min(g.start + chunk, total); }
    return g;
}

// ---- balanced partition ---------------------------------------------------------------------
// Several sequences on one GPU (kFlagBalanced): the cached positions of all (sequence, head group)
// pairs, laid end to end in the order pair = sequence * n_hgroups + head group, are cut into
// gridDim.x equal shares, one per CTA; a CTA's work items are the pieces of pairs inside its share.
// Every CTA streams the same number of bytes, nothing is drawn from a queue, and the only cost of a
// ragged batch is one more merge wherever a share crosses the end of a pair.  Piece k of a pair (in
// position order) is the pair's split k; the pair's remaining splits are marked empty (the rows are
// dealt to the CTAs in equal runs).  `per` is raised where needed so that no pair is cut into more than
// max_chunks pieces (CTAs at the end of the grid then stay idle).
struct BalancedShare {
    long long total;   // positions of all pairs
    int per;           // positions per CTA, a multiple of the tile
};

__device__ __forceinline__ BalancedShare balanced_share(const FastArgs& a, const FastPlan& plan, int lane) {
    long long sum = 0;
    int longest = 0;
    for (int b0 = 0; b0 < a.batch; b0 += 32) {
        const int s = (b0 + lane < a.batch) ? a.kv_offsets[b0 + lane] + 1 : 0;
        sum += s;
        longest = max(longest, s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
        longest = max(longest, __shfl_xor_sync(0xffffffffu, longest, o));
    }
    BalancedShare bs;
    bs.total = sum * plan.n_hgroups;
    long long per = (bs.total + gridDim.x - 1) / gridDim.x;
    const int slots = max(1, a.max_chunks - 1);             // a pair of S positions meets at most ceil(S / per) + 1 shares
    per = max(per, (long long)((longest + slots - 1) / slots));
    per = max(per, 1ll);
    bs.per = (int)((per + plan.tile - 1) / plan.tile) * plan.tile;
    return bs;
}

// The piece that starts at position x of the laid-out pairs and ends at `hi` or at its pair's end,
// whichever comes first (lo <= x < hi <= total).  Warp-cooperative: all lanes call it with the same
// arguments and get the same answer.  `ends_pair` tells whether the piece is its pair's last.
__device__ __forceinline__ ItemGeometry balanced_piece(const FastArgs& a, const FastPlan& plan, const BalancedShare& bs,
                                                       long long x, long long hi, int lane, bool& ends_pair) {
    ItemGeometry g;
    g.b = g.hgroup = g.c = g.start = g.end = 0;
    ends_pair = false;
    long long base = 0;
    for (int b0 = 0; b0 < a.batch; b0 += 32) {
        const int s = (b0 + lane < a.batch) ? a.kv_offsets[b0 + lane] + 1 : 0;
        const long long mine = (long long)s * plan.n_hgroups;
        long long incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const long long v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        const long long first = base + incl - mine;          // where this lane's sequence starts
        const unsigned hit = __ballot_sync(0xffffffffu, s > 0 && x >= first && x < base + incl);
        if (hit) {
            const int src = __ffs(hit) - 1;
            const int len = __shfl_sync(0xffffffffu, s, src);
            const long long seq_first = __shfl_sync(0xffffffffu, first, src);
            const long long off = x - seq_first;
            g.b = b0 + src;
            g.hgroup = (int)(off / len);
            g.start = (int)(off - (long long)g.hgroup * len);
            const long long pair_first = seq_first + (long long)g.hgroup * len;
            const long long pair_end = pair_first + len;
            const long long e = min(hi, pair_end);
            g.end = g.start + (int)(e - x);
            g.c = (int)(x / bs.per) - (int)(pair_first / bs.per);
            ends_pair = (e == pair_end);
            return g;
        }
        base += __shfl_sync(0xffffffffu, incl, 31);
    }
    return g;   // not reached for x < total
}

// Fused append: the newest row of a sequence for the item's head group (`new_row`, hg * D halves,
// rotated at `pos` unless rope_type < 0 or `rotate` is false) goes to its place in the cache and to
// row `r` of the tile at `tile_dst` (swizzled layout), four bytes per lane and step.
template <int D>
__device__ __forceinline__ void append_row_to_tile_and_cache(const __half* __restrict__ new_row, __half* __restrict__ cache_row,
                                                             uint32_t tile_dst, int r, int hg, int blk_bytes, bool rotate,
                                                             const __half* cos_table, const __half* sin_table, int pos,
                                                             int rope_type, int rotary_dim, int lane) {
    for (int idx = lane; idx < hg * D / 2; idx += 32) {
        const int head = (2 * idx) / D, d = 2 * idx - head * D;
        const __half* x = new_row + head * D;
        const __half y0 = rotate ? rope_channel(x, d, D, cos_table, sin_table, pos, rope_type, rotary_dim) : x[d];
        const __half y1 = rotate ? rope_channel(x, d + 1, D, cos_table, sin_table, pos, rope_type, rotary_dim) : x[d + 1];
        const __half2 y = __halves2half2(y0, y1);
        const uint32_t w = *reinterpret_cast<const uint32_t*>(&y);
        reinterpret_cast<uint32_t*>(cache_row)[idx] = w;
        const int chunk = idx >> 2;                                  // 16-byte chunk of the row
        const uint32_t addr = tile_dst + (chunk >> 3) * blk_bytes + r * 128 + ((((chunk & 7) ^ (r & 7))) << 4) + (idx & 3) * 4;
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(addr), "r"(w) : "memory");
    }
}

template <int D, int CW, bool kRope = false, bool kColSplitKernel = false>
__device__ __forceinline__ void fast_partial_body(const FastArgs& a)
{
    constexpr bool kCompact = (CW == kCompactConsumerWarps);
    // Full shape: the boxes of a tile (one per 128-byte column block) are issued by as many lanes in one
    // warp instruction; issued by one lane in turn they cost the loader about as long as the tile's share of
    // the stream lasts (one million positions: 157.5 vs 167.1 us per layer, sixteen 256-wide sequences 172.9
    // vs 177.7).  The compact shape keeps the one lane: its launches live on how soon the FIRST tile lands,
    // and six tiles' boxes requested at once delay it (32k context: 10.07 vs 9.85 us per layer).
    constexpr bool kTmaLanes = (VTEB_TMA_LANES != 0) && !kCompact;
    constexpr int kLoaderWarpK = CW;          // loads K rows, owns the work queue
    constexpr int kLoaderWarpV = CW + 1;      // loads V rows, follows the K loader's headers
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const FastPlan plan = make_fast_plan(a.num_q_heads, a.num_kv_heads, D, kCompact ? 1 : 0);
    const int group = a.num_q_heads / a.num_kv_heads;

    volatile int* abort_word = reinterpret_cast<volatile int*>(smem_raw + kAbortOffset);
    TileHeader* headers = reinterpret_cast<TileHeader*>(smem_raw + kHeaderOffset);
    float* merge = reinterpret_cast<float*>(smem_raw + kCtrlBytes);
    uint32_t* q_store = reinterpret_cast<uint32_t*>(smem_raw + kCtrlBytes + plan.merge_bytes);
    // stages start on the next 1024-byte shared address (the plan reserves the slack)
    unsigned char* stages = smem_raw + kCtrlBytes + plan.merge_bytes + plan.q_bytes;
    stages += (kStageAlign - (smem_u32(stages) & (kStageAlign - 1))) & (kStageAlign - 1);

    const uint32_t bar0 = smem_u32(smem_raw);
    const uint32_t full0 = bar0 + kBarFull * 1, empty0 = bar0 + kBarEmpty, hdr0 = bar0 + kBarHeader;
    const uint32_t merge_bar0 = bar0 + kBarMerge;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nstages = plan.nstages;

    // The first item's geometry needs one global load (the sequence's kv offset): start it
    // before the barrier set-up so its latency is hidden.
    const bool balanced = !kCompact && (a.flags & kFlagBalanced) != 0;   // the compact shape serves one sequence: no such code in it
    int total_items = a.batch * plan.n_hgroups * a.max_chunks;
    ItemGeometry first_geom;
    first_geom.b = first_geom.hgroup = first_geom.c = first_geom.start = first_geom.end = 0;
    BalancedShare share;
    share.total = 0; share.per = 1;
    long long share_lo = 0, share_hi = 0;      // this CTA's positions of the laid-out pairs (balanced partition)
    bool first_ends_pair = false;
    if (balanced) {
        share = balanced_share(a, plan, threadIdx.x & 31);
        share_lo = min((long long)blockIdx.x * share.per, share.total);
        share_hi = min(share_lo + share.per, share.total);
        // below, "blockIdx.x < total_items" reads "this CTA has a first item"
        total_items = (share_hi > share_lo) ? (int)gridDim.x : 0;
        if (share_hi > share_lo) first_geom = balanced_piece(a, plan, share, share_lo, share_hi, threadIdx.x & 31, first_ends_pair);
    } else if ((int)blockIdx.x < total_items) {
        first_geom = decode_item(a, plan, blockIdx.x);
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(full0 + 8 * s, 65);   // asynchronous-copy arrivals of the loader lanes + the header writer
            mbar_init(empty0 + 8 * s, plan.active_warps);
            mbar_init(hdr0 + 8 * s, 1);
        }
        mbar_init(merge_bar0, plan.active_warps);
        mbar_init(merge_bar0 + 8, plan.active_warps);
        mbar_init(bar0 + kBarFinal, plan.active_warps);
        mbar_init(bar0 + kBarFinal + 8, 1);
        *abort_word = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
#ifdef VTEB_TRACE
    TraceCtx tr; tr.base = nullptr;
    {
        __shared__ int trace_launch;
        const int sel = (blockIdx.x == 0) ? 0 : (blockIdx.x == gridDim.x / 2) ? 1 : (blockIdx.x + 3 == gridDim.x) ? 2 : -1;
        if (threadIdx.x == 0 && sel >= 0) trace_launch = atomicAdd(a.status + 15 + sel, 1);
        __syncthreads();
        if (sel >= 0 && trace_launch < 64)
            tr.base = reinterpret_cast<unsigned long long*>(a.status - 1) + 32 +
                      (((size_t)trace_launch * 3 + sel) * 10 + (threadIdx.x >> 5)) * 32;
    }
    VTEB_TR_GT(tr, 0);
    VTEB_TR(tr, 1);
#endif
    __syncthreads();
    grid_launch_dependents();

    const long long pos_stride = 2ll * a.num_kv_heads * D;      // bytes between positions
    const bool use_tensor_maps = (a.flags & kFlagTensorMaps) != 0;
    const int rows_per_seq = (int)(a.kv_batch_stride / (a.num_kv_heads * D));   // tensor-map rows per sequence
    const int n_col_blocks = plan.row_bytes >> 7;

    // ===================================================================== K loader
    if (warp == kLoaderWarpK) {
        if ((a.flags & kFlagPrefetchQ) && lane == 0 && (int)blockIdx.x < total_items && first_geom.c == 0) {
            // Q of the first item is read right after the dependency wait; when it is not in L2 by then
            // (nothing produced it recently) the consumers start a DRAM latency late.  A prefetch moves no
            // data into the SM, so it may run ahead of the kernel that writes Q: L2 is where that write lands.
            // Only the CTA that owns split 0 of a (sequence, head group) asks: the others share its rows.
            const __half* q0 = a.q + ((long long)first_geom.b * a.num_q_heads + (long long)first_geom.hgroup * plan.hg * group) * D;
            const unsigned qbytes = (unsigned)(plan.hg * group * D * 2);
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(q0), "r"(qbytes) : "memory");
        }
        int stage = 0, filled = 0;
        uint32_t empty_parity = 0;
        bool dep_done = false;
        int item = blockIdx.x;
        long long cursor = share_lo;               // balanced partition: where the next piece starts
        bool alive = true;
        while (alive) {
            const bool stop = balanced ? (cursor >= share_hi) : (item >= total_items);
            ItemGeometry g = first_geom;
            if (!stop && item != (int)blockIdx.x) {
                bool ends_pair;
                g = balanced ? balanced_piece(a, plan, share, cursor, share_hi, lane, ends_pair) : decode_item(a, plan, item);
            }
            const int ntiles = stop ? 1 : max(1, (g.end - g.start + plan.tile - 1) / plan.tile);
            if ((a.flags & kFlagPrefetchQ) && !stop && item != (int)blockIdx.x && g.c == 0 && g.end > g.start && lane == 0) {
                // a later item: the loader runs several tiles ahead of the consumers, so asking L2 for the
                // item's Q rows now means their loads at the item's first tile do not go to DRAM
                const __half* qn = a.q + ((long long)g.b * a.num_q_heads + (long long)g.hgroup * plan.hg * group) * D;
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(qn), "r"((unsigned)(plan.hg * group * D * 2)) : "memory");
            }
            for (int t = 0; t < ntiles; ++t) {
                if (filled >= nstages) {
                    if (!mbar_wait_bounded(empty0 + 8 * stage, (empty_parity >> stage) & 1u, abort_word)) {
                        raise_abort(abort_word, a.status, kStatusEmptyTimeout);
                        alive = false;
                        break;
                    }
                    empty_parity ^= (1u << stage);
                }
                const uint32_t bar = full0 + 8 * stage;
                const bool empty_item = !stop && g.end <= g.start;
                const int pos0 = stop ? 0 : g.start + t * plan.tile;
                const int nvalid = (stop || empty_item) ? 0 : min(plan.tile, g.end - pos0);
                // The newest cache row may be written by the kernel launched just before
                // this one: wait for that kernel before touching the sequence's last position.
                if (!dep_done && !stop && !empty_item && g.end == a.kv_offsets[g.b] + 1 && pos0 + nvalid >= g.end) {
                    grid_dependency_wait();
                    dep_done = true;
                }
                if (lane == 0) {
                    TileHeader h;
                    h.b = stop ? 0 : g.b; h.hgroup = stop ? 0 : g.hgroup; h.c = stop ? 0 : g.c;
                    h.blk0 = t * (plan.tile / kBlockPos); h.nvalid = nvalid; h.pos0 = pos0;
                    h.last_pos = stop ? 0 : g.end - 1;
                    h.flags = stop ? kTileStop
                                   : ((t == 0 ? kTileFirst : 0) | (t == ntiles - 1 ? kTileLast : 0) | (empty_item ? kTileEmpty : 0));
                    headers[stage] = h;
                    mbar_arrive(hdr0 + 8 * stage);
                    mbar_arrive(bar);
                }
                if (nvalid > 0) {
                    const int nrows = vteb_round_up(nvalid, kBlockPos);
                    const unsigned char* src = reinterpret_cast<const unsigned char*>(a.k_cache) +
                        2ll * ((long long)g.b * a.kv_batch_stride + (long long)g.hgroup * plan.hg * D) +
                        (long long)pos0 * pos_stride;
                    const unsigned char* src_last = src + (long long)(g.end - 1 - pos0) * pos_stride;
                    const uint32_t dst = smem_u32(stages + (size_t)stage * plan.stage_bytes);
                    bool append_here = false;
                    if constexpr (kRope) {
                        append_here = a.k_new != nullptr && g.end == a.kv_offsets[g.b] + 1 && pos0 + nvalid >= g.end;
                    }
                    if (append_here) {
                        // The tile ends with the sequence's newest position, whose row is not in the cache yet:
                        // older rows come from the cache (masked rows are filled from the new row, which is
                        // finite), then the new row is rotated and written to the cache and into the tile.
                        const __half* knew = a.k_new + ((long long)g.b * a.num_kv_heads + (long long)g.hgroup * plan.hg) * D;
                        copy_rows_async(src, reinterpret_cast<const unsigned char*>(knew), dst, nrows, nvalid - 1, plan.row_bytes,
                                        plan.blk_bytes, pos_stride, lane);
                        asm volatile("cp.async.wait_all;" ::: "memory");
                        __syncwarp();
                        __half* cache_row = const_cast<__half*>(a.k_cache) + (long long)g.b * a.kv_batch_stride +
                                            (long long)(g.end - 1) * a.num_kv_heads * D + (long long)g.hgroup * plan.hg * D;
                        append_row_to_tile_and_cache<D>(knew, cache_row, dst, nvalid - 1, plan.hg, plan.blk_bytes, true, a.rope_cos,
                                                        a.rope_sin, g.end - 1, a.rope_type, a.rotary_dim, lane);
                        mbar_arrive(bar);                       // every lane: releases its own stores
                    } else if (use_tensor_maps && nvalid == plan.tile) {
                        // a whole tile: one elected lane issues one box per 128-byte column block
                        if constexpr (kTmaLanes) {
                            // one box per lane: the column blocks of a tile are issued by one warp instruction
                            if (lane == 0) mbar_arrive_expect_tx(bar, plan.tile * plan.row_bytes);
                            else mbar_arrive(bar);
                            if (lane < n_col_blocks)
                                tma_load_box_2d(dst + lane * plan.blk_bytes, a.tmap_k, g.hgroup * plan.hg * D + lane * 64,
                                                g.b * rows_per_seq + pos0, bar);
                        } else if (lane == 0) {
                            mbar_arrive_expect_tx(bar, plan.tile * plan.row_bytes);
                            const int x0 = g.hgroup * plan.hg * D, y = g.b * rows_per_seq + pos0;
                            for (int cb = 0; cb < n_col_blocks; ++cb)
                                tma_load_box_2d(dst + cb * plan.blk_bytes, a.tmap_k, x0 + cb * 64, y, bar);
                        } else {
                            mbar_arrive(bar);
                        }
                    } else {
                        copy_rows_async(src, src_last, dst, nrows, nvalid, plan.row_bytes, plan.blk_bytes, pos_stride, lane);
                        async_copy_arrive(bar);
                    }
                } else {
                    mbar_arrive(bar);      // no copies belong to this tile
                }
                ++filled;
                if (filled <= 8) VTEB_TR(tr, 11 + filled);
                if (filled == 1) VTEB_TR(tr, 2);
                if (filled == nstages) VTEB_TR(tr, 3);
                if (!stop) VTEB_TR(tr, 4);
                stage = (stage + 1 == nstages) ? 0 : stage + 1;
            }
            if (stop || !alive) break;
            if (balanced) {
                // the next piece of this CTA's share; `item` only has to differ from blockIdx.x from now on
                cursor += g.end - g.start;
                item = -1;
                continue;
            }
            // Later items come from the shared ticket, which the previous combine
            // launch reset: it may only be touched once that launch has completed.
            if (!dep_done) { grid_dependency_wait(); dep_done = true; }
            if (a.flags & kFlagDirectOutput) { item = total_items; continue; }   // unsplit: one item per CTA, go publish the stop tile
            // (taken only now, not while the current item's tiles were being issued: a CTA that reserves its
            // next item early keeps it from CTAs that run dry first, and with one to four items per CTA that
            // costs more than the atomic's round trip: 193 -> 210 us per layer on the 64-sequence batch)
            int next = 0;
            if (lane == 0) next = gridDim.x + atomicAdd(a.ticket, 1);
            item = __shfl_sync(0xffffffffu, next, 0);
        }
        if (a.next_k_cache != nullptr && plan.n_hgroups == 1 && total_items <= (int)gridDim.x && (int)blockIdx.x < total_items) {
            const ItemGeometry g = first_geom;
            if (g.end > g.start && (long long)(g.end - g.start) * pos_stride * total_items <= kL2PrefetchMaxBytes)
                prefetch_range_l2(reinterpret_cast<const unsigned char*>(a.next_k_cache) +
                                      2ll * (long long)g.b * a.kv_batch_stride + (long long)g.start * pos_stride,
                                  (long long)(g.end - g.start) * pos_stride, lane);
        }
        if (!dep_done) grid_dependency_wait();
        if (balanced && alive) {
            // Splits past a pair's last piece hold nothing: mark them empty for the combine, as the
            // reference's kernel does for chunks past the sequence (flash_attention_split_kv_partial.hip.template:59-69).
            // The (sequence, query head) rows are dealt to the CTAs in equal runs, whatever their shares hold, so
            // that no CTA has more than a few rows to mark and one prefix sum of the lengths serves a whole run.  After the dependency wait: the launch before this
            // one may still have read the partial buffers.
            const int heads_pair = plan.hg * group;
            const int rows = a.batch * a.num_q_heads;
            const int rows_per_cta = (rows + gridDim.x - 1) / gridDim.x;
            const int row0 = blockIdx.x * rows_per_cta, row1 = min(rows, row0 + rows_per_cta);
            if (row0 < row1) {
                int b = row0 / a.num_q_heads;
                long long before = 0;                                  // positions of the sequences ahead of b
                for (int b0 = 0; b0 < b; b0 += 32)
                    before += (b0 + lane < b) ? a.kv_offsets[b0 + lane] + 1 : 0;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) before += __shfl_xor_sync(0xffffffffu, before, o);
                int len = a.kv_offsets[b] + 1;
                for (int row = row0; row < row1;) {
                    if (row >= (b + 1) * a.num_q_heads) { before += len; ++b; len = a.kv_offsets[b] + 1; }
                    // the rows of one pair share their number of pieces: one pair (or what this run holds of it) per turn
                    const int hgroup = (row - b * a.num_q_heads) / heads_pair;
                    const int row_end = min(row1, b * a.num_q_heads + (hgroup + 1) * heads_pair);
                    const long long pair_first = before * plan.n_hgroups + (long long)hgroup * len;
                    const int live = (int)((pair_first + len - 1) / share.per) - (int)(pair_first / share.per) + 1;
                    const int idle = a.max_chunks - live;
                    for (int i = lane; i < (row_end - row) * idle; i += 32) {
                        const int r = i / idle;
                        const long long stat = (long long)(row + r) * a.max_chunks + live + (i - r * idle);
                        a.partial_m[stat] = kNeutralM;
                        a.partial_l[stat] = 0.f;
                        if (a.flags & kFlagWriteEmptyO)
                            for (int d = 0; d < D; ++d) a.partial_o[stat * D + d] = 0.f;
                    }
                    row = row_end;
                }
            }
        }
        VTEB_TR(tr, 5);
        asm volatile("cp.async.wait_all;" ::: "memory");   // own copies have landed before the warp leaves
        VTEB_TR(tr, 8);
        VTEB_TR_GT(tr, 9);
        return;
    }

    // ===================================================================== V loader
    if (warp == kLoaderWarpV) {
        int stage = 0;
        uint32_t hdr_parity = 0;
        bool dep_done = false;
        for (;;) {
            if (!mbar_wait_bounded(hdr0 + 8 * stage, (hdr_parity >> stage) & 1u, abort_word)) break;
            hdr_parity ^= (1u << stage);
            const TileHeader hd = headers[stage];
            const uint32_t bar = full0 + 8 * stage;
            if (hd.nvalid > 0) {
                if (!dep_done && hd.last_pos == a.kv_offsets[hd.b] && hd.pos0 + hd.nvalid > hd.last_pos) {
                    grid_dependency_wait();
                    dep_done = true;
                }
                const int nrows = vteb_round_up(hd.nvalid, kBlockPos);
                const unsigned char* src = reinterpret_cast<const unsigned char*>(a.v_cache) +
                    2ll * ((long long)hd.b * a.kv_batch_stride + (long long)hd.hgroup * plan.hg * D) +
                    (long long)hd.pos0 * pos_stride;
                const unsigned char* src_last = src + (long long)(hd.last_pos - hd.pos0) * pos_stride;
                const uint32_t dst = smem_u32(stages + (size_t)stage * plan.stage_bytes) + plan.tile * plan.row_bytes;
                bool append_here = false;
                if constexpr (kRope) {
                    append_here = a.v_new != nullptr && hd.last_pos == a.kv_offsets[hd.b] && hd.pos0 + hd.nvalid > hd.last_pos;
                }
                if (append_here) {
                    const __half* vnew = a.v_new + ((long long)hd.b * a.num_kv_heads + (long long)hd.hgroup * plan.hg) * D;
                    copy_rows_async(src, reinterpret_cast<const unsigned char*>(vnew), dst, nrows, hd.nvalid - 1, plan.row_bytes,
                                    plan.blk_bytes, pos_stride, lane);
                    asm volatile("cp.async.wait_all;" ::: "memory");
                    __syncwarp();
                    __half* cache_row = const_cast<__half*>(a.v_cache) + (long long)hd.b * a.kv_batch_stride +
                                        (long long)hd.last_pos * a.num_kv_heads * D + (long long)hd.hgroup * plan.hg * D;
                    append_row_to_tile_and_cache<D>(vnew, cache_row, dst, hd.nvalid - 1, plan.hg, plan.blk_bytes, false, nullptr,
                                                    nullptr, 0, -1, 0, lane);
                    mbar_arrive(bar);
                } else if (use_tensor_maps && hd.nvalid == plan.tile) {
                    if constexpr (kTmaLanes) {
                        if (lane == 0) mbar_arrive_expect_tx(bar, plan.tile * plan.row_bytes);
                        else mbar_arrive(bar);
                        if (lane < n_col_blocks)
                            tma_load_box_2d(dst + lane * plan.blk_bytes, a.tmap_v, hd.hgroup * plan.hg * D + lane * 64,
                                            hd.b * rows_per_seq + hd.pos0, bar);
                    } else if (lane == 0) {
                        mbar_arrive_expect_tx(bar, plan.tile * plan.row_bytes);
                        const int x0 = hd.hgroup * plan.hg * D, y = hd.b * rows_per_seq + hd.pos0;
                        for (int cb = 0; cb < n_col_blocks; ++cb)
                            tma_load_box_2d(dst + cb * plan.blk_bytes, a.tmap_v, x0 + cb * 64, y, bar);
                    } else {
                        mbar_arrive(bar);
                    }
                } else {
                    copy_rows_async(src, src_last, dst, nrows, hd.nvalid, plan.row_bytes, plan.blk_bytes, pos_stride, lane);
                    async_copy_arrive(bar);
                }
            } else {
                mbar_arrive(bar);
            }
            if (hd.flags & kTileStop) break;
            stage = (stage + 1 == nstages) ? 0 : stage + 1;
        }
        if (a.next_v_cache != nullptr && plan.n_hgroups == 1 && total_items <= (int)gridDim.x && (int)blockIdx.x < total_items) {
            const ItemGeometry g = first_geom;
            if (g.end > g.start && (long long)(g.end - g.start) * pos_stride * total_items <= kL2PrefetchMaxBytes)
                prefetch_range_l2(reinterpret_cast<const unsigned char*>(a.next_v_cache) +
                                      2ll * (long long)g.b * a.kv_batch_stride + (long long)g.start * pos_stride,
                                  (long long)(g.end - g.start) * pos_stride, lane);
        }
        if (!dep_done) grid_dependency_wait();
        asm volatile("cp.async.wait_all;" ::: "memory");
        VTEB_TR(tr, 8);
        VTEB_TR_GT(tr, 9);
        return;
    }

    if (warp >= plan.active_warps) return;

    // ===================================================================== consumers
    // warp = (sub * DS + dhalf) * hg + hh
    // 128-wide heads, and 256-wide heads in the full shape, take the transposed form of the block (consumer_block.cuh); its state is `tt`.
    constexpr bool kT = (VTEB_TRANSPOSED != 0) && (D == 128 || (D == 256 && !kCompact));
    constexpr int DS = (D == 256 && !kT) ? 2 : 1;       // warps sharing one (head, block), split by output columns
    const int hh = warp % plan.hg;                      // KV head within the group
    const int dhalf = (warp / plan.hg) % DS;            // which part of the output columns this warp owns
    const int sub = warp / (plan.hg * DS);              // which of the wph interleaved block streams
    int next_blk = sub;                   // index, within the item, of this warp's next block: sub, sub + wph, ...
    const int g = lane >> 2, t = lane & 3;
    const float scale2 = a.scale * kLog2e;
    constexpr int KS = D / 16;            // k-steps of the QK^T product
    constexpr int NT = D / 8 / DS;        // 8-wide output column tiles owned by this warp
    constexpr int DW = D / DS;            // output columns owned by this warp
    const int blocks_per_tile = plan.tile / kBlockPos;

    // Q operand fragments of this warp's KV head: word i of lane L at q_frag[i * 32].
    // Every warp of the head writes the same values; they are rewritten only after
    // the item's merge barrier, when no warp of the CTA still reads the old ones.
    uint32_t* q_frag = q_store + hh * (KS * 2 * 32) + lane;
    auto load_q = [&](int b, int hgroup) {
        const int kv_head = hgroup * plan.hg + hh;
        const uint32_t* qrow = reinterpret_cast<const uint32_t*>(
            a.q + ((long long)b * a.num_q_heads + (long long)kv_head * group + g) * D);
        uint32_t tmp[KS * 2];
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            tmp[2 * ks] = (g < group) ? qrow[ks * 8 + t] : 0u;
            tmp[2 * ks + 1] = (g < group) ? qrow[ks * 8 + 4 + t] : 0u;
        }
        if constexpr (kRope) {
            // q holds the un-rotated projection: rotate it at the sequence's current position, in
            // fp32, and round to fp16 exactly as the standalone rotation kernel would have stored it
            if (g < group)
                rope_rotate_q_words<KS>(tmp, a.rope_cos, a.rope_sin, a.kv_offsets[b], a.rope_type, a.rotary_dim, t);
        }
#pragma unroll
        for (int i = 0; i < KS * 2; ++i) q_frag[i * 32] = tmp[i];
        __syncwarp();
    };

    ConsumerState<NT, kLoAcc> st;
    ConsumerStateT<D / 16> tt;
    st.reset();
    tt.reset();
    // Column split (the `..._compact_cs_d128_kernel` instantiation; three warps per KV head, partials wanted):
    // every warp of a head computes the scores of all the item's blocks and accumulates its own 16-column
    // tiles only, so the item ends without a cross-warp merge.  The scores are computed three times over,
    // which pays only while an item is one block long (28 layers per graph, us per layer: 512-position
    // context 5.62 vs 5.85, 2,048: 5.88 vs 6.37, 4,096 = two blocks per item: 6.42 vs 6.35, 32k = 14 blocks:
    // 13.3 vs 9.9), so the dispatcher picks this kernel for contexts whose splits cannot exceed 16 positions.  (A kernel of its own: the mere presence of this
    // path in the compact kernel changed its register allocation and cost the 32k workload 0.5 us per layer.)
    // The warps that are alone on their
    // scheduler (sub 1) take four of the eight tiles, the others two each; the accumulators are the first four tiles of `tt`.
    const bool colsplit = kColSplitKernel && plan.wph == 3 && !(a.flags & kFlagDirectOutput);
    const int cs_mt0 = (sub == 0) ? 0 : (sub == 1) ? 2 : 6, cs_nmt = (sub == 1) ? 4 : 2;
    bool cs_pending = false;              // the head's warps have yet to meet before Q may be rewritten
    int stage = 0;
    uint32_t full_parity = 0, merge_parity = 0;
    bool merge_pending = false;           // previous item's readers may still use the exchange area
    bool first_item = true;

    // Lane-constant parts of the ldmatrix addresses.
    // K, per 16-half k-step: matrices (rows 0-7, chunk 0), (rows 0-7, chunk 1), (rows 8-15, chunk 0),
    // (rows 8-15, chunk 1); V, per 16 output columns: (rows 0-7, chunk 0), (rows 8-15, chunk 0),
    // (rows 0-7, chunk 1), (rows 8-15, chunk 1).  A lane's row has r & 7 == lane & 7, so the
    // swizzle term of its address is a lane constant XORed with the k-step's chunk pair.
    const int blk_bytes = plan.blk_bytes;
    const uint32_t k_lane_off = ((lane & 7) + ((lane >> 4) << 3)) * 128 + hh * (D / 64) * blk_bytes;
    const uint32_t k_lane_x = ((((lane >> 3) & 1) ^ (lane & 7)) << 4);
    const uint32_t v_lane_off = ((lane & 7) + (((lane >> 3) & 1) << 3)) * 128 +
                                (hh * (D / 64) + dhalf * (DW / 64)) * blk_bytes + plan.tile * plan.row_bytes;
    const uint32_t v_lane_x = (((lane >> 4) ^ (lane & 7)) << 4);

    // The first item is known without the loader: fetch its Q while the first tile is in flight.
    grid_dependency_wait();
    VTEB_TR(tr, 2);
    if ((int)blockIdx.x < total_items) load_q(first_geom.b, first_geom.hgroup);
    VTEB_TR(tr, 3);
#ifdef VTEB_TRACE
    bool trace_first_full = true;
    int trace_tile = 0;
    long long trace_wait = 0;
#endif

    for (;;) {
#ifdef VTEB_TRACE
        const long long trace_w0 = clock64();
#endif
        if (!mbar_wait_bounded(full0 + 8 * stage, (full_parity >> stage) & 1u, abort_word)) {
            raise_abort(abort_word, a.status, kStatusFullTimeout);
            return;
        }
#ifdef VTEB_TRACE
        trace_wait += clock64() - trace_w0;
        if (trace_first_full) { VTEB_TR(tr, 4); trace_first_full = false; }
        if (trace_tile < 8) VTEB_TR(tr, 12 + trace_tile);
#endif
        full_parity ^= (1u << stage);
        const TileHeader* hd = headers + stage;
        const int flags = hd->flags;
        if (flags & kTileStop) break;
        // Copy what is needed later: the loader may rewrite the header once every
        // consumer warp has released the stage.
        const int item_b = hd->b, item_hgroup = hd->hgroup, item_c = hd->c;
        const int nvalid = hd->nvalid, blk0 = hd->blk0;

        if (flags & kTileFirst) {
            st.reset();
            tt.reset();
            if (cs_pending) {
                // every consumer warp has left the previous item: its Q fragments may be overwritten
                if (!mbar_wait_bounded(merge_bar0, merge_parity & 1u, abort_word)) {
                    raise_abort(abort_word, a.status, kStatusMergeTimeout);
                    return;
                }
                merge_parity ^= 1u;
                cs_pending = false;
            }
            if (!first_item) load_q(item_b, item_hgroup);
            first_item = false;
        }

        const uint32_t tile_base = smem_u32(stages + (size_t)stage * plan.stage_bytes);
        if (flags & kTileFirst) next_blk = sub;
        if constexpr (kColSplitKernel) {
            if (colsplit) {
                for (int r0 = 0; r0 < nvalid; r0 += kBlockPos) {
                    float sr[4];
                    qk_block_t<D>(q_frag, (tile_base + r0 * 128 + k_lane_off) | k_lane_x, blk_bytes, sr);
                    softmax_pv_t_cols<4>(tt, sr, (tile_base + r0 * 128 + v_lane_off) | v_lane_x, blk_bytes, nvalid - r0, scale2, g,
                                         cs_mt0, cs_nmt);
                }
                next_blk = blk0 + blocks_per_tile;          // nothing left for the loop below
            }
        }
        for (; next_blk < blk0 + blocks_per_tile; next_blk += plan.wph) {
            const int r0 = (next_blk - blk0) * kBlockPos;
            if (r0 >= nvalid) break;
            if constexpr (kT) {
                float sr[4];
                qk_block_t<D>(q_frag, (tile_base + r0 * 128 + k_lane_off) | k_lane_x, blk_bytes, sr);
                softmax_pv_t<D / 16>(tt, sr, (tile_base + r0 * 128 + v_lane_off) | v_lane_x, blk_bytes, nvalid - r0, scale2, g);
            } else {
                float sn[2][2];
                qk_block<D, kQkChains>(q_frag, (tile_base + r0 * 128 + k_lane_off) | k_lane_x, blk_bytes, sn);
                softmax_pv<NT, kLoAcc>(st, sn, (tile_base + r0 * 128 + v_lane_off) | v_lane_x, blk_bytes, nvalid - r0, scale2, t);
            }
        }
        if (flags & kTileLast) {
            st.fold_lo();
            VTEB_TR(tr, 5);
        }

#ifdef VTEB_TRACE
        if (trace_tile < 8) VTEB_TR(tr, 20 + trace_tile);
        ++trace_tile;
#endif
        // Hand the stage back to the loader.
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * stage);

        if (flags & kTileLast) {
            stage = (stage + 1 == nstages) ? 0 : stage + 1;
            if constexpr (kColSplitKernel) {
                if (colsplit) {
                    // every warp holds the finished state of its columns: restate it against the rows' true
                    // maximum and store it; the warps with sub 0 store m and l
                    const bool empty = (flags & kTileEmpty) != 0;
                    const bool write_o = !empty || (a.flags & kFlagWriteEmptyO);
                    const long long stat_base = ((long long)item_b * a.num_q_heads + (long long)item_hgroup * plan.hg * group +
                                                 (long long)hh * group) * a.max_chunks + item_c;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int r = 2 * t + h;
                        float l_head = sum_over_g(tt.l[h]);
#if VTEB_LAZY_MAX > 0
                        const float m_head = max_over_g(tt.mt[h]);
#else
                        const float m_head = tt.m[h];
#endif
                        const float f = fast_exp2(tt.m[h] - m_head);
                        l_head *= f;
                        if (r < group) {
                            const long long stat = stat_base + (long long)r * a.max_chunks;
                            if (write_o) {
                                float* orow = a.partial_o + stat * D + g;
#pragma unroll
                                for (int i = 0; i < 4; ++i)
                                    if (i < cs_nmt) {
                                        orow[(cs_mt0 + i) * 16] = tt.o[i][h] * f;
                                        orow[(cs_mt0 + i) * 16 + 8] = tt.o[i][2 + h] * f;
                                    }
                            }
                            if (sub == 0 && g == 0) {
                                a.partial_m[stat] = empty ? kNeutralM : m_head * kLn2;
                                a.partial_l[stat] = empty ? 0.f : l_head;
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(merge_bar0);
                    cs_pending = true;
                    VTEB_TR(tr, 6);
                    VTEB_TR(tr, 7);
                    continue;
                }
            }
            // ---- exchange (m, l, o) between the warps of each KV head and store the item
            const int pitch = D + kMergePad;           // floats per (warp, row): o[D], 4 unused, m, l, true maximum, 1 unused
            if (plan.wph == 1 && !kT) {
                // One warp per KV head: nothing to merge, the warp stores its own state.
                // (The transposed form goes through the exchange area here too: its registers hold
                // one column of eight heads, which no global store takes well.)
                float l_own = st.l;
                l_own += __shfl_xor_sync(0xffffffffu, l_own, 1);
                l_own += __shfl_xor_sync(0xffffffffu, l_own, 2);
                const bool empty1 = (flags & kTileEmpty) != 0;
#if VTEB_LAZY_MAX > 0
                {   // restate (m, l, o) against the row's true maximum, as the partial buffers promise
                    const float m_true = st.true_max();
                    const float f = fast_exp2(st.m - m_true);
                    l_own *= f;
#pragma unroll
                    for (int n = 0; n < NT; ++n) { st.o[n][0] *= f; st.o[n][1] *= f; }
                    st.m = m_true;
                }
#endif
                if (g < group && (a.flags & kFlagDirectOutput)) {
                    // unsplit: this warp holds the whole sequence's state for its rows
                    const long long row = (long long)item_b * a.num_q_heads + (long long)item_hgroup * plan.hg * group +
                                          (long long)hh * group + g;
                    const float inv = 1.f / fmaxf(l_own, 1e-20f);
#pragma unroll
                    for (int n = 0; n < NT; ++n)
                        store_out2(a.output, a.out_kind, row * D + dhalf * DW + n * 8 + 2 * t,
                                   make_float2(st.o[n][0] * inv, st.o[n][1] * inv));
                } else if (g < group) {
                    const long long stat = ((long long)item_b * a.num_q_heads + (long long)item_hgroup * plan.hg * group +
                                            (long long)hh * group + g) * a.max_chunks + item_c;
                    if (!empty1 || (a.flags & kFlagWriteEmptyO)) {
                        float* out = a.partial_o + stat * D + dhalf * DW + 2 * t;
#pragma unroll
                        for (int n = 0; n < NT; ++n)
                            *reinterpret_cast<float2*>(out + n * 8) = make_float2(st.o[n][0], st.o[n][1]);
                    }
                    if (t == 0 && dhalf == 0) {
                        a.partial_m[stat] = empty1 ? kNeutralM : st.m * kLn2;
                        a.partial_l[stat] = empty1 ? 0.f : l_own;
                    }
                }
                continue;
            }
            if (merge_pending) {
                // everyone must have finished reading the previous item's exchange area
                if (!mbar_wait_bounded(merge_bar0 + 8, (merge_parity >> 1) & 1u, abort_word)) {
                    raise_abort(abort_word, a.status, kStatusMergeTimeout);
                    return;
                }
                merge_parity ^= 2u;
            }
            if constexpr (kT) {
                // thread (g, t): heads 2t, 2t+1; columns 16*mt + g and + 8.  Rows of the exchange area are per (warp, head).
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int r = 2 * t + h;
                    const float l_head = sum_over_g(tt.l[h]);
#if VTEB_LAZY_MAX > 0
                    const float m_head = max_over_g(tt.mt[h]);
#else
                    const float m_head = tt.m[h];
#endif
                    if (r < group) {
                        float* dst = merge + ((size_t)warp * group + r) * pitch;
#pragma unroll
                        for (int mt = 0; mt < D / 16; ++mt) {
                            dst[mt * 16 + g] = tt.o[mt][h];
                            dst[mt * 16 + g + 8] = tt.o[mt][2 + h];
                        }
                        if (g == 0) { dst[D + 4] = tt.m[h]; dst[D + 5] = l_head; dst[D + kMergeTrueMax] = m_head; }
                    }
                }
            } else {
                float l_quad = st.l;
                l_quad += __shfl_xor_sync(0xffffffffu, l_quad, 1);
                l_quad += __shfl_xor_sync(0xffffffffu, l_quad, 2);
                const float m_true = st.true_max();
                if (g < group) {
                    float* dst = merge + ((size_t)warp * group + g) * pitch;
#pragma unroll
                    for (int n = 0; n < NT; ++n)
                        *reinterpret_cast<float2*>(dst + dhalf * DW + n * 8 + 2 * t) = make_float2(st.o[n][0], st.o[n][1]);
                    if (t == 0) { dst[D + 4] = st.m; dst[D + 5] = l_quad; dst[D + kMergeTrueMax] = m_true; }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(merge_bar0);
            if (!mbar_wait_bounded(merge_bar0, merge_parity & 1u, abort_word)) {
                raise_abort(abort_word, a.status, kStatusMergeTimeout);
                return;
            }
            merge_parity ^= 1u;
            VTEB_TR(tr, 6);

            if constexpr (VTEB_MERGE_PAIRS == 2 && D <= 128) {
            // Two (KV head, query row) pairs per warp pass, one per half-warp: a lane derives its pair's
            // weights from broadcast reads and merges D / 16 consecutive columns.  With 12 query heads and six
            // warps the CTA's merge is one pass instead of two.
            const bool empty = (flags & kTileEmpty) != 0;
            const int heads_item = plan.hg * group;                    // query heads of this item
            const long long stat0 = ((long long)item_b * a.num_q_heads + (long long)item_hgroup * heads_item) * a.max_chunks + item_c;
            const bool write_o = !empty || (a.flags & kFlagWriteEmptyO);
            for (int hq0 = 2 * warp; hq0 < heads_item; hq0 += 2 * plan.active_warps) {
                const int hq = hq0 + (lane >> 4), l16 = lane & 15;
                const bool pair_ok = hq < heads_item;
                const int hqc = pair_ok ? hq : hq0;                     // an idle half-warp reads the first pair's rows
                const int kvh = hqc / group, row = hqc - kvh * group;
                const float* src0 = merge + ((size_t)kvh * group + row) * pitch;        // warp (sub 0, half 0, kvh)
                const size_t hstride = (size_t)plan.hg * group * pitch;                  // same sub, next column half
                const size_t wstride = hstride * DS;                                     // next sub of the same head
                constexpr int FPL = D / 16, NV = FPL / 4;                                // floats / float4s per lane
                const int col0 = l16 * FPL;
                float mw[CW], lw[CW];            // reference maximum and sum of each warp's row
                float4 ow[CW][NV];
#pragma unroll
                for (int w = 0; w < CW; ++w) {
                    const bool on = w < plan.wph;
                    const float* src = src0 + (on ? w : 0) * wstride;
                    mw[w] = on ? src[D + 4] : kNeutralM;
                    lw[w] = on ? src[D + 5] : 0.f;
#pragma unroll
                    for (int i = 0; i < NV; ++i) {
                        const int col = col0 + 4 * i;                  // lies in column half col / DW, written by that half's warp
                        ow[w][i] = on ? *reinterpret_cast<const float4*>(src + (col / DW) * hstride + col) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
                float mm = kNeutralM;   // the rows' true maximum (with a lazy maximum the reference values lag behind it)
#pragma unroll
                for (int w = 0; w < CW; ++w) mm = fmaxf(mm, (w < plan.wph) ? src0[w * wstride + D + kMergeTrueMax] : kNeutralM);
                float ll = 0.f;
                float4 acc[NV];
#pragma unroll
                for (int i = 0; i < NV; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int w = 0; w < CW; ++w) {
                    const float wt = fast_exp2(mw[w] - mm);       // absent warps: exp2(-1e30 - mm) = 0 (or 1 * zeros)
                    ll = fmaf(lw[w], wt, ll);
#pragma unroll
                    for (int i = 0; i < NV; ++i) {
                        acc[i].x = fmaf(ow[w][i].x, wt, acc[i].x); acc[i].y = fmaf(ow[w][i].y, wt, acc[i].y);
                        acc[i].z = fmaf(ow[w][i].z, wt, acc[i].z); acc[i].w = fmaf(ow[w][i].w, wt, acc[i].w);
                    }
                }
                if (!pair_ok) continue;
                if (a.flags & kFlagDirectOutput) {
                    const long long orow = (long long)item_b * a.num_q_heads + (long long)item_hgroup * heads_item + hq;
                    const float inv = 1.f / fmaxf(ll, 1e-20f);
#pragma unroll
                    for (int i = 0; i < NV; ++i)
                        store_out4(a.output, a.out_kind, orow * D + col0 + 4 * i,
                                   make_float4(acc[i].x * inv, acc[i].y * inv, acc[i].z * inv, acc[i].w * inv));
                    continue;
                }
                const long long stat = stat0 + (long long)hq * a.max_chunks;
                if (write_o) {
#pragma unroll
                    for (int i = 0; i < NV; ++i)
                        *reinterpret_cast<float4*>(a.partial_o + stat * D + col0 + 4 * i) = acc[i];
                }
                if (l16 == 0) {
                    a.partial_m[stat] = empty ? kNeutralM : mm * kLn2;
                    a.partial_l[stat] = empty ? 0.f : ll;
                }
            }
            } else {
            // One (KV head, query row) pair per warp pass: all lanes derive the pair's
            // weights from broadcast reads, then each lane merges its float4 columns.
            const bool empty = (flags & kTileEmpty) != 0;
            const int heads_item = plan.hg * group;                    // query heads of this item
            const long long stat0 = ((long long)item_b * a.num_q_heads + (long long)item_hgroup * heads_item) * a.max_chunks + item_c;
            const bool write_o = !empty || (a.flags & kFlagWriteEmptyO);
            for (int hq = warp; hq < heads_item; hq += plan.active_warps) {
                const int kvh = hq / group, row = hq - kvh * group;
                const float* src0 = merge + ((size_t)kvh * group + row) * pitch;        // warp (sub 0, half 0, kvh)
                const size_t hstride = (size_t)plan.hg * group * pitch;                  // same sub, next column half
                const size_t wstride = hstride * DS;                                     // next sub of the same head
                constexpr int NV = (D + 127) / 128;                                      // float4 columns per lane
                const bool col_ok = (D >= 128) || lane < D / 4;
                float mw[CW], lw[CW];            // reference maximum and sum of each warp's row
                float4 ow[CW][NV];
#pragma unroll
                for (int w = 0; w < CW; ++w) {
                    const bool on = w < plan.wph;
                    const float* src = src0 + (on ? w : 0) * wstride;
                    mw[w] = on ? src[D + 4] : kNeutralM;
                    lw[w] = on ? src[D + 5] : 0.f;
#pragma unroll
                    for (int i = 0; i < NV; ++i)   // float4 group i lies in column half (i * 128) / DW, written by that half's warp
                        ow[w][i] = (on && col_ok) ? *reinterpret_cast<const float4*>(src + ((i * 128) / DW) * hstride + i * 128 + lane * 4)
                                                  : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                float mm = kNeutralM;   // the rows' true maximum (with a lazy maximum the reference values lag behind it)
#pragma unroll
                for (int w = 0; w < CW; ++w) mm = fmaxf(mm, (w < plan.wph) ? src0[w * wstride + D + kMergeTrueMax] : kNeutralM);
                float ll = 0.f;
                float4 acc[NV];
#pragma unroll
                for (int i = 0; i < NV; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int w = 0; w < CW; ++w) {
                    const float wt = fast_exp2(mw[w] - mm);       // absent warps: exp2(-1e30 - mm) = 0 (or 1 * zeros)
                    ll = fmaf(lw[w], wt, ll);
#pragma unroll
                    for (int i = 0; i < NV; ++i) {
                        acc[i].x = fmaf(ow[w][i].x, wt, acc[i].x); acc[i].y = fmaf(ow[w][i].y, wt, acc[i].y);
                        acc[i].z = fmaf(ow[w][i].z, wt, acc[i].z); acc[i].w = fmaf(ow[w][i].w, wt, acc[i].w);
                    }
                }
                if (a.flags & kFlagDirectOutput) {
                    const long long row = (long long)item_b * a.num_q_heads + (long long)item_hgroup * heads_item + hq;
                    const float inv = 1.f / fmaxf(ll, 1e-20f);
                    if (col_ok) {
#pragma unroll
                        for (int i = 0; i < NV; ++i)
                            store_out4(a.output, a.out_kind, row * D + i * 128 + lane * 4,
                                       make_float4(acc[i].x * inv, acc[i].y * inv, acc[i].z * inv, acc[i].w * inv));
                    }
                    continue;
                }
                const long long stat = stat0 + (long long)hq * a.max_chunks;
                if (write_o && col_ok) {
#pragma unroll
                    for (int i = 0; i < NV; ++i)
                        *reinterpret_cast<float4*>(a.partial_o + stat * D + i * 128 + lane * 4) = acc[i];
                }
                if (lane == 0) {
                    a.partial_m[stat] = empty ? kNeutralM : mm * kLn2;
                    a.partial_l[stat] = empty ? 0.f : ll;
                }
            }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(merge_bar0 + 8);
            merge_pending = true;
            VTEB_TR(tr, 7);
        } else {
            stage = (stage + 1 == nstages) ? 0 : stage + 1;
        }
    }

    VTEB_TR(tr, 8);
    VTEB_TR_GT(tr, 9);
#ifdef VTEB_TRACE
    if (tr.base != nullptr && lane == 0) tr.base[11] = (unsigned long long)trace_wait;
#endif
    if (kCompact || a.out_kind == 0 || (a.flags & kFlagDirectOutput)) return;
    // ===================================================================== in-launch combine
    // (needs all eight consumer warps; the host only asks for it then)
    // 1. every consumer warp's partial stores are fenced, then counted on a CTA barrier
    __threadfence();
    __syncwarp();
    if (lane == 0) mbar_arrive(bar0 + kBarFinal);
    if (!mbar_wait_bounded(bar0 + kBarFinal, 0, abort_word)) {
        raise_abort(abort_word, a.status, kStatusMergeTimeout);
        return;
    }
    // 2. one thread waits until every CTA of the grid has done the same
    volatile int* grid_ok = reinterpret_cast<volatile int*>(smem_raw + kGridOkOffset);
    if (warp == 0 && lane == 0) {
        *grid_ok = grid_barrier_bounded(a.ticket + 2, gridDim.x) ? 1 : 0;
        mbar_arrive(bar0 + kBarFinal + 8);
    }
    if (!mbar_wait_bounded(bar0 + kBarFinal + 8, 0, abort_word) || *grid_ok == 0) {
        raise_abort(abort_word, a.status, kStatusGridTimeout);
        return;
    }
    // 3. the grid's CTAs share the (sequence, head, 32-column) slices of the combine
    if (blockIdx.x == 0 && threadIdx.x == 0) *a.ticket = 0;     // work queue starts from zero next launch
    const int dsplit = D / 32;
    const int n_slices = a.batch * a.num_q_heads * dsplit;
    for (int slice = blockIdx.x; slice < n_slices; slice += gridDim.x)
        combine_slice<true>(a.partial_m, a.partial_l, a.partial_o, a.output, a.out_kind, D, a.max_chunks, dsplit, slice, merge);
}

// compact shape: the register cap (two warps per register-file partition, 5,120 registers each) is
// what leaves room for the combine launch's CTAs on the same SM
#ifndef VTEB_COMPACT_MAXNREG
#define VTEB_COMPACT_MAXNREG 160
#endif
#define VTEB_COMPACT_BOUNDS __maxnreg__(VTEB_COMPACT_MAXNREG)

#define VTEB_FAST_PARTIAL_CS(NAME, DIM, CWARPS, BOUNDS, COLSPLIT)                                     \
    extern "C" __global__ void BOUNDS NAME(                                                           \
        const __half* __restrict__ q, const __half* __restrict__ k_cache,                             \
        const __half* __restrict__ v_cache, float* __restrict__ partial_m,                            \
        float* __restrict__ partial_l, float* __restrict__ partial_o, int num_q_heads,                \
        int num_kv_heads, int head_dim, float scale, const int* __restrict__ kv_cache_offset_ptr,     \
        int kv_batch_stride, int max_chunks, int batch, int min_chunk, int flags,                     \
        const int* __restrict__ seq_order, int* __restrict__ ticket, int* __restrict__ status,        \
        const __half* __restrict__ next_k_cache, const __half* __restrict__ next_v_cache,             \
        void* __restrict__ output, int out_kind, const __grid_constant__ KvTensorMap tmap_k,          \
        const __grid_constant__ KvTensorMap tmap_v)                                                   \
    {                                                                                                 \
        FastArgs a;                                                                                   \
        a.q = q; a.k_cache = k_cache; a.v_cache = v_cache;                                            \
        a.partial_m = partial_m; a.partial_l = partial_l; a.partial_o = partial_o;                    \
        a.num_q_heads = num_q_heads; a.num_kv_heads = num_kv_heads; a.scale = scale;                  \
        a.kv_offsets = kv_cache_offset_ptr; a.kv_batch_stride = kv_batch_stride;                      \
        a.max_chunks = max_chunks; a.batch = batch; a.min_chunk = min_chunk; a.flags = flags;         \
        a.seq_order = seq_order; a.ticket = ticket; a.status = status;                                \
        a.next_k_cache = next_k_cache; a.next_v_cache = next_v_cache;                                 \
        a.output = output; a.out_kind = out_kind;                                                     \
        a.rope_cos = nullptr; a.rope_sin = nullptr; a.rope_type = 0; a.rotary_dim = 0;                \
        a.k_new = nullptr; a.v_new = nullptr;                                                         \
        a.tmap_k = &tmap_k; a.tmap_v = &tmap_v;                                                       \
        (void)head_dim;                                                                               \
        fast_partial_body<DIM, CWARPS, false, COLSPLIT>(a);                                           \
    }

// The same kernel with the Q rotation folded into the Q load: `q` is the un-rotated projection,
// four more arguments name the tables (fp16 [max_seq, head_dim], or [max_seq, rotary_dim] for
// rope_type 2), the rotation type and the rotated width.
#define VTEB_FAST_PARTIAL_ROPE(NAME, DIM, CWARPS, BOUNDS)                                             \
    extern "C" __global__ void BOUNDS NAME(                                                           \
        const __half* __restrict__ q, const __half* __restrict__ k_cache,                             \
        const __half* __restrict__ v_cache, float* __restrict__ partial_m,                            \
        float* __restrict__ partial_l, float* __restrict__ partial_o, int num_q_heads,                \
        int num_kv_heads, int head_dim, float scale, const int* __restrict__ kv_cache_offset_ptr,     \
        int kv_batch_stride, int max_chunks, int batch, int min_chunk, int flags,                     \
        const int* __restrict__ seq_order, int* __restrict__ ticket, int* __restrict__ status,        \
        const __half* __restrict__ next_k_cache, const __half* __restrict__ next_v_cache,             \
        void* __restrict__ output, int out_kind, const __grid_constant__ KvTensorMap tmap_k,          \
        const __grid_constant__ KvTensorMap tmap_v,                                                   \
        const __half* __restrict__ cos_cache, const __half* __restrict__ sin_cache,                   \
        int rope_type, int rotary_dim, const __half* __restrict__ k_new,                              \
        const __half* __restrict__ v_new)                                                             \
    {                                                                                                 \
        FastArgs a;                                                                                   \
        a.q = q; a.k_cache = k_cache; a.v_cache = v_cache;                                            \
        a.partial_m = partial_m; a.partial_l = partial_l; a.partial_o = partial_o;                    \
        a.num_q_heads = num_q_heads; a.num_kv_heads = num_kv_heads; a.scale = scale;                  \
        a.kv_offsets = kv_cache_offset_ptr; a.kv_batch_stride = kv_batch_stride;                      \
        a.max_chunks = max_chunks; a.batch = batch; a.min_chunk = min_chunk; a.flags = flags;         \
        a.seq_order = seq_order; a.ticket = ticket; a.status = status;                                \
        a.next_k_cache = next_k_cache; a.next_v_cache = next_v_cache;                                 \
        a.output = output; a.out_kind = out_kind;                                                     \
        a.rope_cos = cos_cache; a.rope_sin = sin_cache; a.rope_type = rope_type;                      \
        a.rotary_dim = rotary_dim; a.k_new = k_new; a.v_new = v_new;                                  \
        a.tmap_k = &tmap_k; a.tmap_v = &tmap_v;                                                       \
        (void)head_dim;                                                                               \
        fast_partial_body<DIM, CWARPS, true>(a);                                                      \
    }

#define VTEB_FAST_PARTIAL(NAME, DIM, CWARPS, BOUNDS) VTEB_FAST_PARTIAL_CS(NAME, DIM, CWARPS, BOUNDS, false)
VTEB_FAST_PARTIAL(vteb_split_kv_partial_d64_kernel, 64, kFullConsumerWarps, __launch_bounds__(kFullThreads, 1))
VTEB_FAST_PARTIAL(vteb_split_kv_partial_d128_kernel, 128, kFullConsumerWarps, __launch_bounds__(kFullThreads, 1))
VTEB_FAST_PARTIAL(vteb_split_kv_partial_d256_kernel, 256, kFullConsumerWarps, __launch_bounds__(kFullThreads, 1))
VTEB_FAST_PARTIAL(vteb_split_kv_partial_compact_d64_kernel, 64, kCompactConsumerWarps, VTEB_COMPACT_BOUNDS)
VTEB_FAST_PARTIAL(vteb_split_kv_partial_compact_d128_kernel, 128, kCompactConsumerWarps, VTEB_COMPACT_BOUNDS)
VTEB_FAST_PARTIAL(vteb_split_kv_partial_compact_d256_kernel, 256, kCompactConsumerWarps, VTEB_COMPACT_BOUNDS)
VTEB_FAST_PARTIAL_CS(vteb_split_kv_partial_compact_cs_d128_kernel, 128, kCompactConsumerWarps, VTEB_COMPACT_BOUNDS, true)
VTEB_FAST_PARTIAL_ROPE(vteb_split_kv_partial_rope_d64_kernel, 64, kFullConsumerWarps, __launch_bounds__(kFullThreads, 1))
VTEB_FAST_PARTIAL_ROPE(vteb_split_kv_partial_rope_d128_kernel, 128, kFullConsumerWarps, __launch_bounds__(kFullThreads, 1))
VTEB_FAST_PARTIAL_ROPE(vteb_split_kv_partial_rope_d256_kernel, 256, kFullConsumerWarps, __launch_bounds__(kFullThreads, 1))
VTEB_FAST_PARTIAL_ROPE(vteb_split_kv_partial_compact_rope_d64_kernel, 64, kCompactConsumerWarps, VTEB_COMPACT_BOUNDS)
VTEB_FAST_PARTIAL_ROPE(vteb_split_kv_partial_compact_rope_d128_kernel, 128, kCompactConsumerWarps, VTEB_COMPACT_BOUNDS)
VTEB_FAST_PARTIAL_ROPE(vteb_split_kv_partial_compact_rope_d256_kernel, 256, kCompactConsumerWarps, VTEB_COMPACT_BOUNDS)
