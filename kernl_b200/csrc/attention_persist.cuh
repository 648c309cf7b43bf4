// Fused attention forward for sm_100a, head dimension 64: PERSISTENT form of the split-row kernel.
//
// attention_split.cuh launches one CTA per 128-row query tile. A launch of one to three waves of
// such CTAs (the benchmark's [8,12,512,64]: 384 tiles on 296 CTA slots) spends about half of every
// CTA's life outside its key loop: barrier and TMEM set-up, the first Q/K/V loads arriving from
// DRAM with nothing to overlap them, the epilogue, CTA exit and the launch of the next CTA. Here a
// CTA lives for the whole launch instead (grid = min(tiles, 2 per SM)), allocates its tensor memory
// and initialises its barriers once, and pulls query tiles from a device-side queue:
//   * the first tile of a CTA is its block index; further tiles come from an atomic counter, so a
//     CTA that drew short tiles (few live key blocks behind a padding mask, early causal tiles)
//     simply draws more of them;
//   * a scheduler warp fetches the NEXT tile while the current one is being computed, stages its
//     mask row in shared memory and works out which key blocks are live; the TMA warp then loads
//     that tile's Q (second Q buffer) and starts its K/V blocks as soon as ring slots free up; the
//     tcgen05 issuer starts the next tile's Q·Kᵀ while the softmax warps are still in the epilogue
//     of the current one. Every barrier phase is a running count over the CTA's life.
// The arithmetic of a tile (64-key blocks, two threads per query row, lazy rescaling, merge of the
// two halves in the epilogue) is that of attention_split.cuh; see there for the reasons.
//
// Warps (384 threads): 0..7 softmax (0..3 first halves of the rows' key columns, 4..7 second
// halves), 8 TMA producer, 9 tcgen05 issuer, 10 scheduler, 11 idle.
// TMEM (256 columns): S ring slot s at 64·s (s = 0, 1), O_a at 128, O_b at 192.
// Shared memory: Q[2] | K ring[4] | V ring[4] | barriers | item slots[2] | (m, l) exchange[2] |
// mask rows[2] (MODE 1).
#pragma once
#include "attention_split.cuh"

namespace kb {

// Work queues. A launch takes the next slot (host-side round robin) and its CTAs draw tile numbers
// from slot[0]; slot[1] counts CTAs that have finished, and the last one puts both words back to
// zero, so a slot is clean again when its launch ends — also when the launch gave up on an expired
// wait. Two launches would have to be in flight kAttnQueueSlots launches apart to share a slot.
constexpr int kAttnQueueSlots = 1024;
__device__ unsigned int g_attn_queue[kAttnQueueSlots][2];

// Optional time stamps for tuning (compiled in with -DKB_ATTN_TRACE only): per CTA and tile, when the
// tile was published, when the softmax warps began it, when its first scores were ready, when its key
// loop and its epilogue ended (%globaltimer, ns); slot 15 of a CTA holds start, end, SM id and tiles.
#ifdef KB_ATTN_TRACE
constexpr int kTraceTiles = 15, kTraceEvents = 8;
__device__ unsigned long long g_attn_trace[296 * (kTraceTiles + 1) * kTraceEvents];
__device__ __forceinline__ unsigned long long trace_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define KB_TRACE(tile, ev, val)                                                                         \
    do {                                                                                                \
        if (blockIdx.x < 296 && (tile) <= kTraceTiles)                                                  \
            g_attn_trace[((size_t)blockIdx.x * (kTraceTiles + 1) + (tile)) * kTraceEvents + (ev)] = (val); \
    } while (0)
#else
#define KB_TRACE(tile, ev, val) do { } while (0)
#endif

struct AttnItem {   // one slot of the CTA's two-deep tile pipeline (shared memory)
    int bh;         // batch * H + head, or -1: no more tiles
    int mt;         // query tile
    int nb;         // key blocks this tile visits
    int nblk;       // key blocks up to the causal limit (before skipping)
    uint32_t act[4];  // MODE 1: live key blocks
};

struct AttnPersistCfg {
    static constexpr int D = 64;
    static constexpr int kThreads = 384;
    static constexpr int kKvStages = 4;
    static constexpr int kQTileBytes = kAttnBlock * D * 2;
    static constexpr int kKvBytes = kBlkN * D * 2;
    static constexpr int kTilesBytes = 2 * kQTileBytes + 2 * kKvStages * kKvBytes;
    static constexpr int kBarBytes = 1024;
    static constexpr int kXchBytes = 2 * 2 * kAttnBlock * 8;  // [tile parity][half][row] (m, l)
    static constexpr int kSmemBase = kTilesBytes + kBarBytes + kXchBytes + 1024;
    // two CTAs share an SM: what a CTA may use of the SM's 228 KB, less the per-CTA reservation
    static constexpr int kSmemLimit = 113 * 1024;
    static constexpr int kMaskMaxCols = (kSmemLimit - kSmemBase) / 8;  // two rows of fp32
    static constexpr int kRegsLaunch = 80, kRegsHigh = 96, kRegsLow = 48;
    static_assert(2 * kRegsHigh + kRegsLow <= 3 * kRegsLaunch, "setmaxnreg totals exceed the CTA's register pool");
};

// Stages one mask row for MODE 1: clamped, in the log2 domain, -inf beyond N (see attention_split.cuh).
// The calling warps cover the columns [first, mask_cols) in steps of `step` (both multiples of 32, so a
// warp always holds half a key block); `bits` collects, warp-uniformly, the key blocks in which this
// warp saw a value above kSkipBelow. Eight loads are in flight per thread before the first is used.
__device__ __forceinline__ void stage_mask_row(const AttnDev& p, int b, int h, float* dst, int mask_cols, int first, int step,
                                               uint32_t (&bits)[4]) {
    const float mlow = mask_lowest(p.mask_dtype);
    const int64_t moff = (int64_t)b * p.mask_strides[0] + (int64_t)h * p.mask_strides[1];
    const int lane = threadIdx.x & 31;
    if (first == 0 && step == 32 && p.mask_vec && p.mask_dtype != KB_F32 && (p.N & 7) == 0 && mask_cols <= 1536) {
        // One warp, 16-bit contiguous 16-byte-aligned row: 256 values per 128-bit load of the warp,
        // all loads (at most six) in flight at once.
        const uint16_t* row = reinterpret_cast<const uint16_t*>(p.mask) + moff;
        uint4 raw[6];
#pragma unroll
        for (int e = 0; e < 6; ++e) {
            const int col = e * 256 + lane * 8;
            raw[e] = make_uint4(0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u);
            if (col < p.N) raw[e] = __ldg(reinterpret_cast<const uint4*>(row + col));
        }
#pragma unroll
        for (int e = 0; e < 6; ++e) {
            const int col = e * 256 + lane * 8;
            if (e * 256 < mask_cols) {
                const uint32_t w4[4] = {raw[e].x, raw[e].y, raw[e].z, raw[e].w};
                float v[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = (p.mask_dtype == KB_F16) ? Elem<__half>::unpack2(w4[i]) : Elem<__nv_bfloat16>::unpack2(w4[i]);
                    v[2 * i] = f.x;
                    v[2 * i + 1] = f.y;
                }
                bool mine = false;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    v[i] = (col + i < p.N) ? fmaxf(v[i], mlow) * kLog2e : -INFINITY;
                    mine = mine || v[i] > kSkipBelow;
                }
                if (col < mask_cols) {
                    *reinterpret_cast<float4*>(dst + col) = make_float4(v[0], v[1], v[2], v[3]);
                    *reinterpret_cast<float4*>(dst + col + 4) = make_float4(v[4], v[5], v[6], v[7]);
                }
                const uint32_t ballot = __ballot_sync(0xffffffffu, mine);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int blk = e * 4 + k;
                    if ((ballot >> (8 * k)) & 0xffu) bits[blk >> 5] |= 1u << (blk & 31);
                }
            }
        }
        return;
    }
    for (int c0 = first; c0 < mask_cols; c0 += 8 * step) {
        float vals[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int col = c0 + e * step + lane;
            vals[e] = (col < p.N) ? mask_load(p.mask, moff + (int64_t)col * p.mask_strides[3], p.mask_dtype) : -INFINITY;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int col = c0 + e * step + lane;
            const float v = (col < p.N) ? fmaxf(vals[e], mlow) * kLog2e : -INFINITY;
            if (col < mask_cols) dst[col] = v;
            const bool live = __any_sync(0xffffffffu, col < p.N && v > kSkipBelow);
            const int blk = (c0 + e * step) >> 6;
            if (live && blk < 128) bits[blk >> 5] |= 1u << (blk & 31);
        }
    }
}

template <typename T, int MODE>
__global__ void __launch_bounds__(AttnPersistCfg::kThreads, 2)
attention_persist_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                         const __grid_constant__ CUtensorMap tmap_v, const AttnDev p, const int num_items,
                         const int mask_cols, unsigned int* const queue, const int sort_batches) {
    using Cfg = AttnPersistCfg;
    constexpr int D = 64;
    constexpr int KVS = Cfg::kKvStages;
    constexpr int QTILE = Cfg::kQTileBytes;
    constexpr int KVB = Cfg::kKvBytes;
    constexpr uint32_t kTmemCols = 256;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t q_smem = smem_u32(smem);
    const uint32_t k_smem = q_smem + 2 * QTILE;
    const uint32_t v_smem = k_smem + KVS * KVB;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kTilesBytes);
    const uint32_t bar_base = smem_u32(bars);
    // item_full[2] slot_free[2] q_full[2] | s_full[2] p_full[2] pv_done[2] | o_final o_free | ep[4] |
    // k_full k_empty v_full v_empty [KVS] each
    auto item_full = [&](int s) { return bar_base + 8u * (0 + s); };
    auto slot_free = [&](int s) { return bar_base + 8u * (2 + s); };
    auto q_full = [&](int s) { return bar_base + 8u * (4 + s); };
    auto s_full = [&](int bf) { return bar_base + 8u * (6 + bf); };
    auto p_full = [&](int bf) { return bar_base + 8u * (8 + bf); };
    auto pv_done = [&](int bf) { return bar_base + 8u * (10 + bf); };
    const uint32_t o_final = bar_base + 8u * 12;
    const uint32_t o_free = bar_base + 8u * 13;
    auto ep_bar = [&](int q) { return bar_base + 8u * (14 + q); };
    constexpr int kKvBar = 18;
    auto k_full = [&](int s) { return bar_base + 8u * (kKvBar + s); };
    auto k_empty = [&](int s) { return bar_base + 8u * (kKvBar + KVS + s); };
    auto v_full = [&](int s) { return bar_base + 8u * (kKvBar + 2 * KVS + s); };
    auto v_empty = [&](int s) { return bar_base + 8u * (kKvBar + 3 * KVS + s); };
    const uint32_t near_end = bar_base + 8u * (kKvBar + 4 * KVS);  // the issuer has issued a tile's last Q·Kᵀ
    constexpr int kNumBars = kKvBar + 4 * KVS + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    AttnItem* items = reinterpret_cast<AttnItem*>(tmem_slot + 4);  // two slots
    uint32_t* warp_bits = reinterpret_cast<uint32_t*>(items + 2);  // [12 warps][4]: live blocks of the first tile, per staging warp
    int* batch_order = reinterpret_cast<int*>(warp_bits + 12 * 4);  // [32]: batches, longest first (sort_batches)
    int* setup_issued = batch_order + 32;  // K/V blocks of the first tile that the set-up has requested already
    static_assert(kNumBars * 8 + 16 + 2 * sizeof(AttnItem) + 12 * 16 + 32 * 4 + 4 <= Cfg::kBarBytes, "barrier area too small");
    float2* xch = reinterpret_cast<float2*>(smem + Cfg::kTilesBytes + Cfg::kBarBytes);
    float* mask_smem = reinterpret_cast<float*>(smem + Cfg::kTilesBytes + Cfg::kBarBytes + Cfg::kXchBytes);  // [2][mask_cols]
    // sort_batches: [12 warps][32 batches] live-block words, in the (not yet used) second mask row
    uint32_t* warp_live = reinterpret_cast<uint32_t*>(mask_smem + mask_cols);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef KB_ATTN_TRACE
    if (threadIdx.x == 0) {
        unsigned smid;
        asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
        KB_TRACE(kTraceTiles, 0, trace_now());
        KB_TRACE(kTraceTiles, 2, (unsigned long long)smid);
    }
#endif
    // A wait that expired in an earlier launch leaves the status word set: such a launch does no
    // work. The word is read here and looked at after the set-up barrier, so that its latency
    // overlaps the set-up instead of preceding it.
    __shared__ int s_skip;
    int status_early = 0;
    if (threadIdx.x == 0 || threadIdx.x == 8 * 32) status_early = *reinterpret_cast<volatile int*>(&g_device_status[0]);

    const int BH = p.B * p.H;
    const int num_n_blocks = (p.N + kBlkN - 1) / kBlkN;
    // tile number -> (batch*head, query tile): the CTA order of the one-tile-per-CTA kernel
    // (attn_work_item: L2-sized head groups, late query tiles first), as a function of the number
    auto locate = [&](int idx, int& bh, int& mt) {
        const int per_group = p.num_pairs * p.head_group;
        const int g = idx / per_group, rem = idx % per_group;
        const int first = g * p.head_group;
        const int gsz = min(p.head_group, BH - first);
        mt = p.num_pairs - 1 - rem / gsz;
        bh = first + rem % gsz;
    };
    // With sort_batches the batch part of a tile number counts batches from the longest (most live
    // key blocks behind its padding mask) to the shortest, so the tiles that CTAs start with are the
    // long ones and those drawn from the queue later are the short ones: the launch ends with
    // little work left per CTA instead of a long tile that somebody started late.
    auto locate_sorted = [&](int idx, int& bh, int& mt) {
        if (!sort_batches) {
            locate(idx, bh, mt);
            return;
        }
        // batch-major: all tiles of the longest batch, then of the next one, ...; inside a batch
        // the heads of one query tile are neighbours (they share no K/V, but a batch's K/V of all
        // heads is small next to L2)
        const int per_batch = p.H * p.num_pairs;
        const int r = idx / per_batch, rem = idx % per_batch;
        mt = p.num_pairs - 1 - rem / p.H;
        bh = batch_order[r] * p.H + rem % p.H;
    };
    // The CTA's first tile is its block index: known without the queue, so its operands are
    // requested during set-up and its mask row is staged by all threads at once.
    int bh0, mt0;
    locate((int)blockIdx.x, bh0, mt0);
    const int nblk0 = p.is_causal ? min(num_n_blocks, (mt0 + 1) * (kAttnBlock / kBlkN)) : num_n_blocks;
    // MODE 1 does not know which key blocks it will visit before the mask has been looked at: it
    // only pulls the first ring of K/V blocks into L2 during set-up
    constexpr int kFirstBurst = 1;  // K/V blocks requested together with Q during set-up
    const int first_kv = (MODE == 1) ? 0 : min(kFirstBurst, nblk0);
    const bool early_q = !(MODE == 1 && sort_batches);  // sorted: the first tile is known after the scan only (requested there)

    {
        if (warp == 8) {
            if (lane == 0) {
                tma_prefetch_desc(&tmap_q);
                tma_prefetch_desc(&tmap_k);
                tma_prefetch_desc(&tmap_v);
                for (int s = 0; s < 2; ++s) {
                    mbar_init(item_full(s), 1);
                    mbar_init(slot_free(s), 9);  // eight softmax warps + the issuer's last Q·Kᵀ of the tile
                    mbar_init(q_full(s), 1);
                }
                for (int s = 0; s < KVS; ++s) {
                    mbar_init(k_full(s), 1);
                    mbar_init(k_empty(s), 1);
                    mbar_init(v_full(s), 1);
                    mbar_init(v_empty(s), 1);
                }
                mbar_init(near_end, 1);
                fence_mbar_init();
                pdl_wait();  // q/k/v may be the output of the kernel before this one
              if (status_early == 0 && early_q) {
                const int b0 = bh0 / p.H, h0 = bh0 % p.H, hk0 = h0 / p.kv_group;
                mbar_arrive_expect_tx(q_full(0), QTILE);
                tma_load_4d(q_smem, &tmap_q, q_full(0), 0, mt0 * kAttnBlock, h0, b0);
                if (MODE == 1) {
                    for (int j = 0; j < min(KVS, nblk0); ++j) {
                        tma_prefetch_l2_4d(&tmap_k, 0, j * kBlkN, hk0, b0);
                        tma_prefetch_l2_4d(&tmap_v, 0, j * kBlkN, hk0, b0);
                    }
                }
                for (int j = 0; j < first_kv; ++j) {
                    mbar_arrive_expect_tx(k_full(j), KVB);
                    tma_load_4d(k_smem + j * KVB, &tmap_k, k_full(j), 0, j * kBlkN, hk0, b0);
                    mbar_arrive_expect_tx(v_full(j), KVB);
                    tma_load_4d(v_smem + j * KVB, &tmap_v, v_full(j), 0, j * kBlkN, hk0, b0);
                }
              }
            }
        } else if (warp == 0) {
            if (lane < 2) {
                mbar_init(s_full(lane), 1);
                mbar_init(p_full(lane), 8);
                mbar_init(pv_done(lane), 1);
            }
            if (lane == 2) mbar_init(o_final, 1);
            if (lane == 3) mbar_init(o_free, 8);
            if (lane >= 4 && lane < 8) mbar_init(ep_bar(lane - 4), 2);
            if (lane == 0) {
                *abort_flag = 0;
                s_skip = status_early;
            }
            fence_mbar_init();
        } else if (warp == 9) {
            tmem_alloc(smem_u32(tmem_slot), kTmemCols);
            tmem_relinquish();
        }
    }
    // Launched with programmatic dependent launch: everything above may run while the previous
    // kernel of the stream drains; nothing of global memory is touched before this point (the TMA
    // thread has made the same wait before its loads).
    pdl_wait();
#ifdef KB_ATTN_TRACE
    if (threadIdx.x == 0) KB_TRACE(kTraceTiles, 3, trace_now());
#endif
    if (MODE == 1 && !sort_batches) {
        // every warp stages its share of the first tile's mask row and leaves the key blocks it
        // found live in its own slot; the scheduler combines the slots after the barrier
        uint32_t bits[4] = {0u, 0u, 0u, 0u};
        stage_mask_row(p, bh0 / p.H, bh0 % p.H, mask_smem, mask_cols, warp * 32, Cfg::kThreads, bits);
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (lane == i) warp_bits[warp * 4 + i] = bits[i];
    }
    if (MODE == 1 && sort_batches) {
        // All batches' mask rows (the mask is the same for every head and query row): which key
        // blocks of each are live. The rows are 16-bit, contiguous and 16-byte aligned (checked by
        // the host), so a warp reads 256 values — four key blocks of one batch — per 128-bit load;
        // warp w takes the 256-value pieces w, w + 12, ... and keeps what it saw in its own row of
        // warp_live (at most 32 batches of at most 32 key blocks).
        warp_live[warp * 32 + lane] = 0u;
        __syncwarp();
        const float mlow_s = mask_lowest(p.mask_dtype);
        constexpr int kW = Cfg::kThreads / 32;
        constexpr int kRounds = 4;  // 12 warps x 4 rounds x 256 values = 12288 >= B x mask_cols
        const int pieces_per_row = (mask_cols + 255) >> 8;
        const int pieces = p.B * pieces_per_row;
        uint4 vals[kRounds];
#pragma unroll
        for (int r = 0; r < kRounds; ++r) {
            const int pc = warp + r * kW;
            const int bb = pc / pieces_per_row, col = (pc % pieces_per_row) * 256 + lane * 8;
            vals[r] = make_uint4(0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u, 0xfc00fc00u);  // -inf in fp16; very negative in bf16
            if (pc < pieces && col < p.N)
                vals[r] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.mask) + (int64_t)bb * p.mask_strides[0] + col));
        }
#pragma unroll
        for (int r = 0; r < kRounds; ++r) {
            const int pc = warp + r * kW;
            const int bb = pc / pieces_per_row, blk0 = (pc % pieces_per_row) * 4;
            const uint32_t w4[4] = {vals[r].x, vals[r].y, vals[r].z, vals[r].w};
            bool mine = false;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = (p.mask_dtype == KB_F16) ? Elem<__half>::unpack2(w4[i]) : Elem<__nv_bfloat16>::unpack2(w4[i]);
                mine = mine || f.x * kLog2e > kSkipBelow || f.y * kLog2e > kSkipBelow;
            }
            const uint32_t ballot = __ballot_sync(0xffffffffu, mine);
            if (lane == 0 && pc < pieces) {
                uint32_t bits = 0u;
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    if ((ballot >> (8 * k)) & 0xffu) bits |= 1u << (blk0 + k);
                warp_live[warp * 32 + bb] |= bits;
            }
        }
        // Every warp now ranks the batches (longest first, ties by number) for itself, which tells
        // it the batch of this CTA's first tile; the threads that hold that batch's mask values put
        // them into mask slot 0, and the TMA thread requests the tile's Q and first K/V blocks —
        // nobody reads the mask from memory a second time or waits for the scheduler warp.
        __syncthreads();
        uint32_t w = 0u;
#pragma unroll
        for (int ww = 0; ww < kW; ++ww) w |= warp_live[ww * 32 + lane];
        const int len = (lane < p.B) ? (w != 0u ? __popc(w) : num_n_blocks) : -1;
        int rank = 0;
        for (int o = 0; o < 32; ++o) {
            const int other = __shfl_sync(0xffffffffu, len, o);
            rank += (other > len || (other == len && o < lane)) ? 1 : 0;
        }
        if (warp == 10 && lane < p.B) batch_order[rank] = lane;  // the scheduler warp keeps the table for the later tiles
        const int per_batch = p.H * p.num_pairs;
        // A grid of two CTAs per SM: CTA c and CTA c + grid/2 usually share an SM (the block scheduler
        // fills every SM once before it doubles up), so the second half takes its tiles in reverse —
        // the SM that runs the longest tile also gets the shortest of the statically assigned ones,
        // and the work per SM is even (8 + 3, 7 + 4, ... key blocks instead of 8 + 5, ..., 5 + 3).
        // Only a heuristic for balance: any placement computes every tile exactly once.
        const int half = (int)gridDim.x >> 1;
        const int first_idx = ((gridDim.x & 1) == 0 && (int)blockIdx.x >= half) ? (int)gridDim.x - 1 - ((int)blockIdx.x - half)
                                                                              : (int)blockIdx.x;
        const int r0 = first_idx / per_batch, rem0 = first_idx % per_batch;
        const int b0 = __ffs((int)__ballot_sync(0xffffffffu, lane < p.B && rank == r0)) - 1;
        const uint32_t live0 = __shfl_sync(0xffffffffu, w, b0);
#pragma unroll
        for (int r = 0; r < kRounds; ++r) {
            const int pc = warp + r * kW;
            const int bb = pc / pieces_per_row, col = (pc % pieces_per_row) * 256 + lane * 8;
            if (pc < pieces && bb == b0 && col < mask_cols) {
                const uint32_t w4[4] = {vals[r].x, vals[r].y, vals[r].z, vals[r].w};
                float v[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = (p.mask_dtype == KB_F16) ? Elem<__half>::unpack2(w4[i]) : Elem<__nv_bfloat16>::unpack2(w4[i]);
                    v[2 * i] = f.x;
                    v[2 * i + 1] = f.y;
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = (col + i < p.N) ? fmaxf(v[i], mlow_s) * kLog2e : -INFINITY;
                *reinterpret_cast<float4*>(mask_smem + col) = make_float4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<float4*>(mask_smem + col + 4) = make_float4(v[4], v[5], v[6], v[7]);
            }
        }
        if (warp == 8 && lane == 0) {
            int issued = 0;
            if (status_early == 0) {
                const int mt_s = p.num_pairs - 1 - rem0 / p.H, h_s = rem0 % p.H, hk_s = h_s / p.kv_group;
                const uint32_t act_s[4] = {live0 != 0u ? live0 : 0xffffffffu, live0 != 0u ? 0u : 0xffffffffu,
                                           live0 != 0u ? 0u : 0xffffffffu, live0 != 0u ? 0u : 0xffffffffu};
                const int nb_s = bits_count_below(act_s, num_n_blocks);
                mbar_arrive_expect_tx(q_full(0), QTILE);
                tma_load_4d(q_smem, &tmap_q, q_full(0), 0, mt_s * kAttnBlock, h_s, b0);
                int jb = bits_next(act_s, 0);
                // Only the first key block with Q: all CTAs start at once, and what they ask for in this
                // burst is served at DRAM speed — Q and the first K decide when the first scores
                // exist; the other blocks of the ring follow from the producer loop right after the
                // barrier (21.5 -> 21.05 µs on the headline shape; leaving V of the first block to the
                // producer loop as well was slightly worse: 21.2 µs).
                for (; issued < min(kFirstBurst, nb_s); ++issued) {
                    mbar_arrive_expect_tx(k_full(issued), KVB);
                    tma_load_4d(k_smem + issued * KVB, &tmap_k, k_full(issued), 0, jb * kBlkN, hk_s, b0);
                    mbar_arrive_expect_tx(v_full(issued), KVB);
                    tma_load_4d(v_smem + issued * KVB, &tmap_v, v_full(issued), 0, jb * kBlkN, hk_s, b0);
                    jb = bits_next(act_s, jb + 1);
                }
            }
            *setup_issued = issued;
        }
        if (warp == 10 && lane == 0) {
            // the first tile is complete as far as the scheduler is concerned: publish it here, so
            // that nobody waits for the scheduler warp to get going after the barrier
            const bool any_live = live0 != 0u;
            AttnItem* item = &items[0];
            item->bh = b0 * p.H + rem0 % p.H;
            item->mt = p.num_pairs - 1 - rem0 / p.H;
            item->act[0] = any_live ? live0 : 0xffffffffu;
            item->act[1] = item->act[2] = item->act[3] = any_live ? 0u : 0xffffffffu;
            item->nblk = num_n_blocks;
            item->nb = any_live ? __popc(live0) : num_n_blocks;
            mbar_arrive(item_full(0));
        }
    }
    if (!(MODE == 1 && sort_batches) && warp == 8 && lane == 0) *setup_issued = first_kv;
#ifdef KB_ATTN_TRACE
    if (threadIdx.x == 0) KB_TRACE(kTraceTiles, 4, trace_now());
#endif
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
#ifdef KB_ATTN_TRACE
    if (threadIdx.x == 0) KB_TRACE(kTraceTiles, 5, trace_now());
#endif

    const bool skip = s_skip != 0;
    if (!skip) {
      const uint32_t tmem_base = *tmem_slot;
      if (warp >= 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Cfg::kRegsLow));
        if (warp == 10) {
            // -------------------------------------------------------------- scheduler (whole warp)
            bool ok = true;
#ifdef KB_ATTN_TRACE
            if (lane == 0) KB_TRACE(kTraceTiles, 6, trace_now());
#endif
            for (int it = (MODE == 1 && sort_batches) ? 1 : 0; ok; ++it) {  // (sorted: the first tile was published during set-up)
                const int slot = it & 1;
                // The next tile is drawn only once the current one is two key blocks from its end (its
                // last Q·Kᵀ has been issued; scores run two blocks ahead of the softmax): a CTA that is
                // busy with a long tile must not reserve another one that an idle CTA could have started
                // at once. Two blocks and the epilogue are enough to stage the next tile behind them.
                if (it >= 1) {
                    if (!mbar_wait(near_end, (uint32_t)((it - 1) & 1), abort_flag, 701)) { ok = false; break; }
                }
                int idx = 0;
                if (lane == 0) idx = (it == 0) ? (int)blockIdx.x : (int)gridDim.x + (int)atomicAdd(&queue[0], 1u);
                idx = __shfl_sync(0xffffffffu, idx, 0);
                if (it >= 2) {  // the slot's previous tile (it - 2) has been read to the end by everybody
                    if (!mbar_wait(slot_free(slot), (uint32_t)(((it >> 1) - 1) & 1), abort_flag, 700)) { ok = false; break; }
                }
                AttnItem* item = &items[slot];
                if (idx >= num_items) {
                    __syncwarp();
                    if (lane == 0) {
                        item->bh = -1;
                        mbar_arrive(item_full(slot));
                    }
                    pdl_launch_dependents();  // this CTA draws no more tiles: a dependent launch may take the slots that free up
                    break;
                }
                int bh, mt;
                locate_sorted(idx, bh, mt);
                const int nblk = p.is_causal ? min(num_n_blocks, (mt + 1) * (kAttnBlock / kBlkN)) : num_n_blocks;
                uint32_t act[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
                int nb = nblk;
                if (MODE == 1) {
                    uint32_t bits[4] = {0u, 0u, 0u, 0u};
                    if (it == 0 && !sort_batches) {  // staged by the whole CTA during set-up
                        for (int w = 0; w < Cfg::kThreads / 32; ++w) {
#pragma unroll
                            for (int i = 0; i < 4; ++i) bits[i] |= warp_bits[w * 4 + i];
                        }
                    } else {
                        stage_mask_row(p, bh / p.H, bh % p.H, mask_smem + slot * mask_cols, mask_cols, 0, 32, bits);
                    }
                    // Nothing is skipped when the whole row is masked (the reference then returns a
                    // plain softmax), nor for causal calls (a row's prefix may hold masked keys only).
                    if ((bits[0] | bits[1] | bits[2] | bits[3]) != 0u && !p.is_causal) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) act[i] = bits[i];
                    }
                    nb = bits_count_below(act, nblk);
                }
                __syncwarp();
#ifdef KB_ATTN_TRACE
                if (lane == 0 && it == 0) KB_TRACE(kTraceTiles, 7, trace_now());
#endif
                if (lane == 0) {
                    item->bh = bh;
                    item->mt = mt;
                    item->nb = nb;
                    item->nblk = nblk;
#pragma unroll
                    for (int i = 0; i < 4; ++i) item->act[i] = act[i];
                    mbar_arrive(item_full(slot));  // release: the mask row and the item are visible to who waits
#ifdef KB_ATTN_TRACE
                    KB_TRACE(it, 0, trace_now());
                    KB_TRACE(it, 5, (unsigned long long)nb);
                    KB_TRACE(it, 6, (unsigned long long)idx);
#endif
                }
            }
        } else if (warp == 8) {
            // -------------------------------------------------------------- TMA producer
            if (elect_one()) {
                bool ok = true;
                int kv_i = 0;  // K/V ring position, running over the CTA's life
                for (int it = 0; ok; ++it) {
                    const int slot = it & 1;
                    if (!mbar_wait(item_full(slot), (uint32_t)((it >> 1) & 1), abort_flag, 710)) { ok = false; break; }
                    const AttnItem item = items[slot];
                    if (item.bh < 0) break;
                    const int b = item.bh / p.H, h = item.bh % p.H, hk = h / p.kv_group;
                    int i = 0;
                    int jb = (MODE == 1) ? bits_next(item.act, 0) : 0;
                    if (it == 0) {
                        // Q and the first blocks of the first tile were requested during set-up
                        const int done = *setup_issued;
                        for (; i < done; ++i) jb = (MODE == 1) ? bits_next(item.act, jb + 1) : jb + 1;
                        kv_i = done;
                    } else {
                        // the scheduler has waited for slot_free: Q buffer `slot` is no longer read
                        mbar_arrive_expect_tx(q_full(slot), QTILE);
                        tma_load_4d(q_smem + slot * QTILE, &tmap_q, q_full(slot), 0, item.mt * kAttnBlock, h, b);
                    }
                    for (; i < item.nb; ++i, ++kv_i) {
                        const int s = kv_i % KVS;
                        const uint32_t ph = (uint32_t)((kv_i / KVS) & 1);
                        if (!mbar_wait(k_empty(s), ph ^ 1, abort_flag, 711)) { ok = false; break; }
                        mbar_arrive_expect_tx(k_full(s), KVB);
                        tma_load_4d(k_smem + s * KVB, &tmap_k, k_full(s), 0, jb * kBlkN, hk, b);
                        if (!mbar_wait(v_empty(s), ph ^ 1, abort_flag, 712)) { ok = false; break; }
                        mbar_arrive_expect_tx(v_full(s), KVB);
                        tma_load_4d(v_smem + s * KVB, &tmap_v, v_full(s), 0, jb * kBlkN, hk, b);
                        jb = (MODE == 1) ? bits_next(item.act, jb + 1) : jb + 1;
                    }
                }
                if (!ok) {
                    for (int i = 0; i < 64; ++i) __nanosleep(2000);  // let copies in flight land before the CTA retires
                }
            }
        } else if (warp == 9) {
            // -------------------------------------------------------------- tcgen05 issuer
            if (elect_one()) {
                constexpr uint32_t idesc_qk = make_idesc_f16(Elem<T>::kIsBf16, 128, kBlkN, 0, 0);
                constexpr uint32_t idesc_pv = make_idesc_f16(Elem<T>::kIsBf16, 128, D, 0, 1);
                constexpr uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
                const uint32_t k_lo = (k_smem & 0x3FFFF) >> 4;
                const uint32_t v_lo = (v_smem & 0x3FFFF) >> 4;
                auto desc = [&](uint32_t lo) { return ((uint64_t)desc_hi << 32) | (uint64_t)lo; };
                bool ok = true;
                int g = 0;     // key blocks issued so far (S ring position and barrier phases)
                int kv_i = 0;  // K/V ring position of the current tile's first block
                for (int it = 0; ok; ++it) {
                    const int slot = it & 1;
                    if (!mbar_wait(item_full(slot), (uint32_t)((it >> 1) & 1), abort_flag, 719)) { ok = false; break; }
                    const int nb = items[slot].nb;
                    if (items[slot].bh < 0) break;
                    if (!mbar_wait(q_full(slot), (uint32_t)((it >> 1) & 1), abort_flag, 720)) { ok = false; break; }
                    const uint32_t q_lo = ((q_smem + slot * QTILE) & 0x3FFFF) >> 4;
                    auto issue_qk = [&](int j) {  // S[(g + j) & 1] = Q · K_jᵀ
                        const uint32_t b_lo = k_lo + (uint32_t)(((kv_i + j) % KVS) * (KVB >> 4));
                        const uint32_t d_tmem = tmem_base + (uint32_t)(((g + j) & 1) * kBlkN);
#pragma unroll
                        for (int ks = 0; ks < D / 16; ++ks)
                            tc_mma_ss(d_tmem, desc(q_lo + (uint32_t)((ks * 32) >> 4)), desc(b_lo + (uint32_t)((ks * 32) >> 4)), idesc_qk,
                                      ks > 0 ? 1u : 0u);
                        tc_commit(s_full((g + j) & 1));
                        tc_commit(k_empty((kv_i + j) % KVS));
                        if (j + 1 == nb) {
                            tc_commit(slot_free(slot));  // the tile's last read of its Q buffer
                            mbar_arrive(near_end);
                        }
                    };
                    auto issue_pv = [&](int j) {  // O_a += P_j[:, 0:32] · V_j[0:32, :],  O_b += P_j[:, 32:64] · V_j[32:64, :]
                        const uint32_t b_lo = v_lo + (uint32_t)(((kv_i + j) % KVS) * (KVB >> 4));
                        const uint32_t s_tmem = tmem_base + (uint32_t)(((g + j) & 1) * kBlkN);
#pragma unroll
                        for (int hf = 0; hf < 2; ++hf) {
#pragma unroll
                            for (int ks = 0; ks < 2; ++ks) {
                                tc_mma_ts(tmem_base + (uint32_t)(128 + hf * 64), s_tmem + (uint32_t)(hf * 32 + ks * 8),
                                          desc(b_lo + (uint32_t)((hf * 2 + ks) * (2048 >> 4))), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
                            }
                        }
                    };
                    // scores run two blocks ahead of the softmax; the first two of a tile are issued
                    // while the softmax warps are still in the previous tile's epilogue
                    for (int jj = 0; jj < 2 && jj < nb && ok; ++jj) {
                        const int kr = kv_i + jj;
                        if (!mbar_wait(k_full(kr % KVS), (uint32_t)((kr / KVS) & 1), abort_flag, 721)) { ok = false; break; }
                        tc_fence_after();
                        issue_qk(jj);
                    }
                    for (int j = 0; j < nb && ok; ++j) {
                        const int kr = kv_i + j;
                        if (!mbar_wait(v_full(kr % KVS), (uint32_t)((kr / KVS) & 1), abort_flag, 722)) { ok = false; break; }
                        const int j2 = j + 2;
                        if (j2 < nb) {
                            if (!mbar_wait(k_full((kv_i + j2) % KVS), (uint32_t)(((kv_i + j2) / KVS) & 1), abort_flag, 723)) { ok = false; break; }
                        }
                        if (!mbar_wait(p_full((g + j) & 1), (uint32_t)(((g + j) >> 1) & 1), abort_flag, 724)) { ok = false; break; }
                        if (j == 0 && it > 0) {  // the previous tile's epilogue has read O out of tensor memory
                            if (!mbar_wait(o_free, (uint32_t)((it - 1) & 1), abort_flag, 725)) { ok = false; break; }
                        }
                        tc_fence_after();
                        issue_pv(j);
                        tc_commit(pv_done((g + j) & 1));
                        if (j2 < nb) issue_qk(j2);  // into the slot that P_j has just been read from (in-order execution)
                        if (j + 1 == nb) tc_commit(o_final);
                        tc_commit(v_empty(kr % KVS));
                    }
                    g += nb;
                    kv_i += nb;
                }
            }
        }
      } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Cfg::kRegsHigh));
        // ------------------------------------------------------------------ softmax warps
        const int hf = (warp >> 2) & 1;  // which 32 key columns of every block
        const int q = warp & 3;          // TMEM lane quarter = 32 query rows
        const int r_in_tile = q * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        const uint32_t o_own = lane_addr + (uint32_t)(128 + hf * 64);
        const float c = p.scale_log2;
        const float mlow = mask_lowest(p.mask_dtype);
        const float unit = (MODE == 0) ? c : 1.0f;
        bool ok = true;
        int g = 0;  // key blocks seen so far
        for (int it = 0; ok; ++it) {
            const int slot = it & 1;
            if (!mbar_wait(item_full(slot), (uint32_t)((it >> 1) & 1), abort_flag, 730)) { ok = false; break; }
            const int bh = items[slot].bh;
            if (bh < 0) break;
#ifdef KB_ATTN_TRACE
            if (threadIdx.x == 0) KB_TRACE(it, 1, trace_now());
#endif
            const int mt = items[slot].mt, nb = items[slot].nb;
            uint32_t act[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) act[i] = (MODE == 1) ? items[slot].act[i] : 0xffffffffu;
            const int b = bh / p.H, h = bh % p.H;
            const int row = mt * kAttnBlock + r_in_tile;
            const float* mask_row = mask_smem + slot * mask_cols;
            const int64_t mask_row_off =
                (MODE == 2 && p.mask != nullptr)
                    ? (int64_t)b * p.mask_strides[0] + (int64_t)h * p.mask_strides[1] + (int64_t)min(row, p.M - 1) * p.mask_strides[2]
                    : 0;
            float m_ref = -INFINITY;
            float l = 0.f;
            int jb = (MODE == 1) ? bits_next(act, 0) : 0;  // key-block number of visit j
            for (int j = 0; j < nb; ++j, jb = (MODE == 1) ? bits_next(act, jb + 1) : jb + 1) {
                const int gj = g + j;
                const int bf = gj & 1;
                const uint32_t ph = (uint32_t)((gj >> 1) & 1);
                const uint32_t s_addr = lane_addr + (uint32_t)(bf * kBlkN + hf * 32);
                if (!mbar_wait(s_full(bf), ph, abort_flag, 731)) { ok = false; break; }
#ifdef KB_ATTN_TRACE
                if (threadIdx.x == 0 && j == 0) KB_TRACE(it, 2, trace_now());
                if (threadIdx.x == 0 && it == 0 && j < 8) KB_TRACE(kTraceTiles - 1, j, trace_now());  // row 14: scores of block j of the first tile ready
#endif
                tc_fence_after();
                uint32_t sr[32];
                tmem_ld_32x32(s_addr, sr);
                tmem_ld_wait();

                const int col0 = jb * kBlkN + hf * 32;
                if (MODE == 1) {
                    const float4* ms = reinterpret_cast<const float4*>(mask_row + col0);
#pragma unroll
                    for (int v4 = 0; v4 < 8; ++v4) {
                        const float4 a = ms[v4];
                        sr[v4 * 4 + 0] = __float_as_uint(fmaf(__uint_as_float(sr[v4 * 4 + 0]), c, a.x));
                        sr[v4 * 4 + 1] = __float_as_uint(fmaf(__uint_as_float(sr[v4 * 4 + 1]), c, a.y));
                        sr[v4 * 4 + 2] = __float_as_uint(fmaf(__uint_as_float(sr[v4 * 4 + 2]), c, a.z));
                        sr[v4 * 4 + 3] = __float_as_uint(fmaf(__uint_as_float(sr[v4 * 4 + 3]), c, a.w));
                    }
                } else if (MODE == 2) {
                    if (p.mask == nullptr) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) sr[i] = __float_as_uint(__uint_as_float(sr[i]) * c);
                    } else {
#pragma unroll
                        for (int hc = 0; hc < 2; ++hc) {
                            const int colc = col0 + hc * 16;
                            float mvals[16];
                            if (p.mask_vec && colc + 16 <= p.N) {
                                if (p.mask_dtype == KB_F32) {
                                    const float4* mp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.mask) + mask_row_off + colc);
#pragma unroll
                                    for (int v4 = 0; v4 < 4; ++v4) {
                                        const float4 f = __ldg(mp + v4);
                                        mvals[v4 * 4 + 0] = f.x; mvals[v4 * 4 + 1] = f.y; mvals[v4 * 4 + 2] = f.z; mvals[v4 * 4 + 3] = f.w;
                                    }
                                } else {
                                    const uint4* mp = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.mask) + mask_row_off + colc);
#pragma unroll
                                    for (int v4 = 0; v4 < 2; ++v4) {
                                        const uint4 w = __ldg(mp + v4);
                                        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                                        for (int i = 0; i < 4; ++i) {
                                            const float2 f = (p.mask_dtype == KB_F16) ? Elem<__half>::unpack2(ww[i]) : Elem<__nv_bfloat16>::unpack2(ww[i]);
                                            mvals[v4 * 8 + 2 * i] = f.x;
                                            mvals[v4 * 8 + 2 * i + 1] = f.y;
                                        }
                                    }
                                }
                            } else {
#pragma unroll
                                for (int i = 0; i < 16; ++i) {
                                    const int col = colc + i;
                                    mvals[i] = (col < p.N) ? mask_load(p.mask, mask_row_off + (int64_t)col * p.mask_strides[3], p.mask_dtype) : 0.f;
                                }
                            }
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                uint32_t& sv = sr[hc * 16 + i];
                                sv = __float_as_uint(fmaf(fmaxf(mvals[i], mlow), kLog2e, __uint_as_float(sv) * c));
                            }
                        }
                    }
                }
                const bool causal_edge = p.is_causal && col0 + 31 > mt * kAttnBlock;
                if ((MODE != 1 && col0 + 32 > p.N) || causal_edge) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int col = col0 + i;
                        if (col >= p.N || (p.is_causal && col > row)) sr[i] = __float_as_uint(-INFINITY);
                    }
                }
                float m4[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) m4[i] = fmaxf(__uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1]));
#pragma unroll
                for (int i = 4; i < 16; ++i) m4[i & 3] = fmax3(m4[i & 3], __uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1]));
                const float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
                float m_new = fmaxf(m_ref, mx);
                if (m_new == -INFINITY) m_new = 0.f;
                const bool grow = (m_new - m_ref) * unit > kLazyThreshold;
                float alpha = 1.0f;
                if (grow) {
                    alpha = (m_ref == -INFINITY) ? 0.f : fast_exp2((m_ref - m_new) * unit);
                    m_ref = m_new;
                    l *= alpha;
                }
                if (j > 0 && __any_sync(0xffffffffu, grow)) {
                    // this half's accumulator must be quiescent before it is rescaled: P·V of the
                    // previous block (ring position gj - 1) complete
                    if (!mbar_wait(pv_done((gj - 1) & 1), (uint32_t)(((gj - 1) >> 1) & 1), abort_flag, 732)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int dch = 0; dch < D / 16; ++dch) {
                        uint32_t orr[16];
                        tmem_ld_32x16(o_own + dch * 16, orr);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
                        tmem_st_32x16(o_own + dch * 16, orr);
                    }
                }
                const float neg_ref = -m_ref * unit;
                const float2 unit2 = make_float2(unit, unit);
                const float2 neg2 = make_float2(neg_ref, neg_ref);
                float2 lp[2] = {{0.f, 0.f}, {0.f, 0.f}};
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float2 a = __ffma2_rn(make_float2(__uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1])), unit2, neg2);
                    float2 e;
                    e.x = fast_exp2(a.x);
                    e.y = fast_exp2(a.y);
                    lp[i & 1] = __fadd2_rn(lp[i & 1], e);
                    pk[i] = Elem<T>::pack2(e.x, e.y);
                }
                tmem_st_32x16(s_addr, pk);
                {
                    const float2 st = __fadd2_rn(lp[0], lp[1]);
                    l += st.x + st.y;
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full(bf));
            }
            if (!ok) break;
            g += nb;
#ifdef KB_ATTN_TRACE
            if (threadIdx.x == 0) KB_TRACE(it, 3, trace_now());
#endif
            // the key loop is over: this warp no longer reads the slot's mask row or item
            __syncwarp();
            if (lane == 0) mbar_arrive(slot_free(slot));
            // ---- epilogue: merge the two halves of every row, O / l -> global
            // a half that never saw a finite score (all of its columns beyond N) must not set the scale
            const float m_own = (l > 0.f) ? m_ref * unit : -INFINITY;
            float2* xrow = xch + (it & 1) * 2 * kAttnBlock;
            xrow[hf * kAttnBlock + r_in_tile] = make_float2(m_own, l);
            __syncwarp();
            if (lane == 0) mbar_arrive(ep_bar(q));
            const uint32_t tph = (uint32_t)(it & 1);
            if (!(mbar_wait(ep_bar(q), tph, abort_flag, 733) && mbar_wait(o_final, tph, abort_flag, 734))) { ok = false; break; }
            tc_fence_after();
            const float2 other = xrow[(hf ^ 1) * kAttnBlock + r_in_tile];
            float m_all = fmaxf(m_own, other.x);
            if (m_all == -INFINITY) m_all = 0.f;
            const float w_own = fast_exp2(m_own - m_all), w_oth = fast_exp2(other.x - m_all);
            const float inv_l = 1.0f / (w_own * l + w_oth * other.y);
            const float wa = (hf == 0 ? w_own : w_oth) * inv_l;  // weight of O_a
            const float wb = (hf == 0 ? w_oth : w_own) * inv_l;  // weight of O_b
            // this warp writes output columns [32·hf, 32·hf + 32) of its 32 rows
            uint32_t oa[32], ob[32];
            tmem_ld_32x32(lane_addr + (uint32_t)(128 + hf * 32), oa);
            tmem_ld_32x32(lane_addr + (uint32_t)(192 + hf * 32), ob);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(o_free);  // the issuer may overwrite O with the next tile's first P·V
            T* o_row = reinterpret_cast<T*>(p.o) + (int64_t)b * p.o_strides[0] + (int64_t)h * p.o_strides[1] +
                       (int64_t)row * p.o_strides[2];
            const bool vec = p.o_strides[3] == 1 && ((((uintptr_t)o_row) & 15) == 0);
            if (row < p.M) {
                float val[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) val[i] = fmaf(__uint_as_float(oa[i]), wa, __uint_as_float(ob[i]) * wb);
                if (hf * 32 + 32 <= p.d_out) attn_store_32<T, false>(o_row, hf * 32, p.o_strides[3], vec, val, p.d_out);
                else attn_store_32<T, true>(o_row, hf * 32, p.o_strides[3], vec, val, p.d_out);
            }
#ifdef KB_ATTN_TRACE
            if (threadIdx.x == 0) KB_TRACE(it, 4, trace_now());
#endif
        }
      }
    }

    tc_fence_before();
    __syncthreads();
    if (!skip && warp == 9) {
        __syncwarp();
        tmem_dealloc(*tmem_slot, kTmemCols);
    }
#ifdef KB_ATTN_TRACE
    if (threadIdx.x == 0) KB_TRACE(kTraceTiles, 1, trace_now());
#endif
    // every CTA reports in, also one that did no work; the last one leaves the queue slot clean
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&queue[1], 1u) == gridDim.x - 1) {
            queue[0] = 0u;
            queue[1] = 0u;
            __threadfence();
        }
    }
}

// Whether the persistent kernel serves a call: a launch of more tiles than CTA slots (otherwise
// every CTA would draw one tile and the queue buys nothing), and for row-broadcast masks a mask
// row short enough for two of them to sit in shared memory next to two CTAs' tiles.
static int attention_persist_mask_cols(int64_t N) {  // one staged mask row: whole key blocks, in steps of 128 values
    const int64_t blocks = (N + kBlkN - 1) / kBlkN;
    return (int)(((blocks * kBlkN + 127) / 128) * 128);
}

static bool attention_persist_applicable(const kb_attn_params& p, int mode) {
    const int64_t tiles = ((p.M + kAttnBlock - 1) / kAttnBlock) * p.B * p.H;
    if (g_attn_persistent == 0) return false;
    if (mode == 1 && (p.N > 8192 || attention_persist_mask_cols(p.N) > AttnPersistCfg::kMaskMaxCols)) return false;
    if (tiles > 0x3fffffff) return false;
    if (g_attn_persistent == 1) return true;
    return tiles > 2 * (int64_t)sm_count();
}

static int g_attn_sort_batches = 1;  // test hook (kb_debug_attention_persistent: bit 1 of the mode switches it off)

// The next queue slot on the current device. g_attn_queue is a host-side handle; its device address
// is looked up once per device (with that device current) and kept.
static unsigned int* attention_queue_slot() {
    static unsigned int* base[64] = {};
    static std::mutex mu;
    static std::atomic<unsigned> next_slot{0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (base[dev] == nullptr) {
            void* ptr = nullptr;
            if (cudaGetSymbolAddress(&ptr, g_attn_queue) != cudaSuccess || ptr == nullptr) {
                cudaGetLastError();
                return nullptr;
            }
            base[dev] = reinterpret_cast<unsigned int*>(ptr);
        }
    }
    return base[dev] + 2 * (next_slot.fetch_add(1) % (unsigned)kAttnQueueSlots);
}

template <typename T, int MODE>
static int launch_attention_persist_tm(const kb_attn_params& p, cudaStream_t stream) {
    using Cfg = AttnPersistCfg;
    constexpr int D = 64;
    CUtensorMap tq, tk, tv;
    const int64_t kv_group = p.kv_group > 1 ? p.kv_group : 1;
    if (p.H % kv_group != 0) return KB_ERR_BAD_ARG;
    auto enc = [&](CUtensorMap* out, const void* ptr, int64_t rows, const int64_t* st, uint32_t box_rows, int64_t heads) -> int {
        if (st[3] != 1) return KB_ERR_UNSUPPORTED;
        const uint64_t dims[4] = {(uint64_t)p.D, (uint64_t)rows, (uint64_t)heads, (uint64_t)p.B};  // the box reaches to 64: zero fill
        auto fix = [](int64_t extent, int64_t stride) -> uint64_t { return (extent == 1) ? 16u : (uint64_t)stride * 2u; };
        const uint64_t strides[4] = {0, fix(rows, st[2]), fix(heads, st[1]), fix(p.B, st[0])};
        const uint32_t box[4] = {64, box_rows, 1, 1};
        return encode_tmap_16bit(out, ptr, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    };
    int st = enc(&tq, p.q, p.M, p.q_strides, kAttnBlock, p.H);
    if (st != KB_OK) return st;
    st = enc(&tk, p.k, p.N, p.k_strides, kBlkN, p.H / kv_group);
    if (st != KB_OK) return st;
    st = enc(&tv, p.v, p.N, p.v_strides, kBlkN, p.H / kv_group);
    if (st != KB_OK) return st;

    AttnDev d;
    d.o = p.o;
    d.mask = p.mask;
    for (int i = 0; i < 4; ++i) {
        d.o_strides[i] = p.o_strides[i];
        d.mask_strides[i] = p.mask ? p.mask_strides[i] : 0;
    }
    d.B = (int)p.B; d.H = (int)p.H; d.M = (int)p.M; d.N = (int)p.N;
    d.scale_log2 = p.sm_scale * kLog2e;
    d.is_causal = p.is_causal ? 1 : 0;
    d.mask_dtype = p.mask ? p.mask_dtype : KB_F32;
    d.mask_vec = 0;
    if (p.mask != nullptr && p.mask_strides[3] == 1 && (((uintptr_t)p.mask) & 15) == 0) {
        const int64_t per16 = (p.mask_dtype == KB_F32) ? 4 : 8;
        d.mask_vec = (p.mask_strides[0] % per16 == 0 && p.mask_strides[1] % per16 == 0 && p.mask_strides[2] % per16 == 0) ? 1 : 0;
    }
    d.num_pairs = (int)((p.M + kAttnBlock - 1) / kAttnBlock);  // query tiles per (batch, head)
    d.head_group = attn_head_group(p.B * p.H, p.N, p.D);
    d.kv_group = (int)kv_group;
    d.d_out = (int)p.D;
    static int regs_ok = 0;  // 0 = not checked, 1 = usable, -1 = register allocation does not fit
    if (regs_ok == 0) {
        // setmaxnreg.inc blocks until the CTA's pool holds the registers: refuse to launch a build
        // whose launch allocation is smaller than the redistribution assumes.
        cudaFuncAttributes fa;
        if (cudaFuncGetAttributes(&fa, attention_persist_kernel<T, MODE>) != cudaSuccess) return KB_ERR_LAUNCH;
        regs_ok = (fa.numRegs < Cfg::kRegsLaunch) ? -1 : 1;
    }
    if (regs_ok < 0) return KB_ERR_UNSUPPORTED;
    const int mask_cols = MODE == 1 ? attention_persist_mask_cols(p.N) : 0;
    const size_t smem_bytes = (size_t)Cfg::kSmemBase + (size_t)mask_cols * 8;
    static PerDeviceOnce attr_once;
    if (attr_once.first_time()) {
        // two CTAs of up to 113 KB share an SM: that needs the largest shared-memory carve-out
        if (cudaFuncSetAttribute(attention_persist_kernel<T, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg::kSmemLimit) != cudaSuccess ||
            cudaFuncSetAttribute(attention_persist_kernel<T, MODE>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 (int)cudaSharedmemCarveoutMaxShared) != cudaSuccess)
            return KB_ERR_LAUNCH;
    }
    if (smem_bytes > (size_t)Cfg::kSmemLimit) return KB_ERR_UNSUPPORTED;
    const int64_t tiles = (int64_t)d.num_pairs * p.B * p.H;
    const int64_t grid = tiles < 2 * (int64_t)sm_count() ? tiles : 2 * (int64_t)sm_count();
    unsigned int* queue = attention_queue_slot();
    if (queue == nullptr) return KB_ERR_LAUNCH;
    // Longest-first order of the batches: for padding masks (one row per batch, shared by heads and
    // query rows) of a size that every CTA can scan during its set-up.
    const int sort_batches = (MODE == 1 && g_attn_sort_batches && !p.is_causal && p.mask_strides[1] == 0 && p.mask_strides[0] != 0 &&
                              p.B > 1 && p.B <= 32 && mask_cols >= 384 && mask_cols <= 2048 &&
                              p.B * (int64_t)((mask_cols + 255) / 256) <= 48 &&  // what twelve warps scan in four loads each
                              (p.mask_dtype == KB_F16 || p.mask_dtype == KB_BF16) && p.mask_strides[3] == 1 && p.N % 8 == 0 &&
                              p.mask_strides[0] % 8 == 0 && (((uintptr_t)p.mask) & 15) == 0)
                                 ? 1 : 0;
    if (launch_pdl(attention_persist_kernel<T, MODE>, (unsigned)grid, (unsigned)Cfg::kThreads, smem_bytes, stream, tq, tk, tv, d,
                   (int)tiles, mask_cols, queue, sort_batches) != cudaSuccess)
        return KB_ERR_LAUNCH;
    return cudaGetLastError() == cudaSuccess ? KB_OK : KB_ERR_LAUNCH;
}

}  // namespace kb
