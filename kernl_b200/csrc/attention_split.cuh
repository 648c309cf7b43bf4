// Fused attention forward for sm_100a, head dimension 64, "split-row" variant.
//
// Two 128-row query tiles per CTA, keys in blocks of 64, K/V through an 8-stage TMA ring, one
// tcgen05 issuer warp per tile, and SIXTEEN softmax warps: every query row is shared by two
// threads of different warps, one owning key columns
// [0,32) of each block, the other [32,64). The two halves never talk to each other inside the key
// loop: each keeps its own running maximum and row sum, writes its own half of P, and its P·V goes
// into its own accumulator in TMEM (O_a from the keys of the first halves, O_b from the second
// halves; two K=32 tcgen05.mma chains instead of one K=64 chain, the same tensor-core work). The
// halves are merged once, in the epilogue: O = (w_a·O_a + w_b·O_b) / (w_a·l_a + w_b·l_b) with
// w_x = 2^(m_x - max(m_a, m_b)).
//
// Why: a softmax warp's block is a serial chain of fixed latencies (barrier poll, TMEM load, the
// dependent maximum reduction, special-function-unit results, TMEM store, hand-off) that one warp
// cannot overlap with itself, and with one row per thread there are only two such warps per SM
// sub-partition. Clock stamps taken inside the kernel showed a block taking ~2200 cycles of which
// the special-function unit was busy for 512. Four warps per sub-partition overlap those chains.
//
// Warps (640 threads): 0..7 tile 0 (0..3 first halves, 4..7 second halves), 8..15 tile 1,
// 16 TMA producer, 17/18 tcgen05 issuers of tile 0/1, 19 mask loader (MODE 1).
// TMEM columns per tile t (base 256·t): S ring slot s at 64·s (s = 0,1; 64 fp32 columns; P of the
// first half overwrites columns [0,16), P of the second half columns [32,48) of the same slot),
// O_a at 128, O_b at 192.
#pragma once
#include "attention.cuh"

namespace kb {

// TILES = 2: the CTA described above (640 threads, all 512 TMEM columns, one CTA per SM). TILES = 1:
// half of it (one query tile, 8 softmax warps + TMA + one issuer = 384 threads, 256 TMEM columns, a
// 4-stage K/V ring), so that TWO CTAs share an SM. A launch that is only one or two waves of
// two-tile CTAs spends a third of its time in per-CTA fixed costs (set-up, first loads from DRAM,
// epilogue, exit) with the SM idle; with two independent CTAs per SM one CTA's fixed costs overlap
// the other's key loop, and the second wave starts per tile, not per pair. Measured faster at every
// launch size, so TILES = 1 is what the dispatcher picks; TILES = 2 loads K/V once for two tiles.
template <int TILES>
struct SplitShape {
    static constexpr int kThreads = TILES * 256 + 128;
    static constexpr int kAuxWarp = TILES * 8;  // first non-softmax warp: TMA producer; issuers follow
    static constexpr int kRegsLaunch = TILES == 2 ? 96 : 80;  // 65536 / 640 and 65536 / (2 x 384), rounded down to 8
    static constexpr int kRegsHigh = TILES == 2 ? 104 : 96;
    static constexpr int kRegsLow = TILES == 2 ? 64 : 48;
    static_assert(TILES * 2 * kRegsHigh + kRegsLow <= (TILES * 2 + 1) * kRegsLaunch, "setmaxnreg totals exceed the CTA's register pool");
    static_assert(kRegsHigh % 8 == 0 && kRegsLow % 8 == 0, "setmaxnreg wants multiples of 8");
};
static int g_split_tiles = 0;  // test hook: 0 = by launch size, 1 / 2 = force the number of query tiles per CTA
static int g_attn_persistent = -1;  // test hook: -1 = dispatcher's choice, 0 = one CTA per tile, 1 = persistent CTAs

// 2^x for a pair of x <= 0 on the FMA pipe (no special-function unit): x = r + f with r = round(x),
// f in [-0.5, 0.5]; 2^f by a cubic (max relative error 7.5e-5, below the rounding of a 16-bit P);
// 2^r by adding r to the exponent field. The magic constant 1.5 * 2^23 makes the fp32 adder do the
// rounding and leaves r in the low mantissa bits of the sum. Inputs below -126 (masked keys are -inf)
// are clamped and come out as 2^-126 * 2^f, which the 16-bit conversion flushes to zero.
__device__ __forceinline__ float2 exp2_poly_pair(float2 x) {
    x.x = fmaxf(x.x, -126.0f);
    x.y = fmaxf(x.y, -126.0f);
    const float2 fl = __fadd2_rn(x, make_float2(12582912.0f, 12582912.0f));
    const float2 r = __fadd2_rn(fl, make_float2(-12582912.0f, -12582912.0f));
    const float2 f = __ffma2_rn(r, make_float2(-1.0f, -1.0f), x);
    float2 pl = __ffma2_rn(make_float2(0.05517137795686722f, 0.05517137795686722f), f,
                           make_float2(0.24261121451854706f, 0.24261121451854706f));
    pl = __ffma2_rn(pl, f, make_float2(0.6932610273361206f, 0.6932610273361206f));
    pl = __ffma2_rn(pl, f, make_float2(0.9999280571937561f, 0.9999280571937561f));
    float2 out;
    out.x = __uint_as_float(__float_as_uint(pl.x) + (__float_as_uint(fl.x) << 23));
    out.y = __uint_as_float(__float_as_uint(pl.y) + (__float_as_uint(fl.y) << 23));
    return out;
}
// Which pairs of a block go to the FMA pipe: bit (i & 3) of this mask, i = pair index. The
// special-function unit evaluates 16 exponentials per clock per SM, which at head dimension 64
// is twice the time the tensor core needs for the same block, so moving some of them looked
// promising; measured on B200 (B8 H12 S4096 fp16) it is not: 0/4 of the pairs 0.571 ms, 1/4 0.591,
// 2/4 0.596, 3/4 0.669. The softmax warps are bound by their own dependent instruction stream, and
// the polynomial adds eleven instructions per pair. Kept switchable, off by default.
#ifndef KB_POLY_MASK
#define KB_POLY_MASK 0x0u
#endif
constexpr unsigned kPolyPairMask = KB_POLY_MASK;
// Key blocks of a MODE 1 launch whose mask is "minus infinity" for every key (the padding behind a
// sequence) contribute exp(-65504 + ...) = 0 to every row and are skipped: not loaded, not multiplied,
// not exponentiated. A block is skipped only if all of its mask values are below kSkipBelow (in the
// log2 domain), far beyond where fp32 exp underflows for any score difference up to 2^14; if the
// whole row is like that (a fully padded sequence, where the mask cancels and the reference
// returns a plain softmax) nothing is skipped. At most 128 blocks (N <= 8192): a 128-bit set.
constexpr float kSkipBelow = -30000.0f * 1.4426950408889634f;
__device__ __forceinline__ int bits_next(const uint32_t (&w)[4], int from) {  // smallest set bit >= from
    int r = 1 << 20;
#pragma unroll
    for (int wi = 3; wi >= 0; --wi) {
        uint32_t m = w[wi];
        const int lo = from - wi * 32;
        if (lo >= 32) m = 0u;
        else if (lo > 0) m &= 0xffffffffu << lo;
        if (m != 0u) r = wi * 32 + __ffs((int)m) - 1;
    }
    return r;
}
__device__ __forceinline__ int bits_count_below(const uint32_t (&w)[4], int limit) {  // set bits with index < limit
    int n = 0;
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
        const int hi = limit - wi * 32;
        uint32_t m = w[wi];
        if (hi <= 0) m = 0u;
        else if (hi < 32) m &= (1u << hi) - 1u;
        n += __popc(m);
    }
    return n;
}
__device__ __forceinline__ void tma_prefetch_l2_4d(const CUtensorMap* map, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(
                     reinterpret_cast<uint64_t>(map)),
                 "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}

template <int TILES>
struct AttnSplitCfgT {
    static constexpr int D = 64;
    static constexpr int kKvStages = TILES == 2 ? 8 : 4;
    static constexpr int kQTileBytes = kAttnBlock * D * 2;
    static constexpr int kKvBytes = kBlkN * D * 2;
    static constexpr int kTilesBytes = TILES * kQTileBytes + 2 * kKvStages * kKvBytes;
    static constexpr int kBarBytes = 1024;
    static constexpr int kXchBytes = 2 * 2 * kAttnBlock * 8;  // [tile][half][row] (m, l)
    // MODE 1 keeps the whole row-broadcast mask of its (batch, head) in shared memory, as fp32 in the
    // log2 domain, staged by all threads during set-up; longer rows take the general path (MODE 2)
    static constexpr int kMaskMaxN = 8192;
    static constexpr int kMaskLoads = (kMaskMaxN + SplitShape<TILES>::kThreads - 1) / SplitShape<TILES>::kThreads;  // per thread
    static constexpr int kSmemBase = kTilesBytes + kBarBytes + kXchBytes + 1024;
    static constexpr int kSmemMax = kSmemBase + kMaskMaxN * 4;
};

using AttnSplitCfg = AttnSplitCfgT<2>;

template <typename T, int MODE, int TILES>
__global__ void __launch_bounds__(SplitShape<TILES>::kThreads, TILES == 2 ? 1 : 2)
attention_split_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v, const AttnDev p) {
    using Cfg = AttnSplitCfgT<TILES>;
    using Shape = SplitShape<TILES>;
    constexpr int kThreads = Shape::kThreads;
    constexpr int W0 = Shape::kAuxWarp;
    constexpr int D = 64;
    constexpr int KVS = Cfg::kKvStages;
    constexpr int QTILE = Cfg::kQTileBytes;
    constexpr int KVB = Cfg::kKvBytes;
    constexpr int NB = 2;
    constexpr uint32_t kTmemCols = TILES * 256;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t q_smem = smem_u32(smem);
    const uint32_t k_smem = q_smem + TILES * QTILE;
    const uint32_t v_smem = k_smem + KVS * KVB;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kTilesBytes);
    const uint32_t bar_base = smem_u32(bars);
    // q_full[2] | o_final[2] | p_full, s_full, pv_done [2][2] each | ep[2][4] |
    // k_full, k_empty, v_full, v_empty [KVS] each
    auto q_full = [&](int t) { return bar_base + 8u * t; };
    auto o_final = [&](int t) { return bar_base + 8u * (2 + t); };
    auto p_full = [&](int t, int bf) { return bar_base + 8u * (4 + t * NB + bf); };
    auto s_full = [&](int t, int bf) { return bar_base + 8u * (8 + t * NB + bf); };
    auto pv_done = [&](int t, int bf) { return bar_base + 8u * (12 + t * NB + bf); };
    auto ep_bar = [&](int t, int q) { return bar_base + 8u * (16 + t * 4 + q); };
    constexpr int kKvBar = 24;
    auto k_full = [&](int s) { return bar_base + 8u * (kKvBar + s); };
    auto k_empty = [&](int s) { return bar_base + 8u * (kKvBar + KVS + s); };
    auto v_full = [&](int s) { return bar_base + 8u * (kKvBar + 2 * KVS + s); };
    auto v_empty = [&](int s) { return bar_base + 8u * (kKvBar + 3 * KVS + s); };
    constexpr int kNumBars = kKvBar + 4 * KVS;
    static_assert(kNumBars * 8 + 32 <= Cfg::kBarBytes, "barrier area too small");
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    uint32_t* act_bits = tmem_slot + 4;  // MODE 1: which key blocks have at least one unmasked key
    float2* xch = reinterpret_cast<float2*>(smem + Cfg::kTilesBytes + Cfg::kBarBytes);
    float* mask_smem = reinterpret_cast<float*>(smem + Cfg::kTilesBytes + Cfg::kBarBytes + Cfg::kXchBytes);  // [N rounded up to 64]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    {
        __shared__ int s_skip;
        if (threadIdx.x == 0) s_skip = *reinterpret_cast<volatile int*>(&g_device_status[0]);
        if (MODE == 1 && threadIdx.x < 4) act_bits[threadIdx.x] = 0u;
        __syncthreads();
        if (s_skip != 0) return;
    }

    const int BH = p.B * p.H;
    int bh, pair;
    attn_work_item(p, BH, bh, pair);
    const int b = bh / p.H, h = bh % p.H;
    const int hk = h / p.kv_group;  // K/V head of this query head
    const int num_m_tiles = (p.M + kAttnBlock - 1) / kAttnBlock;
    const int num_n_blocks = (p.N + kBlkN - 1) / kBlkN;
    int mt[2], nblk[2];
    int ntl = 0;
    for (int t = 0; t < 2; ++t) {
        mt[t] = pair * TILES + t;
        if (t < TILES && mt[t] < num_m_tiles) {
            ntl = t + 1;
            nblk[t] = p.is_causal ? min(num_n_blocks, (mt[t] + 1) * (kAttnBlock / kBlkN)) : num_n_blocks;
        } else {
            nblk[t] = 0;
        }
    }
    const int max_blk = max(nblk[0], nblk[1]);

    // Set-up is spread over three warps so that the first loads are in flight as early as possible:
    // the TMA warp initialises the barriers its loads complete on and issues both Q tiles and the
    // first ring of K/V blocks at once; warp 0 initialises the other barriers, one per lane; warp 17
    // allocates TMEM. Everybody else meets them at the barrier below.
    // MODE 1 does not know which key blocks it will visit before the mask has been looked at: it
    // only pulls the first ring of K/V blocks into L2 and issues the real loads after the set-up barrier.
    const int first_kv = (MODE == 1) ? 0 : min(KVS, max_blk);
    if (warp == W0) {
        if (lane == 0) {
            tma_prefetch_desc(&tmap_q);
            tma_prefetch_desc(&tmap_k);
            tma_prefetch_desc(&tmap_v);
            for (int t = 0; t < 2; ++t) mbar_init(q_full(t), 1);
            for (int s = 0; s < KVS; ++s) {
                mbar_init(k_full(s), 1);
                mbar_init(k_empty(s), ntl);  // one arrival per live tile's issuer
                mbar_init(v_full(s), 1);
                mbar_init(v_empty(s), ntl);
            }
            fence_mbar_init();
            pdl_wait();  // q/k/v may be the output of the kernel before this one
            for (int t = 0; t < ntl; ++t) {
                mbar_arrive_expect_tx(q_full(t), QTILE);
                tma_load_4d(q_smem + t * QTILE, &tmap_q, q_full(t), 0, mt[t] * kAttnBlock, h, b);
                if (MODE == 1 && t == 0) {
                    for (int j = 0; j < min(KVS, max_blk); ++j) {
                        tma_prefetch_l2_4d(&tmap_k, 0, j * kBlkN, hk, b);
                        tma_prefetch_l2_4d(&tmap_v, 0, j * kBlkN, hk, b);
                    }
                }
                if (t == 0 && first_kv > 0) {  // K_0 right behind the first Q tile: the first Q·Kᵀ needs just these two
                    mbar_arrive_expect_tx(k_full(0), KVB);
                    tma_load_4d(k_smem, &tmap_k, k_full(0), 0, 0, hk, b);
                }
            }
            for (int j = 0; j < first_kv; ++j) {
                if (j > 0) {
                    mbar_arrive_expect_tx(k_full(j), KVB);
                    tma_load_4d(k_smem + j * KVB, &tmap_k, k_full(j), 0, j * kBlkN, hk, b);
                }
                mbar_arrive_expect_tx(v_full(j), KVB);
                tma_load_4d(v_smem + j * KVB, &tmap_v, v_full(j), 0, j * kBlkN, hk, b);
            }
        }
    } else if (warp == 0) {
        if (lane < 2) mbar_init(o_final(lane), 1);
        if (lane < 4) {
            mbar_init(p_full(lane >> 1, lane & 1), 8);
            mbar_init(s_full(lane >> 1, lane & 1), 1);
            mbar_init(pv_done(lane >> 1, lane & 1), 1);
        }
        if (lane < 8) mbar_init(ep_bar(lane >> 2, lane & 3), 2);
        if (lane == 0) *abort_flag = 0;
        fence_mbar_init();
    } else if (warp == W0 + 1) {
        tmem_alloc(smem_u32(tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    // Launched with programmatic dependent launch: everything above (barriers, TMEM, descriptors)
    // may run while the previous kernel of the stream drains; nothing of global memory is touched
    // before this point.
    pdl_wait();
    if (MODE == 1) {
        // every thread stages its share of the mask row: clamped, in the log2 domain, -inf beyond N
        const float mlow = mask_lowest(p.mask_dtype);
        const int64_t moff = (int64_t)b * p.mask_strides[0] + (int64_t)h * p.mask_strides[1];
        const int ncols = max_blk * kBlkN;
        float vals[Cfg::kMaskLoads];
#pragma unroll
        for (int e = 0; e < Cfg::kMaskLoads; ++e) {
            const int col = e * kThreads + (int)threadIdx.x;
            vals[e] = (col < p.N && col < ncols) ? mask_load(p.mask, moff + (int64_t)col * p.mask_strides[3], p.mask_dtype) : -INFINITY;
        }
#pragma unroll
        for (int e = 0; e < Cfg::kMaskLoads; ++e) {
            const int col = e * kThreads + (int)threadIdx.x;  // a warp covers half of one key block
            if (e * kThreads < ncols) {
                const bool inside = col < p.N && col < ncols;
                const float v = inside ? fmaxf(vals[e], mlow) * kLog2e : -INFINITY;
                if (col < ncols) mask_smem[col] = v;
                const bool live = __any_sync(0xffffffffu, inside && v > kSkipBelow);
                if (live && lane == 0) atomicOr(&act_bits[col >> 11], 1u << ((col >> 6) & 31));
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // the key blocks this CTA visits: all of them, or (MODE 1) those with an unmasked key
    uint32_t act[4] = {0u, 0u, 0u, 0u};
    int n_union = max_blk, n_tile[2] = {nblk[0], nblk[1]};
    if (MODE == 1) {
#pragma unroll
        for (int i = 0; i < 4; ++i) act[i] = act_bits[i];
        // Causal rows see a prefix of the keys, which may consist of masked keys only even when the
        // row as a whole has live ones: no skipping then.
        if ((act[0] | act[1] | act[2] | act[3]) == 0u || p.is_causal) {
#pragma unroll
            for (int i = 0; i < 4; ++i) act[i] = 0xffffffffu;
        }
        n_union = bits_count_below(act, max_blk);
        n_tile[0] = bits_count_below(act, nblk[0]);
        n_tile[1] = bits_count_below(act, nblk[1]);
    }
    auto next_blk = [&](int from) { return MODE == 1 ? bits_next(act, from) : from; };

    if (warp >= W0) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Shape::kRegsLow));
      if (warp == W0) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one()) {
            bool ok = true;
            int jb = next_blk(first_kv);
            for (int i = first_kv; i < n_union && ok; ++i) {  // (MODE 0/2: the first ring was issued during set-up)
                const int s = i % KVS;
                const uint32_t ph = (uint32_t)((i / KVS) & 1);
                if (!mbar_wait(k_empty(s), ph ^ 1, abort_flag, 600)) { ok = false; break; }
                mbar_arrive_expect_tx(k_full(s), KVB);
                tma_load_4d(k_smem + s * KVB, &tmap_k, k_full(s), 0, jb * kBlkN, hk, b);
                if (!mbar_wait(v_empty(s), ph ^ 1, abort_flag, 601)) { ok = false; break; }
                mbar_arrive_expect_tx(v_full(s), KVB);
                tma_load_4d(v_smem + s * KVB, &tmap_v, v_full(s), 0, jb * kBlkN, hk, b);
                jb = next_blk(jb + 1);
            }
            if (!ok) {
                for (int i = 0; i < 64; ++i) __nanosleep(2000);
            }
        }
      } else if (warp >= W0 + 1 && warp <= W0 + TILES) {
        // ------------------------------------------------------------------ MMA issuers, one per tile
        const int t = warp - (W0 + 1);
        if (elect_one()) {
            constexpr uint32_t idesc_qk = make_idesc_f16(Elem<T>::kIsBf16, 128, kBlkN, 0, 0);
            constexpr uint32_t idesc_pv = make_idesc_f16(Elem<T>::kIsBf16, 128, D, 0, 1);
            constexpr uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
            const uint32_t q_lo = ((q_smem + t * QTILE) & 0x3FFFF) >> 4;
            const uint32_t k_lo = (k_smem & 0x3FFFF) >> 4;
            const uint32_t v_lo = (v_smem & 0x3FFFF) >> 4;
            const uint32_t t_base = tmem_base + (uint32_t)(t * 256);
            auto desc = [&](uint32_t lo) { return ((uint64_t)desc_hi << 32) | (uint64_t)lo; };
            auto issue_qk = [&](int j) {  // S[t][j & 1] = Q_t · K_jᵀ
                const uint32_t b_lo = k_lo + (uint32_t)((j % KVS) * (KVB >> 4));
                const uint32_t d_tmem = t_base + (uint32_t)((j & 1) * kBlkN);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    tc_mma_ss(d_tmem, desc(q_lo + (uint32_t)((ks * 32) >> 4)), desc(b_lo + (uint32_t)((ks * 32) >> 4)), idesc_qk,
                              ks > 0 ? 1u : 0u);
            };
            auto issue_pv = [&](int j) {  // O_a += P_j[:, 0:32] · V_j[0:32, :],  O_b += P_j[:, 32:64] · V_j[32:64, :]
                const uint32_t b_lo = v_lo + (uint32_t)((j % KVS) * (KVB >> 4));
                const uint32_t s_tmem = t_base + (uint32_t)((j & 1) * kBlkN);
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
#pragma unroll
                    for (int ks = 0; ks < 2; ++ks) {
                        tc_mma_ts(t_base + (uint32_t)(128 + hf * 64), s_tmem + (uint32_t)(hf * 32 + ks * 8),
                                  desc(b_lo + (uint32_t)((hf * 2 + ks) * (2048 >> 4))), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
                    }
                }
            };
            // j below counts visited blocks (ring positions), not key-block numbers; a tile's blocks are
            // a prefix of the CTA's visit list (causal tiles stop early)
            const int my_blk = (t < ntl) ? n_tile[t] : 0;
            const int max_blk = n_union;
            bool ok = true;
            if (t < ntl && !mbar_wait(q_full(t), 0, abort_flag, 610)) ok = false;
            for (int jj = 0; jj < NB && jj < max_blk && ok && t < ntl; ++jj) {
                if (!mbar_wait(k_full(jj % KVS), (uint32_t)((jj / KVS) & 1), abort_flag, 611)) { ok = false; break; }
                if (jj < my_blk) {
                    tc_fence_after();
                    issue_qk(jj);
                    tc_commit(s_full(t, jj & 1));
                    tc_commit(k_empty(jj % KVS));
                } else {
                    mbar_arrive(k_empty(jj % KVS));  // a block this tile does not need (shorter causal range)
                }
            }
            for (int j = 0; j < max_blk && ok && t < ntl; ++j) {
                const int s = j % KVS;
                if (!mbar_wait(v_full(s), (uint32_t)((j / KVS) & 1), abort_flag, 612)) { ok = false; break; }
                const int j2 = j + NB;
                if (j2 < max_blk) {
                    if (!mbar_wait(k_full(j2 % KVS), (uint32_t)((j2 / KVS) & 1), abort_flag, 613)) { ok = false; break; }
                }
                if (j < my_blk) {
                    if (!mbar_wait(p_full(t, j & 1), (uint32_t)((j >> 1) & 1), abort_flag, 614)) { ok = false; break; }
                    tc_fence_after();
                    issue_pv(j);
                    tc_commit(pv_done(t, j & 1));
                    if (j2 < my_blk) {
                        issue_qk(j2);  // into the slot that P_j has just been read from (in-order execution)
                        tc_commit(s_full(t, j & 1));
                    }
                    if (j + 1 == my_blk) tc_commit(o_final(t));
                    tc_commit(v_empty(s));
                    if (j2 < max_blk) {
                        if (j2 < my_blk) tc_commit(k_empty(j2 % KVS));
                        else mbar_arrive(k_empty(j2 % KVS));
                    }
                } else {
                    mbar_arrive(v_empty(s));
                    if (j2 < max_blk) mbar_arrive(k_empty(j2 % KVS));
                }
            }
        }
      }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Shape::kRegsHigh));
        // ------------------------------------------------------------------ softmax warps
        const int t = warp >> 3;
        const int hf = (warp >> 2) & 1;  // which 32 key columns of every block
        const int q = warp & 3;          // TMEM lane quarter = 32 query rows
        if (t < ntl && nblk[t] > 0) {
            const int nb = n_tile[t];
            const int r_in_tile = q * 32 + lane;
            const int row = mt[t] * kAttnBlock + r_in_tile;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(t * 256);
            const uint32_t o_own = lane_addr + (uint32_t)(128 + hf * 64);
            const float c = p.scale_log2;
            const float mlow = mask_lowest(p.mask_dtype);
            const int64_t mask_row_off =
                (MODE == 2 && p.mask != nullptr)
                    ? (int64_t)b * p.mask_strides[0] + (int64_t)h * p.mask_strides[1] + (int64_t)min(row, p.M - 1) * p.mask_strides[2]
                    : 0;
            const float unit = (MODE == 0) ? c : 1.0f;
            float m_ref = -INFINITY;
            float l = 0.f;
            bool ok = true;
            int jb = next_blk(0);  // key-block number of visit j
            for (int j = 0; j < nb; ++j, jb = next_blk(jb + 1)) {
                const int bf = j & 1;
                const uint32_t ph = (uint32_t)((j >> 1) & 1);
                const uint32_t s_addr = lane_addr + (uint32_t)(bf * kBlkN + hf * 32);
                if (!mbar_wait(s_full(t, bf), ph, abort_flag, 630 + t)) { ok = false; break; }
                tc_fence_after();
                uint32_t sr[32];
                tmem_ld_32x32(s_addr, sr);
                tmem_ld_wait();

                const int col0 = jb * kBlkN + hf * 32;
                if (MODE == 1) {
                    const float4* ms = reinterpret_cast<const float4*>(mask_smem + col0);
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
                const bool causal_edge = p.is_causal && col0 + 31 > mt[t] * kAttnBlock;
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
                    // This half's accumulator must be quiescent before it is rescaled: P·V of block j-1
                    // complete, the ((j-1)>>1)-th completion of the barrier of parity (j-1)&1. S_j
                    // being ready implies P·V of block j-2 (hence j-3) complete, i.e. every earlier
                    // completion of this barrier, so the parity cannot be mistaken for an older phase.
                    if (!mbar_wait(pv_done(t, (j - 1) & 1), (uint32_t)(((j - 1) >> 1) & 1), abort_flag, 650 + t)) { ok = false; break; }
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
                    if ((kPolyPairMask >> (i & 3)) & 1u) {
                        e = exp2_poly_pair(a);
                    } else {
                        e.x = fast_exp2(a.x);
                        e.y = fast_exp2(a.y);
                    }
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
                if (lane == 0) mbar_arrive(p_full(t, bf));
            }
            // The key loop is over: a dependent kernel's CTAs may take the slots that free up from
            // here on and set themselves up (they read nothing before this grid has completed). The
            // first caller in a CTA counts; no thread calls it earlier, so a dependent never
            // competes with CTAs of this launch that have not started yet.
            pdl_launch_dependents();
            // ---- epilogue: merge the two halves of every row, O / l -> global
            // (m, l) of this half to the partner warp (same rows, other half) through shared memory
            // a half that never saw a finite score (all of its columns beyond N) must not set the scale
            const float m_own = (l > 0.f) ? m_ref * unit : -INFINITY;
            xch[(t * 2 + hf) * kAttnBlock + r_in_tile] = make_float2(m_own, l);
            __syncwarp();
            if (lane == 0) mbar_arrive(ep_bar(t, q));
            if (ok && mbar_wait(ep_bar(t, q), 0, abort_flag, 660 + t) && mbar_wait(o_final(t), 0, abort_flag, 670 + t)) {
                tc_fence_after();
                const float2 other = xch[(t * 2 + (hf ^ 1)) * kAttnBlock + r_in_tile];
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
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == W0 + 1) {
        __syncwarp();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

template <typename T, int MODE, int TILES>
static int launch_attention_split_tmt(const kb_attn_params& p, cudaStream_t stream) {
    using Cfg = AttnSplitCfgT<TILES>;
    using Shape = SplitShape<TILES>;
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
    const int num_m_tiles = (int)((p.M + kAttnBlock - 1) / kAttnBlock);
    d.num_pairs = (num_m_tiles + TILES - 1) / TILES;  // work items per (batch, head): tile pairs, or tiles
    d.head_group = attn_head_group(p.B * p.H, p.N, p.D);
    d.kv_group = (int)kv_group;
    d.d_out = (int)p.D;
    static int regs_ok = 0;  // 0 = not checked, 1 = usable, -1 = register allocation does not fit
    if (regs_ok == 0) {
        // setmaxnreg.inc blocks until the CTA's pool holds the registers: refuse to launch a build
        // whose launch allocation is smaller than the redistribution assumes.
        cudaFuncAttributes fa;
        if (cudaFuncGetAttributes(&fa, attention_split_kernel<T, MODE, TILES>) != cudaSuccess) return KB_ERR_LAUNCH;
        regs_ok = (fa.numRegs < Shape::kRegsLaunch) ? -1 : 1;
    }
    if (regs_ok < 0) return KB_ERR_UNSUPPORTED;
    static PerDeviceOnce attr_once;
    if (attr_once.first_time()) {
        if (cudaFuncSetAttribute(attention_split_kernel<T, MODE, TILES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg::kSmemMax) != cudaSuccess)
            return KB_ERR_LAUNCH;
    }
    const int64_t grid = (int64_t)d.num_pairs * p.B * p.H;
    if (grid > 0x7fffffff) return KB_ERR_UNSUPPORTED;
    const int num_n_blocks = (int)((p.N + kBlkN - 1) / kBlkN);
    const size_t smem_bytes = (size_t)Cfg::kSmemBase + (MODE == 1 ? (size_t)num_n_blocks * kBlkN * 4 : 0);
    if (launch_pdl(attention_split_kernel<T, MODE, TILES>, (unsigned)grid, (unsigned)Shape::kThreads, smem_bytes, stream, tq,
                   tk, tv, d) != cudaSuccess)
        return KB_ERR_LAUNCH;
    return cudaGetLastError() == cudaSuccess ? KB_OK : KB_ERR_LAUNCH;
}

// One tile per CTA, two CTAs per SM, is the shape the dispatcher uses: measured against the two-tile
// CTA it is 2 % (B8 H12 S4096) to 20 % (B64 H12 S512) faster on launches of many waves as well, not
// only on small ones — two independent CTAs hide each other's latencies better than two tiles inside
// one CTA share K/V. The two-tile shape stays selectable (kb_debug_split_tiles) and tested.
template <typename T, int MODE>
static int launch_attention_split_tm(const kb_attn_params& p, cudaStream_t stream) {
    if (g_split_tiles == 2) return launch_attention_split_tmt<T, MODE, 2>(p, stream);
    return launch_attention_split_tmt<T, MODE, 1>(p, stream);
}

// The persistent form of this kernel (attention_persist.cuh) takes the launches it is made for.
static bool attention_persist_applicable(const kb_attn_params& p, int mode);
template <typename T, int MODE>
static int launch_attention_persist_tm(const kb_attn_params& p, cudaStream_t stream);

template <typename T>
static int launch_attention_split_t(const kb_attn_params& p, cudaStream_t stream) {
    const int mode = (p.mask == nullptr && p.sm_scale > 0.f) ? 0
                     : (p.mask != nullptr && p.mask_strides[2] == 0 && p.N <= AttnSplitCfg::kMaskMaxN) ? 1 : 2;
    if (g_split_tiles == 0 && attention_persist_applicable(p, mode)) {
        if (mode == 0) return launch_attention_persist_tm<T, 0>(p, stream);
        if (mode == 1) return launch_attention_persist_tm<T, 1>(p, stream);
        return launch_attention_persist_tm<T, 2>(p, stream);
    }
    if (mode == 0) return launch_attention_split_tm<T, 0>(p, stream);
    if (mode == 1) return launch_attention_split_tm<T, 1>(p, stream);
    return launch_attention_split_tm<T, 2>(p, stream);
}

static int launch_attention_split(const kb_attn_params& p, cudaStream_t stream) {
    if (p.D > 64 || p.D % 8 != 0) return KB_ERR_UNSUPPORTED;
    if (p.dtype == KB_F16) return launch_attention_split_t<__half>(p, stream);
    if (p.dtype == KB_BF16) return launch_attention_split_t<__nv_bfloat16>(p, stream);
    return KB_ERR_UNSUPPORTED;
}

// The fused-attention entry: head dimensions up to 64 -> the split-row kernels above, up to 128 ->
// attention.cuh (multiples of 8; the kernels compute on 64 / 128 columns, the missing ones are zeros).
static int launch_attention(const kb_attn_params& p, cudaStream_t stream) {
    if (p.N <= 0) return KB_ERR_UNSUPPORTED;
    if (p.M > 0x7fffffff || p.N > 0x7fffffff || p.B * p.H > 0x7fffffff) return KB_ERR_UNSUPPORTED;
    if (p.D % 8 != 0 || p.D > 128) return KB_ERR_UNSUPPORTED;
    if (p.D <= 64) return launch_attention_split(p, stream);
    return launch_attention128(p, stream);
}

}  // namespace kb
