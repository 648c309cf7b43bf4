// Fused attention forward for sm_100a, variant with 64-key blocks and double-buffered scores.
//
// Same maths as attention.cuh and the same two softmax warpgroups (one 128-row query tile each) and
// TMA warp, with one tcgen05 issuer warp PER TILE (warps 9 and 10; warp 11 stages broadcast masks), but the keys are streamed in blocks of 64 and
// every tile owns TWO score buffers in TMEM. The issuer keeps the scores two blocks ahead of the
// softmax: S_{j+2} = Q·K_{j+2}ᵀ is issued into the buffer that P_j has just left, so a softmax group
// that finishes block j finds S_{j+1} already complete and never waits for the tensor core, and
// O += P_j·V_j runs behind its back. What bounds a long sequence is then the softmax group's own
// instruction stream instead of the round trip softmax -> issuer -> tensor core -> softmax.
//
// TMEM columns: S[t][b] at (2t+b)*64 (64 fp32 columns; P_j, 16-bit, overwrites the first 32),
// O[t] at 256 + 128t (D columns, +16 for the row sums when D = 64, see kSumOnTc in attention.cuh).
#pragma once
#include "attention.cuh"

namespace kb {

constexpr int kBlkN = 64;

template <int D>
struct Attn64Cfg {
    static constexpr int kKvStages = D == 64 ? 8 : 4;
    static constexpr int kQTileBytes = kAttnBlock * D * 2;
    static constexpr int kKvBytes = kBlkN * D * 2;
    static constexpr bool kSumOnTc = (D == 64);
    static constexpr int kOnesBytes = kSumOnTc ? kBlkN * 128 : 0;
    static constexpr int kOCols = kSumOnTc ? D + 16 : D;
    static constexpr int kTilesBytes = 2 * kQTileBytes + 2 * kKvStages * kKvBytes + kOnesBytes;
    static constexpr int kSmemBytes = kTilesBytes + 512 + 1024 + 1024;
};

template <typename T, int D, int MODE>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_tc64_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, const AttnDev p) {
    using Cfg = Attn64Cfg<D>;
    constexpr int KVS = Cfg::kKvStages;
    constexpr int QTILE = Cfg::kQTileBytes;
    constexpr int KVB = Cfg::kKvBytes;
    constexpr int QSLAB = kAttnBlock * 128;  // one 64-column slab of a Q tile
    constexpr int KSLAB = kBlkN * 128;       // one 64-column slab of a K or V block
    constexpr bool kSumOnTc = Cfg::kSumOnTc;
    constexpr bool kHalfExp = kSumOnTc && !Elem<T>::kIsBf16;
    constexpr int OCOLS = Cfg::kOCols;
    constexpr uint32_t kTmemCols = 512;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t q_smem = smem_u32(smem);
    const uint32_t k_smem = q_smem + 2 * QTILE;
    const uint32_t v_smem = k_smem + KVS * KVB;
    const uint32_t ones_smem = v_smem + KVS * KVB;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kTilesBytes);
    const uint32_t bar_base = smem_u32(bars);
    auto q_full = [&](int t) { return bar_base + 8u * t; };
    // P_j written (softmax -> issuer), one barrier per block parity: a softmax group may finish block
    // j+1 before the issuer has looked at block j, and a single barrier's phase parity could not tell
    // those two completions apart
    auto p_full = [&](int t, int bf) { return bar_base + 8u * (2 + t * 2 + bf); };
    auto o_final = [&](int t) { return bar_base + 8u * (6 + t); };
    auto s_full = [&](int t, int bf) { return bar_base + 8u * (8 + t * 2 + bf); };
    auto m_full = [&](int t, int bf) { return bar_base + 8u * (12 + t * 2 + bf); };
    auto m_empty = [&](int t, int bf) { return bar_base + 8u * (16 + t * 2 + bf); };
    auto k_full = [&](int s) { return bar_base + 8u * (20 + s); };
    auto k_empty = [&](int s) { return bar_base + 8u * (20 + KVS + s); };
    auto v_full = [&](int s) { return bar_base + 8u * (20 + 2 * KVS + s); };
    auto v_empty = [&](int s) { return bar_base + 8u * (20 + 3 * KVS + s); };
    // completion of O_t += P_j·V_j, one barrier per block parity (see the rescale path below)
    auto pv_done = [&](int t, int bf) { return bar_base + 8u * (20 + 4 * KVS + t * 2 + bf); };
    constexpr int kNumBars = 24 + 4 * KVS;
    static_assert(kNumBars * 8 + 16 <= 512, "barrier area too small");
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* mask_smem = reinterpret_cast<float*>(smem + Cfg::kTilesBytes + 512);  // [tile][buffer][64]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    {
        __shared__ int s_skip;
        if (threadIdx.x == 0) s_skip = *reinterpret_cast<volatile int*>(&g_device_status[0]);
        __syncthreads();
        if (s_skip != 0) return;
    }

    const int BH = p.B * p.H;
    int bh, pair;
    attn_work_item(p, BH, bh, pair);
    const int b = bh / p.H, h = bh % p.H;
    const int num_m_tiles = (p.M + kAttnBlock - 1) / kAttnBlock;
    const int num_n_blocks = (p.N + kBlkN - 1) / kBlkN;
    int mt[2], nblk[2];
    int ntl = 0;
    for (int t = 0; t < 2; ++t) {
        mt[t] = pair * 2 + t;
        if (mt[t] < num_m_tiles) {
            ntl = t + 1;
            nblk[t] = p.is_causal ? min(num_n_blocks, (mt[t] + 1) * (kAttnBlock / kBlkN)) : num_n_blocks;
        } else {
            nblk[t] = 0;
        }
    }
    const int max_blk = max(nblk[0], nblk[1]);

    if (threadIdx.x == 0) {
        for (int t = 0; t < 2; ++t) {
            mbar_init(q_full(t), 1);
            mbar_init(o_final(t), 1);
            for (int bf = 0; bf < 2; ++bf) {
                mbar_init(s_full(t, bf), 1);
                mbar_init(pv_done(t, bf), 1);
                mbar_init(p_full(t, bf), 4);
                mbar_init(m_full(t, bf), 1);
                mbar_init(m_empty(t, bf), 4);
            }
        }
        for (int s = 0; s < KVS; ++s) {
            mbar_init(k_full(s), 1);
            mbar_init(k_empty(s), ntl);  // one arrival per live tile's issuer
            mbar_init(v_full(s), 1);
            mbar_init(v_empty(s), ntl);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (kSumOnTc) {
        const uint32_t one2 = Elem<T>::pack2(1.0f, 1.0f);
        uint32_t* ones = reinterpret_cast<uint32_t*>(smem + 2 * QTILE + 2 * KVS * KVB);
        for (int i = threadIdx.x; i < Cfg::kOnesBytes / 4; i += kAttnThreads) ones[i] = one2;
        fence_proxy_async_smem();
    }
    if (warp == 9) {
        tmem_alloc(smem_u32(tmem_slot), kTmemCols);
        tmem_relinquish();
    }
    if (warp == 8 && lane == 0) {
        tma_prefetch_desc(&tmap_q);
        tma_prefetch_desc(&tmap_k);
        tma_prefetch_desc(&tmap_v);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp >= 8) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kAttnRegsLow));
      if (warp == 8) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one()) {
            bool ok = true;
            for (int t = 0; t < ntl; ++t) {
                mbar_arrive_expect_tx(q_full(t), QTILE);
                for (int c = 0; c < D / 64; ++c)
                    tma_load_4d(q_smem + t * QTILE + c * QSLAB, &tmap_q, q_full(t), c * 64, mt[t] * kAttnBlock, h, b);
            }
            for (int j = 0; j < max_blk && ok; ++j) {
                const int s = j % KVS;
                const uint32_t ph = (uint32_t)((j / KVS) & 1);
                if (!mbar_wait(k_empty(s), ph ^ 1, abort_flag, 100)) { ok = false; break; }
                mbar_arrive_expect_tx(k_full(s), KVB);
                for (int c = 0; c < D / 64; ++c)
                    tma_load_4d(k_smem + s * KVB + c * KSLAB, &tmap_k, k_full(s), c * 64, j * kBlkN, h, b);
                if (!mbar_wait(v_empty(s), ph ^ 1, abort_flag, 101)) { ok = false; break; }
                mbar_arrive_expect_tx(v_full(s), KVB);
                for (int c = 0; c < D / 64; ++c)
                    tma_load_4d(v_smem + s * KVB + c * KSLAB, &tmap_v, v_full(s), c * 64, j * kBlkN, h, b);
            }
            if (!ok) {
                for (int i = 0; i < 64; ++i) __nanosleep(2000);
            }
        }
      } else if (warp == 9 || warp == 10) {
        // ------------------------------------------------------------------ MMA issuers, one per tile
        // A single thread pushing the tcgen05 work of both tiles is itself a bottleneck (its serial
        // stream of barrier polls, fences, sixteen MMA issues and commits per key block is slower
        // than the softmax groups), so warp 9 serves tile 0 and warp 10 serves tile 1. A K or V
        // stage is released when BOTH have arrived on its "empty" barrier.
        const int t = warp - 9;
        if (elect_one()) {
            constexpr uint32_t idesc_qk = make_idesc_f16(Elem<T>::kIsBf16, 128, kBlkN, 0, 0);
            constexpr uint32_t idesc_pv = make_idesc_f16(Elem<T>::kIsBf16, 128, OCOLS, 0, 1);
            constexpr uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
            const uint32_t q_lo = ((q_smem + t * QTILE) & 0x3FFFF) >> 4;
            const uint32_t k_lo = (k_smem & 0x3FFFF) >> 4;
            const uint32_t v_lo = ((v_smem & 0x3FFFF) >> 4) | (kSumOnTc ? 0u : ((uint32_t)(KSLAB >> 4) << 16));
            auto desc = [&](uint32_t lo) { return ((uint64_t)desc_hi << 32) | (uint64_t)lo; };
            auto issue_qk = [&](int j) {  // S[t][j&1] = Q_t · K_jᵀ
                const uint32_t b_lo = k_lo + (uint32_t)((j % KVS) * (KVB >> 4));
                const uint32_t d_tmem = tmem_base + (uint32_t)((t * 2 + (j & 1)) * kBlkN);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t a_off = (uint32_t)(((ks / 4) * QSLAB + (ks % 4) * 32) >> 4);
                    const uint32_t b_off = (uint32_t)(((ks / 4) * KSLAB + (ks % 4) * 32) >> 4);
                    tc_mma_ss(d_tmem, desc(q_lo + a_off), desc(b_lo + b_off), idesc_qk, ks > 0 ? 1u : 0u);
                }
            };
            auto issue_pv = [&](int j) {  // O_t (+)= P_j · V_j
                const int s = j % KVS;
                uint32_t b_lo = v_lo + (uint32_t)(s * (KVB >> 4));
                if (kSumOnTc) b_lo |= (uint32_t)((ones_smem - (v_smem + s * KVB)) >> 4) << 16;
                const uint32_t d_tmem = tmem_base + (uint32_t)(256 + t * 128);
                const uint32_t a_tmem = tmem_base + (uint32_t)((t * 2 + (j & 1)) * kBlkN);
#pragma unroll
                for (int ks = 0; ks < kBlkN / 16; ++ks) {
                    tc_mma_ts(d_tmem, a_tmem + (uint32_t)(ks * 8), desc(b_lo + (uint32_t)(ks * (2048 >> 4))), idesc_pv,
                              (j > 0 || ks > 0) ? 1u : 0u);
                }
            };
            const int my_blk = (t < ntl) ? nblk[t] : 0;
            bool ok = true;
            if (t < ntl && !mbar_wait(q_full(t), 0, abort_flag, 200)) ok = false;
            // prologue: scores of blocks 0 and 1
            for (int jj = 0; jj < 2 && jj < max_blk && ok && t < ntl; ++jj) {
                if (!mbar_wait(k_full(jj % KVS), (uint32_t)((jj / KVS) & 1), abort_flag, 201)) { ok = false; break; }
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
                if (!mbar_wait(v_full(s), (uint32_t)((j / KVS) & 1), abort_flag, 202)) { ok = false; break; }
                const int j2 = j + 2;
                if (j2 < max_blk) {
                    if (!mbar_wait(k_full(j2 % KVS), (uint32_t)((j2 / KVS) & 1), abort_flag, 203)) { ok = false; break; }
                }
                if (j < my_blk) {
                    if (!mbar_wait(p_full(t, j & 1), (uint32_t)((j >> 1) & 1), abort_flag, 204)) { ok = false; break; }
                    tc_fence_after();
                    issue_pv(j);
                    tc_commit(pv_done(t, j & 1));
                    if (j2 < my_blk) {
                        issue_qk(j2);  // into the buffer that P_j has just been read from (in-order execution)
                        tc_commit(s_full(t, j & 1));
                    }
                    if (j + 1 == my_blk) tc_commit(o_final(t));
                    tc_commit(v_empty(s));
                    if (j2 < max_blk) {
                        if (j2 < my_blk) tc_commit(k_empty(j2 % KVS));
                        else mbar_arrive(k_empty(j2 % KVS));
                    }
                } else {
                    // blocks beyond this tile's causal range: hand the stages back untouched, but only
                    // once they have been loaded, so that the arrival lands in the right phase
                    mbar_arrive(v_empty(s));
                    if (j2 < max_blk) mbar_arrive(k_empty(j2 % KVS));
                }
            }
        }
      } else if (MODE == 1 && warp == 11) {
        // ------------------------------------------------------------------ mask loader (warp 11)
        const float mlow = mask_lowest(p.mask_dtype);
        const int64_t moff = (int64_t)b * p.mask_strides[0] + (int64_t)h * p.mask_strides[1];
        bool ok = true;
        for (int j = 0; j < max_blk && ok; ++j) {
            const int bf = j & 1;
            const uint32_t ph = (uint32_t)((j >> 1) & 1);
            for (int t = 0; t < ntl && ok; ++t) {
                if (j >= nblk[t]) continue;
                if (!mbar_wait(m_empty(t, bf), ph ^ 1, abort_flag, 400 + t)) { ok = false; break; }
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int idx = lane + e * 32;
                    const int col = j * kBlkN + idx;
                    float a = -INFINITY;
                    if (col < p.N)
                        a = fmaxf(mask_load(p.mask, moff + (int64_t)col * p.mask_strides[3], p.mask_dtype), mlow) * kLog2e;
                    mask_smem[(t * 2 + bf) * kBlkN + idx] = a;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(m_full(t, bf));
            }
        }
      }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kAttnRegsHigh));
        // ------------------------------------------------------------------ softmax groups
        const int t = warp >> 2;
        const int q = warp & 3;
        if (t < ntl && nblk[t] > 0) {
            const int row = mt[t] * kAttnBlock + q * 32 + lane;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
            const uint32_t o_addr = lane_addr + (uint32_t)(256 + t * 128);
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
            for (int j = 0; j < nblk[t]; ++j) {
                const int bf = j & 1;
                const uint32_t s_addr = lane_addr + (uint32_t)((t * 2 + bf) * kBlkN);
                if (!mbar_wait(s_full(t, bf), (uint32_t)((j >> 1) & 1), abort_flag, 300 + t)) { ok = false; break; }
                tc_fence_after();
                uint32_t sr[2][32];
                tmem_ld_32x32(s_addr, sr[0]);
                tmem_ld_32x32(s_addr + 32, sr[1]);
                tmem_ld_wait();

                const int col0 = j * kBlkN;
                const bool causal_edge = p.is_causal && col0 + kBlkN - 1 > mt[t] * kAttnBlock;
                if (MODE == 1) {
                    if (!mbar_wait(m_full(t, bf), (uint32_t)((j >> 1) & 1), abort_flag, 320 + t)) { ok = false; break; }
                    const float4* ms = reinterpret_cast<const float4*>(mask_smem + (t * 2 + bf) * kBlkN);
#pragma unroll
                    for (int cch = 0; cch < 2; ++cch) {
#pragma unroll
                        for (int v4 = 0; v4 < 8; ++v4) {
                            const float4 a = ms[cch * 8 + v4];
                            sr[cch][v4 * 4 + 0] = __float_as_uint(fmaf(__uint_as_float(sr[cch][v4 * 4 + 0]), c, a.x));
                            sr[cch][v4 * 4 + 1] = __float_as_uint(fmaf(__uint_as_float(sr[cch][v4 * 4 + 1]), c, a.y));
                            sr[cch][v4 * 4 + 2] = __float_as_uint(fmaf(__uint_as_float(sr[cch][v4 * 4 + 2]), c, a.z));
                            sr[cch][v4 * 4 + 3] = __float_as_uint(fmaf(__uint_as_float(sr[cch][v4 * 4 + 3]), c, a.w));
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(m_empty(t, bf));
                } else if (MODE == 2) {
                    if (p.mask == nullptr) {
#pragma unroll
                        for (int cch = 0; cch < 2; ++cch) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) sr[cch][i] = __float_as_uint(__uint_as_float(sr[cch][i]) * c);
                        }
                    } else {
#pragma unroll
                        for (int hc = 0; hc < 4; ++hc) {
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
                                uint32_t& sv = sr[hc >> 1][(hc & 1) * 16 + i];
                                sv = __float_as_uint(fmaf(fmaxf(mvals[i], mlow), kLog2e, __uint_as_float(sv) * c));
                            }
                        }
                    }
                }
                if ((MODE != 1 && col0 + kBlkN > p.N) || causal_edge) {
#pragma unroll
                    for (int cch = 0; cch < 2; ++cch) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int col = col0 + cch * 32 + i;
                            if (col >= p.N || (p.is_causal && col > row)) sr[cch][i] = __float_as_uint(-INFINITY);
                        }
                    }
                }
                float mx2[2];
#pragma unroll
                for (int cch = 0; cch < 2; ++cch) {
                    float mloc = fmaxf(__uint_as_float(sr[cch][0]), __uint_as_float(sr[cch][1]));
#pragma unroll
                    for (int i = 2; i < 32; i += 2) mloc = fmax3(mloc, __uint_as_float(sr[cch][i]), __uint_as_float(sr[cch][i + 1]));
                    mx2[cch] = mloc;
                }
                const float mx = fmaxf(mx2[0], mx2[1]);
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
                    // O_t must be quiescent before it is rescaled: P·V of block j-1 complete. That is
                    // the ((j-1)>>1)-th completion of the barrier of parity (j-1)&1. S_j being ready
                    // implies P·V of block j-2 (hence j-3) complete, i.e. every earlier completion of
                    // this barrier, so the phase parity below cannot be mistaken for an older phase
                    // even though most blocks never wait here.
                    if (!mbar_wait(pv_done(t, (j - 1) & 1), (uint32_t)(((j - 1) >> 1) & 1), abort_flag, 330 + t)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int dch = 0; dch < OCOLS / 16; ++dch) {
                        uint32_t orr[16];
                        tmem_ld_32x16(o_addr + dch * 16, orr);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
                        tmem_st_32x16(o_addr + dch * 16, orr);
                    }
                }
                const float neg_ref = -m_ref * unit;
                float lp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int cch = 0; cch < 2; ++cch) {
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float a0 = fmaf(__uint_as_float(sr[cch][2 * i]), unit, neg_ref);
                        const float a1 = fmaf(__uint_as_float(sr[cch][2 * i + 1]), unit, neg_ref);
                        if (kHalfExp) {
                            const uint32_t h2 = Elem<T>::pack2(a0, a1);
                            asm("ex2.approx.f16x2 %0, %1;" : "=r"(pk[i]) : "r"(h2));
                        } else {
                            const float e0 = fast_exp2(a0);
                            const float e1 = fast_exp2(a1);
                            if (!kSumOnTc) lp[i & 3] += e0 + e1;
                            pk[i] = Elem<T>::pack2(e0, e1);
                        }
                    }
                    tmem_st_32x16(s_addr + cch * 16, pk);
                }
                if (!kSumOnTc) l += (lp[0] + lp[1]) + (lp[2] + lp[3]);
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full(t, bf));
            }
            // ---- epilogue: O / l -> global
            if (ok && mbar_wait(o_final(t), 0, abort_flag, 310 + t)) {
                tc_fence_after();
                if (kSumOnTc) {
                    uint32_t lr[16];
                    tmem_ld_32x16(o_addr + D, lr);
                    tmem_ld_wait();
                    l = __uint_as_float(lr[0]);
                }
                const float inv_l = 1.0f / l;
                T* o_row = reinterpret_cast<T*>(p.o) + (int64_t)b * p.o_strides[0] + (int64_t)h * p.o_strides[1] +
                           (int64_t)row * p.o_strides[2];
                const bool vec = p.o_strides[3] == 1 && ((((uintptr_t)o_row) & 15) == 0);
#pragma unroll
                for (int dch = 0; dch < D / 32; ++dch) {
                    uint32_t orr[32];
                    tmem_ld_32x32(o_addr + dch * 32, orr);
                    tmem_ld_wait();
                    if (row < p.M) {
                        if (vec) {
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                uint4 w;
                                w.x = Elem<T>::pack2(__uint_as_float(orr[v * 8 + 0]) * inv_l, __uint_as_float(orr[v * 8 + 1]) * inv_l);
                                w.y = Elem<T>::pack2(__uint_as_float(orr[v * 8 + 2]) * inv_l, __uint_as_float(orr[v * 8 + 3]) * inv_l);
                                w.z = Elem<T>::pack2(__uint_as_float(orr[v * 8 + 4]) * inv_l, __uint_as_float(orr[v * 8 + 5]) * inv_l);
                                w.w = Elem<T>::pack2(__uint_as_float(orr[v * 8 + 6]) * inv_l, __uint_as_float(orr[v * 8 + 7]) * inv_l);
                                reinterpret_cast<uint4*>(o_row + dch * 32)[v] = w;
                            }
                        } else {
                            for (int i = 0; i < 32; ++i)
                                o_row[(int64_t)(dch * 32 + i) * p.o_strides[3]] =
                                    Elem<T>::from_f32(__uint_as_float(orr[i]) * inv_l);
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        __syncwarp();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

template <typename T, int D, int MODE>
static int launch_attention64_tdm(const kb_attn_params& p, cudaStream_t stream) {
    using Cfg = Attn64Cfg<D>;
    CUtensorMap tq, tk, tv;
    auto enc = [&](CUtensorMap* out, const void* ptr, int64_t rows, const int64_t* st, uint32_t box_rows) -> int {
        if (st[3] != 1) return KB_ERR_UNSUPPORTED;
        const uint64_t dims[4] = {(uint64_t)D, (uint64_t)rows, (uint64_t)p.H, (uint64_t)p.B};
        auto fix = [](int64_t extent, int64_t stride) -> uint64_t { return (extent == 1) ? 16u : (uint64_t)stride * 2u; };
        const uint64_t strides[4] = {0, fix(rows, st[2]), fix(p.H, st[1]), fix(p.B, st[0])};
        const uint32_t box[4] = {64, box_rows, 1, 1};
        return encode_tmap_16bit(out, ptr, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    };
    int st = enc(&tq, p.q, p.M, p.q_strides, kAttnBlock);
    if (st != KB_OK) return st;
    st = enc(&tk, p.k, p.N, p.k_strides, kBlkN);
    if (st != KB_OK) return st;
    st = enc(&tv, p.v, p.N, p.v_strides, kBlkN);
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
    d.num_pairs = (num_m_tiles + 1) / 2;
    d.head_group = attn_head_group(p.B * p.H, p.N, p.D);
    static PerDeviceOnce attr_once;
    if (attr_once.first_time()) {
        if (cudaFuncSetAttribute(attention_tc64_kernel<T, D, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg::kSmemBytes) != cudaSuccess)
            return KB_ERR_LAUNCH;
    }
    const int64_t grid = (int64_t)d.num_pairs * p.B * p.H;
    if (grid > 0x7fffffff) return KB_ERR_UNSUPPORTED;
    attention_tc64_kernel<T, D, MODE><<<(unsigned)grid, kAttnThreads, Cfg::kSmemBytes, stream>>>(tq, tk, tv, d);
    return cudaGetLastError() == cudaSuccess ? KB_OK : KB_ERR_LAUNCH;
}

template <typename T, int D>
static int launch_attention64_td(const kb_attn_params& p, cudaStream_t stream) {
    if (p.mask == nullptr && p.sm_scale > 0.f) return launch_attention64_tdm<T, D, 0>(p, stream);
    if (p.mask != nullptr && p.mask_strides[2] == 0) return launch_attention64_tdm<T, D, 1>(p, stream);
    return launch_attention64_tdm<T, D, 2>(p, stream);
}

// Which kernel serves a call: 0 = by head dimension (below), 1 = 128-key blocks, 2 = 64-key blocks,
// 3 = 64-key blocks with two threads per query row (head dimension 64 only).
static int g_attn_variant = 0;
static int launch_attention_split(const kb_attn_params& p, cudaStream_t stream);

static int launch_attention(const kb_attn_params& p, cudaStream_t stream) {
    if (p.N <= 0) return KB_ERR_UNSUPPORTED;
    if (p.M > 0x7fffffff || p.N > 0x7fffffff || p.B * p.H > 0x7fffffff) return KB_ERR_UNSUPPORTED;
    if (p.D == 64 && (g_attn_variant == 3 || g_attn_variant == 0)) return launch_attention_split(p, stream);
    const bool use64 = g_attn_variant == 2 || g_attn_variant == 3;
    if (!use64) return launch_attention128(p, stream);
    if (p.dtype == KB_F16) {
        if (p.D == 64) return launch_attention64_td<__half, 64>(p, stream);
        if (p.D == 128) return launch_attention64_td<__half, 128>(p, stream);
    } else if (p.dtype == KB_BF16) {
        if (p.D == 64) return launch_attention64_td<__nv_bfloat16, 64>(p, stream);
        if (p.D == 128) return launch_attention64_td<__nv_bfloat16, 128>(p, stream);
    }
    return KB_ERR_UNSUPPORTED;
}

}  // namespace kb
