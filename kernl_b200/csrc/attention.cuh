// Fused attention forward for sm_100a: O = softmax(sm_scale·Q·Kᵀ + mask [causal]) · V.
//
// One CTA owns TWO query tiles of 128 rows of one (batch, head) and streams the keys/values in
// blocks of 128. Roles (384 threads = 3 warpgroups):
//   warps 0..3    softmax group of tile 0 (one query row per thread)
//   warps 4..7    softmax group of tile 1
//   warp 8        TMA producer: both Q tiles once, then the K and V blocks through two small rings
//   warp 9        tcgen05 issuer (one elected thread):  S_t = Q_t·K_jᵀ  (operands in shared memory)
//                 and  O_t += P_t·V_j  (P read from TMEM, V from shared memory, N-major)
//   warps 10..11  idle (they only give their registers away)
// The third warpgroup shrinks its register allowance (setmaxnreg) so that the softmax threads can
// hold a whole 128-wide score row in registers.
// While one group runs its exponentials, the tensor core works on the other tile (ping-pong).
// TMEM columns: S_0 [0,128)  S_1 [128,256)  O_0 [256,256+D)  O_1 [384,384+D); P_t (16-bit, two
// per column) overwrites the first 64 columns of S_t once the thread has its row in registers.
//
// Online softmax in the log2 domain with LAZY rescaling: the running reference maximum of a row
// only moves (and O is only rescaled in TMEM) when the true maximum has grown by more than 2^8,
// so P stays below 256 — exactly representable range for fp16/bf16 — and most iterations skip
// the O round trip. The final O is divided by the fp32 row sum.
//
// Semantics follow src/kernl/implementations/attention.py:122-435 of the reference: scale before
// mask (:345), additive mask with -inf clamped to the lowest finite value of the mask's dtype
// (:380,:516), causal = keep col <= row, top-left aligned (:347), P rounded to the input dtype
// before P·V (:424), fp32 statistics and accumulation (:290-295).
#pragma once
#include "common.cuh"

namespace kb {

constexpr int kAttnThreads = 384;
constexpr int kAttnBlock = 128;  // rows per query tile and keys per block
constexpr int kBlkN = 64;        // keys per block of the head-dimension-64 kernel (attention_split.cuh)
// Register re-balancing between the warpgroups (setmaxnreg). The CTA is launched with
// 65536 / 384 -> 168 registers per thread; the third warpgroup shrinks to kAttnRegsLow and the two
// softmax warpgroups grow to kAttnRegsHigh. The increase waits (without bound) until the CTA's own
// pool has the registers, so the totals MUST fit the launch allocation: 2*high + low <= 3*168.
constexpr int kAttnRegsLaunch = 168;
constexpr int kAttnRegsLow = 40;
constexpr int kAttnRegsHigh = 232;
static_assert(2 * kAttnRegsHigh + kAttnRegsLow <= 3 * kAttnRegsLaunch, "setmaxnreg totals exceed the CTA's register pool");
static_assert(kAttnRegsLow % 8 == 0 && kAttnRegsHigh % 8 == 0, "setmaxnreg wants multiples of 8");
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLazyThreshold = 8.0f;

struct AttnDev {
    void* o;
    const void* mask;
    int64_t o_strides[4];
    int64_t mask_strides[4];
    int B, H, M, N;
    float scale_log2;  // sm_scale * log2(e)
    int is_causal;
    int mask_dtype;
    int mask_vec;   // mask rows can be read with aligned 128-bit loads
    int num_pairs;  // ceil(ceil(M/128)/2)
    int head_group; // heads whose CTAs are interleaved (see attn_work_item)
    int kv_group;   // query heads per K/V head (grouped-query attention), >= 1
    int d_out;      // head dimension of the caller's tensors (a multiple of 8, at most the kernel's D): the
                    // tensor maps end there — TMA fills the columns beyond with zeros, which add nothing to
                    // q·kᵀ — and only these output columns are stored
};

// Stores 32 output columns [col0, col0 + 32) of one row. GUARD: the caller's head dimension ends
// inside or before the chunk (d_out < col0 + 32), so only whole 8-column pieces below d_out are
// written; the unguarded form is the hot path and carries no per-store condition (a guard inside the
// store loop of the head-dimension-64 kernel cost 2.7 µs of a 21 µs launch).
template <typename T, bool GUARD>
__device__ __forceinline__ void attn_store_32(T* __restrict__ o_row, int col0, int64_t col_stride, bool vec,
                                              const float (&val)[32], int d_out) {
    if (vec) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            if (GUARD && col0 + v * 8 >= d_out) continue;
            uint4 w;
            w.x = Elem<T>::pack2(val[v * 8 + 0], val[v * 8 + 1]);
            w.y = Elem<T>::pack2(val[v * 8 + 2], val[v * 8 + 3]);
            w.z = Elem<T>::pack2(val[v * 8 + 4], val[v * 8 + 5]);
            w.w = Elem<T>::pack2(val[v * 8 + 6], val[v * 8 + 7]);
            reinterpret_cast<uint4*>(o_row + col0)[v] = w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {  // (fully unrolled: val stays in registers)
            if (GUARD && col0 + i >= d_out) continue;
            o_row[(int64_t)(col0 + i) * col_stride] = Elem<T>::from_f32(val[i]);
        }
    }
}

// CTA -> (batch*head, query-tile pair). Heads are taken in groups of p.head_group; inside a group
// the order is pair-major with the late (causally heavier) pairs first, so the tail of a causal
// launch is made of light tiles, and consecutive CTAs are different heads of the same group. The
// group is sized on the host so that the K/V of all its heads (what the resident CTAs stream) stay
// in L2: with one group over all heads, 148 resident CTAs of a long-sequence launch streamed the
// K/V of 148 heads and DRAM read traffic was ten times the algorithmic bytes.
__device__ __forceinline__ void attn_work_item(const AttnDev& p, int BH, int& bh, int& pair) {
    const int per_group = p.num_pairs * p.head_group;
    const int g = (int)(blockIdx.x / per_group);
    const int rem = (int)(blockIdx.x % per_group);
    const int first = g * p.head_group;
    const int gsz = min(p.head_group, BH - first);
    pair = p.num_pairs - 1 - rem / gsz;
    bh = first + rem % gsz;
}
static int attn_head_group(int64_t BH, int64_t N, int64_t D) {
    const int64_t kv_bytes = 2 * N * D * 2;
    int64_t g = ((int64_t)32 << 20) / (kv_bytes > 0 ? kv_bytes : 1);
    if (g < 1) g = 1;
    if (g > BH) g = BH;
    return (int)g;
}

template <int D>
struct AttnCfg {
    static constexpr int kKvStages = D == 64 ? 3 : 2;
    static constexpr int kTileBytes = kAttnBlock * D * 2;  // one Q tile / one K block / one V block
    // D = 64 only: the row sums of P come out of the tensor core. V gets 16 extra columns of ones
    // (one 128-byte-swizzled slab of ones in shared memory, shared by every stage), so O has D+16
    // columns and column D accumulates sum_k P[r,k] of exactly the 16-bit P that multiplies V.
    static constexpr bool kSumOnTc = (D == 64);
    static constexpr int kOnesBytes = kSumOnTc ? kAttnBlock * 128 : 0;
    static constexpr int kOCols = kSumOnTc ? D + 16 : D;
    static constexpr int kSmemBytes = (2 + 2 * kKvStages) * kTileBytes + kOnesBytes + 512 + 2048 + 1024;
};

__device__ __forceinline__ float mask_lowest(int mask_dtype) {
    if (mask_dtype == KB_F16) return -65504.0f;
    if (mask_dtype == KB_BF16) return -3.3895313892515355e38f;
    return -3.4028234663852886e38f;
}

__device__ __forceinline__ float mask_load(const void* base, int64_t off, int mask_dtype) {
    if (mask_dtype == KB_F16) return __half2float(reinterpret_cast<const __half*>(base)[off]);
    if (mask_dtype == KB_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[off]);
    return reinterpret_cast<const float*>(base)[off];
}

__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// MODE 0: no mask and positive scale (maximum taken on raw scores, one FFMA + EX2 per element);
// MODE 1: additive mask that is the same for every query row (padding masks): warps 10-11 stage
//         it per key block in shared memory, already clamped, scaled by log2(e) and with -inf for
//         columns beyond N; MODE 2: anything else (per-row masks read from global memory with
//         128-bit loads where the layout allows, non-positive scale).
template <typename T, int D, int MODE>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const AttnDev p) {
    using Cfg = AttnCfg<D>;
    constexpr int KVS = Cfg::kKvStages;
    constexpr int TILE = Cfg::kTileBytes;
    constexpr int CHUNK = kAttnBlock * 64 * 2;  // one 64-column (128-byte swizzled) slab of a tile
    constexpr uint32_t kTmemCols = 512;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t q_smem = smem_u32(smem);
    const uint32_t k_smem = q_smem + 2 * TILE;
    const uint32_t v_smem = k_smem + KVS * TILE;
    constexpr bool kSumOnTc = Cfg::kSumOnTc;
    // With fp16 inputs the exponentials themselves are taken two at a time in half precision
    // (ex2.approx.f16x2): the argument s - m_ref is at most 2^3 (lazy rescaling), where fp16 still
    // resolves 2^-8, and P is rounded to fp16 for the tensor core anyway. bf16 keeps fp32 exponentials.
    constexpr bool kHalfExp = kSumOnTc && !Elem<T>::kIsBf16;
    constexpr int OCOLS = Cfg::kOCols;
    const uint32_t ones_smem = v_smem + KVS * TILE;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (2 + 2 * KVS) * TILE + Cfg::kOnesBytes);
    const uint32_t bar_base = smem_u32(bars);
    // barrier slots
    auto q_full = [&](int t) { return bar_base + 8u * t; };
    auto k_full = [&](int s) { return bar_base + 8u * (2 + s); };
    auto k_empty = [&](int s) { return bar_base + 8u * (2 + KVS + s); };
    auto v_full = [&](int s) { return bar_base + 8u * (2 + 2 * KVS + s); };
    auto v_empty = [&](int s) { return bar_base + 8u * (2 + 3 * KVS + s); };
    auto s_full = [&](int t) { return bar_base + 8u * (2 + 4 * KVS + t); };
    auto p_full = [&](int t) { return bar_base + 8u * (4 + 4 * KVS + t); };
    auto o_final = [&](int t) { return bar_base + 8u * (6 + 4 * KVS + t); };
    auto m_full = [&](int t, int bf) { return bar_base + 8u * (8 + 4 * KVS + t * 2 + bf); };
    auto m_empty = [&](int t, int bf) { return bar_base + 8u * (12 + 4 * KVS + t * 2 + bf); };
    constexpr int kNumBars = 16 + 4 * KVS;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* mask_smem = reinterpret_cast<float*>(smem + (2 + 2 * KVS) * TILE + Cfg::kOnesBytes + 512);  // [tile][buffer][128]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // A wait that expired in an earlier CTA or launch leaves the status word set: do no work until
    // the host has read (and cleared) it, so that one failure cannot cost a second per CTA.
    {
        __shared__ int s_skip;
        if (threadIdx.x == 0) s_skip = *reinterpret_cast<volatile int*>(&g_device_status[0]);
        __syncthreads();
        if (s_skip != 0) return;
    }

    // Work assignment: heavy (late) query tiles first so that causal work is balanced.
    const int BH = p.B * p.H;
    int bh, pair;
    attn_work_item(p, BH, bh, pair);
    const int b = bh / p.H, h = bh % p.H;
    const int num_m_tiles = (p.M + kAttnBlock - 1) / kAttnBlock;
    const int num_n_blocks = (p.N + kAttnBlock - 1) / kAttnBlock;
    int mt[2], nblk[2];
    int ntl = 0;  // live tiles in this CTA (1 or 2)
    for (int t = 0; t < 2; ++t) {
        mt[t] = pair * 2 + t;
        if (mt[t] < num_m_tiles) {
            ntl = t + 1;
            nblk[t] = p.is_causal ? min(num_n_blocks, mt[t] + 1) : num_n_blocks;
        } else {
            nblk[t] = 0;
        }
    }
    const int max_blk = max(nblk[0], nblk[1]);

    if (threadIdx.x == 0) {
        for (int t = 0; t < 2; ++t) {
            mbar_init(q_full(t), 1);
            mbar_init(s_full(t), 1);
            mbar_init(p_full(t), 4);
            mbar_init(o_final(t), 1);
            for (int bf = 0; bf < 2; ++bf) {
                mbar_init(m_full(t, bf), 2);   // the two loader warps
                mbar_init(m_empty(t, bf), 4);  // the four warps of the tile's softmax group
            }
        }
        for (int s = 0; s < KVS; ++s) {
            mbar_init(k_full(s), 1);
            mbar_init(k_empty(s), 1);
            mbar_init(v_full(s), 1);
            mbar_init(v_empty(s), 1);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (kSumOnTc) {
        const uint32_t one2 = Elem<T>::pack2(1.0f, 1.0f);
        uint32_t* ones = reinterpret_cast<uint32_t*>(smem + (2 + 2 * KVS) * TILE);
        for (int i = threadIdx.x; i < Cfg::kOnesBytes / 4; i += kAttnThreads) ones[i] = one2;
        fence_proxy_async_smem();  // the tensor core reads shared memory through the async proxy
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
                mbar_arrive_expect_tx(q_full(t), TILE);
                for (int c = 0; c < D / 64; ++c)
                    tma_load_4d(q_smem + t * TILE + c * CHUNK, &tmap_q, q_full(t), c * 64,
                                mt[t] * kAttnBlock, h, b);
            }
            for (int j = 0; j < max_blk && ok; ++j) {
                const int s = j % KVS;
                const uint32_t ph = (uint32_t)((j / KVS) & 1);
                if (!mbar_wait(k_empty(s), ph ^ 1, abort_flag, 100)) { ok = false; break; }
                mbar_arrive_expect_tx(k_full(s), TILE);
                for (int c = 0; c < D / 64; ++c)
                    tma_load_4d(k_smem + s * TILE + c * CHUNK, &tmap_k, k_full(s), c * 64,
                                j * kAttnBlock, h / p.kv_group, b);
                if (!mbar_wait(v_empty(s), ph ^ 1, abort_flag, 101)) { ok = false; break; }
                mbar_arrive_expect_tx(v_full(s), TILE);
                for (int c = 0; c < D / 64; ++c)
                    tma_load_4d(v_smem + s * TILE + c * CHUNK, &tmap_v, v_full(s), c * 64,
                                j * kAttnBlock, h / p.kv_group, b);
            }
            if (!ok) {
                for (int i = 0; i < 64; ++i) __nanosleep(2000);
            }
        }
    } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one()) {
            constexpr uint32_t idesc_qk = make_idesc_f16(Elem<T>::kIsBf16, 128, 128, 0, 0);
            constexpr uint32_t idesc_pv = make_idesc_f16(Elem<T>::kIsBf16, 128, OCOLS, 0, 1);
            bool ok = true;
            // Descriptor halves that never change: high word = stride offset 1024 B, version 1, 128-byte
            // swizzle; low word = address >> 4 (+ the leading offset for the N-major V operand).
            constexpr uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
            const uint32_t q_lo = (q_smem & 0x3FFFF) >> 4;
            const uint32_t k_lo = (k_smem & 0x3FFFF) >> 4;
            // leading offset of the V operand = distance to the next 64-column slab along N: the second
            // slab of D (D = 128) or the slab of ones (D = 64, added per stage below)
            const uint32_t v_lo = ((v_smem & 0x3FFFF) >> 4) | (kSumOnTc ? 0u : ((uint32_t)(CHUNK >> 4) << 16));
            auto desc = [&](uint32_t lo) { return ((uint64_t)desc_hi << 32) | (uint64_t)lo; };
            auto issue_qk = [&](int t, int s) {
                const uint32_t a_lo = q_lo + (uint32_t)(t * (TILE >> 4));
                const uint32_t b_lo = k_lo + (uint32_t)(s * (TILE >> 4));
                const uint32_t d_tmem = tmem_base + (uint32_t)(t * 128);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t off = (uint32_t)(((ks / 4) * CHUNK + (ks % 4) * 32) >> 4);
                    tc_mma_ss(d_tmem, desc(a_lo + off), desc(b_lo + off), idesc_qk, ks > 0 ? 1u : 0u);
                }
            };
            auto issue_pv = [&](int t, int s, bool accumulate) {
                uint32_t b_lo = v_lo + (uint32_t)(s * (TILE >> 4));
                if (kSumOnTc) b_lo |= (uint32_t)((ones_smem - (v_smem + s * TILE)) >> 4) << 16;
                const uint32_t d_tmem = tmem_base + (uint32_t)(256 + t * 128);
                const uint32_t a_tmem = tmem_base + (uint32_t)(t * 128);
#pragma unroll
                for (int ks = 0; ks < kAttnBlock / 16; ++ks) {
                    // 16 keys = 16 rows of 128 bytes = 2048 B; the second 64-wide slab of D is CHUNK bytes away
                    tc_mma_ts(d_tmem, a_tmem + (uint32_t)(ks * 8), desc(b_lo + (uint32_t)(ks * (2048 >> 4))), idesc_pv,
                              (accumulate || ks > 0) ? 1u : 0u);
                }
            };
            for (int t = 0; t < ntl && ok; ++t)
                if (!mbar_wait(q_full(t), 0, abort_flag, 200)) ok = false;
            if (ok && max_blk > 0) {
                if (!mbar_wait(k_full(0), 0, abort_flag, 201)) ok = false;
                if (ok) {
                    tc_fence_after();
                    for (int t = 0; t < ntl; ++t) {
                        if (nblk[t] > 0) {
                            issue_qk(t, 0);
                            tc_commit(s_full(t));
                        }
                    }
                    tc_commit(k_empty(0));
                }
            }
            for (int j = 0; j < max_blk && ok; ++j) {
                const int s = j % KVS;
                const uint32_t ph = (uint32_t)((j / KVS) & 1);
                const int s1 = (j + 1) % KVS;
                const uint32_t ph1 = (uint32_t)(((j + 1) / KVS) & 1);
                if (!mbar_wait(v_full(s), ph, abort_flag, 202)) { ok = false; break; }
                if (j + 1 < max_blk) {
                    if (!mbar_wait(k_full(s1), ph1, abort_flag, 203)) { ok = false; break; }
                }
                for (int t = 0; t < ntl; ++t) {
                    if (j >= nblk[t]) continue;
                    if (!mbar_wait(p_full(t), (uint32_t)(j & 1), abort_flag, 204)) { ok = false; break; }
                    tc_fence_after();
                    issue_pv(t, s, j > 0);
                    if (j + 1 < nblk[t]) {
                        issue_qk(t, s1);
                        tc_commit(s_full(t));
                    } else {
                        tc_commit(o_final(t));
                    }
                }
                if (!ok) break;
                tc_commit(v_empty(s));
                if (j + 1 < max_blk) tc_commit(k_empty(s1));
            }
        }
      } else if (MODE == 1) {
        // ------------------------------------------------------------------ mask loaders (warps 10, 11)
        const int li = (int)threadIdx.x - 320;  // 0..63, two columns each
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
                    const int idx = li + e * 64;
                    const int col = j * kAttnBlock + idx;
                    float a = -INFINITY;
                    if (col < p.N)
                        a = fmaxf(mask_load(p.mask, moff + (int64_t)col * p.mask_strides[3], p.mask_dtype), mlow) * kLog2e;
                    mask_smem[(t * 2 + bf) * kAttnBlock + idx] = a;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(m_full(t, bf));
            }
        }
      }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kAttnRegsHigh));
        // ------------------------------------------------------------------ softmax groups
        const int t = warp >> 2;        // tile handled by this group
        const int q = warp & 3;         // TMEM lane quadrant of this warp
        if (t < ntl && nblk[t] > 0) {
            const int row = mt[t] * kAttnBlock + q * 32 + lane;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
            const uint32_t s_addr = lane_addr + (uint32_t)(t * 128);
            const uint32_t o_addr = lane_addr + (uint32_t)(256 + t * 128);
            const float c = p.scale_log2;
            const float mlow = mask_lowest(p.mask_dtype);
            const int64_t mask_row_off =
                (MODE == 2 && p.mask != nullptr)
                    ? (int64_t)b * p.mask_strides[0] + (int64_t)h * p.mask_strides[1] + (int64_t)min(row, p.M - 1) * p.mask_strides[2]
                    : 0;
            // In MODE 0 the running maximum is kept in raw score units and the exponent is
            // (s - m_ref) * c; otherwise scores are first moved to the log2 domain (s*c + mask).
            const float unit = (MODE == 0) ? c : 1.0f;
            float m_ref = -INFINITY;
            float l = 0.f;
            bool ok = true;
            for (int j = 0; j < nblk[t]; ++j) {
                if (!mbar_wait(s_full(t), (uint32_t)(j & 1), abort_flag, 300 + t)) { ok = false; break; }
                tc_fence_after();
                uint32_t sr[4][32];
#pragma unroll
                for (int cch = 0; cch < 4; ++cch) tmem_ld_32x32(s_addr + cch * 32, sr[cch]);
                tmem_ld_wait();

                const int col0 = j * kAttnBlock;
                const bool causal_edge = p.is_causal && col0 + kAttnBlock - 1 > mt[t] * kAttnBlock;
                if (MODE == 1) {
                    const int bf = j & 1;
                    if (!mbar_wait(m_full(t, bf), (uint32_t)((j >> 1) & 1), abort_flag, 320 + t)) { ok = false; break; }
                    const float4* ms = reinterpret_cast<const float4*>(mask_smem + (t * 2 + bf) * kAttnBlock);
#pragma unroll
                    for (int cch = 0; cch < 4; ++cch) {
#pragma unroll
                        for (int v4 = 0; v4 < 8; ++v4) {
                            const float4 a = ms[cch * 8 + v4];  // same address in every lane: broadcast
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
                        for (int cch = 0; cch < 4; ++cch) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) sr[cch][i] = __float_as_uint(__uint_as_float(sr[cch][i]) * c);
                        }
                    } else {
#pragma unroll
                        for (int hc = 0; hc < 8; ++hc) {
                            const int colc = col0 + hc * 16;
                            float mvals[16];
                            if (p.mask_vec && colc + 16 <= p.N) {
                                // 16 consecutive mask values of this row as 128-bit loads
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
                // columns beyond N (already -inf in MODE 1) and, on the diagonal block, above the diagonal
                if ((MODE != 1 && col0 + kAttnBlock > p.N) || causal_edge) {
#pragma unroll
                    for (int cch = 0; cch < 4; ++cch) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int col = col0 + cch * 32 + i;
                            if (col >= p.N || (p.is_causal && col > row)) sr[cch][i] = __float_as_uint(-INFINITY);
                        }
                    }
                }
                // ---- row maximum (three-input max halves the instruction count)
                float mx4[4];
#pragma unroll
                for (int cch = 0; cch < 4; ++cch) {
                    float mloc = fmaxf(__uint_as_float(sr[cch][0]), __uint_as_float(sr[cch][1]));
#pragma unroll
                    for (int i = 2; i < 32; i += 2) mloc = fmax3(mloc, __uint_as_float(sr[cch][i]), __uint_as_float(sr[cch][i + 1]));
                    mx4[cch] = mloc;
                }
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
                // ---- lazy rescale
                float m_new = fmaxf(m_ref, mx);
                if (m_new == -INFINITY) m_new = 0.f;  // row with nothing visible yet
                const bool grow = (m_new - m_ref) * unit > kLazyThreshold;  // also true on the first block
                float alpha = 1.0f;
                if (grow) {
                    alpha = (m_ref == -INFINITY) ? 0.f : fast_exp2((m_ref - m_new) * unit);
                    m_ref = m_new;
                    l *= alpha;
                }
                if (j > 0 && __any_sync(0xffffffffu, grow)) {
                    // S_j complete implies P·V of block j-1 complete (issued earlier, same thread), so O is quiescent.
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
                // ---- exponentials, row sum (four independent partial sums), pack to 16 bit, write P over
                //      the first 64 columns of S
                const float neg_ref = -m_ref * unit;
                float lp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int cch = 0; cch < 4; ++cch) {
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
                if (lane == 0) mbar_arrive(p_full(t));
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
                        float val[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) val[i] = __uint_as_float(orr[i]) * inv_l;
                        if (dch * 32 + 32 <= p.d_out) attn_store_32<T, false>(o_row, dch * 32, p.o_strides[3], vec, val, p.d_out);
                        else attn_store_32<T, true>(o_row, dch * 32, p.o_strides[3], vec, val, p.d_out);
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
static int launch_attention_tdm(const kb_attn_params& p, cudaStream_t stream) {
    using Cfg = AttnCfg<D>;
    CUtensorMap tq, tk, tv;
    const int64_t kv_group = p.kv_group > 1 ? p.kv_group : 1;
    if (p.H % kv_group != 0) return KB_ERR_BAD_ARG;
    auto enc = [&](CUtensorMap* out, const void* ptr, int64_t rows, const int64_t* st, int64_t heads) -> int {
        if (st[3] != 1) return KB_ERR_UNSUPPORTED;
        const uint64_t dims[4] = {(uint64_t)p.D, (uint64_t)rows, (uint64_t)heads, (uint64_t)p.B};  // boxes reach to D: zero fill
        // A dimension of extent 1 may carry any stride in the caller's tensor; TMA still wants a
        // multiple of 16 bytes, and the value is never used, so substitute a harmless one.
        auto fix = [](int64_t extent, int64_t stride) -> uint64_t {
            return (extent == 1) ? 16u : (uint64_t)stride * 2u;
        };
        const uint64_t strides[4] = {0, fix(rows, st[2]), fix(heads, st[1]), fix(p.B, st[0])};
        const uint32_t box[4] = {64, (uint32_t)kAttnBlock, 1, 1};
        return encode_tmap_16bit(out, ptr, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    };
    int st = enc(&tq, p.q, p.M, p.q_strides, p.H);
    if (st != KB_OK) return st;
    st = enc(&tk, p.k, p.N, p.k_strides, p.H / kv_group);
    if (st != KB_OK) return st;
    st = enc(&tv, p.v, p.N, p.v_strides, p.H / kv_group);
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
        const int64_t per16 = (p.mask_dtype == KB_F32) ? 4 : 8;  // elements per 16 bytes
        d.mask_vec = (p.mask_strides[0] % per16 == 0 && p.mask_strides[1] % per16 == 0 && p.mask_strides[2] % per16 == 0) ? 1 : 0;
    }
    const int num_m_tiles = (int)((p.M + kAttnBlock - 1) / kAttnBlock);
    d.num_pairs = (num_m_tiles + 1) / 2;
    d.head_group = attn_head_group(p.B * p.H, p.N, p.D);
    d.kv_group = (int)kv_group;
    d.d_out = (int)p.D;

    static PerDeviceOnce attr_once;
    if (attr_once.first_time()) {
        if (cudaFuncSetAttribute(attention_tc_kernel<T, D, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 Cfg::kSmemBytes) != cudaSuccess)
            return KB_ERR_LAUNCH;
    }
    const int64_t grid = (int64_t)d.num_pairs * p.B * p.H;
    if (grid > 0x7fffffff) return KB_ERR_UNSUPPORTED;
    attention_tc_kernel<T, D, MODE><<<(unsigned)grid, kAttnThreads, Cfg::kSmemBytes, stream>>>(tq, tk, tv, d);
    return cudaGetLastError() == cudaSuccess ? KB_OK : KB_ERR_LAUNCH;
}

template <typename T, int D>
static int launch_attention_td(const kb_attn_params& p, cudaStream_t stream) {
    if (p.mask == nullptr && p.sm_scale > 0.f) return launch_attention_tdm<T, D, 0>(p, stream);
    if (p.mask != nullptr && p.mask_strides[2] == 0) return launch_attention_tdm<T, D, 1>(p, stream);
    return launch_attention_tdm<T, D, 2>(p, stream);
}

static int launch_attention128(const kb_attn_params& p, cudaStream_t stream) {
    if (p.N <= 0) return KB_ERR_UNSUPPORTED;
    if (p.M > 0x7fffffff || p.N > 0x7fffffff || p.B * p.H > 0x7fffffff) return KB_ERR_UNSUPPORTED;
    // head dimensions up to 64 are served by attention_split.cuh; 72 ... 128 run here on the D = 128 kernel
    if (p.D <= 64 || p.D > 128 || p.D % 8 != 0) return KB_ERR_UNSUPPORTED;
    if (p.dtype == KB_F16) return launch_attention_td<__half, 128>(p, stream);
    if (p.dtype == KB_BF16) return launch_attention_td<__nv_bfloat16, 128>(p, stream);
    return KB_ERR_UNSUPPORTED;
}

}  // namespace kb
