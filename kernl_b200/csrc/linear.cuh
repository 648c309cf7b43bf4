// Fused linear layer y = act(x · Wᵀ + bias) for sm_100a.
//
// Persistent, warp-specialised tcgen05 GEMM:
//   warp 0      TMA producer: x tile [128 x 64] and W tile [BN x 64] per stage, 128-byte swizzle
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (M=128, N=BN, K=16) x 4 per stage,
//               accumulators in TMEM, double-buffered (2 x BN columns) so that the epilogue of tile
//               i overlaps the main loop of tile i+1
//   warps 2..9  epilogue (two warps per TMEM lane quadrant, each taking half of the tile's columns):
//               tcgen05.ld of the accumulator (one row per thread), + bias, activation in fp32,
//               convert, store
// Split-K: when a problem has fewer output tiles than SMs (few rows: the weight matrix is then
// streamed from HBM by too few SMs), the K range of every tile is cut into `splits` work items; the
// items add their fp32 partial tiles into a caller-provided, zero-initialised workspace with vector
// atomics, and a small second kernel applies bias + activation, converts, and writes the zeros back.
// (Letting the last-arriving epilogue warp finish its slice inside the GEMM kernel was tried and was
// slower: the finishing warps serialise on L2 round trips that a separate, fully parallel pass hides.)
// Both operands are K-major (x is [M,K], W is [N,K]) which is exactly what tcgen05 wants, so
// no transposes are needed. Ragged M / N / K edges rely on TMA zero fill for loads and on
// predicated stores.
#pragma once
#include "common.cuh"

namespace kb {

constexpr int kGemmBM = 128;
constexpr int kGemmBK = 64;
constexpr int kGemmThreads = 320;
constexpr int kGemmEpilogueWarps = 8;

template <int BN>
struct GemmCfg {
    static constexpr int kStages = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
    static constexpr int kABytes = kGemmBM * kGemmBK * 2;
    static constexpr int kBBytes = BN * kGemmBK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
    // tiles + barriers/flags + slack for the 1024-byte alignment of the tiles
    static constexpr int kSmemBytes = kStages * kStageBytes + 256 + 1024;
};

// Activations of the epilogue, evaluated on the fp32 accumulator (+bias).
// tanh uses the hardware tanh.approx (relative error about 2^-11, far below the rounding of the
// 16-bit output); GELU (the erf form of the reference, activation_func.py) is described below.
__device__ __forceinline__ float act_tanh(float z) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(z));
    return y;
}
// GELU(z) = z·Φ(z) written as relu(z) − |z|·Φ(−|z|), with Φ(−a) = ½·erfc(a/√2) = 2^P(a): P is a
// degree-6 fit of log2(½·erfc(a/√2)) on [0, 5.5] (weighted for the error that reaches the output),
// |z| is clamped to 5.5 (beyond it |z|·Φ(−|z|) < 1.1e-7). Maximum absolute error against the
// erf form in double precision: 1.1e-7 over [−8, 8], at one
// special-function instruction and eight arithmetic ones per value; the f32x2 form evaluates two
// values per instruction. (The erf form cost more issue slots than a short main loop leaves to the
// epilogue warps.)
constexpr float kGeluP0 = -0.999993085861206f, kGeluP1 = -1.1512017250061035f, kGeluP2 = -0.4587709605693817f,
                kGeluP3 = -0.053412117063999176f, kGeluP4 = 0.008080724626779556f, kGeluP5 = -0.0007692216895520687f,
                kGeluP6 = 3.3092990634031594e-05f;
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float act_gelu(float z) {
    const float a = fminf(fabsf(z), 5.5f);
    float pl = fmaf(kGeluP6, a, kGeluP5);
    pl = fmaf(pl, a, kGeluP4);
    pl = fmaf(pl, a, kGeluP3);
    pl = fmaf(pl, a, kGeluP2);
    pl = fmaf(pl, a, kGeluP1);
    pl = fmaf(pl, a, kGeluP0);
    return fmaf(-a, ex2_approx(pl), fmaxf(z, 0.0f));
}
__device__ __forceinline__ float2 act_gelu2(float2 z) {
    const float2 a = make_float2(fminf(fabsf(z.x), 5.5f), fminf(fabsf(z.y), 5.5f));
    float2 pl = __ffma2_rn(make_float2(kGeluP6, kGeluP6), a, make_float2(kGeluP5, kGeluP5));
    pl = __ffma2_rn(pl, a, make_float2(kGeluP4, kGeluP4));
    pl = __ffma2_rn(pl, a, make_float2(kGeluP3, kGeluP3));
    pl = __ffma2_rn(pl, a, make_float2(kGeluP2, kGeluP2));
    pl = __ffma2_rn(pl, a, make_float2(kGeluP1, kGeluP1));
    pl = __ffma2_rn(pl, a, make_float2(kGeluP0, kGeluP0));
    const float2 g = make_float2(ex2_approx(pl.x), ex2_approx(pl.y));
    return __ffma2_rn(make_float2(-a.x, -a.y), g, make_float2(fmaxf(z.x, 0.0f), fmaxf(z.y, 0.0f)));
}
__device__ __forceinline__ float act_fast_gelu(float z) {
    return 0.5f * z * (1.0f + act_tanh(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float act_silu(float z) { return __fdividef(z, 1.0f + __expf(-z)); }

__device__ __forceinline__ void tile_coords(int t, int num_m, int num_n, int& m_idx, int& n_idx) {
    // Grouped rasterisation: 8 row-tiles share each sweep over the column tiles so that the
    // CTAs running at the same time reuse W and x tiles out of L2.
    constexpr int kGroupM = 8;
    const int group_size = kGroupM * num_n;
    const int group_id = t / group_size;
    const int first_m = group_id * kGroupM;
    const int gsz = min(num_m - first_m, kGroupM);
    const int r = t % group_size;
    m_idx = first_m + r % gsz;
    n_idx = r / gsz;
}

// Epilogue of one 32-column chunk of one output row: z = acc + bias; optional store of z
// (pre-activation); y = act(z) as 16-bit, 128-bit stores when the chunk is whole and aligned.
template <typename T>
__device__ __forceinline__ void epilogue_chunk(const float (&accv)[32], const T* __restrict__ bias,
                                               T* __restrict__ y_row, T* __restrict__ a_row, int col0,
                                               int N, bool row_ok, int activation) {
    const bool full_chunk = (col0 + 32 <= N);
    float z[32];
    if (bias != nullptr) {
        if (full_chunk && (((uintptr_t)(bias + col0)) & 15) == 0) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const uint4 bw = __ldg(reinterpret_cast<const uint4*>(bias + col0) + v);
                const uint32_t w[4] = {bw.x, bw.y, bw.z, bw.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 bf = Elem<T>::unpack2(w[i]);
                    z[v * 8 + 2 * i] = accv[v * 8 + 2 * i] + bf.x;
                    z[v * 8 + 2 * i + 1] = accv[v * 8 + 2 * i + 1] + bf.y;
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float b = (col0 + j < N) ? Elem<T>::to_f32(bias[col0 + j]) : 0.f;
                z[j] = accv[j] + b;
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) z[j] = accv[j];
    }
    if (!row_ok) return;
    const bool vec = full_chunk && ((((uintptr_t)(y_row + col0)) & 15) == 0) &&
                     (a_row == nullptr || (((uintptr_t)(a_row + col0)) & 15) == 0);
    if (a_row != nullptr) {
        if (vec) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                uint4 o;
                o.x = Elem<T>::pack2(z[v * 8 + 0], z[v * 8 + 1]);
                o.y = Elem<T>::pack2(z[v * 8 + 2], z[v * 8 + 3]);
                o.z = Elem<T>::pack2(z[v * 8 + 4], z[v * 8 + 5]);
                o.w = Elem<T>::pack2(z[v * 8 + 6], z[v * 8 + 7]);
                reinterpret_cast<uint4*>(a_row + col0)[v] = o;
            }
        } else {
            for (int j = 0; j < 32; ++j)
                if (col0 + j < N) a_row[col0 + j] = Elem<T>::from_f32(z[j]);
        }
    }
    // The switch sits outside the element loop so that each case unrolls over registers.
    switch (activation) {
        case KB_ACT_TANH:
#pragma unroll
            for (int j = 0; j < 32; ++j) z[j] = act_tanh(z[j]);
            break;
        case KB_ACT_GELU:
#pragma unroll
            for (int j = 0; j < 32; ++j) z[j] = act_gelu(z[j]);
            break;
        case KB_ACT_FAST_GELU:
#pragma unroll
            for (int j = 0; j < 32; ++j) z[j] = act_fast_gelu(z[j]);
            break;
        case KB_ACT_RELU:
#pragma unroll
            for (int j = 0; j < 32; ++j) z[j] = fmaxf(z[j], 0.0f);
            break;
        case KB_ACT_SILU:
#pragma unroll
            for (int j = 0; j < 32; ++j) z[j] = act_silu(z[j]);
            break;
        default: break;
    }
    if (vec) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            uint4 o;
            o.x = Elem<T>::pack2(z[v * 8 + 0], z[v * 8 + 1]);
            o.y = Elem<T>::pack2(z[v * 8 + 2], z[v * 8 + 3]);
            o.z = Elem<T>::pack2(z[v * 8 + 4], z[v * 8 + 5]);
            o.w = Elem<T>::pack2(z[v * 8 + 6], z[v * 8 + 7]);
            reinterpret_cast<uint4*>(y_row + col0)[v] = o;
        }
    } else {
        for (int j = 0; j < 32; ++j)
            if (col0 + j < N) y_row[col0 + j] = Elem<T>::from_f32(z[j]);
    }
}

// z = act(z) in place for NV values (an even count) of one output row.
template <int NV>
__device__ __forceinline__ void apply_activation(float (&z)[NV], int activation) {
    switch (activation) {
        case KB_ACT_TANH:
#pragma unroll
            for (int j = 0; j < NV; ++j) z[j] = act_tanh(z[j]);
            break;
        case KB_ACT_GELU:
#pragma unroll
            for (int j = 0; j < NV; j += 2) {
                const float2 g = act_gelu2(make_float2(z[j], z[j + 1]));
                z[j] = g.x;
                z[j + 1] = g.y;
            }
            break;
        case KB_ACT_FAST_GELU:
#pragma unroll
            for (int j = 0; j < NV; ++j) z[j] = act_fast_gelu(z[j]);
            break;
        case KB_ACT_RELU:
#pragma unroll
            for (int j = 0; j < NV; ++j) z[j] = fmaxf(z[j], 0.0f);
            break;
        case KB_ACT_SILU:
#pragma unroll
            for (int j = 0; j < NV; ++j) z[j] = act_silu(z[j]);
            break;
        default: break;
    }
}

// Gated epilogue (KB_ACT_SWIGLU) of one 32-column chunk: the rows of W are interleaved in blocks of
// eight — block 2j holds gate rows 8j..8j+7, block 2j+1 the matching up rows — so a chunk carries
// two gate/up block pairs and yields 16 output columns y[col0/2 + i] = silu(gate_i) * up_i, computed
// from the fp32 accumulators (the [M, 2F] intermediate never exists). N is a multiple of 16, so a
// chunk holds whole pairs or none.
template <typename T>
__device__ __forceinline__ void epilogue_chunk_swiglu(const float (&accv)[32], const T* __restrict__ bias,
                                                      T* __restrict__ y_row, int col0, int N, bool row_ok) {
    float z[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) z[j] = accv[j];
    if (bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col0 + j < N) z[j] += Elem<T>::to_f32(__ldg(bias + col0 + j));
    }
    if (!row_ok) return;
    float o[16];
#pragma unroll
    for (int blk = 0; blk < 2; ++blk)
#pragma unroll
        for (int i = 0; i < 8; ++i) o[blk * 8 + i] = act_silu(z[blk * 16 + i]) * z[blk * 16 + 8 + i];
    T* dst = y_row + col0 / 2;
    const bool aligned = (((uintptr_t)dst) & 15) == 0;
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
        if (col0 + blk * 16 >= N) break;
        if (aligned) {
            uint4 v;
            v.x = Elem<T>::pack2(o[blk * 8 + 0], o[blk * 8 + 1]);
            v.y = Elem<T>::pack2(o[blk * 8 + 2], o[blk * 8 + 3]);
            v.z = Elem<T>::pack2(o[blk * 8 + 4], o[blk * 8 + 5]);
            v.w = Elem<T>::pack2(o[blk * 8 + 6], o[blk * 8 + 7]);
            reinterpret_cast<uint4*>(dst)[blk] = v;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[blk * 8 + i] = Elem<T>::from_f32(o[blk * 8 + i]);
        }
    }
}

template <typename T, int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
linear_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                 const T* __restrict__ bias, T* __restrict__ y, T* __restrict__ act_inputs, int M,
                 int N, int K, int64_t y_row_stride, int activation, int splits, int kps,
                 float* __restrict__ ws) {
    using Cfg = GemmCfg<BN>;
    constexpr int STAGES = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::kStageBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // Launched with programmatic dependent launch: the barriers and the descriptor prefetch touch no
    // global memory and may run while the previous kernel of the stream drains (a few-row GEMM of a
    // latency-bound graph is itself only a few microseconds long).
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), kGemmEpilogueWarps);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tmap_x);
        tma_prefetch_desc(&tmap_w);
    }
    pdl_wait();
    // A wait that expired in an earlier CTA or launch leaves the status word set: do no work until
    // the host has read (and cleared) it, so that one failure cannot cost a second per CTA.
    {
        __shared__ int s_skip;
        if (threadIdx.x == 0) s_skip = *reinterpret_cast<volatile int*>(&g_device_status[0]);
        __syncthreads();
        if (s_skip != 0) return;
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), Cfg::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int num_m = (M + kGemmBM - 1) / kGemmBM;
    const int num_n = (N + BN - 1) / BN;
    const int num_tiles = num_m * num_n;
    const int num_k = (K + kGemmBK - 1) / kGemmBK;
    // work item w -> (tile = w % num_tiles, split = w / num_tiles); split s covers k-blocks
    // [s*kps, min(num_k, (s+1)*kps)), never empty by construction of `splits`
    const int num_items = num_tiles * splits;

    if (warp == 0) {
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < num_items && ok; w += gridDim.x) {
                int m_idx, n_idx;
                tile_coords(w % num_tiles, num_m, num_n, m_idx, n_idx);
                const int kb0 = (w / num_tiles) * kps, kb1 = min(num_k, kb0 + kps);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, 100)) { ok = false; break; }
                    mbar_arrive_expect_tx(full_bar(stage), Cfg::kStageBytes);
                    const uint32_t a_dst = smem_base + stage * Cfg::kStageBytes;
                    tma_load_2d(a_dst, &tmap_x, full_bar(stage), kb * kGemmBK, m_idx * kGemmBM);
                    tma_load_2d(a_dst + Cfg::kABytes, &tmap_w, full_bar(stage), kb * kGemmBK,
                                n_idx * BN);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                // Give copies that are still in flight a bounded chance to land before the CTA's
                // shared memory is released.
                for (int i = 0; i < 64; ++i) __nanosleep(2000);
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t idesc = make_idesc_f16(Elem<T>::kIsBf16, kGemmBM, BN, 0, 0);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < num_items && ok; w += gridDim.x) {
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1, abort_flag, 200)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                const int kb0 = (w / num_tiles) * kps, kb1 = min(num_k, kb0 + kps);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, 201)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_base + stage * Cfg::kStageBytes;
                    const uint64_t a_desc = make_smem_desc_sw128(a_addr, 16, 1024);
                    const uint64_t b_desc = make_smem_desc_sw128(a_addr + Cfg::kABytes, 16, 1024);
#pragma unroll
                    for (int k = 0; k < kGemmBK / 16; ++k) {
                        // +32 bytes along K inside the 128-byte swizzle row = +2 in the address field
                        tc_mma_ss(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc,
                                  (kb > kb0 || k > 0) ? 1u : 0u);
                    }
                    tc_commit(empty_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                tc_commit(tfull_bar(acc));
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
        }
    } else {
        const int q = warp & 3;  // TMEM lane quadrant this warp may access
        const int col_half = (warp - 2) >> 2;  // which half of the tile's columns this warp handles
        constexpr int kHalfCols = BN / 2 >= 32 ? BN / 2 : 32;
        const int c_begin = col_half * kHalfCols;
        const int c_end = (BN >= 64) ? c_begin + kHalfCols : (col_half == 0 ? BN : 0);
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < num_items && ok; w += gridDim.x) {
            int m_idx, n_idx;
            tile_coords(w % num_tiles, num_m, num_n, m_idx, n_idx);
            if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, 300)) { ok = false; break; }
            tc_fence_after();
            const int row = m_idx * kGemmBM + q * 32 + lane;
            const int n0 = n_idx * BN;
            T* y_row = y + (int64_t)row * y_row_stride;
            T* a_row = act_inputs ? act_inputs + (int64_t)row * y_row_stride : nullptr;
#pragma unroll 1
            for (int c0 = c_begin; c0 < c_end; c0 += 32) {
                if (n0 + c0 >= N) break;
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c0), r);
                tmem_ld_wait();
                const int col0 = n0 + c0;
                const bool full_chunk = (col0 + 32 <= N);
                if (splits > 1) {
                    // partial tile: fp32 vector atomics into the workspace [M, N]
                    if (row < M) {
                        float* wrow = ws + (int64_t)row * N + col0;
                        if (full_chunk && ((((uintptr_t)wrow) & 15) == 0)) {
#pragma unroll
                            for (int v = 0; v < 8; ++v) {
                                atomicAdd(reinterpret_cast<float4*>(wrow) + v,
                                          make_float4(__uint_as_float(r[v * 4 + 0]), __uint_as_float(r[v * 4 + 1]),
                                                      __uint_as_float(r[v * 4 + 2]), __uint_as_float(r[v * 4 + 3])));
                            }
                        } else {
                            for (int j = 0; j < 32; ++j)
                                if (col0 + j < N) atomicAdd(wrow + j, __uint_as_float(r[j]));
                        }
                    }
                    continue;
                }
                float accv[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) accv[j] = __uint_as_float(r[j]);
                if (activation == KB_ACT_SWIGLU) epilogue_chunk_swiglu<T>(accv, bias, y_row, col0, N, row < M);
                else epilogue_chunk<T>(accv, bias, y_row, a_row, col0, N, row < M, activation);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(acc));
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
    }

    // Teardown: every role falls through to here, also after an abandoned wait. This CTA takes no
    // more work: a dependent launch may have the slots that free up.
    pdl_launch_dependents();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// Second pass of a split-K launch: y = act(workspace + bias), four columns per thread; the sums are
// replaced by zeros as they are read, so the workspace is clean again for the next call.
template <typename T>
__global__ void __launch_bounds__(256)
linear_splitk_finish_kernel(float* __restrict__ ws, const T* __restrict__ bias, T* __restrict__ y,
                            T* __restrict__ act_inputs, int M, int N, int64_t y_row_stride, int activation) {
    // (no early trigger: what follows is often another GEMM, whose CTAs would sit on the SMs with all
    // their registers and shared memory while this kernel's CTAs still look for room)
    pdl_wait();
    const int nq = (N + 3) / 4;
    const int64_t total = (int64_t)M * nq;
    const bool vec4 = (N % 4) == 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int row = (int)(i / nq), c0 = (int)(i % nq) * 4;
        float z[4] = {0.f, 0.f, 0.f, 0.f};
        float* wp = ws + (int64_t)row * N + c0;
        if (vec4) {
            const float4 f = __ldcg(reinterpret_cast<const float4*>(wp));
            __stcg(reinterpret_cast<float4*>(wp), make_float4(0.f, 0.f, 0.f, 0.f));
            z[0] = f.x; z[1] = f.y; z[2] = f.z; z[3] = f.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (c0 + j < N) { z[j] = __ldcg(wp + j); __stcg(wp + j, 0.f); }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (bias != nullptr && c0 + j < N) z[j] += Elem<T>::to_f32(bias[c0 + j]);
        if (act_inputs) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (c0 + j < N) act_inputs[(int64_t)row * y_row_stride + c0 + j] = Elem<T>::from_f32(z[j]);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float v = z[j];
            switch (activation) {
                case KB_ACT_TANH: v = act_tanh(v); break;
                case KB_ACT_GELU: v = act_gelu(v); break;
                case KB_ACT_FAST_GELU: v = act_fast_gelu(v); break;
                case KB_ACT_RELU: v = fmaxf(v, 0.f); break;
                case KB_ACT_SILU: v = act_silu(v); break;
                default: break;
            }
            if (c0 + j < N) y[(int64_t)row * y_row_stride + c0 + j] = Elem<T>::from_f32(v);
        }
    }
}

// Second pass of a split-K launch with the gated epilogue (KB_ACT_SWIGLU): four output columns per
// thread, read from the gate block and the up block eight columns further (see epilogue_chunk_swiglu).
template <typename T>
__global__ void __launch_bounds__(256)
linear_splitk_finish_swiglu_kernel(float* __restrict__ ws, const T* __restrict__ bias, T* __restrict__ y, int M,
                                   int N, int64_t y_row_stride) {
    pdl_wait();
    const int nq = N / 8;  // N / 2 output columns, four per thread
    const int64_t total = (int64_t)M * nq;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int row = (int)(i / nq), oc0 = (int)(i % nq) * 4;
        const int gc = (oc0 >> 3) * 16 + (oc0 & 7);  // gate column; the up column is gc + 8
        float* wp = ws + (int64_t)row * N + gc;
        const float4 g4 = __ldcg(reinterpret_cast<const float4*>(wp));
        const float4 u4 = __ldcg(reinterpret_cast<const float4*>(wp + 8));
        __stcg(reinterpret_cast<float4*>(wp), zero);
        __stcg(reinterpret_cast<float4*>(wp + 8), zero);
        float g[4] = {g4.x, g4.y, g4.z, g4.w}, u[4] = {u4.x, u4.y, u4.z, u4.w};
        if (bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                g[j] += Elem<T>::to_f32(bias[gc + j]);
                u[j] += Elem<T>::to_f32(bias[gc + 8 + j]);
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) y[(int64_t)row * y_row_stride + oc0 + j] = Elem<T>::from_f32(act_silu(g[j]) * u[j]);
    }
}

// Split-K workspace: fp32 partial sums [M, N]. It must be all zero before the first call that uses
// it; every call leaves it zero again (the finishing kernel writes the zeros back as it reads).
static int64_t splitk_workspace_bytes(int64_t M, int64_t N) { return ((M * N * (int64_t)sizeof(float)) + 15) / 16 * 16; }
// Splitting pays only while the extra pass over the output is small next to streaming W once:
// few row tiles and a bounded output.
static bool splitk_allowed(int64_t M, int64_t N) { return M <= 1024 && M * N <= (int64_t)4 << 20; }

struct LinearPlan {
    int bn;      // column-tile width
    int splits;  // K splits per tile (1 = none)
    int kps;     // k-blocks per split
};

// Cost model, in units of "bytes staged per SM": waves of work items x k-blocks per item (+2 for the
// fixed per-item cost) x bytes per k-block. Wide tiles re-stream x less often; splitting K fills the
// SMs when there are few tiles (few rows: the op is then bound by streaming W from HBM once, and
// what counts is how many SMs pull on it and how many bytes each keeps in flight).
static LinearPlan plan_linear(int64_t M, int64_t N, int64_t K, bool has_ws, int forced_bn, int forced_splits) {
    const int sms = gemm_sms();
    const int64_t num_m = (M + kGemmBM - 1) / kGemmBM;
    const int num_k = (int)((K + kGemmBK - 1) / kGemmBK);
    LinearPlan best{32, 1, num_k};
    double best_cost = 1e300;
    for (int bn : {256, 128, 64, 32}) {
        if (forced_bn != 0 && bn != forced_bn) continue;
        const int64_t tiles = num_m * ((N + bn - 1) / bn);
        const int max_splits = has_ws ? (num_k / 2 < 1 ? 1 : (num_k / 2 > 32 ? 32 : num_k / 2)) : 1;
        for (int s = 1; s <= max_splits; ++s) {
            if (forced_splits != 0 && s != forced_splits && !(forced_splits > max_splits && s == max_splits)) continue;
            const int kps = (num_k + s - 1) / s;
            const int eff = (num_k + kps - 1) / kps;  // splits that are not empty
            if (eff != s) continue;
            const int64_t waves = (tiles * s + sms - 1) / sms;
            double cost = (double)waves * ((double)kps + 2.0) * (double)(kGemmBM + bn);
            if (s > 1) {
                // Splitting K is not free: every split adds its tile into the fp32 workspace with
                // atomics (8 bytes of traffic per output element and split) and a second kernel reads
                // the sums back, applies the epilogue and clears the workspace. Measured on B200: about
                // 2.6 µs for the extra launch plus the traffic at ~2 TB/s, against ~0.13 µs per k-block of
                // a 128x32 tile (0.0008 µs per cost unit). With the earlier, far smaller penalty the
                // heuristic split [512,768]x[3072,768] (25 µs instead of 10) and [128,4096]x[11008,4096]
                // (33 µs instead of 21).
                const double mn = (double)M * (double)N;
                const double extra_us = 2.6 + (double)s * mn * 8.0 / 2.0e6 + mn * 6.0 / 3.0e6;
                cost += extra_us / 0.0008;
            }
            if (cost < best_cost) {
                best_cost = cost;
                best = LinearPlan{bn, s, kps};
            }
        }
    }
    return best;
}

template <typename T, int BN>
static int launch_linear_bn(const kb_linear_params& p, cudaStream_t stream, const LinearPlan& plan) {
    using Cfg = GemmCfg<BN>;
    CUtensorMap tmap_x, tmap_w;
    {
        const uint64_t dims[2] = {(uint64_t)p.K, (uint64_t)p.M};
        const uint64_t strides[2] = {0, (uint64_t)p.x_row_stride * 2};
        const uint32_t box[2] = {kGemmBK, kGemmBM};
        int st = encode_tmap_16bit(&tmap_x, p.x, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
        if (st != KB_OK) return st;
    }
    {
        const uint64_t dims[2] = {(uint64_t)p.K, (uint64_t)p.N};
        const uint64_t strides[2] = {0, (uint64_t)p.K * 2};
        const uint32_t box[2] = {kGemmBK, BN};
        int st = encode_tmap_16bit(&tmap_w, p.w, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
        if (st != KB_OK) return st;
    }
    static PerDeviceOnce attr_once;
    if (attr_once.first_time()) {
        cudaError_t e = cudaFuncSetAttribute(linear_tc_kernel<T, BN>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        if (e != cudaSuccess) return KB_ERR_LAUNCH;
    }
    const int64_t num_tiles = ((p.M + kGemmBM - 1) / kGemmBM) * ((p.N + BN - 1) / BN);
    const int64_t items = num_tiles * plan.splits;
    const int grid = (int)(items < gemm_sms() ? items : gemm_sms());
    float* ws = reinterpret_cast<float*>(p.workspace);
    // Programmatic launch for the few-row problems of latency-bound graphs only: there the kernel
    // before is small as well. Behind a kernel of thousands of CTAs, 148 early-resident GEMM CTAs
    // (all of an SM's shared memory, most of its registers) would take the room its later waves need.
    cudaError_t le;
    if (p.M <= 1024)
        le = launch_pdl(linear_tc_kernel<T, BN>, dim3((unsigned)grid), dim3(kGemmThreads), (size_t)Cfg::kSmemBytes, stream, tmap_x,
                        tmap_w, (const T*)p.bias, (T*)p.y, (T*)p.act_inputs, (int)p.M, (int)p.N, (int)p.K, p.y_row_stride,
                        p.activation, plan.splits, plan.kps, ws);
    else {
        linear_tc_kernel<T, BN><<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(
            tmap_x, tmap_w, (const T*)p.bias, (T*)p.y, (T*)p.act_inputs, (int)p.M, (int)p.N, (int)p.K, p.y_row_stride,
            p.activation, plan.splits, plan.kps, ws);
        le = cudaSuccess;
    }
    if (le != cudaSuccess) return KB_ERR_LAUNCH;
    if (cudaGetLastError() != cudaSuccess) return KB_ERR_LAUNCH;
    if (plan.splits > 1) {
        const bool gated = p.activation == KB_ACT_SWIGLU;
        const int64_t total = gated ? p.M * (p.N / 8) : p.M * ((p.N + 3) / 4);
        int64_t blocks = (total + 255) / 256;
        if (blocks > (int64_t)sm_count() * 8) blocks = (int64_t)sm_count() * 8;
        if (gated)
            launch_pdl(linear_splitk_finish_swiglu_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, ws, (const T*)p.bias,
                       (T*)p.y, (int)p.M, (int)p.N, p.y_row_stride);
        else
            launch_pdl(linear_splitk_finish_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, ws, (const T*)p.bias, (T*)p.y,
                       (T*)p.act_inputs, (int)p.M, (int)p.N, p.y_row_stride, p.activation);
        if (cudaGetLastError() != cudaSuccess) return KB_ERR_LAUNCH;
    }
    return KB_OK;
}

// Large problems go to CTA pairs on 256 x 256 tiles (linear_pair.cuh).
static bool linear_pair_applicable(const kb_linear_params& p);
template <typename T>
static int launch_linear_pair_t(const kb_linear_params& p, cudaStream_t stream);

template <typename T>
static int launch_linear_t(const kb_linear_params& p, cudaStream_t stream, int forced_bn, int forced_splits) {
    if (forced_bn == 0 && forced_splits == 0 && linear_pair_applicable(p)) return launch_linear_pair_t<T>(p, stream);
    const bool has_ws = p.workspace != nullptr && p.workspace_bytes >= splitk_workspace_bytes(p.M, p.N) &&
                        (((uintptr_t)p.workspace) & 15) == 0 && (splitk_allowed(p.M, p.N) || forced_splits > 1);
    const LinearPlan plan = plan_linear(p.M, p.N, p.K, has_ws, forced_bn, forced_splits);
    switch (plan.bn) {
        case 256: return launch_linear_bn<T, 256>(p, stream, plan);
        case 128: return launch_linear_bn<T, 128>(p, stream, plan);
        case 64: return launch_linear_bn<T, 64>(p, stream, plan);
        default: return launch_linear_bn<T, 32>(p, stream, plan);
    }
}

static int launch_linear(const kb_linear_params& p, cudaStream_t stream, int forced_bn, int forced_splits) {
    if (p.dtype == KB_F16) return launch_linear_t<__half>(p, stream, forced_bn, forced_splits);
    if (p.dtype == KB_BF16) return launch_linear_t<__nv_bfloat16>(p, stream, forced_bn, forced_splits);
    return KB_ERR_UNSUPPORTED;
}

// y = silu(g) * u with gu = [g | u] along columns.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ y, int64_t M, int64_t N) {
    pdl_wait();
    pdl_launch_dependents();
    const int64_t nvec = N / 8;
    const int64_t total = M * nvec;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t m = i / nvec, c = (i % nvec) * 8;
        const uint4 g = *reinterpret_cast<const uint4*>(gu + m * 2 * N + c);
        const uint4 u = *reinterpret_cast<const uint4*>(gu + m * 2 * N + N + c);
        const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 gf = Elem<T>::unpack2(gw[k]), uf = Elem<T>::unpack2(uw[k]);
            ow[k] = Elem<T>::pack2(gf.x / (1.f + __expf(-gf.x)) * uf.x, gf.y / (1.f + __expf(-gf.y)) * uf.y);
        }
        *reinterpret_cast<uint4*>(y + m * N + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

}  // namespace kb
