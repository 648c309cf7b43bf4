// Fused linear layer y = act(x · Wᵀ + bias) for sm_100a, large problems: CTA PAIRS on 256 x 256 tiles.
//
// linear.cuh gives every SM its own 128 x 256 tile: per 64-wide k-block an SM pulls 16 KB of x and
// 32 KB of W through shared memory for 512 tensor-core cycles, and neighbouring SMs load the same W
// tile again from L2 (ncu on [8192,4096]x[11008,4096]: 2.7x the algorithmic DRAM bytes, tensor pipe
// 79 % busy). Here two CTAs of a cluster (two neighbouring SMs) share one 256 x 256 output tile and
// issue `tcgen05.mma.cta_group::2`: each CTA stages its own 128 rows of x and only HALF of the W tile
// (128 of its 256 rows), the tensor cores of both SMs read both halves, and each CTA ends up with its
// 128 rows of the result in its own tensor memory. Per SM and k-block that is 32 KB through shared
// memory instead of 48 KB, and every W byte is fetched once per pair instead of once per SM.
//
// Roles per CTA (576 threads): warp 0 TMA producer, warp 1 tcgen05 issuer (only the pair's leader —
// cluster rank 0 — issues; the other CTA's warp 1 only allocates tensor memory), warps 2..17
// epilogue: warp w reads the tensor-memory lanes of quadrant w % 4 (its 32 rows) and the 64 columns
// (w - 2) / 4 of the CTA's 128 x 256 accumulator. Sixteen warps, because with a short K loop the
// epilogue is the longer of the two pipelines: clock stamps at K = 768 showed eight warps needing
// 7500-9000 cycles per tile (tensor-memory reads, conversion and stores each saturate their unit in
// turn, all warps in the same phase) against 6144 tensor-pipe cycles of the main loop. Barriers:
//   full[s]    in the LEADER's shared memory: the leader's producer arrives with the byte count of all
//              four copies of a stage; both CTAs' TMA copies complete on it (the second CTA addresses
//              it through the cluster's shared window);
//   empty[s]   in each CTA: `tcgen05.commit` of the leader, multicast to both CTAs;
//   tfull[a]   in each CTA: accumulator a complete (multicast commit);
//   tempty[a]  in the leader: all 32 epilogue warps of the pair have read accumulator a (a warp
//              arrives as soon as its 64 columns are in registers, before it converts and stores them).
// Accumulators are double-buffered (2 x 256 columns = all of tensor memory), the ring has six stages.
// Every bulk copy has one destination CTA: the pair's sharing happens inside the tensor-core instruction.
#pragma once
#include "linear.cuh"

namespace kb {

constexpr int kPairBN = 256;          // columns of the pair's widest tile (the kernel is also built for 192)
constexpr int kPairHalfN = 128;       // W rows staged by each CTA at that width
#ifndef KB_PAIR_STAGES
#define KB_PAIR_STAGES 6
#endif
constexpr int kPairStages = KB_PAIR_STAGES;
constexpr int kPairABytes = kGemmBM * kGemmBK * 2;     // 16 KB: this CTA's 128 rows of x
constexpr int kPairBBytes = kPairHalfN * kGemmBK * 2;  // 16 KB: this CTA's half of the W tile
constexpr int kPairStageBytes = kPairABytes + kPairBBytes;
constexpr int kPairEpilogueWarps = 16;
constexpr int kPairThreads = (2 + kPairEpilogueWarps) * 32;
// Output staging of the epilogue: per epilogue warp 32 rows x kPairPassCols columns of 16-bit
// results, in 16-byte pieces; piece c of row r sits at r * row_bytes + (c ^ f(r)) * 16 with f chosen so
// that the row-wise writes and the piece-wise reads are both free of bank conflicts (64-byte rows:
// f = (r >> 1) & 3; 32-byte rows: f = (r >> 2) & 1). Behind it the warp's 64 bias values as fp32.
#ifndef KB_PAIR_PASS_COLS
#define KB_PAIR_PASS_COLS 16
#endif
constexpr int kPairPassCols = KB_PAIR_PASS_COLS;
static_assert(kPairPassCols == 16 || kPairPassCols == 32, "columns per staging pass");
constexpr int kPairRowBytes = kPairPassCols * 2;
constexpr int kPairOutWarpBytes = 32 * kPairRowBytes;
constexpr int kPairBiasWarpBytes = 64 * 4;
constexpr int kPairOutBytes = kPairEpilogueWarps * (kPairOutWarpBytes + kPairBiasWarpBytes);
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 256 + kPairOutBytes + 1024;
__device__ __forceinline__ int pair_stage_offset(int r, int piece) {
    return kPairPassCols == 32 ? r * 64 + ((piece ^ ((r >> 1) & 3)) * 16) : r * 32 + ((piece ^ ((r >> 2) & 1)) * 16);
}
static_assert(kPairSmemBytes <= 227 * 1024, "shared memory of the pair kernel");
constexpr uint32_t kPairTmemCols = 512;
// The address, in the cluster's shared window, of the leader's (rank 0) copy of one of this CTA's own
// shared-memory locations: both CTAs lay out their shared memory identically.
__device__ __forceinline__ uint32_t in_leader(uint32_t own_smem_addr) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(own_smem_addr), "r"(0u));
    return r;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on a barrier of the pair's other CTA. CTA-scope release (the default): what the arrival
// orders are this warp's tensor-memory reads, which tcgen05.wait::ld and the tcgen05 fence before it
// have completed — no global data is handed over. A cluster-scope release also waits for the warp's
// earlier global stores to be acknowledged, which showed as 3.3 stall cycles per issued instruction.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load whose completion is counted on a barrier that may live in the pair's other CTA.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A[smem of both CTAs] * B[smem of both CTAs]: M = 256 (128 rows per CTA)
__device__ __forceinline__ void tc_mma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive (once all MMAs issued so far have completed) on the barrier at this offset in BOTH CTAs.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"((uint16_t)3)
                 : "memory");
}

// Optional clock stamps for tuning (compiled in with -DKB_GEMM_TRACE only): per CTA and for its first
// eight tiles, clock64 of: 0 issuer starts waiting for the accumulator, 1 has it, 2 has issued the
// tile's last MMA; 3 epilogue warp 2 starts waiting for the accumulator, 4 has it, 5 is done with it;
// 6 the same warp's first 64 columns are stored (8 / 9 / 10: its first tensor-memory load has
// landed / values are in shared memory / the warp has synchronised). Event 7 of tile 0 is the CTA's start.
#ifdef KB_GEMM_TRACE
__device__ long long g_gemm_trace[148 * 8 * 16];
#define KB_GTRACE(tile, ev)                                                                   \
    do {                                                                                      \
        if (blockIdx.x < 148 && (tile) < 8) g_gemm_trace[(blockIdx.x * 8 + (tile)) * 16 + (ev)] = clock64(); \
    } while (0)
#else
#define KB_GTRACE(tile, ev) do { } while (0)
#endif

// BN: columns of the pair's tile, 256 or 192. Each CTA stages BN / 2 rows of W per stage (the stage
// keeps its 32 KB stride), the accumulators sit at tensor-memory columns 0 and 256 whatever BN, and an
// epilogue warp owns BN / 4 columns. The narrower tile exists for problems of a few rounds: 384 tiles
// of 256 columns on 74 pairs run 5.2 rounds as 6, 512 tiles of 192 columns run 6.9 rounds as 7.
template <typename T, int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
linear_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                   const T* __restrict__ bias, T* __restrict__ y, T* __restrict__ act_inputs, int M, int N, int K,
                   int64_t y_row_stride, int activation) {
    constexpr int STAGES = kPairStages;
    static_assert(BN == 256 || BN == 192, "tile width of the pair kernel");
    constexpr int kHalfN = BN / 2;                     // W rows this CTA stages
    constexpr int kStageTx = kPairABytes + kHalfN * kGemmBK * 2;  // bytes one CTA's copies put into a stage
    constexpr int CW = BN / 4;                         // columns per epilogue warp
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * kPairStageBytes);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    uint8_t* out_stage = smem + STAGES * kPairStageBytes + 256;

    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0 = the pair's leader
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

    // A wait that expired earlier leaves the status word set: such a launch does no work. Both CTAs
    // of a pair must take the same decision (they allocate tensor memory together), so the leader's
    // reading counts for both: it is exchanged through the cluster barrier below.
    __shared__ int s_skip;
    if (threadIdx.x == 0) {
        KB_GTRACE(0, 7);
        s_skip = *reinterpret_cast<volatile int*>(&g_device_status[0]);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull_bar(a), 1);
            mbar_init(tempty_bar(a), 2 * kPairEpilogueWarps);  // the epilogue warps of both CTAs
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tmap_x);
        tma_prefetch_desc(&tmap_w);
    }
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers exist before anybody signals across the pair
    // the leader's decision, read from its shared memory through the cluster window
    int skip;
    {
        const uint32_t leader_skip = in_leader(smem_u32(&s_skip));
        asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(skip) : "r"(leader_skip) : "memory");
    }
    if (skip == 0) {
        if (warp == 1) {
            tmem_alloc_pair(smem_u32(tmem_slot), kPairTmemCols);
            tmem_relinquish_pair();
        }
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
    }
    const uint32_t tmem_base = (skip == 0) ? *tmem_slot : 0u;

    const int num_m = (M + 2 * kGemmBM - 1) / (2 * kGemmBM);  // 256-row tiles
    const int num_n = (N + BN - 1) / BN;
    const int num_tiles = num_m * num_n;
    const int num_k = (K + kGemmBK - 1) / kGemmBK;

    if (skip == 0 && warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = pair; t < num_tiles && ok; t += num_pairs) {
                int m_idx, n_idx;
                tile_coords(t, num_m, num_n, m_idx, n_idx);
                const int row0 = m_idx * 2 * kGemmBM + (int)rank * kGemmBM;    // this CTA's rows of x
                const int wrow0 = n_idx * BN + (int)rank * kHalfN;    // this CTA's rows of W
                for (int kb = 0; kb < num_k; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, 110)) { ok = false; break; }
                    // the leader's barrier counts the bytes of both CTAs' copies of this stage
                    if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * kStageTx);
                    const uint32_t a_dst = smem_base + stage * kPairStageBytes;
                    const uint32_t leader_full = in_leader(full_bar(stage));
                    tma_load_2d_pair(a_dst, &tmap_x, leader_full, kb * kGemmBK, row0);
                    tma_load_2d_pair(a_dst + kPairABytes, &tmap_w, leader_full, kb * kGemmBK, wrow0);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                for (int i = 0; i < 64; ++i) __nanosleep(2000);  // let copies in flight land
            }
        }
    } else if (skip == 0 && warp == 1) {
        // ------------------------------------------------------------------ tcgen05 issuer (leader only)
        if (rank == 0 && elect_one()) {
            constexpr uint32_t idesc = make_idesc_f16(Elem<T>::kIsBf16, 2 * kGemmBM, BN, 0, 0);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            int ti = 0;
            for (int t = pair; t < num_tiles && ok; t += num_pairs, ++ti) {
                KB_GTRACE(ti, 0);
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1, abort_flag, 210)) { ok = false; break; }
                KB_GTRACE(ti, 1);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * kPairBN);
                for (int kb = 0; kb < num_k; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag, 211)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_base + stage * kPairStageBytes;
                    const uint64_t a_desc = make_smem_desc_sw128(a_addr, 16, 1024);
                    const uint64_t b_desc = make_smem_desc_sw128(a_addr + kPairABytes, 16, 1024);
#pragma unroll
                    for (int k = 0; k < kGemmBK / 16; ++k)
                        tc_mma_ss_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    tc_commit_pair(empty_bar(stage));  // frees this stage in both CTAs
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                tc_commit_pair(tfull_bar(acc));  // both CTAs' epilogues may read accumulator `acc`
                KB_GTRACE(ti, 2);
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
        }
    } else if (skip == 0) {
        // ------------------------------------------------------------------ epilogue (both CTAs)
        const int q = warp & 3;                 // TMEM lane quadrant this warp may access
        const int c_begin = ((warp - 2) >> 2) * CW;  // the warp's CW columns of the tile
        const uint32_t leader_tempty[2] = {in_leader(tempty_bar(0)), in_leader(tempty_bar(1))};
        // whole 16-byte pieces of y: plain activations, no pre-activation output, aligned rows
        const bool staged = activation != KB_ACT_SWIGLU && act_inputs == nullptr && (N & 7) == 0 && (y_row_stride & 7) == 0 &&
                            (((uintptr_t)y) & 15) == 0;
        uint8_t* mine = out_stage + (warp - 2) * (kPairOutWarpBytes + kPairBiasWarpBytes);
        float* bias_s = reinterpret_cast<float*>(mine + kPairOutWarpBytes);
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        int ti = 0;
        // the warp's bias values of a tile (lane l: columns 2l, 2l + 1 of the warp's 64)
        auto load_bias = [&](int tile) -> float2 {
            float2 b2 = make_float2(0.f, 0.f);
            if (bias != nullptr && tile < num_tiles) {
                int m_i, n_i;
                tile_coords(tile, num_m, num_n, m_i, n_i);
                const int c = n_i * BN + c_begin + 2 * lane;
                if (2 * lane < CW && c < N) b2.x = Elem<T>::to_f32(bias[c]);
                if (2 * lane < CW && c + 1 < N) b2.y = Elem<T>::to_f32(bias[c + 1]);
            }
            return b2;
        };
        if (staged) reinterpret_cast<float2*>(bias_s)[lane] = load_bias(pair);
        for (int t = pair; t < num_tiles && ok; t += num_pairs, ++ti) {
            int m_idx, n_idx;
            tile_coords(t, num_m, num_n, m_idx, n_idx);
            const int n0 = n_idx * BN;
            // the next tile's bias is requested now and put into shared memory when this tile is done
            float2 bias_next = make_float2(0.f, 0.f);
            if (staged) bias_next = load_bias(t + num_pairs);
            if (warp == 2 && lane == 0) KB_GTRACE(ti, 3);
            if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, 310)) { ok = false; break; }
            if (warp == 2 && lane == 0) KB_GTRACE(ti, 4);
            tc_fence_after();
            const int row = m_idx * 2 * kGemmBM + (int)rank * kGemmBM + q * 32 + lane;
            T* y_row = y + (int64_t)row * y_row_stride;
            T* a_row = act_inputs ? act_inputs + (int64_t)row * y_row_stride : nullptr;
            if (staged) {
                // Results go through shared memory so that the warp writes whole row segments (eight
                // rows x 64 bytes per store instruction) instead of 32 rows x 16 bytes: a
                // thread-per-row store touches 32 cache lines per instruction.
                const int row_base = m_idx * 2 * kGemmBM + (int)rank * kGemmBM + q * 32;
                // all CW columns in one tensor-memory round trip; with them in registers the
                // accumulator goes back to the issuer at once. (Fetching the second half while the
                // first is converted and stored was slower: the accumulator came back later.)
                uint32_t r2[CW];
                const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * kPairBN + c_begin);
                {
                    uint32_t (&lo)[32] = *reinterpret_cast<uint32_t(*)[32]>(&r2[0]);
                    tmem_ld_32x32(t_addr, lo);
                    if (CW == 64) {
                        uint32_t (&hi)[32] = *reinterpret_cast<uint32_t(*)[32]>(&r2[CW - 32]);
                        tmem_ld_32x32(t_addr + 32, hi);
                    } else {
                        uint32_t (&hi)[16] = *reinterpret_cast<uint32_t(*)[16]>(&r2[CW - 16]);
                        tmem_ld_32x16(t_addr + 32, hi);
                    }
                }
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();  // (also: every lane's bias values are in bias_s)
                if (lane == 0) mbar_arrive_cluster(leader_tempty[acc]);
                if (warp == 2 && lane == 0) KB_GTRACE(ti, 8);
                constexpr int kPieces = kPairPassCols / 8;     // 16-byte pieces per staged row
                constexpr int kRowsPerStore = 32 / kPieces;  // rows one store instruction covers
#pragma unroll
                for (int ps = 0; ps < CW / kPairPassCols; ++ps) {
                    const int pc0 = c_begin + ps * kPairPassCols;  // first column of the pass, inside the tile
                    if (n0 + pc0 >= N) break;
                    float z[kPairPassCols];
#pragma unroll
                    for (int v = 0; v < kPairPassCols / 4; ++v) {
                        const float4 b4 = reinterpret_cast<const float4*>(bias_s)[ps * (kPairPassCols / 4) + v];
                        z[v * 4 + 0] = __uint_as_float(r2[ps * kPairPassCols + v * 4 + 0]) + b4.x;
                        z[v * 4 + 1] = __uint_as_float(r2[ps * kPairPassCols + v * 4 + 1]) + b4.y;
                        z[v * 4 + 2] = __uint_as_float(r2[ps * kPairPassCols + v * 4 + 2]) + b4.z;
                        z[v * 4 + 3] = __uint_as_float(r2[ps * kPairPassCols + v * 4 + 3]) + b4.w;
                    }
                    apply_activation<kPairPassCols>(z, activation);
#pragma unroll
                    for (int v = 0; v < kPieces; ++v) {
                        uint4 o;
                        o.x = Elem<T>::pack2(z[v * 8 + 0], z[v * 8 + 1]);
                        o.y = Elem<T>::pack2(z[v * 8 + 2], z[v * 8 + 3]);
                        o.z = Elem<T>::pack2(z[v * 8 + 4], z[v * 8 + 5]);
                        o.w = Elem<T>::pack2(z[v * 8 + 6], z[v * 8 + 7]);
                        *reinterpret_cast<uint4*>(mine + pair_stage_offset(lane, v)) = o;
                    }
                    if (warp == 2 && lane == 0 && ps == 0) KB_GTRACE(ti, 9);
                    __syncwarp();
                    if (warp == 2 && lane == 0 && ps == 0) KB_GTRACE(ti, 10);
#pragma unroll
                    for (int it = 0; it < 32 / kRowsPerStore; ++it) {
                        const int rr = it * kRowsPerStore + lane / kPieces, pc = lane % kPieces;
                        const uint4 o = *reinterpret_cast<const uint4*>(mine + pair_stage_offset(rr, pc));
                        const int grow = row_base + rr, gcol = n0 + pc0 + pc * 8;
                        if (grow < M && gcol < N) *reinterpret_cast<uint4*>(y + (int64_t)grow * y_row_stride + gcol) = o;
                    }
                    if (warp == 2 && lane == 0 && ps == 0) KB_GTRACE(ti, 6);
                    __syncwarp();
                }
                reinterpret_cast<float2*>(bias_s)[lane] = bias_next;  // (all reads of this tile's values are behind the last __syncwarp)
            } else {
#pragma unroll 1
                // (a 32-column chunk at a time: with 48 columns per warp, warps pair up on chunks — the
                // even warp of a pair of column groups takes the chunk that straddles them)
                for (int c0 = (c_begin / 32) * 32; c0 < c_begin + CW; c0 += 32) {
                    if (n0 + c0 >= N) break;
                    if (c0 < c_begin || c0 + 32 > c_begin + CW) {
                        if ((((warp - 2) >> 2) & 1) != 0) continue;  // the straddling chunk belongs to the even group
                    }
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * kPairBN + c0), r);
                    tmem_ld_wait();
                    float accv[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) accv[j] = __uint_as_float(r[j]);
                    if (activation == KB_ACT_SWIGLU) epilogue_chunk_swiglu<T>(accv, bias, y_row, n0 + c0, N, row < M);
                    else epilogue_chunk<T>(accv, bias, y_row, a_row, n0 + c0, N, row < M, activation);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(leader_tempty[acc]);  // counted in the leader, whose issuer reuses the accumulator
            }
            if (warp == 2 && lane == 0) KB_GTRACE(ti, 5);
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
    }

    // Teardown: every role of both CTAs falls through to here, also after an abandoned wait. Neither
    // CTA may retire while the other can still signal its barriers or use its tensor memory.
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (skip == 0 && warp == 1) {
        __syncwarp();
        tmem_dealloc_pair(tmem_base, kPairTmemCols);
    }
}

static int g_linear_pair = 1;  // test hook (kb_debug_linear_pair): 0 = never use the pair kernel, 192 / 256 = force that tile width

// The pair kernel serves problems with at least one 256 x 256 tile per pair of SMs and no split-K.
static bool linear_pair_applicable(const kb_linear_params& p) {
    if (g_linear_pair == 0) return false;
    const int64_t tiles = ((p.M + 255) / 256) * ((p.N + kPairBN - 1) / kPairBN);
    return p.M >= 512 && p.N >= 256 && p.K >= 256 && tiles >= gemm_sms() / 2;
}

// Tile width: rounds of tiles on the pairs x (columns of a tile + a fixed cost per tile, in columns).
// 192 columns only where that is clearly cheaper (a launch of a few rounds whose last one is nearly
// empty) and the epilogue can take its staged path (whole 16-byte pieces, no gated or pre-activation output).
static int linear_pair_tile_width(const kb_linear_params& p, int pairs) {
    if (g_linear_pair == 192 || g_linear_pair == 256) return g_linear_pair;
    const bool staged = p.activation != KB_ACT_SWIGLU && p.act_inputs == nullptr && (p.N & 7) == 0 && (p.y_row_stride & 7) == 0 &&
                        (((uintptr_t)p.y) & 15) == 0;
    if (!staged) return 256;
    auto cost = [&](int bn) {
        const int64_t tiles = ((p.M + 255) / 256) * ((p.N + bn - 1) / bn);
        return (double)((tiles + pairs - 1) / pairs) * (bn + 24);
    };
    return cost(192) < 0.95 * cost(256) ? 192 : 256;
}

template <typename T, int BN>
static int launch_linear_pair_tb(const kb_linear_params& p, cudaStream_t stream) {
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
        const uint32_t box[2] = {kGemmBK, BN / 2};
        int st = encode_tmap_16bit(&tmap_w, p.w, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
        if (st != KB_OK) return st;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kPairThreads);
    cfg.dynamicSmemBytes = kPairSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // pairs that can be resident at once, per device (the grid is persistent: one pair per slot)
    static int max_pairs[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return KB_ERR_LAUNCH;
    if (max_pairs[dev] == 0) {
        if (cudaFuncSetAttribute(linear_pair_kernel<T, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes) != cudaSuccess)
            return KB_ERR_LAUNCH;
        cfg.gridDim = dim3(2 * (unsigned)(sm_count() / 2));
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, linear_pair_kernel<T, BN>, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            return KB_ERR_LAUNCH;
        }
        max_pairs[dev] = n < sm_count() / 2 ? n : sm_count() / 2;
    }
    const int64_t tiles = ((p.M + 255) / 256) * ((p.N + BN - 1) / BN);
    int pairs = (int)(tiles < max_pairs[dev] ? tiles : max_pairs[dev]);
    if (pairs > gemm_sms() / 2) pairs = gemm_sms() / 2;  // a caller-set limit leaves SMs to a concurrent collective
    cfg.gridDim = dim3(2 * (unsigned)pairs);
    if (cudaLaunchKernelEx(&cfg, linear_pair_kernel<T, BN>, tmap_x, tmap_w, (const T*)p.bias, (T*)p.y, (T*)p.act_inputs, (int)p.M,
                           (int)p.N, (int)p.K, p.y_row_stride, p.activation) != cudaSuccess)
        return KB_ERR_LAUNCH;
    return cudaGetLastError() == cudaSuccess ? KB_OK : KB_ERR_LAUNCH;
}

template <typename T>
static int launch_linear_pair_t(const kb_linear_params& p, cudaStream_t stream) {
    const int pairs = gemm_sms() / 2;
    if (linear_pair_tile_width(p, pairs > 0 ? pairs : 1) == 192) return launch_linear_pair_tb<T, 192>(p, stream);
    return launch_linear_pair_tb<T, 256>(p, stream);
}

}  // namespace kb
