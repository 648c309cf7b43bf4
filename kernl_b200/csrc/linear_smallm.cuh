// Linear layer for very few rows (M <= 16): y = act(x · Wᵀ + bias), the decode-step shape.
//
// With a handful of rows the op is a single pass over W from HBM (2·N·K bytes; x is a few dozen KB and
// lives in L1/L2), so what matters is how many bytes every SM keeps in flight and how little
// fixed cost a launch carries — not the tensor-core generation. The tcgen05 GEMM pays for a tensor
// map, a TMEM allocation, a 128-row tile of which 8 rows are real, and a second kernel to finish its
// split-K sums: about 6 µs of fixed cost on a 14 µs stream. This kernel has none of that:
//   * one CTA of 8 warps per 16 output columns; the warps split K in interleaved 64-byte pieces,
//     so the 8 warps together read 512 contiguous bytes of each weight row per round;
//   * every thread loads 16 bytes (8 consecutive k) of one weight row per 8-column group with
//     streaming loads, four rounds ahead, and feeds them as the B fragments of two
//     mma.sync.m16n8k16 (the k order inside an MMA is permuted consistently for A and B, which a dot
//     product does not notice); x rows are the A fragments, read through L1;
//   * launched with programmatic dependent launch: its set-up overlaps the tail of the kernel that
//     produces x;
//   * the 8 partial 16x16 tiles meet in shared memory, 256 threads add them and apply bias and
//     activation. No workspace, no atomics, no second launch.
// Same contract as the reference's linear_layer (src/kernl/implementations/linear_layer.py:213-282).
#pragma once
#include "linear.cuh"

namespace kb {

constexpr int kSmallMThreads = 256;
constexpr int kSmallMCols = 16;    // output columns per CTA
constexpr int kSmallMRounds = 4;   // 32-element k pieces in flight per warp

// HI: rows 8..15 exist (M > 8); otherwise their A fragments are zero and are not loaded.
// Up to eight rows (HI = false) the kernel fits three CTAs per SM (80 registers): more weight bytes in
// flight per SM. Decode step of the 7B shape: 8 layers 1.76 -> 1.69 ms, 32 layers 5.43 -> 5.40 ms;
// four CTAs per SM (64 registers) measured no better than three.
template <typename T, bool HI>
__global__ void __launch_bounds__(kSmallMThreads, HI ? 2 : 3)
linear_smallm_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias, T* __restrict__ y,
                     T* __restrict__ act_inputs, int M, int N, int K, int64_t x_row_stride, int64_t y_row_stride,
                     int activation) {
    __shared__ float red[kSmallMThreads / 32][16][kSmallMCols + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    const int n0 = blockIdx.x * kSmallMCols;

    // rows of W this thread reads (one per 8-column group) and rows of x (g and g + 8)
    const T* wrow[2];
    bool wlive[2];
#pragma unroll
    for (int grp = 0; grp < 2; ++grp) {
        const int n = n0 + grp * 8 + g;
        wlive[grp] = n < N;
        wrow[grp] = w + (int64_t)(wlive[grp] ? n : 0) * K;
    }
    const bool lo_live = g < M, hi_live = HI && (g + 8 < M);
    const T* xlo = x + (int64_t)(lo_live ? g : 0) * x_row_stride;
    const T* xhi = x + (int64_t)(hi_live ? g + 8 : 0) * x_row_stride;

    float acc[2][4];
#pragma unroll
    for (int grp = 0; grp < 2; ++grp)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[grp][i] = 0.f;

    // piece p covers k in [32p, 32p + 32); warp `warp` takes pieces warp, warp + 8, ...; inside a piece
    // this thread owns the 8 elements at 32p + 8c.
    const int pieces = (K + 31) / 32;
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    uint4 bw[kSmallMRounds][2];
    auto load_w = [&](int p0) {
#pragma unroll
        for (int r = 0; r < kSmallMRounds; ++r) {
            const int k = (p0 + r * 8) * 32 + c * 8;
#pragma unroll
            for (int grp = 0; grp < 2; ++grp) bw[r][grp] = (k < K && wlive[grp]) ? ld_stream_nc_16B(wrow[grp] + k) : zero4;
        }
    };
    pdl_wait();  // (W could in principle have been written by the previous kernel, e.g. a dtype conversion)
    pdl_launch_dependents();
    load_w(warp);
    for (int p0 = warp; p0 < pieces; p0 += 8 * kSmallMRounds) {
        uint4 alo[kSmallMRounds], ahi[kSmallMRounds];
#pragma unroll
        for (int r = 0; r < kSmallMRounds; ++r) {
            const int k = (p0 + r * 8) * 32 + c * 8;
            const bool kin = k < K;  // K is a multiple of 8, so a thread's 8 elements are in or out as a whole
            alo[r] = (kin && lo_live) ? __ldg(reinterpret_cast<const uint4*>(xlo + k)) : zero4;
            if (HI) ahi[r] = (kin && hi_live) ? __ldg(reinterpret_cast<const uint4*>(xhi + k)) : zero4;
            else ahi[r] = zero4;
        }
#pragma unroll
        for (int r = 0; r < kSmallMRounds; ++r) {
#pragma unroll
            for (int grp = 0; grp < 2; ++grp) {
                mma_16816<T>(acc[grp], alo[r].x, ahi[r].x, alo[r].y, ahi[r].y, bw[r][grp].x, bw[r][grp].y);
                mma_16816<T>(acc[grp], alo[r].z, ahi[r].z, alo[r].w, ahi[r].w, bw[r][grp].z, bw[r][grp].w);
            }
        }
        if (p0 + 8 * kSmallMRounds < pieces) load_w(p0 + 8 * kSmallMRounds);
    }
    // accumulator fragment: c0,c1 -> (row g, cols 2c, 2c+1); c2,c3 -> (row g+8, same cols)
#pragma unroll
    for (int grp = 0; grp < 2; ++grp) {
        red[warp][g][grp * 8 + 2 * c] = acc[grp][0];
        red[warp][g][grp * 8 + 2 * c + 1] = acc[grp][1];
        red[warp][g + 8][grp * 8 + 2 * c] = acc[grp][2];
        red[warp][g + 8][grp * 8 + 2 * c + 1] = acc[grp][3];
    }
    __syncthreads();
    const int m = threadIdx.x >> 4, nn = threadIdx.x & 15;
    const int n = n0 + nn;
    if (activation == KB_ACT_SWIGLU) {
        // the CTA's first eight columns are a gate block, the other eight the matching up block
        // (rows of W interleaved in blocks of eight): eight outputs at columns n0 / 2 ...
        if (m < M && nn < 8 && n < N) {
            float zg = 0.f, zu = 0.f;
#pragma unroll
            for (int wi = 0; wi < kSmallMThreads / 32; ++wi) {
                zg += red[wi][m][nn];
                zu += red[wi][m][nn + 8];
            }
            if (bias != nullptr) {
                zg += Elem<T>::to_f32(bias[n]);
                zu += Elem<T>::to_f32(bias[n + 8]);
            }
            y[(int64_t)m * y_row_stride + (n0 >> 1) + nn] = Elem<T>::from_f32(act_silu(zg) * zu);
        }
        return;
    }
    if (m < M && n < N) {
        float z = 0.f;
#pragma unroll
        for (int wi = 0; wi < kSmallMThreads / 32; ++wi) z += red[wi][m][nn];
        if (bias != nullptr) z += Elem<T>::to_f32(bias[n]);
        if (act_inputs != nullptr) act_inputs[(int64_t)m * y_row_stride + n] = Elem<T>::from_f32(z);
        float v = z;
        switch (activation) {
            case KB_ACT_TANH: v = act_tanh(v); break;
            case KB_ACT_GELU: v = act_gelu(v); break;
            case KB_ACT_FAST_GELU: v = act_fast_gelu(v); break;
            case KB_ACT_RELU: v = fmaxf(v, 0.f); break;
            case KB_ACT_SILU: v = act_silu(v); break;
            default: break;
        }
        y[(int64_t)m * y_row_stride + n] = Elem<T>::from_f32(v);
    }
}

static bool smallm_applicable(const kb_linear_params& p) {
    return p.M >= 1 && p.M <= 16 && p.K % 8 == 0 && p.x_row_stride % 8 == 0 && (((uintptr_t)p.x) & 15) == 0 &&
           (((uintptr_t)p.w) & 15) == 0 && p.N <= (int64_t)0x7fffffff / 2 && p.K <= 0x7fffffff;
}

template <typename T>
static int launch_linear_smallm_t(const kb_linear_params& p, cudaStream_t stream) {
    const unsigned grid = (unsigned)((p.N + kSmallMCols - 1) / kSmallMCols);
    if (p.M > 8)
        launch_pdl(linear_smallm_kernel<T, true>, grid, kSmallMThreads, 0, stream, (const T*)p.x, (const T*)p.w,
                   (const T*)p.bias, (T*)p.y, (T*)p.act_inputs, (int)p.M, (int)p.N, (int)p.K, p.x_row_stride,
                   p.y_row_stride, p.activation);
    else
        launch_pdl(linear_smallm_kernel<T, false>, grid, kSmallMThreads, 0, stream, (const T*)p.x, (const T*)p.w,
                   (const T*)p.bias, (T*)p.y, (T*)p.act_inputs, (int)p.M, (int)p.N, (int)p.K, p.x_row_stride,
                   p.y_row_stride, p.activation);
    return cudaGetLastError() == cudaSuccess ? KB_OK : KB_ERR_LAUNCH;
}

static int launch_linear_smallm(const kb_linear_params& p, cudaStream_t stream) {
    if (p.dtype == KB_F16) return launch_linear_smallm_t<__half>(p, stream);
    if (p.dtype == KB_BF16) return launch_linear_smallm_t<__nv_bfloat16>(p, stream);
    return KB_ERR_UNSUPPORTED;
}

}  // namespace kb
