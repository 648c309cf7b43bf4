// LayerNorm / RMSNorm forward for sm_100a. HBM-bound: x is read once and y written once.
//
// Fast path: one warp per row, the whole row held in registers as 128-bit vectors (8 elements of
// a 16-bit type per load), statistics by warp shuffles in fp32 in one sweep over the registers
// (shifted sums, no second trip to memory). Algorithmic traffic per row is 2*cols*2 bytes.
// Generic path: arbitrary strides / column counts, one warp per row, re-reads the row (served by
// L1/L2) — correctness path for the strided cases the reference accepts
// (src/kernl/implementations/layer_norm.py:321-324).
#pragma once
#include "common.cuh"

namespace kb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ uint4 ld_stream_16B(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream_16B(void* p, uint4 v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
}

// WPR warps share one row (1: a warp per row, for many rows; 4: the whole CTA on one row, for the
// few rows of a decode step, where a single warp walking 4096 columns is a 19 µs chain of dependent
// loads). CHUNKS = ceil(cols / (256 * WPR)): each lane owns CHUNKS vectors of 8 elements; vector c of
// lane l of warp w covers columns ((c*WPR + w)*32 + l)*8 .. +8. cols must be a multiple of 8.
template <typename T, int CHUNKS, bool RMS, int WPR = 1>
__global__ void __launch_bounds__(128)
norm_fwd_rowwarp_kernel(const T* __restrict__ x, T* __restrict__ y, const T* __restrict__ gamma,
                        const T* __restrict__ beta, float* __restrict__ mean_out,
                        float* __restrict__ rstd_out, int64_t rows, int cols, int64_t x_row_stride,
                        int64_t y_row_stride, float eps, const T* __restrict__ residual,
                        T* __restrict__ sum_out) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float red_s[2][4];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wir = warp % WPR;  // this warp's position inside its row
    const int64_t row = (int64_t)blockIdx.x * (4 / WPR) + warp / WPR;
    if (row >= rows) return;  // (WPR > 1: the whole CTA leaves together)
    const T* xr = x + row * x_row_stride;
    T* yr = y + row * y_row_stride;
#define KB_NORM_COL(c) ((((c) * WPR + wir) * 32 + lane) * 8)

    uint4 v[CHUNKS];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int col = KB_NORM_COL(c);
        if (col < cols) v[c] = ld_stream_16B(xr + col);
        else v[c] = make_uint4(0, 0, 0, 0);
    }
    // Short rows: fetch gamma/beta now, next to the row itself, instead of after the statistics, where
    // their (L1/L2) latency would sit at the end of a warp that has nothing left to overlap it with.
    constexpr bool kEarlyAffine = CHUNKS <= 4;
    uint4 gv[kEarlyAffine ? CHUNKS : 1], bv[kEarlyAffine ? CHUNKS : 1];
    if (kEarlyAffine) {
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            const int col = KB_NORM_COL(c);
            gv[c] = make_uint4(0, 0, 0, 0);
            bv[c] = make_uint4(0, 0, 0, 0);
            if (col < cols) {
                gv[c] = *reinterpret_cast<const uint4*>(gamma + col);
                if (!RMS && beta != nullptr) bv[c] = *reinterpret_cast<const uint4*>(beta + col);
            }
        }
    }
    if (residual != nullptr) {
        // pre-norm residual stream: s = x + residual (rounded to the 16-bit type, as a separate add
        // kernel would store it), written out once and normalised from the registers
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            const int col = KB_NORM_COL(c);
            if (col < cols) {
                const uint4 r = ld_stream_16B(residual + row * (int64_t)cols + col);
                const uint32_t xw[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
                const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
                uint32_t sw[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 a = Elem<T>::unpack2(xw[i]), b = Elem<T>::unpack2(rw[i]);
                    sw[i] = Elem<T>::pack2(a.x + b.x, a.y + b.y);
                }
                v[c] = make_uint4(sw[0], sw[1], sw[2], sw[3]);
                st_stream_16B(sum_out + row * (int64_t)cols + col, v[c]);
            }
        }
    }

    const float inv_n = 1.0f / (float)cols;
    float mean = 0.f, rstd;
    {
        // One sweep over the registers. LayerNorm accumulates sum(x-K) and sum((x-K)^2) with K = the
        // row's first element: shifting by a value of the row itself keeps the subtraction
        // E[(x-K)^2] - E[x-K]^2 well conditioned even when |mean| >> std (rows like -20 +- 0.5).
        float shift = 0.f;
        if (!RMS) {
            if (WPR == 1) {
                shift = __shfl_sync(0xffffffffu, Elem<T>::unpack2(v[0].x).x, 0);
            } else {  // every thread reads the row's first element itself (the sum, when a residual is added)
                float x0 = Elem<T>::to_f32(xr[0]);
                if (residual != nullptr) x0 = Elem<T>::to_f32(Elem<T>::from_f32(x0 + Elem<T>::to_f32(residual[row * (int64_t)cols])));
                shift = x0;
            }
        }
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            const int col = KB_NORM_COL(c);
            if (col < cols) {
                const uint32_t w[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = Elem<T>::unpack2(w[i]);
                    const float a = f.x - shift, b = f.y - shift;
                    if (!RMS) s1 += a + b;
                    s2 = fmaf(a, a, fmaf(b, b, s2));
                }
            }
        }
        s2 = warp_sum(s2);
        if (!RMS) s1 = warp_sum(s1);
        if (WPR > 1) {  // WPR == 4: the CTA is one row
            if (lane == 0) {
                red_s[0][warp] = s1;
                red_s[1][warp] = s2;
            }
            __syncthreads();
            s1 = (red_s[0][0] + red_s[0][1]) + (red_s[0][2] + red_s[0][3]);
            s2 = (red_s[1][0] + red_s[1][1]) + (red_s[1][2] + red_s[1][3]);
        }
        s2 *= inv_n;
        if (!RMS) {
            const float d = s1 * inv_n;
            mean = shift + d;
            s2 = fmaxf(s2 - d * d, 0.f);
        }
        rstd = rsqrtf(s2 + eps);
    }
    if (lane == 0 && wir == 0) {
        if (mean_out) mean_out[row] = mean;
        if (rstd_out) rstd_out[row] = rstd;
    }

#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int col = KB_NORM_COL(c);
        if (col < cols) {
            uint4 g, b = make_uint4(0, 0, 0, 0);
            if (kEarlyAffine) {
                g = gv[c];
                b = bv[c];
            } else {
                g = *reinterpret_cast<const uint4*>(gamma + col);
                if (!RMS && beta != nullptr) b = *reinterpret_cast<const uint4*>(beta + col);
            }
            const uint32_t xw[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
            const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
            const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
            uint32_t ow[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 xf = Elem<T>::unpack2(xw[i]);
                const float2 gf = Elem<T>::unpack2(gw[i]);
                const float2 bf = Elem<T>::unpack2(bw[i]);
                const float o0 = (xf.x - mean) * rstd * gf.x + bf.x;
                const float o1 = (xf.y - mean) * rstd * gf.y + bf.y;
                ow[i] = Elem<T>::pack2(o0, o1);
            }
            st_stream_16B(yr + col, make_uint4(ow[0], ow[1], ow[2], ow[3]));
        }
    }
}

// Generic strided path: one warp per row, three sweeps over the row.
template <typename T, bool RMS>
__global__ void __launch_bounds__(128)
norm_fwd_generic_kernel(const T* __restrict__ x, T* __restrict__ y, const T* __restrict__ gamma,
                        const T* __restrict__ beta, float* __restrict__ mean_out,
                        float* __restrict__ rstd_out, int64_t rows, int64_t cols,
                        int64_t x_row_stride, int64_t x_col_stride, int64_t y_row_stride,
                        int64_t y_col_stride, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= rows) return;
    const T* xr = x + row * x_row_stride;
    T* yr = y + row * y_row_stride;
    const float inv_n = 1.0f / (float)cols;
    float mean = 0.f;
    if (!RMS) {
        float s = 0.f;
        for (int64_t c = lane; c < cols; c += 32) s += Elem<T>::to_f32(xr[c * x_col_stride]);
        mean = warp_sum(s) * inv_n;
    }
    float s2 = 0.f;
    for (int64_t c = lane; c < cols; c += 32) {
        const float d = Elem<T>::to_f32(xr[c * x_col_stride]) - mean;
        s2 += d * d;
    }
    const float rstd = rsqrtf(warp_sum(s2) * inv_n + eps);
    if (lane == 0) {
        if (mean_out) mean_out[row] = mean;
        if (rstd_out) rstd_out[row] = rstd;
    }
    for (int64_t c = lane; c < cols; c += 32) {
        const float xv = Elem<T>::to_f32(xr[c * x_col_stride]);
        const float g = Elem<T>::to_f32(gamma[c]);
        const float b = (!RMS && beta != nullptr) ? Elem<T>::to_f32(beta[c]) : 0.f;
        yr[c * y_col_stride] = Elem<T>::from_f32((xv - mean) * rstd * g + b);
    }
}

template <typename T, bool RMS>
static int launch_norm_t(const kb_norm_params& p, cudaStream_t stream) {
    const T* x = (const T*)p.x;
    T* y = (T*)p.y;
    const T* g = (const T*)p.gamma;
    const T* b = (const T*)p.beta;
    constexpr int kWarps = 4;
    const unsigned grid = (unsigned)((p.rows + kWarps - 1) / kWarps);
    const bool vec_ok = p.x_col_stride == 1 && p.y_col_stride == 1 && (p.cols % 8) == 0 &&
                        (p.x_row_stride % 8) == 0 && (p.y_row_stride % 8) == 0 &&
                        ((uintptr_t)p.x % 16) == 0 && ((uintptr_t)p.y % 16) == 0 &&
                        ((uintptr_t)p.gamma % 16) == 0 &&
                        (p.beta == nullptr || ((uintptr_t)p.beta % 16) == 0) && p.cols <= 6144;
    if (vec_ok && p.rows <= 1024) {
        // few rows (a decode step, BERT at batch 1): one CTA per row, so that every row is read by 128
        // threads at once instead of one warp walking it
        const int chunks4 = (int)((p.cols + 1023) / 1024);
        const unsigned grid4 = (unsigned)p.rows;
#define KB_NORM_CASE4(C)                                                                         \
    if (chunks4 <= C) {                                                                          \
        return launch_pdl(norm_fwd_rowwarp_kernel<T, C, RMS, 4>, grid4, kWarps * 32, 0, stream,  \
                   x, y, g, b, p.mean, p.rstd, p.rows, (int)p.cols, p.x_row_stride,              \
                   p.y_row_stride, p.eps, (const T*)p.residual, (T*)p.sum_out) == cudaSuccess    \
                   ? KB_OK : KB_ERR_LAUNCH;                                                      \
    }
        KB_NORM_CASE4(1)
        KB_NORM_CASE4(2)
        KB_NORM_CASE4(4)
        KB_NORM_CASE4(6)
#undef KB_NORM_CASE4
    }
    if (vec_ok) {
        const int chunks = (int)((p.cols + 255) / 256);
#define KB_NORM_CASE(C)                                                                          \
    if (chunks <= C) {                                                                           \
        return launch_pdl(norm_fwd_rowwarp_kernel<T, C, RMS>, grid, kWarps * 32, 0, stream,      \
                   x, y, g, b, p.mean, p.rstd, p.rows, (int)p.cols, p.x_row_stride,              \
                   p.y_row_stride, p.eps, (const T*)p.residual, (T*)p.sum_out) == cudaSuccess    \
                   ? KB_OK : KB_ERR_LAUNCH;                                                      \
    }
        KB_NORM_CASE(1)
        KB_NORM_CASE(2)
        KB_NORM_CASE(3)
        KB_NORM_CASE(4)
        KB_NORM_CASE(6)
        KB_NORM_CASE(8)
        KB_NORM_CASE(12)
        KB_NORM_CASE(16)
        KB_NORM_CASE(24)
#undef KB_NORM_CASE
    }
    if (p.residual != nullptr) return KB_ERR_UNSUPPORTED;  // the fused add needs the vector layout
    return launch_pdl(norm_fwd_generic_kernel<T, RMS>, grid, kWarps * 32, 0, stream, x, y, g, b, p.mean, p.rstd, p.rows,
                      p.cols, p.x_row_stride, p.x_col_stride, p.y_row_stride, p.y_col_stride, p.eps) == cudaSuccess
               ? KB_OK : KB_ERR_LAUNCH;
}

static int launch_norm(const kb_norm_params& p, cudaStream_t stream) {
    if (p.dtype == KB_F16)
        return p.is_rms ? launch_norm_t<__half, true>(p, stream) : launch_norm_t<__half, false>(p, stream);
    if (p.dtype == KB_BF16)
        return p.is_rms ? launch_norm_t<__nv_bfloat16, true>(p, stream)
                        : launch_norm_t<__nv_bfloat16, false>(p, stream);
    return KB_ERR_UNSUPPORTED;
}

}  // namespace kb
