// All-reduce (sum) + residual add over NVLink peer memory, for the row-parallel linears of a
// tensor-parallel decoder (o_proj, down_proj): out = residual + sum_r partial_r.
//
// Every rank's GEMM writes its partial result straight into a buffer that all peers have mapped
// (symmetric memory). This kernel then, on every rank:
//   1. tells each peer "my partial of epoch e is complete" (system-scope release store of e into
//      the peer's flag word for this rank),
//   2. waits until every peer has said the same (bounded spin, acquire loads of its own flag words),
//   3. pulls every peer's partial with plain 128-bit loads over NVLink (no TMA, no multicast, no
//      multimem), adds them in fp32 in rank order — identical on every rank — adds the residual,
//      and writes the 16-bit result locally,
//   4. tells each peer "I have finished reading your buffer" and waits for the same from everyone,
//      so that the next GEMM may overwrite the partial buffers without any buffer rotation.
// It is a one-shot all-reduce: each rank reads (world-1) x message bytes. That is the right trade
// for the latency-bound decode messages (a few rows of 4096); large prefill messages go through
// NCCL. Nothing here can spin forever: an expired wait sets the device status word and the kernel
// carries on (its output is then meaningless, the host sees the status).
//
// Flag block per rank (uint32, peer-mapped, zero-initialised once): [0,8) ready[src],
// [8,16) done[src], [16] epoch of the last finished call, [17] block ticket.
#pragma once
#include "common.cuh"

namespace kb {

constexpr int kArMaxWorld = 8;
constexpr int kArThreads = 256;

struct ArDev {
    const void* bufs[kArMaxWorld];
    uint32_t* flags[kArMaxWorld];
    const void* residual;
    void* out;
    int64_t n;  // elements, multiple of 8
    int rank, world;
    // optional fused RMSNorm of the reduced rows (norm_weight != nullptr)
    const void* norm_weight;
    void* norm_out;
    int cols;  // row length, multiple of 8, <= kArNormMaxCols; n % cols == 0
    float eps;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_peer_16B(const void* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

// Spin until *flag == want, at most a few seconds (peer_wait_limit). Returns false (and records it) on expiry.
__device__ __forceinline__ bool ar_wait_flag(const uint32_t* flag, uint32_t want, int site) {
    const long long t0 = clock64();
    for (uint32_t spins = 0;; ++spins) {
        if (ld_acquire_sys(flag) == want) return true;
        if ((spins & 0x3F) == 0x3F && clock64() - t0 > peer_wait_limit()) {
            if (atomicCAS(&g_device_status[0], 0, KB_DEV_WAIT_EXPIRED) == 0) {
                g_device_status[1] = site;
                g_device_status[2] = (int)blockIdx.x;
                g_device_status[3] = (int)want;
            }
            return false;
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kArThreads)
allreduce_residual_kernel(const ArDev p) {
    __shared__ uint32_t s_epoch;
    __shared__ int s_last;
    uint32_t* my = p.flags[p.rank];
    if (threadIdx.x == 0) s_epoch = *reinterpret_cast<volatile uint32_t*>(my + 16) + 1u;
    __syncthreads();
    const uint32_t epoch = s_epoch;
    const int tid = threadIdx.x;

    // 1. my partial is complete (the GEMM that wrote it precedes this kernel on the stream)
    if (blockIdx.x == 0 && tid < p.world && tid != p.rank) {
        __threadfence_system();
        st_release_sys(p.flags[tid] + p.rank, epoch);
    }
    // 2. every peer's partial is complete
    if (tid < p.world && tid != p.rank) ar_wait_flag(my + tid, epoch, 500 + tid);
    __syncthreads();

    // 3. sum in rank order, add the residual, store
    const int64_t nvec = p.n / 8;
    for (int64_t i = (int64_t)blockIdx.x * kArThreads + tid; i < nvec; i += (int64_t)gridDim.x * kArThreads) {
        float acc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = 0.f;
        for (int r = 0; r < p.world; ++r) {
            const uint4 w = ld_peer_16B(reinterpret_cast<const uint4*>(p.bufs[r]) + i);
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = Elem<T>::unpack2(ww[k]);
                acc[2 * k] += f.x;
                acc[2 * k + 1] += f.y;
            }
        }
        if (p.residual != nullptr) {
            const uint4 w = *(reinterpret_cast<const uint4*>(p.residual) + i);
            const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = Elem<T>::unpack2(ww[k]);
                acc[2 * k] += f.x;
                acc[2 * k + 1] += f.y;
            }
        }
        uint4 o;
        o.x = Elem<T>::pack2(acc[0], acc[1]);
        o.y = Elem<T>::pack2(acc[2], acc[3]);
        o.z = Elem<T>::pack2(acc[4], acc[5]);
        o.w = Elem<T>::pack2(acc[6], acc[7]);
        *(reinterpret_cast<uint4*>(p.out) + i) = o;
    }

    // 4. the last block to finish reading tells the peers, waits for theirs, closes the epoch
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        s_last = (atomicAdd(reinterpret_cast<unsigned int*>(my + 17), 1u) == gridDim.x - 1) ? 1 : 0;
    }
    __syncthreads();
    if (s_last) {
        if (tid < p.world && tid != p.rank) {
            st_release_sys(p.flags[tid] + 8 + p.rank, epoch);
            ar_wait_flag(my + 8 + tid, epoch, 520 + tid);
        }
        __syncthreads();
        if (tid == 0) {
            my[17] = 0;
            __threadfence();
            *reinterpret_cast<volatile uint32_t*>(my + 16) = epoch;
        }
    }
}

// Same protocol, plus the RMSNorm that follows the residual add in a pre-norm decoder block:
//   out = residual + sum_r partial_r      (the new residual stream, rounded to T)
//   norm_out = out * rsqrt(mean(out^2) + eps) * weight   (computed from the rounded values, i.e.
//              what a separate RMSNorm kernel reading `out` would produce)
// One CTA per row (grid-strided), the row held in registers between the sum and the scaling.
constexpr int kArNormMaxCols = 8192;
constexpr int kArNormVecs = kArNormMaxCols / 8 / kArThreads;  // 4

template <typename T>
__global__ void __launch_bounds__(kArThreads)
allreduce_residual_rmsnorm_kernel(const ArDev p) {
    __shared__ uint32_t s_epoch;
    __shared__ int s_last;
    __shared__ float s_red[kArThreads / 32];
    uint32_t* my = p.flags[p.rank];
    if (threadIdx.x == 0) s_epoch = *reinterpret_cast<volatile uint32_t*>(my + 16) + 1u;
    __syncthreads();
    const uint32_t epoch = s_epoch;
    const int tid = threadIdx.x;

    if (blockIdx.x == 0 && tid < p.world && tid != p.rank) {
        __threadfence_system();
        st_release_sys(p.flags[tid] + p.rank, epoch);
    }
    if (tid < p.world && tid != p.rank) ar_wait_flag(my + tid, epoch, 540 + tid);
    __syncthreads();

    const int vec_per_row = p.cols / 8;
    const int64_t rows = p.n / p.cols;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        uint4 keep[kArNormVecs];
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < kArNormVecs; ++c) {
            const int vi = c * kArThreads + tid;
            if (vi < vec_per_row) {
                const int64_t i = row * vec_per_row + vi;
                float acc[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] = 0.f;
                for (int r = 0; r < p.world; ++r) {
                    const uint4 w = ld_peer_16B(reinterpret_cast<const uint4*>(p.bufs[r]) + i);
                    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float2 f = Elem<T>::unpack2(ww[k]);
                        acc[2 * k] += f.x;
                        acc[2 * k + 1] += f.y;
                    }
                }
                if (p.residual != nullptr) {
                    const uint4 w = *(reinterpret_cast<const uint4*>(p.residual) + i);
                    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float2 f = Elem<T>::unpack2(ww[k]);
                        acc[2 * k] += f.x;
                        acc[2 * k + 1] += f.y;
                    }
                }
                uint4 o;
                o.x = Elem<T>::pack2(acc[0], acc[1]);
                o.y = Elem<T>::pack2(acc[2], acc[3]);
                o.z = Elem<T>::pack2(acc[4], acc[5]);
                o.w = Elem<T>::pack2(acc[6], acc[7]);
                *(reinterpret_cast<uint4*>(p.out) + i) = o;
                keep[c] = o;
                const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 f = Elem<T>::unpack2(ow[k]);
                    ss += f.x * f.x + f.y * f.y;
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if ((tid & 31) == 0) s_red[tid >> 5] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kArThreads / 32; ++w) tot += s_red[w];
        __syncthreads();  // s_red is reused by the next row
        const float rstd = rsqrtf(tot / (float)p.cols + p.eps);
#pragma unroll
        for (int c = 0; c < kArNormVecs; ++c) {
            const int vi = c * kArThreads + tid;
            if (vi < vec_per_row) {
                const uint4 g = *(reinterpret_cast<const uint4*>(p.norm_weight) + vi);
                const uint32_t xw[4] = {keep[c].x, keep[c].y, keep[c].z, keep[c].w};
                const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
                uint32_t yw[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 f = Elem<T>::unpack2(xw[k]);
                    const float2 w = Elem<T>::unpack2(gw[k]);
                    yw[k] = Elem<T>::pack2(f.x * rstd * w.x, f.y * rstd * w.y);
                }
                *(reinterpret_cast<uint4*>(p.norm_out) + row * vec_per_row + vi) =
                    make_uint4(yw[0], yw[1], yw[2], yw[3]);
            }
        }
    }

    __syncthreads();
    if (tid == 0) {
        __threadfence();
        s_last = (atomicAdd(reinterpret_cast<unsigned int*>(my + 17), 1u) == gridDim.x - 1) ? 1 : 0;
    }
    __syncthreads();
    if (s_last) {
        if (tid < p.world && tid != p.rank) {
            st_release_sys(p.flags[tid] + 8 + p.rank, epoch);
            ar_wait_flag(my + 8 + tid, epoch, 560 + tid);
        }
        __syncthreads();
        if (tid == 0) {
            my[17] = 0;
            __threadfence();
            *reinterpret_cast<volatile uint32_t*>(my + 16) = epoch;
        }
    }
}

template <typename T>
static int launch_allreduce_t(const ArDev& d, cudaStream_t stream) {
    if (d.norm_weight != nullptr) {
        int64_t rows = d.n / d.cols;
        if (rows > 128) rows = 128;
        allreduce_residual_rmsnorm_kernel<T><<<(unsigned)rows, kArThreads, 0, stream>>>(d);
        return cudaGetLastError() == cudaSuccess ? KB_OK : KB_ERR_LAUNCH;
    }
    const int64_t nvec = d.n / 8;
    int64_t blocks = (nvec + kArThreads - 1) / kArThreads;
    if (blocks > 64) blocks = 64;  // latency-bound messages: a few dozen CTAs saturate NVLink reads
    if (blocks < 1) blocks = 1;
    allreduce_residual_kernel<T><<<(unsigned)blocks, kArThreads, 0, stream>>>(d);
    return cudaGetLastError() == cudaSuccess ? KB_OK : KB_ERR_LAUNCH;
}

}  // namespace kb
