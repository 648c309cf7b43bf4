// Decode-shape ("skinny") attention for sm_100a: few query rows against many keys.
// With one query row the tensor cores are pointless (M=1) and the op is bound by streaming K and V
// from HBM once, so this is a CUDA-core split-KV kernel:
//   part 1  grid (splits, M, B*H): each CTA scores a chunk of keys for one query row (one key per
//           thread, 128-bit loads), runs the online softmax over the chunk in blocks of 128 keys and
//           accumulates exp(S-m)·V; it writes (m, l, acc[D]) fp32 to scratch
//   part 2  grid (M, B*H): merges the chunks with the online-softmax recurrence and writes O
// Same maths as src/kernl/implementations/attention_skinny.py:58-366 of the reference (which keeps
// its partial outputs in fp16; fp32 here). Additive masks and the causal flag are honoured in-kernel.
#pragma once
#include "common.cuh"
#include "attention.cuh"

namespace kb {

constexpr int kDecThreads = 128;
constexpr int kDecMaxSplits = 256;
constexpr int kDecMaxD = 256;

struct DecDev {
    const void* q; const void* k; const void* v; void* o; const void* mask;
    int64_t q_strides[4], k_strides[4], v_strides[4], o_strides[4], mask_strides[4];
    int B, H, M, N, D;
    float scale_log2;
    int is_causal, mask_dtype;
    int num_splits, chunk;  // chunk = keys per split, multiple of 128
    int kv_group;           // query heads per K/V head, >= 1
    const long long* kv_len_dev;  // optional: number of keys that exist (device side), else N
    float* scratch;         // [B*H, M, num_splits, D+2]
};

// Keys per CTA: 128 when there are few (batch x head x row) problems, so that the key dimension
// supplies the parallelism; doubled (up to 1024) while the launch still has about one full wave of
// CTAs (16 per SM). Longer chunks amortise a CTA's fixed phases (q load, three barriers per 128 keys,
// the final cross-warp sum) and leave fewer partial results for the second kernel to merge.
static void decode_split(int64_t N, int64_t problems, int* num_splits, int* chunk) {
    int64_t c = 128;
    while ((N + c - 1) / c > kDecMaxSplits) c *= 2;
    const int64_t want = 2000;
    while (c < 1024 && problems * ((N + 2 * c - 1) / (2 * c)) >= want) c *= 2;
    *chunk = (int)c;
    *num_splits = (int)((N + c - 1) / c);
    if (*num_splits < 1) *num_splits = 1;
}

static int64_t decode_scratch_bytes(int64_t B, int64_t H, int64_t M, int64_t N, int64_t D) {
    if (B < 0 || H < 0 || M < 0 || N < 0 || D <= 0) return -1;
    int splits, chunk;
    decode_split(N, B * H * M, &splits, &chunk);
    return B * H * M * (int64_t)splits * (D + 2) * (int64_t)sizeof(float);
}

// Keys that exist: all N, or the device-side count of a partly filled cache.
__device__ __forceinline__ int decode_live_keys(const DecDev& p) {
    if (p.kv_len_dev == nullptr) return p.N;
    const long long n = *p.kv_len_dev;
    return n < 0 ? 0 : (n < (long long)p.N ? (int)n : p.N);
}

template <typename T>
__global__ void __launch_bounds__(kDecThreads)
attn_decode_part1_kernel(const DecDev p) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float q_s[kDecMaxD];
    __shared__ float sc_s[kDecThreads];
    __shared__ float red_s[kDecThreads / 32];
    const int split = blockIdx.x, row = blockIdx.y, bh = blockIdx.z;
    const int b = bh / p.H, h = bh % p.H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int D = p.D;

    const T* qp = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_strides[0] + (int64_t)h * p.q_strides[1] +
                  (int64_t)row * p.q_strides[2];
    for (int d = tid; d < D; d += kDecThreads) q_s[d] = Elem<T>::to_f32(qp[(int64_t)d * p.q_strides[3]]) * p.scale_log2;
    __syncthreads();

    const int hk = h / p.kv_group;
    const T* kbase = reinterpret_cast<const T*>(p.k) + (int64_t)b * p.k_strides[0] + (int64_t)hk * p.k_strides[1];
    const T* vbase = reinterpret_cast<const T*>(p.v) + (int64_t)b * p.v_strides[0] + (int64_t)hk * p.v_strides[1];
    const bool k_vec = p.k_strides[3] == 1 && (p.k_strides[2] % 8) == 0 && (((uintptr_t)kbase) & 15) == 0 && (D % 8) == 0;
    const float mlow = mask_lowest(p.mask_dtype);
    const int64_t mask_off = p.mask ? (int64_t)b * p.mask_strides[0] + (int64_t)h * p.mask_strides[1] +
                                          (int64_t)row * p.mask_strides[2]
                                    : 0;

    float m_run = -INFINITY, l_run = 0.f;
    float acc[kDecMaxD / kDecThreads];
#pragma unroll
    for (int i = 0; i < kDecMaxD / kDecThreads; ++i) acc[i] = 0.f;

    const int key_begin = split * p.chunk;
    const int key_end = min(decode_live_keys(p), key_begin + p.chunk);  // a chunk beyond the live keys scores nothing: (m, l) = (-inf, 0)
    for (int k0 = key_begin; k0 < key_end; k0 += kDecThreads) {
        // ---- one key per thread: score in the log2 domain
        const int key = k0 + tid;
        float s = -INFINITY;
        if (key < key_end && !(p.is_causal && key > row)) {
            const T* kr = kbase + (int64_t)key * p.k_strides[2];
            float dot = 0.f;
            if (k_vec) {
                for (int d = 0; d < D; d += 8) {
                    const uint4 w = __ldg(reinterpret_cast<const uint4*>(kr + d));
                    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = Elem<T>::unpack2(ww[i]);
                        dot = fmaf(f.x, q_s[d + 2 * i], dot);
                        dot = fmaf(f.y, q_s[d + 2 * i + 1], dot);
                    }
                }
            } else {
                for (int d = 0; d < D; ++d) dot = fmaf(Elem<T>::to_f32(kr[(int64_t)d * p.k_strides[3]]), q_s[d], dot);
            }
            s = dot;
            if (p.mask) {
                float mv = mask_load(p.mask, mask_off + (int64_t)key * p.mask_strides[3], p.mask_dtype);
                s = fmaf(fmaxf(mv, mlow), kLog2e, s);
            }
        }
        // ---- block maximum
        float mx = s;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) red_s[warp] = mx;
        __syncthreads();
        mx = fmaxf(fmaxf(red_s[0], red_s[1]), fmaxf(red_s[2], red_s[3]));
        __syncthreads();
        float m_new = fmaxf(m_run, mx);
        if (m_new == -INFINITY) m_new = 0.f;
        const float alpha = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_new);
        const float pe = fast_exp2(s - m_new);
        // P is rounded to the input dtype before P·V, as the reference does (attention_skinny.py:262).
        sc_s[tid] = Elem<T>::to_f32(Elem<T>::from_f32(pe));
        float ps = pe;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        if (lane == 0) red_s[warp] = ps;
        __syncthreads();
        l_run = l_run * alpha + (red_s[0] + red_s[1] + red_s[2] + red_s[3]);
        m_run = m_new;
        // ---- P·V: thread d accumulates output dimension d over the block's keys
        const int nk = min(kDecThreads, key_end - k0);
#pragma unroll
        for (int i = 0; i < kDecMaxD / kDecThreads; ++i) {
            const int d = tid + i * kDecThreads;
            if (d < D) {
                float a = acc[i] * alpha;
                const T* vp = vbase + (int64_t)k0 * p.v_strides[2] + (int64_t)d * p.v_strides[3];
                for (int kk = 0; kk < nk; ++kk) a = fmaf(sc_s[kk], Elem<T>::to_f32(vp[(int64_t)kk * p.v_strides[2]]), a);
                acc[i] = a;
            }
        }
        __syncthreads();
    }
    float* out = p.scratch + (((int64_t)bh * p.M + row) * p.num_splits + split) * (D + 2);
    if (tid == 0) { out[0] = m_run; out[1] = l_run; }
#pragma unroll
    for (int i = 0; i < kDecMaxD / kDecThreads; ++i) {
        const int d = tid + i * kDecThreads;
        if (d < D) out[2 + d] = acc[i];
    }
}

// Coalesced variant of part 1 for the common layout (unit stride on the head dimension, rows 16-byte
// aligned, D = 8 * LPK with LPK lanes per key in {8, 16, 32}): the lanes of a warp cover 32/LPK whole
// keys per step with one 128-bit load each, so every load instruction of a warp reads 512 contiguous
// bytes of K (or V) and each byte is requested exactly once. Scores are reduced over the LPK lanes
// with shuffles; for P·V each lane accumulates its 8 output dimensions over the keys it sees and the
// 128/LPK key groups of the CTA are summed through shared memory at the end.
template <typename T, int LPK>
__global__ void __launch_bounds__(kDecThreads)
attn_decode_part1_vec_kernel(const DecDev p) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int D = LPK * 8;
    constexpr int KPW = 32 / LPK;                 // keys per warp per step
    constexpr int KPS = KPW * (kDecThreads / 32);  // keys per CTA per step
    constexpr int GROUPS = kDecThreads / LPK;      // key groups in the CTA
    __shared__ float sc_s[kDecThreads];
    __shared__ float red_s[kDecThreads / 32];
    __shared__ float acc_s[GROUPS][D + 4];
    // K and V tiles of 128 keys, staged with asynchronous 16-byte copies: a thread issues all of its
    // 2 x 16 copies for a tile up front and holds no registers for them, so a CTA has its whole
    // tile (64 KB at D = 128) in flight and three CTAs share an SM. With plain loads into registers
    // the kernel was bound by memory latency (ncu: 42 % of the warps resident, 22 long-scoreboard
    // stall cycles per issued instruction, 3.7 TB/s). Chunk j (16 bytes) of row r sits at
    // r * LPK + (j ^ ((r & 1) << 2)), which makes both read patterns below bank-conflict free.
    extern __shared__ uint4 kv_tiles[];
    uint4* k_tile = kv_tiles;
    uint4* v_tile = kv_tiles + kDecThreads * LPK;
    const int split = blockIdx.x, row = blockIdx.y, bh = blockIdx.z;
    const int b = bh / p.H, h = bh % p.H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int dl = lane % LPK;    // which 8-wide slice of the head dimension
    const int group = tid / LPK;  // == warp * KPW + sub

    // Scores on the tensor core: one mma.sync.m16n8k16 chain per group of 8 keys, q in row 0 of the A
    // operand (rows 1..15 are zero), the 8 keys as the columns of B. K is [key][d] with d contiguous,
    // which is exactly the "col" layout of B; every thread feeds the 16 bytes it loads (8 consecutive
    // d of one key) into two MMAs, with the same permutation of d inside an MMA for q and K. One
    // load and two MMAs per 16 bytes instead of one load, 8 conversions, 8 FMAs and log2(LPK)
    // shuffles: the scalar version spent ~45 instructions per 32 bytes of K/V and ran out of issue slots
    // at two thirds of the HBM bandwidth.
    const int g8 = lane >> 2, c4 = lane & 3;
    uint4 qf[D / 32];
    {
        const T* qp = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_strides[0] + (int64_t)h * p.q_strides[1] +
                      (int64_t)row * p.q_strides[2];
#pragma unroll
        for (int i = 0; i < D / 32; ++i)
            qf[i] = (g8 == 0) ? __ldg(reinterpret_cast<const uint4*>(qp + 32 * i + 8 * c4)) : make_uint4(0u, 0u, 0u, 0u);
    }
    const int hk = h / p.kv_group;
    const T* kbase0 = reinterpret_cast<const T*>(p.k) + (int64_t)b * p.k_strides[0] + (int64_t)hk * p.k_strides[1];
    const T* vbase0 = reinterpret_cast<const T*>(p.v) + (int64_t)b * p.v_strides[0] + (int64_t)hk * p.v_strides[1];
    auto stage_tile = [&](uint4* tile, const T* base, int64_t row_stride, int k0, int key_end) {
#pragma unroll 4
        for (int it = 0; it < LPK; ++it) {
            const int idx = it * kDecThreads + tid;
            const int r = idx / LPK, j = idx % LPK;
            const int key = k0 + r;
            const bool live = key < key_end;
            const T* src = base + (int64_t)(live ? key : k0) * row_stride + j * 8;
            const uint32_t dst = smem_u32(tile + r * LPK + (j ^ ((r & 1) << 2)));
            // src-size 0 for rows beyond the chunk: the 16 bytes are zero-filled, nothing is read
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(live ? 16 : 0) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const float mlow = mask_lowest(p.mask_dtype);
    const int64_t mask_off = p.mask ? (int64_t)b * p.mask_strides[0] + (int64_t)h * p.mask_strides[1] +
                                          (int64_t)row * p.mask_strides[2]
                                    : 0;
    float m_run = -INFINITY, l_run = 0.f;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;

    const int key_begin = split * p.chunk;
    const int key_end = min(decode_live_keys(p), key_begin + p.chunk);  // a chunk beyond the live keys scores nothing: (m, l) = (-inf, 0)
    for (int k0 = key_begin; k0 < key_end; k0 += kDecThreads) {
        stage_tile(k_tile, kbase0, p.k_strides[2], k0, key_end);
        stage_tile(v_tile, vbase0, p.v_strides[2], k0, key_end);
        asm volatile("cp.async.wait_group 1;" ::: "memory");  // this thread's K copies have landed
        __syncthreads();                                       // ... and everybody else's
        // ---- scores of the block's 128 keys: step s, warp w, group row g8 -> tile row 32 s + 8 w + g8
#pragma unroll
        for (int s = 0; s < kDecThreads / 32; ++s) {
            const int r = s * 32 + warp * 8 + g8;
            uint4 kf[D / 32];
#pragma unroll
            for (int i = 0; i < D / 32; ++i) kf[i] = k_tile[r * LPK + ((4 * i + c4) ^ ((r & 1) << 2))];
            float cacc[4] = {0.f, 0.f, 0.f, 0.f};
            // mma.sync.aligned needs the whole warp converged; the lanes that stored the previous
            // group's scores (g8 == 0, below) may still be apart from the others. Without this
            // barrier the kernel produced garbage for some CTAs whenever the GPU was busy.
            __syncwarp();
#pragma unroll
            for (int i = 0; i < D / 32; ++i) {
                mma_16816<T>(cacc, qf[i].x, 0u, qf[i].y, 0u, kf[i].x, kf[i].y);
                mma_16816<T>(cacc, qf[i].z, 0u, qf[i].w, 0u, kf[i].z, kf[i].w);
            }
            if (g8 == 0) {  // row 0 of the accumulator: lane c4 holds the scores of keys 2 c4 and 2 c4 + 1 of the group
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int kk = s * 32 + warp * 8 + 2 * c4 + e;
                    const int key2 = k0 + kk;
                    float sc = -INFINITY;
                    if (key2 < key_end && !(p.is_causal && key2 > row)) {
                        sc = cacc[e] * p.scale_log2;
                        if (p.mask) {
                            const float mv = mask_load(p.mask, mask_off + (int64_t)key2 * p.mask_strides[3], p.mask_dtype);
                            sc = fmaf(fmaxf(mv, mlow), kLog2e, sc);
                        }
                    }
                    sc_s[kk] = sc;
                }
            }
        }
        __syncthreads();
        // ---- block maximum and exponentials (one key per thread)
        const float sv = sc_s[tid];
        float mx = sv;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) red_s[warp] = mx;
        __syncthreads();
        mx = fmaxf(fmaxf(red_s[0], red_s[1]), fmaxf(red_s[2], red_s[3]));
        float m_new = fmaxf(m_run, mx);
        if (m_new == -INFINITY) m_new = 0.f;
        const float alpha = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_new);
        const float pe = fast_exp2(sv - m_new);
        __syncthreads();  // everyone has read sc_s and red_s
        // P is rounded to the input dtype before P·V, as the reference does (attention_skinny.py:262)
        sc_s[tid] = Elem<T>::to_f32(Elem<T>::from_f32(pe));
        float ps = pe;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        if (lane == 0) red_s[warp] = ps;
        __syncthreads();
        asm volatile("cp.async.wait_group 0;" ::: "memory");  // this thread's V copies have landed
        l_run = l_run * alpha + (red_s[0] + red_s[1] + red_s[2] + red_s[3]);
        m_run = m_new;
        __syncthreads();  // every thread's V copies are visible
        // ---- P·V with the same key-to-lane mapping
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] *= alpha;
#pragma unroll 4
        for (int s = 0; s < kDecThreads / KPS; ++s) {
            const int kk = s * KPS + group;
            const int key = k0 + kk;
            if (key < key_end) {
                const float pk = sc_s[kk];
                const uint4 w = v_tile[kk * LPK + (dl ^ ((kk & 1) << 2))];
                const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = Elem<T>::unpack2(ww[i]);
                    acc[2 * i] = fmaf(pk, f.x, acc[2 * i]);
                    acc[2 * i + 1] = fmaf(pk, f.y, acc[2 * i + 1]);
                }
            }
        }
        __syncthreads();  // sc_s and both tiles are rewritten by the next block
    }
    // ---- sum the key groups and write (m, l, acc[D])
#pragma unroll
    for (int i = 0; i < 8; ++i) acc_s[group][dl * 8 + i] = acc[i];
    __syncthreads();
    float* out = p.scratch + (((int64_t)bh * p.M + row) * p.num_splits + split) * (D + 2);
    if (tid == 0) { out[0] = m_run; out[1] = l_run; }
    for (int d = tid; d < D; d += kDecThreads) {
        float a = 0.f;
#pragma unroll
        for (int g = 0; g < GROUPS; ++g) a += acc_s[g][d];
        out[2 + d] = a;
    }
}

template <typename T>
__global__ void __launch_bounds__(kDecThreads)
attn_decode_part2_kernel(const DecDev p) {
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x, bh = blockIdx.y;
    const int b = bh / p.H, h = bh % p.H;
    const int D = p.D;
    const float* in = p.scratch + ((int64_t)bh * p.M + row) * p.num_splits * (D + 2);
    float m_tot = -INFINITY;
    for (int s = 0; s < p.num_splits; ++s) m_tot = fmaxf(m_tot, in[(int64_t)s * (D + 2)]);
    float l_tot = 0.f;
    for (int s = 0; s < p.num_splits; ++s) {
        const float ms = in[(int64_t)s * (D + 2)];
        if (ms != -INFINITY) l_tot += in[(int64_t)s * (D + 2) + 1] * fast_exp2(ms - m_tot);
    }
    T* op = reinterpret_cast<T*>(p.o) + (int64_t)b * p.o_strides[0] + (int64_t)h * p.o_strides[1] +
            (int64_t)row * p.o_strides[2];
    for (int d = threadIdx.x; d < D; d += kDecThreads) {
        float a = 0.f;
        for (int s = 0; s < p.num_splits; ++s) {
            const float ms = in[(int64_t)s * (D + 2)];
            if (ms != -INFINITY) a += in[(int64_t)s * (D + 2) + 2 + d] * fast_exp2(ms - m_tot);
        }
        op[(int64_t)d * p.o_strides[3]] = Elem<T>::from_f32(a / l_tot);
    }
}

template <typename T, int LPK>
static void launch_decode_vec(dim3 grid, cudaStream_t stream, const DecDev& d) {
    constexpr size_t smem = 2 * (size_t)kDecThreads * LPK * sizeof(uint4);  // K tile + V tile
    static PerDeviceOnce attr_once;
    if (attr_once.first_time()) {
        cudaFuncSetAttribute(attn_decode_part1_vec_kernel<T, LPK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }
    launch_pdl(attn_decode_part1_vec_kernel<T, LPK>, grid, kDecThreads, smem, stream, d);
}

static int launch_attention_decode(const kb_attn_params& p, void* scratch, int64_t scratch_bytes, cudaStream_t stream) {
    if (p.N <= 0 || p.D > kDecMaxD) return KB_ERR_UNSUPPORTED;
    if (p.M > 65535 || p.B * p.H > 65535) return KB_ERR_UNSUPPORTED;
    if (scratch == nullptr) return KB_ERR_BAD_ARG;
    const int64_t need = decode_scratch_bytes(p.B, p.H, p.M, p.N, p.D);
    if (scratch_bytes < need) return KB_ERR_BAD_ARG;
    DecDev d;
    d.q = p.q; d.k = p.k; d.v = p.v; d.o = p.o; d.mask = p.mask;
    for (int i = 0; i < 4; ++i) {
        d.q_strides[i] = p.q_strides[i]; d.k_strides[i] = p.k_strides[i]; d.v_strides[i] = p.v_strides[i];
        d.o_strides[i] = p.o_strides[i]; d.mask_strides[i] = p.mask ? p.mask_strides[i] : 0;
    }
    d.B = (int)p.B; d.H = (int)p.H; d.M = (int)p.M; d.N = (int)p.N; d.D = (int)p.D;
    d.scale_log2 = p.sm_scale * kLog2e;
    d.is_causal = p.is_causal ? 1 : 0;
    d.mask_dtype = p.mask ? p.mask_dtype : KB_F32;
    decode_split(p.N, p.B * p.H * p.M, &d.num_splits, &d.chunk);
    d.kv_group = p.kv_group > 1 ? p.kv_group : 1;
    if (p.H % d.kv_group != 0) return KB_ERR_BAD_ARG;
    d.kv_len_dev = reinterpret_cast<const long long*>(p.kv_len_dev);
    d.scratch = reinterpret_cast<float*>(scratch);
    const dim3 g1((unsigned)d.num_splits, (unsigned)p.M, (unsigned)(p.B * p.H));
    const dim3 g2((unsigned)p.M, (unsigned)(p.B * p.H));
    const bool vec_ok = (p.D == 64 || p.D == 128 || p.D == 256) && p.q_strides[3] == 1 && p.k_strides[3] == 1 &&
                        p.v_strides[3] == 1 && (p.k_strides[2] % 8) == 0 && (p.v_strides[2] % 8) == 0 &&
                        (p.k_strides[1] % 8) == 0 && (p.v_strides[1] % 8) == 0 && (p.k_strides[0] % 8) == 0 &&
                        (p.v_strides[0] % 8) == 0 && (((uintptr_t)p.k) & 15) == 0 && (((uintptr_t)p.v) & 15) == 0 &&
                        (((uintptr_t)p.q) & 15) == 0 && (p.q_strides[0] % 8) == 0 && (p.q_strides[1] % 8) == 0 &&
                        (p.q_strides[2] % 8) == 0;
    if (p.dtype == KB_F16) {
        if (vec_ok && p.D == 64) launch_decode_vec<__half, 8>(g1, stream, d);
        else if (vec_ok && p.D == 128) launch_decode_vec<__half, 16>(g1, stream, d);
        else if (vec_ok && p.D == 256) launch_decode_vec<__half, 32>(g1, stream, d);
        else launch_pdl(attn_decode_part1_kernel<__half>, g1, kDecThreads, 0, stream, d);
        launch_pdl(attn_decode_part2_kernel<__half>, g2, kDecThreads, 0, stream, d);
    } else {
        if (vec_ok && p.D == 64) launch_decode_vec<__nv_bfloat16, 8>(g1, stream, d);
        else if (vec_ok && p.D == 128) launch_decode_vec<__nv_bfloat16, 16>(g1, stream, d);
        else if (vec_ok && p.D == 256) launch_decode_vec<__nv_bfloat16, 32>(g1, stream, d);
        else launch_pdl(attn_decode_part1_kernel<__nv_bfloat16>, g1, kDecThreads, 0, stream, d);
        launch_pdl(attn_decode_part2_kernel<__nv_bfloat16>, g2, kDecThreads, 0, stream, d);
    }
    return cudaGetLastError() == cudaSuccess ? KB_OK : KB_ERR_LAUNCH;
}

}  // namespace kb
