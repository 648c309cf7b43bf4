// Rotary position embedding fused with the KV-cache write, for the Llama-shaped decoder.
// Input: the output of the fused QKV projection, [tokens, 3, heads, D] (16-bit). For every token
// the kernel rotates q and k on interleaved pairs (x[2i], x[2i+1]) by the angle of the token's
// position, writes q to [B, S, heads, D] and writes the rotated k and the untouched v into the
// caches [B, heads, max_seq, D] at that position — one launch instead of the dozen elementwise
// kernels and two index-copies of an eager implementation. The start position comes from device
// memory when given (so that a captured decode step stays valid as the position advances).
// Semantics: experimental/llama-v2/kernel/pytorch_reference.py:37-80 of the reference (interleaved
// pairs, theta = 10000); its Triton counterpart is the RoPE epilogue of fused_kernel_proj_qkv.py.
#pragma once
#include "common.cuh"

namespace kb {

struct RopeDev {
    const void* qkv;
    void* q_out;
    void* k_cache;
    void* v_cache;
    const float* cos_t;  // [max_seq, D/2]
    const float* sin_t;
    const long long* pos_dev;  // optional: start position on the device
    long long pos_host;
    int B, S, H, D, max_seq;
};

// One thread per (token, head, 8 consecutive elements = 4 rotation pairs).
template <typename T>
__global__ void __launch_bounds__(256)
rope_kv_write_kernel(const RopeDev p) {
    pdl_wait();
    pdl_launch_dependents();
    const int vec_per_head = p.D / 8;
    const long long total = (long long)p.B * p.S * p.H * vec_per_head;
    const long long start = p.pos_dev ? *p.pos_dev : p.pos_host;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int v = (int)(i % vec_per_head);
        const int h = (int)((i / vec_per_head) % p.H);
        const long long tok = i / ((long long)vec_per_head * p.H);  // b * S + s
        const int s = (int)(tok % p.S);
        const int b = (int)(tok / p.S);
        const long long pos = start + s;
        if (pos < 0 || pos >= p.max_seq) continue;
        const T* base = reinterpret_cast<const T*>(p.qkv) + tok * (3LL * p.H * p.D) + (long long)h * p.D + v * 8;
        const uint4 qw = *reinterpret_cast<const uint4*>(base);
        const uint4 kw = *reinterpret_cast<const uint4*>(base + (long long)p.H * p.D);
        const uint4 vw = *reinterpret_cast<const uint4*>(base + 2LL * p.H * p.D);
        const float4 c = *reinterpret_cast<const float4*>(p.cos_t + pos * (p.D / 2) + v * 4);
        const float4 sn = *reinterpret_cast<const float4*>(p.sin_t + pos * (p.D / 2) + v * 4);
        const float cs[4] = {c.x, c.y, c.z, c.w}, ss[4] = {sn.x, sn.y, sn.z, sn.w};
        const uint32_t qi[4] = {qw.x, qw.y, qw.z, qw.w}, ki[4] = {kw.x, kw.y, kw.z, kw.w};
        uint32_t qo[4], ko[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 qf = Elem<T>::unpack2(qi[j]);
            const float2 kf = Elem<T>::unpack2(ki[j]);
            qo[j] = Elem<T>::pack2(qf.x * cs[j] - qf.y * ss[j], qf.x * ss[j] + qf.y * cs[j]);
            ko[j] = Elem<T>::pack2(kf.x * cs[j] - kf.y * ss[j], kf.x * ss[j] + kf.y * cs[j]);
        }
        T* qdst = reinterpret_cast<T*>(p.q_out) + (tok * p.H + h) * (long long)p.D + v * 8;
        *reinterpret_cast<uint4*>(qdst) = make_uint4(qo[0], qo[1], qo[2], qo[3]);
        const long long coff = (((long long)b * p.H + h) * p.max_seq + pos) * p.D + v * 8;
        *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.k_cache) + coff) = make_uint4(ko[0], ko[1], ko[2], ko[3]);
        *reinterpret_cast<uint4*>(reinterpret_cast<T*>(p.v_cache) + coff) = vw;
    }
}

template <typename T>
static int launch_rope_t(const RopeDev& d, cudaStream_t stream) {
    const long long total = (long long)d.B * d.S * d.H * (d.D / 8);
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    launch_pdl(rope_kv_write_kernel<T>, (unsigned)blocks, 256, 0, stream, d);
    return cudaGetLastError() == cudaSuccess ? KB_OK : KB_ERR_LAUNCH;
}

}  // namespace kb
