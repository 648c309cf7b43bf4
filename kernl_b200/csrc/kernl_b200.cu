// C ABI of the kernl_b200 kernels (declared in include/kernl_b200.h) and the host helpers they
// share. All kernels live in this single translation unit so that they share one device status word.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/kernl_b200_debug.h"
#include "common.cuh"
#include "norm.cuh"
#include "linear.cuh"
#include "linear_pair.cuh"
#include "linear_smallm.cuh"
#include "attention.cuh"
#include "attention_split.cuh"
#include "attention_persist.cuh"
#include "attention_decode.cuh"
#include "allreduce.cuh"
#include "rope.cuh"

namespace kb {

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

static PFN_encodeTiled get_encode_fn() {
    static PFN_encodeTiled fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_encodeTiled>(p);
    });
    return fn;
}

int encode_tmap_16bit(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swz,
                      CUtensorMapL2promotion l2) {
    PFN_encodeTiled fn = get_encode_fn();
    if (fn == nullptr) return KB_ERR_NO_DEVICE;
    if (((uintptr_t)base & 15) != 0) return KB_ERR_UNSUPPORTED;
    cuuint64_t gdims[5];
    cuuint64_t gstrides[4];
    cuuint32_t gbox[5], estr[5];
    for (int i = 0; i < rank; ++i) {
        gdims[i] = dims[i];
        gbox[i] = box[i];
        estr[i] = 1;
        if (i > 0) {
            if (strides_bytes[i] % 16 != 0) return KB_ERR_UNSUPPORTED;
            gstrides[i - 1] = strides_bytes[i];
        }
    }
    // CU_TENSOR_MAP_DATA_TYPE_FLOAT16 and BFLOAT16 move bytes identically; zero fill for OOB.
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gdims,
                    gstrides, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, l2,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? KB_OK : KB_ERR_UNSUPPORTED;
}

// Both answers are per device (a process may drive several GPUs), cached per device index.
int sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) return 148;
    if (dev >= 0 && dev < 64) cached[dev] = v;
    return v;
}

static std::atomic<int> g_gemm_sm_limit{0};  // 0 = no limit
int gemm_sms() {
    const int all = sm_count(), lim = g_gemm_sm_limit.load(std::memory_order_relaxed);
    return (lim > 0 && lim < all) ? lim : all;
}

static int check_device() {
    static int state[64] = {};  // per device: 0 unknown, 1 ok, -1 not an sm_100 device
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return KB_ERR_NO_DEVICE;
    }
    const bool cacheable = dev >= 0 && dev < 64;
    if (!cacheable || state[dev] == 0) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
            cudaGetLastError();
            return KB_ERR_NO_DEVICE;
        }
        if (!cacheable) return major == 10 ? KB_OK : KB_ERR_NO_DEVICE;
        state[dev] = (major == 10) ? 1 : -1;
    }
    return state[dev] == 1 ? KB_OK : KB_ERR_NO_DEVICE;
}

static int g_forced_bn = 0;
static int g_forced_splits = 0;

}  // namespace kb

using namespace kb;

extern "C" {

int kb_version(void) { return 100; }

int kb_gemm_sm_limit(int sms) {
    if (sms < 0) return KB_ERR_BAD_ARG;
    g_gemm_sm_limit.store(sms, std::memory_order_relaxed);
    return KB_OK;
}

const char* kb_status_str(int status) {
    switch (status) {
        case KB_OK: return "ok";
        case KB_ERR_BAD_ARG: return "bad argument";
        case KB_ERR_UNSUPPORTED: return "unsupported shape, stride, alignment or dtype";
        case KB_ERR_LAUNCH: return "CUDA launch error";
        case KB_ERR_TIMEOUT: return "a bounded device-side wait expired";
        case KB_ERR_NO_DEVICE: return "no sm_100 CUDA device";
        case KB_ERR_TOO_LARGE: return "size beyond the fixed maximum of this entry point";
        default: return "unknown status";
    }
}

int kb_device_status_read(int32_t* status_out) {
    if (status_out == nullptr) return KB_ERR_BAD_ARG;
    int st = check_device();
    if (st != KB_OK) return st;
    int h[4] = {0, 0, 0, 0};
    if (cudaDeviceSynchronize() != cudaSuccess) return KB_ERR_LAUNCH;
    if (cudaMemcpyFromSymbol(h, g_device_status, sizeof(h)) != cudaSuccess) return KB_ERR_LAUNCH;
    for (int i = 0; i < 4; ++i) status_out[i] = h[i];
    if (h[0] != 0) {
        int z[4] = {0, 0, 0, 0};
        if (cudaMemcpyToSymbol(g_device_status, z, sizeof(z)) != cudaSuccess) return KB_ERR_LAUNCH;
        return KB_ERR_TIMEOUT;
    }
    return KB_OK;
}

int kb_norm_fwd(const kb_norm_params* p, void* stream) {
    if (p == nullptr || p->x == nullptr || p->y == nullptr || p->gamma == nullptr) return KB_ERR_BAD_ARG;
    if (p->rows < 0 || p->cols <= 0) return KB_ERR_BAD_ARG;
    if (p->residual != nullptr && p->sum_out == nullptr) return KB_ERR_BAD_ARG;
    if (p->residual != nullptr && ((((uintptr_t)p->residual) | ((uintptr_t)p->sum_out)) & 15)) return KB_ERR_UNSUPPORTED;
    if (p->rows == 0) return KB_OK;
    int st = check_device();
    if (st != KB_OK) return st;
    st = launch_norm(*p, (cudaStream_t)stream);
    if (st != KB_OK) return st;
    return cudaGetLastError() == cudaSuccess ? KB_OK : KB_ERR_LAUNCH;
}

// Test and measurement hooks (include/kernl_b200_debug.h; not part of the stable ABI; process-wide).
void kb_debug_force_bn(int bn) { g_forced_bn = bn; }
void kb_debug_split_tiles(int v) { g_split_tiles = v; }
void kb_debug_attention_persistent(int mode) {
    g_attn_persistent = mode == 2 ? 1 : mode;
    g_attn_sort_batches = mode == 2 ? 0 : 1;
}
void kb_debug_pdl(int on) { g_use_pdl = on ? 1 : 0; }
void kb_debug_linear_pair(int mode) { g_linear_pair = (mode == 192 || mode == 256) ? mode : (mode ? 1 : 0); }
void kb_debug_force_splits(int splits) { g_forced_splits = splits; }
#ifdef KB_ATTN_TRACE
// Tuning builds only: copies the persistent attention kernel's time stamps to the host.
int kb_debug_attention_trace_read(void* host_buf, int64_t bytes) {
    if (cudaDeviceSynchronize() != cudaSuccess) return KB_ERR_LAUNCH;
    const size_t n = sizeof(unsigned long long) * 296 * (kTraceTiles + 1) * kTraceEvents;
    if (bytes < (int64_t)n) return KB_ERR_BAD_ARG;
    return cudaMemcpyFromSymbol(host_buf, g_attn_trace, n) == cudaSuccess ? KB_OK : KB_ERR_LAUNCH;
}
#endif
#ifdef KB_GEMM_TRACE
// Tuning builds only: copies the CTA-pair GEMM's clock stamps to the host.
int kb_debug_gemm_trace_read(void* host_buf, int64_t bytes) {
    if (cudaDeviceSynchronize() != cudaSuccess) return KB_ERR_LAUNCH;
    const size_t n = sizeof(long long) * 148 * 8 * 16;
    if (bytes < (int64_t)n) return KB_ERR_BAD_ARG;
    return cudaMemcpyFromSymbol(host_buf, g_gemm_trace, n) == cudaSuccess ? KB_OK : KB_ERR_LAUNCH;
}
#endif
int kb_debug_wait_limit(int64_t in_kernel_cycles, int64_t peer_cycles) {
    int st = check_device();
    if (st != KB_OK) return st;
    const long long a = in_kernel_cycles > 0 ? (long long)in_kernel_cycles : kWaitLimitCycles;
    const long long b = peer_cycles > 0 ? (long long)peer_cycles : kPeerWaitLimitCycles;
    if (cudaDeviceSynchronize() != cudaSuccess) return KB_ERR_LAUNCH;
    if (cudaMemcpyToSymbol(g_wait_limit_cycles, &a, sizeof(a)) != cudaSuccess) return KB_ERR_LAUNCH;
    if (cudaMemcpyToSymbol(g_peer_wait_limit_cycles, &b, sizeof(b)) != cudaSuccess) return KB_ERR_LAUNCH;
    return cudaDeviceSynchronize() == cudaSuccess ? KB_OK : KB_ERR_LAUNCH;
}

int kb_linear_fwd(const kb_linear_params* p, void* stream) {
    if (p == nullptr || p->x == nullptr || p->w == nullptr || p->y == nullptr) return KB_ERR_BAD_ARG;
    if (p->M < 0 || p->N <= 0 || p->K <= 0) return KB_ERR_BAD_ARG;
    if (p->activation < KB_ACT_NONE || p->activation > KB_ACT_SWIGLU) return KB_ERR_BAD_ARG;
    if (p->activation == KB_ACT_SWIGLU && (p->N % 16 != 0 || p->act_inputs != nullptr)) return KB_ERR_BAD_ARG;
    if (p->M == 0) return KB_OK;
    if (p->K % 8 != 0 || p->x_row_stride % 8 != 0) return KB_ERR_UNSUPPORTED;
    if (((uintptr_t)p->x & 15) || ((uintptr_t)p->w & 15)) return KB_ERR_UNSUPPORTED;
    if (p->M > 0x7fffffff || p->N > 0x7fffffff || p->K > 0x7fffffff) return KB_ERR_UNSUPPORTED;
    int st = check_device();
    if (st != KB_OK) return st;
    // a handful of rows: one pass over W, no tensor map / TMEM / split-K finish (unless a test forces
    // a tile shape or a split count of the GEMM kernel)
    if (g_forced_bn == 0 && g_forced_splits == 0 && smallm_applicable(*p)) return launch_linear_smallm(*p, (cudaStream_t)stream);
    return launch_linear(*p, (cudaStream_t)stream, g_forced_bn, g_forced_splits);
}

int64_t kb_linear_workspace_bytes(int64_t M, int64_t N) {
    if (M <= 0 || N <= 0) return 0;
    return splitk_workspace_bytes(M, N);
}

int kb_silu_mul(const void* gu, void* y, int64_t M, int64_t N, int32_t dtype, void* stream) {
    if (gu == nullptr || y == nullptr || M < 0 || N <= 0) return KB_ERR_BAD_ARG;
    if (M == 0) return KB_OK;
    if (N % 8 != 0 || ((uintptr_t)gu & 15) || ((uintptr_t)y & 15)) return KB_ERR_UNSUPPORTED;
    int st = check_device();
    if (st != KB_OK) return st;
    const int64_t total = M * (N / 8);
    const int threads = 256;
    int64_t blocks = (total + threads - 1) / threads;
    if (blocks > (int64_t)sm_count() * 16) blocks = (int64_t)sm_count() * 16;
    if (dtype == KB_F16)
        launch_pdl(silu_mul_kernel<__half>, (unsigned)blocks, threads, 0, (cudaStream_t)stream, (const __half*)gu, (__half*)y, M, N);
    else if (dtype == KB_BF16)
        launch_pdl(silu_mul_kernel<__nv_bfloat16>, (unsigned)blocks, threads, 0, (cudaStream_t)stream,
                   (const __nv_bfloat16*)gu, (__nv_bfloat16*)y, M, N);
    else
        return KB_ERR_UNSUPPORTED;
    return cudaGetLastError() == cudaSuccess ? KB_OK : KB_ERR_LAUNCH;
}

static int check_attn(const kb_attn_params* p) {
    if (p == nullptr || p->q == nullptr || p->k == nullptr || p->v == nullptr || p->o == nullptr)
        return KB_ERR_BAD_ARG;
    if (p->B < 0 || p->H < 0 || p->M < 0 || p->N < 0 || p->D <= 0) return KB_ERR_BAD_ARG;
    if (p->dtype != KB_F16 && p->dtype != KB_BF16) return KB_ERR_UNSUPPORTED;
    if (p->mask != nullptr && p->mask_dtype != KB_F16 && p->mask_dtype != KB_BF16 && p->mask_dtype != KB_F32)
        return KB_ERR_UNSUPPORTED;
    if (p->kv_group < 0 || (p->kv_group > 1 && p->H % p->kv_group != 0)) return KB_ERR_BAD_ARG;
    return KB_OK;
}

int kb_attention_fwd(const kb_attn_params* p, void* stream) {
    int st = check_attn(p);
    if (st != KB_OK) return st;
    if (p->kv_len_dev != nullptr) return KB_ERR_UNSUPPORTED;  // a device-side key count is a decode-entry feature
    if (p->B == 0 || p->H == 0 || p->M == 0) return KB_OK;
    st = check_device();
    if (st != KB_OK) return st;
    return launch_attention(*p, (cudaStream_t)stream);
}

int64_t kb_attention_decode_scratch_bytes(int64_t B, int64_t H, int64_t M, int64_t N, int64_t D) {
    return decode_scratch_bytes(B, H, M, N, D);
}

int kb_attention_decode_fwd(const kb_attn_params* p, void* scratch, int64_t scratch_bytes, void* stream) {
    int st = check_attn(p);
    if (st != KB_OK) return st;
    if (p->B == 0 || p->H == 0 || p->M == 0) return KB_OK;
    st = check_device();
    if (st != KB_OK) return st;
    return launch_attention_decode(*p, scratch, scratch_bytes, (cudaStream_t)stream);
}

int kb_rope_kv_write(const kb_rope_params* p, void* stream) {
    if (p == nullptr || p->qkv == nullptr || p->q_out == nullptr || p->k_cache == nullptr || p->v_cache == nullptr ||
        p->cos == nullptr || p->sin == nullptr)
        return KB_ERR_BAD_ARG;
    if (p->B < 0 || p->S < 0 || p->H <= 0 || p->D <= 0 || p->max_seq <= 0) return KB_ERR_BAD_ARG;
    if (p->D % 8 != 0) return KB_ERR_UNSUPPORTED;
    if ((((uintptr_t)p->qkv) | ((uintptr_t)p->q_out) | ((uintptr_t)p->k_cache) | ((uintptr_t)p->v_cache) |
         ((uintptr_t)p->cos) | ((uintptr_t)p->sin)) & 15)
        return KB_ERR_UNSUPPORTED;
    if (p->B == 0 || p->S == 0) return KB_OK;
    int st = check_device();
    if (st != KB_OK) return st;
    RopeDev d;
    d.qkv = p->qkv; d.q_out = p->q_out; d.k_cache = p->k_cache; d.v_cache = p->v_cache;
    d.cos_t = p->cos; d.sin_t = p->sin;
    d.pos_dev = reinterpret_cast<const long long*>(p->pos_dev);
    d.pos_host = p->pos_host;
    d.B = (int)p->B; d.S = (int)p->S; d.H = (int)p->H; d.D = (int)p->D; d.max_seq = (int)p->max_seq;
    if (p->dtype == KB_F16) return launch_rope_t<__half>(d, (cudaStream_t)stream);
    if (p->dtype == KB_BF16) return launch_rope_t<__nv_bfloat16>(d, (cudaStream_t)stream);
    return KB_ERR_UNSUPPORTED;
}

int kb_allreduce_residual_fwd(const kb_allreduce_params* p, void* stream) {
    if (p == nullptr || p->out == nullptr) return KB_ERR_BAD_ARG;
    if (p->world < 1 || p->world > KB_ALLREDUCE_MAX_WORLD || p->rank < 0 || p->rank >= p->world) return KB_ERR_BAD_ARG;
    if (p->count < 0 || p->count % 8 != 0) return KB_ERR_UNSUPPORTED;
    if (p->count * 2 > KB_ALLREDUCE_MAX_BYTES) return KB_ERR_TOO_LARGE;
    if (p->dtype != KB_F16 && p->dtype != KB_BF16) return KB_ERR_UNSUPPORTED;
    if (p->count == 0) return KB_OK;
    ArDev d;
    for (int r = 0; r < KB_ALLREDUCE_MAX_WORLD; ++r) {
        d.bufs[r] = r < p->world ? p->partials[r] : nullptr;
        d.flags[r] = r < p->world ? p->flags[r] : nullptr;
        if (r < p->world && (p->partials[r] == nullptr || p->flags[r] == nullptr)) return KB_ERR_BAD_ARG;
        if (r < p->world && (((uintptr_t)p->partials[r]) & 15)) return KB_ERR_UNSUPPORTED;
    }
    if ((((uintptr_t)p->out) & 15) || (p->residual != nullptr && (((uintptr_t)p->residual) & 15))) return KB_ERR_UNSUPPORTED;
    d.residual = p->residual;
    d.out = p->out;
    d.n = p->count;
    d.rank = p->rank;
    d.world = p->world;
    d.norm_weight = p->norm_weight;
    d.norm_out = p->norm_out;
    d.cols = (int)p->cols;
    d.eps = p->eps;
    if (p->norm_weight != nullptr) {
        if (p->norm_out == nullptr || p->cols <= 0) return KB_ERR_BAD_ARG;
        if (p->cols % 8 != 0 || p->cols > kArNormMaxCols || p->count % p->cols != 0) return KB_ERR_UNSUPPORTED;
        if ((((uintptr_t)p->norm_weight) | ((uintptr_t)p->norm_out)) & 15) return KB_ERR_UNSUPPORTED;
    }
    int st = check_device();
    if (st != KB_OK) return st;
    return p->dtype == KB_F16 ? launch_allreduce_t<__half>(d, (cudaStream_t)stream)
                              : launch_allreduce_t<__nv_bfloat16>(d, (cudaStream_t)stream);
}

// Peer-mapped buffers for kb_allreduce_residual_fwd. Plain CUDA IPC: the owner allocates with
// cudaMalloc and exports a 64-byte handle, every peer process opens it (which enables peer access
// over NVLink). No multicast / NVLS object is created for these buffers.
int kb_peer_alloc(int64_t bytes, void** out) {
    if (out == nullptr || bytes <= 0) return KB_ERR_BAD_ARG;
    int st = check_device();
    if (st != KB_OK) return st;
    void* p = nullptr;
    if (cudaMalloc(&p, (size_t)bytes) != cudaSuccess) { cudaGetLastError(); return KB_ERR_LAUNCH; }
    if (cudaMemset(p, 0, (size_t)bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
        cudaFree(p);
        return KB_ERR_LAUNCH;
    }
    *out = p;
    return KB_OK;
}
int kb_peer_free(void* p) { return (p == nullptr || cudaFree(p) == cudaSuccess) ? KB_OK : KB_ERR_LAUNCH; }
int kb_peer_export(void* p, void* handle64) {
    if (p == nullptr || handle64 == nullptr) return KB_ERR_BAD_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) { cudaGetLastError(); return KB_ERR_LAUNCH; }
    memcpy(handle64, &h, 64);
    return KB_OK;
}
int kb_peer_open(const void* handle64, void** out) {
    if (handle64 == nullptr || out == nullptr) return KB_ERR_BAD_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void* p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); return KB_ERR_LAUNCH; }
    *out = p;
    return KB_OK;
}
int kb_peer_close(void* p) { return (p == nullptr || cudaIpcCloseMemHandle(p) == cudaSuccess) ? KB_OK : KB_ERR_LAUNCH; }

// -------------------------------------------------------------------------------------------------
// Decode attention without any allocation by the caller.
//
// kb_attention_decode_fwd needs a scratch buffer for the per-chunk partial results, which its caller
// has to get from somewhere. Some callers have no device allocator to ask: a custom-op hook of a
// serving runtime that is handed nothing but input and output buffers, or a process whose device
// memory has been reserved up front by another framework's pool so that a cudaMalloc of its own
// would fail or fragment the pool. For them the scratch lives in the library image itself.
//
// The array below is device memory that every GPU loading this library carries until the process
// exits (kStaticScratchBytes per GPU). Its name is only a host-side handle: the device address is
// obtained with cudaGetSymbolAddress, once per device, with that device current, and cached.
// -------------------------------------------------------------------------------------------------
namespace kb {
constexpr size_t kStaticScratchBytes = 4u << 20;  // 4 MiB
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_static_scratch_addr[kMaxDevices] = {nullptr};
static std::mutex g_static_scratch_mutex;

// Device address of the static scratch on the CURRENT device (looked up on the first call per device).
static int static_scratch_for_current_device(void** out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return KB_ERR_NO_DEVICE;
    if (dev < 0 || dev >= kMaxDevices) return KB_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_addr[dev] == nullptr) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_decode_static_scratch) != cudaSuccess || ptr == nullptr) {
            cudaGetLastError();
            return KB_ERR_LAUNCH;
        }
        g_static_scratch_addr[dev] = ptr;
    }
    *out = g_static_scratch_addr[dev];
    return KB_OK;
}
}  // namespace kb

int64_t kb_attention_decode_static_max_bytes(void) { return (int64_t)kb::kStaticScratchBytes; }

int kb_attention_decode_fwd_static(const kb_attn_params* p, void* stream) {
    int st = check_attn(p);
    if (st != KB_OK) return st;
    if (p->B == 0 || p->H == 0 || p->M == 0) return KB_OK;
    const int64_t need = decode_scratch_bytes(p->B, p->H, p->M, p->N, p->D);
    if (need < 0) return KB_ERR_BAD_ARG;
    if (need > (int64_t)kb::kStaticScratchBytes) return KB_ERR_TOO_LARGE;
    st = check_device();
    if (st != KB_OK) return st;
    void* scratch = nullptr;
    st = kb::static_scratch_for_current_device(&scratch);
    if (st != KB_OK) return st;
    // Nothing in the scratch has to start at zero: the first kernel writes every slot that the
    // second one reads, so stale contents of an earlier call are never observed.
    return launch_attention_decode(*p, scratch, (int64_t)kb::kStaticScratchBytes, (cudaStream_t)stream);
}

}  // extern "C"
