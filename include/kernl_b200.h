/*
 * kernl_b200 — C ABI of the B200 (sm_100a) fused transformer-inference kernels.
 *
 * Every entry point is asynchronous on the CUDA stream it is given, allocates nothing,
 * never synchronises the device (except kb_device_status_read) and returns a KB_* status.
 * Pointers are device pointers unless stated otherwise. Strides are in ELEMENTS.
 * `stream` is a cudaStream_t passed as void* so that this header needs no CUDA include.
 *
 * Each function cites the interface of the reference project (ELS-RD/kernl) that it
 * replaces, as <file>:<line> relative to that project's root.
 */
#ifndef KERNL_B200_H
#define KERNL_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes -------------------------------------------------------------------- */
#define KB_OK               0
#define KB_ERR_BAD_ARG     (-1)  /* null pointer, negative size, bad enum                   */
#define KB_ERR_UNSUPPORTED (-2)  /* shape/stride/dtype outside what the kernels implement   */
#define KB_ERR_LAUNCH      (-3)  /* CUDA runtime/driver reported an error at launch         */
#define KB_ERR_TIMEOUT     (-4)  /* a bounded device-side wait expired (see status word)    */
#define KB_ERR_NO_DEVICE   (-5)  /* no CUDA device / not an sm_100 device                   */
#define KB_ERR_TOO_LARGE   (-6)  /* size beyond a documented fixed maximum                  */

/* ---- element types ------------------------------------------------------------------- */
#define KB_F16  0
#define KB_BF16 1
#define KB_F32  2   /* accepted for attention masks only */

/* ---- activations fused in the linear epilogue.
 * Reference: src/kernl/implementations/activation_func.py:28-49 (tanh, relu, fast_gelu, gelu);
 * SILU has no counterpart there (needed by the Llama-shaped decoder). ---------------------- */
#define KB_ACT_NONE      0
#define KB_ACT_TANH      1
#define KB_ACT_GELU      2   /* exact erf form  */
#define KB_ACT_FAST_GELU 3   /* tanh approximation */
#define KB_ACT_RELU      4
#define KB_ACT_SILU      5
/* Gated feed-forward: the rows of W are interleaved in blocks of eight (block 2j = gate rows
 * 8j..8j+7, block 2j+1 = the matching up rows), N counts all of them (a multiple of 16), and y is
 * [M, N/2] with y[:, 8j+i] = silu(gate) * up — the silu(w1 x) * (w3 x) of the reference's fused
 * feed-forward experiment (experimental/llama-v2/kernel/fused_kernel_ff.py:10-114). No act_inputs. */
#define KB_ACT_SWIGLU    6

/* ---------------------------------------------------------------------------------------
 * LayerNorm / RMSNorm forward.
 * Replaces: src/kernl/implementations/layer_norm.py:279-335 (LayerNorm.forward launching
 * _layer_norm_fwd_fused_single_pass, :114-205).
 *   y[r,c] = (x[r,c]-mean_r) * rstd_r * gamma[c] + beta[c]         (is_rms == 0)
 *   y[r,c] =  x[r,c] * rsqrt(mean(x_r^2)+eps) * gamma[c]           (is_rms != 0, beta unused)
 * Statistics are computed in fp32 with the biased variance. The fp16 eps clamp
 * (eps = max(eps, 1.6e-5), layer_norm.py:295-296) is the CALLER's job: eps is used as given.
 * mean / rstd are optional fp32 [rows] side outputs (NULL to skip).
 * residual / sum_out (an addition over the reference, for pre-norm decoders): the kernel first forms
 * s = x + residual, stores s to sum_out and normalises s. Needs unit column strides, cols % 8 == 0,
 * cols <= 6144.
 * ------------------------------------------------------------------------------------- */
typedef struct {
    const void* x;          /* [rows, cols], strides x_row_stride / x_col_stride          */
    void*       y;          /* [rows, cols], strides y_row_stride / y_col_stride          */
    const void* gamma;      /* [cols] contiguous                                          */
    const void* beta;       /* [cols] contiguous or NULL                                  */
    float*      mean;       /* [rows] or NULL                                             */
    float*      rstd;       /* [rows] or NULL                                             */
    int64_t     rows, cols;
    int64_t     x_row_stride, x_col_stride;
    int64_t     y_row_stride, y_col_stride;
    float       eps;
    int32_t     is_rms;
    int32_t     dtype;      /* KB_F16 / KB_BF16 (x, y, gamma, beta share it)              */
    const void* residual;   /* optional [rows, cols] contiguous: normalise x + residual   */
    void*       sum_out;    /* required with residual: receives x + residual (contiguous) */
} kb_norm_params;

int kb_norm_fwd(const kb_norm_params* p, void* stream);

/* ---------------------------------------------------------------------------------------
 * Fused linear: y = act(x · Wᵀ + bias), fp32 accumulation on tcgen05 tensor cores.
 * Replaces: src/kernl/implementations/linear_layer.py:213-282 (LinearLayer.forward launching
 * kernel_fma, :91-210). W is [N,K] contiguous (linear_layer.py:244); x is [M,K] with unit K
 * stride and a row stride that is a multiple of 8 elements; K must be a multiple of 8.
 * act_inputs (optional, [M,N], row stride = y_row_stride) receives the pre-activation values
 * (linear_layer.py:193-195).
 * workspace: when the problem has fewer output tiles than SMs (few rows), K is split across work
 * items that accumulate fp32 partial sums into `workspace`. The workspace must be ALL ZERO before
 * the first call that uses it and is left all zero by every call (kb_linear_workspace_bytes gives
 * the size a problem needs); without a workspace, or with one that is too small, the same result
 * is computed unsplit. The reference fixes SPLIT_K = 1 (linear_layer.py:121-122).
 * ------------------------------------------------------------------------------------- */
typedef struct {
    const void* x;          /* [M,K]                                                       */
    const void* w;          /* [N,K] contiguous                                            */
    const void* bias;       /* [N] or NULL                                                 */
    void*       y;          /* [M,N]; [M,N/2] with KB_ACT_SWIGLU                           */
    void*       act_inputs; /* [M,N] or NULL                                               */
    int64_t     M, N, K;
    int64_t     x_row_stride;
    int64_t     y_row_stride;
    int32_t     activation; /* KB_ACT_*                                                    */
    int32_t     dtype;      /* KB_F16 / KB_BF16                                            */
    void*       workspace;  /* optional scratch for split-K, 16-byte aligned, or NULL      */
    int64_t     workspace_bytes; /* split-K needs >= kb_linear_workspace_bytes(M, N)       */
} kb_linear_params;

int kb_linear_fwd(const kb_linear_params* p, void* stream);
int64_t kb_linear_workspace_bytes(int64_t M, int64_t N);

/* Gated linear unit for SwiGLU feed-forward blocks: y[m,n] = silu(g[m,n]) * u[m,n], where
 * gu = [M, 2*N] holds g in columns [0,N) and u in columns [N,2N). No counterpart in the
 * reference's dispatched path; semantics follow experimental/llama-v2/kernel/fused_kernel_ff.py:10-114. */
int kb_silu_mul(const void* gu, void* y, int64_t M, int64_t N, int32_t dtype, void* stream);

/* Rotary embedding fused with the KV-cache write (Llama-shaped decoder). qkv is the fused
 * projection output [B*S, 3, H, D]; q (rotated) goes to q_out [B, S, H, D]; rotated k and v go to
 * k_cache / v_cache [B, H, max_seq, D] at positions start .. start+S-1, where start is read from
 * pos_dev (device int64) when it is not NULL, else pos_host. cos/sin: fp32 [max_seq, D/2].
 * Rotation on interleaved pairs as in the reference's experimental Llama kernels
 * (experimental/llama-v2/kernel/pytorch_reference.py:37-80, fused_kernel_proj_qkv.py:116-347);
 * nothing in the reference's dispatched path corresponds to it. D must be a multiple of 8. */
typedef struct {
    const void* qkv; void* q_out; void* k_cache; void* v_cache;
    const float* cos; const float* sin;
    const int64_t* pos_dev; int64_t pos_host;
    int64_t B, S, H, D, max_seq;
    int32_t dtype;
} kb_rope_params;

int kb_rope_kv_write(const kb_rope_params* p, void* stream);

/* ---------------------------------------------------------------------------------------
 * Fused attention forward: O = softmax(sm_scale · Q·Kᵀ + mask [causal]) · V, online softmax.
 * Replaces: src/kernl/implementations/attention.py:438-529 (Attention.forward launching
 * _fwd_kernel, :122-435).
 *   q [B,H,M,D], k/v [B,H,N,D] ([B,H/kv_group,N,D] with grouped queries), o [B,H,M,D]; D a multiple
 *   of 8 up to 128 (the reference takes the powers of two from 16, attention.py:521; the kernels
 *   compute on 64 or 128 columns and TMA fills the missing ones with zeros);
 *   unit D stride required for q,k,v,o;
 *   the other q/k/v strides must be multiples of 8 elements.
 *   mask: additive, logical shape [B|1, H|1, M|1, N]; a broadcast dimension is passed with
 *   stride 0. -inf entries are clamped to the lowest finite value of mask_dtype
 *   (attention.py:380,516). is_causal keeps col <= row, top-left aligned (attention.py:347).
 * ------------------------------------------------------------------------------------- */
typedef struct {
    const void* q; const void* k; const void* v; void* o;
    const void* mask;        /* or NULL                                                    */
    int64_t B, H, M, N, D;
    int64_t q_strides[4];    /* batch, head, row, dim                                      */
    int64_t k_strides[4];
    int64_t v_strides[4];
    int64_t o_strides[4];
    int64_t mask_strides[4]; /* batch, head, row, col ; 0 = broadcast                       */
    float   sm_scale;
    int32_t is_causal;
    int32_t dtype;           /* KB_F16 / KB_BF16 for q,k,v,o                               */
    int32_t mask_dtype;      /* KB_F16 / KB_BF16 / KB_F32                                  */
    /* Grouped-query attention: kv_group consecutive query heads share one K/V head, i.e. query
     * head h reads K/V head h / kv_group, k and v are [B, H / kv_group, N, D] and H % kv_group == 0.
     * 0 or 1 = one K/V head per query head (the reference's only case). Replaces the eager
     * `repeat_kv` copy that grouped-query models otherwise make before attention. */
    int32_t kv_group;
    /* Decode entry points only (NULL elsewhere): device int64 holding how many of the N keys exist
     * (a KV cache filled up to that slot); keys beyond it are neither loaded nor scored. The value
     * is read by the kernel, so a captured CUDA graph follows a growing cache. It plays the part
     * of `start_position` in the reference's experimental Llama attention
     * (experimental/llama-v2/kernel/fused_kernel_attention.py:30,63,76). Values above N count as N. */
    const int64_t* kv_len_dev;
} kb_attn_params;

int kb_attention_fwd(const kb_attn_params* p, void* stream);

/* Decode-shape ("skinny") attention: few query rows, many keys; the keys are split into
 * chunks handled by different CTAs and merged with the online-softmax recurrence.
 * Replaces: src/kernl/implementations/attention_skinny.py:369-536 (SkinnyAttention.forward
 * launching _fwd_part_1 :58-272 and _fwd_part_2 :275-366). Same tensor conventions as
 * kb_attention_fwd but arbitrary strides. `scratch` must hold kb_attention_decode_scratch_bytes()
 * bytes; it needs no initialisation. */
int64_t kb_attention_decode_scratch_bytes(int64_t B, int64_t H, int64_t M, int64_t N, int64_t D);
int kb_attention_decode_fwd(const kb_attn_params* p, void* scratch, int64_t scratch_bytes, void* stream);

/* ---------------------------------------------------------------------------------------
 * All-reduce (sum over ranks) fused with a residual add, over NVLink peer memory:
 *   out = residual + sum_r partials[r]        (fp32 accumulation, rank order, 16-bit in/out)
 * for the row-parallel linears of a tensor-parallel decoder. The reference has no multi-GPU path at
 * all (single process, single GPU), so this entry point has no counterpart there.
 *   partials[r]  rank r's partial-sum buffer as mapped into THIS process (partials[rank] is local);
 *                each rank's GEMM writes its partial there before the call
 *   flags[r]     rank r's flag block (>= 32 uint32, peer-mapped, zeroed once at set-up)
 * Every rank of the group must make the same sequence of calls. One-shot algorithm (each rank reads
 * every peer's buffer): meant for latency-bound messages; count*2 bytes <= 1 MiB is enforced.
 * The call returns only after every peer has finished reading this rank's partial, so the buffer
 * may be overwritten right away. All device-side waits are bounded (status word on expiry).
 * ------------------------------------------------------------------------------------- */
#define KB_ALLREDUCE_MAX_WORLD 8
#define KB_ALLREDUCE_MAX_BYTES (1 << 20)
typedef struct {
    const void* partials[KB_ALLREDUCE_MAX_WORLD];
    uint32_t*   flags[KB_ALLREDUCE_MAX_WORLD];
    const void* residual;   /* [count] local, or NULL                                      */
    void*       out;        /* [count] local                                               */
    int64_t     count;      /* elements, multiple of 8                                     */
    int32_t     rank, world;
    int32_t     dtype;      /* KB_F16 / KB_BF16                                            */
    /* Optional fused RMSNorm of the reduced rows (the norm that opens the next decoder block): when
     * norm_weight != NULL, count is rows x cols, cols % 8 == 0, cols <= 8192, and
     * norm_out[r, :] = out[r, :] * rsqrt(mean(out[r, :]^2) + eps) * norm_weight, computed from the
     * 16-bit values stored in out. */
    const void* norm_weight; /* [cols]                                                     */
    void*       norm_out;    /* [count], local                                             */
    int64_t     cols;
    float       eps;
} kb_allreduce_params;

int kb_allreduce_residual_fwd(const kb_allreduce_params* p, void* stream);

/* Set-up helpers for the peer-mapped buffers above (the only entry points of this library that
 * allocate; they synchronise and are meant to be called once, outside any stream capture):
 * the owner allocates (zero-filled) and exports a 64-byte CUDA IPC handle, every other process of
 * the node opens it and receives a pointer valid in its own address space. No NVLS / multicast
 * object is involved. */
int kb_peer_alloc(int64_t bytes, void** out);
int kb_peer_free(void* p);
int kb_peer_export(void* p, void* handle64);
int kb_peer_open(const void* handle64, void** out);
int kb_peer_close(void* p);

/* Decode attention for callers that cannot allocate device memory. Same computation and arguments
 * as kb_attention_decode_fwd, but the scratch is a fixed array inside the library (4 MiB of device
 * memory on every GPU that loads the library, held until the process exits), so the caller passes
 * only its inputs and its output. This entry point has no counterpart in the reference; it exists
 * for hosts that own no device allocator — e.g. a custom-op hook of a serving runtime that hands a
 * plugin nothing but tensors, or a process whose memory another framework's pool has already
 * reserved — and it calls no cudaMalloc/cudaFree nor any allocating library routine.
 *   - Limit: kb_attention_decode_scratch_bytes(B,H,M,N,D) must not exceed
 *     kb_attention_decode_static_max_bytes(); larger problems return KB_ERR_TOO_LARGE and launch
 *     nothing (use kb_attention_decode_fwd with your own scratch instead).
 *   - The first call on each device looks up the array's device address (the device must be
 *     current); make that first call before starting any stream capture.
 *   - All calls share the one array: calls that can overlap on the GPU (different streams,
 *     different threads) race on it and must be serialised by the caller. Contents left by an
 *     earlier call are harmless: every slot that is read has been rewritten by the same call. */
int64_t kb_attention_decode_static_max_bytes(void);
int kb_attention_decode_fwd_static(const kb_attn_params* p, void* stream);

/* ---- device status word ---------------------------------------------------------------
 * Kernels with bounded waits record a non-zero code here instead of trapping or hanging.
 * kb_device_status_read synchronises the current device, returns the word and clears it. */
int kb_device_status_read(int32_t* status_out);

/* ---- SMs for the persistent GEMM kernels ------------------------------------------------
 * The fused-linear kernels for large problems are persistent: one CTA (or CTA pair) per SM for the
 * whole launch, so a collective that should run AT THE SAME TIME (the all-reduce of one half of a
 * batch while the other half computes) finds no SM until the GEMM ends. kb_gemm_sm_limit(n) makes
 * later launches use at most n SMs (0 = all, the default); the setting is process-wide and read
 * when a launch is enqueued. Nothing in the reference corresponds to it (it has no multi-GPU path). */
int kb_gemm_sm_limit(int sms);

const char* kb_status_str(int status);
int kb_version(void);

#ifdef __cplusplus
}
#endif
#endif /* KERNL_B200_H */
