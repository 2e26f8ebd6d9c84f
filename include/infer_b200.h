/*
 * infer_b200.h - C ABI of libinfer_b200.so, the sm_100a paged KV-cache path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (cudaStream_t passed as void*; NULL = the legacy default stream).  No entry point
 * allocates, frees or synchronises: outputs, pools and scratch memory belong to the
 * caller, which makes each call capturable in a CUDA graph with static buffers, the
 * scheme the reference engine uses for decode (infer/engine/model_runner.py:135-198).
 * All functions return 0 on success and a negative INFER_ERR_* code otherwise;
 * no C++ exception crosses this boundary.
 *
 * Layouts (bit-identical to the reference engine's, infer/engine/model_runner.py:47-126):
 *   pools          [num_blocks, block_size, n_kv_heads, 128], contiguous, bf16 or e4m3 bytes
 *   scales (e4m3)  fp32 [num_blocks, n_kv_heads], one per (page, kv head)
 *   slot_mapping   int32 [n_tokens], flat slot = page * block_size + offset; < 0 = skip row
 *   block_tables   int32 [batch, bt_stride], page ids, rows padded with -1 (never read
 *                  beyond ceil(context_len / block_size))
 *   context_lens   int32 [batch], keys per sequence INCLUDING the token appended this step;
 *                  0 = the row is skipped and its output left untouched
 *   cu_seqlens_*   int32 [batch + 1]
 */
#ifndef INFER_B200_H
#define INFER_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define INFER_API __attribute__((visibility("default")))
#else
#define INFER_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum {
    INFER_OK = 0,
    INFER_ERR_NULL = -1,       /* a required pointer is NULL */
    INFER_ERR_ALIGN = -2,      /* a pointer or stride is not 16-byte aligned */
    INFER_ERR_STRIDE = -3,     /* a row stride is smaller than the row */
    INFER_ERR_GEOMETRY = -4,   /* unsupported shape: head_dim != 128, block_size % 256 != 0,
                                  n_q_heads % n_kv_heads != 0, group > 8, batch > 2048 ... */
    INFER_ERR_WORKSPACE = -5,  /* scratch buffer missing, misaligned or too small */
    INFER_ERR_CUDA = -6,       /* a CUDA call failed; see infer_last_cuda_error() */
    INFER_ERR_DTYPE = -7,      /* pool dtype not valid for this entry point */
    INFER_ERR_DEVICE = -8,     /* the kernel reported a bounded wait that ran out */
    INFER_ERR_TOO_LARGE = -9   /* the problem needs more than the built-in scratch of
                                  infer_paged_decode_noalloc */
};

enum { INFER_KV_BF16 = 0, INFER_KV_E4M3 = 1 };

/* Opaque pool handle: geometry + the TMA descriptors of the K and V pools.  It owns no
 * device memory.  Replaces the per-layer cache views the reference hands to its
 * attention modules (infer/engine/model_runner.py:58-64) and backs the KVCachePool class
 * (include/kvcache.hpp:32-97). */
typedef struct infer_kv_pool infer_kv_pool_t;

INFER_API int infer_kv_pool_create(infer_kv_pool_t** pool, void* k_cache, void* v_cache,
                         float* k_scale, float* v_scale, int64_t num_blocks, int block_size,
                         int n_kv_heads, int head_dim, int dtype);
INFER_API int infer_kv_pool_destroy(infer_kv_pool_t* pool);

/* KV append.  Replaces store_kvcache / store_kvcache_kernel (infer/ops/attention.py:16-45):
 * row i of k and v ([n_tokens, n_kv_heads, 128] bf16, row pitch k_row_stride / v_row_stride
 * ELEMENTS, so column slices of a fused qkv output are accepted as the reference accepts
 * them) goes to flat slot slot_mapping[i].  An e4m3 pool quantises on write with one scale
 * per (page, kv head) and needs infer_kv_append_workspace_bytes() of scratch. */
INFER_API int infer_kv_append(const infer_kv_pool_t* pool, const void* k, const void* v,
                    int64_t k_row_stride, int64_t v_row_stride, const int32_t* slot_mapping,
                    int64_t n_tokens, void* workspace, size_t workspace_bytes, void* stream);
INFER_API size_t infer_kv_append_workspace_bytes(const infer_kv_pool_t* pool);

/* Fused per-head RMSNorm + rotary embedding + KV append: one pass over the fused qkv rows
 * instead of the four the reference model makes before attention (q_norm and k_norm,
 * infer/models/Qwen3.py:116-121 with infer/ops/norm.py:63-73; the in-place rotary embedding of
 * q and k, infer/models/Qwen3.py:127 with src/operators/rope/rope.cu:109-133, GPT-NeoX
 * pairing, rot_dim = 128; store_kvcache, infer/ops/attention.py:109).  q, k, v: bf16
 * [n_tokens, heads, 128] with free row strides (ELEMENTS); q_out bf16 [n_tokens, n_q_heads, 128]
 * (may be q itself); weights bf16 [128]; positions int64 [n_tokens]; cos_sin_cache bf16
 * [max_position, 128] = 64 cosines then 64 sines per position, as the reference builds it
 * (infer/ops/rope.py:108-115).  k is written normalised and rotated to its slot, v is copied;
 * bf16 pools only.  Rounding follows the reference step by step (fp32 variance and scaling,
 * bf16 before the weight multiply, bf16 products and sum in the rotation). */
INFER_API int infer_qk_norm_rope_append(const infer_kv_pool_t* pool, void* q_out, int64_t q_out_row_stride,
                              const void* q, const void* k, const void* v, int64_t q_row_stride,
                              int64_t k_row_stride, int64_t v_row_stride, const void* q_norm_weight,
                              const void* k_norm_weight, float eps, const int64_t* positions,
                              const void* cos_sin_cache, int64_t max_position,
                              const int32_t* slot_mapping, int64_t n_tokens, int n_q_heads, void* stream);

/* Advances the decode-step metadata on the device: every row with context_lens[b] > 0 grows by
 * one token, slot_mapping[b] becomes the slot of that token (read off block_tables, -1 if the
 * page is missing), positions[b] (optional) its position + position_base; rows with
 * context_lens[b] <= 0 get slot -1.  Replaces the per-step host loops and uploads of
 * ModelRunner.prepare_decode (infer/engine/model_runner.py:110-126), whose position value is
 * len(seq), i.e. position_base = 1. */
INFER_API int infer_decode_step_advance(int32_t* context_lens, int32_t* slot_mapping, int64_t* positions,
                              const int32_t* block_tables, int64_t bt_stride, int batch,
                              int block_size, int position_base, void* stream);

/* Paged decode attention.  Replaces the decode branch of Attention.forward
 * (flash_attn_with_kvcache(q[:,None], k_cache, v_cache, cache_seqlens, block_table,
 * softmax_scale, causal=True), infer/ops/attention.py:117-121) and fills the empty
 * flash_attn_decode stub (src/operators/flashattn/flashattn_decode.cu:1-13).
 * q, out: bf16 [batch, n_q_heads, 128] contiguous. */
INFER_API int infer_paged_decode(const infer_kv_pool_t* pool, void* out, const void* q,
                       const int32_t* context_lens, const int32_t* block_tables,
                       int64_t bt_stride, int batch, int n_q_heads, float softmax_scale,
                       void* workspace, size_t workspace_bytes, void* stream);
INFER_API size_t infer_paged_decode_workspace_bytes(const infer_kv_pool_t* pool, int batch, int n_q_heads);

/* Paged chunked-prefill attention.  Replaces the prefill branch
 * (flash_attn_varlen_func(q, k_cache, v_cache, cu_seqlens_q/k, max_seqlen_q/k,
 * softmax_scale, causal=True, block_table), infer/ops/attention.py:110-116).  Keys of
 * sequence b are its first cu_seqlens_k[b+1]-cu_seqlens_k[b] cached tokens (append the
 * chunk first); the causal mask is aligned to the bottom-right corner.
 * q, out: bf16 [total_q, n_q_heads, 128] contiguous; total_q = cu_seqlens_q[batch]. */
INFER_API int infer_paged_prefill(const infer_kv_pool_t* pool, void* out, const void* q, int64_t total_q,
                        const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                        const int32_t* block_tables, int64_t bt_stride, int batch,
                        int max_seqlen_q, int max_seqlen_k, int n_q_heads,
                        float softmax_scale, void* stream);

/* Dense causal attention.  Replaces flash_attn_prefill_impl
 * (src/operators/flashattn/flashattn.cu:269-328; schema src/bindings.cpp:9):
 * Q, O bf16 [B, Hq, S, 128], K, V bf16 [B, Hkv, S, 128], scale 1/sqrt(128) computed
 * inside, GQA by kv_head = head / (Hq/Hkv). */
INFER_API int infer_flash_attn_prefill(const void* q, const void* k, const void* v, void* o,
                             int batch, int n_q_heads, int n_kv_heads, int seq_len, void* stream);

/* Paged decode attention for callers that cannot provide scratch memory.  It has no
 * counterpart in the reference.  Same arguments and results as infer_paged_decode, minus the
 * workspace: the partial results of contexts that are split over several thread blocks go to
 * a 2 MiB array that is part of the library image on the device (every GPU that loads the
 * library holds those 2 MiB until the process exits).
 *
 * It is meant for two kinds of caller: an engine that has already handed every free byte of
 * device memory to the KV pools - the reference sizes its pool from whatever is left after
 * warm-up (infer/engine/model_runner.py:47-58), so a later cudaMalloc for scratch may fail -
 * and a host runtime that binds this C ABI through a thin shim (cgo, JNI, ctypes) and only
 * ever holds device pointers it was lent, with no device allocator of its own.
 *
 * The function calls no cudaMalloc/cudaFree and no allocating library routine.  The first
 * call on a device looks up the device address of the built-in array (the device must be
 * current, and must be the one the pool was created on); make that first call before any
 * stream capture.  Every call on a device shares the one array, which keeps the previous
 * call's contents; the function clears the status word that must start at zero, everything
 * else is rewritten before it is read.  Two calls that overlap on the GPU (different
 * streams, or concurrent graphs) race on the array: serialise them.
 *
 * Limits: the scratch layout for the pool's geometry and this GPU must fit 2 MiB (up to 8 query
 * heads per KV head, GPUs of up to about 240 SMs) and batch <= 2048; anything
 * larger returns INFER_ERR_TOO_LARGE without launching. */
INFER_API int infer_paged_decode_noalloc(const infer_kv_pool_t* pool, void* out, const void* q,
                               const int32_t* context_lens, const int32_t* block_tables,
                               int64_t bt_stride, int batch, int n_q_heads, float softmax_scale,
                               void* stream);

/* Reads (and clears) the status word of the prefill kernels on the current device
 * (synchronises the stream): INFER_ERR_DEVICE if a bounded wait inside infer_paged_prefill or
 * infer_flash_attn_prefill ran out since the last call, INFER_OK otherwise.  The word lives in
 * the library's device image; the first prefill call on a device looks its address up, so make
 * that call before any stream capture.  A debugging read, like infer_paged_decode_status. */
INFER_API int infer_prefill_status(void* stream);

/* Reads the device status word the last decode call on this workspace left behind
 * (synchronises the stream).  0 = no bounded wait ran out. */
INFER_API int infer_paged_decode_status(const void* workspace, void* stream);

INFER_API const char* infer_strerror(int code);
INFER_API int infer_last_cuda_error(void);
INFER_API int infer_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* INFER_B200_H */
