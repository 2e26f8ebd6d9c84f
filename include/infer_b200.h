/*
 * infer_b200.h - C ABI of libinfer_b200.so, the sm_100a paged KV-cache path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (cudaStream_t passed as void*; NULL = the legacy default stream).  No entry point
 * allocates or frees device memory: outputs, pools and scratch memory belong to the
 * caller.  The per-step entry points of decode - infer_kv_append,
 * infer_qk_norm_rope_append, infer_decode_step_advance, infer_paged_decode - make no
 * CUDA call but kernel launches on the given stream (plus one memset node in
 * infer_paged_decode_noalloc) and read no device data on the host, so they
 * can be captured in a CUDA graph with static buffers, the scheme the reference engine
 * uses for decode (infer/engine/model_runner.py:135-198).  The prefill entry points
 * encode a tensor map for q on the host in every call (the address of q is baked into the
 * launch) and are meant for eager launches, which is how the reference runs prefill
 * (infer/engine/model_runner.py:128-134); a captured prefill is only valid for the q
 * address it was captured with.  The two *_status functions synchronise the stream.
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
    INFER_ERR_TOO_LARGE = -9,  /* the problem needs more than the built-in scratch of
                                  infer_paged_decode_noalloc */
    INFER_ERR_STATE = -10      /* page allocator: out of pages, unknown or duplicate sequence id,
                                  or a call out of order; see infer_block_manager_last_error() */
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
 * per (page, kv head) and needs infer_kv_append_workspace_bytes() of 16-byte aligned scratch
 * that belongs to THIS pool: the caller zero-fills it once before its first use, every call
 * leaves it in the state the next call on the same pool expects, and it must be zero-filled
 * again before it serves a pool of another geometry.  Appends to one pool that share the
 * scratch must not overlap on the GPU.  bf16 pools need no scratch (NULL, 0). */
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
 * q, out: bf16 [batch, n_q_heads, 128] contiguous.  Any n_q_heads that is a multiple of the
 * pool's kv heads with at most 8 query heads per kv head (group sizes 1..8, e.g. 40 over 8).
 * q and out may also be pinned host memory given by its device-valid address (with unified addressing the
 * pointer itself): the kernel then reads the queries and writes the output rows over PCIe, which saves a
 * host-fed caller two copies.  The same holds for q, k, v and out of infer_paged_decode_append.
 * workspace: infer_paged_decode_workspace_bytes() of 16-byte aligned device memory that the
 * caller zero-fills ONCE before its first use; a call leaves the part that has to be zero
 * (a status word and the ticket counters of contexts split over thread blocks) at zero
 * again.  Calls that share a workspace must not overlap on the GPU (one stream, or one
 * graph): give every stream that runs decode its own. */
INFER_API int infer_paged_decode(const infer_kv_pool_t* pool, void* out, const void* q,
                       const int32_t* context_lens, const int32_t* block_tables,
                       int64_t bt_stride, int batch, int n_q_heads, float softmax_scale,
                       void* workspace, size_t workspace_bytes, void* stream);

/* One decode step in one launch, bf16 pools: infer_kv_append of the step's new rows followed by
 * infer_paged_decode.  Replaces the two calls the reference makes per layer and decode step,
 * store_kvcache(k, v, k_cache, v_cache, slot_mapping) and flash_attn_with_kvcache(...)
 * (infer/ops/attention.py:109 and :117-121; the decode batch is one row per sequence,
 * infer/engine/model_runner.py:110-126).
 * k, v: bf16 [batch, n_kv_heads, 128], heads contiguous, k_row_stride / v_row_stride elements between the rows
 * of consecutive sequences (column slices of a fused qkv output are fine); row b is the token at position
 * context_lens[b] - 1 of sequence b, whose slot is read off block_tables (no slot_mapping).  Rows of sequences
 * with context_lens[b] <= 0 or without a page for that position are not written.  The pools end up
 * byte for byte as after infer_kv_append, the output as after infer_paged_decode.  context_lens and
 * block_tables may be written by the kernel directly in front of this call in the stream.
 * INFER_ERR_DTYPE for an e4m3 pool (append and decode stay two calls there).  Workspace, stream and
 * capture rules as for infer_paged_decode. */
INFER_API int infer_paged_decode_append(const infer_kv_pool_t* pool, void* out, const void* q, const void* k,
                              const void* v, int64_t k_row_stride, int64_t v_row_stride,
                              const int32_t* context_lens, const int32_t* block_tables, int64_t bt_stride,
                              int batch, int n_q_heads, float softmax_scale, void* workspace,
                              size_t workspace_bytes, void* stream);
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
 * call's contents; the function clears what must start at zero (the status word and the
 * ticket counters, one memset), everything else is rewritten before it is read.  A bounded
 * wait that ran out is reported by infer_paged_decode_status(NULL, stream).  Two calls that overlap on the GPU (different
 * streams, or concurrent graphs) race on the array: serialise them.
 *
 * Limits: the scratch layout for the pool's geometry and this GPU must fit 2 MiB - a 4352-byte
 * header plus 2080 bytes per (thread block = SM, partial row), where a tile carries
 * (kv heads per tile) x (query heads per kv head) partial rows.  On 148 SMs that is up to 13
 * rows: every bf16 pool fits (one kv head per tile, at most 8 rows; GPUs of up to 250 SMs),
 * and an e4m3 pool fits by taking fewer kv heads per tile than its default.  batch <= 2048.
 * Anything larger returns INFER_ERR_TOO_LARGE without launching. */
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

/* Reads the device status word the decode calls on this workspace left behind (synchronises
 * the stream): INFER_OK = no bounded wait ran out; INFER_ERR_DEVICE = one did since the last
 * read, the outputs of that call are undefined, and the word and the ticket counters have
 * been cleared so that the workspace can be used again.  workspace == NULL reads the
 * built-in array of infer_paged_decode_noalloc on the current device. */
INFER_API int infer_paged_decode_status(const void* workspace, void* stream);

/* Page allocator with prefix sharing (host-only).  Replaces BlockManager / Block and the page
 * arithmetic of Sequence (infer/engine/block_mannager.py:26-133, infer/engine/sequence.py:15-84):
 * pages leave the front of a FIFO free list; a full page is keyed by the XXH64 digest of the
 * previous page's digest and its token ids; a prompt whose leading pages carry known digests
 * and the same token ids shares those pages (reference counts); a page returns to the back of
 * the free list when its count reaches zero.  Same page ids as the reference for the same call
 * sequence.  Sequences live inside the manager under the caller's ids.
 *   allocate      whole-prompt allocation (BlockManager.allocate); returns the number of cached
 *                 (shared) tokens, or a negative error
 *   append        for every new token: Sequence.append_token, then BlockManager.may_append (a
 *                 new page when the token is the first of one, a digest when it fills one);
 *                 n_new == 0 runs may_append alone
 *   can_allocate / can_append   1 or 0 (negative on error), as the reference scheduler asks
 *                 (infer/engine/scheduler.py:27,44)
 *   deallocate    BlockManager.deallocate, used for finished and for preempted sequences
 *   block_table / free_ids / ref_counts   copy up to cap entries, return the full count
 *   set_free_order  replaces the order of the (entirely free) free list: workload generators
 *                 use it to scatter pages over the pool */
typedef struct infer_block_manager infer_block_manager_t;
INFER_API int infer_block_manager_create(infer_block_manager_t** mgr, int64_t num_blocks, int block_size);
INFER_API int infer_block_manager_destroy(infer_block_manager_t* mgr);
INFER_API int infer_block_manager_can_allocate(const infer_block_manager_t* mgr, int64_t n_tokens);
INFER_API int64_t infer_block_manager_allocate(infer_block_manager_t* mgr, int64_t seq_id, const int64_t* token_ids,
                                     int64_t n_tokens);
INFER_API int infer_block_manager_can_append(const infer_block_manager_t* mgr, int64_t seq_id);
INFER_API int infer_block_manager_append(infer_block_manager_t* mgr, int64_t seq_id, const int64_t* token_ids,
                               int64_t n_new);
INFER_API int infer_block_manager_deallocate(infer_block_manager_t* mgr, int64_t seq_id);
INFER_API int64_t infer_block_manager_block_table(const infer_block_manager_t* mgr, int64_t seq_id, int32_t* out,
                                        int64_t cap);
INFER_API int64_t infer_block_manager_num_tokens(const infer_block_manager_t* mgr, int64_t seq_id);
INFER_API int64_t infer_block_manager_num_free(const infer_block_manager_t* mgr);
INFER_API int64_t infer_block_manager_free_ids(const infer_block_manager_t* mgr, int32_t* out, int64_t cap);
INFER_API int64_t infer_block_manager_ref_counts(const infer_block_manager_t* mgr, int32_t* out, int64_t cap);
INFER_API int infer_block_manager_set_free_order(infer_block_manager_t* mgr, const int32_t* ids, int64_t n);
INFER_API const char* infer_block_manager_last_error(const infer_block_manager_t* mgr);

INFER_API const char* infer_strerror(int code);
INFER_API int infer_last_cuda_error(void);
INFER_API int infer_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* INFER_B200_H */
