/*
 * infer_b200_selftest.h - diagnostic entry points of libinfer_b200.so.
 *
 * Not part of the drop-in surface: nothing here replaces a reference interface.  The test
 * suite uses these calls to run the product kernels in every tile shape they support, to
 * run the cross-check prefill kernel, and to make a bounded device-side wait run out on
 * purpose (a producer that arms no copy) so that the error-reporting path is exercised
 * without faulting or hanging the GPU.  Arguments that also appear in infer_b200.h have the
 * same meaning there.
 */
#ifndef INFER_B200_SELFTEST_H
#define INFER_B200_SELFTEST_H

#include "infer_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* infer_paged_decode with the tile shape chosen by the caller.
 *   heads_per_tile  0 = the default; 1, 2, 4 or 8 kv heads per tile (must divide n_kv_heads)
 *   wait_limit      polls before a barrier wait gives up (0 = the default, about a second)
 *   stall_producer  non-zero: the producer warp arms no copy, so the first wait of every
 *                   consumer runs out after wait_limit polls; the kernel then sets the status
 *                   word that infer_paged_decode_status() reports as INFER_ERR_DEVICE.  The
 *                   output is undefined in that case. */
INFER_API int infer_selftest_paged_decode(const infer_kv_pool_t* pool, void* out, const void* q,
                                const int32_t* context_lens, const int32_t* block_tables,
                                int64_t bt_stride, int batch, int n_q_heads, float softmax_scale,
                                void* workspace, size_t workspace_bytes, void* stream,
                                int heads_per_tile, uint32_t wait_limit, int stall_producer);

/* infer_paged_prefill / infer_flash_attn_prefill on a chosen kernel.
 *   kernel          0 = the tcgen05 kernel (the product path); 1 = the mma.sync cross-check kernel
 *   wait_limit, stall_producer   as above (tcgen05 kernel only); the status is read with
 *                   infer_prefill_status(). */
INFER_API int infer_selftest_paged_prefill(const infer_kv_pool_t* pool, void* out, const void* q, int64_t total_q,
                                 const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                 const int32_t* block_tables, int64_t bt_stride, int batch,
                                 int max_seqlen_q, int max_seqlen_k, int n_q_heads, float softmax_scale,
                                 void* stream, int kernel, uint32_t wait_limit, int stall_producer);
INFER_API int infer_selftest_flash_attn_prefill(const void* q, const void* k, const void* v, void* o, int batch,
                                      int n_q_heads, int n_kv_heads, int seq_len, void* stream, int kernel);

#ifdef __cplusplus
}
#endif
#endif /* INFER_B200_SELFTEST_H */
