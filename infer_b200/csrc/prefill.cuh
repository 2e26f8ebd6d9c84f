// Shared declarations of the prefill kernels (paged chunked prefill and the dense op).
#pragma once

#include "common.cuh"

namespace ib {

struct PrefillParams {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    int64_t q_row_stride;     // elements between consecutive query rows
    int64_t q_head_stride;    // elements between query heads
    int64_t q_batch_stride;   // dense only: elements between batches
    const int32_t* cu_q;      // paged only
    const int32_t* cu_k;      // paged only
    const int32_t* block_tables;
    int64_t bt_stride;
    int n_q_heads;
    int n_kv_heads;
    int group;
    int block_size;
    int seq_len;              // dense only
    float scale_log2;
    int* status;              // may be null
    uint32_t wait_limit;      // polls before a barrier wait gives up
    int stall_producer;       // self-test only: the producer loads nothing, so every wait runs out
};

// mma.sync path (prefill_mma.cu): 64 query rows per CTA.
int launch_prefill_mma(bool paged, const PrefillParams& p, const CUtensorMap& mk, const CUtensorMap& mv, int max_q,
                       int batch, cudaStream_t st);
// tcgen05 path (prefill_tc.cu): 128 query rows per CTA, accumulators in tensor memory.
int launch_prefill_tc(bool paged, const PrefillParams& p, const CUtensorMap& mq, const CUtensorMap& mk,
                      const CUtensorMap& mv, int max_q, int batch, cudaStream_t st);

}  // namespace ib
