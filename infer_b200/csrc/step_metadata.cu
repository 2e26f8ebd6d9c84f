// Device-side decode-step metadata.
//
// The reference rebuilds context_lens, slot_mapping and positions for every decode step in
// Python loops and uploads them as separate pinned tensors (ModelRunner.prepare_decode,
// infer/engine/model_runner.py:110-126).  All three follow from the previous step: every live
// sequence grows by one token, and the slot of that token is read off the block table that is
// already on the device.  This kernel advances them in place, so a replayed decode graph
// needs no host data unless a sequence crosses into a new page (then the host writes that one
// block-table entry).
#include "common.cuh"

namespace ib {

__global__ void decode_step_advance_kernel(int32_t* __restrict__ context_lens, int32_t* __restrict__ slot_mapping,
                                           int64_t* __restrict__ positions, const int32_t* __restrict__ block_tables,
                                           int64_t bt_stride, int batch, int block_size, int position_base) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= batch) return;
    const int prev = context_lens[b];
    if (prev <= 0) {                 // padding row of a captured batch: stays empty, append skips it
        slot_mapping[b] = -1;
        if (positions) positions[b] = 0;
        return;
    }
    const int n = prev + 1;          // length including the token appended this step
    const int pos = n - 1;
    const int idx = pos / block_size;
    const int page = idx < bt_stride ? block_tables[int64_t(b) * bt_stride + idx] : -1;
    context_lens[b] = n;
    slot_mapping[b] = page >= 0 ? page * block_size + pos % block_size : -1;
    if (positions) positions[b] = int64_t(pos) + position_base;
}

}  // namespace ib

extern "C" int infer_decode_step_advance(int32_t* context_lens, int32_t* slot_mapping, int64_t* positions,
                                         const int32_t* block_tables, int64_t bt_stride, int batch, int block_size,
                                         int position_base, void* stream_) {
    if (!context_lens || !slot_mapping || !block_tables) return INFER_ERR_NULL;
    if (batch < 0 || bt_stride <= 0 || block_size <= 0) return INFER_ERR_GEOMETRY;
    if (batch == 0) return INFER_OK;
    ib::decode_step_advance_kernel<<<(batch + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream_)>>>(
        context_lens, slot_mapping, positions, block_tables, bt_stride, batch, block_size, position_base);
    return ib::check_launch();
}
