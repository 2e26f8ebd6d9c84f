// Work decomposition shared by the paged decode kernels.
//
// A "tile" is TT consecutive tokens of one sequence for one group of HPC kv heads.  Tiles
// are numbered sequence by sequence, head group by head group:
//     first(b, hg) = NG * tiles_before(b) + hg * tiles(b),   NG = n_kv_heads / HPC.
// CTA c of a grid of `grid` CTAs owns the tile range [c * chunk, (c + 1) * chunk) with
// chunk = ceil(total / grid), so every CTA streams the same number of KV bytes whatever
// the mix of context lengths.  Not quite the same number: beginning and finishing a (sequence,
// head group) - query rows and length to fetch, the warps' merge, the output row or the partial
// and its ticket - costs a CTA about as much time as `seg_overhead` tiles (measured: CTAs with 12
// segments in their range finished 20 us after CTAs with 3), so every (b, hg) is given that many
// tiles of nothing in front of its real ones, and it is this padded numbering that is cut into
// equal ranges.  A range that only holds padding of a (b, hg) has nothing to do for it.  A range is cut into segments at (sequence, head group)
// boundaries.  A segment that covers its whole (b, hg) writes the output row directly;
// otherwise it leaves an un-normalised partial (running max, sum, accumulator) in one of
// the CTA's two scratch slots: slot 0 when the segment continues a (b, hg) begun by an
// earlier CTA, slot 1 when it begins one that a later CTA continues.  Every CTA that leaves
// a partial then takes a ticket from the counter of that (b, hg) (indexed by the first CTA
// of its span); the CTA that draws the last ticket merges slot 1 of the first CTA with slot
// 0 of the following ones and writes the output rows.  No CTA waits for another.
#pragma once

#include "common.cuh"

namespace ib {

constexpr int kStatusMagic = 0x5AFE0000;   // status word == magic | code after a bounded wait ran out
constexpr int kMaxDecodeGrid = 1024;       // ticket counters in the scratch header

struct DecodeParams {
    const __nv_bfloat16* q;
    __nv_bfloat16* out;
    const int32_t* context_lens;
    const int32_t* block_tables;
    int64_t bt_stride;
    const void* k_cache;
    const void* v_cache;
    const float* k_scale;
    const float* v_scale;
    int batch;
    int n_q_heads;
    int n_kv_heads;
    int group;        // query heads per kv head
    int block_size;
    int num_blocks;
    float scale_log2; // softmax_scale * log2(e)
    uint32_t wait_limit;   // polls before a barrier wait gives up
    int stall_producer;    // self-test only: the producer arms no copy, so every wait runs out
    int seg_overhead;      // what starting and finishing a (sequence, head group) costs a CTA, in tiles (see below)
    // fused append (bf16 pools): the step's new rows [batch][n_kv_heads][128], row b going to position
    // context_lens[b] - 1 of sequence b; null = the pools already hold them
    const __nv_bfloat16* new_k;
    const __nv_bfloat16* new_v;
    int64_t new_k_stride, new_v_stride;   // elements between the rows of consecutive sequences
    // scratch
    int* status;      // one word
    int* counters;    // [kMaxDecodeGrid] tickets, zero between launches
    float* ws_ml;     // [grid * 2][rows][2]
    float* ws_o;      // [grid * 2][rows][128]
};

// Scratch layout: 64-byte header (status word), ticket counters, partial maxima/sums, partial
// accumulators.  Everything up to ml_off must be zero when a launch starts; a launch that ends
// normally leaves it zero.
struct DecodeLayout {
    size_t status_off, counters_off, ml_off, o_off, total;
};

inline DecodeLayout decode_layout(int grid, int rows) {
    DecodeLayout l;
    l.status_off = 0;
    l.counters_off = 64;
    l.ml_off = (l.counters_off + size_t(kMaxDecodeGrid) * 4 + 255) / 256 * 256;
    l.o_off = (l.ml_off + size_t(grid) * 2 * rows * 2 * 4 + 255) / 256 * 256;
    l.total = l.o_off + size_t(grid) * 2 * rows * kHeadDim * 4;
    return l;
}

#ifdef __CUDACC__

// Exclusive prefix of tiles per sequence into shared memory (s_tp[batch] = total).
// Every thread of the CTA must call it (blockDim.x a multiple of 32, at most 1024); ends with
// a __syncthreads().  Warp-shuffle scan, then the warp totals through shared memory.
// With s_rem (one byte per sequence, optional) it also records how many tokens the sequence's last tile holds
// (context_len mod tile_tokens; 0 = a full tile), for a producer that copies only the rows that exist.
__device__ inline void build_tile_prefix(const int32_t* __restrict__ context_lens, int batch, int tile_tokens,
                                         int* s_tp, int* s_scratch /* 32 ints */, uint8_t* s_rem = nullptr,
                                         int seg_overhead = 0) {
    const int nt = blockDim.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int per = (batch + nt - 1) / nt;
    const int lo = min(batch, tid * per), hi = min(batch, lo + per);
    int sum = 0;
    // tiles of a sequence in the padded numbering (per head group); an empty sequence has none
    auto padded = [&](int len) { return len > 0 ? (len + tile_tokens - 1) / tile_tokens + seg_overhead : 0; };
    for (int i = lo; i < hi; ++i) sum += padded(context_lens[i]);
    int incl = sum;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += v;
    }
    if (lane == 31) s_scratch[warp] = incl;
    __syncthreads();
    int run = incl - sum;
    for (int w = 0; w < warp; ++w) run += s_scratch[w];
    for (int i = lo; i < hi; ++i) {
        s_tp[i] = run;
        const int n = max(context_lens[i], 0);
        run += padded(n);
        if (s_rem != nullptr) s_rem[i] = uint8_t(n % tile_tokens);
    }
    if (tid == nt - 1) s_tp[batch] = run;
    __syncthreads();
}

struct Segment {
    int b, hg, t0, t1, ntiles;   // real tiles [t0, t1) of the (b, hg)'s ntiles; t0 == t1: only padding lies in the range
    int span;                    // how far the segment reaches in the padded numbering
};

// Segment of the (b, hg) that contains tile g of the padded numbering, cut at `hi`.
__device__ __forceinline__ Segment locate_segment(const int* s_tp, int batch, int ng, int g, int hi, int seg_overhead) {
    // last b with ng * s_tp[b] <= g  (skips empty sequences, whose prefix equals the next one's)
    int lo_b = 0, hi_b = batch;   // invariant: ng*s_tp[lo_b] <= g < ng*s_tp[hi_b]
    while (hi_b - lo_b > 1) {
        const int mid = (lo_b + hi_b) >> 1;
        if (ng * s_tp[mid] <= g) lo_b = mid; else hi_b = mid;
    }
    Segment s;
    s.b = lo_b;
    const int padded = s_tp[lo_b + 1] - s_tp[lo_b];
    const int rel = g - ng * s_tp[lo_b];
    s.hg = rel / padded;
    const int v0 = rel - s.hg * padded, v1 = min(padded, v0 + (hi - g));
    s.span = v1 - v0;
    s.ntiles = padded - seg_overhead;
    s.t0 = max(v0 - seg_overhead, 0);
    s.t1 = max(v1 - seg_overhead, 0);
    return s;
}

#endif  // __CUDACC__

}  // namespace ib
