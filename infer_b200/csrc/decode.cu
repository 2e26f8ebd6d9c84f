// Paged decode attention (one query token per sequence) over the page pools.
//
//  * decode_tma_kernel   bf16 pools.  One persistent CTA per SM: a producer warp walks the
//    block tables and stages K/V tiles (128 (head, token) rows = 32 KiB of K + 32 KiB of V)
//    into a 3-stage shared-memory ring with TMA; eight consumer warps each own 16 tokens of
//    one kv head per tile, run q.K^T and P.V on mma.sync with the query-head group in the M
//    dimension, and keep the online-softmax state (max, sum, accumulator) in registers,
//    merging row statistics with quad shuffles.
//  * decode_tma_fp8_kernel   e4m3 pools: the same ring; K and V bytes go to the tensor cores
//    as f16, the page scales are folded into the softmax exponent and its correction factor.
//
// The work split (equal KV bytes per CTA, two scratch slots per CTA, the last CTA of a split
// sequence merging its partials) is described in decode_common.cuh.
#include <mutex>
#include <utility>

#include "decode_common.cuh"

namespace ib {

constexpr int kStages = 3;
constexpr int kTileBytes = 32768;                 // K (or V) bytes per stage: 128 rows x 256 B
constexpr int kConsumerWarps = 8;
constexpr int kTmaThreads = (kConsumerWarps + 1) * 32;
constexpr int kMergeSlotFloats = 36 * 32;         // 32 accumulators + up to two maxima and two sums per lane

// =========================================================================== merge of split (b, hg)
// Called by all 256 consumer threads of a CTA right after it left a partial for segment `sg`
// (uniformly: a segment is partial for every warp or for none).  The CTA draws a ticket from
// the counter of that (sequence, head group); the one that draws the last ticket finds every
// other partial already in memory, merges them and writes the output rows.  rows = HPC * group;
// row r belongs to query head hg * rows + r.
__device__ __forceinline__ void merge_if_last(const DecodeParams& p, const int* s_tp, int ng, const Segment& sg,
                                              int chunk, int rows, volatile int* s_flag) {
    // first real tile of the (b, hg) in the padded numbering; the CTAs c0..c1 hold its real tiles
    const int first = ng * s_tp[sg.b] + sg.hg * (sg.ntiles + p.seg_overhead) + p.seg_overhead;
    const int c0 = first / chunk, c1 = (first + sg.ntiles - 1) / chunk;
    asm volatile("bar.sync 1, 256;" ::: "memory");          // every partial store of this CTA is ordered before ...
    if (threadIdx.x == 0) {
        __threadfence();                                     // ... this fence, which is cumulative: they are visible before the ticket is
        const int ticket = atomicAdd(p.counters + c0, 1);
        const int last = ticket == c1 - c0;
        if (last) p.counters[c0] = 0;                        // all participants have drawn: ready for the next launch
        *s_flag = last;
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (!*s_flag) return;
    __threadfence();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = warp; r < rows; r += kConsumerWarps) {
        float mm = -INFINITY;
        for (int c = c0; c <= c1; ++c) {
            const int slot = c * 2 + (c == c0 ? 1 : 0);
            mm = fmaxf(mm, __ldcg(p.ws_ml + (int64_t(slot) * rows + r) * 2));
        }
        float ll = 0.f;
        float4 oo = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int c = c0; c <= c1; ++c) {
            const int slot = c * 2 + (c == c0 ? 1 : 0);
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.ws_ml + (int64_t(slot) * rows + r) * 2));
            const float a = ml.x == -INFINITY ? 0.f : exp2f(ml.x - mm);
            const float4 o = __ldcg(reinterpret_cast<const float4*>(p.ws_o + (int64_t(slot) * rows + r) * kHeadDim + lane * 4));
            ll += ml.y * a;
            oo.x += o.x * a; oo.y += o.y * a; oo.z += o.z * a; oo.w += o.w * a;
        }
        const float inv = 1.f / ll;
        uint2 packed;
        packed.x = pack_bf16(oo.x * inv, oo.y * inv);
        packed.y = pack_bf16(oo.z * inv, oo.w * inv);
        *reinterpret_cast<uint2*>(p.out + (int64_t(sg.b) * p.n_q_heads + sg.hg * rows + r) * kHeadDim + lane * 4) = packed;
    }
}

// =========================================================================== TMA kernel

struct TmaSmem {
    // dynamic shared memory, 1024-byte aligned base:
    //   [kStages][2][kTileBytes] tiles | merge slots | tile prefix | scan scratch | barriers
    static constexpr int tiles = kStages * 2 * kTileBytes;
    static constexpr int merge = tiles;
    static constexpr int prefix = merge + 4 * kMergeSlotFloats * 4;
    static constexpr int scan = prefix + (kMaxBatch + 1) * 4 + 12;
    static constexpr int bars = scan + kTmaThreads * 4;
    static constexpr int pages = bars + 2 * kStages * 8 + 16;      // page of the tile in each stage (fused append)
    static constexpr int patch = pages + 16;                        // 512 bytes per consumer warp: a new k row and v row
    static constexpr int rem = patch + kConsumerWarps * 512;        // tokens in every sequence's last tile, one byte each
    static constexpr int total = rem + kMaxBatch;
};

// Tensor maps with boxes of 16, 32, 64 and 128 token rows: the last tile of a sequence is copied with the smallest
// box that holds its tokens (the rows behind them belong to nobody, or to the future).
constexpr int kTailMaps = 4;
struct TailMaps {
    CUtensorMap k[kTailMaps];
    CUtensorMap v[kTailMaps];
};
static_assert(TmaSmem::patch % 16 == 0, "the staging rows are written by 16-byte asynchronous copies");

__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

template <int HPC>
__global__ void __launch_bounds__(kTmaThreads, 1) decode_tma_kernel(DecodeParams p,
                                                                    const __grid_constant__ CUtensorMap map_k,
                                                                    const __grid_constant__ CUtensorMap map_v,
                                                                    const __grid_constant__ TailMaps tails) {
    constexpr int TT = 128 / HPC;          // tokens per tile
    constexpr int WPH = kConsumerWarps / HPC;   // consumer warps per kv head
    constexpr int SUB = TT * 128;          // bytes of one (head, half) sub-tile
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* s_merge = reinterpret_cast<float*>(smem + TmaSmem::merge);
    int* s_tp = reinterpret_cast<int*>(smem + TmaSmem::prefix);
    int* s_scan = reinterpret_cast<int*>(smem + TmaSmem::scan);
    volatile int* s_flag = s_scan + 32;             // "this CTA drew the last ticket" (the scan only uses 32 words)
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(smem + TmaSmem::bars);
    volatile int* s_page = reinterpret_cast<volatile int*>(smem + TmaSmem::pages);
    const uint32_t tiles_u32 = smem_u32(smem);
    const uint32_t full0 = smem_u32(s_bar), empty0 = full0 + kStages * 8;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full0 + s * 8, 1);
            mbar_init(empty0 + s * 8, kConsumerWarps);
        }
        fence_mbar_init();
        fence_proxy_async();
    }
    // With the append fused in, the lengths this launch reads include the token it appends, and whatever wrote
    // them may be the kernel directly in front: wait for it before the first look at them.  (Two attention
    // launches never share an SM - each takes nearly all of its shared memory - so nothing is lost.)
    if (p.new_k != nullptr) pdl_wait();
    uint8_t* s_rem = smem + TmaSmem::rem;
    build_tile_prefix(p.context_lens, p.batch, TT, s_tp, s_scan, s_rem, p.seg_overhead);   // ends with __syncthreads
    // Everything above only reads step metadata; the pools and q may still be written by the
    // kernel in front of this one (the append) when this kernel was launched programmatically.
    pdl_launch_dependents();
    pdl_wait();

    const int ng = p.n_kv_heads / HPC;
    const int total = ng * s_tp[p.batch];
    const int chunk = max(1, (total + int(gridDim.x) - 1) / int(gridDim.x));
    const int lo = min(total, int(blockIdx.x) * chunk), hi = min(total, lo + chunk);

    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------ producer
        if (lane != 0) return;
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        uint32_t it = 0;
        bool ok = true;
        for (int g = lo; g < hi && ok;) {
            const Segment sg = locate_segment(s_tp, p.batch, ng, g, hi, p.seg_overhead);
            const int32_t* table = p.block_tables + int64_t(sg.b) * p.bt_stride;
            for (int t = sg.t0; t < sg.t1; ++t, ++it) {
                const uint32_t s = it % kStages, ph = (it / kStages) & 1;
                if (!mbar_wait(empty0 + s * 8, ph ^ 1, p.wait_limit)) { ok = false; break; }
                const int tok0 = t * TT;
                const int page = table[tok0 / p.block_size];
                const int slot0 = page * p.block_size + tok0 % p.block_size;
                const uint32_t bar = full0 + s * 8;
                const uint32_t kdst = tiles_u32 + s * (2 * kTileBytes), vdst = kdst + kTileBytes;
                if (p.stall_producer) continue;          // self-test: nothing is armed, every wait on this stage runs out
                s_page[s] = page;                         // for the warp that appends into this tile; released by the arrival below
                // a sequence's last tile: only the rows that exist (in boxes of 16, 32 or 64 rows); what the stage
                // holds behind them is masked by the consumers like any row past the context's end
                const CUtensorMap* mk = &map_k;
                const CUtensorMap* mv = &map_v;
                uint32_t bytes = 2 * kTileBytes;
                if (t == sg.ntiles - 1) {
                    const int rem = s_rem[sg.b];
#pragma unroll
                    for (int i = kTailMaps - 1; i >= 0; --i)
                        if (rem != 0 && (16 << i) < TT && rem <= (16 << i)) {
                            mk = &tails.k[i];
                            mv = &tails.v[i];
                            bytes = 4 * HPC * (16 << i) * 128;
                        }
                }
                mbar_expect_tx(bar, bytes);
#pragma unroll
                for (int hl = 0; hl < HPC; ++hl) {
                    const int head = sg.hg * HPC + hl;
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        tma_load_3d(kdst + (hl * 2 + half) * SUB, mk, bar, half * 64, head, slot0);
                        tma_load_3d(vdst + (hl * 2 + half) * SUB, mv, bar, half * 64, head, slot0);
                    }
                }
            }
            g += sg.span;
        }
        // Do not leave while a copy may still be in flight: wait for the last armed stages.
        const uint32_t armed = p.stall_producer ? 0u : (it < uint32_t(kStages) ? it : uint32_t(kStages));
        for (uint32_t j = 0; j < armed; ++j) {
            const uint32_t i2 = it - 1 - j;
            if (!mbar_wait(full0 + (i2 % kStages) * 8, (i2 / kStages) & 1, p.wait_limit)) ok = false;
        }
        if (!ok) atomicExch(p.status, kStatusMagic | 1);
        return;
    }

    // ---------------------------------------------------------------- consumers
    const int hl = warp / WPH, tw = warp % WPH;
    const int gid = lane >> 2, tig = lane & 3;
    const int mi = lane >> 3, mr = lane & 7;
    uint32_t it = 0;
    bool ok = true;

    // A wait that runs out only clears `ok`: the warp keeps walking the same tiles and
    // barriers as its siblings (without computing) so that no named barrier is left short.
    for (int g = lo; g < hi;) {
        const Segment sg = locate_segment(s_tp, p.batch, ng, g, hi, p.seg_overhead);
        if (sg.t0 == sg.t1) {                      // only padding of this (b, hg) lies in the range
            g += sg.span;
            continue;
        }
        const int ctx = p.context_lens[sg.b];
        const int head = sg.hg * HPC + hl;
        // Query fragments: rows 0..group-1 of the 16-row A operand, zero elsewhere.
        uint32_t qa[8][2];
        {
            const uint32_t* qrow = reinterpret_cast<const uint32_t*>(
                p.q + (int64_t(sg.b) * p.n_q_heads + head * p.group + gid) * kHeadDim);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                qa[kk][0] = gid < p.group ? qrow[kk * 8 + tig] : 0u;
                qa[kk][1] = gid < p.group ? qrow[kk * 8 + 4 + tig] : 0u;
            }
        }
        float o[16][4];
#pragma unroll
        for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
        float m_run = -INFINITY, l_run = 0.f;

        // Fused append.  The token at position ctx - 1 is not in the pool yet: its k and v rows come with the call.
        // Every warp of a segment that ends its sequence starts an asynchronous copy of this head's two rows into
        // its 512 bytes of staging memory (lanes 0-15 sixteen bytes of k each, lanes 16-31 of v): no register and
        // no instruction waits for them (with plain loads here, and a register holding the rows, the step measured
        // slower than two launches: such a load takes about a microsecond to return while the SM streams tiles).
        // The warp whose 16 tokens of the last tile include the position moves the rows, once the tile has arrived,
        // into the tile in shared memory, where the products below find them, and into the pool, where the next
        // step will.  The last tile of a (sequence, head) belongs to one CTA and a tile's rows to one warp, so each
        // row is written once; what the bulk copy brought for that row (stale or half-written) is replaced.
        const bool appends = p.new_k != nullptr && sg.t1 == sg.ntiles;
        const uint32_t stage_row = tiles_u32 + TmaSmem::patch + warp * 512 + lane * 16;
        if (appends) {
            cp_async_wait_all();                     // an earlier segment's copy into the same bytes (long done)
            const __nv_bfloat16* src = lane < 16 ? p.new_k + int64_t(sg.b) * p.new_k_stride
                                                 : p.new_v + int64_t(sg.b) * p.new_v_stride;
            cp_async_16(stage_row, src + head * kHeadDim + (lane & 15) * 8);
        }

        for (int t = sg.t0; t < sg.t1; ++t, ++it) {
            const uint32_t s = it % kStages, ph = (it / kStages) & 1;
            if (ok && !mbar_wait(full0 + s * 8, ph, p.wait_limit)) ok = false;
            const int tok_w = t * TT + tw * 16;            // first token of this warp's 16
            const int valid = ctx - tok_w;                  // tokens of the 16 that exist
            if (ok && valid > 0) {
                const uint32_t kbase = tiles_u32 + s * (2 * kTileBytes) + (hl * 2) * SUB;
                const uint32_t vbase = kbase + kTileBytes;
                if (appends && t == sg.ntiles - 1 && ((ctx - 1) % TT) / 16 == tw) {
                    cp_async_wait_all();
                    const uint4 new_row = ld_shared_v4(stage_row);
                    const int c = lane & 15, r = (ctx - 1) % TT;
                    st_shared_v4((lane < 16 ? kbase : vbase) + (c >> 3) * SUB + swz128(r, c & 7), new_row);
                    fence_proxy_async();          // this stage's next filling is a bulk copy: order the write before it
                    __syncwarp();
                    const int page = s_page[s];
                    if (page >= 0 && page < p.num_blocks) {
                        const int64_t slot = int64_t(page) * p.block_size + (ctx - 1) % p.block_size;
                        __nv_bfloat16* pool = static_cast<__nv_bfloat16*>(const_cast<void*>(lane < 16 ? p.k_cache : p.v_cache));
                        *reinterpret_cast<uint4*>(pool + (slot * p.n_kv_heads + head) * kHeadDim + c * 8) = new_row;
                    }
                }
                float sc[2][4];
#pragma unroll
                for (int j = 0; j < 2; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const int row = tw * 16 + (mi >> 1) * 8 + mr;
                    const int chunk16 = (kk & 3) * 2 + (mi & 1);
                    uint32_t b00, b01, b10, b11;
                    ldsm_x4(kbase + (kk >> 2) * SUB + swz128(row, chunk16), b00, b01, b10, b11);
                    mma_bf16(sc[0], qa[kk][0], 0u, qa[kk][1], 0u, b00, b01);
                    mma_bf16(sc[1], qa[kk][0], 0u, qa[kk][1], 0u, b10, b11);
                }
                if (valid < 16) {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        if (j * 8 + 2 * tig >= valid) sc[j][0] = -INFINITY;
                        if (j * 8 + 2 * tig + 1 >= valid) sc[j][1] = -INFINITY;
                    }
                }
                float mx = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m_run, mx * p.scale_log2);
                const float alpha = fast_exp2(m_run - m_new);
                const float p00 = fast_exp2(fmaf(sc[0][0], p.scale_log2, -m_new));
                const float p01 = fast_exp2(fmaf(sc[0][1], p.scale_log2, -m_new));
                const float p10 = fast_exp2(fmaf(sc[1][0], p.scale_log2, -m_new));
                const float p11 = fast_exp2(fmaf(sc[1][1], p.scale_log2, -m_new));
                l_run = l_run * alpha + (p00 + p01) + (p10 + p11);
                m_run = m_new;
                const uint32_t pa0 = pack_bf16(p00, p01), pa2 = pack_bf16(p10, p11);
#pragma unroll
                for (int j = 0; j < 16; ++j) { o[j][0] *= alpha; o[j][1] *= alpha; }
#pragma unroll
                for (int n2 = 0; n2 < 8; ++n2) {
                    const int row = tw * 16 + (mi & 1) * 8 + mr;
                    const int chunk16 = (n2 & 3) * 2 + (mi >> 1);
                    uint32_t v0, v1, v2, v3;
                    ldsm_x4_trans(vbase + (n2 >> 2) * SUB + swz128(row, chunk16), v0, v1, v2, v3);
                    if (valid < 16) {
                        // rows past the context may hold anything (0 * NaN): clear them
                        const uint32_t keep_lo = (2 * tig < valid ? 0x0000ffffu : 0u) | (2 * tig + 1 < valid ? 0xffff0000u : 0u);
                        const uint32_t keep_hi = (8 + 2 * tig < valid ? 0x0000ffffu : 0u) | (9 + 2 * tig < valid ? 0xffff0000u : 0u);
                        v0 &= keep_lo; v2 &= keep_lo;
                        v1 &= keep_hi; v3 &= keep_hi;
                    }
                    mma_bf16(o[2 * n2], pa0, 0u, pa2, 0u, v0, v1);
                    mma_bf16(o[2 * n2 + 1], pa0, 0u, pa2, 0u, v2, v3);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + s * 8);
        }
        // row sum over the quad that shares a query row
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);

        // merge of the WPH warps that share a kv head
        auto put = [&](float* slot) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                slot[(2 * j) * 32 + lane] = o[j][0];
                slot[(2 * j + 1) * 32 + lane] = o[j][1];
            }
            slot[32 * 32 + lane] = m_run;
            slot[33 * 32 + lane] = l_run;
        };
        auto take = [&](const float* slot) {
            const float m2 = slot[32 * 32 + lane], l2 = slot[33 * 32 + lane];
            const float mm = fmaxf(m_run, m2);
            const float a1 = m_run == -INFINITY ? 0.f : fast_exp2(m_run - mm);
            const float a2 = m2 == -INFINITY ? 0.f : fast_exp2(m2 - mm);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                o[j][0] = o[j][0] * a1 + slot[(2 * j) * 32 + lane] * a2;
                o[j][1] = o[j][1] * a1 + slot[(2 * j + 1) * 32 + lane] * a2;
            }
            l_run = l_run * a1 + l2 * a2;
            m_run = mm;
        };
        if (WPH == 8) {
            // eight warps, four slots, three barriers: warps 4-7 hand over to warps 0-3, warps 1-3 hand over (each in
            // the slot it has just read, which nobody else looks at) to warp 0
            if (tw >= 4) put(s_merge + (tw - 4) * kMergeSlotFloats);
            consumer_bar();
            if (tw < 4) take(s_merge + tw * kMergeSlotFloats);
            if (tw >= 1 && tw < 4) put(s_merge + tw * kMergeSlotFloats);
            consumer_bar();
            if (tw == 0) {
                take(s_merge + 1 * kMergeSlotFloats);
                take(s_merge + 2 * kMergeSlotFloats);
                take(s_merge + 3 * kMergeSlotFloats);
            }
            consumer_bar();                       // the slots are written again at the end of the next segment
        } else if (WPH > 1) {
#pragma unroll
            for (int stride = WPH / 2; stride >= 1; stride >>= 1) {
                float* slot = s_merge + (hl * stride + (tw % stride)) * kMergeSlotFloats;
                if (tw >= stride && tw < 2 * stride) put(slot);
                consumer_bar();
                if (tw < stride) take(slot);
                consumer_bar();
            }
        }

        if (ok && tw == 0 && gid < p.group) {
            const bool complete = sg.t0 == 0 && sg.t1 == sg.ntiles;
            const int qh = head * p.group + gid;
            if (complete) {
                const float inv = 1.f / l_run;
                uint32_t* dst = reinterpret_cast<uint32_t*>(p.out + (int64_t(sg.b) * p.n_q_heads + qh) * kHeadDim);
#pragma unroll
                for (int j = 0; j < 16; ++j) dst[j * 4 + tig] = pack_bf16(o[j][0] * inv, o[j][1] * inv);
            } else {
                const int rows = HPC * p.group;
                const int64_t slot = int64_t(blockIdx.x) * 2 + (sg.t0 > 0 ? 0 : 1);
                const int r = hl * p.group + gid;
                float2* dst = reinterpret_cast<float2*>(p.ws_o + (slot * rows + r) * kHeadDim);
#pragma unroll
                for (int j = 0; j < 16; ++j) dst[j * 4 + tig] = make_float2(o[j][0], o[j][1]);
                if (tig == 0) {
                    p.ws_ml[(slot * rows + r) * 2 + 0] = m_run;
                    p.ws_ml[(slot * rows + r) * 2 + 1] = l_run;
                }
            }
        }
        if (!(sg.t0 == 0 && sg.t1 == sg.ntiles)) merge_if_last(p, s_tp, ng, sg, chunk, HPC * p.group, s_flag);
        g += sg.span;
    }
    if (!ok && lane == 0) atomicExch(p.status, kStatusMagic | 2);
}

// =========================================================================== TMA kernel, e4m3 pools
// Same work split and ring as decode_tma_kernel<1>, with a tile of one whole 256-token page of
// one kv head (32 KiB of K + 32 KiB of V).  K and V bytes go from shared memory to the tensor
// cores as f16 (e4m3 -> f16 is exact), q is converted to f16 once per segment.  The products
// are token-major (the 16 MMA rows are tokens, the 8 columns the group's query heads), which
// halves the number of products and accumulator registers against head-major ones (131 against
// 138 us on the benchmark's lengths).
// The page's K scale is folded into the softmax exponent; the V scale is handled by keeping
// the accumulator in units of the current page's V scale and folding scale changes into the
// online-softmax correction, so no per-element dequantisation multiply is needed.
constexpr int kFp8TileTokens = 256;

// HPC kv heads per tile (1, 2, 4 or 8): a tile is 256 / HPC tokens of HPC adjacent heads, loaded head by
// head (one TMA box of 128-byte rows each) into [head][token][128 B].  With several heads the boxes fetch
// adjacent 128-byte pieces of every token row back to back, which is what the bf16 kernel's two column
// halves do; with one head every row is a lone 128-byte line at a pitch of Hkv * 128 B (measured: 8
// heads per token 112 us, the same bytes as a single-head pool 98 us).  Eight consumer warps,
// 32 tokens per warp and tile; sixteen warps of 16 tokens were measured slower.
template <int HPC>
struct Fp8Smem {
    static constexpr int threads = kTmaThreads;
    static constexpr int merge = TmaSmem::tiles;
    static constexpr int prefix = merge + 4 * kMergeSlotFloats * 4;
    static constexpr int scan = prefix + (kMaxBatch + 1) * 4 + 12;
    static constexpr int bars = scan + threads * 4;
    static constexpr int meta = bars + 2 * kStages * 8 + 16;      // [kStages][HPC][2] floats: k scale, v scale
    static constexpr int rem = meta + kStages * HPC * 8;           // tokens in every sequence's last tile, one byte each
    static constexpr int total = rem + kMaxBatch;
};

template <int HPC>
__global__ void __launch_bounds__(kTmaThreads, 1) decode_tma_fp8_kernel(DecodeParams p,
                                                                          const __grid_constant__ CUtensorMap map_k,
                                                                          const __grid_constant__ CUtensorMap map_v,
                                                                          const __grid_constant__ TailMaps tails) {
    static_assert(HPC == 1 || HPC == 2 || HPC == 4 || HPC == 8, "1, 2, 4 or 8 kv heads per tile");
    constexpr int W = kConsumerWarps;
    constexpr int TT = kFp8TileTokens / HPC;     // tokens per tile
    constexpr int WPH = W / HPC;                 // consumer warps per head
    constexpr int TPW = TT / WPH;                // tokens per warp and tile
    constexpr int NH = TPW / 16;                 // 16-token MMA tiles per warp and tile
    constexpr int kHeadBytes = TT * 128;         // one head's K (or V) rows of a tile
    static_assert(TPW == 32, "32 tokens per warp and tile");
    using L = Fp8Smem<HPC>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* s_merge = reinterpret_cast<float*>(smem + L::merge);
    int* s_tp = reinterpret_cast<int*>(smem + L::prefix);
    int* s_scan = reinterpret_cast<int*>(smem + L::scan);
    volatile int* s_flag = s_scan + 32;             // "this CTA drew the last ticket" (the scan only uses 32 words)
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(smem + L::bars);
    volatile float* s_meta = reinterpret_cast<volatile float*>(smem + L::meta);
    const uint32_t tiles_u32 = smem_u32(smem);
    const uint32_t full0 = smem_u32(s_bar), empty0 = full0 + kStages * 8;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full0 + s * 8, 1);
            mbar_init(empty0 + s * 8, W);
        }
        fence_mbar_init();
        fence_proxy_async();
    }
    uint8_t* s_rem = smem + L::rem;
    build_tile_prefix(p.context_lens, p.batch, TT, s_tp, s_scan, s_rem, p.seg_overhead);
    pdl_launch_dependents();
    pdl_wait();

    const int ng = p.n_kv_heads / HPC;
    const int total = ng * s_tp[p.batch];
    const int chunk = max(1, (total + int(gridDim.x) - 1) / int(gridDim.x));
    const int lo = min(total, int(blockIdx.x) * chunk), hi = min(total, lo + chunk);

    if (warp == W) {
        // ------------------------------------------------------------ producer
        if (lane != 0) return;
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        uint32_t it = 0;
        bool ok = true;
        for (int g = lo; g < hi && ok;) {
            const Segment sg = locate_segment(s_tp, p.batch, ng, g, hi, p.seg_overhead);
            const int32_t* table = p.block_tables + int64_t(sg.b) * p.bt_stride;
            for (int t = sg.t0; t < sg.t1; ++t, ++it) {
                const uint32_t s = it % kStages, ph = (it / kStages) & 1;
                const int tok0 = t * TT;
                const int page = table[tok0 / p.block_size];
                const int slot0 = page * p.block_size + tok0 % p.block_size;
                const bool page_ok = page >= 0 && page < p.num_blocks;
                float ks[HPC], vs[HPC];
#pragma unroll
                for (int hl = 0; hl < HPC; ++hl) {
                    ks[hl] = page_ok ? p.k_scale[int64_t(page) * p.n_kv_heads + sg.hg * HPC + hl] : 0.f;
                    vs[hl] = page_ok ? p.v_scale[int64_t(page) * p.n_kv_heads + sg.hg * HPC + hl] : 0.f;
                }
                if (!mbar_wait(empty0 + s * 8, ph ^ 1, p.wait_limit)) { ok = false; break; }
#pragma unroll
                for (int hl = 0; hl < HPC; ++hl) {
                    s_meta[(s * HPC + hl) * 2 + 0] = ks[hl];
                    s_meta[(s * HPC + hl) * 2 + 1] = vs[hl];
                }
                const uint32_t bar = full0 + s * 8;
                const uint32_t kdst = tiles_u32 + s * (2 * kTileBytes), vdst = kdst + kTileBytes;
                if (p.stall_producer) continue;          // self-test: nothing is armed, every wait on this stage runs out
                // a sequence's last tile: only the rows that exist (see decode_tma_kernel)
                const CUtensorMap* mk = &map_k;
                const CUtensorMap* mv = &map_v;
                uint32_t bytes = 2 * kTileBytes;
                if (t == sg.ntiles - 1) {
                    const int rem = s_rem[sg.b];
#pragma unroll
                    for (int i = kTailMaps - 1; i >= 0; --i)
                        if (rem != 0 && (16 << i) < TT && rem <= (16 << i)) {
                            mk = &tails.k[i];
                            mv = &tails.v[i];
                            bytes = 2 * HPC * (16 << i) * 128;
                        }
                }
                mbar_expect_tx(bar, bytes);               // release: the scales above are visible to the waiters
#pragma unroll
                for (int hl = 0; hl < HPC; ++hl) {        // the heads' boxes back to back: adjacent lines of every token row
                    tma_load_3d(kdst + hl * kHeadBytes, mk, bar, 0, sg.hg * HPC + hl, slot0);
                    tma_load_3d(vdst + hl * kHeadBytes, mv, bar, 0, sg.hg * HPC + hl, slot0);
                }
            }
            g += sg.span;
        }
        const uint32_t armed = p.stall_producer ? 0u : (it < uint32_t(kStages) ? it : uint32_t(kStages));
        for (uint32_t j = 0; j < armed; ++j) {
            const uint32_t i2 = it - 1 - j;
            if (!mbar_wait(full0 + (i2 % kStages) * 8, (i2 / kStages) & 1, p.wait_limit)) ok = false;
        }
        if (!ok) atomicExch(p.status, kStatusMagic | 1);
        return;
    }

    // ---------------------------------------------------------------- consumers: 32 tokens per warp and tile
    // Token-major products: the 16 rows of an MMA are TOKENS (all used), the 8 columns the query
    // heads of the group.  S^T[token][head] = K Q^T takes 16 products per 32 tokens, and
    // O^T[dim][head] += V^T P^T another 16, half of what head-major products need, with 32
    // accumulator registers instead of 64.  A lane holds, for the heads (2t, 2t+1) of its quad
    // position t, the scores of four tokens and the output dims (16c + 2g, 16c + 2g + 1), c = 0..7.
    const int hl = warp / WPH, tw = warp % WPH;      // head of the tile, warp within that head
    const int gid = lane >> 2, tig = lane & 3;
    const int mi = lane >> 3, mr = lane & 7;
    uint32_t it = 0;
    bool ok = true;

    for (int g = lo; g < hi;) {
        const Segment sg = locate_segment(s_tp, p.batch, ng, g, hi, p.seg_overhead);
        if (sg.t0 == sg.t1) {                      // only padding of this (b, hg) lies in the range
            g += sg.span;
            continue;
        }
        const int ctx = p.context_lens[sg.b];
        const int head = sg.hg * HPC + hl;
        // B fragments of Q^T in f16: column gid is query head gid of the group.  MMA k-slots
        // (2t, 2t+1, 2t+8, 2t+9) of a 16-dim chunk carry dims (4t, 4t+1, 4t+2, 4t+3): the order in
        // which ldmatrix hands out e4m3 bytes.
        uint32_t qb[8][2];
        {
            const __nv_bfloat16* qrow = p.q + (int64_t(sg.b) * p.n_q_heads + head * p.group + gid) * kHeadDim;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                qb[c][0] = qb[c][1] = 0u;
                if (gid < p.group) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(qrow + c * 16 + tig * 4);
                    const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
                    const __nv_bfloat162 y = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
                    qb[c][0] = pack_f16(__low2float(x), __high2float(x));
                    qb[c][1] = pack_f16(__low2float(y), __high2float(y));
                }
            }
        }
        float o[8][4];                           // O^T: tile c, rows (dims 16c + 2g, 16c + 2g + 1), columns (heads 2t, 2t+1)
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
        float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // per head (2t, 2t+1)
        float s_cur = 0.f;                       // V scale the accumulator is currently expressed in

        for (int t = sg.t0; t < sg.t1; ++t, ++it) {
            const uint32_t s = it % kStages, ph = (it / kStages) & 1;
            if (ok && !mbar_wait(full0 + s * 8, ph, p.wait_limit)) ok = false;
            const float c_k = s_meta[(s * HPC + hl) * 2 + 0] * p.scale_log2;
            const float vs = s_meta[(s * HPC + hl) * 2 + 1];
            const int row0 = tw * TPW;                      // this warp's tokens of the tile
            const int valid = ctx - (t * TT + row0);
            if (ok && valid > 0) {
                const uint32_t kbase = tiles_u32 + s * (2 * kTileBytes) + hl * kHeadBytes;
                const uint32_t vbase = kbase + kTileBytes;
                // S^T: NH 16-token tiles, each with an even-chunk and an odd-chunk accumulator
                float sc[NH][2][4];
#pragma unroll
                for (int h = 0; h < NH; ++h)
#pragma unroll
                    for (int e = 0; e < 2; ++e) sc[h][e][0] = sc[h][e][1] = sc[h][e][2] = sc[h][e][3] = 0.f;
#pragma unroll
                for (int c2 = 0; c2 < 4; ++c2) {
#pragma unroll
                    for (int h = 0; h < NH; ++h) {
                        uint32_t r0, r1, r2, r3;   // (tokens 0-7, chunk 2c2), (0-7, 2c2+1), (8-15, 2c2), (8-15, 2c2+1) of half h
                        ldsm_x4(kbase + swz128(row0 + h * 16 + (mi >> 1) * 8 + mr, c2 * 2 + (mi & 1)), r0, r1, r2, r3);
                        uint32_t a0, a1, a2, a3;
                        e4m3x4_to_f16x2x2(r0, a0, a2);      // token gid: dims (4t, 4t+1) and (4t+2, 4t+3) of chunk 2c2
                        e4m3x4_to_f16x2x2(r2, a1, a3);      // token gid + 8
                        mma_f16(sc[h][0], a0, a1, a2, a3, qb[2 * c2][0], qb[2 * c2][1]);
                        e4m3x4_to_f16x2x2(r1, a0, a2);      // chunk 2c2 + 1
                        e4m3x4_to_f16x2x2(r3, a1, a3);
                        mma_f16(sc[h][1], a0, a1, a2, a3, qb[2 * c2 + 1][0], qb[2 * c2 + 1][1]);
                    }
                }
                // sv[h][x][y]: token 16h + 8x + gid, head 2 tig + y
                float sv[NH][2][2];
#pragma unroll
                for (int h = 0; h < NH; ++h)
#pragma unroll
                    for (int x = 0; x < 2; ++x) {
                        const bool dead = h * 16 + x * 8 + gid >= valid;
                        sv[h][x][0] = dead ? -INFINITY : sc[h][0][2 * x] + sc[h][1][2 * x];
                        sv[h][x][1] = dead ? -INFINITY : sc[h][0][2 * x + 1] + sc[h][1][2 * x + 1];
                    }
                float alpha[2];
                uint32_t pp[NH][2];                         // P as f16 pairs (head 2t, head 2t+1): [h][x] = token 16h + 8x + gid
                float pr[NH][2][2];
#pragma unroll
                for (int y = 0; y < 2; ++y) {
                    float mx = fmaxf(sv[0][0][y], sv[0][1][y]);
                    if (NH == 2) mx = fmaxf(mx, fmaxf(sv[NH - 1][0][y], sv[NH - 1][1][y]));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                    // with c_k == 0 (all-zero page) every visible logit is 0; masked ones stay -inf
                    const float m_new = fmaxf(m_run[y], c_k > 0.f ? mx * c_k : 0.f);
                    alpha[y] = fast_exp2(m_run[y] - m_new);
                    float rs = 0.f;
#pragma unroll
                    for (int h = 0; h < NH; ++h)
#pragma unroll
                        for (int x = 0; x < 2; ++x) {
                            pr[h][x][y] = sv[h][x][y] == -INFINITY ? 0.f : fast_exp2(fmaf(sv[h][x][y], c_k, -m_new));
                            rs += pr[h][x][y];
                        }
                    l_run[y] = l_run[y] * alpha[y] + rs;
                    m_run[y] = m_new;
                }
#pragma unroll
                for (int h = 0; h < NH; ++h)
#pragma unroll
                    for (int x = 0; x < 2; ++x) pp[h][x] = pack_f16(pr[h][x][0], pr[h][x][1]);
                if (vs > 0.f && vs != s_cur) {       // re-express the accumulator in this page's V scale
                    if (s_cur > 0.f) {
                        const float f = __fdividef(s_cur, vs);
                        alpha[0] *= f;
                        alpha[1] *= f;
                    }
                    s_cur = vs;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    o[j][0] *= alpha[0]; o[j][2] *= alpha[0];
                    o[j][1] *= alpha[1]; o[j][3] *= alpha[1];
                }
#pragma unroll
                for (int h = 0; h < NH; ++h) {
                    // B fragments of P^T: transposing the two 8x8 blocks (tokens x heads) turns "token gid, heads
                    // 2t 2t+1" into "head gid, tokens 2t 2t+1"
                    const uint32_t pb0 = movmatrix_trans(pp[h][0]), pb1 = movmatrix_trans(pp[h][1]);
                    const int vh = valid - h * 16;          // tokens of this half that exist
#pragma unroll
                    for (int c2 = 0; c2 < 4; ++c2) {
                        uint32_t r0, r1, r2, r3;   // (tokens 0-7, chunk 2c2), (8-15, 2c2), (0-7, 2c2+1), (8-15, 2c2+1)
                        ldsm_x4_trans(vbase + swz128(row0 + h * 16 + (mi & 1) * 8 + mr, c2 * 2 + (mi >> 1)), r0, r1, r2, r3);
                        if (vh < 16) {
                            const uint32_t keep_lo = (2 * tig < vh ? 0x0000ffffu : 0u) | (2 * tig + 1 < vh ? 0xffff0000u : 0u);
                            const uint32_t keep_hi = (8 + 2 * tig < vh ? 0x0000ffffu : 0u) | (9 + 2 * tig < vh ? 0xffff0000u : 0u);
                            r0 &= keep_lo; r2 &= keep_lo;
                            r1 &= keep_hi; r3 &= keep_hi;
                        }
                        // a transposed register holds (tok 2t, dims 2g 2g+1 | tok 2t+1, dims 2g 2g+1): bytes (0,2) are the
                        // even dim's two tokens (A rows 0-7 of the tile), bytes (1,3) the odd dim's (A rows 8-15)
                        // one byte permute (0,2,1,3) per register, then the low half converts to A rows 0-7, the high half to 8-15
                        uint32_t a0, a1, a2, a3;
                        e4m3x4_to_f16x2x2(__byte_perm(r0, 0, 0x3120), a0, a1);
                        e4m3x4_to_f16x2x2(__byte_perm(r1, 0, 0x3120), a2, a3);
                        mma_f16(o[2 * c2], a0, a1, a2, a3, pb0, pb1);
                        e4m3x4_to_f16x2x2(__byte_perm(r2, 0, 0x3120), a0, a1);
                        e4m3x4_to_f16x2x2(__byte_perm(r3, 0, 0x3120), a2, a3);
                        mma_f16(o[2 * c2 + 1], a0, a1, a2, a3, pb0, pb1);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + s * 8);
        }
        // row sums over the warp's tokens (lanes of equal t); m_run is already equal in those lanes
#pragma unroll
        for (int y = 0; y < 2; ++y) {
            l_run[y] += __shfl_xor_sync(0xffffffffu, l_run[y], 4);
            l_run[y] += __shfl_xor_sync(0xffffffffu, l_run[y], 8);
            l_run[y] += __shfl_xor_sync(0xffffffffu, l_run[y], 16);
        }
        // back to true units before warps (which may sit on different pages) are merged
#pragma unroll
        for (int j = 0; j < 8; ++j) { o[j][0] *= s_cur; o[j][1] *= s_cur; o[j][2] *= s_cur; o[j][3] *= s_cur; }

        // merge the partial results of a head's warps through shared slots (four in all): warps [n, 2n) of
        // every head hand theirs to warps [0, n)
#pragma unroll
        for (int n = WPH / 2; n >= 1; n >>= 1) {
            float* slot = s_merge + (hl * (WPH / 2) + (tw % n)) * kMergeSlotFloats;
            if (tw >= n && tw < 2 * n) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int k = 0; k < 4; ++k) slot[(4 * j + k) * 32 + lane] = o[j][k];
                slot[32 * 32 + lane] = m_run[0];
                slot[33 * 32 + lane] = m_run[1];
                slot[34 * 32 + lane] = l_run[0];
                slot[35 * 32 + lane] = l_run[1];
            }
            consumer_bar();
            if (tw < n) {
#pragma unroll
                for (int y = 0; y < 2; ++y) {
                    const float m2 = slot[(32 + y) * 32 + lane], l2 = slot[(34 + y) * 32 + lane];
                    const float mm = fmaxf(m_run[y], m2);
                    const float a1 = m_run[y] == -INFINITY ? 0.f : fast_exp2(m_run[y] - mm);
                    const float a2 = m2 == -INFINITY ? 0.f : fast_exp2(m2 - mm);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        o[j][y] = o[j][y] * a1 + slot[(4 * j + y) * 32 + lane] * a2;
                        o[j][y + 2] = o[j][y + 2] * a1 + slot[(4 * j + y + 2) * 32 + lane] * a2;
                    }
                    l_run[y] = l_run[y] * a1 + l2 * a2;
                    m_run[y] = mm;
                }
            }
            consumer_bar();
        }

        if (ok && tw == 0) {
            // tile c holds dims (16c + 2g, 16c + 2g + 1) in (o[c][y], o[c][y + 2]) for head 2t + y
            const bool complete = sg.t0 == 0 && sg.t1 == sg.ntiles;
#pragma unroll
            for (int y = 0; y < 2; ++y) {
                const int hq = 2 * tig + y;
                if (hq >= p.group) continue;
                const int qh = head * p.group + hq;
                if (complete) {
                    const float inv = 1.f / l_run[y];
                    uint32_t* dst = reinterpret_cast<uint32_t*>(p.out + (int64_t(sg.b) * p.n_q_heads + qh) * kHeadDim);
#pragma unroll
                    for (int c = 0; c < 8; ++c) dst[c * 8 + gid] = pack_bf16(o[c][y] * inv, o[c][y + 2] * inv);
                } else {
                    const int rows = HPC * p.group, r = hl * p.group + hq;
                    const int64_t slot = int64_t(blockIdx.x) * 2 + (sg.t0 > 0 ? 0 : 1);
                    float2* dst = reinterpret_cast<float2*>(p.ws_o + (slot * rows + r) * kHeadDim);
#pragma unroll
                    for (int c = 0; c < 8; ++c) dst[c * 8 + gid] = make_float2(o[c][y], o[c][y + 2]);
                    if (gid == 0) {
                        p.ws_ml[(slot * rows + r) * 2 + 0] = m_run[y];
                        p.ws_ml[(slot * rows + r) * 2 + 1] = l_run[y];
                    }
                }
            }
        }
        if (!(sg.t0 == 0 && sg.t1 == sg.ntiles)) merge_if_last(p, s_tp, ng, sg, chunk, HPC * p.group, s_flag);
        g += sg.span;
    }
    if (!ok && lane == 0) atomicExch(p.status, kStatusMagic | 2);
}

// =========================================================================== host side
struct DecodeConfig {
    int hpc;          // kv heads per tile
    int grid;
    int rows;         // partial rows per scratch slot
};

// force_hpc: 0 = the measured default, else heads per tile (self-test entry point only).
// ws_limit: bytes of scratch the caller has (0 = no limit); the e4m3 kernel takes fewer heads per tile
// when the partial-result slots of more would not fit.
static DecodeConfig decode_config(const infer_kv_pool* pool, int n_q_heads, size_t ws_limit, int force_hpc) {
    DecodeConfig c;
    const int group = n_q_heads / pool->n_kv_heads;
    const bool forced = (force_hpc == 1 || force_hpc == 2 || force_hpc == 4 || force_hpc == 8) &&
                        pool->n_kv_heads % force_hpc == 0;
    if (pool->dtype == INFER_KV_E4M3) {
        // several adjacent heads per tile when the head count allows: their boxes fetch neighbouring lines
        // (measured on 8 heads: 1 head 111 us, 2 heads 98.7, 4 heads 96.5, 8 heads 105)
        c.hpc = pool->n_kv_heads % 4 == 0 ? 4 : (pool->n_kv_heads % 2 == 0 ? 2 : 1);
        if (forced) c.hpc = force_hpc;
        while (ws_limit && c.hpc > 1 && decode_layout(pool->sm_count, c.hpc * group).total > ws_limit) c.hpc /= 2;
    } else {
        // One kv head per tile (128 tokens x 256 B rows) measured fastest at every head count:
        // fewer, larger TMA boxes beat streaming all heads of a token row together.
        c.hpc = forced ? force_hpc : 1;
    }
    c.grid = pool->sm_count < kMaxDecodeGrid ? pool->sm_count : kMaxDecodeGrid;
    c.rows = c.hpc * group;
    return c;
}

static TailMaps tail_maps(const infer_kv_pool* pool) {
    TailMaps tails;
    for (int i = 0; i < kTailMaps; ++i) {
        tails.k[i] = pool->maps[i].k;
        tails.v[i] = pool->maps[i].v;
    }
    return tails;
}

template <int HPC>
static int launch_bf16(const DecodeParams& p, const infer_kv_pool* pool, int grid, cudaStream_t st) {
    int idx = 0;
    while ((16 << idx) != 128 / HPC) ++idx;
    const TailMaps tails = tail_maps(pool);
    IB_CUDA(launch_pdl(decode_tma_kernel<HPC>, dim3(grid), dim3(kTmaThreads), TmaSmem::total + 1024, st, p,
                       pool->maps[idx].k, pool->maps[idx].v, tails));
    return INFER_OK;
}

template <int HPC>
static int launch_fp8(const DecodeParams& p, const infer_kv_pool* pool, int grid, cudaStream_t st) {
    int idx = 0;
    while ((16 << idx) != kFp8TileTokens / HPC) ++idx;
    IB_CUDA(launch_pdl(decode_tma_fp8_kernel<HPC>, dim3(grid), dim3(kTmaThreads), Fp8Smem<HPC>::total + 1024, st, p,
                       pool->maps[idx].k, pool->maps[idx].v, tail_maps(pool)));
    return INFER_OK;
}

template <int HPC>
static cudaError_t allow_smem() {
    cudaError_t e = cudaFuncSetAttribute(decode_tma_kernel<HPC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         TmaSmem::total + 1024);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(decode_tma_fp8_kernel<HPC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                Fp8Smem<HPC>::total + 1024);
}

// Raises the dynamic shared-memory limit of every decode kernel on the current device.  Called once
// per pool creation so that the per-step entry points make no call but the launches.
int decode_prepare_device() {
    cudaError_t e = allow_smem<1>();
    if (e == cudaSuccess) e = allow_smem<2>();
    if (e == cudaSuccess) e = allow_smem<4>();
    if (e == cudaSuccess) e = allow_smem<8>();
    if (e != cudaSuccess) {
        set_cuda_error(e);
        return INFER_ERR_CUDA;
    }
    return INFER_OK;
}

// Tiles of padding in front of every (sequence, head group) in the numbering that is cut into equal ranges.
// Swept on the GPU, us per launch at 0 / 1 / 2 / 3 / 4 tiles: Qwen3-8B batch 64 171.5 / 165.9 / 163.8 / 163.3 / 165.9,
// long-context batch 256 830 / 802 / 784 / 776 / 778, one KV head of the batch-64 workload 30.7 / 29.7 / 29.0 / 28.0 /
// 27.9, the 8-sequence Qwen3-0.6B case 12.4 / 11.4 / 9.3 / 10.0 / 9.9.
constexpr int kSegOverheadTiles = 3;

// The step's new k and v rows for a launch that also appends them (null: the pools already hold them).
struct NewRows {
    const void* k = nullptr;
    const void* v = nullptr;
    int64_t k_stride = 0, v_stride = 0;
};

static int paged_decode(const infer_kv_pool_t* pool, void* out, const void* q, const int32_t* context_lens,
                        const int32_t* block_tables, int64_t bt_stride, int batch, int n_q_heads, float softmax_scale,
                        void* workspace, size_t workspace_bytes, cudaStream_t st, int force_hpc, uint32_t wait_limit,
                        int stall_producer, const NewRows& rows = NewRows()) {
    if (!pool || !out || !q || !context_lens || !block_tables) return INFER_ERR_NULL;
    if (rows.k || rows.v) {
        if (!rows.k || !rows.v) return INFER_ERR_NULL;
        if (pool->dtype != INFER_KV_BF16) return INFER_ERR_DTYPE;
        const int64_t row = int64_t(pool->n_kv_heads) * kHeadDim;
        if (rows.k_stride < row || rows.v_stride < row) return INFER_ERR_STRIDE;
        if (!aligned16(rows.k) || !aligned16(rows.v) || rows.k_stride % 8 || rows.v_stride % 8) return INFER_ERR_ALIGN;
    }
    if (batch < 0 || batch > kMaxBatch || n_q_heads <= 0 || n_q_heads % pool->n_kv_heads != 0 || bt_stride <= 0)
        return INFER_ERR_GEOMETRY;
    const int group = n_q_heads / pool->n_kv_heads;
    if (group > kMaxGroup) return INFER_ERR_GEOMETRY;
    if (!aligned16(out) || !aligned16(q)) return INFER_ERR_ALIGN;
    if (batch == 0) return INFER_OK;
    const DecodeConfig cfg = decode_config(pool, n_q_heads, workspace_bytes, force_hpc);
    const DecodeLayout lay = decode_layout(cfg.grid, cfg.rows);
    if (!workspace || !aligned16(workspace) || workspace_bytes < lay.total) return INFER_ERR_WORKSPACE;

    DecodeParams p;
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.out = static_cast<__nv_bfloat16*>(out);
    p.context_lens = context_lens;
    p.block_tables = block_tables;
    p.bt_stride = bt_stride;
    p.k_cache = pool->k_cache;
    p.v_cache = pool->v_cache;
    p.k_scale = pool->k_scale;
    p.v_scale = pool->v_scale;
    p.batch = batch;
    p.n_q_heads = n_q_heads;
    p.n_kv_heads = pool->n_kv_heads;
    p.group = group;
    p.block_size = pool->block_size;
    p.num_blocks = int(pool->num_blocks);
    p.scale_log2 = softmax_scale * 1.4426950408889634f;
    p.wait_limit = wait_limit;
    p.stall_producer = stall_producer;
    p.seg_overhead = kSegOverheadTiles;
    p.new_k = static_cast<const __nv_bfloat16*>(rows.k);
    p.new_v = static_cast<const __nv_bfloat16*>(rows.v);
    p.new_k_stride = rows.k_stride;
    p.new_v_stride = rows.v_stride;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    p.status = reinterpret_cast<int*>(ws + lay.status_off);
    p.counters = reinterpret_cast<int*>(ws + lay.counters_off);
    p.ws_ml = reinterpret_cast<float*>(ws + lay.ml_off);
    p.ws_o = reinterpret_cast<float*>(ws + lay.o_off);

    int rc;
    if (pool->dtype == INFER_KV_E4M3) {
        switch (cfg.hpc) {
            case 1: rc = launch_fp8<1>(p, pool, cfg.grid, st); break;
            case 2: rc = launch_fp8<2>(p, pool, cfg.grid, st); break;
            case 4: rc = launch_fp8<4>(p, pool, cfg.grid, st); break;
            default: rc = launch_fp8<8>(p, pool, cfg.grid, st); break;
        }
    } else {
        switch (cfg.hpc) {
            case 1: rc = launch_bf16<1>(p, pool, cfg.grid, st); break;
            case 2: rc = launch_bf16<2>(p, pool, cfg.grid, st); break;
            case 4: rc = launch_bf16<4>(p, pool, cfg.grid, st); break;
            default: rc = launch_bf16<8>(p, pool, cfg.grid, st); break;
        }
    }
    return rc != INFER_OK ? rc : check_launch();
}

// ------------------------------------------------------------------ entry point without scratch
// Scratch of infer_paged_decode_noalloc: lives in the library's device image, one copy per
// GPU that loads the library.  In host code the NAME below is only a handle for
// cudaGetSymbolAddress; kernels must be given the address that call returns.
constexpr size_t kBuiltinScratchBytes = size_t(2) << 20;
static __device__ __align__(256) unsigned char g_builtin_scratch[kBuiltinScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_builtin_scratch_addr[kMaxDevices];   // device address per device ordinal, 0 = not looked up yet
static std::mutex g_builtin_scratch_mutex;

// Device address of the built-in array on the current device (looked up once per device); dev_out
// receives the device ordinal.
static int builtin_scratch(void** addr_out, int* dev_out) {
    int dev = -1;
    IB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) {
        set_cuda_error(cudaErrorInvalidDevice);
        return INFER_ERR_CUDA;
    }
    std::lock_guard<std::mutex> lock(g_builtin_scratch_mutex);
    if (!g_builtin_scratch_addr[dev]) {
        void* addr = nullptr;
        IB_CUDA(cudaGetSymbolAddress(&addr, g_builtin_scratch));
        g_builtin_scratch_addr[dev] = addr;
    }
    *addr_out = g_builtin_scratch_addr[dev];
    *dev_out = dev;
    return INFER_OK;
}

}  // namespace ib

extern "C" {

size_t infer_paged_decode_workspace_bytes(const infer_kv_pool_t* pool, int batch, int n_q_heads) {
    (void)batch;
    if (!pool || n_q_heads <= 0 || n_q_heads % pool->n_kv_heads != 0) return 0;
    // sized for the widest tile (eight kv heads' partial rows per slot) so that no tile shape outgrows it
    const int group = n_q_heads / pool->n_kv_heads;
    const int grid = pool->sm_count < ib::kMaxDecodeGrid ? pool->sm_count : ib::kMaxDecodeGrid;
    return ib::decode_layout(grid, 8 * group).total;
}

int infer_paged_decode(const infer_kv_pool_t* pool, void* out, const void* q, const int32_t* context_lens,
                       const int32_t* block_tables, int64_t bt_stride, int batch, int n_q_heads,
                       float softmax_scale, void* workspace, size_t workspace_bytes, void* stream_) {
    return ib::paged_decode(pool, out, q, context_lens, block_tables, bt_stride, batch, n_q_heads, softmax_scale,
                            workspace, workspace_bytes, static_cast<cudaStream_t>(stream_), 0, ib::kDefaultWaitLimit, 0);
}

int infer_paged_decode_append(const infer_kv_pool_t* pool, void* out, const void* q, const void* k, const void* v,
                              int64_t k_row_stride, int64_t v_row_stride, const int32_t* context_lens,
                              const int32_t* block_tables, int64_t bt_stride, int batch, int n_q_heads,
                              float softmax_scale, void* workspace, size_t workspace_bytes, void* stream_) {
    if (!k || !v) return INFER_ERR_NULL;
    ib::NewRows rows;
    rows.k = k;
    rows.v = v;
    rows.k_stride = k_row_stride;
    rows.v_stride = v_row_stride;
    return ib::paged_decode(pool, out, q, context_lens, block_tables, bt_stride, batch, n_q_heads, softmax_scale,
                            workspace, workspace_bytes, static_cast<cudaStream_t>(stream_), 0, ib::kDefaultWaitLimit, 0, rows);
}

int infer_selftest_paged_decode(const infer_kv_pool_t* pool, void* out, const void* q, const int32_t* context_lens,
                                const int32_t* block_tables, int64_t bt_stride, int batch, int n_q_heads,
                                float softmax_scale, void* workspace, size_t workspace_bytes, void* stream_,
                                int heads_per_tile, uint32_t wait_limit, int stall_producer) {
    return ib::paged_decode(pool, out, q, context_lens, block_tables, bt_stride, batch, n_q_heads, softmax_scale,
                            workspace, workspace_bytes, static_cast<cudaStream_t>(stream_), heads_per_tile,
                            wait_limit ? wait_limit : ib::kDefaultWaitLimit, stall_producer);
}

int infer_paged_decode_status(const void* workspace, void* stream_) {
    using namespace ib;
    void* ws = const_cast<void*>(workspace);
    if (!ws) {                       // the built-in array of infer_paged_decode_noalloc on the current device
        int dev = -1;
        const int rc = builtin_scratch(&ws, &dev);
        if (rc != INFER_OK) return rc;
    }
    int word = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream_);
    IB_CUDA(cudaMemcpyAsync(&word, ws, sizeof(int), cudaMemcpyDeviceToHost, st));
    IB_CUDA(cudaStreamSynchronize(st));
    if ((word & 0xFFFF0000) != kStatusMagic) return INFER_OK;
    // a launch that gave up may have left tickets behind: clear the word and the counters
    IB_CUDA(cudaMemsetAsync(ws, 0, decode_layout(1, 1).ml_off, st));
    return INFER_ERR_DEVICE;
}

int infer_paged_decode_noalloc(const infer_kv_pool_t* pool, void* out, const void* q, const int32_t* context_lens,
                               const int32_t* block_tables, int64_t bt_stride, int batch, int n_q_heads,
                               float softmax_scale, void* stream_) {
    using namespace ib;
    if (!pool || !out || !q || !context_lens || !block_tables) return INFER_ERR_NULL;
    if (n_q_heads <= 0 || n_q_heads % pool->n_kv_heads != 0 || batch < 0) return INFER_ERR_GEOMETRY;
    if (batch > kMaxBatch) return INFER_ERR_TOO_LARGE;
    const DecodeConfig cfg = decode_config(pool, n_q_heads, kBuiltinScratchBytes, 0);
    const DecodeLayout lay = decode_layout(cfg.grid, cfg.rows);
    if (lay.total > kBuiltinScratchBytes) return INFER_ERR_TOO_LARGE;

    void* scratch = nullptr;
    int dev = -1;
    const int rc = builtin_scratch(&scratch, &dev);   // once per device, with that device current
    if (rc != INFER_OK) return rc;
    if (dev != pool->device) {
        set_cuda_error(cudaErrorInvalidDevice);
        return INFER_ERR_CUDA;
    }
    // the array keeps the previous call's bytes: the status word and the ticket counters have to start at zero
    IB_CUDA(cudaMemsetAsync(scratch, 0, lay.ml_off, static_cast<cudaStream_t>(stream_)));
    return infer_paged_decode(pool, out, q, context_lens, block_tables, bt_stride, batch, n_q_heads, softmax_scale,
                              scratch, kBuiltinScratchBytes, stream_);
}

}  // extern "C"
