// Paged decode attention (one query token per sequence) over the page pools.
//
//  * decode_tma_kernel   bf16 pools.  One persistent CTA per SM: a producer warp walks the
//    block tables and stages K/V tiles (128 (head, token) rows = 32 KiB of K + 32 KiB of V)
//    into a 3-stage shared-memory ring with TMA; eight consumer warps each own 16 tokens of
//    one kv head per tile, run q.K^T and P.V on mma.sync with the query-head group in the M
//    dimension, and keep the online-softmax state (max, sum, accumulator) in registers,
//    merging row statistics with quad shuffles.
//  * decode_simple_kernel   e4m3 pools (dequantise on load) - plain loads, CUDA cores.
//  * decode_reduce_kernel   merges the partials of (sequence, head group)s that span CTAs.
//
// The work split (equal KV bytes per CTA, two scratch slots per CTA) is described in
// decode_common.cuh.
#include <cstdlib>
#include <mutex>
#include <utility>

#include "decode_common.cuh"

namespace ib {

// =========================================================================== simple kernel
template <int G, bool FP8>
__global__ void __launch_bounds__(128) decode_simple_kernel(DecodeParams p) {
    constexpr int TT = 64;
    __shared__ int s_tp[kMaxBatch + 1];
    __shared__ int s_scan[128];
    __shared__ float s_m[4][G], s_l[4][G];
    __shared__ float s_o[4][G][kHeadDim];

    build_tile_prefix(p.context_lens, p.batch, TT, s_tp, s_scan);
    pdl_launch_dependents();
    pdl_wait();
    const int ng = p.n_kv_heads;
    const int total = ng * s_tp[p.batch];
    const int chunk = max(1, (total + int(gridDim.x) - 1) / int(gridDim.x));
    if (blockIdx.x == 0) {
        for (int i = threadIdx.x; i <= p.batch; i += blockDim.x) p.prefix[i] = s_tp[i];
        if (threadIdx.x == 0) {
            p.header[1] = total;
            p.header[2] = chunk;
            p.header[3] = gridDim.x;
        }
    }
    const int lo = min(total, int(blockIdx.x) * chunk), hi = min(total, lo + chunk);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int elem = FP8 ? 1 : 2;

    for (int g = lo; g < hi;) {
        const Segment sg = locate_segment(s_tp, p.batch, ng, g, hi);
        const int ctx = p.context_lens[sg.b];
        const int head = sg.hg;
        float q[G][4], o[G][4], m[G], l[G];
#pragma unroll
        for (int j = 0; j < G; ++j) {
            const uint2 raw = *reinterpret_cast<const uint2*>(
                p.q + (int64_t(sg.b) * p.n_q_heads + head * G + j) * kHeadDim + lane * 4);
            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
            const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
            q[j][0] = __low2float(a); q[j][1] = __high2float(a);
            q[j][2] = __low2float(c); q[j][3] = __high2float(c);
            o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
            m[j] = -INFINITY;
            l[j] = 0.f;
        }
        for (int t = sg.t0; t < sg.t1; ++t) {
            for (int i = 0; i < 16; ++i) {
                const int tok = t * TT + warp * 16 + i;
                if (tok >= ctx) break;
                const int page = p.block_tables[int64_t(sg.b) * p.bt_stride + tok / p.block_size];
                if (page < 0 || page >= p.num_blocks) continue;
                const int64_t slot = int64_t(page) * p.block_size + tok % p.block_size;
                const int64_t off = ((slot * p.n_kv_heads + head) * kHeadDim + lane * 4) * elem;
                float kf[4], vf[4];
                if (FP8) {
                    const uint32_t kr = *reinterpret_cast<const uint32_t*>(static_cast<const uint8_t*>(p.k_cache) + off);
                    const uint32_t vr = *reinterpret_cast<const uint32_t*>(static_cast<const uint8_t*>(p.v_cache) + off);
                    const float ks = p.k_scale[int64_t(page) * p.n_kv_heads + head];
                    const float vs = p.v_scale[int64_t(page) * p.n_kv_heads + head];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        __half_raw hk = __nv_cvt_fp8_to_halfraw((kr >> (8 * e)) & 0xff, __NV_E4M3);
                        __half_raw hv = __nv_cvt_fp8_to_halfraw((vr >> (8 * e)) & 0xff, __NV_E4M3);
                        kf[e] = __half2float(*reinterpret_cast<__half*>(&hk)) * ks;
                        vf[e] = __half2float(*reinterpret_cast<__half*>(&hv)) * vs;
                    }
                } else {
                    const uint2 kr = *reinterpret_cast<const uint2*>(static_cast<const uint8_t*>(p.k_cache) + off);
                    const uint2 vr = *reinterpret_cast<const uint2*>(static_cast<const uint8_t*>(p.v_cache) + off);
                    const __nv_bfloat162 k0 = *reinterpret_cast<const __nv_bfloat162*>(&kr.x);
                    const __nv_bfloat162 k1 = *reinterpret_cast<const __nv_bfloat162*>(&kr.y);
                    const __nv_bfloat162 v0 = *reinterpret_cast<const __nv_bfloat162*>(&vr.x);
                    const __nv_bfloat162 v1 = *reinterpret_cast<const __nv_bfloat162*>(&vr.y);
                    kf[0] = __low2float(k0); kf[1] = __high2float(k0); kf[2] = __low2float(k1); kf[3] = __high2float(k1);
                    vf[0] = __low2float(v0); vf[1] = __high2float(v0); vf[2] = __low2float(v1); vf[3] = __high2float(v1);
                }
#pragma unroll
                for (int j = 0; j < G; ++j) {
                    float s = q[j][0] * kf[0] + q[j][1] * kf[1] + q[j][2] * kf[2] + q[j][3] * kf[3];
#pragma unroll
                    for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
                    s *= p.scale_log2;
                    const float mn = fmaxf(m[j], s);
                    const float alpha = exp2f(m[j] - mn);
                    const float pr = exp2f(s - mn);
                    l[j] = l[j] * alpha + pr;
#pragma unroll
                    for (int e = 0; e < 4; ++e) o[j][e] = o[j][e] * alpha + pr * vf[e];
                    m[j] = mn;
                }
            }
        }
        // merge the four warps
        __syncthreads();
#pragma unroll
        for (int j = 0; j < G; ++j) {
            if (lane == 0) { s_m[warp][j] = m[j]; s_l[warp][j] = l[j]; }
#pragma unroll
            for (int e = 0; e < 4; ++e) s_o[warp][j][lane * 4 + e] = o[j][e];
        }
        __syncthreads();
        const bool complete = sg.t0 == 0 && sg.t1 == sg.ntiles;
        const int slot = int(blockIdx.x) * 2 + (sg.t0 > 0 ? 0 : 1);
        const int d = threadIdx.x;
        for (int j = 0; j < G; ++j) {
            float mm = fmaxf(fmaxf(s_m[0][j], s_m[1][j]), fmaxf(s_m[2][j], s_m[3][j]));
            float ll = 0.f, oo = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float a = s_m[w][j] == -INFINITY ? 0.f : exp2f(s_m[w][j] - mm);
                ll += s_l[w][j] * a;
                oo += s_o[w][j][d] * a;
            }
            if (complete) {
                p.out[(int64_t(sg.b) * p.n_q_heads + head * G + j) * kHeadDim + d] = __float2bfloat16(oo / ll);
            } else {
                p.ws_o[(int64_t(slot) * G + j) * kHeadDim + d] = oo;
                if (d == 0) {
                    p.ws_ml[(int64_t(slot) * G + j) * 2 + 0] = mm;
                    p.ws_ml[(int64_t(slot) * G + j) * 2 + 1] = ll;
                }
            }
        }
        g += sg.t1 - sg.t0;
    }
}

// =========================================================================== reduce kernel
// grid = batch * NG, 128 threads: warp w merges rows w, w + 4, ...; a lane owns 4 output dims.
__global__ void __launch_bounds__(128) decode_reduce_kernel(DecodeParams p, int rows) {
    pdl_launch_dependents();   // the next step's append may become resident; it waits for this grid itself
    pdl_wait();
    const int ng = p.n_kv_heads / p.hpc;
    const int b = blockIdx.x / ng, hg = blockIdx.x - b * ng;
    const int nt = p.prefix[b + 1] - p.prefix[b];
    if (nt == 0) return;
    const int chunk = p.header[2];
    const int s = ng * p.prefix[b] + hg * nt, e = s + nt;
    const int c0 = s / chunk, c1 = (e - 1) / chunk;
    if (c0 == c1) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = warp; r < rows; r += 4) {
        float mm = -INFINITY;
        for (int c = c0; c <= c1; ++c) {
            const int slot = c * 2 + (c == c0 ? 1 : 0);
            mm = fmaxf(mm, p.ws_ml[(int64_t(slot) * rows + r) * 2]);
        }
        float ll = 0.f;
        float4 oo = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int c = c0; c <= c1; ++c) {
            const int slot = c * 2 + (c == c0 ? 1 : 0);
            const float2 ml = *reinterpret_cast<const float2*>(p.ws_ml + (int64_t(slot) * rows + r) * 2);
            const float a = ml.x == -INFINITY ? 0.f : exp2f(ml.x - mm);
            const float4 o = *reinterpret_cast<const float4*>(p.ws_o + (int64_t(slot) * rows + r) * kHeadDim + lane * 4);
            ll += ml.y * a;
            oo.x += o.x * a; oo.y += o.y * a; oo.z += o.z * a; oo.w += o.w * a;
        }
        const float inv = 1.f / ll;
        uint2 packed;
        packed.x = pack_bf16(oo.x * inv, oo.y * inv);
        packed.y = pack_bf16(oo.z * inv, oo.w * inv);
        *reinterpret_cast<uint2*>(p.out + (int64_t(b) * p.n_q_heads + hg * rows + r) * kHeadDim + lane * 4) = packed;
    }
}

// =========================================================================== TMA kernel
constexpr int kStages = 3;
constexpr int kTileBytes = 32768;                 // K (or V) bytes per stage: 128 rows x 256 B
constexpr int kConsumerWarps = 8;
constexpr int kTmaThreads = (kConsumerWarps + 1) * 32;
constexpr int kMergeSlotFloats = 36 * 32;         // 32 accumulators + up to two maxima and two sums per lane

struct TmaSmem {
    // dynamic shared memory, 1024-byte aligned base:
    //   [kStages][2][kTileBytes] tiles | merge slots | tile prefix | scan scratch | barriers
    static constexpr int tiles = kStages * 2 * kTileBytes;
    static constexpr int merge = tiles;
    static constexpr int prefix = merge + 4 * kMergeSlotFloats * 4;
    static constexpr int scan = prefix + (kMaxBatch + 1) * 4 + 12;
    static constexpr int bars = scan + kTmaThreads * 4;
    static constexpr int total = bars + 2 * kStages * 8 + 16;
};

__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

template <int HPC>
__global__ void __launch_bounds__(kTmaThreads, 1) decode_tma_kernel(DecodeParams p,
                                                                    const __grid_constant__ CUtensorMap map_k,
                                                                    const __grid_constant__ CUtensorMap map_v) {
    constexpr int TT = 128 / HPC;          // tokens per tile
    constexpr int WPH = kConsumerWarps / HPC;   // consumer warps per kv head
    constexpr int SUB = TT * 128;          // bytes of one (head, half) sub-tile
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* s_merge = reinterpret_cast<float*>(smem + TmaSmem::merge);
    int* s_tp = reinterpret_cast<int*>(smem + TmaSmem::prefix);
    int* s_scan = reinterpret_cast<int*>(smem + TmaSmem::scan);
    uint64_t* s_bar = reinterpret_cast<uint64_t*>(smem + TmaSmem::bars);
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
    build_tile_prefix(p.context_lens, p.batch, TT, s_tp, s_scan);   // ends with __syncthreads
    // Everything above only reads step metadata; the pools and q may still be written by the
    // kernel in front of this one (the append) when this kernel was launched programmatically.
    pdl_launch_dependents();
    pdl_wait();

    const int ng = p.n_kv_heads / HPC;
    const int total = ng * s_tp[p.batch];
    const int chunk = max(1, (total + int(gridDim.x) - 1) / int(gridDim.x));
    if (blockIdx.x == 0) {
        for (int i = threadIdx.x; i <= p.batch; i += blockDim.x) p.prefix[i] = s_tp[i];
        if (threadIdx.x == 0) {
            p.header[1] = total;
            p.header[2] = chunk;
            p.header[3] = gridDim.x;
        }
    }
    const int lo = min(total, int(blockIdx.x) * chunk), hi = min(total, lo + chunk);

    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------ producer
        if (lane != 0) return;
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        uint32_t it = 0;
        bool ok = true;
        for (int g = lo; g < hi && ok;) {
            const Segment sg = locate_segment(s_tp, p.batch, ng, g, hi);
            const int32_t* table = p.block_tables + int64_t(sg.b) * p.bt_stride;
            for (int t = sg.t0; t < sg.t1; ++t, ++it) {
                const uint32_t s = it % kStages, ph = (it / kStages) & 1;
                if (!mbar_wait(empty0 + s * 8, ph ^ 1)) { ok = false; break; }
                const int tok0 = t * TT;
                const int page = table[tok0 / p.block_size];
                const int slot0 = page * p.block_size + tok0 % p.block_size;
                const uint32_t bar = full0 + s * 8;
                const uint32_t kdst = tiles_u32 + s * (2 * kTileBytes), vdst = kdst + kTileBytes;
                mbar_expect_tx(bar, 2 * kTileBytes);
#pragma unroll
                for (int hl = 0; hl < HPC; ++hl) {
                    const int head = sg.hg * HPC + hl;
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        tma_load_3d(kdst + (hl * 2 + half) * SUB, &map_k, bar, half * 64, head, slot0);
                        tma_load_3d(vdst + (hl * 2 + half) * SUB, &map_v, bar, half * 64, head, slot0);
                    }
                }
            }
            g += sg.t1 - sg.t0;
        }
        // Do not leave while a copy may still be in flight: wait for the last armed stages.
        const uint32_t armed = it < uint32_t(kStages) ? it : uint32_t(kStages);
        for (uint32_t j = 0; j < armed; ++j) {
            const uint32_t i2 = it - 1 - j;
            if (!mbar_wait(full0 + (i2 % kStages) * 8, (i2 / kStages) & 1)) ok = false;
        }
        if (!ok) atomicExch(p.header, kStatusMagic | 1);
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
        const Segment sg = locate_segment(s_tp, p.batch, ng, g, hi);
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

        for (int t = sg.t0; t < sg.t1; ++t, ++it) {
            const uint32_t s = it % kStages, ph = (it / kStages) & 1;
            if (ok && !mbar_wait(full0 + s * 8, ph)) ok = false;
            const int tok_w = t * TT + tw * 16;            // first token of this warp's 16
            const int valid = ctx - tok_w;                  // tokens of the 16 that exist
            if (ok && valid > 0) {
                const uint32_t kbase = tiles_u32 + s * (2 * kTileBytes) + (hl * 2) * SUB;
                const uint32_t vbase = kbase + kTileBytes;
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

        // tree merge of the WPH warps that share a kv head
        if (WPH > 1) {
#pragma unroll
            for (int stride = WPH / 2; stride >= 1; stride >>= 1) {
                float* slot = s_merge + (hl * stride + (tw % stride)) * kMergeSlotFloats;
                if (tw >= stride && tw < 2 * stride) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        slot[(2 * j) * 32 + lane] = o[j][0];
                        slot[(2 * j + 1) * 32 + lane] = o[j][1];
                    }
                    slot[32 * 32 + lane] = m_run;
                    slot[33 * 32 + lane] = l_run;
                }
                consumer_bar();
                if (tw < stride) {
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
                }
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
        g += sg.t1 - sg.t0;
    }
    if (!ok && lane == 0) atomicExch(p.header, kStatusMagic | 2);
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
    static constexpr int total = meta + kStages * HPC * 8;
};

template <int HPC>
__global__ void __launch_bounds__(kTmaThreads, 1) decode_tma_fp8_kernel(DecodeParams p,
                                                                          const __grid_constant__ CUtensorMap map_k,
                                                                          const __grid_constant__ CUtensorMap map_v) {
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
    build_tile_prefix(p.context_lens, p.batch, TT, s_tp, s_scan);
    pdl_launch_dependents();
    pdl_wait();

    const int ng = p.n_kv_heads / HPC;
    const int total = ng * s_tp[p.batch];
    const int chunk = max(1, (total + int(gridDim.x) - 1) / int(gridDim.x));
    if (blockIdx.x == 0) {
        for (int i = threadIdx.x; i <= p.batch; i += blockDim.x) p.prefix[i] = s_tp[i];
        if (threadIdx.x == 0) {
            p.header[1] = total;
            p.header[2] = chunk;
            p.header[3] = gridDim.x;
        }
    }
    const int lo = min(total, int(blockIdx.x) * chunk), hi = min(total, lo + chunk);

    if (warp == W) {
        // ------------------------------------------------------------ producer
        if (lane != 0) return;
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        uint32_t it = 0;
        bool ok = true;
        for (int g = lo; g < hi && ok;) {
            const Segment sg = locate_segment(s_tp, p.batch, ng, g, hi);
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
                if (!mbar_wait(empty0 + s * 8, ph ^ 1)) { ok = false; break; }
#pragma unroll
                for (int hl = 0; hl < HPC; ++hl) {
                    s_meta[(s * HPC + hl) * 2 + 0] = ks[hl];
                    s_meta[(s * HPC + hl) * 2 + 1] = vs[hl];
                }
                const uint32_t bar = full0 + s * 8;
                const uint32_t kdst = tiles_u32 + s * (2 * kTileBytes), vdst = kdst + kTileBytes;
                mbar_expect_tx(bar, 2 * kTileBytes);      // release: the scales above are visible to the waiters
#pragma unroll
                for (int hl = 0; hl < HPC; ++hl) {        // the heads' boxes back to back: adjacent lines of every token row
                    tma_load_3d(kdst + hl * kHeadBytes, &map_k, bar, 0, sg.hg * HPC + hl, slot0);
                    tma_load_3d(vdst + hl * kHeadBytes, &map_v, bar, 0, sg.hg * HPC + hl, slot0);
                }
            }
            g += sg.t1 - sg.t0;
        }
        const uint32_t armed = it < uint32_t(kStages) ? it : uint32_t(kStages);
        for (uint32_t j = 0; j < armed; ++j) {
            const uint32_t i2 = it - 1 - j;
            if (!mbar_wait(full0 + (i2 % kStages) * 8, (i2 / kStages) & 1)) ok = false;
        }
        if (!ok) atomicExch(p.header, kStatusMagic | 1);
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
        const Segment sg = locate_segment(s_tp, p.batch, ng, g, hi);
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
            if (ok && !mbar_wait(full0 + s * 8, ph)) ok = false;
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
        g += sg.t1 - sg.t0;
    }
    if (!ok && lane == 0) atomicExch(p.header, kStatusMagic | 2);
}

// =========================================================================== host side
struct DecodeConfig {
    int impl;   // 1 = simple, 2 = tma
    int hpc;
    int tile_tokens;
    int grid;
    int rows;   // partial rows per scratch slot
};

static void set_cuda_error_if(cudaError_t e) {
    if (e != cudaSuccess) set_cuda_error(e);
}

static int env_int(const char* name, int dflt) {
    const char* s = std::getenv(name);
    return s && *s ? std::atoi(s) : dflt;
}

// ws_limit: bytes of scratch the caller has (0 = no limit); the e4m3 kernel takes fewer heads per tile
// when the partial-result slots of more would not fit.
static DecodeConfig decode_config(const infer_kv_pool* pool, int n_q_heads, size_t ws_limit = 0) {
    DecodeConfig c;
    const int group = n_q_heads / pool->n_kv_heads;
    c.impl = 2;
    const int forced = env_int("INFER_B200_DECODE_IMPL", 0);   // development switch: 1 = plain-load kernel
    if (forced == 1 || forced == 2) c.impl = forced;
    if (c.impl == 2 && pool->dtype == INFER_KV_E4M3) {
        // several adjacent heads per tile when the head count allows: their boxes fetch neighbouring lines
        // (measured on 8 heads: 1 head 111 us, 2 heads 98.7, 4 heads 96.5, 8 heads 105)
        c.hpc = pool->n_kv_heads % 4 == 0 ? 4 : (pool->n_kv_heads % 2 == 0 ? 2 : 1);
        const int want8 = env_int("INFER_B200_FP8_HPC", 0);         // development switch
        if ((want8 == 1 || want8 == 2 || want8 == 4 || want8 == 8) && pool->n_kv_heads % want8 == 0) c.hpc = want8;
        while (ws_limit && c.hpc > 1 && decode_layout(pool->sm_count, c.hpc * group).total > ws_limit) c.hpc /= 2;
        c.tile_tokens = kFp8TileTokens / c.hpc;
        c.grid = pool->sm_count;
    } else if (c.impl == 2) {
        // One kv head per tile (128 tokens x 256 B rows) measured fastest at every head count:
        // fewer, larger TMA boxes beat streaming all heads of a token row together.
        int hpc = 1;
        const int want = env_int("INFER_B200_DECODE_HPC", 0);
        if ((want == 1 || want == 2 || want == 4 || want == 8) && pool->n_kv_heads % want == 0) hpc = want;
        c.hpc = hpc;
        c.tile_tokens = 128 / hpc;
        c.grid = pool->sm_count;
    } else {
        c.hpc = 1;
        c.tile_tokens = 64;
        c.grid = pool->sm_count * 8;
    }
    c.rows = c.hpc * group;
    return c;
}

template <int G, bool FP8>
static void launch_simple(const DecodeParams& p, int grid, cudaStream_t st) {
    set_cuda_error_if(launch_pdl(decode_simple_kernel<G, FP8>, dim3(grid), dim3(128), 0, st, p));
}

template <int HPC>
static int launch_tma(const DecodeParams& p, const infer_kv_pool* pool, int grid, cudaStream_t st) {
    int idx = 0;
    while ((16 << idx) != 128 / HPC) ++idx;
    const int smem = TmaSmem::total + 1024;
    IB_CUDA(cudaFuncSetAttribute(decode_tma_kernel<HPC>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    IB_CUDA(launch_pdl(decode_tma_kernel<HPC>, dim3(grid), dim3(kTmaThreads), smem, st, p, pool->maps[idx].k,
                       pool->maps[idx].v));
    return INFER_OK;
}

}  // namespace ib

extern "C" {

size_t infer_paged_decode_workspace_bytes(const infer_kv_pool_t* pool, int batch, int n_q_heads) {
    (void)batch;
    if (!pool || n_q_heads <= 0 || n_q_heads % pool->n_kv_heads != 0) return 0;
    // sized for either kernel so that a development switch never outgrows the buffer
    const int group = n_q_heads / pool->n_kv_heads;
    const size_t a = ib::decode_layout(pool->sm_count, 8 * group).total;
    const size_t b = ib::decode_layout(pool->sm_count * 8, group).total;
    return a > b ? a : b;
}

int infer_paged_decode(const infer_kv_pool_t* pool, void* out, const void* q, const int32_t* context_lens,
                       const int32_t* block_tables, int64_t bt_stride, int batch, int n_q_heads,
                       float softmax_scale, void* workspace, size_t workspace_bytes, void* stream_) {
    using namespace ib;
    if (!pool || !out || !q || !context_lens || !block_tables) return INFER_ERR_NULL;
    if (batch < 0 || batch > kMaxBatch || n_q_heads <= 0 || n_q_heads % pool->n_kv_heads != 0 || bt_stride <= 0)
        return INFER_ERR_GEOMETRY;
    const int group = n_q_heads / pool->n_kv_heads;
    if (group > kMaxGroup || (group & (group - 1)) != 0) return INFER_ERR_GEOMETRY;
    if (!aligned16(out) || !aligned16(q)) return INFER_ERR_ALIGN;
    if (batch == 0) return INFER_OK;
    const DecodeConfig cfg = decode_config(pool, n_q_heads, workspace_bytes);
    const DecodeLayout lay = decode_layout(cfg.grid, cfg.rows);
    if (!workspace || !aligned16(workspace) || workspace_bytes < lay.total) return INFER_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream_);

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
    p.hpc = cfg.hpc;
    p.tile_tokens = cfg.tile_tokens;
    p.scale_log2 = softmax_scale * 1.4426950408889634f;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    p.header = reinterpret_cast<int*>(ws + lay.header_off);
    p.prefix = reinterpret_cast<int*>(ws + lay.prefix_off);
    p.ws_ml = reinterpret_cast<float*>(ws + lay.ml_off);
    p.ws_o = reinterpret_cast<float*>(ws + lay.o_off);

    if (cfg.impl == 2 && pool->dtype == INFER_KV_E4M3) {
        if (cfg.hpc == 8 || cfg.hpc == 4) {
            const int mi = cfg.hpc == 8 ? 1 : 2;
            if (cfg.hpc == 8) {
                const int smem_t = Fp8Smem<8>::total + 1024;
                IB_CUDA(cudaFuncSetAttribute(decode_tma_fp8_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_t));
                IB_CUDA(launch_pdl(decode_tma_fp8_kernel<8>, dim3(cfg.grid), dim3(kTmaThreads), smem_t, st, p, pool->maps[mi].k,
                                   pool->maps[mi].v));
            } else {
                const int smem_t = Fp8Smem<4>::total + 1024;
                IB_CUDA(cudaFuncSetAttribute(decode_tma_fp8_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_t));
                IB_CUDA(launch_pdl(decode_tma_fp8_kernel<4>, dim3(cfg.grid), dim3(kTmaThreads), smem_t, st, p, pool->maps[mi].k,
                                   pool->maps[mi].v));
            }
        } else if (cfg.hpc == 2) {
            const int smem_t = Fp8Smem<2>::total + 1024;
            IB_CUDA(cudaFuncSetAttribute(decode_tma_fp8_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_t));
            IB_CUDA(launch_pdl(decode_tma_fp8_kernel<2>, dim3(cfg.grid), dim3(kTmaThreads), smem_t, st, p, pool->maps[3].k,
                               pool->maps[3].v));
        } else {
            const int smem_t = Fp8Smem<1>::total + 1024;
            IB_CUDA(cudaFuncSetAttribute(decode_tma_fp8_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_t));
            IB_CUDA(launch_pdl(decode_tma_fp8_kernel<1>, dim3(cfg.grid), dim3(kTmaThreads), smem_t, st, p, pool->maps[4].k,
                               pool->maps[4].v));
        }
    } else if (cfg.impl == 2) {
        int rc = INFER_OK;
        switch (cfg.hpc) {
            case 1: rc = launch_tma<1>(p, pool, cfg.grid, st); break;
            case 2: rc = launch_tma<2>(p, pool, cfg.grid, st); break;
            case 4: rc = launch_tma<4>(p, pool, cfg.grid, st); break;
            default: rc = launch_tma<8>(p, pool, cfg.grid, st); break;
        }
        if (rc != INFER_OK) return rc;
    } else {
        const bool fp8 = pool->dtype == INFER_KV_E4M3;
#define IB_SIMPLE(G) (fp8 ? launch_simple<G, true>(p, cfg.grid, st) : launch_simple<G, false>(p, cfg.grid, st))
        switch (group) {
            case 1: IB_SIMPLE(1); break;
            case 2: IB_SIMPLE(2); break;
            case 4: IB_SIMPLE(4); break;
            default: IB_SIMPLE(8); break;
        }
#undef IB_SIMPLE
    }
    int rc = check_launch();
    if (rc != INFER_OK) return rc;
    IB_CUDA(launch_pdl(decode_reduce_kernel, dim3(batch * (pool->n_kv_heads / cfg.hpc)), dim3(128), 0, st, p, cfg.rows));
    return check_launch();
}

int infer_paged_decode_status(const void* workspace, void* stream_) {
    if (!workspace) return INFER_ERR_NULL;
    int word = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream_);
    IB_CUDA(cudaMemcpyAsync(&word, workspace, sizeof(int), cudaMemcpyDeviceToHost, st));
    IB_CUDA(cudaStreamSynchronize(st));
    return (word & 0xFFFF0000) == ib::kStatusMagic ? INFER_ERR_DEVICE : INFER_OK;
}

// ------------------------------------------------------------------ entry point without scratch
namespace ib {

// Scratch of infer_paged_decode_noalloc: lives in the library's device image, one copy per
// GPU that loads the library.  In host code the NAME below is only a handle for
// cudaGetSymbolAddress; kernels must be given the address that call returns.
constexpr size_t kBuiltinScratchBytes = size_t(2) << 20;
static __device__ __align__(256) unsigned char g_builtin_scratch[kBuiltinScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_builtin_scratch_addr[kMaxDevices];   // device address per device ordinal, 0 = not looked up yet
static std::mutex g_builtin_scratch_mutex;

}  // namespace ib

int infer_paged_decode_noalloc(const infer_kv_pool_t* pool, void* out, const void* q, const int32_t* context_lens,
                               const int32_t* block_tables, int64_t bt_stride, int batch, int n_q_heads,
                               float softmax_scale, void* stream_) {
    using namespace ib;
    if (!pool || !out || !q || !context_lens || !block_tables) return INFER_ERR_NULL;
    if (n_q_heads <= 0 || n_q_heads % pool->n_kv_heads != 0 || batch < 0) return INFER_ERR_GEOMETRY;
    if (batch > kMaxBatch) return INFER_ERR_TOO_LARGE;
    const DecodeConfig cfg = decode_config(pool, n_q_heads, kBuiltinScratchBytes);
    if (decode_layout(cfg.grid, cfg.rows).total > kBuiltinScratchBytes) return INFER_ERR_TOO_LARGE;

    int dev = -1;
    IB_CUDA(cudaGetDevice(&dev));
    if (dev != pool->device || dev < 0 || dev >= kMaxDevices) {
        set_cuda_error(cudaErrorInvalidDevice);
        return INFER_ERR_CUDA;
    }
    void* scratch = nullptr;
    {
        // once per device, with that device current: resolve the array's device address
        std::lock_guard<std::mutex> lock(g_builtin_scratch_mutex);
        if (!g_builtin_scratch_addr[dev]) {
            void* addr = nullptr;
            IB_CUDA(cudaGetSymbolAddress(&addr, g_builtin_scratch));
            g_builtin_scratch_addr[dev] = addr;
        }
        scratch = g_builtin_scratch_addr[dev];
    }
    // the array keeps the previous call's bytes: the status word has to start at zero
    IB_CUDA(cudaMemsetAsync(scratch, 0, 64, static_cast<cudaStream_t>(stream_)));
    return infer_paged_decode(pool, out, q, context_lens, block_tables, bt_stride, batch, n_q_heads, softmax_scale,
                              scratch, kBuiltinScratchBytes, stream_);
}

}  // extern "C"
