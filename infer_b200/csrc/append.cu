// KV append: scatter new k/v rows through slot_mapping into the page pools.
//
// bf16 pools: a pure byte copy, one 16-byte load and one 16-byte store per thread and
// row chunk, K and V in the same thread, two chunks in flight per thread.
// e4m3 pools: four kernels (snapshot scales, raise scales by the new rows' amax,
// re-encode pages whose scale grew, write the new rows) so that the result depends on no
// scheduling order and matches the CPU oracle bit for bit.  The three row kernels work on
// strips of 8 tokens per warp: 16-byte loads, 8 in flight per lane, one atomic per run of
// tokens that share a page.
#include "common.cuh"

namespace ib {

// --------------------------------------------------------------------------- bf16
__global__ void __launch_bounds__(256) append_bf16_kernel(
    const uint4* __restrict__ k, const uint4* __restrict__ v, int64_t k_pitch16, int64_t v_pitch16,
    uint4* __restrict__ k_cache, uint4* __restrict__ v_cache, const int32_t* __restrict__ slot_mapping,
    int64_t n_tokens, int chunks, int64_t num_slots) {
    pdl_launch_dependents();   // an attention kernel behind this one may run its prologue already
    pdl_wait();                // launched programmatically itself: the kernel in front may still be reading the pools
    const int64_t total = n_tokens * chunks;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t u0 = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; u0 < total; u0 += 2 * stride) {
        const int64_t u1 = u0 + stride;
        const bool has1 = u1 < total;
        const int64_t t0 = u0 / chunks, t1 = has1 ? u1 / chunks : t0;
        const int c0 = int(u0 - t0 * chunks), c1 = has1 ? int(u1 - t1 * chunks) : c0;
        const int64_t s0 = slot_mapping[t0];
        const int64_t s1 = slot_mapping[t1];
        const bool ok0 = s0 >= 0 && s0 < num_slots;
        const bool ok1 = has1 && s1 >= 0 && s1 < num_slots;
        uint4 ka, va, kb, vb;
        if (ok0) {
            ka = __ldg(k + t0 * k_pitch16 + c0);
            va = __ldg(v + t0 * v_pitch16 + c0);
        }
        if (ok1) {
            kb = __ldg(k + t1 * k_pitch16 + c1);
            vb = __ldg(v + t1 * v_pitch16 + c1);
        }
        if (ok0) {
            k_cache[s0 * chunks + c0] = ka;
            v_cache[s0 * chunks + c0] = va;
        }
        if (ok1) {
            k_cache[s1 * chunks + c1] = kb;
            v_cache[s1 * chunks + c1] = vb;
        }
    }
}

// --------------------------------------------------------------------------- e4m3
struct Fp8Args {
    const __nv_bfloat16* src[2];   // k, v
    int64_t pitch[2];              // elements
    uint8_t* cache[2];
    float* scale[2];
    float* snap[2];                // workspace copies of the scales of touched pages
    const int32_t* slot_mapping;
    int64_t n_tokens;
    int64_t num_slots;
    int n_kv_heads;
    int block_size;
};

__device__ __forceinline__ bool fp8_locate(const Fp8Args& a, int64_t item, int& which, int64_t& tok, int& head,
                                           int64_t& slot) {
    // item = (tok * Hkv + head) * 2 + which
    which = int(item & 1);
    const int64_t th = item >> 1;
    tok = th / a.n_kv_heads;
    head = int(th - tok * a.n_kv_heads);
    slot = a.slot_mapping[tok];
    return slot >= 0 && slot < a.num_slots;
}

__global__ void fp8_snapshot_kernel(Fp8Args a) {
    const int64_t item = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (item >= a.n_tokens * a.n_kv_heads * 2) return;
    int which, head;
    int64_t tok, slot;
    if (!fp8_locate(a, item, which, tok, head, slot)) return;
    const int64_t e = (slot / a.block_size) * a.n_kv_heads + head;
    a.snap[which][e] = a.scale[which][e];
}

// Work unit of the three row kernels below: kStrip consecutive tokens x (k|v) x a pair of KV
// heads.  One warp per unit: lane / 16 picks the head of the pair, lane % 16 the 16-byte chunk
// of its 128-element row, so a warp reads 512 contiguous bytes per token and keeps kStrip
// loads in flight per lane.  Consecutive tokens mostly share a page, which lets the half-warp
// issue one atomic (amax) or one claim test (rescale) per run of equal pages, not per row.
constexpr int kStrip = 8;

struct StripUnit {
    int which, head, sub;
    int64_t tok0;
    bool active;
};

__device__ __forceinline__ int64_t strip_units(const Fp8Args& a) {
    return ((a.n_tokens + kStrip - 1) / kStrip) * 2 * ((a.n_kv_heads + 1) / 2);
}

__device__ __forceinline__ StripUnit strip_locate(const Fp8Args& a, int64_t unit, int lane) {
    const int pairs = (a.n_kv_heads + 1) / 2;
    StripUnit u;
    u.which = int(unit & 1);
    const int64_t sp = unit >> 1;
    const int64_t strip = sp / pairs;
    u.head = int(sp - strip * pairs) * 2 + (lane >> 4);
    u.sub = lane & 15;
    u.tok0 = strip * kStrip;
    u.active = u.head < a.n_kv_heads;
    return u;
}

__device__ __forceinline__ float amax8(const uint4& r) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        // a bf16 is the upper half of the fp32 with the same value
        m = fmaxf(m, fmaxf(fabsf(__uint_as_float(w[i] << 16)), fabsf(__uint_as_float(w[i] & 0xffff0000u))));
    }
    return m;
}

// scale[page, head] = max(scale, amax(rows of this call on that page) / 448)
__global__ void __launch_bounds__(256) fp8_amax_kernel(Fp8Args a) {
    const int64_t unit = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (unit >= strip_units(a)) return;
    const int lane = threadIdx.x & 31;
    const StripUnit u = strip_locate(a, unit, lane);
    int64_t page[kStrip];
    uint4 raw[kStrip];
#pragma unroll
    for (int t = 0; t < kStrip; ++t) {
        const int64_t tok = u.tok0 + t;
        int64_t slot = -1;
        if (tok < a.n_tokens) slot = a.slot_mapping[tok];
        const bool ok = u.active && slot >= 0 && slot < a.num_slots;
        page[t] = ok ? slot / a.block_size : -1;
        raw[t] = make_uint4(0, 0, 0, 0);
        if (ok) raw[t] = __ldg(reinterpret_cast<const uint4*>(a.src[u.which] + tok * a.pitch[u.which] + u.head * kHeadDim) + u.sub);
    }
    float m[kStrip];
#pragma unroll
    for (int t = 0; t < kStrip; ++t) {
        m[t] = amax8(raw[t]);
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) m[t] = fmaxf(m[t], __shfl_xor_sync(0xffffffffu, m[t], o));
    }
    if (u.sub != 0 || !u.active) return;
    int64_t cur = -1;
    float best = 0.0f;
#pragma unroll
    for (int t = 0; t <= kStrip; ++t) {
        const int64_t p = t < kStrip ? page[t] : -2;
        if (p != cur) {
            if (cur >= 0)   // non-negative floats order like their bit patterns
                atomicMax(reinterpret_cast<int*>(a.scale[u.which] + cur * a.n_kv_heads + u.head),
                          __float_as_int(__fdiv_rn(best, 448.0f)));
            cur = p;
            best = 0.0f;
        }
        if (t < kStrip) best = fmaxf(best, m[t]);
    }
}

__device__ __forceinline__ uint32_t rescale4(uint32_t q, float ratio) {
    uint32_t out = 0;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>((q >> (16 * i)) & 0xffff), __NV_E4M3);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
        out |= uint32_t(__nv_cvt_float2_to_fp8x2(make_float2(__fmul_rn(f.x, ratio), __fmul_rn(f.y, ratio)),
                                                 __NV_SATFINITE, __NV_E4M3)) << (16 * i);
    }
    return out;
}

// The first half-warp to claim a (page, head) whose scale grew re-encodes all of that page's
// rows for that head (rare: most half-warps leave after two loads per distinct page).
__global__ void __launch_bounds__(256) fp8_rescale_kernel(Fp8Args a) {
    const int64_t unit = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (unit >= strip_units(a)) return;
    const int lane = threadIdx.x & 31;
    const StripUnit u = strip_locate(a, unit, lane);
    const unsigned half_mask = 0xffffu << (lane & 16);
    int64_t cur = -1;
    for (int t = 0; t < kStrip; ++t) {
        const int64_t tok = u.tok0 + t;
        int64_t slot = -1;
        if (tok < a.n_tokens) slot = a.slot_mapping[tok];
        const bool ok = u.active && slot >= 0 && slot < a.num_slots;
        const int64_t page = ok ? slot / a.block_size : -1;
        if (page == cur || page < 0) continue;        // uniform within the half-warp
        cur = page;
        const int64_t e = page * a.n_kv_heads + u.head;
        float ratio = -1.0f;
        if (u.sub == 0) {
            const float now = a.scale[u.which][e];
            const float seen = a.snap[u.which][e];
            if (seen > 0.0f && now > seen) {                       // a candidate: claim it exactly once
                const float old = atomicExch(a.snap[u.which] + e, -1.0f);
                if (old > 0.0f) ratio = __fdiv_rn(old, now);
            }
        }
        ratio = __shfl_sync(half_mask, ratio, lane & 16);
        if (ratio < 0.0f) continue;
        // rows of this head: block_size rows of 128 bytes, pitch Hkv * 128
        uint8_t* base = a.cache[u.which] + (page * a.block_size * a.n_kv_heads + u.head) * int64_t(kHeadDim);
        const int64_t pitch = int64_t(a.n_kv_heads) * kHeadDim;
        for (int i = u.sub; i < a.block_size * 8; i += 16) {
            uint4* p = reinterpret_cast<uint4*>(base + (i >> 3) * pitch + (i & 7) * 16);
            uint4 q = *p;
            q.x = rescale4(q.x, ratio);
            q.y = rescale4(q.y, ratio);
            q.z = rescale4(q.z, ratio);
            q.w = rescale4(q.w, ratio);
            *p = q;
        }
    }
}

// quantise the new rows with their page's final scale
__global__ void __launch_bounds__(256) fp8_write_kernel(Fp8Args a) {
    const int64_t unit = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (unit >= strip_units(a)) return;
    const int lane = threadIdx.x & 31;
    const StripUnit u = strip_locate(a, unit, lane);
    if (!u.active) return;
    int64_t slot[kStrip];
    uint4 raw[kStrip];
    float s[kStrip];
#pragma unroll
    for (int t = 0; t < kStrip; ++t) {
        const int64_t tok = u.tok0 + t;
        slot[t] = -1;
        if (tok < a.n_tokens) slot[t] = a.slot_mapping[tok];
        if (slot[t] >= a.num_slots) slot[t] = -1;
        raw[t] = make_uint4(0, 0, 0, 0);
        s[t] = 0.0f;
        if (slot[t] >= 0) {
            raw[t] = __ldg(reinterpret_cast<const uint4*>(a.src[u.which] + tok * a.pitch[u.which] + u.head * kHeadDim) + u.sub);
            s[t] = a.scale[u.which][(slot[t] / a.block_size) * a.n_kv_heads + u.head];
        }
    }
#pragma unroll
    for (int t = 0; t < kStrip; ++t) {
        if (slot[t] < 0) continue;
        const uint32_t w[4] = {raw[t].x, raw[t].y, raw[t].z, raw[t].w};
        uint32_t out[2] = {0, 0};
        if (s[t] > 0.0f) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float lo = __fdiv_rn(__uint_as_float(w[i] << 16), s[t]);
                const float hi = __fdiv_rn(__uint_as_float(w[i] & 0xffff0000u), s[t]);
                out[i >> 1] |= uint32_t(__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3)) << (16 * (i & 1));
            }
        }
        *reinterpret_cast<uint2*>(a.cache[u.which] + (slot[t] * a.n_kv_heads + u.head) * int64_t(kHeadDim) + u.sub * 8) =
            make_uint2(out[0], out[1]);
    }
}

}  // namespace ib

extern "C" {

size_t infer_kv_append_workspace_bytes(const infer_kv_pool_t* pool) {
    if (!pool || pool->dtype != INFER_KV_E4M3) return 0;
    return size_t(2) * pool->num_blocks * pool->n_kv_heads * sizeof(float);
}

int infer_kv_append(const infer_kv_pool_t* pool, const void* k, const void* v, int64_t k_row_stride,
                    int64_t v_row_stride, const int32_t* slot_mapping, int64_t n_tokens, void* workspace,
                    size_t workspace_bytes, void* stream_) {
    if (!pool) return INFER_ERR_NULL;
    if (n_tokens < 0) return INFER_ERR_GEOMETRY;
    if (n_tokens == 0) return INFER_OK;
    if (!k || !v || !slot_mapping) return INFER_ERR_NULL;
    const int64_t row = int64_t(pool->n_kv_heads) * ib::kHeadDim;
    if (k_row_stride < row || v_row_stride < row) return INFER_ERR_STRIDE;
    if (!ib::aligned16(k) || !ib::aligned16(v) || k_row_stride % 8 || v_row_stride % 8) return INFER_ERR_ALIGN;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);

    if (pool->dtype == INFER_KV_BF16) {
        const int chunks = int(row * 2 / 16);
        const int64_t total = n_tokens * chunks;
        int64_t blocks = (total + 511) / 512;   // two chunks per thread
        const int64_t cap = int64_t(pool->sm_count) * 32;
        if (blocks > cap) blocks = cap;
        // programmatic launch: the CTAs may become resident while the previous kernel drains
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(unsigned(blocks));
        cfg.blockDim = dim3(256);
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        IB_CUDA(cudaLaunchKernelEx(&cfg, ib::append_bf16_kernel, static_cast<const uint4*>(k), static_cast<const uint4*>(v),
                                   int64_t(k_row_stride / 8), int64_t(v_row_stride / 8), static_cast<uint4*>(pool->k_cache),
                                   static_cast<uint4*>(pool->v_cache), slot_mapping, n_tokens, chunks, pool->num_slots));
        return ib::check_launch();
    }

    const size_t need = infer_kv_append_workspace_bytes(pool);
    if (!workspace || workspace_bytes < need || !ib::aligned16(workspace)) return INFER_ERR_WORKSPACE;
    ib::Fp8Args a;
    a.src[0] = static_cast<const __nv_bfloat16*>(k);
    a.src[1] = static_cast<const __nv_bfloat16*>(v);
    a.pitch[0] = k_row_stride;
    a.pitch[1] = v_row_stride;
    a.cache[0] = static_cast<uint8_t*>(pool->k_cache);
    a.cache[1] = static_cast<uint8_t*>(pool->v_cache);
    a.scale[0] = pool->k_scale;
    a.scale[1] = pool->v_scale;
    a.snap[0] = static_cast<float*>(workspace);
    a.snap[1] = a.snap[0] + pool->num_blocks * pool->n_kv_heads;
    a.slot_mapping = slot_mapping;
    a.n_tokens = n_tokens;
    a.num_slots = pool->num_slots;
    a.n_kv_heads = pool->n_kv_heads;
    a.block_size = pool->block_size;
    const int64_t items = n_tokens * pool->n_kv_heads * 2;
    if (items >= (int64_t(1) << 31)) return INFER_ERR_GEOMETRY;
    ib::fp8_snapshot_kernel<<<unsigned((items + 255) / 256), 256, 0, stream>>>(a);
    const int64_t units = ((n_tokens + ib::kStrip - 1) / ib::kStrip) * 2 * ((pool->n_kv_heads + 1) / 2);
    const unsigned strip_blocks = unsigned((units * 32 + 255) / 256);
    ib::fp8_amax_kernel<<<strip_blocks, 256, 0, stream>>>(a);
    ib::fp8_rescale_kernel<<<strip_blocks, 256, 0, stream>>>(a);
    ib::fp8_write_kernel<<<strip_blocks, 256, 0, stream>>>(a);
    return ib::check_launch();
}

}  // extern "C"
