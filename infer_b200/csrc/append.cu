// KV append: scatter new k/v rows through slot_mapping into the page pools.
//
// bf16 pools: a pure byte copy, one 16-byte load and one 16-byte store per thread and
// row chunk, K and V in the same thread, two chunks in flight per thread.
// e4m3 pools: four small kernels (snapshot scales, raise scales by the new rows' amax,
// re-encode pages whose scale grew, write the new rows) so that the result depends on no
// scheduling order and matches the CPU oracle bit for bit.
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

// one warp per (token, head, k|v): scale = max(scale, amax(row) / 448)
__global__ void fp8_amax_kernel(Fp8Args a) {
    const int64_t item = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (item >= a.n_tokens * a.n_kv_heads * 2) return;
    const int lane = threadIdx.x & 31;
    int which, head;
    int64_t tok, slot;
    if (!fp8_locate(a, item, which, tok, head, slot)) return;
    const uint2 raw = *reinterpret_cast<const uint2*>(a.src[which] + tok * a.pitch[which] + head * kHeadDim + lane * 4);
    const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    float m = fmaxf(fmaxf(fabsf(__low2float(p0)), fabsf(__high2float(p0))),
                    fmaxf(fabsf(__low2float(p1)), fabsf(__high2float(p1))));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) {
        const float s = __fdiv_rn(m, 448.0f);
        // non-negative floats order like their bit patterns
        atomicMax(reinterpret_cast<int*>(a.scale[which] + (slot / a.block_size) * a.n_kv_heads + head),
                  __float_as_int(s));
    }
}

__device__ __forceinline__ uint32_t rescale4(uint32_t q, float ratio) {
    uint32_t out = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>((q >> (8 * i)) & 0xff), __NV_E4M3);
        const float x = __fmul_rn(__half2float(*reinterpret_cast<const __half*>(&h)), ratio);
        out |= uint32_t(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3)) << (8 * i);
    }
    return out;
}

// one warp per (token, head, k|v); the first warp to claim a page/head whose scale grew
// re-encodes all of that page's rows for that head (rare: most warps leave after two loads).
__global__ void __launch_bounds__(256) fp8_rescale_kernel(Fp8Args a) {
    const int64_t item = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (item >= a.n_tokens * a.n_kv_heads * 2) return;
    const int lane = threadIdx.x & 31;
    int which, head;
    int64_t tok, slot;
    if (!fp8_locate(a, item, which, tok, head, slot)) return;
    const int64_t page = slot / a.block_size;
    const int64_t e = page * a.n_kv_heads + head;
    float ratio = -1.0f;
    if (lane == 0) {
        const float now = a.scale[which][e];
        const float seen = a.snap[which][e];
        if (seen > 0.0f && now > seen) {                       // a candidate: claim it exactly once
            const float old = atomicExch(a.snap[which] + e, -1.0f);
            if (old > 0.0f) ratio = __fdiv_rn(old, now);
        }
    }
    ratio = __shfl_sync(0xffffffffu, ratio, 0);
    if (ratio < 0.0f) return;
    // rows of this head: block_size rows of 128 bytes, pitch Hkv * 128
    uint8_t* base = a.cache[which] + (page * a.block_size * a.n_kv_heads + head) * int64_t(kHeadDim);
    const int64_t pitch = int64_t(a.n_kv_heads) * kHeadDim;
    for (int i = lane; i < a.block_size * 8; i += 32) {
        uint4* p = reinterpret_cast<uint4*>(base + (i >> 3) * pitch + (i & 7) * 16);
        uint4 q = *p;
        q.x = rescale4(q.x, ratio);
        q.y = rescale4(q.y, ratio);
        q.z = rescale4(q.z, ratio);
        q.w = rescale4(q.w, ratio);
        *p = q;
    }
}

// one warp per (token, head, k|v): quantise the row with the page's final scale
__global__ void fp8_write_kernel(Fp8Args a) {
    const int64_t item = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (item >= a.n_tokens * a.n_kv_heads * 2) return;
    const int lane = threadIdx.x & 31;
    int which, head;
    int64_t tok, slot;
    if (!fp8_locate(a, item, which, tok, head, slot)) return;
    const float s = a.scale[which][(slot / a.block_size) * a.n_kv_heads + head];
    const uint2 raw = *reinterpret_cast<const uint2*>(a.src[which] + tok * a.pitch[which] + head * kHeadDim + lane * 4);
    const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    const float x[4] = {__low2float(p0), __high2float(p0), __low2float(p1), __high2float(p1)};
    uint32_t out = 0;
    if (s > 0.0f) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            out |= uint32_t(__nv_cvt_float_to_fp8(__fdiv_rn(x[i], s), __NV_SATFINITE, __NV_E4M3)) << (8 * i);
    }
    *reinterpret_cast<uint32_t*>(a.cache[which] + (slot * a.n_kv_heads + head) * int64_t(kHeadDim) + lane * 4) = out;
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
    ib::fp8_amax_kernel<<<unsigned((items * 32 + 255) / 256), 256, 0, stream>>>(a);
    ib::fp8_rescale_kernel<<<unsigned((items * 32 + 255) / 256), 256, 0, stream>>>(a);
    ib::fp8_write_kernel<<<unsigned((items * 32 + 255) / 256), 256, 0, stream>>>(a);
    return ib::check_launch();
}

}  // extern "C"
