// Fused per-head RMSNorm + rotary embedding + KV append.
//
// One pass over a fused qkv row replaces four passes of the reference model code
// (infer/models/Qwen3.py:112-131): q_norm and k_norm (infer/ops/norm.py:63-73), the in-place
// rotary embedding of q and k (src/operators/rope/rope.cu:43-133, GPT-NeoX pairing) and
// store_kvcache (infer/ops/attention.py:16-45).  q is written normalised and rotated to
// q_out (which may be the input itself); k is normalised, rotated and written straight into
// its page slot; v is copied into its page slot.  Every rounding step of the reference is
// kept: the variance and the normalisation run in fp32, the normalised value is rounded to
// bf16 before the bf16 multiply by the weight, and the rotation is three bf16 operations per
// output (two products, one sum), as rope.cu computes it in its scalar type.
//
// One warp per (token, head): a lane owns dims {2l, 2l+1, 64+2l, 65+2l}, i.e. two rotation
// pairs, so the pairing (i, i + 64) never leaves the thread.
#include "common.cuh"

namespace ib {

struct FusedArgs {
    const __nv_bfloat16* q;
    const __nv_bfloat16* k;
    const __nv_bfloat16* v;
    __nv_bfloat16* q_out;
    int64_t q_pitch, k_pitch, v_pitch, q_out_pitch;   // elements between token rows
    const __nv_bfloat16* q_weight;
    const __nv_bfloat16* k_weight;
    const int64_t* positions;
    const __nv_bfloat16* cos_sin;    // [max_position, 128]: 64 cosines, then 64 sines
    const int32_t* slot_mapping;
    __nv_bfloat16* k_cache;
    __nv_bfloat16* v_cache;
    int64_t n_tokens;
    int64_t num_slots;
    int64_t max_position;
    int n_q_heads;
    int n_kv_heads;
    float eps;
};

__device__ __forceinline__ float bf(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ __nv_bfloat16 rb(float x) { return __float2bfloat16_rn(x); }

// normalise + rotate the four values of this lane; returns them as two packed bf16 pairs
__device__ __forceinline__ void norm_rope(const __nv_bfloat16* row, const __nv_bfloat16* weight, const __nv_bfloat16* cs,
                                          float eps, int lane, uint32_t& lo_out, uint32_t& hi_out) {
    const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(row + 2 * lane);
    const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(row + 64 + 2 * lane);
    const float x0 = __low2float(lo), x1 = __high2float(lo), y0 = __low2float(hi), y1 = __high2float(hi);
    float ss = x0 * x0 + x1 * x1 + y0 * y0 + y1 * y1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = rsqrtf(ss * (1.0f / kHeadDim) + eps);
    const __nv_bfloat162 wl = *reinterpret_cast<const __nv_bfloat162*>(weight + 2 * lane);
    const __nv_bfloat162 wh = *reinterpret_cast<const __nv_bfloat162*>(weight + 64 + 2 * lane);
    // bf16(bf16(x * inv) * w)
    const __nv_bfloat16 a0 = rb(bf(rb(x0 * inv)) * __low2float(wl)), a1 = rb(bf(rb(x1 * inv)) * __high2float(wl));
    const __nv_bfloat16 b0 = rb(bf(rb(y0 * inv)) * __low2float(wh)), b1 = rb(bf(rb(y1 * inv)) * __high2float(wh));
    const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(cs + 2 * lane);
    const __nv_bfloat162 s = *reinterpret_cast<const __nv_bfloat162*>(cs + 64 + 2 * lane);
    const float c0 = __low2float(c), c1 = __high2float(c), s0 = __low2float(s), s1 = __high2float(s);
    // out_x = bf16(bf16(x c) - bf16(y s)),  out_y = bf16(bf16(y c) + bf16(x s))
    const __nv_bfloat16 ox0 = rb(bf(rb(bf(a0) * c0)) - bf(rb(bf(b0) * s0)));
    const __nv_bfloat16 ox1 = rb(bf(rb(bf(a1) * c1)) - bf(rb(bf(b1) * s1)));
    const __nv_bfloat16 oy0 = rb(bf(rb(bf(b0) * c0)) + bf(rb(bf(a0) * s0)));
    const __nv_bfloat16 oy1 = rb(bf(rb(bf(b1) * c1)) + bf(rb(bf(a1) * s1)));
    __nv_bfloat162 plo, phi;
    plo.x = ox0; plo.y = ox1;
    phi.x = oy0; phi.y = oy1;
    lo_out = *reinterpret_cast<uint32_t*>(&plo);
    hi_out = *reinterpret_cast<uint32_t*>(&phi);
}

__global__ void __launch_bounds__(256) fused_norm_rope_append_kernel(FusedArgs a) {
    pdl_launch_dependents();
    const int heads = a.n_q_heads + 2 * a.n_kv_heads;
    const int64_t item = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (item >= a.n_tokens * heads) return;
    const int lane = threadIdx.x & 31;
    const int64_t tok = item / heads;
    const int h = int(item - tok * heads);
    if (h < a.n_q_heads) {
        const int64_t pos = min(max(a.positions[tok], int64_t(0)), a.max_position - 1);
        uint32_t lo, hi;
        norm_rope(a.q + tok * a.q_pitch + h * kHeadDim, a.q_weight, a.cos_sin + pos * kHeadDim, a.eps, lane, lo, hi);
        __nv_bfloat16* dst = a.q_out + tok * a.q_out_pitch + h * kHeadDim;
        *reinterpret_cast<uint32_t*>(dst + 2 * lane) = lo;
        *reinterpret_cast<uint32_t*>(dst + 64 + 2 * lane) = hi;
        return;
    }
    const int64_t slot = a.slot_mapping[tok];
    if (slot < 0 || slot >= a.num_slots) return;             // padding row of a captured batch
    if (h < a.n_q_heads + a.n_kv_heads) {
        const int kh = h - a.n_q_heads;
        const int64_t pos = min(max(a.positions[tok], int64_t(0)), a.max_position - 1);
        uint32_t lo, hi;
        norm_rope(a.k + tok * a.k_pitch + kh * kHeadDim, a.k_weight, a.cos_sin + pos * kHeadDim, a.eps, lane, lo, hi);
        __nv_bfloat16* dst = a.k_cache + (slot * a.n_kv_heads + kh) * int64_t(kHeadDim);
        *reinterpret_cast<uint32_t*>(dst + 2 * lane) = lo;
        *reinterpret_cast<uint32_t*>(dst + 64 + 2 * lane) = hi;
    } else {
        const int vh = h - a.n_q_heads - a.n_kv_heads;
        const uint2 raw = *reinterpret_cast<const uint2*>(a.v + tok * a.v_pitch + vh * kHeadDim + lane * 4);
        *reinterpret_cast<uint2*>(a.v_cache + (slot * a.n_kv_heads + vh) * int64_t(kHeadDim) + lane * 4) = raw;
    }
}

}  // namespace ib

extern "C" int infer_qk_norm_rope_append(const infer_kv_pool_t* pool, void* q_out, int64_t q_out_row_stride, const void* q,
                                         const void* k, const void* v, int64_t q_row_stride, int64_t k_row_stride,
                                         int64_t v_row_stride, const void* q_norm_weight, const void* k_norm_weight,
                                         float eps, const int64_t* positions, const void* cos_sin_cache,
                                         int64_t max_position, const int32_t* slot_mapping, int64_t n_tokens,
                                         int n_q_heads, void* stream_) {
    using namespace ib;
    if (!pool) return INFER_ERR_NULL;
    if (pool->dtype != INFER_KV_BF16) return INFER_ERR_DTYPE;
    if (n_tokens < 0 || n_q_heads <= 0 || max_position <= 0) return INFER_ERR_GEOMETRY;
    if (n_tokens == 0) return INFER_OK;
    if (!q_out || !q || !k || !v || !q_norm_weight || !k_norm_weight || !positions || !cos_sin_cache || !slot_mapping)
        return INFER_ERR_NULL;
    const int64_t qrow = int64_t(n_q_heads) * kHeadDim, kvrow = int64_t(pool->n_kv_heads) * kHeadDim;
    if (q_row_stride < qrow || q_out_row_stride < qrow || k_row_stride < kvrow || v_row_stride < kvrow) return INFER_ERR_STRIDE;
    if (!aligned16(q_out) || !aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(cos_sin_cache) ||
        (reinterpret_cast<uintptr_t>(q_norm_weight) & 3) || (reinterpret_cast<uintptr_t>(k_norm_weight) & 3) ||
        q_row_stride % 8 || q_out_row_stride % 8 || k_row_stride % 8 || v_row_stride % 8)
        return INFER_ERR_ALIGN;
    FusedArgs a;
    a.q = static_cast<const __nv_bfloat16*>(q);
    a.k = static_cast<const __nv_bfloat16*>(k);
    a.v = static_cast<const __nv_bfloat16*>(v);
    a.q_out = static_cast<__nv_bfloat16*>(q_out);
    a.q_pitch = q_row_stride;
    a.k_pitch = k_row_stride;
    a.v_pitch = v_row_stride;
    a.q_out_pitch = q_out_row_stride;
    a.q_weight = static_cast<const __nv_bfloat16*>(q_norm_weight);
    a.k_weight = static_cast<const __nv_bfloat16*>(k_norm_weight);
    a.positions = positions;
    a.cos_sin = static_cast<const __nv_bfloat16*>(cos_sin_cache);
    a.slot_mapping = slot_mapping;
    a.k_cache = static_cast<__nv_bfloat16*>(pool->k_cache);
    a.v_cache = static_cast<__nv_bfloat16*>(pool->v_cache);
    a.n_tokens = n_tokens;
    a.num_slots = pool->num_slots;
    a.max_position = max_position;
    a.n_q_heads = n_q_heads;
    a.n_kv_heads = pool->n_kv_heads;
    a.eps = eps;
    const int64_t warps = n_tokens * (n_q_heads + 2 * pool->n_kv_heads);
    const int64_t blocks = (warps + 7) / 8;
    if (blocks >= (int64_t(1) << 31)) return INFER_ERR_GEOMETRY;
    fused_norm_rope_append_kernel<<<unsigned(blocks), 256, 0, static_cast<cudaStream_t>(stream_)>>>(a);
    return check_launch();
}
