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
// Eight lanes per (token, head), four heads per warp: a lane owns dims [8l, 8l+8) and
// [64+8l, 64+8l+8) (two 16-byte loads), i.e. eight rotation pairs, so the pairing (i, i + 64)
// never leaves the thread and the sum of squares needs three shuffles.
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

// What a lane holds of one (token, head): dims [8 sub, 8 sub + 8) and [64 + 8 sub, 64 + 8 sub + 8) of the row,
// and the cosines / sines of those rotation pairs.
struct RowPart {
    uint4 x, y, c, s;
};

// normalise + rotate the sixteen values of this lane (sub = lane within the head's group of 8).
// Packed bf16 arithmetic: a bf16 product or sum is the fp32 result rounded once, which is exactly
// the reference's "compute in the tensor's dtype" step.
__device__ __forceinline__ void norm_rope(const RowPart& r, const __nv_bfloat16* weight, float eps, int sub, uint4& lo_out,
                                          uint4& hi_out) {
    const uint4 wlr = *reinterpret_cast<const uint4*>(weight + 8 * sub);
    const uint4 whr = *reinterpret_cast<const uint4*>(weight + 64 + 8 * sub);
    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&r.x);
    const __nv_bfloat162* y2 = reinterpret_cast<const __nv_bfloat162*>(&r.y);
    const __nv_bfloat162* wl2 = reinterpret_cast<const __nv_bfloat162*>(&wlr);
    const __nv_bfloat162* wh2 = reinterpret_cast<const __nv_bfloat162*>(&whr);
    const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&r.c);
    const __nv_bfloat162* s2 = reinterpret_cast<const __nv_bfloat162*>(&r.s);
    float2 xf[4], yf[4];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        xf[i] = __bfloat1622float2(x2[i]);
        yf[i] = __bfloat1622float2(y2[i]);
        ss += xf[i].x * xf[i].x + xf[i].y * xf[i].y + yf[i].x * yf[i].x + yf[i].y * yf[i].y;
    }
    // only the eight lanes of this head's group take part: other groups of the warp may be V heads
    const uint32_t group_mask = 0xffu << ((threadIdx.x & 31) & ~7);
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) ss += __shfl_xor_sync(group_mask, ss, o);
    const float inv = rsqrtf(ss * (1.0f / kHeadDim) + eps);
    __nv_bfloat162* ox = reinterpret_cast<__nv_bfloat162*>(&lo_out);
    __nv_bfloat162* oy = reinterpret_cast<__nv_bfloat162*>(&hi_out);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        // bf16(bf16(x * inv) * w)
        const __nv_bfloat162 a = __hmul2_rn(__floats2bfloat162_rn(xf[i].x * inv, xf[i].y * inv), wl2[i]);
        const __nv_bfloat162 b = __hmul2_rn(__floats2bfloat162_rn(yf[i].x * inv, yf[i].y * inv), wh2[i]);
        // out_x = bf16(bf16(x c) - bf16(y s)),  out_y = bf16(bf16(y c) + bf16(x s))
        // (the _rn forms are never contracted into a fused multiply-add, which would skip a rounding)
        ox[i] = __hsub2_rn(__hmul2_rn(a, c2[i]), __hmul2_rn(b, s2[i]));
        oy[i] = __hadd2_rn(__hmul2_rn(b, c2[i]), __hmul2_rn(a, s2[i]));
    }
}

// Two (token, head) items per lane group, kItems groups apart, so that the loads of both are in
// flight together: the kernel waits on memory, not on arithmetic (ncu: 14 long-scoreboard
// stall cycles per issued instruction with one item per group).
constexpr int kItemsPerGroup = 2;

__global__ void __launch_bounds__(256) fused_norm_rope_append_kernel(FusedArgs a) {
    pdl_launch_dependents();
    const int heads = a.n_q_heads + 2 * a.n_kv_heads;
    const int qk_heads = a.n_q_heads + a.n_kv_heads;
    const uint32_t total = uint32_t(a.n_tokens) * uint32_t(heads);       // the host keeps this below 2^28
    const uint32_t groups = (total + kItemsPerGroup - 1) / kItemsPerGroup;
    const uint32_t group = (blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    const int sub = threadIdx.x & 7;

    // phase 1: where the items are, and every load they need
    bool live[kItemsPerGroup], slot_ok[kItemsPerGroup];
    int h[kItemsPerGroup];
    int64_t tok[kItemsPerGroup], slot[kItemsPerGroup];
    RowPart part[kItemsPerGroup];
#pragma unroll
    for (int j = 0; j < kItemsPerGroup; ++j) {
        const uint32_t item = group + uint32_t(j) * groups;
        // an item past the end still takes part in the shuffles of its warp
        live[j] = group < groups && item < total;
        const uint32_t it = live[j] ? item : total - 1;
        tok[j] = it / uint32_t(heads);
        h[j] = int(it - uint32_t(tok[j]) * uint32_t(heads));
        slot[j] = a.slot_mapping[tok[j]];
        slot_ok[j] = slot[j] >= 0 && slot[j] < a.num_slots;      // false: padding row of a captured batch
        const __nv_bfloat16* src = h[j] < a.n_q_heads ? a.q + tok[j] * a.q_pitch + h[j] * kHeadDim
                                 : h[j] < qk_heads    ? a.k + tok[j] * a.k_pitch + (h[j] - a.n_q_heads) * kHeadDim
                                                      : a.v + tok[j] * a.v_pitch + (h[j] - qk_heads) * kHeadDim;
        part[j].x = *reinterpret_cast<const uint4*>(src + 8 * sub);
        part[j].y = *reinterpret_cast<const uint4*>(src + 64 + 8 * sub);
        if (h[j] < qk_heads) {
            const int64_t pos = min(max(a.positions[tok[j]], int64_t(0)), a.max_position - 1);
            const __nv_bfloat16* cs = a.cos_sin + pos * kHeadDim;
            part[j].c = *reinterpret_cast<const uint4*>(cs + 8 * sub);
            part[j].s = *reinterpret_cast<const uint4*>(cs + 64 + 8 * sub);
        }
    }
    // phase 2: arithmetic and stores
#pragma unroll
    for (int j = 0; j < kItemsPerGroup; ++j) {
        if (h[j] < qk_heads) {
            const bool is_q = h[j] < a.n_q_heads;
            uint4 lo, hi;
            norm_rope(part[j], is_q ? a.q_weight : a.k_weight, a.eps, sub, lo, hi);
            if (!live[j] || (!is_q && !slot_ok[j])) continue;
            __nv_bfloat16* dst = is_q ? a.q_out + tok[j] * a.q_out_pitch + h[j] * kHeadDim
                                      : a.k_cache + (slot[j] * a.n_kv_heads + (h[j] - a.n_q_heads)) * int64_t(kHeadDim);
            *reinterpret_cast<uint4*>(dst + 8 * sub) = lo;
            *reinterpret_cast<uint4*>(dst + 64 + 8 * sub) = hi;
        } else {
            if (!live[j] || !slot_ok[j]) continue;
            __nv_bfloat16* dst = a.v_cache + (slot[j] * a.n_kv_heads + (h[j] - qk_heads)) * int64_t(kHeadDim);
            *reinterpret_cast<uint4*>(dst + 8 * sub) = part[j].x;
            *reinterpret_cast<uint4*>(dst + 64 + 8 * sub) = part[j].y;
        }
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
        !aligned16(q_norm_weight) || !aligned16(k_norm_weight) ||
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
    const int64_t items = n_tokens * (n_q_heads + 2 * pool->n_kv_heads);
    const int64_t groups = (items + kItemsPerGroup - 1) / kItemsPerGroup;   // eight lanes each
    const int64_t blocks = (groups + 31) / 32;
    if (items >= (int64_t(1) << 28)) return INFER_ERR_GEOMETRY;           // 32-bit item arithmetic in the kernel
    fused_norm_rope_append_kernel<<<unsigned(blocks), 256, 0, static_cast<cudaStream_t>(stream_)>>>(a);
    return check_launch();
}
