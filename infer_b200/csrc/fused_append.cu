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
// Eight lanes per (token, head), four heads per warp and load instruction: a lane owns dims
// [8l, 8l+8) and [64+8l, 64+8l+8) (two 16-byte loads), i.e. eight rotation pairs, so the pairing
// (i, i + 64) never leaves the thread and the sum of squares needs three shuffles.
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

// Work item of a warp: one token and a batch of up to 4 * kQuads of its heads (q heads first, then
// k, then v).  Lane l works on head (l / 8) of each quad of four heads and owns dims [8 s, 8 s + 8)
// and [64 + 8 s, 64 + 8 s + 8), s = l % 8.  The position's cosines and sines are loaded once per
// item, the loads of all kQuads rows are issued before any arithmetic (6 KiB in flight per warp),
// and a token's heads are consecutive in memory, so every load instruction of a warp covers 1 KiB
// of one contiguous fused qkv row.
constexpr int kQuads = 6;

__global__ void __launch_bounds__(256) fused_norm_rope_append_kernel(FusedArgs a) {
    pdl_launch_dependents();
    const int heads = a.n_q_heads + 2 * a.n_kv_heads;
    const int qk_heads = a.n_q_heads + a.n_kv_heads;
    const int batches = (heads + 4 * kQuads - 1) / (4 * kQuads);
    const int lane = threadIdx.x & 31, sub = lane & 7, grp = lane >> 3;
    const int64_t n_items = a.n_tokens * batches;
    const int64_t n_warps = (int64_t(gridDim.x) * blockDim.x) >> 5;
    for (int64_t item = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; item < n_items; item += n_warps) {
        const int64_t tok = item / batches;
        const int h0 = int(item - tok * batches) * 4 * kQuads;
        const int64_t pos = min(max(a.positions[tok], int64_t(0)), a.max_position - 1);
        const int64_t slot = a.slot_mapping[tok];
        const bool slot_ok = slot >= 0 && slot < a.num_slots;      // false: padding row of a captured batch
        // phase 1: every load of the item
        RowPart part[kQuads];
        int h[kQuads];
#pragma unroll
        for (int j = 0; j < kQuads; ++j) {
            h[j] = h0 + 4 * j + grp;
            const int hh = min(h[j], heads - 1);                   // a lane group past the last head re-reads it and stores nothing
            const __nv_bfloat16* src = hh < a.n_q_heads ? a.q + tok * a.q_pitch + hh * kHeadDim
                                     : hh < qk_heads    ? a.k + tok * a.k_pitch + (hh - a.n_q_heads) * kHeadDim
                                                        : a.v + tok * a.v_pitch + (hh - qk_heads) * kHeadDim;
            part[j].x = *reinterpret_cast<const uint4*>(src + 8 * sub);
            part[j].y = *reinterpret_cast<const uint4*>(src + 64 + 8 * sub);
        }
        const __nv_bfloat16* cs = a.cos_sin + pos * kHeadDim;
        const uint4 c = *reinterpret_cast<const uint4*>(cs + 8 * sub);
        const uint4 sn = *reinterpret_cast<const uint4*>(cs + 64 + 8 * sub);
        // phase 2: arithmetic and stores
#pragma unroll
        for (int j = 0; j < kQuads; ++j) {
            if (h[j] >= heads) continue;                           // uniform over the 8 lanes of a group
            if (h[j] < qk_heads) {
                const bool is_q = h[j] < a.n_q_heads;
                part[j].c = c;
                part[j].s = sn;
                uint4 lo, hi;
                norm_rope(part[j], is_q ? a.q_weight : a.k_weight, a.eps, sub, lo, hi);
                if (!is_q && !slot_ok) continue;
                __nv_bfloat16* dst = is_q ? a.q_out + tok * a.q_out_pitch + h[j] * kHeadDim
                                          : a.k_cache + (slot * a.n_kv_heads + (h[j] - a.n_q_heads)) * int64_t(kHeadDim);
                *reinterpret_cast<uint4*>(dst + 8 * sub) = lo;
                *reinterpret_cast<uint4*>(dst + 64 + 8 * sub) = hi;
            } else if (slot_ok) {
                __nv_bfloat16* dst = a.v_cache + (slot * a.n_kv_heads + (h[j] - qk_heads)) * int64_t(kHeadDim);
                *reinterpret_cast<uint4*>(dst + 8 * sub) = part[j].x;
                *reinterpret_cast<uint4*>(dst + 64 + 8 * sub) = part[j].y;
            }
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
    const int heads = n_q_heads + 2 * pool->n_kv_heads;
    const int64_t items = n_tokens * ((heads + 4 * kQuads - 1) / (4 * kQuads));      // one warp each
    int64_t blocks = (items + 7) / 8;
    const int64_t cap = int64_t(pool->sm_count) * 16;                              // grid-stride beyond that
    if (blocks > cap) blocks = cap;
    fused_norm_rope_append_kernel<<<unsigned(blocks), 256, 0, static_cast<cudaStream_t>(stream_)>>>(a);
    return check_launch();
}
