// KV append: scatter new k/v rows through slot_mapping into the page pools.
//
// bf16 pools: a pure byte copy, one 16-byte load and one 16-byte store per thread and
// row chunk, K and V in the same thread, two chunks in flight per thread.
// e4m3 pools: the scale of a (page, head) must be final before any of its new rows is
// quantised.  A small kernel first cuts the token list into runs (consecutive tokens going to
// consecutive slots of one page) and finds out whether any page receives more than one run.
//   * No page does (every prefill chunk, every decode step): fp8_run_kernel's persistent thread
//     blocks take (run, head, k|v) units off the list the first kernel wrote; a block reads its
//     run's rows ONCE into registers, takes their amax, settles the scale (re-encoding the page's
//     older rows when a positive scale grew) and quantises from the registers.
//   * Otherwise (slots scattered over pages; also a call of more than 1024 tokens in runs of fewer than 64 rows on
//     average): three kernels - collect the new rows' amax / 448 per
//     (page, head) with atomics; raise the scales and re-encode pages whose scale grew; write the
//     new rows - on strips of 8 tokens per warp.
// Both ways give the bytes and scales of the CPU oracle bit for bit, whatever the scheduling.
// Calls of more than 1024 tokens launch the kernels of both ways; those of the way not taken return at once
// (the host never reads device data).  Calls of at most 1024 tokens (a decode step) are ONE launch
// (fp8_small_kernel): every block finds the runs for itself in shared memory.
#include <climits>

#include "common.cuh"

namespace ib {

// --------------------------------------------------------------------------- bf16
__global__ void __launch_bounds__(256) append_bf16_kernel(
    const uint4* __restrict__ k, const uint4* __restrict__ v, int64_t k_pitch16, int64_t v_pitch16,
    uint4* __restrict__ k_cache, uint4* __restrict__ v_cache, const int32_t* __restrict__ slot_mapping,
    int64_t n_tokens, int chunks, int64_t num_slots) {
    // Launched programmatically: the kernel in front (the previous step's attention, or the kernel
    // that advances the step metadata) may still be running.  Wait for it first, and only then let
    // the attention kernel behind this one start: its prologue reads context_lens, which the kernel
    // in front may have been writing.
    pdl_wait();
    pdl_launch_dependents();
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
struct Fp8Side {
    const __nv_bfloat16* src;      // new rows
    int64_t pitch;                 // elements
    uint8_t* cache;
    float* scale;                  // [num_blocks, Hkv]
    float* cand;                   // workspace [num_blocks, Hkv]: this call's amax / 448 per (page, head)
};

// Control words at the end of the workspace.
enum { kCtlConflictAcc = 0, kCtlDone = 1, kCtlConflict = 2, kCtlRunAcc = 3, kCtlRuns = 4, kCtlWords = 16 };

struct Fp8Args {
    Fp8Side k, v;
    const int32_t* slot_mapping;
    int64_t n_tokens;
    int64_t num_slots;
    int n_kv_heads;
    int block_size;
    uint64_t page_magic;           // ceil(2^64 / block_size): page = mulhi(slot, page_magic), exact for slot < 2^32
    int* count;                    // workspace [num_blocks]: runs of this call per page (zero between calls)
    int2* run_list;                // workspace [num_blocks]: (first token, its slot) of every run (valid when no page got two)
    int num_blocks;
    int* ctl;                      // workspace [kCtlWords]: see the enum above

    __device__ __forceinline__ int64_t page_of(int64_t slot) const {
        return int64_t(__umul64hi(uint64_t(slot), page_magic));
    }
};

// Work unit of the three kernels below: a strip of kStrip consecutive tokens x (k|v) x a pair
// of KV heads.  blockIdx.y fixes (k|v, head pair); the warps of a grid row walk the strips with
// a warp stride.  lane / 16 picks the head of the pair, lane % 16 the 16-byte chunk of its
// 128-element row, so a warp reads 512 contiguous bytes per token and keeps kStrip loads in
// flight per lane, and fetches the next strip's slots while the current strip's rows are in
// flight.  All lanes of a warp see the same tokens, so every branch on a page number is
// warp-uniform; consecutive tokens mostly share a page, which lets the warp do one reduction
// and one atomic (amax), one claim (rescale) or one reciprocal (write) per run of equal
// pages, not per row.
constexpr int kStrip = 8;
constexpr int kWarpsPerCta = 8;

struct StripLane {
    Fp8Side side;
    const __nv_bfloat16* src;      // this lane's 8 elements of token 0
    int head, sub;
    bool active;                   // false: the odd head of the last pair when Hkv is odd
};

__device__ __forceinline__ StripLane strip_lane(const Fp8Args& a, int lane, int by) {
    StripLane u;
    u.side = (by & 1) ? a.v : a.k;                  // selected by value: no indexed access to the parameter block
    u.head = int(by >> 1) * 2 + (lane >> 4);
    u.sub = lane & 15;
    u.active = u.head < a.n_kv_heads;
    u.src = u.side.src + u.head * kHeadDim + u.sub * 8;
    return u;
}

// Raw slots of a strip's tokens (not yet range-checked); -1 for rows or strips beyond the call.
// Full strips of a 16-byte aligned slot_mapping come in as two 16-byte loads.
__device__ __forceinline__ void strip_slots(const Fp8Args& a, int64_t strip, int64_t strips, int (&slot)[kStrip]) {
    const int64_t tok0 = strip * kStrip;
    if (strip < strips && tok0 + kStrip <= a.n_tokens && (reinterpret_cast<uintptr_t>(a.slot_mapping) & 15) == 0) {
        const int4 lo = __ldg(reinterpret_cast<const int4*>(a.slot_mapping + tok0));
        const int4 hi = __ldg(reinterpret_cast<const int4*>(a.slot_mapping + tok0) + 1);
        slot[0] = lo.x; slot[1] = lo.y; slot[2] = lo.z; slot[3] = lo.w;
        slot[4] = hi.x; slot[5] = hi.y; slot[6] = hi.z; slot[7] = hi.w;
        return;
    }
#pragma unroll
    for (int t = 0; t < kStrip; ++t) {
        slot[t] = -1;
        if (strip < strips && tok0 + t < a.n_tokens) slot[t] = __ldg(a.slot_mapping + tok0 + t);
    }
}

// True when the strip's tokens go to kStrip consecutive slots of one page (the usual case in
// a prefill chunk); page receives that page.  Warp-uniform.
__device__ __forceinline__ bool strip_is_one_run(const Fp8Args& a, const int (&slot)[kStrip], int64_t& page) {
    bool run = slot[0] >= 0 && int64_t(slot[0]) + kStrip <= a.num_slots;
#pragma unroll
    for (int t = 1; t < kStrip; ++t) run = run && slot[t] == slot[0] + t;
    if (!run) return false;
    page = a.page_of(slot[0]);
    return a.page_of(slot[0] + kStrip - 1) == page;
}

// general path: out-of-range slots become -1
__device__ __forceinline__ void strip_normalise(const Fp8Args& a, int (&slot)[kStrip]) {
#pragma unroll
    for (int t = 0; t < kStrip; ++t) slot[t] = (slot[t] >= 0 && slot[t] < a.num_slots) ? slot[t] : -1;
}

__device__ __forceinline__ uint4 strip_row(const StripLane& u, int64_t tok) {
    return __ldg(reinterpret_cast<const uint4*>(u.src + tok * u.side.pitch));
}

// largest magnitude of 8 bf16 values, as a bf16 pair (maxNum semantics: a NaN operand is dropped)
__device__ __forceinline__ __nv_bfloat162 amax8(const uint4& r) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
    return __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])), __hmax2(__habs2(h[2]), __habs2(h[3])));
}

// half-warp reduction of a row maximum, then one atomic per (page, head) by the half-warp's leader
__device__ __forceinline__ void amax_flush(const Fp8Args& a, const StripLane& u, int64_t page, __nv_bfloat162 best) {
    float m = fmaxf(__low2float(best), __high2float(best));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (u.sub == 0 && u.active && m > 0.0f)   // non-negative floats order like their bit patterns
        atomicMax(reinterpret_cast<int*>(u.side.cand + page * a.n_kv_heads + u.head), __float_as_int(__fdiv_rn(m, 448.0f)));
}

// cand[page, head] = max over this call's rows on that page of amax(row) / 448
// The warps of grid row `by` ((k|v) x head pair) walk the strips first_strip, first_strip + stride, ...
__device__ __forceinline__ void fp8_amax_body(const Fp8Args& a, int by, int64_t first_strip, int64_t stride) {
    const int64_t strips = (a.n_tokens + kStrip - 1) / kStrip;
    const int lane = threadIdx.x & 31;
    const StripLane u = strip_lane(a, lane, by);
    int64_t strip = first_strip;
    int next[kStrip];
    strip_slots(a, strip, strips, next);
    for (; strip < strips; strip += stride) {
        int slot[kStrip];
#pragma unroll
        for (int t = 0; t < kStrip; ++t) slot[t] = next[t];
        int64_t page;
        const bool one_run = strip_is_one_run(a, slot, page);
        if (!one_run) strip_normalise(a, slot);
        uint4 raw[kStrip];
#pragma unroll
        for (int t = 0; t < kStrip; ++t) {
            raw[t] = make_uint4(0, 0, 0, 0);
            if (u.active && (one_run || slot[t] >= 0)) raw[t] = strip_row(u, strip * kStrip + t);
        }
        strip_slots(a, strip + stride, strips, next);
        const __nv_bfloat162 zero = __float2bfloat162_rn(0.0f);
        if (one_run) {
            __nv_bfloat162 best = zero;
#pragma unroll
            for (int t = 0; t < kStrip; ++t) best = __hmax2(best, amax8(raw[t]));
            amax_flush(a, u, page, best);
            continue;
        }
        int64_t cur = -1;
        __nv_bfloat162 best = zero;
#pragma unroll
        for (int t = 0; t <= kStrip; ++t) {
            const int64_t p = t < kStrip ? (slot[t] >= 0 ? a.page_of(slot[t]) : -1) : -2;
            if (p != cur) {                            // warp-uniform
                if (cur >= 0) amax_flush(a, u, cur, best);
                cur = p;
                best = zero;
            }
            if (t < kStrip) best = __hmax2(best, amax8(raw[t]));
        }
    }
}

__global__ void __launch_bounds__(256, 3) fp8_amax_kernel(Fp8Args a) {
    pdl_launch_dependents();
    pdl_wait();
    if (a.ctl[kCtlConflict] == 0) return;      // every page got one run: fp8_run_kernel did the work
    fp8_amax_body(a, int(blockIdx.y), int64_t(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5), int64_t(gridDim.x) * kWarpsPerCta);
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

// The start of a run of tokens on `page`: the half-warp whose leader takes the candidate out
// of the workspace (exactly one per touched (page, head), however many runs the page has)
// raises the scale and, when a positive scale grew, re-encodes that page's rows for that head.
__device__ __forceinline__ void rescale_claim(const Fp8Args& a, const StripLane& u, int64_t page, int lane) {
    const int64_t e = page * a.n_kv_heads + u.head;
    float ratio = -1.0f;
    if (u.sub == 0 && u.active) {
        const float c = atomicExch(u.side.cand + e, 0.0f);
        if (c > 0.0f) {
            const float old = u.side.scale[e];
            if (c > old) {
                u.side.scale[e] = c;
                if (old > 0.0f) ratio = __fdiv_rn(old, c);
            }
        }
    }
    ratio = __shfl_sync(0xffffu << (lane & 16), ratio, lane & 16);
    if (ratio < 0.0f) return;
    // rows of this head: block_size rows of 128 bytes, pitch Hkv * 128
    uint8_t* base = u.side.cache + (page * a.block_size * a.n_kv_heads + u.head) * int64_t(kHeadDim);
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

// Raises scale[page, head] to the call's candidate; a warp looks at a page only where a run
// of tokens on that page starts (the token in front maps elsewhere).
__device__ __forceinline__ void fp8_rescale_body(const Fp8Args& a, int by, int64_t first_strip, int64_t stride) {
    const int64_t strips = (a.n_tokens + kStrip - 1) / kStrip;
    const int lane = threadIdx.x & 31;
    const StripLane u = strip_lane(a, lane, by);
    for (int64_t strip = first_strip; strip < strips; strip += stride) {
        int slot[kStrip];
        strip_slots(a, strip, strips, slot);
        int64_t cur = -1;                              // page of the token in front of the strip
        if (strip > 0) {
            const int s = __ldg(a.slot_mapping + strip * kStrip - 1);
            if (s >= 0 && s < a.num_slots) cur = a.page_of(s);
        }
        int64_t page;
        if (strip_is_one_run(a, slot, page)) {
            if (page != cur) rescale_claim(a, u, page, lane);
            continue;
        }
        strip_normalise(a, slot);
#pragma unroll
        for (int t = 0; t < kStrip; ++t) {
            page = slot[t] >= 0 ? a.page_of(slot[t]) : -1;
            const bool starts = page >= 0 && page != cur;   // warp-uniform
            cur = page;
            if (starts) rescale_claim(a, u, page, lane);
        }
    }
}

__global__ void __launch_bounds__(256) fp8_rescale_kernel(Fp8Args a) {
    pdl_launch_dependents();
    pdl_wait();                // the candidates of the kernel in front
    if (a.ctl[kCtlConflict] == 0) return;
    fp8_rescale_body(a, int(blockIdx.y), int64_t(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5), int64_t(gridDim.x) * kWarpsPerCta);
}

__device__ __forceinline__ uint64_t pk2(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ uint64_t fmul2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// x / s, correctly rounded, for numerators that are bf16 values.  With r = RN(1 / s) the
// sequence q0 = RN(x r), q = RN(q0 + RN(x - s q0) r) returns RN(x / s) for every one of the
// 128 significands of x and all 2^23 significands of s (checked exhaustively on the host);
// scales outside [2^-64, 2^64] take the general division.  Quotients too small for the
// sequence's intermediate results to be normal numbers round to zero in e4m3 either way.
// Two quotients per instruction (packed fp32 pairs, each half rounded like the scalar form).
struct Divisor {
    float s;
    uint64_t r2, neg_s2;
    bool fast;
    __device__ __forceinline__ explicit Divisor(float s_) : s(s_), r2(0), neg_s2(0), fast(s_ >= 0x1p-64f && s_ <= 0x1p64f) {
        if (fast) {
            const float r = __frcp_rn(s_);
            r2 = pk2(r, r);
            neg_s2 = pk2(-s_, -s_);
        }
    }
    // a 32-bit word holding two bf16 values -> their two quotients
    __device__ __forceinline__ float2 divide2(uint32_t w) const {
        const float lo = __uint_as_float(w << 16), hi = __uint_as_float(w & 0xffff0000u);
        float2 q;
        if (fast) {
            const uint64_t x2 = pk2(lo, hi);
            const uint64_t q0 = fmul2(x2, r2);
            const uint64_t q2 = ffma2(ffma2(neg_s2, q0, x2), r2, q0);
            asm("mov.b64 {%0, %1}, %2;" : "=f"(q.x), "=f"(q.y) : "l"(q2));
        } else {
            q = make_float2(__fdiv_rn(lo, s), __fdiv_rn(hi, s));
        }
        return q;
    }
    // two 32-bit words (four bf16 values) -> the four e4m3 bytes of their quotients: one conversion
    // instruction per pair (round to nearest even, saturating), the halves joined by register naming
    __device__ __forceinline__ uint32_t quantise4(uint32_t w0, uint32_t w1) const {
        const float2 a = divide2(w0), b = divide2(w1);
        uint32_t out;
        asm("{\n\t.reg .b16 lo, hi;\n\t"
            "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
            "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
            "mov.b32 %0, {lo, hi};\n\t}"
            : "=r"(out)
            : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
        return out;
    }
    __device__ __forceinline__ uint2 quantise8(const uint4& raw) const {
        if (!(s > 0.0f)) return make_uint2(0, 0);
        return make_uint2(quantise4(raw.x, raw.y), quantise4(raw.z, raw.w));
    }
    // The same for a scale known to be in the range of the short sequence (`fast`): straight-line code, so a
    // loop over many rows carries no test per quotient.  Callers test `fast` once, outside their loop.
    __device__ __forceinline__ uint32_t quantise4_fast(uint32_t w0, uint32_t w1) const {
        const uint64_t x0 = pk2(__uint_as_float(w0 << 16), __uint_as_float(w0 & 0xffff0000u));
        const uint64_t x1 = pk2(__uint_as_float(w1 << 16), __uint_as_float(w1 & 0xffff0000u));
        const uint64_t a0 = fmul2(x0, r2), b0 = fmul2(x1, r2);
        const uint64_t a = ffma2(ffma2(neg_s2, a0, x0), r2, a0), b = ffma2(ffma2(neg_s2, b0, x1), r2, b0);
        uint32_t out;
        asm("{\n\t.reg .b16 lo, hi;\n\t.reg .f32 ax, ay, bx, by;\n\t"
            "mov.b64 {ax, ay}, %1;\n\tmov.b64 {bx, by}, %2;\n\t"
            "cvt.rn.satfinite.e4m3x2.f32 lo, ay, ax;\n\t"
            "cvt.rn.satfinite.e4m3x2.f32 hi, by, bx;\n\t"
            "mov.b32 %0, {lo, hi};\n\t}"
            : "=r"(out)
            : "l"(a), "l"(b));
        return out;
    }
    __device__ __forceinline__ uint2 quantise8_fast(const uint4& raw) const {
        return make_uint2(quantise4_fast(raw.x, raw.y), quantise4_fast(raw.z, raw.w));
    }
};

// quantise the new rows with their page's final scale
__device__ __forceinline__ void fp8_write_body(const Fp8Args& a, int by, int64_t first_strip, int64_t stride) {
    const int64_t strips = (a.n_tokens + kStrip - 1) / kStrip;
    const int lane = threadIdx.x & 31;
    const StripLane u = strip_lane(a, lane, by);
    uint8_t* const dst = u.side.cache + u.head * kHeadDim + u.sub * 8;
    const int64_t dst_pitch = int64_t(a.n_kv_heads) * kHeadDim;
    int64_t strip = first_strip;
    int next[kStrip];
    strip_slots(a, strip, strips, next);
    for (; strip < strips; strip += stride) {
        int slot[kStrip];
#pragma unroll
        for (int t = 0; t < kStrip; ++t) slot[t] = next[t];
        int64_t page;
        const bool one_run = strip_is_one_run(a, slot, page);
        if (!one_run) strip_normalise(a, slot);
        uint4 raw[kStrip];
#pragma unroll
        for (int t = 0; t < kStrip; ++t) {
            raw[t] = make_uint4(0, 0, 0, 0);
            if (u.active && (one_run || slot[t] >= 0)) raw[t] = strip_row(u, strip * kStrip + t);
        }
        // the scale of the strip's first page travels with the rows; later pages (rare) load theirs in the loop
        int64_t cur = one_run ? page : (slot[0] >= 0 ? a.page_of(slot[0]) : -1);
        float s = (cur >= 0 && u.active) ? u.side.scale[cur * a.n_kv_heads + u.head] : 0.0f;
        strip_slots(a, strip + stride, strips, next);
        Divisor div(s);
        if (one_run) {
            if (u.active) {
                uint8_t* row = dst + slot[0] * dst_pitch;
#pragma unroll
                for (int t = 0; t < kStrip; ++t) *reinterpret_cast<uint2*>(row + t * dst_pitch) = div.quantise8(raw[t]);
            }
            continue;
        }
#pragma unroll
        for (int t = 0; t < kStrip; ++t) {
            if (slot[t] < 0) continue;                 // warp-uniform
            page = a.page_of(slot[t]);
            if (page != cur) {                         // warp-uniform
                cur = page;
                s = u.active ? u.side.scale[cur * a.n_kv_heads + u.head] : 0.0f;
                div = Divisor(s);
            }
            if (u.active) *reinterpret_cast<uint2*>(dst + slot[t] * dst_pitch) = div.quantise8(raw[t]);
        }
    }
}

__global__ void __launch_bounds__(256, 3) fp8_write_kernel(Fp8Args a) {
    pdl_launch_dependents();
    pdl_wait();                // the final scales and re-encoded pages of the kernel in front
    if (a.ctl[kCtlConflict] == 0) return;
    fp8_write_body(a, int(blockIdx.y), int64_t(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5), int64_t(gridDim.x) * kWarpsPerCta);
}

// --------------------------------------------------------------------------- runs
__device__ __forceinline__ bool slot_valid(const Fp8Args& a, int s) { return s >= 0 && int64_t(s) < a.num_slots; }

// Token i starts a run when its slot is valid and the token in front does not sit in the slot in
// front of it on the same page.
__device__ __forceinline__ bool is_run_start(const Fp8Args& a, int64_t i, int& slot) {
    slot = __ldg(a.slot_mapping + i);
    const int prev = i > 0 ? __ldg(a.slot_mapping + i - 1) : -1;       // both loads in flight together
    if (!slot_valid(a, slot)) return false;
    return !(slot_valid(a, prev) && prev + 1 == slot && a.page_of(prev) == a.page_of(slot));
}

// Counts the runs every page receives and lists the runs' first tokens (a page that gets one run
// at most means at most num_blocks runs, so the list has room for all of them in the case that
// uses it).  The block that finishes last publishes whether any page got more than one run
// (kCtlConflict) and how many runs there are (kCtlRuns) - both written afresh by every call - and
// clears the accumulators.
__global__ void __launch_bounds__(256) fp8_classify_kernel(Fp8Args a) {
    pdl_launch_dependents();
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const int lane = threadIdx.x & 31;
    int slot = -1;
    const bool starts = i < a.n_tokens && is_run_start(a, i, slot);
    int conflict = 0;
    if (starts) conflict = atomicAdd(a.count + a.page_of(slot), 1) > 0;
    // one atomic per warp for the list positions
    const uint32_t ballot = __ballot_sync(0xffffffffu, starts);
    int base = 0;
    if (ballot && lane == 0) base = atomicAdd(a.ctl + kCtlRunAcc, __popc(ballot));
    base = __shfl_sync(0xffffffffu, base, 0);
    if (starts) {
        const int idx = base + __popc(ballot & ((1u << lane) - 1));
        if (idx < a.num_blocks) a.run_list[idx] = make_int2(int(i), slot);
    }
    conflict = __syncthreads_or(conflict);
    if (threadIdx.x == 0) {
        if (conflict) atomicOr(a.ctl + kCtlConflictAcc, 1);
        __threadfence();
        if (atomicAdd(a.ctl + kCtlDone, 1) == int(gridDim.x) - 1) {
            __threadfence();
            int scattered = atomicExch(a.ctl + kCtlConflictAcc, 0);
            const int runs = atomicExch(a.ctl + kCtlRunAcc, 0);
            // A large call whose runs are short (fewer than 64 rows on average: the step of a decode batch of
            // more than 1024 sequences) also goes to the strip kernels: fp8_run_kernel gives a whole thread block
            // to every (run, head, k|v), most of it idle on a one-row run (measured: 2048 rows on pages of their
            // own 266 us, 46 us as units of single warps, less again on strips).
            if (a.n_tokens > 1024 && int64_t(runs) * 64 > a.n_tokens) scattered = 1;
            a.ctl[kCtlConflict] = scattered;
            a.ctl[kCtlRuns] = runs;
            a.ctl[kCtlDone] = 0;
        }
    }
}

// Groups of threads walk the units (run, head, k|v), the 2 * Hkv units of a run side by side so that neighbouring
// groups read neighbouring 256-byte pieces of the same rows at the same time.  A row of one head is 256 bytes =
// 16 lanes x 16 bytes, THREADS / 16 rows per load instruction, 16 loads in flight per thread: a block of 256
// threads holds a whole 256-row run (64 KiB) in registers, so the rows are read from memory once; a single warp
// (the form the calls of few tokens use: a decode step's runs are one row long) holds 32 rows.  Rows past what
// the registers hold are read a second time, from L2.
// (Measured slower on 32768 rows x 8 heads, 43.2 us for the kernel of persistent 256-thread blocks: the rows parked
// in shared memory by 512 threads, two blocks per SM, 51 us - 24.5 M executed instructions against 18.9 M;
// asynchronous copies into three 64 KiB buffers, one 17-warp block per SM, 70.8 us; no rows held at all, pass 2
// re-reading them from L2, with 3, 4 or 6 blocks per SM, 56 / 53 / 53 us per call against 50.5; the loads of a
// unit issued before its run's length is known, 52.3 against 50.4.)

// Scratch of one group of threads working on a unit (a block, or one warp of a block).
struct RunScratch {
    int len;
    float red[8], scale, ratio;
};

template <int THREADS>
__device__ __forceinline__ void group_sync() {
    if (THREADS == 32) __syncwarp();
    else __syncthreads();
}

// The units first_unit, first_unit + unit_step, ... of the runs in run_list (global or shared memory), worked on
// by a group of THREADS threads (tid = index in the group): a whole block, or one warp on its own.
template <int THREADS>
__device__ __forceinline__ void fp8_run_units(const Fp8Args& a, const int2* run_list, int n_runs, int64_t first_unit,
                                              int64_t unit_step, int tid, RunScratch& sc, bool reset_counts) {
    constexpr int kRowsPerLoad = THREADS / 16, kHeld = 16 * kRowsPerLoad, kWarps = THREADS / 32;
    const int sides = 2 * a.n_kv_heads;
    const int64_t n_units = int64_t(n_runs) * sides;
    const int lane16 = tid & 15, rsub = tid >> 4;
    const int64_t dst_pitch = int64_t(a.n_kv_heads) * kHeadDim;
    for (int64_t unit = first_unit; unit < n_units; unit += unit_step) {
        const int run = int(unit / sides), y = int(unit - int64_t(run) * sides);
        const int head = y >> 1;
        const Fp8Side side = (y & 1) ? a.v : a.k;
        const int2 first = run_list[run];
        const int64_t start = first.x;
        const int slot0 = first.y;
        const int64_t page = a.page_of(slot0);
        if (reset_counts && y == 0 && tid == 0) a.count[page] = 0;          // nobody reads the counts any more
        // length of the run: the first offset whose token does not continue it
        int len = 1;
        for (int base = 1;; base += THREADS) {
            if (tid == 0) sc.len = INT_MAX;
            group_sync<THREADS>();
            const int64_t i = start + base + tid;
            bool cont = i < a.n_tokens;
            if (cont) {
                const int s = __ldg(a.slot_mapping + i);
                cont = s == slot0 + base + tid && int64_t(s) < a.num_slots && a.page_of(s) == page;
            }
            if (!cont) atomicMin(&sc.len, base + tid);
            group_sync<THREADS>();
            const int first_bad = sc.len;
            group_sync<THREADS>();
            if (first_bad != INT_MAX) { len = first_bad; break; }
            len = base + THREADS;
        }
        // pass 1: the rows (the first kHeld stay in registers) and their largest magnitude
        const __nv_bfloat16* src = side.src + head * kHeadDim + lane16 * 8;
        uint4 raw[16];
        __nv_bfloat162 best = __float2bfloat162_rn(0.0f);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int row = rsub + j * kRowsPerLoad;
            raw[j] = make_uint4(0, 0, 0, 0);
            if (row < len) raw[j] = __ldg(reinterpret_cast<const uint4*>(src + (start + row) * side.pitch));
        }
        // the page's present scale travels with the rows
        const int64_t e = page * a.n_kv_heads + head;
        const float old = side.scale[e];
#pragma unroll
        for (int j = 0; j < 16; ++j) best = __hmax2(best, amax8(raw[j]));
        for (int row = kHeld + rsub; row < len; row += kRowsPerLoad)
            best = __hmax2(best, amax8(__ldg(reinterpret_cast<const uint4*>(src + (start + row) * side.pitch))));
        float m = fmaxf(__low2float(best), __high2float(best));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if ((tid & 31) == 0) sc.red[tid >> 5] = m;
        group_sync<THREADS>();
        if (tid == 0) {
#pragma unroll
            for (int w = 1; w < kWarps; ++w) m = fmaxf(m, sc.red[w]);
            float s = old, ratio = -1.0f;
            if (m > 0.0f) {
                const float c = __fdiv_rn(m, 448.0f);
                if (c > old) {
                    side.scale[e] = c;
                    s = c;
                    if (old > 0.0f) ratio = __fdiv_rn(old, c);
                }
            }
            sc.scale = s;
            sc.ratio = ratio;
        }
        group_sync<THREADS>();
        const float scale = sc.scale, ratio = sc.ratio;
        if (ratio >= 0.0f) {
            // the page's scale grew: re-encode what the page holds for this head (rows this run is about
            // to overwrite included, which is harmless), before any new row is written
            uint8_t* base = side.cache + (page * a.block_size * a.n_kv_heads + head) * int64_t(kHeadDim);
            for (int i = tid; i < a.block_size * 8; i += THREADS) {
                uint4* p = reinterpret_cast<uint4*>(base + (i >> 3) * dst_pitch + (i & 7) * 16);
                uint4 q = *p;
                q.x = rescale4(q.x, ratio);
                q.y = rescale4(q.y, ratio);
                q.z = rescale4(q.z, ratio);
                q.w = rescale4(q.w, ratio);
                *p = q;
            }
            group_sync<THREADS>();
        }
        // pass 2: quantise with the final scale
        const Divisor div(scale);
        uint8_t* dst = side.cache + int64_t(slot0) * dst_pitch + head * kHeadDim + lane16 * 8;
        if (div.fast) {                                // uniform over the block: one test for the whole run
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int row = rsub + j * kRowsPerLoad;
                if (row < len) *reinterpret_cast<uint2*>(dst + row * dst_pitch) = div.quantise8_fast(raw[j]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int row = rsub + j * kRowsPerLoad;
                if (row < len) *reinterpret_cast<uint2*>(dst + row * dst_pitch) = div.quantise8(raw[j]);
            }
        }
        for (int row = kHeld + rsub; row < len; row += kRowsPerLoad)
            *reinterpret_cast<uint2*>(dst + row * dst_pitch) =
                div.quantise8(__ldg(reinterpret_cast<const uint4*>(src + (start + row) * side.pitch)));
        group_sync<THREADS>();                          // s_red, sc.scale and sc.ratio are reused by the next unit
    }
}



// Calls of more than 1024 tokens: persistent blocks of 256 threads, a block per unit, over the run list the
// classification kernel wrote.
__global__ void __launch_bounds__(256, 2) fp8_run_kernel(Fp8Args a) {
    __shared__ RunScratch s_scratch;
    pdl_launch_dependents();
    pdl_wait();                                   // the run list, the counts and the conflict flag of the kernel in front
    const int tid = threadIdx.x;
    if (a.ctl[kCtlConflict] != 0) {
        // some page got several runs: the three strip kernels do the work; all that is left to do here
        // is to put the run counts back to zero
        const int64_t stride = int64_t(gridDim.x) * 256;
        for (int64_t i = int64_t(blockIdx.x) * 256 + tid; i < a.n_tokens; i += stride) {
            int slot;
            if (is_run_start(a, i, slot)) a.count[a.page_of(slot)] = 0;
        }
        return;
    }
    fp8_run_units<256>(a, a.run_list, a.ctl[kCtlRuns], blockIdx.x, gridDim.x, tid, s_scratch, true);
}

// Calls of at most kSmallTokens tokens (a decode step, a short prompt) in ONE launch.  Every block cuts the whole
// token list into runs for itself, in shared memory - a few kilobytes of slot_mapping out of L2 - and finds out
// whether some page receives two runs (a hash table of the runs' pages); all blocks come to the same list and the
// same answer, so no block has to wait for another.  Then every warp takes (run, head, k|v) units of its own.  If
// some page did get two runs, block 0 alone runs the three strip phases, separated by block-wide barriers.
constexpr int kSmallTokens = 1024;

__global__ void __launch_bounds__(256, 2) fp8_small_kernel(Fp8Args a, int grid_rows) {
    constexpr int kPer = kSmallTokens / 256;      // consecutive tokens per thread
    constexpr int kHash = 2 * kSmallTokens;
    __shared__ int2 s_runs[kSmallTokens];
    __shared__ int s_hash[kHash];                 // page + 1 of a run, 0 = free
    __shared__ int s_warp_runs[8], s_conflict;
    __shared__ RunScratch s_scratch[8];
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < kHash; i += 256) s_hash[i] = 0;
    if (tid == 0) s_conflict = 0;
    int slot[kPer], mine = 0;
    bool starts[kPer];
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
        const int64_t i = int64_t(tid) * kPer + j;
        starts[j] = i < a.n_tokens && is_run_start(a, i, slot[j]);
        mine += starts[j];
    }
    int incl = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += v;
    }
    if (lane == 31) s_warp_runs[warp] = incl;
    __syncthreads();                              // also: the hash table is clear
    int at = incl - mine, n_runs = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        if (w < warp) at += s_warp_runs[w];
        n_runs += s_warp_runs[w];
    }
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
        if (!starts[j]) continue;
        s_runs[at++] = make_int2(tid * kPer + j, slot[j]);
        const int key = int(a.page_of(slot[j])) + 1;
        for (uint32_t h = (uint32_t(key) * 2654435761u) >> 21;; h = (h + 1) & (kHash - 1)) {
            const int seen = atomicCAS(&s_hash[h], 0, key);
            if (seen == key) s_conflict = 1;
            if (seen == 0 || seen == key) break;
        }
    }
    __syncthreads();
    if (s_conflict) {
        if (blockIdx.x != 0) return;
        for (int by = 0; by < grid_rows; ++by) fp8_amax_body(a, by, warp, kWarpsPerCta);
        __syncthreads();
        for (int by = 0; by < grid_rows; ++by) fp8_rescale_body(a, by, warp, kWarpsPerCta);
        __syncthreads();
        for (int by = 0; by < grid_rows; ++by) fp8_write_body(a, by, warp, kWarpsPerCta);
        return;
    }
    fp8_run_units<32>(a, s_runs, n_runs, int64_t(blockIdx.x) * 8 + warp, int64_t(gridDim.x) * 8, lane, s_scratch[warp], false);
}

}  // namespace ib

extern "C" {

size_t infer_kv_append_workspace_bytes(const infer_kv_pool_t* pool) {
    if (!pool || pool->dtype != INFER_KV_E4M3) return 0;
    // candidates of k and v per (page, head), runs per page, the run list, control words
    return (size_t(2) * pool->num_blocks * pool->n_kv_heads + size_t(3) * pool->num_blocks + ib::kCtlWords) * 4 + 8;
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
    float* cand = static_cast<float*>(workspace);
    a.k = {static_cast<const __nv_bfloat16*>(k), k_row_stride, static_cast<uint8_t*>(pool->k_cache), pool->k_scale, cand};
    a.v = {static_cast<const __nv_bfloat16*>(v), v_row_stride, static_cast<uint8_t*>(pool->v_cache), pool->v_scale,
           cand + pool->num_blocks * pool->n_kv_heads};
    a.slot_mapping = slot_mapping;
    a.n_tokens = n_tokens;
    a.num_slots = pool->num_slots;
    a.n_kv_heads = pool->n_kv_heads;
    a.block_size = pool->block_size;
    a.page_magic = ~uint64_t(0) / uint64_t(pool->block_size) + 1;
    if (pool->num_slots >= (int64_t(1) << 32)) return INFER_ERR_GEOMETRY;
    a.count = reinterpret_cast<int*>(cand + 2 * pool->num_blocks * pool->n_kv_heads);
    // the run list holds 8-byte entries: start it on the next 8-byte boundary after the counts
    a.run_list = reinterpret_cast<int2*>((reinterpret_cast<uintptr_t>(a.count + pool->num_blocks) + 7) & ~uintptr_t(7));
    a.ctl = reinterpret_cast<int*>(a.run_list + pool->num_blocks);
    a.num_blocks = int(pool->num_blocks);
    const int rows = 2 * ((pool->n_kv_heads + 1) / 2);             // grid rows of the strip phases: (k|v) x head pair
    if (n_tokens <= ib::kSmallTokens) {
        // one launch: every block finds the runs for itself, every warp takes units (at most n_tokens * 2 Hkv of them)
        int64_t grid = (n_tokens * 2 * pool->n_kv_heads + 7) / 8;
        if (grid > int64_t(pool->sm_count) * 2) grid = int64_t(pool->sm_count) * 2;
        IB_CUDA(ib::launch_pdl(ib::fp8_small_kernel, dim3(unsigned(grid)), dim3(256), 0, stream, a, rows));
        return ib::check_launch();
    }
    // runs: count and list them, then persistent thread blocks take (run, head, k|v) units
    ib::fp8_classify_kernel<<<unsigned((n_tokens + 255) / 256), 256, 0, stream>>>(a);
    IB_CUDA(ib::launch_pdl(ib::fp8_run_kernel, dim3(unsigned(pool->sm_count) * 2), dim3(256), 0, stream, a));
    // strips: only when some page received several runs (the kernels return at once otherwise)
    const int64_t strips = (n_tokens + ib::kStrip - 1) / ib::kStrip;
    int64_t per_row = (strips + ib::kWarpsPerCta - 1) / ib::kWarpsPerCta;
    // The strip kernels stride over their strips, so any grid works; they only have work when slots are
    // scattered, and otherwise every block of theirs just reads a flag and leaves: 6 blocks per SM keeps
    // that cheap and still fills the machine when they do run.
    const int64_t cap = (int64_t(pool->sm_count) * 6 + rows - 1) / rows;
    if (per_row > cap) per_row = cap;
    const dim3 blocks{unsigned(per_row), unsigned(rows), 1u};
    IB_CUDA(ib::launch_pdl(ib::fp8_amax_kernel, blocks, dim3(256), 0, stream, a));
    IB_CUDA(ib::launch_pdl(ib::fp8_rescale_kernel, blocks, dim3(256), 0, stream, a));
    IB_CUDA(ib::launch_pdl(ib::fp8_write_kernel, blocks, dim3(256), 0, stream, a));
    return ib::check_launch();
}

}  // extern "C"
