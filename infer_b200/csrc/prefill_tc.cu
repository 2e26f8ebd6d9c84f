// Causal attention over many query rows on the 5th-generation tensor cores (tcgen05).
//
// One CTA = 128 query rows of one (sequence, query head).  Per 128-key tile:
//   S = Q K^T        tcgen05.mma, A = Q and B = K from shared memory (K-major, 128-byte
//                    swizzle, written by TMA), accumulator in tensor memory (128 columns)
//   softmax          four warps, one thread per query row = one TMEM lane: tcgen05.ld of the
//                    row, running max / sum in registers, P written back to tensor memory as
//                    packed bf16 (two keys per 32-bit column)
//   O += P V         tcgen05.mma, A = P from tensor memory, B = V (MN-major: dims contiguous), the
//                    accumulator stays in tensor memory for the whole key loop
// The softmax keeps a reference maximum per row and only moves it (rescaling the row of O in
// tensor memory and the running sum) when the true maximum has grown by more than 2^8; the
// result is exact because O and the sum always share the same reference.  S and P are
// double-buffered, so S_{j+1} and P V_j run on the tensor core while the softmax of the next
// tile proceeds.  Warp roles: 0-7 softmax (two threads per query row, each owning 64 of a
// tile's 128 columns; they exchange their row maxima through shared memory once per tile),
// 8 TMA producer, 9 MMA issue and TMEM allocation.  Every barrier wait is bounded; a wait that runs out raises a CTA-wide
// abort flag, every role drains to the common epilogue, TMEM is freed and a status is set.
#include "prefill.cuh"

namespace ib {

constexpr int kTcRows = 128;                 // query rows per CTA
constexpr int kTcKeys = 128;                 // keys per tile
constexpr int kTcHalf = 128 * 128;           // bytes of one [128 rows][64 elems] swizzled sub-tile
constexpr int kTcTile = 2 * kTcHalf;         // 32 KiB: Q, K, V or P tile
constexpr int kTcSoftmaxWarps = 8;            // two threads per query row: columns 0-63 and 64-127 of a tile
constexpr int kTcProducerWarp = kTcSoftmaxWarps, kTcMmaWarp = kTcSoftmaxWarps + 1;
constexpr int kTcThreads = (kTcSoftmaxWarps + 2) * 32;
constexpr int kTcStages = 3;                  // K and V tiles in flight
// tensor memory columns: S0 0-127, S1 128-255, O 256-383, P0 384-447, P1 448-511
constexpr uint32_t kTmemO = 256, kTmemP = 384;

struct TcSmem {
    static constexpr int q = 0;
    static constexpr int k = q + kTcTile;                  // kTcStages stages
    static constexpr int v = k + kTcStages * kTcTile;      // kTcStages stages
    static constexpr int bars = v + kTcStages * kTcTile;   // 8-byte mbarriers
    static constexpr int n_bars = 24;
    static constexpr int misc = bars + n_bars * 8;   // tmem base, abort flag
    static constexpr int xchg = misc + 16;           // [2 tile parities][2 column halves][128 rows] bf16 row maxima
    static constexpr int total = xchg + 2 * 2 * 128 * 2;
};

enum TcBar { Q_FULL = 0, K_FULL = 1, K_EMPTY = 4, V_FULL = 7, V_EMPTY = 10, S_FULL = 13, S_EMPTY = 15, P_FULL = 17,
             P_EMPTY = 19, PV_DONE = 21, DRAIN = 22 };
constexpr float kLazyLog2 = 8.f;              // the reference maximum may lag the true one by 2^8

// ---- tcgen05 wrappers
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc), "r"(0u)
        : "memory");
}
// same, with the A operand in tensor memory (16-bit elements packed two per column)
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(acc), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
        "%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
        "%29,%30,%31};"
        ::"r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
          "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
          "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]), "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle, 8-row groups 1024 bytes apart.
//   K-major operands ([rows][64 elems] sub-tiles): lbo unused.
//   MN-major operand (V as [keys][64 dims]): lbo = distance between the two 64-dim halves.
__device__ __forceinline__ uint64_t tc_desc(uint32_t smem_addr, uint32_t lbo_bytes) {
    uint64_t d = 0;
    d |= uint64_t((smem_addr >> 4) & 0x3FFF);
    d |= uint64_t((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= uint64_t((1024 >> 4) & 0x3FFF) << 32;
    d |= uint64_t(1) << 46;        // descriptor version for sm_100
    d |= uint64_t(2) << 61;        // SWIZZLE_128B
    return d;
}
// kind::f16 instruction descriptor: D f32, A and B bf16, M = N = 128.
constexpr uint32_t tc_idesc(bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
}

// Bounded wait that also gives up as soon as another thread raised the abort flag.
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63) == 63) {
            if (*abort_flag) return false;
            __nanosleep(i > 4096 ? 256 : 32);
        }
    }
    *abort_flag = 1;
    return false;
}

template <bool PAGED>
__global__ void __launch_bounds__(kTcThreads, 1) prefill_tc_kernel(PrefillParams p,
                                                                   const __grid_constant__ CUtensorMap map_q,
                                                                   const __grid_constant__ CUtensorMap map_k,
                                                                   const __grid_constant__ CUtensorMap map_v) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t base = smem_u32(smem);
    const uint32_t bar0 = base + TcSmem::bars;
    volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(smem + TcSmem::misc);
    volatile int* s_abort = reinterpret_cast<volatile int*>(smem + TcSmem::misc + 4);
    auto bar = [&](int which, int idx = 0) { return bar0 + uint32_t(which + idx) * 8; };

    const int b = blockIdx.z, h = blockIdx.y;
    const int qt = int(gridDim.x) - 1 - int(blockIdx.x);    // longest rows first
    int lq, lk, q0 = 0;
    int64_t q_base;
    if (PAGED) {
        q0 = p.cu_q[b];
        lq = p.cu_q[b + 1] - q0;
        lk = p.cu_k[b + 1] - p.cu_k[b];
        q_base = int64_t(q0) * p.q_row_stride + int64_t(h) * p.q_head_stride;
    } else {
        lq = lk = p.seq_len;
        q_base = int64_t(b) * p.q_batch_stride + int64_t(h) * p.q_head_stride;
    }
    if (qt * kTcRows >= lq) return;                          // whole CTA leaves before any barrier or TMEM use
    const int shift = lk - lq;
    const int last_row = min(lq, qt * kTcRows + kTcRows) - 1;
    const int n_kt = (shift + last_row) / kTcKeys + 1;
    const int kvh = h / p.group;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(bar(Q_FULL), 1);
        for (int i = 0; i < kTcStages; ++i) {
            mbar_init(bar(K_FULL, i), 1);
            mbar_init(bar(K_EMPTY, i), 1);
            mbar_init(bar(V_FULL, i), 1);
            mbar_init(bar(V_EMPTY, i), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar(S_FULL, i), 1);
            mbar_init(bar(S_EMPTY, i), kTcSoftmaxWarps * 32);
            mbar_init(bar(P_FULL, i), kTcSoftmaxWarps * 32);
            mbar_init(bar(P_EMPTY, i), 1);
        }
        mbar_init(bar(PV_DONE), 1);
        mbar_init(bar(DRAIN), 1);
        *s_abort = 0;
        fence_mbar_init();
        fence_proxy_async();
    }
    if (warp == kTcMmaWarp) {
        // all 512 columns: S0, S1, O, P0, P1 (one CTA per SM by shared-memory use)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(base + uint32_t(TcSmem::misc)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *s_tmem;
    bool ok = true;

    if (warp == kTcProducerWarp) {
        // ================================================================= TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&map_q);
            tma_prefetch_desc(&map_k);
            tma_prefetch_desc(&map_v);
            mbar_expect_tx(bar(Q_FULL), kTcTile);
            for (int half = 0; half < 2; ++half) {
                if (PAGED) tma_load_3d(base + TcSmem::q + half * kTcHalf, &map_q, bar(Q_FULL), half * 64, h, q0 + qt * kTcRows);
                else tma_load_3d(base + TcSmem::q + half * kTcHalf, &map_q, bar(Q_FULL), half * 64, qt * kTcRows, b * p.n_q_heads + h);
            }
            auto load_tile = [&](const CUtensorMap* map, uint32_t dst, uint32_t full, int j) {
                int c1, c2;
                if (PAGED) {
                    const int tok0 = j * kTcKeys;
                    const int page = p.block_tables[int64_t(b) * p.bt_stride + tok0 / p.block_size];
                    c1 = kvh;
                    c2 = page * p.block_size + tok0 % p.block_size;
                } else {
                    c1 = j * kTcKeys;
                    c2 = b * p.n_kv_heads + kvh;
                }
                mbar_expect_tx(full, kTcTile);
                tma_load_3d(dst, map, full, 0, c1, c2);
                tma_load_3d(dst + kTcHalf, map, full, 64, c1, c2);
            };
            int k_issued = 0, v_issued = 0;
            // order K0, K1, V0, K2, V1, ...: K of the next tile is needed before V of this one
            for (int j = 0; j <= n_kt && ok; ++j) {
                if (j < n_kt) {
                    if (tc_wait(bar(K_EMPTY, j % kTcStages), ((j / kTcStages) & 1) ^ 1, s_abort)) {
                        load_tile(&map_k, base + TcSmem::k + (j % kTcStages) * kTcTile, bar(K_FULL, j % kTcStages), j);
                        ++k_issued;
                    } else ok = false;
                }
                if (j >= 1 && ok) {
                    const int jv = j - 1;
                    if (tc_wait(bar(V_EMPTY, jv % kTcStages), ((jv / kTcStages) & 1) ^ 1, s_abort)) {
                        load_tile(&map_v, base + TcSmem::v + (jv % kTcStages) * kTcTile, bar(V_FULL, jv % kTcStages), jv);
                        ++v_issued;
                    } else ok = false;
                }
            }
            // never leave with a copy in flight: wait (bounded) for everything that was armed
            mbar_wait(bar(Q_FULL), 0);
            for (int j = max(0, k_issued - kTcStages); j < k_issued; ++j) mbar_wait(bar(K_FULL, j % kTcStages), (j / kTcStages) & 1);
            for (int j = max(0, v_issued - kTcStages); j < v_issued; ++j) mbar_wait(bar(V_FULL, j % kTcStages), (j / kTcStages) & 1);
        }
    } else if (warp == kTcMmaWarp) {
        // ================================================================= MMA issue
        constexpr uint32_t idesc_s = tc_idesc(false), idesc_pv = tc_idesc(true);
        const uint32_t q_addr = base + TcSmem::q;
        auto issue_s = [&](int j) {      // S[j&1] = Q K_j^T
            if (!tc_wait(bar(K_FULL, j % kTcStages), (j / kTcStages) & 1, s_abort)) return false;
            if (!tc_wait(bar(S_EMPTY, j & 1), ((j >> 1) & 1) ^ 1, s_abort)) return false;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t k_addr = base + TcSmem::k + (j % kTcStages) * kTcTile;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint32_t off = (kk >> 2) * kTcHalf + (kk & 3) * 32;
                    tc_mma(tmem + (j & 1) * 128, tc_desc(q_addr + off, 16), tc_desc(k_addr + off, 16), idesc_s, kk > 0);
                }
                tc_commit(bar(S_FULL, j & 1));
                tc_commit(bar(K_EMPTY, j % kTcStages));
            }
            __syncwarp();
            return true;
        };
        if (!tc_wait(bar(Q_FULL), 0, s_abort)) ok = false;
        if (ok) ok = issue_s(0);
        for (int j = 0; j < n_kt && ok; ++j) {
            if (j + 1 < n_kt) ok = issue_s(j + 1);
            if (ok && !tc_wait(bar(V_FULL, j % kTcStages), (j / kTcStages) & 1, s_abort)) ok = false;
            if (ok && PAGED && j == n_kt - 1) {
                // keys past the end of the context: P is 0 there, but 0 * (stale bytes) must not
                // produce NaN, so clear those V rows before the tensor core reads them
                const int valid = lk - j * kTcKeys;
                if (valid < kTcKeys) {
                    uint8_t* vt = smem + TcSmem::v + (j % kTcStages) * kTcTile;
                    for (int i = valid * 8 + lane; i < kTcKeys * 8; i += 32) {
                        *reinterpret_cast<uint4*>(vt + i * 16) = make_uint4(0, 0, 0, 0);
                        *reinterpret_cast<uint4*>(vt + kTcHalf + i * 16) = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async();
                    __syncwarp();
                }
            }
            if (ok && !tc_wait(bar(P_FULL, j & 1), (j >> 1) & 1, s_abort)) ok = false;
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t v_addr = base + TcSmem::v + (j % kTcStages) * kTcTile;
                const uint32_t pj_tmem = tmem + kTmemP + (j & 1) * 64;
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t b_off = ks * 16 * 128;                         // 16 key rows of V
                    // 16 keys of P = 8 packed columns
                    tc_mma_ts(tmem + kTmemO, pj_tmem + ks * 8, tc_desc(v_addr + b_off, kTcHalf), idesc_pv,
                              (j > 0 || ks > 0) ? 1u : 0u);
                }
                tc_commit(bar(PV_DONE));
                tc_commit(bar(V_EMPTY, j % kTcStages));
                tc_commit(bar(P_EMPTY, j & 1));
            }
            __syncwarp();
        }
        // all tensor-core work issued by this warp must have retired before TMEM is freed
        if (lane == 0) tc_commit(bar(DRAIN));
        __syncwarp();
        mbar_wait(bar(DRAIN), 0);
    } else {
        // ================================================================= softmax, two threads per row
        const int r = (warp & 3) * 32 + lane;                      // row in the tile == TMEM lane
        const int ch = warp >> 2;                                  // column half: keys / dims [64 ch, 64 ch + 64)
        const uint32_t lane_sel = uint32_t((warp & 3) * 32) << 16;
        const int row = qt * kTcRows + r;
        const int pos = shift + row;
        const int cta_first_pos = shift + qt * kTcRows;
        const uint32_t o_addr = tmem + lane_sel + kTmemO + ch * 64;
        __nv_bfloat16* s_xchg = reinterpret_cast<__nv_bfloat16*>(smem + TcSmem::xchg);
        float m_ref = -INFINITY, l_run = 0.f;                      // reference maximum (log2 domain), partial row sum
        auto softmax_bar = [] { asm volatile("bar.sync 2, 256;" ::: "memory"); };

        // Every thread executes exactly one softmax_bar() per tile, whatever happened to its
        // waits: the named barrier is not bounded, so nobody may skip it.
        for (int j = 0; j < n_kt; ++j) {
            if (ok && !tc_wait(bar(S_FULL, j & 1), (j >> 1) & 1, s_abort)) ok = false;
            uint32_t sv[64];
            float mx = -INFINITY;
            const int key0 = j * kTcKeys + ch * 64;
            const int limit = pos - key0;                            // local columns <= limit are visible
            if (ok) {
                tc_fence_after();
                const uint32_t s_addr = tmem + lane_sel + (j & 1) * 128 + ch * 64;
                tc_ld32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
                tc_ld32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
                tc_wait_ld();
                tc_fence_before();
                mbar_arrive(bar(S_EMPTY, j & 1));                    // S_{j+2} may overwrite this buffer
                if (j * kTcKeys + kTcKeys - 1 > cta_first_pos) {     // tile touches the diagonal or the context end
#pragma unroll
                    for (int i = 0; i < 64; ++i) {
                        if (i > limit) sv[i] = 0xff800000u;          // -inf
                        mx = fmaxf(mx, __uint_as_float(sv[i]));
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 64; ++i) mx = fmaxf(mx, __uint_as_float(sv[i]));
                }
                // The two threads of a row must agree on the maximum bit for bit: both use the
                // two halves' maxima rounded up to bf16 (any upper-ish reference is valid).
                const __nv_bfloat16 mxr = __float2bfloat16_ru(mx);
                s_xchg[((j & 1) * 2 + ch) * 128 + r] = mxr;
                mx = __bfloat162float(mxr);
            }
            softmax_bar();
            if (!ok) continue;
            mx = fmaxf(mx, __bfloat162float(s_xchg[((j & 1) * 2 + (ch ^ 1)) * 128 + r])) * p.scale_log2;
            // move the reference only when the maximum outgrew it by more than 2^kLazyLog2
            const bool move = mx > m_ref + kLazyLog2 || (m_ref == -INFINITY && mx > -INFINITY);
            if (__any_sync(0xffffffffu, move)) {
                const float m_new = move ? mx : m_ref;
                const float alpha = m_ref == -INFINITY ? 0.f : fast_exp2(m_ref - m_new);
                if (j > 0) {
                    // O holds tiles < j once P V_{j-1} has retired; P V_j cannot start before P_FULL below
                    if (!tc_wait(bar(PV_DONE), (j - 1) & 1, s_abort)) { ok = false; continue; }
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        uint32_t v[32];
                        tc_ld32(o_addr + c * 32, v);
                        tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                        tc_st32(o_addr + c * 32, v);
                    }
                    tc_wait_st();
                }
                l_run *= alpha;
                m_ref = m_new;
            }
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;

            if (!tc_wait(bar(P_EMPTY, j & 1), ((j >> 1) & 1) ^ 1, s_abort)) { ok = false; continue; }
            uint32_t pk[32];                                         // this thread's 64 keys, two per column
            float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float e0 = fast_exp2(fmaf(__uint_as_float(sv[2 * i]), p.scale_log2, -m_use));
                const float e1 = fast_exp2(fmaf(__uint_as_float(sv[2 * i + 1]), p.scale_log2, -m_use));
                rs0 += e0;
                rs1 += e1;
                pk[i] = pack_bf16(e0, e1);
            }
            l_run += rs0 + rs1;
            tc_st32(tmem + lane_sel + kTmemP + (j & 1) * 64 + ch * 32, pk);
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(bar(P_FULL, j & 1));
        }
        // O is complete once the last P V has retired
        if (ok && !tc_wait(bar(PV_DONE), (n_kt - 1) & 1, s_abort)) ok = false;
        // row sum = the two halves' partial sums (same reference maximum in both); every
        // tensor-core read of the tiles has retired, so the Q tile's memory is free for the exchange
        float* s_sum = reinterpret_cast<float*>(smem + TcSmem::q);
        s_sum[ch * 128 + r] = l_run;
        softmax_bar();
        l_run += s_sum[(ch ^ 1) * 128 + r];
        if (ok) {
            tc_fence_after();
            const float inv = 1.f / l_run;
            __nv_bfloat16* dst = p.out + q_base + int64_t(row) * p.q_row_stride + ch * 64;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t v[32];
                tc_ld32(o_addr + c * 32, v);
                tc_wait_ld();
                if (row < lq) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c * 32 + i) = w;
                    }
                }
            }
            tc_fence_before();
        }
    }

    // ===================================================================== common epilogue
    tc_fence_before();
    __syncthreads();
    if (warp == kTcMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
    if (threadIdx.x == 0 && *s_abort && p.status) atomicExch(p.status, 0x5AFE0005);
}

int launch_prefill_tc(bool paged, const PrefillParams& p, const CUtensorMap& mq, const CUtensorMap& mk,
                      const CUtensorMap& mv, int max_q, int batch, cudaStream_t st) {
    if (max_q <= 0 || batch <= 0) return INFER_OK;
    dim3 grid((max_q + kTcRows - 1) / kTcRows, p.n_q_heads, batch);
    const int smem = TcSmem::total + 1024;
    if (paged) {
        IB_CUDA(cudaFuncSetAttribute(prefill_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        prefill_tc_kernel<true><<<grid, kTcThreads, smem, st>>>(p, mq, mk, mv);
    } else {
        IB_CUDA(cudaFuncSetAttribute(prefill_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        prefill_tc_kernel<false><<<grid, kTcThreads, smem, st>>>(p, mq, mk, mv);
    }
    return check_launch();
}

}  // namespace ib
