// Causal attention over many query rows on the 5th-generation tensor cores (tcgen05).
//
// One CTA works on TWO query tiles of 128 rows that share every K/V tile: the two query heads
// of a GQA pair over the same 128 rows (even group size), or two consecutive 128-row blocks
// of one head.  Per 128-key tile and query tile:
//   S = Q K^T        tcgen05.mma, A = Q and B = K from shared memory (K-major, 128-byte
//                    swizzle, written by TMA), accumulator in tensor memory (128 columns)
//   softmax          one warpgroup per query tile, one thread per query row = one TMEM lane:
//                    tcgen05.ld of the whole row into registers, running max / sum in
//                    registers, P written to tensor memory as packed bf16
//   O += P V         tcgen05.mma, A = P from tensor memory, B = V (MN-major: dims contiguous),
//                    the accumulator stays in tensor memory for the whole key loop
// Tensor memory (512 columns): ONE S buffer that the two query tiles take turns on (a row of
// S only lives there from the end of its product until its warpgroup has copied it to
// registers), P of tile 0, P of tile 1 (64 columns each), O of tile 0, O of tile 1.  Because P
// has its own columns, S_i(j+1) does not have to wait for P V_i(j): the tensor core computes
// the next S of a tile while that tile's warpgroup is still in the softmax of the current
// one, so neither waits for the other in the steady state.
// The softmax keeps a reference maximum per row and only moves it (rescaling the row of O in
// tensor memory and the running sum) when the true maximum has grown by more than 2^8; the
// result is exact because O and the sum always share the same reference.
// Warp roles: 0-3 softmax of tile 0, 4-7 softmax of tile 1, 8 TMA producer, 9 issue of the S
// products and TMEM allocation, 10 issue of the P V products, 11 idle (8-11 make up the third
// warpgroup, which hands 64 registers per
// thread to the softmax warpgroups with setmaxnreg so that a whole 128-column row of S fits in
// registers).  The softmax arithmetic uses packed f32x2 instructions and 3-input max.  Every
// barrier wait is bounded; a wait that runs out raises a CTA-wide abort flag, every role
// drains to the common epilogue, TMEM is freed and a status is set.
#include <atomic>

#include "prefill.cuh"

namespace ib {

constexpr int kTcRows = 128;                 // query rows per query tile (= TMEM lanes)
constexpr int kTcKeys = 128;                 // keys per K/V tile
constexpr int kTcHalf = 128 * 128;           // bytes of one [128 rows][64 elems] swizzled sub-tile
constexpr int kTcTile = 2 * kTcHalf;         // 32 KiB: one Q, K or V tile
constexpr int kTcQTiles = 2;                 // query tiles per CTA, each with its own softmax warpgroup
constexpr int kTcSoftmaxWarps = 4 * kTcQTiles;
constexpr int kTcProducerWarp = kTcSoftmaxWarps, kTcMmaWarp = kTcSoftmaxWarps + 1;
constexpr int kTcThreads = (kTcSoftmaxWarps + 4) * 32;   // third warpgroup: producer, MMA issue, two idle warps
constexpr int kTcKStages = 3, kTcVStages = 2;
// tensor memory columns: S (shared by the two tiles) at 0, P of tile i (bf16, two keys per column) at
// 128 + 64 i, O of tile i at 256 + 128 i
constexpr uint32_t kTmemP = 128, kTmemO = 256;

struct TcSmem {
    static constexpr int q = 0;                              // kTcQTiles tiles
    static constexpr int k = q + kTcQTiles * kTcTile;
    static constexpr int v = k + kTcKStages * kTcTile;
    static constexpr int bars = v + kTcVStages * kTcTile;    // 8-byte mbarriers
    static constexpr int n_bars = 24;
    static constexpr int misc = bars + n_bars * 8;           // tmem base, abort flag
    static constexpr int total = misc + 16;
};

enum TcBar { Q_FULL = 0, K_FULL = 1, K_EMPTY = 4, V_FULL = 7, V_EMPTY = 9, S_FULL = 11, P_FULL = 13, PV_DONE = 15,
             DRAIN = 17 /* two */, S_FREE = 19 };
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

// packed pairs of f32 (sm_100 executes add/mul/fma on two floats per instruction)
__device__ __forceinline__ uint64_t pk2(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void upk2(uint64_t v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t fadd2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
// One lane of the (converged) warp, chosen by the hardware: unlike a test of the lane number
// this keeps the compiler's view of the branch uniform, which matters for the instructions that
// feed tcgen05.mma its descriptors (measured: 1208 -> 1230 TFLOP/s).
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
// Bounded wait that also gives up as soon as another thread raised the abort flag.  One test
// in front of the polling loop: a wait on a phase that is already complete then costs a test
// and a branch (about 35 clocks) instead of a trip through the loop (about 210 as measured).
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t limit) {
    if (mbar_try_wait(bar, parity)) return true;
    uint32_t i = 0;
#pragma unroll 1
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++i & 63) == 0) {
            if (*abort_flag) return false;
            if (i >= limit) break;
            __nanosleep(i > 4096 ? 256 : 32);
        }
    }
    *abort_flag = 1;
    return false;
}

// Which (head, row block) the two query tiles of a CTA are.
struct TcTile {
    int head, row0, n_kt, lq_left;   // lq_left: valid rows of the tile (<= 0: tile inactive)
};

template <bool PAGED>
__global__ void __launch_bounds__(kTcThreads, 1) prefill_tc_kernel(PrefillParams p, int pair_heads,
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

    const int b = blockIdx.z;
    const int xb = int(gridDim.x) - 1 - int(blockIdx.x);    // longest rows first
    int lq, lk, q0 = 0;
    if (PAGED) {
        q0 = p.cu_q[b];
        lq = p.cu_q[b + 1] - q0;
        lk = p.cu_k[b + 1] - p.cu_k[b];
    } else {
        lq = lk = p.seq_len;
    }
    const int shift = lk - lq;
    TcTile tile[kTcQTiles];
#pragma unroll
    for (int i = 0; i < kTcQTiles; ++i) {
        tile[i].head = pair_heads ? int(blockIdx.y) * 2 + i : int(blockIdx.y);
        tile[i].row0 = pair_heads ? xb * kTcRows : (xb * kTcQTiles + i) * kTcRows;
        tile[i].lq_left = lq - tile[i].row0;
        tile[i].n_kt = tile[i].lq_left > 0 ? (shift + min(lq, tile[i].row0 + kTcRows) - 1) / kTcKeys + 1 : 0;
    }
    if (tile[0].n_kt == 0) return;                           // whole CTA leaves before any barrier or TMEM use
    const int n_max = max(tile[0].n_kt, tile[1].n_kt);
    const int kvh = tile[0].head / p.group;                  // both tiles read the same kv head
    // Roles are numbered as in the header comment, but the third warpgroup's roles (producer, MMA
    // issue) sit in the FIRST four hardware warps: when several warps of a scheduler are ready the
    // oldest one goes first, and the MMA issue warp, which has little to do but whose every
    // instruction is on the tensor core's critical path, must not queue behind the softmax warps.
    const int warp = (int(threadIdx.x >> 5) + kTcSoftmaxWarps) % (kTcThreads / 32), lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(bar(Q_FULL), 1);
        for (int i = 0; i < kTcKStages; ++i) {
            mbar_init(bar(K_FULL, i), 1);
            mbar_init(bar(K_EMPTY, i), 1);
        }
        for (int i = 0; i < kTcVStages; ++i) {
            mbar_init(bar(V_FULL, i), 1);
            mbar_init(bar(V_EMPTY, i), 1);
        }
        for (int i = 0; i < kTcQTiles; ++i) {
            mbar_init(bar(S_FULL, i), 1);
            mbar_init(bar(P_FULL, i), 128);
            mbar_init(bar(PV_DONE, i), 1);
        }
        mbar_init(bar(DRAIN, 0), 1);
        mbar_init(bar(DRAIN, 1), 1);
        mbar_init(bar(S_FREE), 128);             // the warpgroup that copied the S buffer to registers
        *s_abort = 0;
        fence_mbar_init();
        fence_proxy_async();
    }
    if (warp == kTcMmaWarp) {
        // all 512 columns (one CTA per SM by shared-memory use)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(base + uint32_t(TcSmem::misc)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = __shfl_sync(0xffffffffu, *s_tmem, 0);   // warp-uniform by construction
    bool ok = true;

    // Register budget: 384 threads x 168 at launch.  The third warpgroup gives 64 registers per
    // thread back, the two softmax warpgroups grow to 200: they hold a 128-column row of S.
    // (each role adjusts its own budget first thing in its branch, so that the compiler sees it)
    if (warp >= kTcSoftmaxWarps) {
    // one instruction for the whole third warpgroup, before its warps take their roles
    asm volatile("setmaxnreg.dec.sync.aligned.u32 104;" ::: "memory");
    if (warp == kTcProducerWarp) {
        // ================================================================= TMA producer
        if (lane == 0 && !p.stall_producer) {
            tma_prefetch_desc(&map_q);
            tma_prefetch_desc(&map_k);
            tma_prefetch_desc(&map_v);
            const int n_q = tile[1].n_kt > 0 ? 2 : 1;
            mbar_expect_tx(bar(Q_FULL), n_q * kTcTile);
            for (int i = 0; i < n_q; ++i)
                for (int half = 0; half < 2; ++half) {
                    const uint32_t dst = base + TcSmem::q + i * kTcTile + half * kTcHalf;
                    if (PAGED) tma_load_3d(dst, &map_q, bar(Q_FULL), half * 64, tile[i].head, q0 + tile[i].row0);
                    else tma_load_3d(dst, &map_q, bar(Q_FULL), half * 64, tile[i].row0, b * p.n_q_heads + tile[i].head);
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
            for (int j = 0; j <= n_max && ok; ++j) {
                if (j < n_max) {
                    if (tc_wait(bar(K_EMPTY, j % kTcKStages), ((j / kTcKStages) & 1) ^ 1, s_abort, p.wait_limit)) {
                        load_tile(&map_k, base + TcSmem::k + (j % kTcKStages) * kTcTile, bar(K_FULL, j % kTcKStages), j);
                        ++k_issued;
                    } else ok = false;
                }
                if (j >= 1 && ok) {
                    const int jv = j - 1;
                    if (tc_wait(bar(V_EMPTY, jv % kTcVStages), ((jv / kTcVStages) & 1) ^ 1, s_abort, p.wait_limit)) {
                        load_tile(&map_v, base + TcSmem::v + (jv % kTcVStages) * kTcTile, bar(V_FULL, jv % kTcVStages), jv);
                        ++v_issued;
                    } else ok = false;
                }
            }
            // never leave with a copy in flight: wait (bounded) for everything that was armed
            mbar_wait(bar(Q_FULL), 0, p.wait_limit);
            for (int j = max(0, k_issued - kTcKStages); j < k_issued; ++j) mbar_wait(bar(K_FULL, j % kTcKStages), (j / kTcKStages) & 1, p.wait_limit);
            for (int j = max(0, v_issued - kTcVStages); j < v_issued; ++j) mbar_wait(bar(V_FULL, j % kTcVStages), (j / kTcVStages) & 1, p.wait_limit);
        }
    } else if (warp == kTcMmaWarp) {
        // ================================================================= MMA issue: the S products
        // S_0(0) S_1(0) S_0(1) S_1(1) ...: an S product may start once the warpgroup of the previous
        // one has copied the S buffer to registers (S_FREE, one phase per S product).  The P V
        // products are issued by the next warp: under the softmax warps' instruction stream the
        // descriptor arithmetic and barrier tests of one issuing thread take longer than the
        // products they lead to, two threads keep the tensor core fed.
        constexpr uint32_t idesc_s = tc_idesc(false);
        const int kt0 = tile[0].n_kt, kt1 = tile[1].n_kt;
        // descriptors differ from operand tile to operand tile only in the 14-bit start address
        // (16-byte units) at the bottom of the low word
        const uint64_t q_desc0 = tc_desc(base + TcSmem::q, 16), k_desc0 = tc_desc(base + TcSmem::k, 16);
        int n_s = 0;                               // S products issued so far
        auto issue_s = [&](int i, int stage) {     // S = Q_i K^T  (K_FULL of that stage already awaited)
            if (n_s > 0 && !tc_wait(bar(S_FREE), (n_s - 1) & 1, s_abort, p.wait_limit)) { ok = false; return; }
            ++n_s;
            tc_fence_after();
            if (elect_one()) {
                const uint64_t qd = q_desc0 + uint64_t(i * (kTcTile >> 4));
                const uint64_t kd = k_desc0 + uint64_t(stage * (kTcTile >> 4));
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint32_t off = ((kk >> 2) * kTcHalf + (kk & 3) * 32) >> 4;
                    tc_mma(tmem, qd + off, kd + off, idesc_s, kk > 0);
                }
                tc_commit(bar(S_FULL, i));
            }
            __syncwarp();
        };
        if (!tc_wait(bar(Q_FULL), 0, s_abort, p.wait_limit)) ok = false;
        int ks = 0, kph = 0;                                           // stage and phase of K_j
        for (int j = 0; j < n_max && ok; ++j) {
            if (!tc_wait(bar(K_FULL, ks), kph, s_abort, p.wait_limit)) { ok = false; break; }
            if (j < kt0) issue_s(0, ks);
            if (ok && j < kt1) issue_s(1, ks);
            if (!ok) break;
            if (elect_one()) tc_commit(bar(K_EMPTY, ks));                 // both S(j) are issued
            __syncwarp();
            if (++ks == kTcKStages) { ks = 0; kph ^= 1; }
        }
        // all tensor-core work issued by this warp must have retired before TMEM is freed
        if (elect_one()) tc_commit(bar(DRAIN, 0));
        __syncwarp();
        mbar_wait(bar(DRAIN, 0), 0, p.wait_limit);
    } else if (warp == kTcMmaWarp + 1) {
        // ================================================================= MMA issue: the P V products
        // P V_0(0) P V_1(0) P V_0(1) ...: each once its warpgroup has written P.
        constexpr uint32_t idesc_pv = tc_idesc(true);
        const int kt0 = tile[0].n_kt, kt1 = tile[1].n_kt;
        const uint64_t v_desc0 = tc_desc(base + TcSmem::v, kTcHalf);
        auto issue_pv = [&](int i, int stage, int j) {   // O_i += P_i V  (V_FULL of that stage already awaited)
            if (!tc_wait(bar(P_FULL, i), j & 1, s_abort, p.wait_limit)) { ok = false; return; }
            tc_fence_after();
            if (elect_one()) {
                const uint64_t vd = v_desc0 + uint64_t(stage * (kTcTile >> 4));
                const uint32_t p_tmem = tmem + kTmemP + i * 64;
#pragma unroll
                for (int kk = 0; kk < 8; ++kk)     // 16 keys: 8 packed columns of P, 16 rows of V
                    tc_mma_ts(tmem + kTmemO + i * 128, p_tmem + kk * 8, vd + uint32_t(kk * 16 * 128 >> 4), idesc_pv,
                              (j > 0 || kk > 0) ? 1u : 0u);
                tc_commit(bar(PV_DONE, i));
            }
            __syncwarp();
        };
        int vs = 0, vph = 0;                                           // stage and phase of V_j
        for (int j = 0; j < n_max && ok; ++j) {
            if (!tc_wait(bar(V_FULL, vs), vph, s_abort, p.wait_limit)) { ok = false; break; }
            if (PAGED && j == n_max - 1) {
                // keys past the end of the context: P is 0 there, but 0 * (stale bytes) must not
                // produce NaN, so clear those V rows before the tensor core reads them
                const int valid = lk - j * kTcKeys;
                if (valid < kTcKeys) {
                    uint8_t* vt = smem + TcSmem::v + vs * kTcTile;
                    for (int x = valid * 8 + lane; x < kTcKeys * 8; x += 32) {
                        *reinterpret_cast<uint4*>(vt + x * 16) = make_uint4(0, 0, 0, 0);
                        *reinterpret_cast<uint4*>(vt + kTcHalf + x * 16) = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async();
                    __syncwarp();
                }
            }
            if (j < kt0) issue_pv(0, vs, j);
            if (ok && j < kt1) issue_pv(1, vs, j);
            if (!ok) break;
            if (elect_one()) tc_commit(bar(V_EMPTY, vs));                 // both products with V_j are issued
            __syncwarp();
            if (++vs == kTcVStages) { vs = 0; vph ^= 1; }
        }
        if (elect_one()) tc_commit(bar(DRAIN, 1));
        __syncwarp();
        mbar_wait(bar(DRAIN, 1), 0, p.wait_limit);
    }
    } else {
        // ================================================================= softmax, one row per thread
        asm volatile("setmaxnreg.inc.sync.aligned.u32 200;" ::: "memory");
        const int g = warp >> 2;                                   // query tile of this warpgroup
        const int r = (warp & 3) * 32 + lane;                      // row in the tile == TMEM lane
        const uint32_t lane_sel = uint32_t((warp & 3) * 32) << 16;
        const int n_kt = tile[g].n_kt;
        const int row = tile[g].row0 + r;
        const int pos = shift + row;
        const int tile_first_pos = shift + tile[g].row0;
        const uint32_t s_addr = tmem + lane_sel;                   // the S buffer is shared by the two tiles
        const uint32_t p_addr = tmem + lane_sel + kTmemP + g * 64;
        const uint32_t o_addr = tmem + lane_sel + kTmemO + g * 128;
        float m_ref = -INFINITY, l_run = 0.f;                      // reference maximum (log2 domain), row sum

        for (int j = 0; j < n_kt; ++j) {
            if (ok && !tc_wait(bar(S_FULL, g), j & 1, s_abort, p.wait_limit)) ok = false;
            if (!ok) continue;
            tc_fence_after();
            const int limit = pos - j * kTcKeys;                     // columns <= limit are visible
            const bool masked = j * kTcKeys + kTcKeys - 1 > tile_first_pos;
            // the whole row of S in registers
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
            uint32_t sv[128];
            tc_ld32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
            tc_ld32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
            tc_ld32(s_addr + 64, *reinterpret_cast<uint32_t(*)[32]>(&sv[64]));
            tc_ld32(s_addr + 96, *reinterpret_cast<uint32_t(*)[32]>(&sv[96]));
            tc_wait_ld();
            // the row is in registers: the tensor core may overwrite the S buffer
            tc_fence_before();
            mbar_arrive(bar(S_FREE));
            if (masked) {
#pragma unroll
                for (int i = 0; i < 128; ++i)
                    if (i > limit) sv[i] = 0xff800000u;              // -inf
            }
#pragma unroll
            for (int i = 0; i < 128; i += 8) {
                mx0 = fmax3(mx0, __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
                mx1 = fmax3(mx1, __uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3]));
                mx2 = fmax3(mx2, __uint_as_float(sv[i + 4]), __uint_as_float(sv[i + 5]));
                mx3 = fmax3(mx3, __uint_as_float(sv[i + 6]), __uint_as_float(sv[i + 7]));
            }
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;
            // move the reference only when the maximum outgrew it by more than 2^kLazyLog2
            const bool move = mx > m_ref + kLazyLog2 || (m_ref == -INFINITY && mx > -INFINITY);
            if (__any_sync(0xffffffffu, move)) {
                const float m_new = move ? mx : m_ref;
                const float alpha = m_ref == -INFINITY ? 0.f : fast_exp2(m_ref - m_new);
                if (j > 0) {
                    // O holds tiles < j once P V_{j-1} has retired; P V_j cannot start before P_FULL below
                    if (!tc_wait(bar(PV_DONE, g), (j - 1) & 1, s_abort, p.wait_limit)) { ok = false; continue; }
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
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
            // the tensor core must be done reading P of the previous key tile (long since, as a rule)
            if (j > 0 && !tc_wait(bar(PV_DONE, g), (j - 1) & 1, s_abort, p.wait_limit)) { ok = false; continue; }
            // P = exp2(S * c - m) as packed bf16
            uint64_t rsa = pk2(0.f, 0.f), rsb = pk2(0.f, 0.f);
            const uint64_t c2 = pk2(p.scale_log2, p.scale_log2), nm2 = pk2(-m_use, -m_use);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t pk[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int c = h * 64 + 2 * i;
                    const uint64_t x2 = ffma2(pk2(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])), c2, nm2);
                    float e0, e1;
                    upk2(x2, e0, e1);
                    e0 = fast_exp2(e0);
                    e1 = fast_exp2(e1);
                    if (i & 1) rsb = fadd2(rsb, pk2(e0, e1)); else rsa = fadd2(rsa, pk2(e0, e1));
                    pk[i] = pack_bf16(e0, e1);
                }
                tc_st32(p_addr + h * 32, pk);
            }
            float rs0, rs1, rs2, rs3;
            upk2(rsa, rs0, rs1);
            upk2(rsb, rs2, rs3);
            l_run += (rs0 + rs1) + (rs2 + rs3);
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(bar(P_FULL, g));
        }
        // O is complete once the last P V has retired
        if (n_kt > 0 && ok && !tc_wait(bar(PV_DONE, g), (n_kt - 1) & 1, s_abort, p.wait_limit)) ok = false;
        if (n_kt > 0 && ok) {
            tc_fence_after();
            const float inv = 1.f / l_run;
            int64_t q_base;
            if (PAGED) q_base = int64_t(q0) * p.q_row_stride + int64_t(tile[g].head) * p.q_head_stride;
            else q_base = int64_t(b) * p.q_batch_stride + int64_t(tile[g].head) * p.q_head_stride;
            __nv_bfloat16* dst = p.out + q_base + int64_t(row) * p.q_row_stride;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t v[32];
                tc_ld32(o_addr + c * 32, v);
                tc_wait_ld();
                if (r < tile[g].lq_left) {
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
    // an even group lets the two query tiles of a CTA be the two heads of a GQA pair (same rows,
    // same kv head); otherwise they are two consecutive row blocks of one head
    const int pair_heads = p.group % 2 == 0 ? 1 : 0;
    dim3 grid = pair_heads ? dim3((max_q + kTcRows - 1) / kTcRows, p.n_q_heads / 2, batch)
                           : dim3((max_q + kTcQTiles * kTcRows - 1) / (kTcQTiles * kTcRows), p.n_q_heads, batch);
    const int smem = TcSmem::total + 1024;
    // the shared-memory limit of the two instantiations is raised once per device
    static std::atomic<bool> prepared[64];
    int dev = 0;
    IB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !prepared[dev].load(std::memory_order_acquire)) {
        IB_CUDA(cudaFuncSetAttribute(prefill_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        IB_CUDA(cudaFuncSetAttribute(prefill_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        if (dev >= 0 && dev < 64) prepared[dev].store(true, std::memory_order_release);
    }
    if (paged) prefill_tc_kernel<true><<<grid, kTcThreads, smem, st>>>(p, pair_heads, mq, mk, mv);
    else prefill_tc_kernel<false><<<grid, kTcThreads, smem, st>>>(p, pair_heads, mq, mk, mv);
    return check_launch();
}

}  // namespace ib
