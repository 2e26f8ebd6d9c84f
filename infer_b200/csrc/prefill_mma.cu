// Causal attention over many query rows (chunked prefill over pages, and the dense
// [B,H,S,128] op) on the mma.sync tensor path: 64 query rows per CTA (16 per warp), K/V
// tiles of 64 tokens staged by a producer warp with TMA into a 3-stage ring, online softmax
// in registers.  The same kernel serves both layouts; only the TMA coordinates differ.
#include "prefill.cuh"

namespace ib {

constexpr int kPfStages = 3;
constexpr int kPfTile = 64;                      // keys per tile
constexpr int kPfTileBytes = kPfTile * 256;      // K (or V) bytes per stage
constexpr int kPfWarps = 4;
constexpr int kPfThreads = (kPfWarps + 1) * 32;
constexpr int kPfSmem = kPfStages * 2 * kPfTileBytes + 2 * kPfStages * 8 + 1024;

template <bool PAGED>
__global__ void __launch_bounds__(kPfThreads) prefill_mma_kernel(PrefillParams p,
                                                                 const __grid_constant__ CUtensorMap map_k,
                                                                 const __grid_constant__ CUtensorMap map_v) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t tiles_u32 = smem_u32(smem);
    const uint32_t full0 = tiles_u32 + kPfStages * 2 * kPfTileBytes, empty0 = full0 + kPfStages * 8;

    const int b = blockIdx.z, h = blockIdx.y;
    const int qt = int(gridDim.x) - 1 - int(blockIdx.x);   // longest rows first
    int lq, lk;
    int64_t q_base;
    if (PAGED) {
        const int q0 = p.cu_q[b];
        lq = p.cu_q[b + 1] - q0;
        lk = p.cu_k[b + 1] - p.cu_k[b];
        q_base = int64_t(q0) * p.q_row_stride + int64_t(h) * p.q_head_stride;
    } else {
        lq = lk = p.seq_len;
        q_base = int64_t(b) * p.q_batch_stride + int64_t(h) * p.q_head_stride;
    }
    if (qt * 64 >= lq) return;
    const int shift = lk - lq;                              // query row i sits at key position shift + i
    const int last_row = min(lq, qt * 64 + 64) - 1;
    const int n_kt = (shift + last_row) / kPfTile + 1;
    const int kvh = h / p.group;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kPfStages; ++s) {
            mbar_init(full0 + s * 8, 1);
            mbar_init(empty0 + s * 8, kPfWarps);
        }
        fence_mbar_init();
        fence_proxy_async();
    }
    __syncthreads();

    if (warp == kPfWarps) {
        if (lane != 0) return;
        bool ok = true;
        int kt = 0;
        for (; kt < n_kt; ++kt) {
            const uint32_t s = kt % kPfStages, ph = (kt / kPfStages) & 1;
            if (!mbar_wait(empty0 + s * 8, ph ^ 1)) { ok = false; break; }
            const uint32_t bar = full0 + s * 8;
            const uint32_t kdst = tiles_u32 + s * (2 * kPfTileBytes), vdst = kdst + kPfTileBytes;
            mbar_expect_tx(bar, 2 * kPfTileBytes);
            int c1, c2;
            if (PAGED) {
                const int tok0 = kt * kPfTile;
                const int page = p.block_tables[int64_t(b) * p.bt_stride + tok0 / p.block_size];
                c1 = kvh;
                c2 = page * p.block_size + tok0 % p.block_size;
            } else {
                c1 = kt * kPfTile;
                c2 = b * p.n_kv_heads + kvh;
            }
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                tma_load_3d(kdst + half * (kPfTile * 128), &map_k, bar, half * 64, c1, c2);
                tma_load_3d(vdst + half * (kPfTile * 128), &map_v, bar, half * 64, c1, c2);
            }
        }
        const int armed = kt < kPfStages ? kt : kPfStages;
        for (int j = 0; j < armed; ++j) {
            const int i2 = kt - 1 - j;
            if (!mbar_wait(full0 + (i2 % kPfStages) * 8, (i2 / kPfStages) & 1)) ok = false;
        }
        if (!ok && p.status) atomicExch(p.status, 0x5AFE0003);
        return;
    }

    // ------------------------------------------------------------------ consumers
    const int gid = lane >> 2, tig = lane & 3;
    const int mi = lane >> 3, mr = lane & 7;
    const int row0 = qt * 64 + warp * 16 + gid, row1 = row0 + 8;    // query rows of this thread
    uint32_t qa[8][4];
    {
        const uint32_t* r0p = reinterpret_cast<const uint32_t*>(p.q + q_base + int64_t(min(row0, lq - 1)) * p.q_row_stride);
        const uint32_t* r1p = reinterpret_cast<const uint32_t*>(p.q + q_base + int64_t(min(row1, lq - 1)) * p.q_row_stride);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
            qa[kk][0] = r0p[kk * 8 + tig];
            qa[kk][1] = r1p[kk * 8 + tig];
            qa[kk][2] = r0p[kk * 8 + 4 + tig];
            qa[kk][3] = r1p[kk * 8 + 4 + tig];
        }
    }
    float o[16][4];
#pragma unroll
    for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int pos0 = shift + row0, pos1 = shift + row1;
    const int warp_first_pos = shift + qt * 64 + warp * 16;
    bool ok = true;

    for (int kt = 0; kt < n_kt; ++kt) {
        const uint32_t s = kt % kPfStages, ph = (kt / kPfStages) & 1;
        if (ok && !mbar_wait(full0 + s * 8, ph)) ok = false;
        const int key0 = kt * kPfTile;
        // keys beyond the last position any row of this warp may see need no work
        if (ok && key0 <= warp_first_pos + 15) {
            const uint32_t kbase = tiles_u32 + s * (2 * kPfTileBytes), vbase = kbase + kPfTileBytes;
            float sc[8][4];
#pragma unroll
            for (int j = 0; j < 8; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
#pragma unroll
                for (int jp = 0; jp < 4; ++jp) {
                    const int row = jp * 16 + (mi >> 1) * 8 + mr;
                    const int chunk16 = (kk & 3) * 2 + (mi & 1);
                    uint32_t b00, b01, b10, b11;
                    ldsm_x4(kbase + (kk >> 2) * (kPfTile * 128) + swz128(row, chunk16), b00, b01, b10, b11);
                    mma_bf16(sc[2 * jp], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b00, b01);
                    mma_bf16(sc[2 * jp + 1], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b10, b11);
                }
            }
            const bool need_mask = key0 + kPfTile - 1 > warp_first_pos;
            if (need_mask) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int key = key0 + j * 8 + 2 * tig;
                    if (key > pos0) sc[j][0] = -INFINITY;
                    if (key + 1 > pos0) sc[j][1] = -INFINITY;
                    if (key > pos1) sc[j][2] = -INFINITY;
                    if (key + 1 > pos1) sc[j][3] = -INFINITY;
                }
            }
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                mx0 = fmaxf(mx0, fmaxf(sc[j][0], sc[j][1]));
                mx1 = fmaxf(mx1, fmaxf(sc[j][2], sc[j][3]));
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m0, mx0 * p.scale_log2), mn1 = fmaxf(m1, mx1 * p.scale_log2);
            // a row with no visible key yet keeps max = -inf; use 0 as the exponent origin then
            const float e0 = mn0 == -INFINITY ? 0.f : mn0, e1 = mn1 == -INFINITY ? 0.f : mn1;
            const float a0 = fast_exp2(m0 - e0), a1 = fast_exp2(m1 - e1);
            float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                sc[j][0] = fast_exp2(fmaf(sc[j][0], p.scale_log2, -e0));
                sc[j][1] = fast_exp2(fmaf(sc[j][1], p.scale_log2, -e0));
                sc[j][2] = fast_exp2(fmaf(sc[j][2], p.scale_log2, -e1));
                sc[j][3] = fast_exp2(fmaf(sc[j][3], p.scale_log2, -e1));
                rs0 += sc[j][0] + sc[j][1];
                rs1 += sc[j][2] + sc[j][3];
            }
            l0 = l0 * a0 + rs0;
            l1 = l1 * a1 + rs1;
            m0 = mn0;
            m1 = mn1;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                o[j][0] *= a0; o[j][1] *= a0;
                o[j][2] *= a1; o[j][3] *= a1;
            }
            const int valid = lk - key0;    // keys of this tile that exist
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const uint32_t pa0 = pack_bf16(sc[2 * ks][0], sc[2 * ks][1]);
                const uint32_t pa1 = pack_bf16(sc[2 * ks][2], sc[2 * ks][3]);
                const uint32_t pa2 = pack_bf16(sc[2 * ks + 1][0], sc[2 * ks + 1][1]);
                const uint32_t pa3 = pack_bf16(sc[2 * ks + 1][2], sc[2 * ks + 1][3]);
#pragma unroll
                for (int n2 = 0; n2 < 8; ++n2) {
                    const int row = ks * 16 + (mi & 1) * 8 + mr;
                    const int chunk16 = (n2 & 3) * 2 + (mi >> 1);
                    uint32_t v0, v1, v2, v3;
                    ldsm_x4_trans(vbase + (n2 >> 2) * (kPfTile * 128) + swz128(row, chunk16), v0, v1, v2, v3);
                    if (PAGED && valid < kPfTile) {
                        const int t = ks * 16 + 2 * tig;
                        const uint32_t keep_lo = (t < valid ? 0x0000ffffu : 0u) | (t + 1 < valid ? 0xffff0000u : 0u);
                        const uint32_t keep_hi = (t + 8 < valid ? 0x0000ffffu : 0u) | (t + 9 < valid ? 0xffff0000u : 0u);
                        v0 &= keep_lo; v2 &= keep_lo;
                        v1 &= keep_hi; v3 &= keep_hi;
                    }
                    mma_bf16(o[2 * n2], pa0, pa1, pa2, pa3, v0, v1);
                    mma_bf16(o[2 * n2 + 1], pa0, pa1, pa2, pa3, v2, v3);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + s * 8);
    }
    if (!ok) {
        if (lane == 0 && p.status) atomicExch(p.status, 0x5AFE0004);
        return;
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const int64_t o_base = q_base;   // out has the layout of q
    if (row0 < lq) {
        const float inv = 1.f / l0;
        uint32_t* dst = reinterpret_cast<uint32_t*>(p.out + o_base + int64_t(row0) * p.q_row_stride);
#pragma unroll
        for (int j = 0; j < 16; ++j) dst[j * 4 + tig] = pack_bf16(o[j][0] * inv, o[j][1] * inv);
    }
    if (row1 < lq) {
        const float inv = 1.f / l1;
        uint32_t* dst = reinterpret_cast<uint32_t*>(p.out + o_base + int64_t(row1) * p.q_row_stride);
#pragma unroll
        for (int j = 0; j < 16; ++j) dst[j * 4 + tig] = pack_bf16(o[j][2] * inv, o[j][3] * inv);
    }
}

int launch_prefill_mma(bool paged, const PrefillParams& p, const CUtensorMap& mk, const CUtensorMap& mv,
                          int max_q, int batch, cudaStream_t st) {
    if (max_q <= 0 || batch <= 0) return INFER_OK;
    dim3 grid((max_q + 63) / 64, p.n_q_heads, batch);
    if (paged) {
        IB_CUDA(cudaFuncSetAttribute(prefill_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPfSmem));
        prefill_mma_kernel<true><<<grid, kPfThreads, kPfSmem, st>>>(p, mk, mv);
    } else {
        IB_CUDA(cudaFuncSetAttribute(prefill_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPfSmem));
        prefill_mma_kernel<false><<<grid, kPfThreads, kPfSmem, st>>>(p, mk, mv);
    }
    return check_launch();
}

}  // namespace ib
