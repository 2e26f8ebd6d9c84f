// Entry points of the prefill attention ops: argument checks, tensor maps, kernel choice.
#include <mutex>

#include "prefill.cuh"

namespace ib {

// The tcgen05 kernel is the product path.  The mma.sync kernel (prefill_mma.cu) is an on-GPU
// cross-check that only the self-test entry points can select.
struct PrefillOptions {
    bool tc = true;
    uint32_t wait_limit = kDefaultWaitLimit;
    int stall_producer = 0;
};

// Status word of the prefill kernels: lives in the library's device image (one per GPU), set to
// 0x5AFE0000 | code by a kernel whose bounded wait ran out, read and cleared by
// infer_prefill_status().  In host code the NAME is only a handle for cudaGetSymbolAddress.
static __device__ int g_prefill_status;
constexpr int kMaxDevices = 64;
static int* g_prefill_status_addr[kMaxDevices];
static std::mutex g_prefill_status_mutex;

// Device address of the status word on the current device; nullptr (the kernels then report
// nothing) if it cannot be looked up.
static int* prefill_status_word() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_prefill_status_mutex);
    if (!g_prefill_status_addr[dev]) {
        void* addr = nullptr;
        if (cudaGetSymbolAddress(&addr, g_prefill_status) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        g_prefill_status_addr[dev] = static_cast<int*>(addr);
    }
    return g_prefill_status_addr[dev];
}

static int paged_prefill(const infer_kv_pool_t* pool, void* out, const void* q, int64_t total_q,
                         const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, const int32_t* block_tables,
                         int64_t bt_stride, int batch, int max_seqlen_q, int max_seqlen_k, int n_q_heads,
                         float softmax_scale, cudaStream_t st, const PrefillOptions& opt) {
    if (!pool || !out || !q || !cu_seqlens_q || !cu_seqlens_k || !block_tables) return INFER_ERR_NULL;
    if (pool->dtype != INFER_KV_BF16) return INFER_ERR_DTYPE;
    if (batch < 0 || n_q_heads <= 0 || n_q_heads % pool->n_kv_heads != 0 || bt_stride <= 0 || max_seqlen_q < 0 ||
        max_seqlen_k < max_seqlen_q || batch > 65535 || n_q_heads > 65535 || total_q < 0 ||
        total_q > int64_t(batch) * max_seqlen_q)
        return INFER_ERR_GEOMETRY;
    if (!aligned16(out) || !aligned16(q)) return INFER_ERR_ALIGN;
    if (total_q == 0 || batch == 0) return INFER_OK;
    PrefillParams p{};
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.out = static_cast<__nv_bfloat16*>(out);
    p.q_row_stride = int64_t(n_q_heads) * kHeadDim;
    p.q_head_stride = kHeadDim;
    p.q_batch_stride = 0;
    p.cu_q = cu_seqlens_q;
    p.cu_k = cu_seqlens_k;
    p.block_tables = block_tables;
    p.bt_stride = bt_stride;
    p.n_q_heads = n_q_heads;
    p.n_kv_heads = pool->n_kv_heads;
    p.group = n_q_heads / pool->n_kv_heads;
    p.block_size = pool->block_size;
    p.seq_len = 0;
    p.scale_log2 = softmax_scale * 1.4426950408889634f;
    p.status = prefill_status_word();
    p.wait_limit = opt.wait_limit;
    p.stall_producer = opt.stall_producer;
    if (opt.tc) {
        CUtensorMap mq;   // q [total_q, Hq, 128]: rows past total_q are filled with zeros
        int rc = encode_map_3d(&mq, q, 2, kHeadDim, uint64_t(n_q_heads), uint64_t(total_q), 256,
                               uint64_t(n_q_heads) * 256, 64, 1, 128);
        if (rc != INFER_OK) return rc;
        return launch_prefill_tc(true, p, mq, pool->maps[3].k, pool->maps[3].v, max_seqlen_q, batch, st);
    }
    return launch_prefill_mma(true, p, pool->maps[2].k, pool->maps[2].v, max_seqlen_q, batch, st);
}

static int dense_prefill(const void* q, const void* k, const void* v, void* o, int batch, int n_q_heads, int n_kv_heads,
                         int seq_len, cudaStream_t st, const PrefillOptions& opt) {
    if (!q || !k || !v || !o) return INFER_ERR_NULL;
    if (batch <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads != 0 || seq_len <= 0 ||
        batch > 65535 || n_q_heads > 65535)
        return INFER_ERR_GEOMETRY;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o)) return INFER_ERR_ALIGN;
    const bool tc = opt.tc;
    const uint32_t box_rows = tc ? 128 : 64;
    CUtensorMap mq, mk, mv;
    // K, V [B, Hkv, S, 128]: dims {128, S, B*Hkv}; a box never crosses into the next head,
    // rows past S are filled with zeros.
    int rc = encode_map_3d(&mk, k, 2, kHeadDim, uint64_t(seq_len), uint64_t(batch) * n_kv_heads, 256,
                           uint64_t(seq_len) * 256, 64, box_rows, 1);
    if (rc == INFER_OK)
        rc = encode_map_3d(&mv, v, 2, kHeadDim, uint64_t(seq_len), uint64_t(batch) * n_kv_heads, 256,
                           uint64_t(seq_len) * 256, 64, box_rows, 1);
    if (rc == INFER_OK && tc)
        rc = encode_map_3d(&mq, q, 2, kHeadDim, uint64_t(seq_len), uint64_t(batch) * n_q_heads, 256,
                           uint64_t(seq_len) * 256, 64, 128, 1);
    if (rc != INFER_OK) return rc;
    PrefillParams p{};
    p.q = static_cast<const __nv_bfloat16*>(q);
    p.out = static_cast<__nv_bfloat16*>(o);
    p.q_row_stride = kHeadDim;
    p.q_head_stride = int64_t(seq_len) * kHeadDim;
    p.q_batch_stride = int64_t(n_q_heads) * seq_len * kHeadDim;
    p.n_q_heads = n_q_heads;
    p.n_kv_heads = n_kv_heads;
    p.group = n_q_heads / n_kv_heads;
    p.block_size = 1;
    p.seq_len = seq_len;
    p.scale_log2 = 1.4426950408889634f / sqrtf(float(kHeadDim));
    p.status = prefill_status_word();
    p.wait_limit = opt.wait_limit;
    p.stall_producer = opt.stall_producer;
    if (tc) return launch_prefill_tc(false, p, mq, mk, mv, seq_len, batch, st);
    return launch_prefill_mma(false, p, mk, mv, seq_len, batch, st);
}

}  // namespace ib

extern "C" {

int infer_prefill_status(void* stream_) {
    int* word_dev = ib::prefill_status_word();
    if (!word_dev) return INFER_ERR_CUDA;
    int word = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream_);
    IB_CUDA(cudaMemcpyAsync(&word, word_dev, sizeof(int), cudaMemcpyDeviceToHost, st));
    IB_CUDA(cudaStreamSynchronize(st));
    if ((word & 0xFFFF0000) != 0x5AFE0000) return INFER_OK;
    IB_CUDA(cudaMemsetAsync(word_dev, 0, sizeof(int), st));
    return INFER_ERR_DEVICE;
}

int infer_paged_prefill(const infer_kv_pool_t* pool, void* out, const void* q, int64_t total_q,
                        const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, const int32_t* block_tables,
                        int64_t bt_stride, int batch, int max_seqlen_q, int max_seqlen_k, int n_q_heads,
                        float softmax_scale, void* stream_) {
    return ib::paged_prefill(pool, out, q, total_q, cu_seqlens_q, cu_seqlens_k, block_tables, bt_stride, batch,
                             max_seqlen_q, max_seqlen_k, n_q_heads, softmax_scale, static_cast<cudaStream_t>(stream_),
                             ib::PrefillOptions{});
}

int infer_flash_attn_prefill(const void* q, const void* k, const void* v, void* o, int batch, int n_q_heads,
                             int n_kv_heads, int seq_len, void* stream_) {
    return ib::dense_prefill(q, k, v, o, batch, n_q_heads, n_kv_heads, seq_len, static_cast<cudaStream_t>(stream_),
                             ib::PrefillOptions{});
}

int infer_selftest_paged_prefill(const infer_kv_pool_t* pool, void* out, const void* q, int64_t total_q,
                                 const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, const int32_t* block_tables,
                                 int64_t bt_stride, int batch, int max_seqlen_q, int max_seqlen_k, int n_q_heads,
                                 float softmax_scale, void* stream_, int kernel, uint32_t wait_limit, int stall_producer) {
    ib::PrefillOptions opt;
    opt.tc = kernel != 1;
    if (wait_limit) opt.wait_limit = wait_limit;
    opt.stall_producer = opt.tc ? stall_producer : 0;
    return ib::paged_prefill(pool, out, q, total_q, cu_seqlens_q, cu_seqlens_k, block_tables, bt_stride, batch,
                             max_seqlen_q, max_seqlen_k, n_q_heads, softmax_scale, static_cast<cudaStream_t>(stream_), opt);
}

int infer_selftest_flash_attn_prefill(const void* q, const void* k, const void* v, void* o, int batch, int n_q_heads,
                                      int n_kv_heads, int seq_len, void* stream_, int kernel) {
    ib::PrefillOptions opt;
    opt.tc = kernel != 1;
    return ib::dense_prefill(q, k, v, o, batch, n_q_heads, n_kv_heads, seq_len, static_cast<cudaStream_t>(stream_), opt);
}

}  // extern "C"
