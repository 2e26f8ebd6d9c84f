// Pool handle: geometry checks and TMA descriptors of the K/V page pools.
#include <atomic>
#include <new>

#include "common.cuh"

namespace ib {

static std::atomic<int> g_last_cuda_error{0};

void set_cuda_error(cudaError_t e) { g_last_cuda_error.store(static_cast<int>(e)); }

int check_launch() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_cuda_error(e);
        return INFER_ERR_CUDA;
    }
    return INFER_OK;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

// The driver entry point is looked up at run time so the library links against the CUDA
// runtime only and still loads on a machine without a driver.
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess) {
            set_cuda_error(e != cudaSuccess ? e : cudaErrorSymbolNotFound);
            p = nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

int encode_map_3d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t d0, uint64_t d1, uint64_t d2,
                  uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return INFER_ERR_CUDA;
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
    cuuint32_t box[3] = {b0, b1, b2};
    cuuint32_t estr[3] = {1, 1, 1};
    CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
    // One head's row is 256 contiguous bytes in a bf16 pool but only 128 in an e4m3 pool, where a
    // 256-byte L2 promotion would drag in the neighbouring head's bytes and double the DRAM traffic.
    const CUtensorMapL2promotion promo = elem_bytes == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B;
    CUresult r = fn(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_cuda_error(cudaErrorInvalidValue);
        return INFER_ERR_CUDA;
    }
    return INFER_OK;
}

}  // namespace ib

extern "C" {

int infer_kv_pool_create(infer_kv_pool_t** out, void* k_cache, void* v_cache, float* k_scale, float* v_scale,
                         int64_t num_blocks, int block_size, int n_kv_heads, int head_dim, int dtype) {
    if (!out || !k_cache || !v_cache) return INFER_ERR_NULL;
    *out = nullptr;
    if (dtype != INFER_KV_BF16 && dtype != INFER_KV_E4M3) return INFER_ERR_DTYPE;
    if (dtype == INFER_KV_E4M3 && (!k_scale || !v_scale)) return INFER_ERR_NULL;
    if (head_dim != ib::kHeadDim || block_size <= 0 || block_size % 256 != 0 || n_kv_heads <= 0 ||
        num_blocks <= 0 || num_blocks * block_size >= (int64_t(1) << 31))
        return INFER_ERR_GEOMETRY;
    if (!ib::aligned16(k_cache) || !ib::aligned16(v_cache)) return INFER_ERR_ALIGN;

    infer_kv_pool* p = new (std::nothrow) infer_kv_pool();
    if (!p) return INFER_ERR_CUDA;
    p->k_cache = k_cache;
    p->v_cache = v_cache;
    p->k_scale = k_scale;
    p->v_scale = v_scale;
    p->num_blocks = num_blocks;
    p->block_size = block_size;
    p->num_slots = num_blocks * block_size;
    p->n_kv_heads = n_kv_heads;
    p->head_dim = head_dim;
    p->dtype = dtype;
    p->elem_bytes = dtype == INFER_KV_BF16 ? 2 : 1;

    cudaError_t e = cudaGetDevice(&p->device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&p->sm_count, cudaDevAttrMultiProcessorCount, p->device);
    if (e != cudaSuccess) {
        ib::set_cuda_error(e);
        delete p;
        return INFER_ERR_CUDA;
    }
    if (ib::decode_prepare_device() != INFER_OK) {
        delete p;
        return INFER_ERR_CUDA;
    }
    // Rows of one head are 128 elements; a swizzled box is 128 bytes wide.
    const uint32_t inner = 128 / p->elem_bytes;
    const uint64_t head_pitch = uint64_t(ib::kHeadDim) * p->elem_bytes;
    const uint64_t slot_pitch = head_pitch * n_kv_heads;
    for (int i = 0; i < 5; ++i) {
        const uint32_t rows = 16u << i;
        int rc = ib::encode_map_3d(&p->maps[i].k, k_cache, p->elem_bytes, ib::kHeadDim, n_kv_heads, p->num_slots,
                                   head_pitch, slot_pitch, inner, 1, rows);
        if (rc == INFER_OK)
            rc = ib::encode_map_3d(&p->maps[i].v, v_cache, p->elem_bytes, ib::kHeadDim, n_kv_heads, p->num_slots,
                                   head_pitch, slot_pitch, inner, 1, rows);
        if (rc != INFER_OK) {
            delete p;
            return rc;
        }
    }
    *out = p;
    return INFER_OK;
}

int infer_kv_pool_destroy(infer_kv_pool_t* pool) {
    delete pool;
    return INFER_OK;
}

const char* infer_strerror(int code) {
    switch (code) {
        case INFER_OK: return "ok";
        case INFER_ERR_NULL: return "a required pointer is NULL";
        case INFER_ERR_ALIGN: return "pointer or stride is not 16-byte aligned";
        case INFER_ERR_STRIDE: return "row stride is smaller than the row";
        case INFER_ERR_GEOMETRY: return "unsupported geometry (head_dim 128, block_size % 256 == 0, "
                                        "n_q_heads % n_kv_heads == 0, group <= 8, batch <= 2048)";
        case INFER_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
        case INFER_ERR_CUDA: return "CUDA error (see infer_last_cuda_error)";
        case INFER_ERR_DTYPE: return "pool dtype not supported by this entry point";
        case INFER_ERR_DEVICE: return "a bounded device-side wait ran out";
        case INFER_ERR_TOO_LARGE: return "problem exceeds the 2 MiB built-in scratch of infer_paged_decode_noalloc "
                                         "(batch <= 2048); use infer_paged_decode with a workspace";
        case INFER_ERR_STATE: return "page allocator: out of pages, unknown or duplicate sequence, or a call out of order";
        default: return "unknown error code";
    }
}

int infer_last_cuda_error(void) { return ib::g_last_cuda_error.load(); }

int infer_abi_version(void) { return 1; }

}  // extern "C"
