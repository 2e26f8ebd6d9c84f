// Operators of the paged KV-cache path over the C ABI: append, paged decode, paged prefill.
// They have no class in the reference (its Python layer calls Triton and flash_attn
// directly, infer/ops/attention.py:96-122); they follow the shape of its operator classes
// (include/operators/*.hpp): typed forward(), type(), name().
#pragma once

#include "../kvcache.hpp"
#include "flashattn.hpp"

namespace infer {

// store_kvcache (infer/ops/attention.py:38-45): k, v [N, Hkv, 128] -> slots of the layer's pools.
template <typename T>
class KVAppendOperator : public Operator {
public:
    void forward(infer_kv_pool_t* pool, const Tensor<T>* k, const Tensor<T>* v, const Tensor<int32_t>* slot_mapping,
                 Tensor<uint8_t>* workspace = nullptr) {
        if (!pool || !k || !v || !slot_mapping) throw std::runtime_error("KVAppendOperator: null argument");
        if (k->dim() != 3 || k->shape() != v->shape() || slot_mapping->numel() != k->size(0))
            throw std::runtime_error("KVAppendOperator: expected k,v [N,Hkv,128] and slot_mapping [N]");
        check_rc(infer_kv_append(pool, k->data_ptr(), v->data_ptr(), static_cast<int64_t>(k->stride(0)),
                                 static_cast<int64_t>(v->stride(0)), slot_mapping->data_ptr(),
                                 static_cast<int64_t>(k->size(0)), workspace ? workspace->data_ptr() : nullptr,
                                 workspace ? workspace->numel() : 0, stream_),
                 "KVAppendOperator");
    }
    OperatorType type() const override { return OperatorType::KV_APPEND; }
    std::string name() const override { return "KV_APPEND"; }
};

// decode branch (infer/ops/attention.py:117-121): q, out [B, Hq, 128].
template <typename T>
class PagedDecodeOperator : public Operator {
public:
    static size_t workspace_bytes(infer_kv_pool_t* pool, int batch, int n_q_heads) {
        return infer_paged_decode_workspace_bytes(pool, batch, n_q_heads);
    }
    void forward(infer_kv_pool_t* pool, const Tensor<T>* q, const Tensor<int32_t>* context_lens,
                 const Tensor<int32_t>* block_tables, float softmax_scale, Tensor<uint8_t>* workspace, Tensor<T>* out) {
        if (!pool || !q || !context_lens || !block_tables || !workspace || !out)
            throw std::runtime_error("PagedDecodeOperator: null argument");
        if (q->dim() != 3 || out->shape() != q->shape() || block_tables->dim() != 2 ||
            block_tables->size(0) != q->size(0) || context_lens->numel() != q->size(0))
            throw std::runtime_error("PagedDecodeOperator: expected q,out [B,Hq,128], context_lens [B], block_tables [B,W]");
        check_rc(infer_paged_decode(pool, out->data_ptr(), q->data_ptr(), context_lens->data_ptr(),
                                    block_tables->data_ptr(), static_cast<int64_t>(block_tables->size(1)),
                                    static_cast<int>(q->size(0)), static_cast<int>(q->size(1)), softmax_scale,
                                    workspace->data_ptr(), workspace->numel(), stream_),
                 "PagedDecodeOperator");
    }
    OperatorType type() const override { return OperatorType::PAGED_DECODE; }
    std::string name() const override { return "PAGED_DECODE"; }
};

// prefill branch (infer/ops/attention.py:110-116): q, out [total_q, Hq, 128].
template <typename T>
class PagedPrefillOperator : public Operator {
public:
    void forward(infer_kv_pool_t* pool, const Tensor<T>* q, const Tensor<int32_t>* cu_seqlens_q,
                 const Tensor<int32_t>* cu_seqlens_k, int max_seqlen_q, int max_seqlen_k,
                 const Tensor<int32_t>* block_tables, float softmax_scale, Tensor<T>* out) {
        if (!pool || !q || !cu_seqlens_q || !cu_seqlens_k || !block_tables || !out)
            throw std::runtime_error("PagedPrefillOperator: null argument");
        if (q->dim() != 3 || out->shape() != q->shape() || block_tables->dim() != 2 ||
            cu_seqlens_q->numel() != cu_seqlens_k->numel() || cu_seqlens_q->numel() != block_tables->size(0) + 1)
            throw std::runtime_error("PagedPrefillOperator: expected q,out [T,Hq,128], cu_seqlens [B+1], block_tables [B,W]");
        check_rc(infer_paged_prefill(pool, out->data_ptr(), q->data_ptr(), static_cast<int64_t>(q->size(0)),
                                     cu_seqlens_q->data_ptr(), cu_seqlens_k->data_ptr(), block_tables->data_ptr(),
                                     static_cast<int64_t>(block_tables->size(1)), static_cast<int>(block_tables->size(0)),
                                     max_seqlen_q, max_seqlen_k, static_cast<int>(q->size(1)), softmax_scale, stream_),
                 "PagedPrefillOperator");
    }
    OperatorType type() const override { return OperatorType::PAGED_PREFILL; }
    std::string name() const override { return "PAGED_PREFILL"; }
};

}  // namespace infer
