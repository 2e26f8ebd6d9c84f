// UnifiedOp<T>: one object with a method per operator, as in include/unifiedOp.hpp:6-100 of
// the reference (attention(Q, K, V, out) keeps its signature); the paged KV-cache methods
// are added next to it.  Constructing it registers the operators.
#pragma once

#include "kvcache.hpp"
#include "opfactory.hpp"

namespace infer {

template <typename T>
class UnifiedOp {
public:
    explicit UnifiedOp(void* stream = nullptr) : stream_(stream) { OperatorFactory::registerOperators<T>(); }

    void attention(const Tensor<T>* Q, const Tensor<T>* K, const Tensor<T>* V, Tensor<T>* output) {
        auto op = OperatorFactory::getFlashAttnOperator<T>();
        if (!op) throw std::runtime_error("FlashAttn operator not found");
        op->set_stream(stream_);
        op->forward(Q, K, V, output);
    }
    void kv_append(KVCachePool<T>& cache, size_t layer, const Tensor<T>* k, const Tensor<T>* v,
                   const Tensor<int32_t>* slot_mapping, Tensor<uint8_t>* workspace = nullptr) {
        auto op = OperatorFactory::getKVAppendOperator<T>();
        if (!op) throw std::runtime_error("KVAppend operator not found");
        op->set_stream(stream_);
        op->forward(cache.handle(layer), k, v, slot_mapping, workspace);
    }
    void paged_decode(KVCachePool<T>& cache, size_t layer, const Tensor<T>* q, const Tensor<int32_t>* context_lens,
                      const Tensor<int32_t>* block_tables, float softmax_scale, Tensor<uint8_t>* workspace,
                      Tensor<T>* out) {
        auto op = OperatorFactory::getPagedDecodeOperator<T>();
        if (!op) throw std::runtime_error("PagedDecode operator not found");
        op->set_stream(stream_);
        op->forward(cache.handle(layer), q, context_lens, block_tables, softmax_scale, workspace, out);
    }
    void paged_prefill(KVCachePool<T>& cache, size_t layer, const Tensor<T>* q, const Tensor<int32_t>* cu_seqlens_q,
                       const Tensor<int32_t>* cu_seqlens_k, int max_seqlen_q, int max_seqlen_k,
                       const Tensor<int32_t>* block_tables, float softmax_scale, Tensor<T>* out) {
        auto op = OperatorFactory::getPagedPrefillOperator<T>();
        if (!op) throw std::runtime_error("PagedPrefill operator not found");
        op->set_stream(stream_);
        op->forward(cache.handle(layer), q, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, block_tables,
                    softmax_scale, out);
    }

private:
    void* stream_;
};

}  // namespace infer
