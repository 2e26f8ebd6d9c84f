// OperatorFactory: registers the operators of the paged KV-cache path and hands out the
// shared instances.  Same shape as include/opfactory.hpp:15-76 of the reference
// (registerOperators<T>() + one typed getter per operator); the reference's other nine
// entries belong to operators outside this path and are not provided.
#pragma once

#include "operators/flashattn.hpp"
#include "operators/paged_attention.hpp"
#include "opregistry.hpp"

namespace infer {

class OperatorFactory {
public:
    template <typename T>
    static void registerOperators() {
        REGISTER_OPERATOR(OperatorType::FLASHATTENTION, FLASHATTENTION, FlashAttnOperator, T);
        REGISTER_OPERATOR(OperatorType::KV_APPEND, KV_APPEND, KVAppendOperator, T);
        REGISTER_OPERATOR(OperatorType::PAGED_DECODE, PAGED_DECODE, PagedDecodeOperator, T);
        REGISTER_OPERATOR(OperatorType::PAGED_PREFILL, PAGED_PREFILL, PagedPrefillOperator, T);
    }
    template <typename T>
    static std::shared_ptr<FlashAttnOperator<T>> getFlashAttnOperator() {
        return OperatorRegistry::getInstance().getOperator<T, FlashAttnOperator>(OperatorType::FLASHATTENTION, "FLASHATTENTION");
    }
    template <typename T>
    static std::shared_ptr<KVAppendOperator<T>> getKVAppendOperator() {
        return OperatorRegistry::getInstance().getOperator<T, KVAppendOperator>(OperatorType::KV_APPEND, "KV_APPEND");
    }
    template <typename T>
    static std::shared_ptr<PagedDecodeOperator<T>> getPagedDecodeOperator() {
        return OperatorRegistry::getInstance().getOperator<T, PagedDecodeOperator>(OperatorType::PAGED_DECODE, "PAGED_DECODE");
    }
    template <typename T>
    static std::shared_ptr<PagedPrefillOperator<T>> getPagedPrefillOperator() {
        return OperatorRegistry::getInstance().getOperator<T, PagedPrefillOperator>(OperatorType::PAGED_PREFILL, "PAGED_PREFILL");
    }
};

}  // namespace infer
