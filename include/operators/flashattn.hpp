// FlashAttnOperator<T>: dense causal attention, Q/O [B, Hq, S, 128], K/V [B, Hkv, S, 128].
// Same class name, forward() signature, type() and name() as the reference's operator
// (include/operators/flashattn.hpp:7-17); the body the reference left commented out
// (src/operators/flashattn/flashattn.cu:331-367) is the C-ABI call below.
#pragma once

#include <stdexcept>
#include <string>

#include "../infer_b200.h"
#include "../operator.hpp"
#include "../tensor.hpp"

namespace infer {

inline void check_rc(int rc, const char* what) {
    if (rc != INFER_OK) throw std::runtime_error(std::string(what) + ": " + infer_strerror(rc));
}

template <typename T>
class FlashAttnOperator : public Operator {
public:
    void forward(const Tensor<T>* Q, const Tensor<T>* K, const Tensor<T>* V, Tensor<T>* output) {
        if (sizeof(T) != 2) throw std::runtime_error("FlashAttnOperator: only bf16 (2-byte) tensors are supported");
        if (!Q || !K || !V || !output) throw std::runtime_error("FlashAttnOperator: null tensor");
        if (Q->dim() != 4 || K->dim() != 4 || K->shape() != V->shape() || output->shape() != Q->shape() ||
            Q->size(3) != 128 || K->size(2) != Q->size(2) || K->size(0) != Q->size(0))
            throw std::runtime_error("FlashAttnOperator: expected Q,O [B,Hq,S,128] and K,V [B,Hkv,S,128]");
        check_rc(infer_flash_attn_prefill(Q->data_ptr(), K->data_ptr(), V->data_ptr(), output->data_ptr(),
                                          static_cast<int>(Q->size(0)), static_cast<int>(Q->size(1)),
                                          static_cast<int>(K->size(1)), static_cast<int>(Q->size(2)), stream_),
                 "FlashAttnOperator");
    }
    OperatorType type() const override { return OperatorType::FLASHATTENTION; }
    std::string name() const override { return "FLASHATTENTION"; }
};

}  // namespace infer
