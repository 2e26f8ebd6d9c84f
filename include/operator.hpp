// Operator base class and operator ids of the C++ surface.
//
// Follows include/operator.hpp:14-46 of the reference: an enum of operator kinds and an
// abstract base with type() and name().  The reference's torch-typed
// `forward(const std::vector<torch::Tensor>&)` is not kept: this surface has no torch types,
// every operator exposes a typed forward() of its own (as the reference's concrete operators
// do).  The three paged-KV entries are new; the others keep their reference values so that
// ids stay stable for code that stores them.
#pragma once

#include <memory>
#include <string>

namespace infer {

enum class OperatorType {
    MATMUL,
    RELU,
    SOFTMAX,
    SILU,
    FLASHATTENTION,
    ADD_RMS_NORM,
    MUL,
    ADD,
    ROPE,
    EMBEDDING,
    KV_APPEND,       // store_kvcache (infer/ops/attention.py:38-45)
    PAGED_DECODE,    // decode branch of Attention.forward (infer/ops/attention.py:117-121)
    PAGED_PREFILL    // prefill branch (infer/ops/attention.py:110-116)
};

enum class DataType { FLOAT32, FLOAT16, BFLOAT16 };

class Operator {
public:
    virtual ~Operator() = default;
    virtual OperatorType type() const = 0;
    virtual std::string name() const = 0;
    // CUDA stream (cudaStream_t) the operator launches on; nullptr = default stream.
    void set_stream(void* stream) { stream_ = stream; }
    void* stream() const { return stream_; }

protected:
    void* stream_ = nullptr;
};

using OperatorPtr = std::shared_ptr<Operator>;

}  // namespace infer
