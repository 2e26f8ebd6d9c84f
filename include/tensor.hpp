// Minimal tensor view used by the C++ operator surface.
//
// The reference's Tensor<T> (include/tensor.hpp:24-385) owns its storage through the
// reference's memory pool; that class is not part of the paged KV-cache path.  This one is a
// non-owning, contiguous, row-major view over memory the caller allocated (device memory for
// everything the operators read or write), with the accessors the operators need.
#pragma once

#include <cstddef>
#include <cstdint>
#include <numeric>
#include <stdexcept>
#include <vector>

namespace infer {

// 16-bit brain float storage type for hosts that do not include cuda_bf16.h; any 2-byte T
// (e.g. __nv_bfloat16) is accepted by the bf16 operators.
struct bfloat16 {
    uint16_t bits;
};

template <typename T>
class Tensor {
public:
    Tensor() = default;
    Tensor(T* data, std::vector<size_t> shape) : data_(data), shape_(std::move(shape)) {}

    T* data_ptr() const { return data_; }
    const std::vector<size_t>& shape() const { return shape_; }
    size_t dim() const { return shape_.size(); }
    size_t size(size_t i) const {
        if (i >= shape_.size()) throw std::out_of_range("Tensor::size: dimension out of range");
        return shape_[i];
    }
    size_t numel() const {
        return shape_.empty() ? 0 : std::accumulate(shape_.begin(), shape_.end(), size_t(1), std::multiplies<size_t>());
    }
    // elements between consecutive indices of dimension i (contiguous row-major)
    size_t stride(size_t i) const {
        size_t s = 1;
        for (size_t d = shape_.size(); d-- > i + 1;) s *= shape_[d];
        return s;
    }

private:
    T* data_ = nullptr;
    std::vector<size_t> shape_;
};

}  // namespace infer
