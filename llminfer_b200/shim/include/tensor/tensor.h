// tensor::Tensor of the reference (code/include/tensor/tensor.h:8-86): dims, dtype and a
// shared Buffer. The members the attention operators use are provided with the reference's
// signatures, including the (dtype, dims..., need_alloc, allocator, ptr) constructors.
#ifndef LLMINFER_SHIM_TENSOR_TENSOR_H
#define LLMINFER_SHIM_TENSOR_TENSOR_H

#include <cuda_runtime_api.h>
#include <memory>
#include <vector>

#include "base/buffer.h"

namespace tensor {

class Tensor {
public:
    Tensor() = default;
    explicit Tensor(base::DataType data_type, int32_t dim0, bool need_alloc = false,
                    std::shared_ptr<base::DeviceAllocator> allocator = nullptr,
                    void* ptr = nullptr);
    explicit Tensor(base::DataType data_type, int32_t dim0, int32_t dim1, bool need_alloc = false,
                    std::shared_ptr<base::DeviceAllocator> allocator = nullptr,
                    void* ptr = nullptr);
    explicit Tensor(base::DataType data_type, int32_t dim0, int32_t dim1, int32_t dim2,
                    bool need_alloc = false,
                    std::shared_ptr<base::DeviceAllocator> allocator = nullptr,
                    void* ptr = nullptr);
    explicit Tensor(base::DataType data_type, int32_t dim0, int32_t dim1, int32_t dim2,
                    int32_t dim3, bool need_alloc = false,
                    std::shared_ptr<base::DeviceAllocator> allocator = nullptr,
                    void* ptr = nullptr);
    explicit Tensor(base::DataType data_type, std::vector<int32_t> dims, bool need_alloc = false,
                    std::shared_ptr<base::DeviceAllocator> allocator = nullptr,
                    void* ptr = nullptr);

    void init_buffer(std::shared_ptr<base::DeviceAllocator> allocator, bool need_alloc, void* ptr);
    bool allocate(std::shared_ptr<base::DeviceAllocator> allocator, bool need_realloc = false);
    bool assgin(std::shared_ptr<base::Buffer> buffer);

    void to_cpu();
    void to_cuda(cudaStream_t stream = nullptr);

    void reshape(const std::vector<int32_t>& dims);
    int32_t dims_size() const { return static_cast<int32_t>(dims_.size()); }
    int32_t get_dim(int32_t index) const;
    const std::vector<int32_t>& dims() const { return dims_; }
    std::vector<size_t> strides() const;

    Tensor clone() const;
    void reset(base::DataType data_type, const std::vector<int32_t>& dims);

    bool is_empty() const;
    size_t size() const { return size_; }
    size_t byte_size() const { return size_ * base::data_type_size(data_type_); }
    base::DataType data_type() const { return data_type_; }
    base::DeviceType device_type() const;
    void set_device_type(base::DeviceType device_type) const;
    std::shared_ptr<base::Buffer> get_buffer() const { return buffer_; }

    template <typename T> T* ptr() {
        return buffer_ ? reinterpret_cast<T*>(buffer_->ptr()) : nullptr;
    }
    template <typename T> const T* ptr() const {
        return buffer_ ? reinterpret_cast<const T*>(buffer_->ptr()) : nullptr;
    }
    template <typename T> T* ptr(int64_t index) {
        CHECK(buffer_ && buffer_->ptr());
        return reinterpret_cast<T*>(buffer_->ptr()) + index;
    }
    template <typename T> const T* ptr(int64_t index) const {
        CHECK(buffer_ && buffer_->ptr());
        return reinterpret_cast<const T*>(buffer_->ptr()) + index;
    }
    template <typename T> T& index(int64_t offset) {
        CHECK(offset >= 0 && static_cast<size_t>(offset) < size_);
        return *(reinterpret_cast<T*>(buffer_->ptr()) + offset);
    }
    template <typename T> const T& index(int64_t offset) const {
        CHECK(offset >= 0 && static_cast<size_t>(offset) < size_);
        return *(reinterpret_cast<const T*>(buffer_->ptr()) + offset);
    }

private:
    size_t size_ = 0;
    std::vector<int32_t> dims_;
    std::shared_ptr<base::Buffer> buffer_;
    base::DataType data_type_ = base::DataType::DataTypeUnknown;
};

}  // namespace tensor

#endif  // LLMINFER_SHIM_TENSOR_TENSOR_H
