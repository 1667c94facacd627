// tensor::Tensor of the operator shim.
#include "tensor/tensor.h"

#include <numeric>

namespace tensor {

namespace {
size_t element_count(const std::vector<int32_t>& dims) {
    if (dims.empty()) return 0;
    size_t n = 1;
    for (int32_t d : dims) n *= static_cast<size_t>(d);
    return n;
}
}  // namespace

Tensor::Tensor(base::DataType data_type, std::vector<int32_t> dims, bool need_alloc,
               std::shared_ptr<base::DeviceAllocator> allocator, void* ptr)
    : size_(element_count(dims)), dims_(std::move(dims)), data_type_(data_type) {
    if (need_alloc && allocator) {
        allocate(allocator);
    } else if (ptr != nullptr) {
        init_buffer(allocator, need_alloc, ptr);
    }
}

Tensor::Tensor(base::DataType data_type, int32_t dim0, bool need_alloc,
               std::shared_ptr<base::DeviceAllocator> allocator, void* ptr)
    : Tensor(data_type, std::vector<int32_t>{dim0}, need_alloc, std::move(allocator), ptr) {}

Tensor::Tensor(base::DataType data_type, int32_t dim0, int32_t dim1, bool need_alloc,
               std::shared_ptr<base::DeviceAllocator> allocator, void* ptr)
    : Tensor(data_type, std::vector<int32_t>{dim0, dim1}, need_alloc, std::move(allocator), ptr) {}

Tensor::Tensor(base::DataType data_type, int32_t dim0, int32_t dim1, int32_t dim2, bool need_alloc,
               std::shared_ptr<base::DeviceAllocator> allocator, void* ptr)
    : Tensor(data_type, std::vector<int32_t>{dim0, dim1, dim2}, need_alloc, std::move(allocator),
             ptr) {}

Tensor::Tensor(base::DataType data_type, int32_t dim0, int32_t dim1, int32_t dim2, int32_t dim3,
               bool need_alloc, std::shared_ptr<base::DeviceAllocator> allocator, void* ptr)
    : Tensor(data_type, std::vector<int32_t>{dim0, dim1, dim2, dim3}, need_alloc,
             std::move(allocator), ptr) {}

void Tensor::init_buffer(std::shared_ptr<base::DeviceAllocator> allocator, bool need_alloc,
                         void* ptr) {
    if (!allocator && !need_alloc) {
        // A view: the memory belongs to somebody else.
        buffer_ = std::make_shared<base::Buffer>(byte_size(), nullptr, ptr, true);
    } else {
        allocate(allocator, true);
    }
}

bool Tensor::allocate(std::shared_ptr<base::DeviceAllocator> allocator, bool need_realloc) {
    if (!allocator || byte_size() == 0) return false;
    if (buffer_ && buffer_->byte_size() >= byte_size() && !need_realloc) return true;
    buffer_ = std::make_shared<base::Buffer>(byte_size(), allocator, nullptr, false);
    return buffer_->ptr() != nullptr;
}

bool Tensor::assgin(std::shared_ptr<base::Buffer> buffer) {
    if (!buffer || buffer->byte_size() < byte_size()) return false;
    buffer_ = std::move(buffer);
    return true;
}

void Tensor::to_cuda(cudaStream_t stream) {
    CHECK(buffer_ != nullptr);
    if (buffer_->device_type() == base::DeviceType::DeviceCUDA) return;
    auto alloc = base::CUDADeviceAllocatorFactory::get_instance();
    auto moved = std::make_shared<base::Buffer>(byte_size(), alloc, nullptr, false);
    alloc->memcpy(moved->ptr(), buffer_->ptr(), byte_size(), base::MemcpyKind::MemcpyCPU2CUDA,
                  stream, false);
    buffer_ = std::move(moved);
}

void Tensor::to_cpu() {
    CHECK(buffer_ != nullptr);
    if (buffer_->device_type() == base::DeviceType::DeviceCPU) return;
    auto alloc = base::CPUDeviceAllocatorFactory::get_instance();
    auto moved = std::make_shared<base::Buffer>(byte_size(), alloc, nullptr, false);
    alloc->memcpy(moved->ptr(), buffer_->ptr(), byte_size(), base::MemcpyKind::MemcpyCUDA2CPU,
                  nullptr, true);
    buffer_ = std::move(moved);
}

void Tensor::reshape(const std::vector<int32_t>& dims) {
    const size_t n = element_count(dims);
    if (buffer_ && n > size_) {
        auto grown = std::make_shared<base::Buffer>(n * base::data_type_size(data_type_),
                                                    buffer_->allocator(), nullptr, false);
        CHECK(grown->ptr() != nullptr);
        grown->copy_from(buffer_.get());
        buffer_ = std::move(grown);
    }
    dims_ = dims;
    size_ = n;
}

int32_t Tensor::get_dim(int32_t index) const {
    CHECK(index >= 0 && index < dims_size());
    return dims_[index];
}

std::vector<size_t> Tensor::strides() const {
    std::vector<size_t> out(dims_.size(), 1);
    for (int i = static_cast<int>(dims_.size()) - 2; i >= 0; --i) {
        out[i] = out[i + 1] * static_cast<size_t>(dims_[i + 1]);
    }
    return out;
}

Tensor Tensor::clone() const {
    Tensor copy = *this;
    CHECK(buffer_ != nullptr);
    std::shared_ptr<base::DeviceAllocator> alloc = buffer_->allocator();
    if (!alloc) {
        if (buffer_->device_type() == base::DeviceType::DeviceCUDA) {
            alloc = base::CUDADeviceAllocatorFactory::get_instance();
        } else {
            alloc = base::CPUDeviceAllocatorFactory::get_instance();
        }
    }
    copy.buffer_ = std::make_shared<base::Buffer>(byte_size(), alloc, nullptr, false);
    copy.buffer_->copy_from(buffer_.get());
    return copy;
}

void Tensor::reset(base::DataType data_type, const std::vector<int32_t>& dims) {
    data_type_ = data_type;
    dims_ = dims;
    size_ = element_count(dims);
    buffer_ = nullptr;
}

bool Tensor::is_empty() const { return size_ == 0 || !buffer_ || buffer_->ptr() == nullptr; }

base::DeviceType Tensor::device_type() const {
    return buffer_ ? buffer_->device_type() : base::DeviceType::DeviceUnknown;
}

void Tensor::set_device_type(base::DeviceType device_type) const {
    if (buffer_) buffer_->set_device_type(device_type);
}

}  // namespace tensor
