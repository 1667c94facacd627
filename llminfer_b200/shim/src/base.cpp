// Allocators, Buffer and CudaConfig of the operator shim.
#include <cstdlib>
#include <cstring>

#include <cuda_runtime.h>

#include "base/alloc.h"
#include "base/buffer.h"
#include "base/cuda_config.h"

namespace base {

void DeviceAllocator::memcpy(void* dest_ptr, const void* src_ptr, size_t byte_size,
                             MemcpyKind kind, void* stream, bool need_sync) const {
    CHECK(dest_ptr != nullptr && src_ptr != nullptr);
    if (byte_size == 0) return;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (kind == MemcpyKind::MemcpyCPU2CPU) {
        std::memcpy(dest_ptr, src_ptr, byte_size);
        return;
    }
    const cudaMemcpyKind k = kind == MemcpyKind::MemcpyCPU2CUDA   ? cudaMemcpyHostToDevice
                             : kind == MemcpyKind::MemcpyCUDA2CPU ? cudaMemcpyDeviceToHost
                                                                  : cudaMemcpyDeviceToDevice;
    const cudaError_t e = s ? cudaMemcpyAsync(dest_ptr, src_ptr, byte_size, k, s)
                            : cudaMemcpy(dest_ptr, src_ptr, byte_size, k);
    CHECK(e == cudaSuccess);
    if (need_sync) CHECK(cudaDeviceSynchronize() == cudaSuccess);
}

void DeviceAllocator::memset_zero(void* ptr, size_t byte_size, void* stream, bool need_sync) {
    CHECK(ptr != nullptr);
    if (device_type_ == DeviceType::DeviceCPU) {
        std::memset(ptr, 0, byte_size);
        return;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    CHECK((s ? cudaMemsetAsync(ptr, 0, byte_size, s) : cudaMemset(ptr, 0, byte_size)) ==
          cudaSuccess);
    if (need_sync) CHECK(cudaDeviceSynchronize() == cudaSuccess);
}

void* CPUDeviceAllocator::allocate(size_t byte_size) {
    return byte_size ? std::malloc(byte_size) : nullptr;
}

void CPUDeviceAllocator::release(void* ptr) { std::free(ptr); }

void* CUDADeviceAllocator::allocate(size_t byte_size) {
    if (byte_size == 0) return nullptr;
    void* p = nullptr;
    CHECK(cudaMalloc(&p, byte_size) == cudaSuccess);
    return p;
}

void CUDADeviceAllocator::release(void* ptr) {
    if (ptr != nullptr) CHECK(cudaFree(ptr) == cudaSuccess);
}

std::shared_ptr<CPUDeviceAllocator> CPUDeviceAllocatorFactory::get_instance() {
    static std::shared_ptr<CPUDeviceAllocator> instance = std::make_shared<CPUDeviceAllocator>();
    return instance;
}

std::shared_ptr<CUDADeviceAllocator> CUDADeviceAllocatorFactory::get_instance() {
    static std::shared_ptr<CUDADeviceAllocator> instance = std::make_shared<CUDADeviceAllocator>();
    return instance;
}

Buffer::Buffer(size_t byte_size, std::shared_ptr<DeviceAllocator> allocator, void* ptr,
               bool use_external)
    : byte_size_(byte_size), allocator_(std::move(allocator)), ptr_(ptr),
      use_external_(use_external) {
    if (ptr_ == nullptr && allocator_ != nullptr) {
        device_type_ = allocator_->device_type();
        use_external_ = false;
        ptr_ = allocator_->allocate(byte_size_);
    }
}

Buffer::~Buffer() {
    if (!use_external_ && ptr_ != nullptr && allocator_ != nullptr) {
        allocator_->release(ptr_);
    }
    ptr_ = nullptr;
}

bool Buffer::allocate() {
    if (allocator_ == nullptr || byte_size_ == 0) return false;
    use_external_ = false;
    ptr_ = allocator_->allocate(byte_size_);
    return ptr_ != nullptr;
}

void Buffer::copy_from(const Buffer& other) const {
    CHECK(allocator_ != nullptr && other.ptr_ != nullptr && ptr_ != nullptr);
    const size_t n = byte_size_ < other.byte_size_ ? byte_size_ : other.byte_size_;
    const bool src_cuda = other.device_type_ == DeviceType::DeviceCUDA;
    const bool dst_cuda = device_type_ == DeviceType::DeviceCUDA;
    const MemcpyKind kind = src_cuda ? (dst_cuda ? MemcpyKind::MemcpyCUDA2CUDA
                                                 : MemcpyKind::MemcpyCUDA2CPU)
                                     : (dst_cuda ? MemcpyKind::MemcpyCPU2CUDA
                                                 : MemcpyKind::MemcpyCPU2CPU);
    allocator_->memcpy(ptr_, other.ptr_, n, kind);
}

void Buffer::copy_from(const Buffer* other) const {
    CHECK(other != nullptr);
    copy_from(*other);
}

}  // namespace base

namespace kernel {

CudaConfig::~CudaConfig() {
    if (stream != nullptr) cudaStreamDestroy(stream);
}

void CudaConfig::create() {
    if (stream == nullptr) CHECK(cudaStreamCreate(&stream) == cudaSuccess);
}

}  // namespace kernel
