// Allocator interface of the reference (code/include/base/alloc.h:17-85), kept as the
// ownership contract of Buffer / Tensor. The CUDA allocator here is a plain cudaMalloc /
// cudaFree pair: the reference's size-class pool (code/source/base/alloc_cu.cpp:7-79) is
// outside the attention path; KV memory is managed by gqa_kv_pool instead.
#ifndef LLMINFER_SHIM_BASE_ALLOC_H
#define LLMINFER_SHIM_BASE_ALLOC_H

#include <memory>

#include "base/base.h"

namespace base {

enum class MemcpyKind : uint8_t {
    MemcpyCPU2CPU = 0,
    MemcpyCPU2CUDA = 1,
    MemcpyCUDA2CPU = 2,
    MemcpyCUDA2CUDA = 3,
};

class DeviceAllocator {
public:
    explicit DeviceAllocator(DeviceType device_type) : device_type_(device_type) {}
    virtual ~DeviceAllocator() = default;
    virtual DeviceType device_type() const { return device_type_; }
    virtual void* allocate(size_t byte_size) = 0;
    virtual void release(void* ptr) = 0;
    virtual void memcpy(void* dest_ptr, const void* src_ptr, size_t byte_size,
                        MemcpyKind memcpy_kind = MemcpyKind::MemcpyCPU2CPU, void* stream = nullptr,
                        bool need_sync = false) const;
    virtual void memset_zero(void* ptr, size_t byte_size, void* stream, bool need_sync = false);

private:
    DeviceType device_type_;
};

class CPUDeviceAllocator : public DeviceAllocator {
public:
    CPUDeviceAllocator() : DeviceAllocator(DeviceType::DeviceCPU) {}
    void* allocate(size_t byte_size) override;
    void release(void* ptr) override;
};

class CUDADeviceAllocator : public DeviceAllocator {
public:
    CUDADeviceAllocator() : DeviceAllocator(DeviceType::DeviceCUDA) {}
    void* allocate(size_t byte_size) override;
    void release(void* ptr) override;
};

class CPUDeviceAllocatorFactory {
public:
    static std::shared_ptr<CPUDeviceAllocator> get_instance();
};

class CUDADeviceAllocatorFactory {
public:
    static std::shared_ptr<CUDADeviceAllocator> get_instance();
};

}  // namespace base

#endif  // LLMINFER_SHIM_BASE_ALLOC_H
