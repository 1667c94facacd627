// One CUDA stream per model, as in the reference (code/include/base/cuda_config.h:18-22).
#ifndef LLMINFER_SHIM_BASE_CUDA_CONFIG_H
#define LLMINFER_SHIM_BASE_CUDA_CONFIG_H

#include <cuda_runtime.h>

namespace kernel {

struct CudaConfig {
    ~CudaConfig();
    void create();
    cudaStream_t stream = nullptr;
};

}  // namespace kernel

#endif  // LLMINFER_SHIM_BASE_CUDA_CONFIG_H
