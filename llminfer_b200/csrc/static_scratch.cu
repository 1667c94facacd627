// gqa_decode_static_scratch: decode attention whose split scratch lives inside the library.
//
// Who needs it. Some callers may not allocate device memory around the attention call: code
// running while a CUDA stream is being captured (cudaMalloc is not a capturable operation and
// may be refused there), real-time serving loops that are forbidden to touch the allocator
// after start-up, and hosts that hand this library a fixed memory budget and no allocator
// callback. gqa_decode() asks such callers for a workspace they would have to size and
// allocate in advance; this entry point asks for nothing but inputs and outputs.
//
// How. The partial records of split units (the scratch that gqa_decode_stream_* writes and
// gqa_decode_combine reads) go to a file-scope __device__ array of GQA_STATIC_SCRATCH_BYTES.
// Every GPU that loads the library reserves that much memory until the process exits. In host
// code the array's name is only a handle: its device address is looked up with
// cudaGetSymbolAddress, once per device, with that device current, and that address is what
// the kernels receive.
//
// Limits. The planner keeps its split inside GQA_STATIC_SCRATCH_BYTES (with lengths known on
// the device only it sizes the records for full sequences and coarsens the split until they
// fit); an explicit split_keys whose records cannot fit is refused with GQA_ERR_WORKSPACE and
// nothing is launched. If device-side lengths outgrow what the plan provided for, the kernels
// skip the records that would fall outside the array and set the caller's status word to
// GQA_STATUS_BAD_INPUT: they never write past it. All calls on a device share the one array: calls that may run
// concurrently on the GPU (different streams, or graphs launched side by side) race on it and
// must be serialised by the caller or use gqa_decode() with separate workspaces. The array keeps
// the previous call's records; nothing in it has to start at zero, because every record that is
// read in a call was written earlier in that same call.
#include "../../include/gqa_b200.h"

#include <mutex>

#include <cuda_runtime.h>

namespace {

static __device__ __align__(256) float g_static_scratch[GQA_STATIC_SCRATCH_BYTES / sizeof(float)];

// Device address of the array on the current device; looked up on the first call per device.
int static_scratch_address(void** out) {
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static void* cached[kMaxDevices] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return GQA_ERR_CUDA;
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < kMaxDevices && cached[dev] != nullptr) {
        *out = cached[dev];
        return GQA_OK;
    }
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) return GQA_ERR_CUDA;
    if (dev >= 0 && dev < kMaxDevices) cached[dev] = ptr;
    *out = ptr;
    return GQA_OK;
}

}  // namespace

extern "C" int gqa_decode_static_scratch(const gqa_decode_params* p) {
    if (p == nullptr) return GQA_ERR_NULL;
    void* scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if (rc != GQA_OK) return rc;
    gqa_decode_params local = *p;
    local.workspace = scratch;
    local.workspace_bytes = GQA_STATIC_SCRATCH_BYTES;
    // An explicit split that cannot fit the array is refused here, before anything is launched.
    gqa_decode_plan_info plan;
    rc = gqa_decode_plan(&local, 0, &plan);
    if (rc != GQA_OK) return rc;
    if (plan.workspace_bytes > GQA_STATIC_SCRATCH_BYTES) return GQA_ERR_WORKSPACE;
    return gqa_decode(&local);
}
