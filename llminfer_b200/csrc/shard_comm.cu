// KV-head-parallel partition and the gather of the attention output across the GPUs of a node.
// See include/gqa_b200.h.
//
// Two gathers are provided. The plain one is ncclAllGather; NCCL is bound at run time (the
// copy already loaded in the process if there is one, else libnccl.so.2 from the loader
// path), so the library has no link-time dependency on it and single-GPU users never load it.
//
// The peer gather moves the (small: tens of KiB) outputs with the GPUs' own stores over
// NVLink. Every rank owns a "window" of device memory that all other ranks map through CUDA
// IPC: two halves of nranks slots each. Data travels as 8-byte words that carry 4 bytes of
// payload and the 4-byte step number (8-byte stores are single transactions, so a word is
// seen either whole or not at all): no fences and no separate flags are needed, a word whose
// upper half shows the current step has arrived. One kernel per rank and step
//   1. stores the rank's output, word by word, into its slot of every rank's window (plain
//      stores to peer memory; no TMA, no multicast),
//   2. polls, with a time limit, the slots of all ranks in its own window until every word
//      shows the step number, and writes the payloads to the caller's buffer.
// Steps alternate between the two halves: a rank can run at most one step ahead of the
// slowest rank (it needs everybody's words to finish a step), so the half it writes for step
// e + 1 is never the one a slower rank is still reading for step e. The step number lives
// in device memory and is advanced by the kernel itself, so a captured CUDA graph can be
// replayed. If a wait runs out (a peer died or never called), the kernel sets the caller's
// status word and the window's own, and returns: nothing hangs.
#include "../../include/gqa_b200.h"

#include <cstdlib>
#include <cstring>
#include <dlfcn.h>
#include <mutex>
#include <new>

#include <cuda_runtime.h>
#include <nccl.h>

#include "decode_kernels.cuh"
#include "peer_window.cuh"
#include "ptx.cuh"

namespace {

struct NcclApi {
    ncclResult_t (*get_unique_id)(ncclUniqueId*);
    ncclResult_t (*comm_init_rank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*comm_destroy)(ncclComm_t);
    ncclResult_t (*all_gather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t,
                               cudaStream_t);
    bool ok;
};

const NcclApi& nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        std::memset(&api, 0, sizeof(api));
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
        if (h == nullptr) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (h == nullptr) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (h == nullptr) return;
        api.get_unique_id =
            reinterpret_cast<decltype(api.get_unique_id)>(dlsym(h, "ncclGetUniqueId"));
        api.comm_init_rank =
            reinterpret_cast<decltype(api.comm_init_rank)>(dlsym(h, "ncclCommInitRank"));
        api.comm_destroy = reinterpret_cast<decltype(api.comm_destroy)>(dlsym(h, "ncclCommDestroy"));
        api.all_gather = reinterpret_cast<decltype(api.all_gather)>(dlsym(h, "ncclAllGather"));
        api.ok = api.get_unique_id && api.comm_init_rank && api.comm_destroy && api.all_gather;
    });
    return api;
}

}  // namespace

namespace {

using gqa::kMaxPeers;
using gqa::PeerGatherArgs;
using gqa::WindowCtrl;
using gqa::window_ctrl;
constexpr int kGatherCtas = 16;
constexpr int kGatherThreads = 256;

__global__ void __launch_bounds__(kGatherThreads) peer_gather_kernel(const PeerGatherArgs a) {
    __shared__ uint32_t s_step;
    __shared__ int s_timed_out;
    gqa::pdl_launch_dependents();
    gqa::pdl_wait();  // the attention output and the step counter come from earlier kernels
    uint8_t* mine = a.windows[a.rank];
    WindowCtrl* ctrl = window_ctrl(mine, a.slot_bytes, a.nranks);
    if (threadIdx.x == 0) {
        s_step = *reinterpret_cast<volatile uint32_t*>(&ctrl->step) + 1;
        s_timed_out = 0;
    }
    __syncthreads();
    const uint32_t step = s_step;
    const uint64_t total = a.words * a.nranks;
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nthreads = (uint64_t)gridDim.x * blockDim.x;

    // 1. my output -> my slot in every rank's window, each word tagged with the step
    for (uint64_t i = tid; i < total; i += nthreads) {
        const int p = (int)(i / a.words);
        const uint64_t w = i - (uint64_t)p * a.words;
        gqa::push_word(gqa::window_slot(a.windows[p], step, a.nranks, a.rank, a.slot_bytes) + w,
                       step, a.send[w]);
    }

    // 2. every word of every rank's slot in my window, as soon as it shows this step
    const unsigned long long start = gqa::global_timer();
    bool timed_out = false;
    for (uint64_t i = tid; i < total && !timed_out; i += nthreads) {
        const int p = (int)(i / a.words);
        const uint64_t w = i - (uint64_t)p * a.words;
        uint32_t data;
        if (gqa::poll_word(gqa::window_slot(mine, step, a.nranks, p, a.slot_bytes) + w, step,
                           start, &data)) {
            a.recv[(uint64_t)p * a.words + w] = data;
        } else {
            timed_out = true;
        }
    }
    if (timed_out) s_timed_out = 1;
    __syncthreads();
    if (threadIdx.x == 0) {
        if (s_timed_out) {
            ctrl->status = 1;
            if (a.status != nullptr) atomicExch(a.status, gqa::kStatusPeerTimeout);
        }
        // The last CTA to finish advances the step counter for the next launch.
        __threadfence();
        const uint32_t ticket = atomicAdd(&ctrl->ticket_out, 1u);
        if (ticket == gridDim.x - 1) {
            ctrl->ticket_out = 0;
            ctrl->step = step;
        }
    }
}

}  // namespace

struct gqa_comm {
    ncclComm_t comm;
    int32_t nranks;
    int32_t rank;
    // peer gather (null / zero until gqa_comm_enable_peer_gather)
    uint8_t* window_local;
    uint8_t* windows[kMaxPeers];
    size_t slot_bytes;
};

namespace {

// GQA_FUSED_GATHER=0 keeps the gather in its own kernel (for measurements).
bool fused_gather_disabled() {
    static const bool off = [] {
        const char* v = std::getenv("GQA_FUSED_GATHER");
        return v != nullptr && v[0] == '0';
    }();
    return off;
}

PeerGatherArgs gather_args(const gqa_comm* comm, const void* send, void* recv, size_t bytes,
                           int32_t* status_dev) {
    PeerGatherArgs a;
    std::memset(&a, 0, sizeof(a));
    for (int p = 0; p < comm->nranks; ++p) a.windows[p] = comm->windows[p];
    a.send = static_cast<const uint32_t*>(send);
    a.recv = static_cast<uint32_t*>(recv);
    a.status = status_dev;
    a.slot_bytes = comm->slot_bytes;
    a.words = bytes / 4;
    a.nranks = comm->nranks;
    a.rank = comm->rank;
    return a;
}

}  // namespace

int gqa::comm_peer_args(const gqa_comm* comm, size_t bytes_per_rank, int32_t* status_dev,
                        PeerGatherArgs* out) {
    if (comm == nullptr || out == nullptr) return GQA_ERR_NULL;
    if (comm->window_local == nullptr) return GQA_ERR_COMM;
    if (bytes_per_rank == 0 || 2 * bytes_per_rank > comm->slot_bytes) return GQA_ERR_SHAPE;
    *out = gather_args(comm, nullptr, nullptr, bytes_per_rank, status_dev);
    return GQA_OK;
}

extern "C" {

int gqa_shard_plan(int32_t num_q_heads, int32_t num_kv_heads, int32_t nranks, int32_t rank,
                   int32_t* first_kv_head, int32_t* num_local_kv_heads, int32_t* first_q_head,
                   int32_t* num_local_q_heads) {
    if (!first_kv_head || !num_local_kv_heads || !first_q_head || !num_local_q_heads) {
        return GQA_ERR_NULL;
    }
    if (num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads != 0) {
        return GQA_ERR_SHAPE;
    }
    if (nranks <= 0 || rank < 0 || rank >= nranks) return GQA_ERR_RANGE;
    if (num_kv_heads % nranks != 0) return GQA_ERR_SHAPE;
    const int32_t group = num_q_heads / num_kv_heads;
    const int32_t local = num_kv_heads / nranks;
    *num_local_kv_heads = local;
    *first_kv_head = rank * local;
    *num_local_q_heads = local * group;
    *first_q_head = rank * local * group;
    return GQA_OK;
}

int gqa_comm_unique_id(void* id_out) {
    if (id_out == nullptr) return GQA_ERR_NULL;
    static_assert(sizeof(ncclUniqueId) == GQA_COMM_ID_BYTES, "id size");
    const NcclApi& api = nccl();
    if (!api.ok) return GQA_ERR_COMM;
    ncclUniqueId id;
    if (api.get_unique_id(&id) != ncclSuccess) return GQA_ERR_COMM;
    std::memcpy(id_out, &id, sizeof(id));
    return GQA_OK;
}

int gqa_comm_init(const void* id, int32_t nranks, int32_t rank, gqa_comm** out) {
    if (id == nullptr || out == nullptr) return GQA_ERR_NULL;
    *out = nullptr;
    if (nranks <= 0 || rank < 0 || rank >= nranks) return GQA_ERR_RANGE;
    const NcclApi& api = nccl();
    if (!api.ok) return GQA_ERR_COMM;
    gqa_comm* c = new (std::nothrow) gqa_comm();
    if (c == nullptr) return GQA_ERR_COMM;
    ncclUniqueId uid;
    std::memcpy(&uid, id, sizeof(uid));
    if (api.comm_init_rank(&c->comm, nranks, uid, rank) != ncclSuccess) {
        delete c;
        return GQA_ERR_COMM;
    }
    c->nranks = nranks;
    c->rank = rank;
    c->window_local = nullptr;
    c->slot_bytes = 0;
    for (int p = 0; p < kMaxPeers; ++p) c->windows[p] = nullptr;
    *out = c;
    return GQA_OK;
}

int gqa_comm_enable_peer_gather(gqa_comm* comm, size_t max_bytes_per_rank) {
    if (comm == nullptr) return GQA_ERR_NULL;
    if (comm->window_local != nullptr) return GQA_OK;
    if (comm->nranks > kMaxPeers || max_bytes_per_rank == 0) return GQA_ERR_SHAPE;
    const NcclApi& api = nccl();
    if (!api.ok) return GQA_ERR_COMM;
    // A slot holds the payload twice over: every 4 payload bytes travel with a 4-byte step tag.
    const size_t slot = (2 * max_bytes_per_rank + 255) / 256 * 256;
    const size_t window_bytes = 2 * (size_t)comm->nranks * slot + sizeof(WindowCtrl);
    uint8_t* local = nullptr;
    cudaIpcMemHandle_t* d_handles = nullptr;
    cudaIpcMemHandle_t handles[kMaxPeers];
    bool ok = cudaMalloc(&local, window_bytes) == cudaSuccess &&
              cudaMemset(local, 0, window_bytes) == cudaSuccess &&
              cudaDeviceSynchronize() == cudaSuccess &&
              cudaIpcGetMemHandle(&handles[comm->rank], local) == cudaSuccess &&
              cudaMalloc(&d_handles, sizeof(cudaIpcMemHandle_t) * kMaxPeers) == cudaSuccess &&
              cudaMemcpy(d_handles + comm->rank, &handles[comm->rank], sizeof(cudaIpcMemHandle_t),
                         cudaMemcpyHostToDevice) == cudaSuccess;
    // Every rank learns every window's handle through one small all-gather.
    ok = ok && api.all_gather(d_handles + comm->rank, d_handles, sizeof(cudaIpcMemHandle_t),
                              ncclInt8, comm->comm, nullptr) == ncclSuccess &&
         cudaDeviceSynchronize() == cudaSuccess &&
         cudaMemcpy(handles, d_handles, sizeof(cudaIpcMemHandle_t) * comm->nranks,
                    cudaMemcpyDeviceToHost) == cudaSuccess;
    if (d_handles != nullptr) cudaFree(d_handles);
    if (!ok) {
        if (local != nullptr) cudaFree(local);
        return GQA_ERR_COMM;
    }
    for (int p = 0; p < comm->nranks; ++p) {
        if (p == comm->rank) {
            comm->windows[p] = local;
            continue;
        }
        void* mapped = nullptr;
        if (cudaIpcOpenMemHandle(&mapped, handles[p], cudaIpcMemLazyEnablePeerAccess) !=
            cudaSuccess) {
            for (int q = 0; q < p; ++q) {
                if (q != comm->rank && comm->windows[q]) cudaIpcCloseMemHandle(comm->windows[q]);
                comm->windows[q] = nullptr;
            }
            cudaFree(local);
            return GQA_ERR_COMM;
        }
        comm->windows[p] = static_cast<uint8_t*>(mapped);
    }
    comm->window_local = local;
    comm->slot_bytes = slot;
    return GQA_OK;
}

int gqa_comm_peer_gather(gqa_comm* comm, const void* send, void* recv, size_t bytes,
                         int32_t* status_dev, void* stream) {
    if (comm == nullptr || send == nullptr || recv == nullptr) return GQA_ERR_NULL;
    if (comm->window_local == nullptr) return GQA_ERR_COMM;
    if (bytes == 0 || bytes % 16 != 0 || 2 * bytes > comm->slot_bytes) return GQA_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(send) | reinterpret_cast<uintptr_t>(recv)) & 15u) {
        return GQA_ERR_ALIGN;
    }
    const PeerGatherArgs a = gather_args(comm, send, recv, bytes, status_dev);
    const cudaError_t e = gqa::launch_pdl(peer_gather_kernel, dim3(kGatherCtas),
                                          dim3(kGatherThreads), 0,
                                          reinterpret_cast<cudaStream_t>(stream), a);
    return e == cudaSuccess ? GQA_OK : GQA_ERR_CUDA;
}

int gqa_comm_peer_gather_fits(const gqa_comm* comm, size_t bytes) {
    if (comm == nullptr) return 0;
    return comm->window_local != nullptr && bytes != 0 && bytes % 16 == 0 &&
                   2 * bytes <= comm->slot_bytes ? 1 : 0;
}

void gqa_comm_disable_peer_gather(gqa_comm* comm) {
    if (comm == nullptr || comm->window_local == nullptr) return;
    cudaDeviceSynchronize();
    for (int p = 0; p < comm->nranks; ++p) {
        if (p != comm->rank && comm->windows[p] != nullptr) cudaIpcCloseMemHandle(comm->windows[p]);
        comm->windows[p] = nullptr;
    }
    cudaFree(comm->window_local);
    comm->window_local = nullptr;
    comm->slot_bytes = 0;
}

void gqa_comm_destroy(gqa_comm* comm) {
    if (comm == nullptr) return;
    gqa_comm_disable_peer_gather(comm);
    const NcclApi& api = nccl();
    if (api.ok && comm->comm != nullptr) api.comm_destroy(comm->comm);
    delete comm;
}

int32_t gqa_comm_nranks(const gqa_comm* comm) { return comm == nullptr ? 0 : comm->nranks; }

int gqa_comm_all_gather(gqa_comm* comm, const void* send, void* recv, size_t bytes, void* stream) {
    if (comm == nullptr || send == nullptr || recv == nullptr) return GQA_ERR_NULL;
    const NcclApi& api = nccl();
    if (!api.ok) return GQA_ERR_COMM;
    if (api.all_gather(send, recv, bytes, ncclInt8, comm->comm,
                       reinterpret_cast<cudaStream_t>(stream)) != ncclSuccess) {
        return GQA_ERR_COMM;
    }
    return GQA_OK;
}

int gqa_decode_sharded_fused(const gqa_decode_params* p, const gqa_fused_front* front,
                             gqa_comm* comm, void* gathered) {
    if (p == nullptr || comm == nullptr || gathered == nullptr) return GQA_ERR_NULL;
    if (p->batch <= 0 || p->num_q_heads <= 0 || p->head_dim <= 0 || p->q_tokens < 0) {
        return GQA_ERR_SHAPE;
    }
    const size_t elem = p->dtype == GQA_DTYPE_F32 ? 4 : 2;
    const size_t tokens = p->q_tokens > 0 ? p->q_tokens : 1;
    const size_t bytes = (size_t)p->batch * tokens * p->num_q_heads * p->head_dim * elem;
    // Which gather runs depends on the communicator's state and the sizes only, which are the
    // same on every rank: the ranks cannot end up in different collectives.
    const bool peer = comm->window_local != nullptr && 2 * bytes <= comm->slot_bytes &&
                      bytes % 16 == 0 && p->out != nullptr &&
                      ((reinterpret_cast<uintptr_t>(p->out) |
                        reinterpret_cast<uintptr_t>(gathered)) & 15u) == 0;
    if (peer && !fused_gather_disabled()) {
        // The combine kernel pushes each row to the peers as soon as it is merged.
        const PeerGatherArgs g = gather_args(comm, p->out, gathered, bytes, p->status_dev);
        bool fused = false;
        const int rc = gqa::decode_with_gather(p, front, &g, &fused);
        if (rc != GQA_OK || fused) return rc;
        return gqa_comm_peer_gather(comm, p->out, gathered, bytes, p->status_dev, p->stream);
    }
    const int rc = front != nullptr ? gqa_decode_fused(p, front) : gqa_decode(p);
    if (rc != GQA_OK) return rc;
    if (peer) {
        return gqa_comm_peer_gather(comm, p->out, gathered, bytes, p->status_dev, p->stream);
    }
    return gqa_comm_all_gather(comm, p->out, gathered, bytes, p->stream);
}

int gqa_decode_sharded(const gqa_decode_params* p, gqa_comm* comm, void* gathered) {
    return gqa_decode_sharded_fused(p, nullptr, comm, gathered);
}

int gqa_decode_seqpar(const gqa_decode_params* p, gqa_comm* comm) {
    if (p == nullptr || comm == nullptr) return GQA_ERR_NULL;
    if (p->batch <= 0 || p->num_q_heads <= 0 || p->head_dim <= 0) return GQA_ERR_SHAPE;
    if (comm->window_local == nullptr) return GQA_ERR_COMM;
    // One record per (sequence, query head) and rank: 128 channel sums, maximum, row sum.
    const size_t bytes = (size_t)p->batch * p->num_q_heads * (p->head_dim + 2) * sizeof(float);
    if (2 * bytes > comm->slot_bytes) return GQA_ERR_SHAPE;
    const PeerGatherArgs g = gather_args(comm, nullptr, nullptr, bytes, p->status_dev);
    return gqa::decode_sequence_parallel(p, &g);
}

}  // extern "C"
