// KV-head-parallel partition and the NCCL all-gather of the attention output.
// See include/gqa_b200.h. NCCL is bound at run time (the copy already loaded in the process
// if there is one, else libnccl.so.2 from the loader path), so the library itself has no
// link-time dependency on it and single-GPU users never load it.
#include "../../include/gqa_b200.h"

#include <cstring>
#include <dlfcn.h>
#include <mutex>
#include <new>

#include <cuda_runtime.h>
#include <nccl.h>

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

struct gqa_comm {
    ncclComm_t comm;
    int32_t nranks;
    int32_t rank;
};

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
    *out = c;
    return GQA_OK;
}

void gqa_comm_destroy(gqa_comm* comm) {
    if (comm == nullptr) return;
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

int gqa_decode_sharded(const gqa_decode_params* p, gqa_comm* comm, void* gathered) {
    if (p == nullptr || comm == nullptr || gathered == nullptr) return GQA_ERR_NULL;
    const int rc = gqa_decode(p);
    if (rc != GQA_OK) return rc;
    const size_t elem = p->dtype == GQA_DTYPE_F32 ? 4 : 2;
    const size_t bytes = (size_t)p->batch * p->num_q_heads * p->head_dim * elem;
    return gqa_comm_all_gather(comm, p->out, gathered, bytes, p->stream);
}

}  // extern "C"
