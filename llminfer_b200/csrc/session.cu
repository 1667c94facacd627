// One decode step driven from host buffers. See include/gqa_b200.h.
//
// The new token's rows are small (tens of KiB), so no copy engine is involved: the caller's
// rows are placed in a pinned, device-mapped block that the front-stage kernel reads over the
// bus directly (it writes the rotated query to device memory, where the attention kernel reads
// it many times), and the attention (or the gather) writes its output straight into a second
// pinned block. The step then waits for the stream and hands the output to the caller.
// GQA_SESSION_COPIES=1 in the environment selects explicit cudaMemcpyAsync staging instead.
#include "../../include/gqa_b200.h"

#include <cstdlib>
#include <cstring>
#include <new>

#include <cuda_runtime.h>

struct gqa_session {
    int32_t max_batch;
    int32_t num_q_heads;
    int32_t num_kv_heads;
    int32_t head_dim;
    int32_t max_seq_len;
    cudaStream_t stream;
    // One pinned block and one device block with the same layout:
    //   [q rows | k rows | v rows | seq_lens int32 | positions int32]
    uint8_t* host_in;
    uint8_t* dev_in;
    size_t in_bytes;
    uint8_t* host_out;  // pinned
    uint8_t* dev_out;
    uint8_t* host_gather;  // pinned, grown on first sharded step
    uint8_t* dev_gather;
    size_t gather_bytes;
    void* workspace;
    size_t workspace_bytes;
    float* sin_table;  // [max_seq_len, head_dim / 2], built once at creation
    float* cos_table;
    bool zero_copy;    // kernels read / write the pinned blocks directly
};

namespace {

size_t q_bytes(const gqa_session* s, int32_t batch) {
    return (size_t)batch * s->num_q_heads * s->head_dim * 2;
}

size_t kv_bytes(const gqa_session* s, int32_t batch) {
    return (size_t)batch * s->num_kv_heads * s->head_dim * 2;
}

void release(gqa_session* s) {
    if (s == nullptr) return;
    if (s->host_in) cudaFreeHost(s->host_in);
    if (s->host_out) cudaFreeHost(s->host_out);
    if (s->host_gather) cudaFreeHost(s->host_gather);
    if (s->dev_gather) cudaFree(s->dev_gather);
    if (s->dev_in) cudaFree(s->dev_in);
    if (s->dev_out) cudaFree(s->dev_out);
    if (s->workspace) cudaFree(s->workspace);
    if (s->sin_table) cudaFree(s->sin_table);
    if (s->cos_table) cudaFree(s->cos_table);
    if (s->stream) cudaStreamDestroy(s->stream);
    delete s;
}

}  // namespace

extern "C" {

int gqa_session_create(int32_t dtype, int32_t max_batch, int32_t num_q_heads,
                       int32_t num_kv_heads, int32_t head_dim, int32_t max_seq_len,
                       gqa_session** out) {
    if (out == nullptr) return GQA_ERR_NULL;
    *out = nullptr;
    if (dtype != GQA_DTYPE_BF16) return GQA_ERR_DTYPE;  // the front stage is BF16 only
    if (max_batch <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim != 128 ||
        max_seq_len <= 0 || num_q_heads % num_kv_heads != 0) {
        return GQA_ERR_SHAPE;
    }
    gqa_session* s = new (std::nothrow) gqa_session();
    if (s == nullptr) return GQA_ERR_CUDA;
    std::memset(s, 0, sizeof(*s));
    s->max_batch = max_batch;
    s->num_q_heads = num_q_heads;
    s->num_kv_heads = num_kv_heads;
    s->head_dim = head_dim;
    s->max_seq_len = max_seq_len;
    const char* copies = std::getenv("GQA_SESSION_COPIES");
    s->zero_copy = !(copies != nullptr && copies[0] == '1');
    s->in_bytes = q_bytes(s, max_batch) + 2 * kv_bytes(s, max_batch) + 2 * (size_t)max_batch * 4;
    int sms = 0, dev = 0;
    bool ok = cudaGetDevice(&dev) == cudaSuccess &&
              cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess;
    // Room for every split plan the planner may choose (it stops refining once the grid is
    // oversubscribed eight times) plus one record per unit.
    const size_t rec = (size_t)(num_q_heads / num_kv_heads) * (head_dim + 2) * sizeof(float);
    s->workspace_bytes = ((size_t)16 * (sms > 0 ? sms : 1) +
                          (size_t)2 * max_batch * num_kv_heads) * rec;
    ok = ok && cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaMallocHost(&s->host_in, s->in_bytes) == cudaSuccess;
    ok = ok && cudaMallocHost(&s->host_out, q_bytes(s, max_batch)) == cudaSuccess;
    ok = ok && cudaMalloc(&s->dev_in, s->in_bytes) == cudaSuccess;
    ok = ok && cudaMalloc(&s->dev_out, q_bytes(s, max_batch)) == cudaSuccess;
    ok = ok && cudaMalloc(&s->workspace, s->workspace_bytes) == cudaSuccess;
    const size_t table_bytes = (size_t)max_seq_len * (head_dim / 2) * sizeof(float);
    ok = ok && cudaMalloc(&s->sin_table, table_bytes) == cudaSuccess;
    ok = ok && cudaMalloc(&s->cos_table, table_bytes) == cudaSuccess;
    ok = ok && gqa_sin_cos_cache(s->sin_table, s->cos_table, head_dim, max_seq_len, s->stream) ==
                   GQA_OK;
    ok = ok && cudaStreamSynchronize(s->stream) == cudaSuccess;
    if (!ok) {
        release(s);
        return GQA_ERR_CUDA;
    }
    *out = s;
    return GQA_OK;
}

void gqa_session_destroy(gqa_session* s) { release(s); }

static int step_impl(gqa_session* s, gqa_comm* comm, int32_t batch, const void* q_host,
                     const void* k_host, const void* v_host, const void* qk_weight_dev,
                     void* k_cache, void* v_cache, const gqa_kv_layout* layout,
                     const int32_t* positions_host, const int32_t* block_table_dev,
                     int32_t blocks_per_seq, int32_t fixed_block, void* out_host) {
    if (s == nullptr || q_host == nullptr || k_host == nullptr || v_host == nullptr ||
        qk_weight_dev == nullptr || k_cache == nullptr || v_cache == nullptr ||
        layout == nullptr || positions_host == nullptr || out_host == nullptr) {
        return GQA_ERR_NULL;
    }
    if (batch <= 0 || batch > s->max_batch) return GQA_ERR_SHAPE;
    const size_t qb = q_bytes(s, batch), kb = kv_bytes(s, batch);
    // Offsets follow the max_batch layout so device pointers stay 16-byte aligned.
    const size_t off_k = q_bytes(s, s->max_batch);
    const size_t off_v = off_k + kv_bytes(s, s->max_batch);
    const size_t off_len = off_v + kv_bytes(s, s->max_batch);
    const size_t off_pos = off_len + (size_t)s->max_batch * 4;
    std::memcpy(s->host_in, q_host, qb);
    std::memcpy(s->host_in + off_k, k_host, kb);
    std::memcpy(s->host_in + off_v, v_host, kb);
    int32_t* lens = reinterpret_cast<int32_t*>(s->host_in + off_len);
    int32_t* poss = reinterpret_cast<int32_t*>(s->host_in + off_pos);
    for (int32_t b = 0; b < batch; ++b) {
        if (positions_host[b] < 0) return GQA_ERR_RANGE;
        poss[b] = positions_host[b];
        lens[b] = positions_host[b] + 1;
    }
    const size_t used = off_pos + (size_t)batch * 4;
    // Pinned memory is mapped into the device's address space at the same address.
    const uint8_t* in = s->zero_copy ? s->host_in : s->dev_in;
    if (!s->zero_copy &&
        cudaMemcpyAsync(s->dev_in, s->host_in, used, cudaMemcpyHostToDevice, s->stream) !=
            cudaSuccess) {
        return GQA_ERR_CUDA;
    }
    bool uniform = true;
    for (int32_t b = 1; b < batch; ++b) uniform = uniform && positions_host[b] == positions_host[0];

    gqa_front_params f;
    std::memset(&f, 0, sizeof(f));
    f.batch = batch;
    f.num_q_heads = s->num_q_heads;
    f.num_kv_heads = s->num_kv_heads;
    f.head_dim = s->head_dim;
    f.blocks_per_seq = blocks_per_seq;
    f.fixed_block = fixed_block;
    f.eps = 1e-6f;
    f.layout = *layout;
    f.q = in;
    f.q_out = s->dev_in;
    f.k_new = in + off_k;
    f.v_new = in + off_v;
    f.qk_weight = qk_weight_dev;
    f.sin_cache = s->sin_table;
    f.cos_cache = s->cos_table;
    f.table_len = s->max_seq_len;
    f.k_cache = k_cache;
    f.v_cache = v_cache;
    f.positions_host = poss;
    // Equal positions travel by value; otherwise the kernels read them from the staged block.
    f.positions_dev = uniform ? nullptr : reinterpret_cast<const int32_t*>(in + off_pos);
    f.block_table_dev = block_table_dev;
    f.stream = s->stream;
    int rc = gqa_qk_norm_rope_append(&f);
    if (rc != GQA_OK) return rc;

    gqa_decode_params p;
    std::memset(&p, 0, sizeof(p));
    p.dtype = GQA_DTYPE_BF16;
    p.batch = batch;
    p.num_q_heads = s->num_q_heads;
    p.num_kv_heads = s->num_kv_heads;
    p.head_dim = s->head_dim;
    p.blocks_per_seq = blocks_per_seq;
    p.fixed_block = fixed_block;
    p.layout = *layout;
    p.q = s->dev_in;
    p.k_cache = k_cache;
    p.v_cache = v_cache;
    const bool out_to_host = s->zero_copy && comm == nullptr;
    p.out = out_to_host ? s->host_out : s->dev_out;
    p.workspace = s->workspace;
    p.workspace_bytes = s->workspace_bytes;
    p.seq_lens_host = lens;
    p.seq_lens_dev = uniform ? nullptr : reinterpret_cast<const int32_t*>(in + off_len);
    p.block_table_dev = block_table_dev;
    p.stream = s->stream;
    // Ahead of the attention in this stream is the front stage, which writes the cache rows
    // of the new positions only.
    p.early_prefetch = 1;
    rc = gqa_decode(&p);
    if (rc != GQA_OK) return rc;

    if (comm != nullptr) {
        const int32_t nranks = gqa_comm_nranks(comm);
        const size_t total = qb * (size_t)nranks;
        if (s->gather_bytes < total) {
            if (s->host_gather) cudaFreeHost(s->host_gather);
            if (s->dev_gather) cudaFree(s->dev_gather);
            s->host_gather = nullptr;
            s->dev_gather = nullptr;
            s->gather_bytes = 0;
            const size_t cap = q_bytes(s, s->max_batch) * (size_t)nranks;
            if (cudaMallocHost(&s->host_gather, cap) != cudaSuccess ||
                cudaMalloc(&s->dev_gather, cap) != cudaSuccess) {
                return GQA_ERR_CUDA;
            }
            s->gather_bytes = cap;
        }
        // The peer-store gather can deliver into the pinned block itself; NCCL gathers on the
        // device and a copy follows.
        bool on_host = false;
        if (s->zero_copy) {
            rc = gqa_comm_peer_gather(comm, s->dev_out, s->host_gather, qb, nullptr, s->stream);
            on_host = rc == GQA_OK;
        }
        if (!on_host) {
            rc = gqa_comm_all_gather(comm, s->dev_out, s->dev_gather, qb, s->stream);
            if (rc != GQA_OK) return rc;
            if (cudaMemcpyAsync(s->host_gather, s->dev_gather, total, cudaMemcpyDeviceToHost,
                                s->stream) != cudaSuccess) {
                return GQA_ERR_CUDA;
            }
        }
        if (cudaStreamSynchronize(s->stream) != cudaSuccess) return GQA_ERR_CUDA;
        std::memcpy(out_host, s->host_gather, total);
        return GQA_OK;
    }
    if (!out_to_host && cudaMemcpyAsync(s->host_out, s->dev_out, qb, cudaMemcpyDeviceToHost,
                                        s->stream) != cudaSuccess) {
        return GQA_ERR_CUDA;
    }
    if (cudaStreamSynchronize(s->stream) != cudaSuccess) return GQA_ERR_CUDA;
    std::memcpy(out_host, s->host_out, qb);
    return GQA_OK;
}

int gqa_session_step(gqa_session* s, int32_t batch, const void* q_host, const void* k_host,
                     const void* v_host, const void* qk_weight_dev, void* k_cache, void* v_cache,
                     const gqa_kv_layout* layout, const int32_t* positions_host,
                     const int32_t* block_table_dev, int32_t blocks_per_seq,
                     int32_t fixed_block, void* out_host) {
    return step_impl(s, nullptr, batch, q_host, k_host, v_host, qk_weight_dev, k_cache, v_cache,
                     layout, positions_host, block_table_dev, blocks_per_seq, fixed_block,
                     out_host);
}

int gqa_session_step_sharded(gqa_session* s, gqa_comm* comm, int32_t batch, const void* q_host,
                             const void* k_host, const void* v_host, const void* qk_weight_dev,
                             void* k_cache, void* v_cache, const gqa_kv_layout* layout,
                             const int32_t* positions_host, const int32_t* block_table_dev,
                             int32_t blocks_per_seq, int32_t fixed_block, void* gathered_host) {
    if (comm == nullptr) return GQA_ERR_NULL;
    return step_impl(s, comm, batch, q_host, k_host, v_host, qk_weight_dev, k_cache, v_cache,
                     layout, positions_host, block_table_dev, blocks_per_seq, fixed_block,
                     gathered_host);
}

}  // extern "C"
