// One decode step driven from host buffers. See include/gqa_b200.h.
//
// The new token's rows are small (tens of KiB), so no copy engine is involved: the caller's
// rows are placed in a pinned, device-mapped block that the front-stage kernel reads over the
// bus directly (it writes the rotated query to device memory, where the attention kernel reads
// it many times), and the attention (or the gather) writes its output straight into a second
// pinned block. The step then waits for the stream and hands the output to the caller.
// GQA_SESSION_COPIES=1 in the environment selects explicit cudaMemcpyAsync staging instead;
// GQA_SESSION_FUSED=1 runs the front stage inside the attention kernel (gqa_decode_fused).
//
// On a KV-head-parallel node the attention's combine kernel pushes the finished rows to the
// other ranks and writes the gathered rows straight into the pinned output block, so a step
// is front stage + attention + combine there too. Which gather runs is decided from the
// communicator's state and the sizes, which are the same on every rank.
#include "../../include/gqa_b200.h"

#include <chrono>
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
    int32_t* status;   // pinned, device-mapped status word of the step's kernels
    cudaEvent_t done;  // recorded behind the step's last launch
    bool zero_copy;    // kernels read / write the pinned blocks directly
    bool fused_front;  // the attention kernel runs the front stage itself
    bool spin_wait;    // wait for a step by polling the event, not by blocking in the driver
    int64_t timing_ns[4];  // last step: staging, launches, wait, copy-out
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
    if (s->status) cudaFreeHost(s->status);
    if (s->done) cudaEventDestroy(s->done);
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
    const char* fused = std::getenv("GQA_SESSION_FUSED");
    s->fused_front = fused != nullptr && fused[0] == '1';
    const char* wait = std::getenv("GQA_SESSION_WAIT");
    s->spin_wait = !(wait != nullptr && wait[0] == 's');  // "sync": cudaStreamSynchronize
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
    ok = ok && cudaEventCreateWithFlags(&s->done, cudaEventDisableTiming) == cudaSuccess;
    ok = ok && cudaMallocHost(&s->status, sizeof(int32_t)) == cudaSuccess;
    if (ok) *s->status = 0;
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

namespace {

// Device address of a caller's host buffer when the kernels can use it where it lies (pinned,
// mapped into this device, 16-byte aligned), else null. Asked every step: a buffer may have
// been freed and its address handed out again as pageable memory since the last one.
void* mapped_address(const void* host) {
    void* device = nullptr;
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, host) == cudaSuccess && attr.type == cudaMemoryTypeHost &&
        attr.devicePointer != nullptr &&
        (reinterpret_cast<uintptr_t>(attr.devicePointer) & 15u) == 0) {
        device = attr.devicePointer;
    } else {
        cudaGetLastError();  // a pageable pointer is not an error worth keeping
    }
    return device;
}

using Clock = std::chrono::steady_clock;

int64_t ns_between(Clock::time_point a, Clock::time_point b) {
    return std::chrono::duration_cast<std::chrono::nanoseconds>(b - a).count();
}

// Waits for everything launched on the session's stream. Polling the event keeps the wake-up
// latency of a blocking wait (tens of microseconds when the host is busy) out of the step; the
// poll gives up after ten seconds and falls back to the blocking call.
int wait_for_step(gqa_session* s) {
    if (!s->spin_wait) {
        return cudaStreamSynchronize(s->stream) == cudaSuccess ? GQA_OK : GQA_ERR_CUDA;
    }
    if (cudaEventRecord(s->done, s->stream) != cudaSuccess) return GQA_ERR_CUDA;
    const Clock::time_point start = Clock::now();
    for (uint32_t spins = 1;; ++spins) {
        const cudaError_t e = cudaEventQuery(s->done);
        if (e == cudaSuccess) return GQA_OK;
        if (e != cudaErrorNotReady) return GQA_ERR_CUDA;
        if ((spins & 1023u) == 0 && ns_between(start, Clock::now()) > 10000000000ll) {
            return cudaStreamSynchronize(s->stream) == cudaSuccess ? GQA_OK : GQA_ERR_CUDA;
        }
    }
}

// What the kernels left in the status word, as a return code.
int status_code(gqa_session* s) {
    const int32_t st = *reinterpret_cast<volatile int32_t*>(s->status);
    if (st == 0) return GQA_OK;
    *s->status = 0;
    return st == GQA_STATUS_BAD_INPUT ? GQA_ERR_RANGE : GQA_ERR_TIMEOUT;
}

}  // namespace

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
    const Clock::time_point t_start = Clock::now();
    const size_t qb = q_bytes(s, batch), kb = kv_bytes(s, batch);
    // Offsets follow the max_batch layout so device pointers stay 16-byte aligned.
    const size_t off_k = q_bytes(s, s->max_batch);
    const size_t off_v = off_k + kv_bytes(s, s->max_batch);
    const size_t off_len = off_v + kv_bytes(s, s->max_batch);
    const size_t off_pos = off_len + (size_t)s->max_batch * 4;
    // Rows the caller keeps in pinned memory are read where they lie; others are staged.
    const uint8_t* q_in = nullptr;
    const uint8_t* k_in = nullptr;
    const uint8_t* v_in = nullptr;
    uint8_t* out_direct = nullptr;
    if (s->zero_copy) {
        q_in = static_cast<const uint8_t*>(mapped_address(q_host));
        k_in = static_cast<const uint8_t*>(mapped_address(k_host));
        v_in = static_cast<const uint8_t*>(mapped_address(v_host));
        out_direct = static_cast<uint8_t*>(mapped_address(out_host));
    }
    if (q_in == nullptr) std::memcpy(s->host_in, q_host, qb);
    if (k_in == nullptr) std::memcpy(s->host_in + off_k, k_host, kb);
    if (v_in == nullptr) std::memcpy(s->host_in + off_v, v_host, kb);
    int32_t* lens = reinterpret_cast<int32_t*>(s->host_in + off_len);
    int32_t* poss = reinterpret_cast<int32_t*>(s->host_in + off_pos);
    for (int32_t b = 0; b < batch; ++b) {
        if (positions_host[b] < 0 || positions_host[b] >= s->max_seq_len) return GQA_ERR_RANGE;
        poss[b] = positions_host[b];
        lens[b] = positions_host[b] + 1;
    }
    const size_t used = off_pos + (size_t)batch * 4;
    // Pinned memory is mapped into the device's address space at the same address.
    const uint8_t* in = s->zero_copy ? s->host_in : s->dev_in;
    if (q_in == nullptr) q_in = in;
    if (k_in == nullptr) k_in = in + off_k;
    if (v_in == nullptr) v_in = in + off_v;
    if (!s->zero_copy &&
        cudaMemcpyAsync(s->dev_in, s->host_in, used, cudaMemcpyHostToDevice, s->stream) !=
            cudaSuccess) {
        return GQA_ERR_CUDA;
    }
    bool uniform = true;
    for (int32_t b = 1; b < batch; ++b) uniform = uniform && positions_host[b] == positions_host[0];
    const Clock::time_point t_staged = Clock::now();

    int rc = GQA_OK;
    gqa_fused_front ff;
    std::memset(&ff, 0, sizeof(ff));
    if (s->fused_front) {
        ff.k_new = k_in;
        ff.v_new = v_in;
        ff.qk_weight = qk_weight_dev;
        ff.sin_cache = s->sin_table;
        ff.cos_cache = s->cos_table;
        ff.table_len = s->max_seq_len;
        ff.eps = 1e-6f;
    } else {
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
        f.q = q_in;
        f.q_out = s->dev_in;
        f.k_new = k_in;
        f.v_new = v_in;
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
        f.status_dev = s->status;
        f.stream = s->stream;
        rc = gqa_qk_norm_rope_append(&f);
        if (rc != GQA_OK) return rc;
    }

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
    p.q = s->fused_front ? static_cast<const void*>(q_in) : s->dev_in;
    p.k_cache = k_cache;
    p.v_cache = v_cache;
    const bool out_to_host = s->zero_copy && comm == nullptr;
    p.out = out_to_host ? (out_direct != nullptr ? out_direct : s->host_out) : s->dev_out;
    p.workspace = s->workspace;
    p.workspace_bytes = s->workspace_bytes;
    p.seq_lens_host = lens;
    p.seq_lens_dev = uniform ? nullptr : reinterpret_cast<const int32_t*>(in + off_len);
    p.block_table_dev = block_table_dev;
    p.status_dev = s->status;
    p.stream = s->stream;
    // Ahead of the attention in this stream is the front stage, which writes the cache rows
    // of the new positions only (fused: nothing that writes the caches at all).
    p.early_prefetch = 1;
    const gqa_fused_front* front = s->fused_front ? &ff : nullptr;

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
        // The peer-store gather (inside the combine kernel when units are split) can deliver
        // into the pinned block itself; NCCL gathers on the device and a copy follows. The
        // choice depends on the communicator and the size only, so every rank makes the same.
        const bool to_host = s->zero_copy && gqa_comm_peer_gather_fits(comm, qb) == 1;
        uint8_t* gather_to = to_host ? (out_direct != nullptr ? out_direct : s->host_gather)
                                     : s->dev_gather;
        rc = gqa_decode_sharded_fused(&p, front, comm, gather_to);
        if (rc != GQA_OK) return rc;
        if (!to_host && cudaMemcpyAsync(s->host_gather, s->dev_gather, total,
                                        cudaMemcpyDeviceToHost, s->stream) != cudaSuccess) {
            return GQA_ERR_CUDA;
        }
        const Clock::time_point t_launched = Clock::now();
        rc = wait_for_step(s);
        if (rc != GQA_OK) return rc;
        const Clock::time_point t_done = Clock::now();
        rc = status_code(s);
        if (rc != GQA_OK) return rc;
        if (!(to_host && out_direct != nullptr)) std::memcpy(out_host, s->host_gather, total);
        const Clock::time_point t_end = Clock::now();
        s->timing_ns[0] = ns_between(t_start, t_staged);
        s->timing_ns[1] = ns_between(t_staged, t_launched);
        s->timing_ns[2] = ns_between(t_launched, t_done);
        s->timing_ns[3] = ns_between(t_done, t_end);
        return GQA_OK;
    }
    rc = front != nullptr ? gqa_decode_fused(&p, front) : gqa_decode(&p);
    if (rc != GQA_OK) return rc;
    if (!out_to_host && cudaMemcpyAsync(s->host_out, s->dev_out, qb, cudaMemcpyDeviceToHost,
                                        s->stream) != cudaSuccess) {
        return GQA_ERR_CUDA;
    }
    const Clock::time_point t_launched = Clock::now();
    rc = wait_for_step(s);
    if (rc != GQA_OK) return rc;
    const Clock::time_point t_done = Clock::now();
    rc = status_code(s);
    if (rc != GQA_OK) return rc;
    if (!(out_to_host && out_direct != nullptr)) std::memcpy(out_host, s->host_out, qb);
    const Clock::time_point t_end = Clock::now();
    s->timing_ns[0] = ns_between(t_start, t_staged);
    s->timing_ns[1] = ns_between(t_staged, t_launched);
    s->timing_ns[2] = ns_between(t_launched, t_done);
    s->timing_ns[3] = ns_between(t_done, t_end);
    return GQA_OK;
}

int gqa_session_last_timing(const gqa_session* s, int64_t* ns_out) {
    if (s == nullptr || ns_out == nullptr) return GQA_ERR_NULL;
    for (int i = 0; i < 4; ++i) ns_out[i] = s->timing_ns[i];
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
