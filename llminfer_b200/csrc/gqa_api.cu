// C ABI of the decode-attention library: validation, split planning, tensor-map set-up and
// kernel launches. See include/gqa_b200.h for the contract of every entry point.
#include "../../include/gqa_b200.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include "decode_kernels.cuh"
#include "peer_window.cuh"
#include "work_map.cuh"

namespace {

using gqa::ceil_div;
using gqa::kChunkKeys;
using gqa::kHeadDim;

constexpr int kMaxGroup = 8;
constexpr int kMaxColumns = 16;  // (query token, query head) columns per unit and launch
constexpr int kPlanWarps = 4;  // warps sharing an item in both streaming kernels

size_t dtype_bytes(int32_t dtype) { return dtype == GQA_DTYPE_F32 ? 4 : 2; }

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int validate_layout(const gqa_kv_layout& l, int32_t dtype, int32_t num_kv_heads) {
    if (l.block_tokens <= 0 || l.num_blocks <= 0) return GQA_ERR_SHAPE;
    if (l.stride_block <= 0 || l.stride_token <= 0 || l.stride_head <= 0) return GQA_ERR_SHAPE;
    const int64_t eb = (int64_t)dtype_bytes(dtype);
    if ((l.stride_block * eb) % 16 || (l.stride_token * eb) % 16 || (l.stride_head * eb) % 16) {
        return GQA_ERR_ALIGN;
    }
    if (l.stride_head < kHeadDim && num_kv_heads > 1) return GQA_ERR_SHAPE;
    return GQA_OK;
}

int32_t tokens_of(const gqa_decode_params* p) { return p->q_tokens > 0 ? p->q_tokens : 1; }

int64_t capacity_of(const gqa_decode_params* p) {
    return p->block_table_dev != nullptr ? (int64_t)p->blocks_per_seq * p->layout.block_tokens
                                         : p->layout.block_tokens;
}

// Everything that can be checked without touching device memory. allow_empty: a sequence may
// have no key at all (an empty slice of a sequence-parallel rank).
int validate_decode(const gqa_decode_params* p, bool allow_empty = false, bool in_passes = false) {
    if (p == nullptr) return GQA_ERR_NULL;
    if (p->dtype != GQA_DTYPE_F32 && p->dtype != GQA_DTYPE_BF16) return GQA_ERR_DTYPE;
    if (p->batch <= 0 || p->num_q_heads <= 0 || p->num_kv_heads <= 0) return GQA_ERR_SHAPE;
    if (p->head_dim != kHeadDim) return GQA_ERR_SHAPE;
    if (p->num_q_heads % p->num_kv_heads != 0) return GQA_ERR_SHAPE;
    if (p->num_q_heads / p->num_kv_heads > kMaxGroup) return GQA_ERR_UNSUPPORTED;
    if (p->q_tokens < 0) return GQA_ERR_SHAPE;
    const int32_t tokens = tokens_of(p);
    if (tokens > 1) {
        if (p->dtype != GQA_DTYPE_BF16) return GQA_ERR_UNSUPPORTED;
        if (!in_passes && tokens * (p->num_q_heads / p->num_kv_heads) > kMaxColumns) {
            return GQA_ERR_UNSUPPORTED;
        }
    }
    int rc = validate_layout(p->layout, p->dtype, p->num_kv_heads);
    if (rc != GQA_OK) return rc;
    if (p->q == nullptr || p->k_cache == nullptr || p->v_cache == nullptr || p->out == nullptr) {
        return GQA_ERR_NULL;
    }
    if (!aligned16(p->q) || !aligned16(p->k_cache) || !aligned16(p->v_cache) ||
        !aligned16(p->out)) {
        return GQA_ERR_ALIGN;
    }
    if (p->seq_lens_host == nullptr && p->seq_lens_dev == nullptr) return GQA_ERR_NULL;
    if (p->split_keys < GQA_SPLIT_EVEN || p->max_ctas < 0 || p->plan_len_hint < 0) return GQA_ERR_RANGE;
    int64_t capacity;  // tokens one sequence can hold
    if (p->block_table_dev != nullptr) {
        if (p->blocks_per_seq <= 0) return GQA_ERR_SHAPE;
        if (p->blocks_per_seq > 1 && p->layout.block_tokens % kChunkKeys != 0) return GQA_ERR_SHAPE;
        capacity = (int64_t)p->blocks_per_seq * p->layout.block_tokens;
    } else {
        if (p->batch != 1) return GQA_ERR_SHAPE;
        if (p->fixed_block < 0 || p->fixed_block >= p->layout.num_blocks) return GQA_ERR_RANGE;
        capacity = p->layout.block_tokens;
    }
    if (p->seq_lens_host != nullptr) {
        for (int32_t b = 0; b < p->batch; ++b) {
            const int32_t len = p->seq_lens_host[b];
            if (len == 0 && allow_empty && p->seq_lens_dev != nullptr) continue;
            if (len < tokens || len > capacity) return GQA_ERR_RANGE;
            if (p->seq_lens_dev == nullptr && len != p->seq_lens_host[0]) return GQA_ERR_UNSUPPORTED;
        }
    } else if (p->batch > gqa::kMaxRaggedBatch) {
        return GQA_ERR_UNSUPPORTED;
    }
    if (p->seq_lens_dev != nullptr && p->batch > gqa::kMaxRaggedBatch) return GQA_ERR_UNSUPPORTED;
    if (p->plan_len_hint > capacity) return GQA_ERR_RANGE;
    return GQA_OK;
}

int device_sm_count(int32_t* out) {
    static std::mutex mu;
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return GQA_ERR_CUDA;
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && cached[dev] > 0) {
        *out = cached[dev];
        return GQA_OK;
    }
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        sms <= 0) {
        return GQA_ERR_CUDA;
    }
    if (dev >= 0 && dev < 64) cached[dev] = sms;
    *out = sms;
    return GQA_OK;
}

gqa::StreamShape stream_shape() { return gqa::kDefaultStreamShape; }

// ---- split planning ------------------------------------------------------------------------
// Cost of a candidate, in "steps": one step is every warp of a CTA consuming one chunk.
// A CTA runs its items back to back (its copies run ahead across items), each item ends with
// a merge of the warps; a split unit additionally pays the combine launch.
constexpr double kItemOverhead = 1.0;
constexpr double kCombineBase = 3.0;
constexpr double kCombinePerSplit = 0.05;
constexpr double kClusterMerge = 1.0;  // cluster barrier + merge through distributed shared memory
constexpr double kEvenMargin = 0.5;    // the even cut has to beat the best split by this much

// Stages that starting on a unit costs a CTA in the even cut (merge of the previous piece's
// warps, the new unit's query rows): every unit counts for that many stages more than it has.
int32_t even_pad_cells() {
    static const int32_t pad = [] {
        const char* v = std::getenv("GQA_EVEN_PAD");
        const int n = v != nullptr ? std::atoi(v) : 8;
        return n < 0 ? 0 : (n > 64 ? 64 : n);
    }();
    return pad;
}

struct PlanInput {
    int32_t batch;
    int32_t num_kv_heads;
    int32_t group;
    const int32_t* lens;  // host lengths or null
    int32_t uniform_len;  // used when lens is null
    int32_t sm_count;
    int32_t max_ctas;
    int32_t split_keys;
    size_t workspace_bytes;  // 0 = unconstrained
    int32_t chunk_align;     // splits start on multiples of this many chunks
    double overhead_scale;   // fixed costs relative to one step (a CUDA-core FP32 step is long)
    // Splits merged inside thread-block clusters (one cluster per unit, one CTA per split):
    const int32_t* cluster_fit;  // [17] clusters of each size the GPU holds at once; null = never
    int32_t cluster_chunks;      // chunks of the longest sequence the kernels may ever see
    // Even cut of all units' stages over the CTAs (BF16 streaming kernel, planner's choice only):
    bool allow_even;
    bool force_even;             // the caller asked for it: no cost comparison
    int32_t capacity_chunks;     // chunks a sequence can hold
};

constexpr int kMaxClusterSize = 16;  // 8 is the portable limit; up to 16 where the GPU takes it

int64_t items_for(const PlanInput& in, int32_t q, int32_t* max_splits) {
    int64_t items = 0;
    int32_t ms = 0;
    for (int32_t b = 0; b < in.batch; ++b) {
        const int32_t len = in.lens ? in.lens[b] : in.uniform_len;
        const int32_t s = ceil_div(ceil_div(len, kChunkKeys), q);
        items += (int64_t)s * in.num_kv_heads;
        ms = s > ms ? s : ms;
        if (!in.lens) {
            items *= in.batch;
            break;
        }
    }
    *max_splits = ms;
    return items;
}

size_t record_bytes(int32_t group) { return (size_t)group * (kHeadDim + 2) * sizeof(float); }

int make_plan(const PlanInput& in, gqa_decode_plan_info* out) {
    int32_t max_chunks = 0;
    for (int32_t b = 0; b < in.batch; ++b) {
        const int32_t len = in.lens ? in.lens[b] : in.uniform_len;
        const int32_t c = ceil_div(len, kChunkKeys);
        max_chunks = c > max_chunks ? c : max_chunks;
        if (!in.lens) break;
    }
    const int32_t g_max = in.max_ctas > 0 && in.max_ctas < in.sm_count ? in.max_ctas : in.sm_count;
    const size_t rec = record_bytes(in.group);
    const int64_t units = (int64_t)in.batch * in.num_kv_heads;

    // CTAs per cluster if splits of q chunks can be merged inside clusters: 2 to 16 splits per
    // unit even at the largest length the kernels may see, the whole grid one wave, and every
    // cluster resident at once. 0 if not.
    auto cluster_for = [&](int32_t q) -> int32_t {
        if (in.cluster_fit == nullptr) return 0;
        const int32_t c = ceil_div(in.cluster_chunks > max_chunks ? in.cluster_chunks : max_chunks, q);
        if (c < 2 || c > kMaxClusterSize) return 0;
        if (units * c > g_max || units > in.cluster_fit[c]) return 0;
        return c;
    };

    auto finish = [&](int32_t q) -> int {
        q = ceil_div(q < 1 ? 1 : q, in.chunk_align) * in.chunk_align;
        int32_t ms = 0;
        const int64_t items = items_for(in, q, &ms);
        if (items > INT32_MAX) return GQA_ERR_SHAPE;
        out->split_chunks = q;
        out->max_splits = ms;
        out->num_items = (int32_t)items;
        out->num_ctas = (int32_t)(items < g_max ? (items > 0 ? items : 1) : g_max);
        out->needs_combine = ms > 1 ? 1 : 0;
        out->cluster_size = ms > 1 ? cluster_for(q) : 0;
        out->even_cut = 0;
        out->workspace_bytes = ms > 1 ? (size_t)items * rec : 0;
        if (in.workspace_bytes != 0 && out->workspace_bytes > in.workspace_bytes) {
            return GQA_ERR_WORKSPACE;
        }
        return GQA_OK;
    };

    if (in.split_keys > 0) return finish(ceil_div(in.split_keys, kChunkKeys));
    if (max_chunks == 0) return finish(1);  // nothing but empty slices

    // Candidates: q = ceil(max_chunks / s) for s = 1, 2, ... while the grid is not yet
    // oversubscribed eight times; evaluated with the uniform upper bound on item size.
    double best_cost = 0.0;
    int32_t best_q = max_chunks;
    bool have = false;
    int32_t last_q = -1;
    for (int32_t s = 1; s <= max_chunks; ++s) {
        const int32_t q = ceil_div(ceil_div(max_chunks, s), in.chunk_align) * in.chunk_align;
        if (q == last_q) continue;
        last_q = q;
        int32_t ms = 0;
        const int64_t items = items_for(in, q, &ms);
        if (in.workspace_bytes != 0 && ms > 1 && (size_t)items * rec > in.workspace_bytes) break;
        const int64_t rounds = (items + g_max - 1) / g_max;
        double cost = (double)rounds *
                      ((double)ceil_div(q, kPlanWarps) + in.overhead_scale * kItemOverhead);
        if (ms > 1) {
            cost += in.overhead_scale *
                    (cluster_for(q) > 0 ? kClusterMerge : kCombineBase + kCombinePerSplit * ms);
        }
        if (!have || cost < best_cost - 1e-9) {
            best_cost = cost;
            best_q = q;
            have = true;
        }
        if (items > (int64_t)8 * g_max) break;
    }
    // The even cut: every CTA streams the same number of stages (cells of chunk_align chunks),
    // pieces of cut units are merged by the combine launch, G + U records. Only for lengths
    // that differ by more than a quarter: with equal lengths uniform splits already fill the
    // GPU evenly and measure a little faster (fewer CTAs change units at the same moment).
    bool ragged = false;
    if (in.lens != nullptr) {
        int32_t lo = INT32_MAX, hi = 0;
        for (int32_t b = 0; b < in.batch; ++b) {
            if (in.lens[b] <= 0) continue;
            lo = in.lens[b] < lo ? in.lens[b] : lo;
            hi = in.lens[b] > hi ? in.lens[b] : hi;
        }
        ragged = hi > 0 && (int64_t)4 * hi > (int64_t)5 * lo;
    }
    if (in.allow_even && (ragged || in.force_even)) {
        const int32_t pad = even_pad_cells();
        int64_t total = 0;
        for (int32_t b = 0; b < in.batch; ++b) {
            const int32_t len = in.lens ? in.lens[b] : in.uniform_len;
            const int32_t cells = ceil_div(ceil_div(len, kChunkKeys), in.chunk_align);
            total += (int64_t)(cells > 0 ? cells + pad : 0) * in.num_kv_heads;
            if (!in.lens) {
                total *= in.batch;
                break;
            }
        }
        const int64_t cap_total = units * (ceil_div(in.capacity_chunks, in.chunk_align) + pad);
        int64_t ctas = (total + kPlanWarps - 1) / kPlanWarps;  // at least one stage per warp
        ctas = ctas < 1 ? 1 : (ctas > g_max ? g_max : ctas);
        const int64_t per_cta = (total + ctas - 1) / ctas;
        // A unit's start is paid for by its padding; a range that starts inside a unit is not.
        const double cost =
            (double)((per_cta + kPlanWarps - 1) / kPlanWarps) * in.chunk_align +
            in.overhead_scale * (kItemOverhead + kCombineBase +
                                 kCombinePerSplit * ((double)ctas / (double)units + 1.0));
        const size_t ws = (size_t)(ctas + units) * rec;
        const bool fits = in.workspace_bytes == 0 || ws <= in.workspace_bytes;
        if (in.force_even && !fits) return GQA_ERR_WORKSPACE;
        if (cap_total < (1 << 30) && ctas + units < INT32_MAX && fits &&
            (in.force_even || !have || cost < best_cost - kEvenMargin)) {
            out->split_chunks = in.chunk_align;
            const int64_t widest = ((int64_t)ceil_div(max_chunks, in.chunk_align) + per_cta - 1) / per_cta + 1;
            out->max_splits = (int32_t)(widest < ctas ? widest : ctas);
            out->num_items = (int32_t)(ctas + units);
            out->num_ctas = (int32_t)ctas;
            out->needs_combine = 1;
            out->cluster_size = 0;
            out->even_cut = 1;
            out->workspace_bytes = ws;
            return GQA_OK;
        }
    }
    if (in.force_even) return GQA_ERR_UNSUPPORTED;  // more cells than the cut can index
    if (!have) return GQA_ERR_WORKSPACE;
    return finish(best_q);
}

// GQA_EVEN_CUT=0 keeps the planner to uniform splits (for measurements).
bool even_cut_disabled() {
    static const bool off = [] {
        const char* v = std::getenv("GQA_EVEN_CUT");
        return v != nullptr && v[0] == '0';
    }();
    return off;
}

// GQA_CLUSTER_MERGE=0 keeps the combine launch for every split plan (for measurements).
bool cluster_merge_disabled() {
    static const bool off = [] {
        const char* v = std::getenv("GQA_CLUSTER_MERGE");
        return v != nullptr && v[0] == '0';
    }();
    return off;
}

// How many clusters of each size (2 .. 16 CTAs of the BF16 streaming kernel) the GPU holds at
// once. Asked from the current device when it is the one being planned for (clusters are placed
// inside GPCs, so fewer may fit than SMs / size); otherwise SMs / size for the portable sizes.
const int32_t* cluster_fit_table(int32_t sm_count) {
    static std::mutex mu;
    static int32_t device_tables[64][kMaxClusterSize + 1];
    static bool ready[64] = {};
    thread_local int32_t guess[kMaxClusterSize + 1];
    int dev = -1, dev_sms = 0;
    const bool on_device = cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 &&
                           cudaDeviceGetAttribute(&dev_sms, cudaDevAttrMultiProcessorCount, dev) ==
                               cudaSuccess && dev_sms == sm_count;
    if (!on_device) {
        cudaGetLastError();
        for (int c = 0; c <= kMaxClusterSize; ++c) guess[c] = c >= 2 && c <= 8 ? sm_count / c : 0;
        return guess;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!ready[dev]) {
        static CUtensorMap dummy;
        for (int c = 0; c <= kMaxClusterSize; ++c) {
            device_tables[dev][c] = 0;
            if (c < 2) continue;
            gqa::DecodeArgs probe;
            std::memset(&probe, 0, sizeof(probe));
            probe.cluster_size = c;
            probe.group = 8;  // the variant with the largest shared-memory footprint
            probe.q_tokens = 2;
            gqa::FusedFrontArgs ff = {};
            device_tables[dev][c] = gqa::stream_bf16_max_clusters(dummy, dummy, probe, &ff, c);
        }
        ready[dev] = true;
    }
    return device_tables[dev];
}

int plan_from_params(const gqa_decode_params* p, int32_t sm_count, gqa_decode_plan_info* out,
                     bool allow_cluster = true, bool allow_even = true);

int plan_from_params(const gqa_decode_params* p, int32_t sm_count, gqa_decode_plan_info* out,
                     bool allow_cluster, bool allow_even) {
    std::memset(out, 0, sizeof(*out));
    PlanInput in;
    in.batch = p->batch;
    in.num_kv_heads = p->num_kv_heads;
    in.group = (p->num_q_heads / p->num_kv_heads) * tokens_of(p);  // columns of a record
    in.lens = p->seq_lens_host;
    in.uniform_len = 0;
    const int64_t capacity = capacity_of(p);
    if (in.lens == nullptr) {
        in.uniform_len = p->plan_len_hint > 0 ? p->plan_len_hint : (int32_t)capacity;
    }
    in.sm_count = sm_count * (p->dtype == GQA_DTYPE_BF16 ? stream_shape().ctas_per_sm : 1);
    in.max_ctas = p->max_ctas;
    const bool force_even = p->split_keys == GQA_SPLIT_EVEN;
    in.split_keys = force_even ? 0 : p->split_keys;
    in.workspace_bytes = p->workspace != nullptr ? p->workspace_bytes : 0;
    const int32_t stage_keys = p->dtype == GQA_DTYPE_BF16 ? stream_shape().keys : kChunkKeys;
    in.chunk_align = stage_keys > kChunkKeys ? stage_keys / kChunkKeys : 1;
    // The FP32 kernel spends roughly ten times longer on a chunk than the BF16 one, so the
    // fixed costs weigh a tenth as much there and finer splits pay off.
    in.overhead_scale = p->dtype == GQA_DTYPE_F32 ? 0.1 : 1.0;
    in.cluster_fit = nullptr;
    in.cluster_chunks = 0;
    if (allow_cluster && p->dtype == GQA_DTYPE_BF16 && !cluster_merge_disabled()) {
        in.cluster_fit = cluster_fit_table(sm_count);
        // Lengths read from the device may grow up to the capacity: size the clusters for it.
        if (p->seq_lens_dev != nullptr) in.cluster_chunks = ceil_div((int32_t)capacity, kChunkKeys);
    }
    if (p->block_table_dev != nullptr && p->blocks_per_seq > 1 &&
        p->layout.block_tokens % stage_keys != 0) {
        return GQA_ERR_SHAPE;
    }
    if (force_even && !(allow_even && p->dtype == GQA_DTYPE_BF16)) return GQA_ERR_UNSUPPORTED;
    in.force_even = force_even;
    in.allow_even = force_even || (allow_even && p->dtype == GQA_DTYPE_BF16 &&
                                   p->split_keys == 0 && !even_cut_disabled());
    in.capacity_chunks = ceil_div((int32_t)capacity, kChunkKeys);
    const int32_t g_max = in.max_ctas > 0 && in.max_ctas < in.sm_count ? in.max_ctas : in.sm_count;
    if (p->seq_lens_host != nullptr || p->seq_lens_dev == nullptr) {
        int rc = make_plan(in, out);
        if (rc != GQA_OK) return rc;
        if (p->seq_lens_dev != nullptr && p->workspace != nullptr &&
            ceil_div((int32_t)capacity, kChunkKeys) > out->split_chunks) {
            // The kernels follow the device lengths: keep the combine launch whenever a
            // sequence could be split, so that the launch sequence does not depend on them.
            out->needs_combine = 1;
        }
        return GQA_OK;
    }
    // Lengths are only known on the device: the split comes from the hint, the scratch is
    // sized for full sequences; a split too fine for the caller's scratch is coarsened.
    PlanInput hint = in;
    hint.workspace_bytes = 0;
    int rc = make_plan(hint, out);
    if (rc != GQA_OK) return rc;
    if (out->even_cut) {
        // The even cut follows the device lengths by itself and its scratch does not depend on
        // them; if the caller's scratch cannot hold it, fall back to uniform splits.
        if (in.workspace_bytes == 0 || out->workspace_bytes <= in.workspace_bytes) return GQA_OK;
        if (force_even) return GQA_ERR_WORKSPACE;
        hint.allow_even = false;
        rc = make_plan(hint, out);
        if (rc != GQA_OK) return rc;
    }
    PlanInput full = in;
    full.allow_even = false;
    full.uniform_len = (int32_t)capacity;
    int32_t chunks = out->split_chunks;
    const int32_t cap_chunks = ceil_div((int32_t)capacity, kChunkKeys);
    for (;;) {
        full.split_keys = chunks * kChunkKeys;
        gqa_decode_plan_info upper;
        rc = make_plan(full, &upper);
        if (rc == GQA_OK) {
            out->split_chunks = upper.split_chunks;
            out->num_items = upper.num_items;
            out->max_splits = upper.max_splits;
            out->needs_combine = upper.needs_combine;
            out->workspace_bytes = upper.workspace_bytes;
            out->num_ctas = upper.num_items < g_max ? upper.num_items : g_max;
            return GQA_OK;
        }
        if (rc != GQA_ERR_WORKSPACE || p->split_keys > 0 || chunks >= cap_chunks) return rc;
        chunks *= 2;
    }
}

// ---- tensor maps ------------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
                cudaSuccess &&
            qres == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(sym);
        }
    });
    return fn;
}

// BF16 cache as a rank-4 tensor (channel, then token/head by ascending stride, then block);
// the box is one 64-channel half of a 32-key chunk of one head, swizzled in 128-byte rows.
int encode_cache_map(const void* base, const gqa_kv_layout& l, int32_t num_kv_heads,
                     int32_t box_keys, bool* head_before_token, CUtensorMap* map) {
    auto fn = encode_fn();
    if (fn == nullptr) return GQA_ERR_CUDA;
    const bool head_first = l.stride_head < l.stride_token;
    *head_before_token = head_first;
    cuuint64_t dims[4];
    cuuint64_t strides[3];
    cuuint32_t box[4];
    cuuint32_t estr[4] = {1, 1, 1, 1};
    dims[0] = kHeadDim;
    box[0] = 64;
    if (head_first) {
        dims[1] = (cuuint64_t)num_kv_heads;
        strides[0] = (cuuint64_t)l.stride_head * 2;
        box[1] = 1;
        dims[2] = (cuuint64_t)l.block_tokens;
        strides[1] = (cuuint64_t)l.stride_token * 2;
        box[2] = (cuuint32_t)box_keys;
    } else {
        dims[1] = (cuuint64_t)l.block_tokens;
        strides[0] = (cuuint64_t)l.stride_token * 2;
        box[1] = (cuuint32_t)box_keys;
        dims[2] = (cuuint64_t)num_kv_heads;
        strides[1] = (cuuint64_t)l.stride_head * 2;
        box[2] = 1;
    }
    dims[3] = (cuuint64_t)l.num_blocks;
    strides[2] = (cuuint64_t)l.stride_block * 2;
    box[3] = 1;
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims,
                          strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? GQA_OK : GQA_ERR_UNSUPPORTED;
}

// Encoding costs a few microseconds; decode steps reuse the same caches, so keep the last few.
struct MapCacheEntry {
    const void* base;
    gqa_kv_layout layout;
    int32_t heads;
    int32_t box_keys;
    bool head_first;
    CUtensorMap map;
};

int cached_cache_map(const void* base, const gqa_kv_layout& l, int32_t heads, int32_t box_keys,
                     bool* head_first, CUtensorMap* map) {
    static std::mutex mu;
    static std::vector<MapCacheEntry> cache;
    static size_t next = 0;
    std::lock_guard<std::mutex> lock(mu);
    for (const auto& e : cache) {
        if (e.base == base && e.heads == heads && e.box_keys == box_keys &&
            std::memcmp(&e.layout, &l, sizeof(gqa_kv_layout)) == 0) {
            *map = e.map;
            *head_first = e.head_first;
            return GQA_OK;
        }
    }
    MapCacheEntry e;
    std::memset(&e, 0, sizeof(e));
    e.base = base;
    e.layout = l;
    e.heads = heads;
    e.box_keys = box_keys;
    const int rc = encode_cache_map(base, l, heads, box_keys, &e.head_first, &e.map);
    if (rc != GQA_OK) return rc;
    if (cache.size() < 32) {
        cache.push_back(e);
    } else {
        cache[next] = e;
        next = (next + 1) % cache.size();
    }
    *map = e.map;
    *head_first = e.head_first;
    return GQA_OK;
}

gqa_kv_layout clean_layout(const gqa_kv_layout& l) {
    gqa_kv_layout c;
    std::memset(&c, 0, sizeof(c));  // padding bytes take part in the cache key
    c.block_tokens = l.block_tokens;
    c.num_blocks = l.num_blocks;
    c.stride_block = l.stride_block;
    c.stride_token = l.stride_token;
    c.stride_head = l.stride_head;
    return c;
}

}  // namespace

namespace {
enum class DecodeMode { kOutput, kSeqPar, kRecords };
// A launch may cover tokens [first, first + count) of the q_tokens of each sequence.
struct TokenPass {
    int32_t first;
    int32_t count;
};
int decode_impl(const gqa_decode_params* p, const gqa_fused_front* front,
                const gqa::PeerGatherArgs* gather, DecodeMode mode, float* records, bool* fused,
                const TokenPass* pass = nullptr);
}  // namespace

int gqa::cached_matrix_map(const void* base, int64_t cols, int64_t rows, int64_t pitch,
                           CUtensorMap* map) {
    struct Entry {
        const void* base;
        int64_t cols, rows, pitch;
        CUtensorMap map;
    };
    static std::mutex mu;
    static std::vector<Entry> cache;
    static size_t next = 0;
    std::lock_guard<std::mutex> lock(mu);
    for (const auto& e : cache) {
        if (e.base == base && e.cols == cols && e.rows == rows && e.pitch == pitch) {
            *map = e.map;
            return GQA_OK;
        }
    }
    auto fn = encode_fn();
    if (fn == nullptr) return GQA_ERR_CUDA;
    Entry e;
    std::memset(&e, 0, sizeof(e));
    e.base = base;
    e.cols = cols;
    e.rows = rows;
    e.pitch = pitch;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)pitch * 2};
    cuuint32_t box[2] = {64, 16};
    cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(&e.map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
                          dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return GQA_ERR_UNSUPPORTED;
    if (cache.size() < 64) {
        cache.push_back(e);
    } else {
        cache[next] = e;
        next = (next + 1) % cache.size();
    }
    *map = e.map;
    return GQA_OK;
}

extern "C" {

const char* gqa_status_string(int status) {
    switch (status) {
        case GQA_OK: return "ok";
        case GQA_ERR_NULL: return "a required pointer is null";
        case GQA_ERR_DTYPE: return "unsupported dtype";
        case GQA_ERR_SHAPE: return "unsupported shape or layout";
        case GQA_ERR_ALIGN: return "pointer or stride is not 16-byte aligned";
        case GQA_ERR_RANGE: return "position or length outside the cache";
        case GQA_ERR_WORKSPACE: return "workspace too small";
        case GQA_ERR_CUDA: return "CUDA call failed or no device";
        case GQA_ERR_UNSUPPORTED: return "request not covered by this build";
        case GQA_ERR_COMM: return "NCCL missing or collective failed";
        case GQA_ERR_POOL: return "KV pool error";
        case GQA_ERR_TIMEOUT: return "bounded device wait ran out";
        default: return "unknown status";
    }
}

int gqa_abi_version(void) { return GQA_B200_ABI_VERSION; }

int gqa_layout_reference(int32_t layer_num, int32_t max_seq_len, int32_t num_kv_heads,
                         int32_t head_dim, gqa_kv_layout* out) {
    if (out == nullptr) return GQA_ERR_NULL;
    if (layer_num <= 0 || max_seq_len <= 0 || num_kv_heads <= 0 || head_dim <= 0) {
        return GQA_ERR_SHAPE;
    }
    std::memset(out, 0, sizeof(*out));
    out->block_tokens = max_seq_len;
    out->num_blocks = layer_num;
    out->stride_head = head_dim;
    out->stride_token = (int64_t)num_kv_heads * head_dim;
    out->stride_block = (int64_t)max_seq_len * out->stride_token;
    return GQA_OK;
}

int gqa_layout_pool(int32_t num_blocks, int32_t block_tokens, int32_t num_kv_heads,
                    int32_t head_dim, gqa_kv_layout* out) {
    if (out == nullptr) return GQA_ERR_NULL;
    if (num_blocks <= 0 || block_tokens <= 0 || num_kv_heads <= 0 || head_dim <= 0) {
        return GQA_ERR_SHAPE;
    }
    if (block_tokens % GQA_CHUNK_KEYS != 0) return GQA_ERR_SHAPE;
    std::memset(out, 0, sizeof(*out));
    out->block_tokens = block_tokens;
    out->num_blocks = num_blocks;
    out->stride_token = head_dim;
    out->stride_head = (int64_t)block_tokens * head_dim;
    out->stride_block = (int64_t)num_kv_heads * out->stride_head;
    return GQA_OK;
}

int gqa_decode_plan(const gqa_decode_params* p, int32_t sm_count, gqa_decode_plan_info* out) {
    if (out == nullptr) return GQA_ERR_NULL;
    int rc = validate_decode(p, false, true);
    if (rc != GQA_OK) return rc;
    if (sm_count <= 0) {
        rc = device_sm_count(&sm_count);
        if (rc != GQA_OK) return rc;
    }
    // More (token, head) columns than one launch holds run as several passes: plan one pass.
    gqa_decode_params planned = *p;
    const int32_t per_pass = kMaxColumns / (p->num_q_heads / p->num_kv_heads);
    if (tokens_of(p) > per_pass) planned.q_tokens = per_pass;
    rc = plan_from_params(&planned, sm_count, out);
    if (rc == GQA_OK && (out->cluster_size > 0 || out->even_cut)) {
        // gqa_decode merges these splits inside clusters and needs no workspace, or cuts the
        // units evenly over the CTAs; the calls that cannot (gathers, records) cut the keys in
        // uniform splits: report the larger of the two workspaces so that one allocation
        // serves them all.
        gqa_decode_plan_info plain;
        if (plan_from_params(&planned, sm_count, &plain, false, false) == GQA_OK &&
            plain.workspace_bytes > out->workspace_bytes) {
            out->workspace_bytes = plain.workspace_bytes;
        }
    }
    return rc;
}

int32_t gqa_cluster_capacity(int32_t cluster_size) {
    if (cluster_size < 2 || cluster_size > kMaxClusterSize) return 0;
    int32_t sms = 0;
    if (device_sm_count(&sms) != GQA_OK) return 0;
    return cluster_fit_table(sms)[cluster_size];
}

int gqa_decode(const gqa_decode_params* p) {
    return gqa::decode_with_gather(p, nullptr, nullptr, nullptr);
}

int gqa_decode_fused(const gqa_decode_params* p, const gqa_fused_front* front) {
    if (front == nullptr) return GQA_ERR_NULL;
    return gqa::decode_with_gather(p, front, nullptr, nullptr);
}

int gqa_decode_partial(const gqa_decode_params* p, float* records) {
    if (records == nullptr) return GQA_ERR_NULL;
    if (!aligned16(records)) return GQA_ERR_ALIGN;
    return decode_impl(p, nullptr, nullptr, DecodeMode::kRecords, records, nullptr);
}

int gqa_merge_partials(const float* records, int32_t nparts, int64_t rows, int32_t head_dim,
                       int32_t dtype, void* out, void* stream) {
    if (records == nullptr || out == nullptr) return GQA_ERR_NULL;
    if (dtype != GQA_DTYPE_F32 && dtype != GQA_DTYPE_BF16) return GQA_ERR_DTYPE;
    if (head_dim != kHeadDim || nparts <= 0 || rows <= 0 || rows > INT32_MAX) return GQA_ERR_SHAPE;
    const cudaError_t e = gqa::launch_merge_partials(records, nparts, rows, dtype == GQA_DTYPE_BF16,
                                                     out, reinterpret_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? GQA_OK : GQA_ERR_CUDA;
}

}  // extern "C"

int gqa::decode_with_gather(const gqa_decode_params* p, const gqa_fused_front* front,
                            const gqa::PeerGatherArgs* gather, bool* fused) {
    if (p != nullptr && p->num_kv_heads > 0 && p->q_tokens > 1 &&
        p->q_tokens * (p->num_q_heads / p->num_kv_heads) > kMaxColumns &&
        p->num_q_heads / p->num_kv_heads <= kMaxGroup && gather == nullptr) {
        // More (token, head) columns than one launch holds: several passes over the cache, each
        // over the next tokens. A later pass may not prefetch early: the pass before it may
        // still be appending its tokens' rows.
        const int32_t per_pass = kMaxColumns / (p->num_q_heads / p->num_kv_heads);
        gqa_decode_params local = *p;
        for (int32_t first = 0; first < p->q_tokens; first += per_pass) {
            const TokenPass pass = {first, p->q_tokens - first < per_pass ? p->q_tokens - first
                                                                          : per_pass};
            if (first > 0) local.early_prefetch = 0;
            const int rc = decode_impl(&local, front, nullptr, DecodeMode::kOutput, nullptr,
                                       nullptr, &pass);
            if (rc != GQA_OK) return rc;
        }
        if (fused != nullptr) *fused = false;
        return GQA_OK;
    }
    return decode_impl(p, front, gather, DecodeMode::kOutput, nullptr, fused);
}

int gqa::decode_sequence_parallel(const gqa_decode_params* p, const gqa::PeerGatherArgs* gather) {
    if (gather == nullptr) return GQA_ERR_NULL;
    return decode_impl(p, nullptr, gather, DecodeMode::kSeqPar, nullptr, nullptr);
}

namespace {

int decode_impl(const gqa_decode_params* p, const gqa_fused_front* front,
                const gqa::PeerGatherArgs* gather, DecodeMode mode, float* records, bool* fused,
                const TokenPass* pass) {
    if (fused != nullptr) *fused = false;
    const bool by_records = mode != DecodeMode::kOutput;
    int rc = validate_decode(p, by_records, pass != nullptr);
    if (rc != GQA_OK) return rc;
    const int32_t all_tokens = tokens_of(p);
    const int32_t tokens = pass != nullptr ? pass->count : all_tokens;
    // Tokens of later passes are not attended by this one: its sequences end before them.
    const int32_t len_offset = pass != nullptr ? all_tokens - pass->first - pass->count : 0;
    if (by_records && tokens > 1) return GQA_ERR_UNSUPPORTED;
    if (front != nullptr) {
        if (p->dtype != GQA_DTYPE_BF16 || by_records) return GQA_ERR_UNSUPPORTED;
        if (front->k_new == nullptr || front->v_new == nullptr || front->qk_weight == nullptr) {
            return GQA_ERR_NULL;
        }
        if ((front->sin_cache == nullptr) != (front->cos_cache == nullptr)) return GQA_ERR_NULL;
        if (front->sin_cache != nullptr && front->table_len <= 0) return GQA_ERR_RANGE;
        if (!aligned16(front->k_new) || !aligned16(front->v_new)) return GQA_ERR_ALIGN;
        // Every CTA of a unit reads the raw rows: they cannot be rotated in place.
        if (front->q_out == p->q) return GQA_ERR_UNSUPPORTED;
    }
    int32_t sms = 0;
    rc = device_sm_count(&sms);
    if (rc != GQA_OK) return rc;
    gqa_decode_plan_info plan;
    {
        gqa_decode_params planned = *p;
        planned.q_tokens = tokens;
        // Splits can be merged inside thread-block clusters (no scratch, no second launch)
        // unless the merged rows have to leave through a gather or as records.
        rc = plan_from_params(&planned, sms, &plan, mode == DecodeMode::kOutput && gather == nullptr,
                              mode == DecodeMode::kOutput);
    }
    if (rc != GQA_OK) return rc;
    const int32_t group = p->num_q_heads / p->num_kv_heads;
    const size_t rec_bytes = (size_t)group * tokens * (kHeadDim + 2) * sizeof(float);
    const int32_t cluster = plan.cluster_size;
    if (cluster > 0) {
        plan.needs_combine = 0;
        plan.workspace_bytes = 0;
        plan.num_ctas = p->batch * p->num_kv_heads * cluster;
    }
    if (by_records && !plan.needs_combine) {
        // Every unit leaves a record for the merge across slices, also when it is not split.
        plan.needs_combine = 1;
        plan.workspace_bytes = (size_t)plan.num_items * rec_bytes;
    }
    if (plan.needs_combine) {
        if (p->workspace == nullptr) return GQA_ERR_NULL;
        if (p->workspace_bytes < plan.workspace_bytes) return GQA_ERR_WORKSPACE;
        if (!aligned16(p->workspace)) return GQA_ERR_ALIGN;
    }
    const int rows = p->batch * tokens * p->num_q_heads;
    if (mode == DecodeMode::kSeqPar && rows > gqa::combine_resident_ctas(rows, sms)) {
        // Every CTA of the merge waits for its peers' records: the grid must be resident.
        return GQA_ERR_UNSUPPORTED;
    }

    gqa::DecodeArgs a;
    std::memset(&a, 0, sizeof(a));
    a.q = p->q;
    a.out = p->out;
    a.workspace = reinterpret_cast<float*>(p->workspace);
    a.k_cache = p->k_cache;
    a.v_cache = p->v_cache;
    a.seq_lens_dev = p->seq_lens_dev;
    a.block_table = p->block_table_dev;
    a.status = p->status_dev;
    a.stride_block = p->layout.stride_block;
    a.stride_token = p->layout.stride_token;
    a.stride_head = p->layout.stride_head;
    a.batch = p->batch;
    a.num_q_heads = p->num_q_heads;
    a.num_kv_heads = p->num_kv_heads;
    a.group = group;
    a.uniform_len = p->seq_lens_dev == nullptr ? p->seq_lens_host[0] - len_offset : 0;
    a.split_chunks = plan.split_chunks;
    a.blocks_per_seq = p->blocks_per_seq;
    a.block_tokens = p->layout.block_tokens;
    a.fixed_block = p->fixed_block;
    a.early_prefetch = p->early_prefetch ? 1 : 0;
    a.always_partial = by_records ? 1 : 0;
    a.q_tokens = tokens;
    a.q_token_stride = all_tokens;
    a.q_token_first = pass != nullptr ? pass->first : 0;
    a.len_offset = len_offset;
    a.len_capacity = (int32_t)capacity_of(p);
    const size_t fit = p->workspace != nullptr ? p->workspace_bytes / rec_bytes : 0;
    a.item_capacity = fit > (size_t)INT32_MAX ? INT32_MAX : (int32_t)fit;
    a.num_blocks = p->layout.num_blocks;
    a.cluster_size = cluster;
    a.even_ctas = plan.even_cut ? plan.num_ctas : 0;
    a.even_pad = plan.even_cut ? even_pad_cells() : 0;
    a.scale_log2 = (1.0f / sqrtf((float)kHeadDim)) * 1.44269504088896340736f;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(p->stream);

    cudaError_t e;
    if (p->dtype == GQA_DTYPE_BF16) {
        CUtensorMap tk, tv;
        bool head_first = false;
        const gqa_kv_layout lay = clean_layout(p->layout);
        const gqa::StreamShape shape = stream_shape();
        rc = cached_cache_map(p->k_cache, lay, p->num_kv_heads, shape.keys, &head_first, &tk);
        if (rc != GQA_OK) return rc;
        rc = cached_cache_map(p->v_cache, lay, p->num_kv_heads, shape.keys, &head_first, &tv);
        if (rc != GQA_OK) return rc;
        a.head_before_token = head_first ? 1 : 0;
        gqa::FusedFrontArgs ff;
        if (front != nullptr) {
            ff.k_new = front->k_new;
            ff.v_new = front->v_new;
            ff.qk_weight = front->qk_weight;
            ff.q_out = front->q_out;
            ff.sin_cache = front->sin_cache;
            ff.cos_cache = front->cos_cache;
            ff.table_len = front->table_len;
            ff.eps = front->eps;
        }
        e = gqa::launch_stream_bf16(tk, tv, a, front != nullptr ? &ff : nullptr, plan.num_ctas,
                                    stream);
    } else {
        e = gqa::launch_stream_f32(a, plan.num_ctas, stream);
    }
    if (e != cudaSuccess) return GQA_ERR_CUDA;
    if (plan.needs_combine) {
        gqa::CombineKind kind = gqa::CombineKind::kLocal;
        gqa::PeerGatherArgs to_records;
        if (mode == DecodeMode::kSeqPar) {
            kind = gqa::CombineKind::kSeqPar;
        } else if (mode == DecodeMode::kRecords) {
            kind = gqa::CombineKind::kRecord;
            std::memset(&to_records, 0, sizeof(to_records));
            to_records.recv = reinterpret_cast<uint32_t*>(records);
            gather = &to_records;
        } else if (gather != nullptr && gqa::combine_can_gather(rows, sms)) {
            kind = gqa::CombineKind::kGather;
        }
        e = gqa::launch_combine(a, p->dtype == GQA_DTYPE_BF16, stream,
                                kind == gqa::CombineKind::kLocal ? nullptr : gather, kind);
        if (e != cudaSuccess) return GQA_ERR_CUDA;
        if (fused != nullptr) *fused = kind == gqa::CombineKind::kGather;
    }
    return GQA_OK;
}

}  // namespace

extern "C" {

int gqa_qk_norm_rope_append(const gqa_front_params* p) {
    if (p == nullptr) return GQA_ERR_NULL;
    if (p->batch <= 0 || p->num_q_heads <= 0 || p->num_kv_heads <= 0 || p->q_tokens < 0) {
        return GQA_ERR_SHAPE;
    }
    if (p->head_dim != kHeadDim) return GQA_ERR_SHAPE;
    int rc = validate_layout(p->layout, GQA_DTYPE_BF16, p->num_kv_heads);
    if (rc != GQA_OK) return rc;
    if (p->q == nullptr || p->q_out == nullptr || p->k_new == nullptr || p->qk_weight == nullptr ||
        p->k_cache == nullptr) {
        return GQA_ERR_NULL;
    }
    if (p->v_new != nullptr && p->v_cache == nullptr) return GQA_ERR_NULL;
    if ((p->sin_cache == nullptr) != (p->cos_cache == nullptr)) return GQA_ERR_NULL;
    if (p->positions_host == nullptr && p->positions_dev == nullptr) return GQA_ERR_NULL;
    if (p->v_new != nullptr && (!aligned16(p->v_new) || !aligned16(p->v_cache))) {
        return GQA_ERR_ALIGN;
    }
    // The reference hands the kernel the cache row itself (its QKV GEMV wrote the raw key
    // there); then the key is rotated where it lies and the layout is not used for addressing.
    const bool k_in_place = p->k_cache == p->k_new && p->v_new == nullptr;
    int64_t capacity;
    if (k_in_place) {
        capacity = INT32_MAX;
    } else if (p->block_table_dev != nullptr) {
        if (p->blocks_per_seq <= 0) return GQA_ERR_SHAPE;
        capacity = (int64_t)p->blocks_per_seq * p->layout.block_tokens;
    } else {
        if (p->batch != 1) return GQA_ERR_SHAPE;
        if (p->fixed_block < 0 || p->fixed_block >= p->layout.num_blocks) return GQA_ERR_RANGE;
        capacity = p->layout.block_tokens;
    }
    const int32_t tokens = p->q_tokens > 0 ? p->q_tokens : 1;
    if (k_in_place && tokens != 1) return GQA_ERR_UNSUPPORTED;
    int32_t uniform_pos = 0;
    if (p->positions_host != nullptr) {
        for (int32_t b = 0; b < p->batch; ++b) {
            const int32_t pos = p->positions_host[b];  // of the first new token
            if (pos < 0 || (int64_t)pos + tokens > capacity) return GQA_ERR_RANGE;
            if (p->sin_cache != nullptr && pos + tokens > p->table_len) return GQA_ERR_RANGE;
            if (p->positions_dev == nullptr && pos != p->positions_host[0]) {
                return GQA_ERR_UNSUPPORTED;
            }
        }
        uniform_pos = p->positions_host[0];
    }
    gqa::FrontArgs f;
    std::memset(&f, 0, sizeof(f));
    f.q_tokens = tokens;
    f.pos_capacity = (int32_t)(capacity > INT32_MAX ? INT32_MAX : capacity);
    f.table_len = p->table_len;
    f.num_blocks = p->layout.num_blocks;
    f.status = p->status_dev;
    f.q = p->q;
    f.q_out = p->q_out;
    f.k_new = p->k_new;
    f.v_new = p->v_new;
    f.qk_weight = p->qk_weight;
    f.k_cache = p->k_cache;
    f.v_cache = p->v_cache;
    f.sin_cache = p->sin_cache;
    f.cos_cache = p->cos_cache;
    f.positions_dev = p->positions_dev;
    f.block_table = p->block_table_dev;
    f.stride_block = p->layout.stride_block;
    f.stride_token = p->layout.stride_token;
    f.stride_head = p->layout.stride_head;
    f.batch = p->batch;
    f.num_q_heads = p->num_q_heads;
    f.num_kv_heads = p->num_kv_heads;
    f.uniform_pos = uniform_pos;
    f.blocks_per_seq = p->blocks_per_seq;
    f.block_tokens = p->layout.block_tokens;
    f.fixed_block = p->fixed_block;
    f.k_in_place = k_in_place ? 1 : 0;
    f.eps = p->eps;
    const cudaError_t e = gqa::launch_front(f, reinterpret_cast<cudaStream_t>(p->stream));
    return e == cudaSuccess ? GQA_OK : GQA_ERR_CUDA;
}

int gqa_sin_cos_cache(float* sin_cache, float* cos_cache, int32_t head_dim, int32_t max_seq_len,
                      void* stream) {
    if (sin_cache == nullptr || cos_cache == nullptr) return GQA_ERR_NULL;
    if (head_dim <= 0 || (head_dim & 1) || max_seq_len <= 0) return GQA_ERR_SHAPE;
    const cudaError_t e = gqa::launch_sin_cos(sin_cache, cos_cache, head_dim, max_seq_len,
                                              reinterpret_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? GQA_OK : GQA_ERR_CUDA;
}

}  // extern "C"
