// How a decode-attention launch is cut into work items, shared by the streaming kernels and
// the combine kernel so that both sides address the same partial records.
//
//   unit  = (sequence b, kv head hk): one pass over that head's cached keys, shared by the
//           `group` query heads that read it;
//   chunk = 32 consecutive keys of a unit;
//   item  = (unit, split): `split_chunks` consecutive chunks of a unit. Item ids are
//           sequence-major, then kv head, then split, so the partial record of an item sits
//           at workspace + item * cols * (head_dim + 2) floats, cols = q_tokens * group:
//           O[cols][head_dim] scaled to the item's own running maximum, then m[cols], then
//           l[cols]. Column c of a unit is query token c / group, query head c % group.
//
// Even cut (DecodeArgs::even_ctas > 0, BF16 streaming kernel): `split_chunks` is then the size
// of a cell (one stage of the kernel). Every unit takes its cells plus even_pad places (the cost
// of starting on a unit, in stages) in one flat sequence in item-id order, and CTA c of
// G = min(even_ctas, T) streams the cells among places [c * T / G, (c + 1) * T / G) of the T
// places: every CTA gets the same amount of work to within one cell, whatever the lengths are.
// Where a CTA's range crosses into another unit a new piece starts; a piece that is not a whole
// unit leaves a partial record at index c + u (u = sequence * kv heads + kv head: the index
// grows by at least one from each piece to the next, and G + U records always suffice), so
// that a unit's records are consecutive: first CTA that holds one of its cells to last. The
// cut follows the lengths the kernels read, not the ones the launch was planned with.
//
// Lengths, block ids and record indices that come from device memory are never trusted: a
// length is clamped to what a sequence can hold, a record that would not fit the caller's
// scratch is not written, and the status word is raised (kStatusBadInput) instead.
#pragma once

#include <cstdint>

namespace gqa {

constexpr int kChunkKeys = 32;
constexpr int kHeadDim = 128;
constexpr int kMaxRaggedBatch = 1024;

// Values of the caller's status word.
constexpr int kStatusStageTimeout = 1;  // a staged chunk did not arrive within the time limit
constexpr int kStatusPeerTimeout = 2;   // a peer's words did not arrive within the time limit
constexpr int kStatusBadInput = 3;      // a device-side length, position or block id was out
                                        // of range (clamped or skipped), or a record did not
                                        // fit the scratch

struct DecodeArgs {
    const void* q;
    void* out;
    float* workspace;
    const void* k_cache;
    const void* v_cache;
    const int32_t* seq_lens_dev;  // null: every sequence has `uniform_len` keys
    const int32_t* block_table;   // null: every chunk reads block `fixed_block`
    int32_t* status;
    int64_t stride_block;
    int64_t stride_token;
    int64_t stride_head;
    int32_t batch;
    int32_t num_q_heads;
    int32_t num_kv_heads;
    int32_t group;
    int32_t uniform_len;
    int32_t split_chunks;
    int32_t blocks_per_seq;
    int32_t block_tokens;
    int32_t fixed_block;
    int32_t head_before_token;  // order of the middle tensor-map coordinates (BF16 path)
    int32_t early_prefetch;     // K/V stages may be requested before the predecessor is done
    int32_t always_partial;     // every item leaves a partial record, even a unit's only one
    int32_t q_tokens;           // query tokens per sequence (token t attends len - (T-1-t) keys)
    int32_t q_token_stride;     // tokens per sequence in q / out / k_new (>= q_tokens: a launch
    int32_t q_token_first;      //   may cover tokens [first, first + q_tokens) of a longer run)
    int32_t len_offset;         // subtracted from every device length (tokens of later passes)
    int32_t len_capacity;       // keys a sequence can hold (device lengths are clamped to it)
    int32_t item_capacity;      // partial records the scratch can hold
    int32_t num_blocks;         // blocks in the cache (block ids are checked against it)
    int32_t cluster_size;       // > 0: one thread-block cluster per unit, one CTA per split
    int32_t even_ctas;          // > 0: even cut of all units' cells over this many CTAs
    int32_t even_pad;           // cells a unit counts for on top of its stages (cost of a start)
    float scale_log2;  // (1 / sqrt(head_dim)) * log2(e)
};

__device__ inline void raise_status(const DecodeArgs& a, int code) {
    if (a.status != nullptr) atomicExch(a.status, code);
}

struct Item {
    int32_t b;
    int32_t hk;
    int32_t split;
    int32_t nsplits;
    int32_t len;
    int32_t chunk_begin;
    int32_t chunk_end;
};

__host__ __device__ inline int32_t ceil_div(int32_t a, int32_t b) { return (a + b - 1) / b; }

// Places a unit of `len` keys takes in the flat item sequence: its splits, or (even cut) its
// cells plus the padding that stands for the cost of starting on a unit.
__device__ inline int32_t unit_places(const DecodeArgs& a, int32_t len) {
    const int32_t n = ceil_div(ceil_div(max(len, 0), kChunkKeys), a.split_chunks);
    return (a.even_ctas > 0 && n > 0) ? n + a.even_pad : n;
}

// Tables for ragged batches, built in shared memory by every CTA: s_len[b] and
// s_base[b] = items of sequences before b (s_base[batch] = total).
struct WorkTables {
    const int32_t* s_len;
    const int32_t* s_base;
};

// Must be called by all threads of the CTA; needs 2 * (batch + 1) ints of shared memory.
__device__ inline WorkTables build_work_tables(const DecodeArgs& a, int32_t* smem_ints) {
    WorkTables t{nullptr, nullptr};
    if (a.seq_lens_dev == nullptr) return t;
    int32_t* s_len = smem_ints;
    int32_t* s_base = smem_ints + (a.batch + 1);
    for (int32_t b = threadIdx.x; b < a.batch; b += blockDim.x) {
        // A sequence holds at least its query tokens and at most the cache's capacity; zero
        // means "no keys here" (an empty slice of a sequence-parallel rank) and yields no item.
        const int32_t raw = a.seq_lens_dev[b] - a.len_offset;
        int32_t len = min(max(raw, 0), a.len_capacity);
        if (len != 0 && len < a.q_tokens) len = 0;
        if (len != raw && blockIdx.x == 0) raise_status(a, kStatusBadInput);
        s_len[b] = len;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        // Warp scan over contiguous segments of the batch.
        const int32_t per = ceil_div(a.batch, 32);
        const int32_t lo = min(a.batch, (int32_t)threadIdx.x * per);
        const int32_t hi = min(a.batch, lo + per);
        int32_t sum = 0;
        for (int32_t b = lo; b < hi; ++b) sum += unit_places(a, s_len[b]) * a.num_kv_heads;
        int32_t incl = sum;
        for (int32_t d = 1; d < 32; d <<= 1) {
            const int32_t up = __shfl_up_sync(0xffffffffu, incl, d);
            if ((int32_t)threadIdx.x >= d) incl += up;
        }
        int32_t run = incl - sum;
        for (int32_t b = lo; b < hi; ++b) {
            s_base[b] = run;
            run += unit_places(a, s_len[b]) * a.num_kv_heads;
        }
        if (threadIdx.x == 31) s_base[a.batch] = incl;
    }
    __syncthreads();
    t.s_len = s_len;
    t.s_base = s_base;
    return t;
}

__device__ inline int32_t total_items(const DecodeArgs& a, const WorkTables& t) {
    if (t.s_base != nullptr) return t.s_base[a.batch];
    return a.batch * a.num_kv_heads * unit_places(a, a.uniform_len);
}

__device__ inline Item decode_item(const DecodeArgs& a, const WorkTables& t, int32_t item) {
    Item it;
    int32_t within;
    if (t.s_base != nullptr) {
        int32_t lo = 0, hi = a.batch;  // largest b with s_base[b] <= item
        while (hi - lo > 1) {
            const int32_t mid = (lo + hi) >> 1;
            if (t.s_base[mid] <= item) lo = mid; else hi = mid;
        }
        it.b = lo;
        it.len = t.s_len[lo];
        within = item - t.s_base[lo];
    } else {
        const int32_t per_seq = a.num_kv_heads * unit_places(a, a.uniform_len);
        it.b = item / per_seq;
        it.len = a.uniform_len;
        within = item - it.b * per_seq;
    }
    const int32_t chunks = ceil_div(it.len, kChunkKeys);
    it.nsplits = unit_places(a, it.len);
    it.hk = within / it.nsplits;
    it.split = within - it.hk * it.nsplits;
    it.chunk_begin = it.split * a.split_chunks;
    it.chunk_end = min(chunks, it.chunk_begin + a.split_chunks);
    return it;
}

// Cluster launches: the cluster is the unit (sequence-major, then kv head), the CTA's rank in
// it is the split. False when the unit has fewer splits than the cluster has CTAs and this CTA
// has nothing to stream. A unit with more splits than CTAs (device lengths outgrew the plan)
// is cut off at the last CTA and reported.
__device__ inline bool cluster_item(const DecodeArgs& a, const WorkTables& t, Item* it) {
    const int32_t unit = blockIdx.x / a.cluster_size;
    it->split = blockIdx.x - unit * a.cluster_size;
    it->b = unit / a.num_kv_heads;
    it->hk = unit - it->b * a.num_kv_heads;
    it->len = t.s_len != nullptr ? t.s_len[it->b] : a.uniform_len;
    const int32_t chunks = ceil_div(it->len, kChunkKeys);
    int32_t nsplits = ceil_div(chunks, a.split_chunks);
    if (nsplits > a.cluster_size) {
        if (threadIdx.x == 0 && it->split == 0) raise_status(a, kStatusBadInput);
        nsplits = a.cluster_size;
    }
    it->nsplits = nsplits;
    it->chunk_begin = it->split * a.split_chunks;
    it->chunk_end = min(chunks, it->chunk_begin + a.split_chunks);
    return it->split < nsplits;
}

// Even cut: CTAs that take part (never more than there are cells, so that none of them is
// empty and the records of a unit stay consecutive; the rest of the grid idles), first cell of
// CTA `cta` (cta == ctas gives the total), and the CTA that holds a cell.
__device__ inline int32_t even_ctas(const DecodeArgs& a, int32_t total) {
    return min(a.even_ctas, total);
}
__device__ inline int32_t even_begin(int32_t cta, int32_t total, int32_t ctas) {
    return (int32_t)((int64_t)min(cta, ctas) * total / max(ctas, 1));
}
__device__ inline int32_t even_owner(int32_t cell, int32_t total, int32_t ctas) {
    return (int32_t)((((int64_t)cell + 1) * ctas - 1) / total);
}

// An item as a CTA meets it on its walk: where its partial record goes and where the walk
// continues. Not valid: the walk has ended.
struct Step {
    Item it;
    int32_t record;
    int32_t next;
    bool valid;
};

// Even cut: the first piece with keys at or after flat place `pos` in the range of CTA `cta`,
// which ends at place `range_end` (places that are a unit's padding hold no keys). In its Item,
// split = the piece's first cell within the unit and nsplits = 1 if the piece is the whole
// unit, else 2.
__device__ inline Step even_piece(const DecodeArgs& a, const WorkTables& t, int32_t pos,
                                  int32_t range_end, int32_t cta) {
    Step s;
    s.valid = false;
    s.record = 0;
    s.next = range_end;
    while (pos < range_end) {
        s.it = decode_item(a, t, pos);
        const int32_t places = min(s.it.nsplits - s.it.split, range_end - pos);
        const int32_t cells = s.it.nsplits - a.even_pad;
        const int32_t first = max(s.it.split - a.even_pad, 0);
        const int32_t end = s.it.split + places - a.even_pad;
        pos += places;
        if (end <= first) continue;  // nothing but padding of this unit
        const int32_t chunks = ceil_div(s.it.len, kChunkKeys);
        s.it.split = first;
        s.it.chunk_begin = first * a.split_chunks;
        s.it.chunk_end = min(chunks, end * a.split_chunks);
        s.it.nsplits = (first == 0 && end == cells) ? 1 : 2;
        s.record = cta + s.it.b * a.num_kv_heads + s.it.hk;
        s.next = pos;
        s.valid = true;
        break;
    }
    return s;
}

// First item and split count of unit (b, hk), for the combine kernel.
__device__ inline void unit_items(const DecodeArgs& a, const WorkTables& t, int32_t b, int32_t hk,
                                  int32_t* first_item, int32_t* nsplits) {
    if (a.even_ctas > 0) {
        const int32_t len = t.s_len != nullptr ? t.s_len[b] : a.uniform_len;
        const int32_t places = unit_places(a, len);
        const int32_t base = t.s_base != nullptr ? t.s_base[b] : b * a.num_kv_heads * places;
        const int32_t total = total_items(a, t);
        *nsplits = 0;
        *first_item = 0;
        if (places > 0) {
            const int32_t lo = base + hk * places + a.even_pad;  // the unit's first cell
            const int32_t ctas = even_ctas(a, total);
            const int32_t c_first = even_owner(lo, total, ctas);
            const int32_t c_last = even_owner(lo + places - a.even_pad - 1, total, ctas);
            *first_item = c_first + b * a.num_kv_heads + hk;
            *nsplits = c_last - c_first + 1;
        }
        return;
    }
    int32_t len, base;
    if (t.s_base != nullptr) {
        len = t.s_len[b];
        base = t.s_base[b];
    } else {
        len = a.uniform_len;
        const int32_t chunks = ceil_div(len, kChunkKeys);
        base = b * a.num_kv_heads * ceil_div(chunks, a.split_chunks);
    }
    const int32_t chunks = ceil_div(len, kChunkKeys);
    *nsplits = ceil_div(chunks, a.split_chunks);
    *first_item = base + hk * (*nsplits);
}

}  // namespace gqa
