// Host-side KV block pool: geometry, free list and per-sequence block tables of the paged
// cache read by the decode kernels. See include/gqa_b200.h. No device memory is touched here;
// the caller owns the K and V arenas and uploads the block table.
#include "../../include/gqa_b200.h"

#include <cstring>
#include <new>
#include <vector>

struct gqa_kv_pool {
    int32_t num_blocks;
    int32_t block_tokens;
    int32_t num_kv_heads;
    int32_t head_dim;
    int32_t dtype;
    int32_t max_seqs;
    int32_t max_blocks_per_seq;
    std::vector<int32_t> free_list;   // stack of free physical blocks
    std::vector<int32_t> table;       // [max_seqs, max_blocks_per_seq], -1 = unassigned
    std::vector<int32_t> seq_blocks;  // blocks held per sequence
};

namespace {

size_t elem_bytes(int32_t dtype) { return dtype == GQA_DTYPE_F32 ? 4 : 2; }

bool geometry_ok(int32_t num_blocks, int32_t block_tokens, int32_t num_kv_heads, int32_t head_dim,
                 int32_t dtype) {
    if (num_blocks <= 0 || block_tokens <= 0 || num_kv_heads <= 0 || head_dim <= 0) return false;
    if (dtype != GQA_DTYPE_F32 && dtype != GQA_DTYPE_BF16) return false;
    if (block_tokens % GQA_CHUNK_KEYS != 0) return false;
    // Every head's share of a block starts on a 1 KiB boundary.
    return ((size_t)block_tokens * head_dim * elem_bytes(dtype)) % 1024 == 0;
}

}  // namespace

extern "C" {

size_t gqa_kv_pool_bytes(int32_t num_blocks, int32_t block_tokens, int32_t num_kv_heads,
                         int32_t head_dim, int32_t dtype) {
    if (!geometry_ok(num_blocks, block_tokens, num_kv_heads, head_dim, dtype)) return 0;
    return (size_t)num_blocks * num_kv_heads * block_tokens * head_dim * elem_bytes(dtype);
}

int gqa_kv_pool_create(int32_t num_blocks, int32_t block_tokens, int32_t num_kv_heads,
                       int32_t head_dim, int32_t dtype, int32_t max_seqs,
                       int32_t max_blocks_per_seq, gqa_kv_pool** out) {
    if (out == nullptr) return GQA_ERR_NULL;
    *out = nullptr;
    if (dtype != GQA_DTYPE_F32 && dtype != GQA_DTYPE_BF16) return GQA_ERR_DTYPE;
    if (!geometry_ok(num_blocks, block_tokens, num_kv_heads, head_dim, dtype)) return GQA_ERR_SHAPE;
    if (max_seqs <= 0 || max_blocks_per_seq <= 0) return GQA_ERR_SHAPE;
    gqa_kv_pool* pool = new (std::nothrow) gqa_kv_pool();
    if (pool == nullptr) return GQA_ERR_POOL;
    pool->num_blocks = num_blocks;
    pool->block_tokens = block_tokens;
    pool->num_kv_heads = num_kv_heads;
    pool->head_dim = head_dim;
    pool->dtype = dtype;
    pool->max_seqs = max_seqs;
    pool->max_blocks_per_seq = max_blocks_per_seq;
    pool->free_list.resize(num_blocks);
    // Lowest block on top of the stack, so a fresh pool hands out 0, 1, 2, ...
    for (int32_t i = 0; i < num_blocks; ++i) pool->free_list[i] = num_blocks - 1 - i;
    pool->table.assign((size_t)max_seqs * max_blocks_per_seq, -1);
    pool->seq_blocks.assign(max_seqs, 0);
    *out = pool;
    return GQA_OK;
}

void gqa_kv_pool_destroy(gqa_kv_pool* pool) { delete pool; }

int gqa_kv_pool_layout(const gqa_kv_pool* pool, gqa_kv_layout* out) {
    if (pool == nullptr || out == nullptr) return GQA_ERR_NULL;
    return gqa_layout_pool(pool->num_blocks, pool->block_tokens, pool->num_kv_heads,
                           pool->head_dim, out);
}

int gqa_kv_pool_reserve(gqa_kv_pool* pool, int32_t seq, int32_t num_tokens) {
    if (pool == nullptr) return GQA_ERR_NULL;
    if (seq < 0 || seq >= pool->max_seqs || num_tokens < 0) return GQA_ERR_POOL;
    const int32_t want = (num_tokens + pool->block_tokens - 1) / pool->block_tokens;
    if (want > pool->max_blocks_per_seq) return GQA_ERR_RANGE;
    const int32_t have = pool->seq_blocks[seq];
    if (want <= have) return GQA_OK;
    if ((size_t)(want - have) > pool->free_list.size()) return GQA_ERR_POOL;  // nothing is taken
    int32_t* row = pool->table.data() + (size_t)seq * pool->max_blocks_per_seq;
    for (int32_t i = have; i < want; ++i) {
        row[i] = pool->free_list.back();
        pool->free_list.pop_back();
    }
    pool->seq_blocks[seq] = want;
    return GQA_OK;
}

int gqa_kv_pool_release(gqa_kv_pool* pool, int32_t seq) {
    if (pool == nullptr) return GQA_ERR_NULL;
    if (seq < 0 || seq >= pool->max_seqs) return GQA_ERR_POOL;
    int32_t* row = pool->table.data() + (size_t)seq * pool->max_blocks_per_seq;
    for (int32_t i = pool->seq_blocks[seq] - 1; i >= 0; --i) {
        pool->free_list.push_back(row[i]);
        row[i] = -1;
    }
    pool->seq_blocks[seq] = 0;
    return GQA_OK;
}

int32_t gqa_kv_pool_free_blocks(const gqa_kv_pool* pool) {
    return pool == nullptr ? -1 : (int32_t)pool->free_list.size();
}

int32_t gqa_kv_pool_seq_blocks(const gqa_kv_pool* pool, int32_t seq) {
    if (pool == nullptr || seq < 0 || seq >= pool->max_seqs) return -1;
    return pool->seq_blocks[seq];
}

const int32_t* gqa_kv_pool_block_table(const gqa_kv_pool* pool) {
    return pool == nullptr ? nullptr : pool->table.data();
}

}  // extern "C"
