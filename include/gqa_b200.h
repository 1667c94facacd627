/*
 * gqa_b200 — C ABI of the B200 (sm_100a) decode-phase grouped-query attention library.
 *
 * One hot path of the LLMInfer engine is provided here and nothing else: Qwen3 decode
 * attention (one query token per sequence against a BF16 or FP32 KV cache), with the
 * QK-Norm + RoPE + KV-append stage in front of it, the KV block pool it reads from and the
 * KV-head-parallel partition across the GPUs of one node. Every entry point takes plain
 * pointers and sizes, returns a status code, never aborts, never synchronises the device
 * (except where stated) and has NO CPU fallback: without a CUDA device the compute entry
 * points return GQA_ERR_CUDA.
 *
 * Each declaration names the interface of the reference engine it stands in for, as
 * file:line inside the reference project.
 */
#ifndef GQA_B200_H
#define GQA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GQA_B200_ABI_VERSION 3

/* ---- status codes ------------------------------------------------------------------- */
#define GQA_OK 0
#define GQA_ERR_NULL (-1)        /* a required pointer is null */
#define GQA_ERR_DTYPE (-2)       /* dtype is not GQA_DTYPE_F32 / GQA_DTYPE_BF16 */
#define GQA_ERR_SHAPE (-3)       /* head counts, head_dim, batch or layout are unsupported */
#define GQA_ERR_ALIGN (-4)       /* a pointer or stride breaks the 16-byte rule */
#define GQA_ERR_RANGE (-5)       /* a position or length is outside the cache */
#define GQA_ERR_WORKSPACE (-6)   /* the workspace is too small for any valid split */
#define GQA_ERR_CUDA (-7)        /* a CUDA call failed (or no device / driver) */
#define GQA_ERR_UNSUPPORTED (-8) /* valid request this build does not cover */
#define GQA_ERR_COMM (-9)        /* NCCL is missing or a collective failed */
#define GQA_ERR_POOL (-10)       /* KV pool: out of blocks, bad sequence or handle */
#define GQA_ERR_TIMEOUT (-11)    /* a bounded device wait ran out (see status word) */

/*
 * Values a kernel leaves in the caller's device status word (status_dev; 0 = nothing happened).
 * The kernels never trap, fault or hang on bad device-side input: they clamp or skip and say so.
 */
#define GQA_STATUS_STAGE_TIMEOUT 1 /* a staged K/V chunk did not arrive within two seconds */
#define GQA_STATUS_PEER_TIMEOUT 2  /* another rank's (or CTA's) words did not arrive in time */
#define GQA_STATUS_BAD_INPUT 3     /* a length, position or block id read from device memory was
                                      out of range (clamped / row skipped), or split partials did
                                      not fit the workspace (those units are left unwritten) */

/* dtype values are the reference's base::DataType values (code/include/base/base.h:51-58). */
#define GQA_DTYPE_F32 1
#define GQA_DTYPE_BF16 2

/* Keys per chunk: the unit in which key ranges are cut, staged and split. */
#define GQA_CHUNK_KEYS 32

const char* gqa_status_string(int status);
int gqa_abi_version(void);

/* ---- KV cache addressing ------------------------------------------------------------- */
/*
 * Element (block, token, kv_head, channel) of a cache lives at
 *     block * stride_block + token * stride_token + kv_head * stride_head + channel
 * (in elements). Two layouts are used:
 *   - the reference's contiguous cache [layer, max_seq_len, kv_dim]
 *     (code/source/model/qwen3_fused.cpp:488-489): block = layer, block_tokens =
 *     max_seq_len, stride_block = max_seq_len * kv_dim, stride_token = kv_dim,
 *     stride_head = head_dim; gqa_layout_reference() fills it in;
 *   - the paged pool [block, kv_head, block_tokens, head_dim], each head's share of a
 *     block contiguous (64 KiB for 256 BF16 tokens); gqa_layout_pool() fills it in.
 * K and V caches share one layout and differ in base pointer only.
 */
typedef struct gqa_kv_layout {
    int32_t block_tokens;
    int32_t num_blocks;
    int64_t stride_block;
    int64_t stride_token;
    int64_t stride_head;
} gqa_kv_layout;

int gqa_layout_reference(int32_t layer_num, int32_t max_seq_len, int32_t num_kv_heads,
                         int32_t head_dim, gqa_kv_layout* out);
int gqa_layout_pool(int32_t num_blocks, int32_t block_tokens, int32_t num_kv_heads,
                    int32_t head_dim, gqa_kv_layout* out);

/* ---- decode attention ---------------------------------------------------------------- */
/*
 * Stands in for kernel::mha_kernel_cu (code/source/op/kernel/cuda/mha_kernel.cu:440-529,
 * declared code/source/op/kernel/cuda/mha_kernel.cuh:7-21) and its three kernels
 * (:44-208 single pass, :210-388 KV split, :399-438 combine), generalised to a batch of
 * sequences and to a paged cache.
 *
 *   q, out          [batch, q_tokens, num_q_heads, head_dim], dtype elements, 16-byte aligned.
 *   q_tokens        query tokens per sequence; 0 means 1 (a decode step). With T > 1 tokens the
 *                   sequence's last T cached positions are the tokens' own: token t attends
 *                   positions 0 .. seq_len - T + t (a causal limit per token), which is what T
 *                   consecutive decode steps compute (the reference prefills token by token
 *                   through its decode kernel, main/main_qwen3.cpp:58-65) in one pass over the
 *                   cache. BF16 only; q_tokens * (num_q_heads / num_kv_heads) <= 16 per launch,
 *                   more tokens run as several passes over the cache.
 *   k_cache/v_cache bases of the caches, `layout` addressing, dtype elements.
 *   seq_lens_host   [batch] cached positions attended (pos + 1) per sequence, or null.
 *   seq_lens_dev    the same on the device, or null. With a device array the kernels read
 *                   lengths from it (a captured graph stays valid as lengths change) and the
 *                   host copy, when also given, is used for split planning only. Without
 *                   it the host lengths must all be equal (they are passed by value). Device
 *                   lengths are clamped to what a sequence can hold; when they outgrow what
 *                   the workspace was planned for, the units whose partials no longer fit are
 *                   skipped and *status_dev is set to GQA_STATUS_BAD_INPUT: plan with the
 *                   largest lengths a replayed graph will see (plan_len_hint, or host lengths).
 *                   Given a workspace and device lengths, the combine launch is kept whenever a
 *                   sequence at full capacity would be split, so the launch sequence does not
 *                   depend on the lengths.
 *   plan_len_hint   planning length when only seq_lens_dev is given (0: block capacity). The
 *                   workspace is then sized for full sequences, with a coarser split than the
 *                   hint asks for if that is what fits p->workspace_bytes.
 *   block_table_dev [batch, blocks_per_seq] physical block of each logical block, or
 *                   null: every sequence then reads block `fixed_block` (the reference's
 *                   layer_id) and batch must be 1.
 *   workspace       FP32 scratch for split partials, gqa_decode_plan() gives the size; may
 *                   be null when the plan needs no split. Contents need no initialisation.
 *   split_keys      0 = choose from lengths and SM count (uniform splits, splits merged inside
 *                   thread-block clusters, or an even cut of all units over the CTAs, see
 *                   gqa_decode_plan_info); otherwise keys per split (rounded up to a multiple
 *                   of GQA_CHUNK_KEYS). With a non-zero split_keys the value of a head's
 *                   output depends on (length, split_keys) only, never on batch size, head
 *                   count or rank count, so equal split_keys give bit-equal results; with 0
 *                   the summation order may depend on all of those. GQA_SPLIT_EVEN asks for
 *                   the even cut whatever the planner would choose (BF16 gqa_decode,
 *                   gqa_decode_fused and the sharded gathers; GQA_ERR_UNSUPPORTED elsewhere,
 *                   GQA_ERR_WORKSPACE when the scratch cannot hold num_ctas + units records).
 *   max_ctas        0 = one CTA per SM; otherwise an upper bound on the grid.
 *   early_prefetch  0 = start reading the cache only when all earlier work of the stream has
 *                   finished. 1 = the caller promises that work still running ahead of this
 *                   call in the stream writes no cache row other than the newest position
 *                   (seq_len - 1) of each sequence and changes neither seq_lens_dev nor the
 *                   block table; K/V rows of older positions are then requested while that
 *                   work is still finishing (the reference's decode step satisfies this: its
 *                   QKV GEMV and QK-Norm write the row of `pos` only).
 *   status_dev      optional device int32, set to a GQA_STATUS_* value by a kernel whose
 *                   bounded wait ran out (it then skips its work instead of hanging) or that
 *                   met out-of-range device-side input.
 *   stream          cudaStream_t (null = default stream), as the reference passes it.
 */
#define GQA_SPLIT_EVEN (-1)  /* gqa_decode_params.split_keys: cut all units evenly over the CTAs */

typedef struct gqa_decode_params {
    int32_t dtype;
    int32_t batch;
    int32_t num_q_heads;
    int32_t num_kv_heads;
    int32_t head_dim;
    int32_t blocks_per_seq;
    int32_t fixed_block;
    int32_t split_keys;
    int32_t max_ctas;
    int32_t plan_len_hint;
    int32_t early_prefetch;
    int32_t q_tokens;
    gqa_kv_layout layout;
    const void* q;
    const void* k_cache;
    const void* v_cache;
    void* out;
    void* workspace;
    size_t workspace_bytes;
    const int32_t* seq_lens_host;
    const int32_t* seq_lens_dev;
    const int32_t* block_table_dev;
    int32_t* status_dev;
    void* stream;
} gqa_decode_params;

typedef struct gqa_decode_plan_info {
    int32_t split_chunks;     /* chunks of GQA_CHUNK_KEYS keys per split */
    int32_t max_splits;       /* splits of the longest sequence */
    int32_t num_items;        /* (sequence, kv head, split) work items (upper bound) */
    int32_t num_ctas;         /* grid of the streaming kernel */
    int32_t needs_combine;    /* 1 when a second, LSE-combine launch follows */
    int32_t cluster_size;     /* > 0: gqa_decode can merge the splits inside thread-block clusters
                                 of this many CTAs (one cluster per (sequence, kv head), one CTA
                                 per split) instead: no combine launch and no workspace, provided
                                 the GPU holds all clusters at once and no gather is fused in */
    size_t workspace_bytes;   /* scratch the chosen plan needs */
    int32_t even_cut;         /* 1: no uniform splits; the stages of all (sequence, kv head) units
                                 form one flat sequence that is cut evenly over num_ctas CTAs, a
                                 partial record per piece of a cut unit (num_items = num_ctas +
                                 units records at most), merged by the combine launch. The cut
                                 follows the lengths the kernels read. split_chunks is then the
                                 granularity of the cut, max_splits the most pieces of a unit */
    int32_t reserved;
} gqa_decode_plan_info;

/*
 * Host only: validates `p` (without touching its device pointers) and chooses the split.
 * sm_count 0 asks the current device. Replaces the reference's fixed rule "split every 32
 * keys once seq_len > 128" (mha_kernel.cu:505-517) and its workspace sizing
 * (code/source/model/qwen3_fused.cpp:502). When p->workspace_bytes is non-zero the plan is
 * kept within it; pass 0 to ask how much the unconstrained plan wants.
 */
int gqa_decode_plan(const gqa_decode_params* p, int32_t sm_count, gqa_decode_plan_info* out);

/*
 * How many thread-block clusters of `cluster_size` CTAs (2 .. 16) of the BF16 streaming kernel
 * the current GPU holds at once; 0 when it takes none of that size. The planner merges splits
 * inside clusters only when every (sequence, kv head) unit gets its cluster in one wave.
 */
int32_t gqa_cluster_capacity(int32_t cluster_size);

/* Launches the attention kernels on p->stream. Asynchronous. */
int gqa_decode(const gqa_decode_params* p);

/*
 * gqa_decode() with the front stage inside the attention kernel: one launch does what
 * kernel::fused_qk_norm_rope_kernel_cu (code/source/op/kernel/cuda/rmsnorm_kernel.cu:205-290),
 * the KV-row placement (code/source/model/model.cpp:90-107, code/source/op/kernel/cuda/
 * matmul_kernel.cu:238-246) and kernel::mha_kernel_cu (code/source/op/kernel/cuda/
 * mha_kernel.cu:440-529) do in sequence. p->q holds the RAW query rows (the QKV projection's
 * output); every CTA normalises and rotates the rows of its own unit (the same operations, hence
 * the same bits, as gqa_qk_norm_rope_append), and the CTA that streams the chunk holding a new
 * token's position computes that token's key row, patches it (and the value row) into its
 * staged tile and appends both to the cache. Positions are implied: token t of sequence b sits
 * at position seq_len_b - q_tokens + t, whose cache rows need not be written beforehand.
 * BF16 only. With p->early_prefetch the caller promises that no work still running ahead in
 * the stream writes these caches, the lengths or the block table at all.
 */
typedef struct gqa_fused_front {
    const void* k_new;     /* [batch, q_tokens, num_kv_heads, head_dim] raw keys */
    const void* v_new;     /* same shape, values */
    const void* qk_weight; /* [2 * head_dim] BF16: query norm weights, then key norm weights */
    void* q_out;           /* optional: the rotated queries, laid out like p->q; must not alias it */
    const float* sin_cache; /* FP32 [table_len, head_dim / 2] as built by gqa_sin_cos_cache, or */
    const float* cos_cache; /* both null: angles are computed in the kernel, same formula */
    int32_t table_len;
    float eps;
} gqa_fused_front;

int gqa_decode_fused(const gqa_decode_params* p, const gqa_fused_front* front);

/*
 * Attention over a SLICE of each sequence's keys that leaves, instead of the output, one record
 * per output row [batch * q_tokens * num_q_heads][head_dim + 2] FP32 in `records`: the row's
 * 128 channel sums relative to the slice's maximum score, that maximum (log2 domain), and the
 * sum of the weights. p describes the slice as gqa_decode describes a whole sequence, except
 * that a length may be 0 (a slice that holds no key of a sequence; its record is 0, -inf, 0).
 * p->out is not written. Always needs a workspace (gqa_decode_plan's, or at least
 * num_items * (num_q_heads / num_kv_heads) * (head_dim + 2) * 4 bytes when the plan asks for
 * none). gqa_merge_partials turns the records of all slices into the output. No counterpart in
 * the reference; it is the arithmetic of gqa_decode_seqpar without the exchange, for callers
 * that move the records themselves.
 */
int gqa_decode_partial(const gqa_decode_params* p, float* records);

/*
 * out[row] = merge of records[part][row], part = 0 .. nparts - 1 in ascending order (the same
 * device function gqa_decode_seqpar applies to the records of the ranks). records is
 * [nparts][rows][head_dim + 2] FP32 on the device, out [rows][head_dim] of `dtype`.
 */
int gqa_merge_partials(const float* records, int32_t nparts, int64_t rows, int32_t head_dim,
                       int32_t dtype, void* out, void* stream);

/*
 * No counterpart in the reference (its caller always allocates kv_split_output,
 * code/source/model/qwen3_fused.cpp:502). The same attention as gqa_decode() for callers that
 * cannot allocate device memory around the call - code running under stream capture, serving
 * loops barred from the allocator after start-up, hosts with a fixed memory budget: p->workspace
 * and p->workspace_bytes are ignored and the split partials go to an array of
 * GQA_STATIC_SCRATCH_BYTES that lives inside the library (each GPU that loads the library holds
 * it until the process exits). The call allocates and frees no device memory.
 *   - The first call on a device looks up the array's device address
 *     (cudaGetSymbolAddress); make that first call outside any stream capture.
 *   - The planner keeps its split within GQA_STATIC_SCRATCH_BYTES (coarsening it when lengths
 *     are known on the device only and records are sized for full sequences); an explicit
 *     split_keys whose records cannot fit returns GQA_ERR_WORKSPACE and launches nothing.
 *     Device-side lengths that outgrow the plan make the kernels skip the records that would
 *     not fit and set *status_dev to GQA_STATUS_BAD_INPUT; nothing is written past the array.
 *   - All calls on one device share the array. Calls that can overlap on the GPU (different
 *     streams, concurrent graph launches) race on it: serialise them, or use gqa_decode() with
 *     one workspace each. Nothing in the array has to be cleared between calls.
 */
#define GQA_STATIC_SCRATCH_BYTES (8u << 20)
int gqa_decode_static_scratch(const gqa_decode_params* p);

/* ---- front stage: QK-Norm + RoPE + KV append ------------------------------------------ */
/*
 * Stands in for kernel::fused_qk_norm_rope_kernel_cu
 * (code/source/op/kernel/cuda/rmsnorm_kernel.cu:205-290) and for the KV-row placement done
 * by Model::slice_kv_cache (code/source/model/model.cpp:90-107) together with the
 * destination select of the QKV GEMV (code/source/op/kernel/cuda/matmul_kernel.cu:238-246).
 *
 * Per sequence b at position pos_b: q[b] is RMS-normalised per head (eps), scaled by
 * qk_weight[0:head_dim], rotated (rotate-half pairs (i, i + head_dim/2)) and written to
 * q_out[b]; k_new[b] likewise with qk_weight[head_dim:2*head_dim], written to the K cache
 * row of pos_b; v_new[b] is copied unchanged to the V cache row. BF16 only, FP32 math,
 * one rounding at the end.
 *   q, q_out        [batch, num_q_heads, head_dim]; may alias (the reference works in place).
 *   k_new, v_new    [batch, num_kv_heads, head_dim]. v_new null = V untouched. When k_new
 *                   and k_cache are the same pointer (and v_new is null) the key already
 *                   lies in its cache row, as in the reference where the QKV GEMV wrote it
 *                   there: it is then normalised and rotated in place and the layout is not
 *                   used for addressing.
 *   sin_cache/cos_cache  FP32 [table_len, head_dim/2] as built by gqa_sin_cos_cache, or
 *                   both null: angles are then computed in the kernel with the same formula.
 *   positions_host  [batch] or null; positions_dev [batch] on the device or null. One of
 *                   them is required; the device array wins.
 *   q_tokens        new tokens per sequence; 0 means 1. Token t of sequence b sits at position
 *                   pos_b + t; q, q_out, k_new, v_new are then [batch, q_tokens, heads, head_dim].
 *   status_dev      optional device int32. A position read from device memory that lies
 *                   outside the cache or the angle tables, or an unassigned block-table entry,
 *                   skips that row and sets it to GQA_STATUS_BAD_INPUT (host positions are
 *                   refused with GQA_ERR_RANGE before the launch).
 */
typedef struct gqa_front_params {
    int32_t batch;
    int32_t num_q_heads;
    int32_t num_kv_heads;
    int32_t head_dim;
    int32_t blocks_per_seq;
    int32_t fixed_block;
    int32_t table_len;
    float eps;
    gqa_kv_layout layout;
    const void* q;
    void* q_out;
    const void* k_new;
    const void* v_new;
    const void* qk_weight;
    void* k_cache;
    void* v_cache;
    const float* sin_cache;
    const float* cos_cache;
    const int32_t* positions_host;
    const int32_t* positions_dev;
    const int32_t* block_table_dev;
    void* stream;
    int32_t* status_dev;
    int32_t q_tokens;
    int32_t reserved;
} gqa_front_params;

int gqa_qk_norm_rope_append(const gqa_front_params* p);

/*
 * Stands in for kernel::sin_cos_cache_precompute_cu
 * (code/source/op/kernel/cuda/rope_kernel.cu:6-46): FP32 tables [max_seq_len, head_dim/2],
 * freq_i = 1 / powf(1e6, 2i / head_dim), sincosf((float)pos * freq_i).
 */
int gqa_sin_cos_cache(float* sin_cache, float* cos_cache, int32_t head_dim, int32_t max_seq_len,
                      void* stream);

/* ---- one decode step from host buffers ------------------------------------------------ */
/*
 * What a caller that keeps only the KV cache on the device does per layer and token: copy
 * the new token's q/k/v rows (host, ideally pinned) to the device, run the front stage and
 * the attention, copy the attention output back and wait for it. The session owns the
 * device staging buffers, the split workspace and a stream, all allocated at creation.
 * Mirrors one iteration of the reference's layer loop around attention
 * (code/source/model/qwen3_fused.cpp:517-553) minus its GEMVs.
 */
typedef struct gqa_session gqa_session;

int gqa_session_create(int32_t dtype, int32_t max_batch, int32_t num_q_heads,
                       int32_t num_kv_heads, int32_t head_dim, int32_t max_seq_len,
                       gqa_session** out);
void gqa_session_destroy(gqa_session* s);

/*
 * q_host/k_host/v_host/out_host: [batch, heads, head_dim] BF16 on the host. positions_host
 * [batch]: the new token's position per sequence; it attends positions 0..pos. Blocks until
 * out_host is filled. Buffers in pinned memory (cudaMallocHost / cudaHostRegister, mapped,
 * 16-byte aligned) are read and written by the kernels where they lie; pageable ones go
 * through the session's own pinned blocks. Cache pointers, layout and block table as in gqa_decode_params.
 */
int gqa_session_step(gqa_session* s, int32_t batch, const void* q_host, const void* k_host,
                     const void* v_host, const void* qk_weight_dev, void* k_cache, void* v_cache,
                     const gqa_kv_layout* layout, const int32_t* positions_host,
                     const int32_t* block_table_dev, int32_t blocks_per_seq,
                     int32_t fixed_block, void* out_host);

/*
 * Host-side time of the last successful step in nanoseconds: [0] placing the rows in the pinned
 * block, [1] issuing the launches, [2] waiting for the GPU, [3] handing the output over. For
 * callers who want to see where a step's end-to-end time goes; no counterpart in the reference.
 * A step whose kernels report a timed-out wait returns GQA_ERR_TIMEOUT, one whose kernels met an
 * out-of-range length, position or block id returns GQA_ERR_RANGE.
 */
int gqa_session_last_timing(const gqa_session* s, int64_t* ns_out);

/*
 * The same step on one rank of a KV-head-parallel group (see gqa_comm below): the session was
 * created with the LOCAL head counts, host rows are this rank's heads, and after the local
 * attention the outputs of all ranks are gathered: by the GPUs' own stores over NVLink straight
 * into pinned host memory when gqa_comm_enable_peer_gather was called (from the combine kernel
 * itself when units are split), else with ncclAllGather on the device and a copy.
 * gathered_host is [nranks, batch, local_q_heads, head_dim]. Collective: every rank of `comm`
 * must call it.
 */
struct gqa_comm;
int gqa_session_step_sharded(gqa_session* s, struct gqa_comm* comm, int32_t batch,
                             const void* q_host, const void* k_host, const void* v_host,
                             const void* qk_weight_dev, void* k_cache, void* v_cache,
                             const gqa_kv_layout* layout, const int32_t* positions_host,
                             const int32_t* block_table_dev, int32_t blocks_per_seq,
                             int32_t fixed_block, void* gathered_host);

/* ---- KV block pool -------------------------------------------------------------------- */
/*
 * Host-side owner of a paged KV cache: block geometry with every head's share of a block
 * 1024-byte aligned (the staging tiles are swizzled in 1 KiB atoms and bulk tensor copies
 * want 16-byte strides), a free list, and one block table row per sequence. Takes the
 * place of the contiguous per-layer caches the reference allocates from its
 * CUDADeviceAllocator pool (code/source/model/qwen3_fused.cpp:483-489,
 * code/source/base/alloc_cu.cpp:7-79). The pool does not allocate device memory: the
 * caller provides K and V arenas of gqa_kv_pool_bytes() each.
 */
typedef struct gqa_kv_pool gqa_kv_pool;

size_t gqa_kv_pool_bytes(int32_t num_blocks, int32_t block_tokens, int32_t num_kv_heads,
                         int32_t head_dim, int32_t dtype);
int gqa_kv_pool_create(int32_t num_blocks, int32_t block_tokens, int32_t num_kv_heads,
                       int32_t head_dim, int32_t dtype, int32_t max_seqs,
                       int32_t max_blocks_per_seq, gqa_kv_pool** out);
void gqa_kv_pool_destroy(gqa_kv_pool* pool);
int gqa_kv_pool_layout(const gqa_kv_pool* pool, gqa_kv_layout* out);
/* Grows sequence `seq` to hold `num_tokens` tokens, taking blocks from the free list. */
int gqa_kv_pool_reserve(gqa_kv_pool* pool, int32_t seq, int32_t num_tokens);
/* Returns every block of `seq` to the free list. */
int gqa_kv_pool_release(gqa_kv_pool* pool, int32_t seq);
int32_t gqa_kv_pool_free_blocks(const gqa_kv_pool* pool);
int32_t gqa_kv_pool_seq_blocks(const gqa_kv_pool* pool, int32_t seq);
/* Host block table [max_seqs, max_blocks_per_seq] (-1 = unassigned); copy it to the device. */
const int32_t* gqa_kv_pool_block_table(const gqa_kv_pool* pool);

/* ---- KV-head-parallel partition -------------------------------------------------------- */
/*
 * New with respect to the reference, which runs on one device
 * (code/source/model/qwen3_fused.cpp:68): rank r of n owns kv heads
 * [first_kv_head, first_kv_head + num_local_kv_heads) together with their query groups.
 * n must divide num_kv_heads.
 */
int gqa_shard_plan(int32_t num_q_heads, int32_t num_kv_heads, int32_t nranks, int32_t rank,
                   int32_t* first_kv_head, int32_t* num_local_kv_heads,
                   int32_t* first_q_head, int32_t* num_local_q_heads);

#define GQA_COMM_ID_BYTES 128
typedef struct gqa_comm gqa_comm;

int32_t gqa_comm_nranks(const gqa_comm* comm);
/* All-gather of `bytes` bytes per rank on `stream`; recv is [nranks][bytes]. */
int gqa_comm_all_gather(gqa_comm* comm, const void* send, void* recv, size_t bytes, void* stream);

/*
 * Collective, once per communicator: sets up the NVLink peer gather for outputs of up to
 * max_bytes_per_rank bytes per rank. Every rank allocates a window of
 * 4 * nranks * max_bytes_per_rank bytes that the other ranks map through CUDA IPC (one process
 * per GPU on one node, all GPUs visible to every process). Afterwards gqa_decode_sharded
 * gathers with the GPUs' own stores (gqa_comm_peer_gather) whenever the output fits, instead
 * of ncclAllGather. Synchronises the device. At most 8 ranks. The same windows carry the
 * exchanges of gqa_oproj_residual_sharded and gqa_decode_seqpar. Words in a window are tagged
 * with a 32-bit step counter kept on the device: a process that runs more than 2^31 exchange
 * steps on one communicator should disable and enable the peer gather again (between steps,
 * on every rank) before the counter wraps.
 */
int gqa_comm_enable_peer_gather(gqa_comm* comm, size_t max_bytes_per_rank);
/* Back to ncclAllGather (every rank must do the same); frees the window. */
void gqa_comm_disable_peer_gather(gqa_comm* comm);
/*
 * One gather step with peer stores on `stream`: recv is [nranks][bytes]; bytes is a multiple
 * of 16 and both buffers are 16-byte aligned. Collective (every rank calls it once per step,
 * in the same order). A rank whose peers do not arrive within two seconds sets *status_dev to
 * 2 (when given), leaves recv unspecified and returns: the kernel never hangs.
 */
int gqa_comm_peer_gather(gqa_comm* comm, const void* send, void* recv, size_t bytes,
                         int32_t* status_dev, void* stream);
/*
 * 1 when an exchange of `bytes` bytes per rank would go through the peer windows, 0 when it
 * would fall back to ncclAllGather (windows not enabled, or too small). Depends on the
 * communicator's state and the size only, so every rank gets the same answer.
 */
int gqa_comm_peer_gather_fits(const gqa_comm* comm, size_t bytes);

/* Rank 0 makes the id; the caller hands it to every rank (any host channel). */
int gqa_comm_unique_id(void* id_out);
/* Collective over all ranks; the current CUDA device is the rank's GPU. */
int gqa_comm_init(const void* id, int32_t nranks, int32_t rank, gqa_comm** out);
void gqa_comm_destroy(gqa_comm* comm);

/*
 * Runs gqa_decode on this rank's heads (p describes the LOCAL shard: local head counts,
 * local caches) and gathers every rank's output over NVLink on p->stream: with the peer-store
 * kernel when gqa_comm_enable_peer_gather was called and the output fits, else with one
 * ncclAllGather. p->out is the local output [batch, local_q_heads, head_dim]; gathered is
 * [nranks, batch, local_q_heads, head_dim]. When units are split and the combine grid
 * (batch * local_q_heads CTAs) fits the GPU at once, the peer stores are issued by the combine
 * kernel itself, row by row as rows are merged, and no separate gather kernel is launched.
 */
int gqa_decode_sharded(const gqa_decode_params* p, gqa_comm* comm, void* gathered);
/* The same with the front stage inside the attention kernel (see gqa_decode_fused). */
int gqa_decode_sharded_fused(const gqa_decode_params* p, const gqa_fused_front* front,
                             gqa_comm* comm, void* gathered);

/*
 * Sequence-parallel decode: every rank holds ALL heads but only a slice of each sequence's
 * cached keys and values (for example every N-th block, or one contiguous part). p describes
 * the LOCAL slice (local caches, local lengths; a rank that holds no key of a sequence passes
 * length 0 for it and contributes the empty record). Each
 * rank attends over its slice; the combine kernel then sends the row's record (128 channel
 * sums relative to the slice's maximum, the maximum and the row sum) to the other ranks
 * through the peer windows and merges all ranks' records in rank order, so p->out
 * [batch, num_q_heads, head_dim] holds the complete attention output, bit-equal on every
 * rank. The way past one KV head per GPU, and a way to balance ragged batches; the reference
 * has no counterpart. Needs gqa_comm_enable_peer_gather(comm, batch * num_q_heads *
 * (head_dim + 2) * 4) and a workspace (gqa_decode_plan's, or at least
 * num_items * (num_q_heads / num_kv_heads) * (head_dim + 2) * 4 bytes when the plan needs
 * none). A wait that runs out sets *status_dev to 2.
 */
int gqa_decode_seqpar(const gqa_decode_params* p, gqa_comm* comm);

/* ---- the projection behind attention ---------------------------------------------------- */

/*
 * Output projection with residual add, the step that follows attention in a decoder layer:
 *     residual[b, n] = bf16(float(residual[b, n]) + sum_c attn_out[b, c] * weight[n, c])
 * Replaces kernel::fused_gemv_add_kernel_cu (code/source/op/kernel/cuda/matmul_kernel.cu:
 * 143-208; single token there, `batch` tokens here, the weights are read once for all of
 * them). FP32 accumulation on tensor cores; the summation order is fixed: the query heads of a
 * KV head are taken in two halves when their number is even (else in one piece); per piece eight
 * accumulators (one per block of 16 columns inside a query head) run over the piece's heads in
 * ascending order and are added in ascending order; lower half + upper half; KV heads are added
 * in ascending order; the residual comes last. Results agree with the reference kernel to one BF16 unit in
 * the last place. The weights travel by TMA: `weight` must stay valid and unchanged in place
 * (a tensor map per matrix is cached by address).
 *
 * In a KV-head-parallel node every rank holds the columns of its own heads
 * (gqa_oproj_residual_sharded): `weight` then points at this rank's first column inside the
 * full matrix (weight_ld = the full row length) or at a packed slice (weight_ld = local
 * columns), attn_out is the rank's LOCAL attention output (no gather of it is needed), and
 * the per-KV-head partial sums are exchanged through the peer windows of
 * gqa_comm_enable_peer_gather (which must have been called with max_bytes_per_rank >=
 * 4 * local_kv_heads * min(batch, 8) * hidden). Every rank ends with the same, complete
 * `residual`, bit-equal to what the unsharded call computes. A wait that runs out sets
 * *status_dev to 2.
 *
 * The CTAs of a launch hand their partial sums to one another, so the grid is sized to be
 * resident all at once on an otherwise idle GPU: run the call on a stream that has the GPU to
 * itself (kernels of other streams that hold SMs at the same time can delay CTAs past the
 * two-second limit of those waits, which then report GQA_STATUS_PEER_TIMEOUT).
 */
typedef struct gqa_oproj_params {
    int32_t batch;        /* tokens (sequences of a decode step) */
    int32_t hidden;       /* output rows; a multiple of 16 */
    int32_t num_q_heads;  /* query heads whose columns this call holds */
    int32_t num_kv_heads; /* KV heads they belong to: divides num_q_heads, quotient <= 16 */
    int32_t head_dim;     /* 128 */
    int32_t reserved;
    int64_t weight_ld;    /* elements between weight rows, >= num_q_heads * 128, % 8 == 0 */
    const void* attn_out; /* [batch, num_q_heads * 128] bf16 */
    const void* weight;   /* bf16, row n column c at weight[n * weight_ld + c] */
    void* residual;       /* [batch, hidden] bf16, read and written */
    void* workspace;      /* gqa_oproj_workspace_bytes() bytes, 16-byte aligned; null if 0 */
    size_t workspace_bytes;
    int32_t* status_dev;  /* may be null */
    void* stream;
} gqa_oproj_params;

/*
 * Workspace of the projection for `num_kv_heads` KV heads held by the caller (0 for one KV
 * head). The caller zero-fills it once after allocating it; every call leaves it zeroed
 * where that matters (per-tile arrival counters), so it can be reused by the next call on
 * the same stream without further care. Calls that overlap on different streams need
 * workspaces of their own. Sums in flight are tagged with a 32-bit launch counter kept in the
 * workspace: a process that makes more than 2^31 calls on one workspace should zero-fill it
 * again (between calls) before the counter wraps.
 */
size_t gqa_oproj_workspace_bytes(int32_t hidden, int32_t num_kv_heads);

int gqa_oproj_residual(const gqa_oproj_params* p);
int gqa_oproj_residual_sharded(const gqa_oproj_params* p, gqa_comm* comm);

/* ---- the projection in front of attention ------------------------------------------------ */

/*
 * Packed QKV projection, the step that precedes QK-Norm + RoPE in a decoder layer:
 *     row n of weight [(Hq + 2 Hkv) * 128, hidden] . x[b]  ->  bf16
 * rows [0, Hq*128) to q_out [batch, Hq*128], the next Hkv*128 rows to k_out, the last Hkv*128
 * rows to v_out (both [batch, Hkv*128]). Replaces kernel::fused_qkv_gemv_kernel_cu
 * (code/source/op/kernel/cuda/matmul_kernel.cu:211-298; single token there). q_out, k_out
 * and v_out are what gqa_qk_norm_rope_append takes as q, k_new and v_new. Same kernel, same
 * numerics contract (one BF16 unit in the last place against the reference kernel) and same
 * workspace rules as gqa_oproj_residual. hidden is a multiple of 128. A rank of a
 * KV-head-parallel node passes the rows of its own heads, packed the same way; there is
 * nothing to exchange.
 */
typedef struct gqa_qkv_params {
    int32_t batch;
    int32_t hidden;       /* input columns */
    int32_t num_q_heads;  /* output rows: (num_q_heads + 2 * num_kv_heads) * 128 */
    int32_t num_kv_heads;
    int32_t head_dim;     /* 128 */
    int32_t reserved;
    int64_t weight_ld;    /* elements between weight rows, >= hidden, % 8 == 0 */
    const void* x;        /* [batch, hidden] bf16 */
    const void* weight;   /* bf16 */
    void* q_out;
    void* k_out;
    void* v_out;
    void* workspace;      /* gqa_qkv_workspace_bytes() bytes, zero-filled once; null if 0 */
    size_t workspace_bytes;
    int32_t* status_dev;  /* may be null */
    void* stream;
} gqa_qkv_params;

size_t gqa_qkv_workspace_bytes(int32_t hidden, int32_t num_q_heads, int32_t num_kv_heads);
int gqa_qkv_gemv(const gqa_qkv_params* p);

#ifdef __cplusplus
}
#endif

#endif /* GQA_B200_H */
