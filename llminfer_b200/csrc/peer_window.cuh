// The peer-gather window: device memory that every rank of a node maps from every other rank
// (CUDA IPC), and the word protocol used to move small outputs through it with plain stores
// over NVLink. Shared by the stand-alone gather kernel (shard_comm.cu) and by the combine
// kernel's fused gather epilogue (decode_f32.cu).
//
// A window holds two halves of `nranks` slots, then the control words. Step e uses half
// e & 1. Payload travels as 8-byte words: low 4 bytes data, high 4 bytes the step number;
// an 8-byte store is a single transaction, so a reader sees a word whole or not at all and a
// word that shows the current step has arrived. No fences, no separate flags.
#pragma once

#include <cstddef>
#include <cstdint>

struct gqa_comm;

namespace gqa {

constexpr int kMaxPeers = 8;
constexpr uint64_t kGatherWaitNs = 2000000000ull;  // bounded poll: two seconds

// Control words at the end of a window.
struct WindowCtrl {
    uint32_t step;        // completed gathers
    uint32_t ticket_out;  // CTAs that finished the current gather
    uint32_t status;      // 1 after a wait ran out
    uint32_t pad;
};

struct PeerGatherArgs {
    uint8_t* windows[kMaxPeers];  // every rank's window as mapped into this process
    const uint32_t* send;         // this rank's payload (stand-alone kernel only)
    uint32_t* recv;               // [nranks][words] gathered payload
    int32_t* status;
    uint64_t slot_bytes;   // capacity of one slot (payload + step words)
    uint64_t words;        // 4-byte payload words per rank in this step
    int32_t nranks;
    int32_t rank;
};

// Host side: the windows of a communicator for an exchange of `bytes_per_rank` payload bytes
// per rank. GQA_ERR_COMM when the peer windows were not set up, GQA_ERR_SHAPE when a slot is
// too small for that payload.
int comm_peer_args(const gqa_comm* comm, size_t bytes_per_rank, int32_t* status_dev,
                   PeerGatherArgs* out);

__device__ __forceinline__ WindowCtrl* window_ctrl(uint8_t* window, uint64_t slot_bytes,
                                                   int nranks) {
    return reinterpret_cast<WindowCtrl*>(window + 2 * (uint64_t)nranks * slot_bytes);
}

__device__ __forceinline__ unsigned long long* window_slot(uint8_t* window, uint32_t step,
                                                           int nranks, int slot,
                                                           uint64_t slot_bytes) {
    return reinterpret_cast<unsigned long long*>(
        window + ((uint64_t)(step & 1u) * nranks + slot) * slot_bytes);
}

__device__ __forceinline__ void push_word(unsigned long long* dst, uint32_t step, uint32_t data) {
    const unsigned long long word = ((unsigned long long)step << 32) | data;
    asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(dst), "l"(word) : "memory");
}

__device__ __forceinline__ unsigned long long load_word(const unsigned long long* src) {
    unsigned long long word;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(word) : "l"(src) : "memory");
    return word;
}

// Polls one word until it shows `step` or the time limit passes (false).
__device__ __forceinline__ bool poll_word(const unsigned long long* src, uint32_t step,
                                          unsigned long long start_ns, uint32_t* data) {
    while (true) {
        unsigned long long word;
        asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(word) : "l"(src) : "memory");
        if ((uint32_t)(word >> 32) == step) {
            *data = (uint32_t)word;
            return true;
        }
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (now - start_ns > kGatherWaitNs) return false;
    }
}

__device__ __forceinline__ unsigned long long global_timer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

}  // namespace gqa
