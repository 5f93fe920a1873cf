// Device side of the peer exchange (jq_peer.cu): the epilogue a kernel runs after storing its outputs into every
// rank's y. Flag words of a rank's buffer: [0, world) arrival flags written by the peers; word 16 a CTA counter and word
// 17 the number of this rank's exchanges on the buffer, both private to the rank.
#pragma once

#include "jq_common.cuh"

namespace jq {

constexpr int PEER_MAX_WORLD = 8;
constexpr int PEER_FLAG_BYTES = 2048;   // flags and counters in the first 128 bytes, then room for PEER_TABLES copies of PeerOut
constexpr int PEER_TABLE_OFFSET = 128;
constexpr int PEER_TABLE_STRIDE = 208;
constexpr int PEER_TABLES = 8;
static_assert(sizeof(PeerOut) <= PEER_TABLE_STRIDE && PEER_TABLE_OFFSET + PEER_TABLES * PEER_TABLE_STRIDE <= PEER_FLAG_BYTES, "the tables fit the flag area");
constexpr int PEER_COUNTER_WORD = 16;
constexpr int PEER_SEQ_WORD = 17;

// Every thread of every CTA of the grid calls this once, after its last store to a peer. The CTA that arrives last
// publishes the exchange: flags_r[rank] = number of this exchange, on every rank r. The CTA barrier orders the CTA's
// stores before thread 0's system-wide fence, which is cumulative: one fence per CTA, not one per thread.
// `shared_word` is a word of shared memory the caller no longer needs.
__device__ __forceinline__ void peer_publish(uint32_t* const* flags, int rank, int world, int* shared_word) {
    int& peer_last_flag = *shared_word;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        int* counter = reinterpret_cast<int*>(flags[rank] + PEER_COUNTER_WORD);
        const int done = atomicAdd(counter, 1);
        peer_last_flag = done == (int)(gridDim.x * gridDim.y * gridDim.z) - 1;
        if (peer_last_flag) {
            *counter = 0;
        }
    }
    __syncthreads();
    if (peer_last_flag && (int)threadIdx.x < 32) {
        const uint32_t seq = flags[rank][PEER_SEQ_WORD] + 1u;  // this exchange's number
        __threadfence_system();
        if ((int)threadIdx.x < world) {
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags[threadIdx.x] + rank), "r"(seq) : "memory");
        }
        __syncwarp();
        if (threadIdx.x == 0) {
            flags[rank][PEER_SEQ_WORD] = seq;
        }
    }
}

// The wait for all ranks' flags of this rank's latest exchange, made by one warp (lane r polls rank r's flag) of a kernel
// that consumes what the exchange delivered, after its griddepcontrol.wait (the kernel that made this rank's part of
// the exchange has then finished and advanced the number). Bounded: gives up after about half a second and records
// 32 + r in *status; the caller carries on with whatever is there.
constexpr unsigned PEER_POLL_LIMIT = 1u << 22;  // polls of about 100 ns each
__device__ __forceinline__ void peer_wait_inline(const uint32_t* flags, int world, int lane, int* status) {
    if (lane < world) {
        const uint32_t seq = *reinterpret_cast<const volatile uint32_t*>(flags + PEER_SEQ_WORD);
        bool arrived = false;
        for (unsigned poll = 0; poll < PEER_POLL_LIMIT && !arrived; poll++) {
            uint32_t seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flags + lane) : "memory");
            arrived = (int32_t)(seen - seq) >= 0;
            if (!arrived) {
                __nanosleep(100);
            }
        }
        if (!arrived) {
            atomicCAS(status, 0, 32 + lane);
        }
    }
    __syncwarp();
}

// Where a kernel that writes one super-block of a Q4_K activation image (jq_q4k_image.cuh, one row of x) puts it when
// the image is shared by the ranks of a row-sharded decoder: the same offset of every rank's image area.
struct PeerImage {
    uint8_t* q4k[PEER_MAX_WORLD];     // every rank's image area (this rank's included)
    uint32_t* flags[PEER_MAX_WORLD];  // every rank's flag words
    int world, rank;
    int first_block;                  // this rank's first super-block of the image
};

// One warp copies `bytes` (a multiple of 16) it has just written at own + offset to the same offset of the other ranks.
__device__ __forceinline__ void peer_copy_block(const PeerImage& pi, size_t offset, int bytes, int lane) {
    __syncwarp();  // the warp's own stores are visible to all its lanes
    const int4* src = reinterpret_cast<const int4*>(pi.q4k[pi.rank] + offset);
    for (int c = lane; c < bytes / 16; c += 32) {
        const int4 v = __ldcg(src + c);
        for (int r = 0; r < pi.world; r++) {
            if (r != pi.rank) {
                reinterpret_cast<int4*>(pi.q4k[r] + offset)[c] = v;
            }
        }
    }
}

}  // namespace jq
