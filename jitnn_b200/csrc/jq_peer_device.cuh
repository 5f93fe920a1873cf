// Device side of the peer exchange (jq_peer.cu): the epilogue a kernel runs after storing its outputs into every
// rank's y. Flag words of a rank's buffer: word r of [0, world) counts what has arrived from rank r, written by rank r with
// release-ordered remote adds; word 17 is the number of exchanges this rank has made on the buffer, private to the rank
// (words 16 and 18 serve the exchanges that travel as marked words, further down).
// Every exchange adds exactly 2^16 to a counter, whatever the grid that makes it: CTA i of G adds
// floor((i + 1) 2^16 / G) - floor(i 2^16 / G), so rank r's part of this rank's exchange number e has arrived once
// counter[r] - e 2^16 >= 0 (32-bit wrap-around arithmetic on both sides).
#pragma once

#include "jq_common.cuh"

namespace jq {

constexpr int PEER_MAX_WORLD = 8;
constexpr int PEER_FLAG_BYTES = 4096;   // counters in the first 128 bytes, then room for PEER_TABLES copies of PeerOut
constexpr int PEER_TABLE_OFFSET = 128;
constexpr int PEER_TABLE_STRIDE = 256;
constexpr int PEER_TABLES = 8;
static_assert(sizeof(PeerOut) <= PEER_TABLE_STRIDE && PEER_TABLE_OFFSET + PEER_TABLES * PEER_TABLE_STRIDE <= PEER_FLAG_BYTES, "the tables fit the flag area");
constexpr int PEER_COUNTER_WORD = 16;  // CTAs of the running kernel that have finished (marked-word exchanges)
constexpr int PEER_SEQ_WORD = 17;
constexpr int PEER_MARK_SEQ_WORD = 18;  // the same for the exchanges that travel as marked words (below)
constexpr uint32_t PEER_UNITS = 1u << 16;  // what one exchange adds to a counter; a grid has at most this many CTAs

constexpr unsigned PEER_POLL_LIMIT = 1u << 22;  // polls of about 100 ns each

// The wait for all ranks' parts of this rank's exchange number `seq`, made by one warp (lane r polls rank r's counter).
// Bounded: gives up after about half a second and records 32 + r in *status; the caller carries on with whatever is there.
__device__ __forceinline__ void peer_wait_for(const uint32_t* flags, uint32_t seq, int world, int lane, int* status) {
    if (lane < world) {
        const uint32_t target = seq * PEER_UNITS;
        bool arrived = false;
        for (unsigned poll = 0; poll < PEER_POLL_LIMIT && !arrived; poll++) {
            uint32_t seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flags + lane) : "memory");
            arrived = (int32_t)(seen - target) >= 0;
            if (!arrived && poll > 16) {
                __nanosleep(100);
            }
        }
        if (!arrived) {
            atomicCAS(status, 0, 32 + lane);
        }
    }
    __syncwarp();
}

// Every thread of every CTA of the grid calls this once, after its last store to a peer. The CTA barrier orders the
// CTA's stores before the release-ordered adds that threads 0 .. world - 1 then make, one per rank, to that rank's
// counter of this rank: a rank that sees the whole count sees every store of every CTA. CTA 0 advances this rank's
// exchange number (a plain store: the kernels behind this one in the stream read it). With `wait` CTA 0 then waits
// (bounded) until the other ranks' parts of the same exchange have arrived here, so that the kernel itself ends only
// when this rank's y is complete and no separate waiting launch is needed. `status` as for peer_wait_for.
// wrote = false: this CTA stored nothing to a peer, so its share needs no ordering and travels as a relaxed add (a release
// at system scope costs microseconds, and the releases of a grid queue up).
__device__ __forceinline__ void peer_publish(uint32_t* const* flags, int rank, int world, bool wait = false, int* status = nullptr, bool wrote = true) {
    const uint32_t G = gridDim.x * gridDim.y * gridDim.z;
    const uint32_t i = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    __syncthreads();
    if ((int)threadIdx.x < world) {
        const uint32_t share = (uint32_t)(((uint64_t)(i + 1) * PEER_UNITS) / G) - (uint32_t)(((uint64_t)i * PEER_UNITS) / G);
        if (wrote) {
            asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(flags[threadIdx.x] + rank), "r"(share) : "memory");
        } else {
            asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(flags[threadIdx.x] + rank), "r"(share) : "memory");
        }
    }
    if (i == 0 && threadIdx.x < 32) {
        uint32_t seq = 0;
        if (threadIdx.x == 0) {
            seq = flags[rank][PEER_SEQ_WORD] + 1u;  // this exchange's number
            flags[rank][PEER_SEQ_WORD] = seq;
        }
        if (wait) {
            seq = __shfl_sync(0xffffffffu, seq, 0);
            peer_wait_for(flags[rank], seq, world, (int)threadIdx.x, status);
        }
    }
}

// The wait for this rank's latest exchange, made by one warp of a kernel that consumes what the exchange delivered,
// after its griddepcontrol.wait (the kernel that made this rank's part of the exchange has then finished and advanced
// the number).
__device__ __forceinline__ void peer_wait_inline(const uint32_t* flags, int world, int lane, int* status) {
    const uint32_t seq = *reinterpret_cast<const volatile uint32_t*>(flags + PEER_SEQ_WORD);
    peer_wait_for(flags, seq, world, lane, status);
}

// ---- exchanges without a fence: marked words ---------------------------------------------------------------------------
// A system-wide release costs a thread block 2.5 to 8 microseconds on this hardware when every block of a grid makes one
// (they queue up). The outputs of a sharded linear therefore travel without any: a rank stores each value for a peer as
// one 8-byte word {value, number of the exchange} into the peer's staging area (an aligned 8-byte store arrives whole),
// and every rank's kernel, once its own rows are done, collects what the others own: it polls each staging word until it
// carries this exchange's number and writes the value into its y. No word depends on another, so nothing needs ordering;
// y is complete when the kernel ends. The numbers of the exchanges grow by one per exchange on a buffer (word 18, private
// to the rank, advanced by the CTA that finishes last), all ranks make the same exchanges in the same order, and an area is not the target
// of two exchanges in a row, so a stale word never carries the current number.

// The number of the exchange this kernel makes; to be read after griddepcontrol.wait (the kernel before has advanced it).
__device__ __forceinline__ uint32_t peer_marks_seq(const PeerOut* po) {
    return *reinterpret_cast<const volatile uint32_t*>(po->flags[po->rank] + PEER_MARK_SEQ_WORD) + 1u;
}

// One output of this rank, element idx = m n_total + col0 + row of y: into its own y, and marked into every peer's staging.
__device__ __forceinline__ void peer_store_marked(const PeerOut* po, int64_t idx, float val, uint32_t seq) {
    const unsigned long long word = ((unsigned long long)seq << 32) | (unsigned long long)__float_as_uint(val);
    for (int r = 0; r < po->world; r++) {
        if (r == po->rank) {
            po->y[r][idx] = val;
        } else {
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(po->stage[r] + idx), "l"(word) : "memory");
        }
    }
}

// Rank that owns column `col` when n columns are split evenly (the first n % world ranks get one more): used to name the
// rank whose values did not arrive.
__device__ __forceinline__ int peer_even_owner(int64_t col, int64_t n, int world) {
    const int64_t base = n / world, extra = n % world;
    const int64_t edge = extra * (base + 1);
    return col < edge ? (int)(col / (base + 1)) : (int)(extra + (base > 0 ? (col - edge) / base : 0));
}

// Every thread of every CTA calls this after its last peer_store_marked: the grid's threads share out the elements of
// y [rows_m, n_total] that other ranks own, wait (bounded by `wait_clocks` in all per thread) for each one's word and move
// the value into y. A wait that runs out records 32 + (owner under the even split) in *status; what has not arrived is
// left as it is in y.
__device__ __forceinline__ void peer_collect(const PeerOut* po, int rows_m, uint32_t seq, int* status) {
    const long long wait_clocks = po->wait_clocks;
    const int64_t G = (int64_t)gridDim.x * gridDim.y * gridDim.z;
    const int64_t i = ((int64_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    const int T = blockDim.x * blockDim.y * blockDim.z;
    const int64_t n_total = po->n_total, lo = po->col0, hi = po->col0 + po->n_own;
    const int64_t total = (int64_t)rows_m * n_total;
    const unsigned long long* stage = po->stage[po->rank];
    float* y = po->y[po->rank];
    long long t0 = 0;
    bool late = false;
    for (int64_t e = i * T + threadIdx.x; e < total; e += G * T) {
        const int64_t col = e % n_total;
        if (col >= lo && col < hi) {
            continue;
        }
        unsigned long long word;
        for (;;) {
            asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(word) : "l"(stage + e) : "memory");
            if ((uint32_t)(word >> 32) == seq || late) {
                break;
            }
            if (t0 == 0) {
                t0 = clock64();
            } else if (clock64() - t0 > wait_clocks) {
                late = true;
                atomicCAS(status, 0, 32 + peer_even_owner(col, n_total, po->world));
            }
        }
        if ((uint32_t)(word >> 32) == seq) {
            y[e] = __uint_as_float((uint32_t)word);
        }
    }
    // The CTA that finishes last advances the number: every CTA has read it by then (a relaxed counter is enough, nothing
    // is published through it).
    if (threadIdx.x == 0) {
        uint32_t* counter = po->flags[po->rank] + PEER_COUNTER_WORD;
        if (atomicAdd(counter, 1u) == (uint32_t)(G - 1)) {
            *counter = 0u;
            po->flags[po->rank][PEER_MARK_SEQ_WORD] = seq;
        }
    }
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
