// Shared declarations of the library: error reporting, the weight handle, launch bookkeeping.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "../../include/jitnn_b200.h"

namespace jq {

// ---- error reporting (thread-local message behind jq_last_error) ------------------------------
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define JQ_CUDA(call)                                   \
    do {                                                \
        cudaError_t e_ = (call);                        \
        if (e_ != cudaSuccess) {                        \
            return ::jq::cuda_fail(e_, #call);          \
        }                                               \
    } while (0)

extern std::atomic<int64_t> g_launches;
inline void count_launch(int n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// Checks the launch that was just issued.
int check_launch(const char* kernel);

// ---- block geometry (DType.java:75-98 of the reference) ---------------------------------------
inline int block_values(int type) {
    switch (type) {
        case JQ_TYPE_Q8_0: case JQ_TYPE_Q4_0: case JQ_TYPE_Q4_1: case JQ_TYPE_Q5_0: case JQ_TYPE_Q5_1: return 32;
        case JQ_TYPE_Q4_K: case JQ_TYPE_Q5_K: case JQ_TYPE_Q6_K: case JQ_TYPE_Q2_K: case JQ_TYPE_Q3_K: return 256;
        default: return 0;
    }
}

inline int block_bytes(int type) {
    switch (type) {
        case JQ_TYPE_Q8_0: return 34;
        case JQ_TYPE_Q4_0: return 18;
        case JQ_TYPE_Q4_1: return 20;
        case JQ_TYPE_Q4_K: return 144;
        case JQ_TYPE_Q5_K: return 176;
        case JQ_TYPE_Q6_K: return 210;
        case JQ_TYPE_Q5_0: return 22;
        case JQ_TYPE_Q5_1: return 24;
        case JQ_TYPE_Q2_K: return 84;
        case JQ_TYPE_Q3_K: return 110;
        default: return 0;
    }
}

// Bytes per block of the quant plane and of the scale plane in the device layout. Formats whose
// blocks are 16-byte multiples (Q4_K, Q5_K) and the dequantise-only formats stay verbatim (aux = 0).
inline int plane_q_bytes(int type) {
    switch (type) {
        case JQ_TYPE_Q8_0: return 32;
        case JQ_TYPE_Q4_0: return 16;
        case JQ_TYPE_Q4_1: return 16;
        case JQ_TYPE_Q6_K: return 208;
        default: return block_bytes(type);
    }
}

inline int plane_aux_bytes(int type) {
    switch (type) {
        case JQ_TYPE_Q8_0: return 2;
        case JQ_TYPE_Q4_0: return 2;
        case JQ_TYPE_Q4_1: return 4;
        case JQ_TYPE_Q6_K: return 2;
        default: return 0;
    }
}

// Q4_K and Q5_K weights are stored tile by tile: 128 consecutive rows form a tile, and within a tile the blocks of one
// 256-element super-block of k lie together, row after row: [tile][super-block b][row in tile][block bytes]. One
// (tile, super-block) unit is then a single contiguous run of 128 x block bytes, which the copy engine moves with one bulk copy.
// The last tile is padded with zero rows. No byte of a block changes; jq_weight_download restores GGUF's order.
constexpr int TILE_ROWS = 128;
__host__ __device__ inline bool tiled_layout(int type) { return type == JQ_TYPE_Q4_K || type == JQ_TYPE_Q5_K; }
// Q6_K keeps its two planes (208 bytes of quants and scales, one fp16 d per block) and orders the blocks of each plane the
// same way, so that 16 rows x one super-block are 3328 contiguous bytes of the quant plane and 32 of the d plane.
__host__ __device__ inline bool tiled_planes(int type) { return type == JQ_TYPE_Q6_K; }
__host__ __device__ inline int64_t tiled_rows(int64_t n) { return (n + TILE_ROWS - 1) / TILE_ROWS * TILE_ROWS; }
// Position of block b of `row` among the blocks of a tiled plane with kb blocks per row.
__host__ __device__ inline int64_t tiled_index(int64_t row, int64_t b, int64_t kb) {
    return ((row >> 7) * kb + b) * TILE_ROWS + (row & (TILE_ROWS - 1));
}
// Byte offset of block b of `row` in a tiled weight with kb blocks of `bytes` bytes per row.
__host__ __device__ inline int64_t tiled_offset(int64_t row, int64_t b, int64_t kb, int bytes) {
    return ((row >> 7) * kb + b) * (int64_t)(TILE_ROWS * bytes) + (row & (TILE_ROWS - 1)) * bytes;
}

inline bool has_linear_kernel(int type) {
    return type == JQ_TYPE_Q8_0 || type == JQ_TYPE_Q4_0 || type == JQ_TYPE_Q4_1 || type == JQ_TYPE_Q4_K ||
           type == JQ_TYPE_Q5_K || type == JQ_TYPE_Q6_K;
}

// What the kernels see of a weight.
struct View {
    const uint8_t* q;    // quant plane, tiled blocks (Q4_K, Q5_K) or verbatim blocks, 256-byte aligned
    const uint8_t* aux;  // scale plane, or nullptr
    int64_t n;           // output rows
    int64_t k;           // input features
    int type;
};

// ---- kernel launchers (one translation unit each) ----------------------------------------------
// kb: blocks per row; the planes of a type with tiled_planes() hold their blocks in tiled order (tiled_rows(n) rows).
int launch_repack(int type, const uint8_t* verbatim, uint8_t* q, uint8_t* aux, int64_t blocks, int64_t kb, cudaStream_t s);
int launch_unpack(int type, const uint8_t* q, const uint8_t* aux, uint8_t* verbatim, int64_t blocks, int64_t kb, cudaStream_t s);
// Verbatim blocks [n, kb] <-> the tiled layout of Q4_K and Q5_K (`tiled` holds tiled_rows(n) rows).
int launch_tile(int type, const uint8_t* verbatim, uint8_t* tiled, int64_t n, int64_t kb, bool inverse, cudaStream_t s);
int launch_dequantize(const View& v, float* dst, cudaStream_t s);
// x_remote: x lies in host memory that the GPU reads across PCIe; kernels then read it once instead of once per thread block.
int launch_gemv(const View& v, const float* x, int rows, const float* bias, float* y, cudaStream_t s, bool x_remote = false);
// gx [m, k] = g [m, n] . dequant(W) (jq_backward.cu).
int launch_linear_backward(const View& v, const float* g, int64_t m, float* gx, cudaStream_t s);
int launch_quantize_q8_0(const float* x, int64_t blocks, uint8_t* out, cudaStream_t s);
// Where a GEMV's outputs go besides (or instead of) y when the linear is sharded by rows over several GPUs: every
// rank's copy of the full output and flag words (jq_peer.cu). world = 0: no peers.
struct PeerOut {
    float* y[8];         // every rank's y [m, n_total] (this rank's included)
    uint32_t* flags[8];  // every rank's flag words
    unsigned long long* stage[8];  // every rank's staging words [m, n_total] (value and exchange number in one 8-byte word), or null:
                                   // the outputs then go straight into y and the exchange is announced through the arrival counters
    int world, rank;
    int64_t n_total, col0;  // this rank's rows are columns col0 .. of y
    int64_t n_own;          // how many of them: rows of this rank's shard
    const PeerOut* table;   // host side only: where a copy of this struct lives in device memory
    int wait_first;         // the kernel's input is what this rank's latest exchange delivered: wait for all ranks' parts before reading it
    int wait_after;         // the kernel ends only when all ranks' parts of its own exchange have arrived in this rank's y (bounded wait by one CTA)
    long long wait_clocks;  // clocks a thread waits in all for the other ranks' marked words
};
// Integer tensor-core GEMV (mma.sync) for Q4_K and Q5_K, rows <= 8 (jq_gemv_q4k_i8.cu); *handled = false leaves the call to
// another kernel. `image` is scratch of gemv_q4k_i8_scratch_bytes(k, rows) bytes.
int launch_gemv_q4k_i8(const View& v, const float* x, int rows, const float* bias, float* y, cudaStream_t s, uint8_t* image, bool* handled,
                       const PeerOut* peer = nullptr, bool x_remote = false);
size_t gemv_q4k_i8_scratch_bytes(int64_t k, int rows);
int launch_gemv_q4k_i8_multi(const View* vs, int count, const float* x, int rows, float* const* ys, cudaStream_t s, uint8_t* image, bool* handled);
// The same for one row of x whose activation image (jq_q4k_image.cuh) a kernel earlier in the stream has already written; a
// second Q4_K weight with the same k can ride in the same launch.
size_t q4k_image_bytes_one_row(int64_t k);
int launch_gemv_q4k_i8_imaged(const View& v, const View* v2, const uint8_t* image, const float* bias, float* y, float* y2, cudaStream_t s, bool* handled,
                              const PeerOut* peer = nullptr, const View* v3 = nullptr, float* y3 = nullptr);
// Status word of the waits a GEMV makes itself for a peer exchange (peer_wait_inline): 0 or 32 + rank, cleared by the call.
int gemv_peer_status(int* status);
int gemv_q6k_status(int* status);  // the same for the Q6_K kernel's weight-ring waits (0 or 25)
// Pieces of the peer exchange (jq_peer.cu) for the row-sharded decoder: the bounded wait for all ranks' flags of this
// rank's latest exchange, and a Q4_K row shard applied to an activation image that is already complete, its outputs
// stored into every rank's y [1, n_total] at payload_offset, followed by that wait.
// staging_offset >= 0: the outputs travel as marked words through that area of the payload and the kernel ends when this
// rank's y is complete (wait_after is then moot); < 0: straight into every rank's y, announced through the arrival counters.
int peer_linear_q4k_imaged(const jq_weight* w, const uint8_t* image, int64_t n_total, int64_t col0, void* const* peer_buffers, int64_t payload_offset,
                           int64_t staging_offset, int rank, int world, cudaStream_t s, bool wait_first, bool wait_after);
// Status word of the waits that the decoder's kernels make themselves (peer_wait_inline): 0 or 32 + rank, cleared by the call.
int decoder_peer_status(int* status);
// Q6_K for one row of x whose activation image (jq_q6k_image.cuh) a kernel earlier in the stream has written.
size_t q6k_image_bytes_one_row(int64_t k);
int launch_gemv_q6k_i8_imaged(const View& v, const uint8_t* image, const float* bias, float* y, cudaStream_t s, bool* handled);
// The same for Q6_K, rows <= 4.
int launch_gemv_q6k_i8(const View& v, const float* x, int rows, const float* bias, float* y, cudaStream_t s, uint8_t* image, bool* handled);
size_t gemv_q6k_i8_scratch_bytes(int64_t k, int rows);
// The same for Q8_0, Q4_0 and Q4_1 (jq_gemv_blk32_i8.cu): rows <= 2, k a multiple of 256.
int launch_gemv_blk32_i8(const View& v, const float* x, int rows, const float* bias, float* y, cudaStream_t s, uint8_t* image, bool* handled);
size_t gemv_blk32_i8_scratch_bytes(int type, int64_t k, int rows);

// Scratch memory of at least `bytes` on the current device, private to work enqueued on `s` (one buffer per
// device and stream, grown on demand and kept until the library is unloaded).
int scratch_for(cudaStream_t s, size_t bytes, uint8_t** out);
// A second, third ... scratch buffer of the same (device, stream), for a caller that needs one while a kernel launcher uses slot 0.
int scratch_for_slot(cudaStream_t s, int slot, size_t bytes, uint8_t** out);

// The same for words that kernels use as counters and leave at zero: a new allocation starts out zeroed (in stream order).
int scratch_zeroed_for_slot(cudaStream_t s, int slot, size_t bytes, uint8_t** out);

// Decode GEMV on tcgen05 (jq_gemv_umma.cu): Q4_K and Q5_K, 1 to 16 rows of x in one pass over the weights.
bool gemv_umma_takes(int type, int64_t k, int rows, int64_t n = 0);
bool gemv_umma_fallback(int type, int64_t k, int rows);  // may stand in for the mma.sync kernel on a shape that one declines
size_t gemv_umma_image_bytes(int64_t k, int rows);
inline size_t gemv_umma_image_bytes_one_row(int64_t k) { return gemv_umma_image_bytes(k, 1); }
int launch_gemv_umma_image(const float* x, int rows, int64_t k, uint8_t* image, cudaStream_t s);
int launch_gemv_umma(const View& v, const View* v2, const float* x, uint8_t* image, int rows, const float* bias, float* y, float* y2, cudaStream_t s,
                     const PeerOut* peer = nullptr, bool no_scratch = false);
int launch_gemv_umma_multi(const View* vs, int count, const float* x, uint8_t* image, int rows, const float* bias, float* const* ys, cudaStream_t s,
                           const PeerOut* peer = nullptr, bool no_scratch = false);
int gemv_umma_status(int* status);
// Option "gemv_tcgen05": 1 sends Q4_K and Q5_K decode (1 to 16 rows) to the tcgen05 kernel instead of the mma.sync one, 2 never,
// 0 where it is faster (many rows of x, many rows of the weight).
extern std::atomic<int64_t> g_opt_gemv_umma;
// Option "wait_limit_us": microseconds after which a bounded device-side wait of the tcgen05 GEMV gives up.
extern std::atomic<int64_t> g_opt_wait_limit_us;
extern std::atomic<int64_t> g_opt_peer_wait_us;  // microseconds a thread waits in all for the other ranks' values of a sharded linear

// Rows of zero padding behind every uploaded weight plane: kernels that work on 16-row tiles read past n.
constexpr int PAD_ROWS = 16;

// Tensor-core prefill (jq_prefill.cu).
bool prefill_supported(const View& v);
int launch_prefill_bf16(const View& v, const uint16_t* x_bf16, int64_t m, const float* bias, float* y, cudaStream_t s);
int launch_f32_to_bf16(const float* x, uint16_t* out, int64_t count, cudaStream_t s);
int prefill_status(int* status);
// Same for the bounded waits of the peer gather (jq_peer.cu): 0, or 32 + the rank whose slice did not arrive.
int peer_status(int* status);

// Option "gemv_generic": non-zero routes every GEMV to the generic CUDA-core kernel (for comparisons).
extern std::atomic<int64_t> g_opt_gemv_generic;
// Option "decoder_graph": zero keeps the decoder's single-token step on eager launches (for comparisons).
extern std::atomic<int64_t> g_opt_decoder_graph;
// Option "decoder_fused": zero keeps the decoder's single-token step on the general kernels (one per operator).
extern std::atomic<int64_t> g_opt_decoder_fused;

}  // namespace jq

// The opaque handle of the C ABI.
struct jq_weight {
    uint32_t magic;
    int device;
    int type;
    int layout;
    int64_t n;
    int64_t k;
    uint8_t* q;
    uint8_t* aux;
    int64_t q_bytes;
    int64_t aux_bytes;
};

#define JQ_WEIGHT_MAGIC 0x4a515754u
