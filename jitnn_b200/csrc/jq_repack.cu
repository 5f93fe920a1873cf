// Load-time repacking between GGUF's verbatim blocks and the device layouts (planes, tiles).
//
// Q8_0 (34 B), Q4_0 (18 B), Q4_1 (20 B) and Q6_K (210 B) blocks are only 2-byte aligned, which rules
// out 128-bit loads. At upload their blocks are split into a plane of quants whose per-block size is a
// multiple of 16 bytes and a plane of fp16 scales; jq_weight_download runs the inverse. No value is
// changed: every byte of a block lands in exactly one plane.
#include "jq_common.cuh"

namespace jq {

// Byte offsets inside a verbatim block: [aux_off, aux_off + aux_bytes) goes to the scale plane, the
// remaining q_bytes (starting at q_off) to the quant plane.
struct Split {
    int block, q_off, q_bytes, aux_off, aux_bytes;
};

static Split split_of(int type) {
    switch (type) {
        case JQ_TYPE_Q8_0: return {34, 2, 32, 0, 2};
        case JQ_TYPE_Q4_0: return {18, 2, 16, 0, 2};
        case JQ_TYPE_Q4_1: return {20, 4, 16, 0, 4};
        case JQ_TYPE_Q6_K: return {210, 0, 208, 208, 2};
        default: return {0, 0, 0, 0, 0};
    }
}

// One thread per 2 bytes of a block (every block size and field offset here is even).
__global__ void repack_kernel(Split sp, const uint16_t* __restrict__ src, uint16_t* __restrict__ q, uint16_t* __restrict__ aux,
                              int64_t blocks, int64_t kb, bool tiled, bool inverse) {
    int64_t halves_per_block = sp.block / 2;
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= blocks * halves_per_block) {
        return;
    }
    int64_t b = i / halves_per_block;
    int off = (int)(i % halves_per_block) * 2;
    if (tiled) {
        b = tiled_index(b / kb, b % kb, kb);  // where the block sits in the planes
    }
    uint16_t* verbatim = const_cast<uint16_t*>(src) + i;
    uint16_t* plane;
    if (off >= sp.aux_off && off < sp.aux_off + sp.aux_bytes) {
        plane = aux + (b * sp.aux_bytes + (off - sp.aux_off)) / 2;
    } else {
        plane = q + (b * sp.q_bytes + (off - sp.q_off)) / 2;
    }
    if (inverse) {
        *verbatim = *plane;
    } else {
        *plane = *verbatim;
    }
}

int launch_repack(int type, const uint8_t* verbatim, uint8_t* q, uint8_t* aux, int64_t blocks, int64_t kb, cudaStream_t s) {
    Split sp = split_of(type);
    if (sp.block == 0) {
        return fail(JQ_ERR_INVALID, "repack: type %d has no plane layout", type);
    }
    int64_t total = blocks * (sp.block / 2);
    if (total == 0) {
        return JQ_OK;
    }
    repack_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(sp, (const uint16_t*)verbatim, (uint16_t*)q, (uint16_t*)aux, blocks, kb, tiled_planes(type), false);
    count_launch();
    return check_launch("repack_kernel");
}

int launch_unpack(int type, const uint8_t* q, const uint8_t* aux, uint8_t* verbatim, int64_t blocks, int64_t kb, cudaStream_t s) {
    Split sp = split_of(type);
    if (sp.block == 0) {
        return fail(JQ_ERR_INVALID, "unpack: type %d has no plane layout", type);
    }
    int64_t total = blocks * (sp.block / 2);
    if (total == 0) {
        return JQ_OK;
    }
    repack_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(sp, (const uint16_t*)verbatim, (uint16_t*)q, (uint16_t*)aux, blocks, kb, tiled_planes(type), true);
    count_launch();
    return check_launch("repack_kernel");
}

// One thread per 16-byte piece of a block: GGUF's order (row after row) <-> the tiled order.
__global__ void tile_kernel(const uint4* __restrict__ verbatim, uint4* __restrict__ tiled, int64_t n, int64_t kb, int pieces, bool inverse) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * kb * pieces) {
        return;
    }
    const int64_t block = i / pieces, row = block / kb, b = block % kb;
    const int piece = (int)(i % pieces);
    uint4* t = tiled + tiled_offset(row, b, kb, pieces * 16) / 16 + piece;
    uint4* v = const_cast<uint4*>(verbatim) + i;
    if (inverse) {
        *v = *t;
    } else {
        *t = *v;
    }
}

int launch_tile(int type, const uint8_t* verbatim, uint8_t* tiled, int64_t n, int64_t kb, bool inverse, cudaStream_t s) {
    if (!tiled_layout(type)) {
        return fail(JQ_ERR_INVALID, "tile: type %d has no tiled layout", type);
    }
    const int pieces = block_bytes(type) / 16;
    const int64_t total = n * kb * pieces;
    if (total == 0) {
        return JQ_OK;
    }
    tile_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>((const uint4*)verbatim, (uint4*)tiled, n, kb, pieces, inverse);
    count_launch();
    return check_launch("tile_kernel");
}

}  // namespace jq
