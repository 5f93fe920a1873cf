// The activation image of the tcgen05 decode GEMV (jq_gemv_umma.cu): its layout and the warp-level routine that
// builds the part of one (super-block of k, row of x). Kernels that produce activations can include this to write the
// image directly instead of a float vector.
//
// Per 256-element super-block of k and row m of x the values are scaled by a power of two s (from the block's largest
// magnitude), rounded to 22-bit fixed point X = rint(x / s * 2^21) and split into three signed base-256 digits
// X = 65536 d2 + 256 d1 + d0. Digit i of row m is column 3m + i of the B operand of tcgen05.mma.kind::i8; one
// 32-element sub-block of k is the K extent of one instruction. The layout is the canonical K-major shared-memory layout
// without swizzle: 8 columns x 16 bytes of k form a 128-byte core matrix; the core matrices of a sub-block are ordered
// [k half][column group of 8]. Behind the eight sub-blocks' digits sit 9 x MPAD floats: for each sub-block the sum of its
// x values (as rounded, times the weight below), then the weight s 2^-21 of digit 0 of each row (NaN if the super-block
// of x holds a value that is not finite, which makes every output NaN, as a product with NaN or Inf is in the reference
// unless Inf meets only weights of one sign).
#pragma once

#include "jq_common.cuh"

namespace jq {
namespace umma {

// N = MMA columns: 8, 16, 32 or 48 hold up to 2, 5, 10, 16 rows of x.
template <int N>
struct ImageCfg {
    static_assert(N == 8 || N == 16 || N == 32 || N == 48, "column counts of the decode GEMV");
    static constexpr int MAX_ROWS = N == 8 ? 2 : (N == 16 ? 5 : (N == 32 ? 10 : 16));
    static constexpr int MPAD = N == 8 ? 4 : (N == 16 ? 8 : (N == 32 ? 12 : 16));  // floats per aux row (16-byte multiples)
    static constexpr int SUB_BYTES = N * 32;                 // digits of one sub-block: N columns x 32 bytes of k
    static constexpr int KHALF_BYTES = (N / 8) * 128;        // distance between the two 16-byte halves of k (leading byte offset)
    static constexpr int XD = 8 * SUB_BYTES;
    static constexpr int AUX = 9 * MPAD * 4;
    static constexpr int BYTES = XD + AUX;                   // per super-block, a multiple of 16
    static_assert(BYTES % 16 == 0, "the image is copied in 16-byte pieces");
};

__host__ __device__ constexpr int columns_for_rows(int rows) { return rows <= 2 ? 8 : (rows <= 5 ? 16 : (rows <= 10 ? 32 : 48)); }
__host__ __device__ constexpr size_t image_block_bytes(int n_cols) {
    return n_cols == 8 ? ImageCfg<8>::BYTES : (n_cols == 16 ? ImageCfg<16>::BYTES : (n_cols == 32 ? ImageCfg<32>::BYTES : ImageCfg<48>::BYTES));
}

// One warp turns the 256 values at xb (super-block b of row m of x) into its part of the image block `img` (global or
// shared memory). lane = 4 sub + tt: elements 8 tt .. 8 tt + 7 of sub-block `sub`. The warp of row 0 also clears the
// columns and aux entries of rows >= rows, so a block is complete once the warps of rows 0 .. rows - 1 have run.
// This lane's eight values of the super-block at xb.
__device__ __forceinline__ void load_lane_values(const float* xb, int lane, float4& lo, float4& hi) {
    const float4* xp = reinterpret_cast<const float4*>(xb) + 2 * lane;
    lo = xp[0];
    hi = xp[1];
}

template <int N>
__device__ __forceinline__ void build_image_from(const float4& lo, const float4& hi, int m, int rows, uint8_t* img, int lane) {
    using C = ImageCfg<N>;
    const int sub = lane >> 2, tt = lane & 3;
    float* aux = reinterpret_cast<float*>(img + C::XD);
    const float xv[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    float am = 0.0f;
    bool bad = false;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        am = fmaxf(am, fabsf(xv[i]));
        bad = bad || (__float_as_uint(xv[i]) & 0x7f800000u) == 0x7f800000u;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    }
    bad = __any_sync(0xffffffffu, bad);
    // s = 2^floor(log2(amax)): the largest |x| / s of the super-block lies in [1, 2)
    uint32_t e = __float_as_uint(am) & 0x7f800000u;
    e = e < 0x0d000000u ? 0x0d000000u : (e > 0x7e800000u ? 0x7e800000u : e);  // keeps 2^21 / s and s 2^-21 normal
    const float inv = __uint_as_float(0x7f000000u - e + (21u << 23));            // 2^21 / s: |X| <= 2^22
    const float wgt = bad ? __uint_as_float(0x7fc00000u) : __uint_as_float(e - (21u << 23));  // s 2^-21
    int X[8];
    int total = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        X[i] = __float2int_rn(xv[i] * inv);
        total += X[i];
    }
    uint8_t* cell = img + sub * C::SUB_BYTES + (tt >> 1) * C::KHALF_BYTES + (tt & 1) * 8;
#pragma unroll
    for (int dgt = 0; dgt < 3; dgt++) {
        uint32_t w0 = 0, w1 = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int d = dgt == 2 ? X[i] : (int)(int8_t)(X[i] & 0xff);  // signed low byte
            X[i] = (X[i] - d) >> 8;
            if (i < 4) {
                w0 |= (uint32_t)(d & 0xff) << (8 * i);
            } else {
                w1 |= (uint32_t)(d & 0xff) << (8 * (i - 4));
            }
        }
        const int col = 3 * m + dgt;
        *reinterpret_cast<uint2*>(cell + (col >> 3) * 128 + (col & 7) * 16) = make_uint2(w0, w1);
    }
    // the sub-block's sum of X (its four octets sit in four consecutive lanes); |sum| <= 2^27, the float keeps 24 bits of it
    total += __shfl_xor_sync(0xffffffffu, total, 1);
    total += __shfl_xor_sync(0xffffffffu, total, 2);
    if (tt == 0) {
        aux[sub * C::MPAD + m] = (float)total * wgt;
    }
    if (lane == 0) {
        aux[8 * C::MPAD + m] = wgt;
    }
    if (m == 0) {
        for (int col = 3 * rows; col < N; col++) {
            *reinterpret_cast<uint2*>(cell + (col >> 3) * 128 + (col & 7) * 16) = make_uint2(0u, 0u);
        }
        for (int i = lane; i < 9 * C::MPAD; i += 32) {
            if (i % C::MPAD >= rows) {
                aux[i] = 0.0f;
            }
        }
    }
}

template <int N>
__device__ __forceinline__ void build_image(const float* xb, int m, int rows, uint8_t* img, int lane) {
    float4 lo, hi;
    load_lane_values(xb, lane, lo, hi);
    build_image_from<N>(lo, hi, m, rows, img, lane);
}

}  // namespace umma
}  // namespace jq
