// The activation image of the tcgen05 decode GEMV (jq_gemv_umma.cu): its layout and the warp-level routine that
// builds the part of one (super-block of k, row of x). Kernels that produce activations can include this to write the
// image directly instead of a float vector.
//
// Per 256-element super-block of k and row m of x the values are scaled by a power of two s (from the block's largest
// magnitude), rounded to 22-bit fixed point X = rint(x / s * 2^21) and split into two signed digits of 11 bits,
// X = 2048 Xh + Xl with -1024 <= Xl < 1024 and |Xh| <= 2048: both are integers that half precision holds exactly. Xh is
// column 2m and Xl column 2m + 1 of the B operand of tcgen05.mma.kind::f16; 16 elements of k are the K extent of one
// instruction, so a super-block is 16 instructions. The layout is the canonical K-major shared-memory layout without
// swizzle: 8 columns x 16 bytes (8 values of k) form a 128-byte core matrix; the core matrices of a step are ordered
// [k half][column group of 8]. Behind the sixteen steps sit 9 x MPAD floats: for each 32-element sub-block the sum of its
// x values (as rounded, times the weight below), then the weight s 2^-21 of the low digit of each row (NaN if the
// super-block of x holds a value that is not finite, which makes every output NaN, as a product with NaN or Inf is in the
// reference unless Inf meets only weights of one sign).
#pragma once

#include <cuda_fp16.h>

#include "jq_common.cuh"

namespace jq {
namespace umma {

// N = MMA columns: 16 or 32 hold up to 8 or 16 rows of x (an MMA of 128 rows takes multiples of 16 columns).
template <int N>
struct ImageCfg {
    static_assert(N == 16 || N == 32, "column counts of the decode GEMV");
    static constexpr int MAX_ROWS = N / 2;
    static constexpr int MPAD = N / 2;                       // floats per aux row (16-byte multiples)
    static constexpr int STEPS = 16;                         // MMA instructions per super-block
    static constexpr int SUB_BYTES = N * 32;                 // one step: N columns x 16 values of k x 2 bytes
    static constexpr int KHALF_BYTES = (N / 8) * 128;        // distance between the two 8-value halves of a step's k (leading byte offset)
    static constexpr int XD = STEPS * SUB_BYTES;
    static constexpr int AUX = 9 * MPAD * 4;
    static constexpr int BYTES = XD + AUX;                   // per super-block, a multiple of 16
    static_assert(BYTES % 16 == 0, "the image is copied in 16-byte pieces");
};

__host__ __device__ constexpr int columns_for_rows(int rows) { return rows <= 8 ? 16 : 32; }
__host__ __device__ constexpr size_t image_block_bytes(int n_cols) {
    return n_cols == 16 ? ImageCfg<16>::BYTES : ImageCfg<32>::BYTES;
}

// This lane's eight values of the super-block at xb: lane = 4 sub + tt holds elements 8 tt .. 8 tt + 7 of sub-block `sub`.
__device__ __forceinline__ void load_lane_values(const float* xb, int lane, float4& lo, float4& hi) {
    const float4* xp = reinterpret_cast<const float4*>(xb) + 2 * lane;
    lo = xp[0];
    hi = xp[1];
}

// One warp turns the 256 values of super-block b of row m of x (lane's values in lo, hi) into its part of the image block
// `img` (global or shared memory). The warp of row 0 also clears the columns and aux entries of rows >= rows, so a block is
// complete once the warps of rows 0 .. rows - 1 have run.
template <int N>
__device__ __forceinline__ void build_image_from(const float4& lo, const float4& hi, int m, int rows, uint8_t* img, int lane) {
    using C = ImageCfg<N>;
    const int sub = lane >> 2, tt = lane & 3;
    float* aux = reinterpret_cast<float*>(img + C::XD);
    const float xv[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    // largest magnitude as an integer (NaN > Inf > every finite value in this order)
    uint32_t amb = 0u;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        amb = max(amb, __float_as_uint(xv[i]) & 0x7fffffffu);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amb = max(amb, __shfl_xor_sync(0xffffffffu, amb, o));
    }
    const bool bad = amb >= 0x7f800000u;
    // s = 2^floor(log2(amax)): the largest |x| / s of the super-block lies in [1, 2)
    uint32_t e = amb & 0x7f800000u;
    e = e < 0x0d000000u ? 0x0d000000u : (e > 0x7e800000u ? 0x7e800000u : e);  // keeps 2^21 / s and s 2^-21 normal
    const float inv = __uint_as_float(0x7f000000u - e + (21u << 23));            // 2^21 / s: |X| <= 2^22
    const float wgt = bad ? __uint_as_float(0x7fc00000u) : __uint_as_float(e - (21u << 23));  // s 2^-21
    int total = 0;
    uint32_t hw[4], lw[4];  // the eight high digits and the eight low digits as half pairs
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int Xa = __float2int_rn(xv[2 * i] * inv), Xb = __float2int_rn(xv[2 * i + 1] * inv);
        if (bad) {
            Xa = Xb = 0;  // what the digits are does not matter (the weights are NaN), but they must be numbers
        }
        total += Xa + Xb;
        const int ha = (Xa + 1024) >> 11, hb = (Xb + 1024) >> 11;
        const int la = Xa - (ha << 11), lb = Xb - (hb << 11);
        const __half2 hp = __halves2half2(__int2half_rn(ha), __int2half_rn(hb));
        const __half2 lp = __halves2half2(__int2half_rn(la), __int2half_rn(lb));
        hw[i] = *reinterpret_cast<const uint32_t*>(&hp);
        lw[i] = *reinterpret_cast<const uint32_t*>(&lp);
    }
    // the lane's eight values are one 16-byte row of a core matrix: step 2 sub + tt / 2, k half tt % 2
    uint8_t* cell = img + (2 * sub + (tt >> 1)) * C::SUB_BYTES + (tt & 1) * C::KHALF_BYTES;
    {
        const int ch = 2 * m, cl = 2 * m + 1;
        *reinterpret_cast<uint4*>(cell + (ch >> 3) * 128 + (ch & 7) * 16) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
        *reinterpret_cast<uint4*>(cell + (cl >> 3) * 128 + (cl & 7) * 16) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
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
        for (int col = 2 * rows; col < N; col++) {
            *reinterpret_cast<uint4*>(cell + (col >> 3) * 128 + (col & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
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
