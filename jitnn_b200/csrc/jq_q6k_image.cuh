// The activation image of the Q6_K integer GEMV (jq_gemv_q6k_i8.cu): its layout and the warp-level routine that
// builds one (super-block, row of x) part of it. Kernels that produce activations include this to write the image
// directly instead of a float vector.
#pragma once

#include "jq_common.cuh"

namespace jq {
namespace q6k {

template <int MT>
struct Cfg {
    static constexpr int COLS = 3 * MT;               // digit columns: column 3m + i is digit i of activation row m
    static constexpr int NG = (COLS + 7) / 8;         // MMA column groups
    static constexpr int NCOL = NG == 1 ? COLS : 8;   // columns stored per group
    // bytes of activation image per super-block: digit fragments of the 16 scale groups, C fragments, column weights.
    // Fragments of several groups sit side by side so that the GEMV reads them with 16-byte loads:
    //   XD  [group / 4][column group][column][lane][group % 4]   4 bytes each: a lane's B operands of four groups
    //   XC  [group / 2][column group][lane][group % 2][2 columns] int32:      a lane's C operands of two groups
    static constexpr size_t XD = (size_t)16 * NG * NCOL * 4 * 4;
    static constexpr size_t XC = (size_t)16 * NG * 8 * 4;
    static constexpr size_t TAB = (size_t)NG * 8 * 4;             // one float per digit column
    static constexpr size_t PB = XD + XC + TAB;
};

// One warp turns the 256 values at xb (one super-block of k of row m of x; nullptr: a row beyond those of x, all zero)
// into its part of the super-block's image at `img` (global or shared memory).
// Lane L holds the 8 activations 8L .. 8L+7: they are k-slots 8 (L % 2) .. + 7 of scale group L / 2 (a group = 16
// consecutive elements of the super-block).
template <int MT>
__device__ __forceinline__ void build_image(const float* xb, int m, uint8_t* img, int lane) {
    using C = Cfg<MT>;
    constexpr int NG = C::NG, NCOL = C::NCOL;
    const int grp = lane >> 1, half = lane & 1;
    uint32_t* xd = reinterpret_cast<uint32_t*>(img);
    int* xc = reinterpret_cast<int*>(img + C::XD);
    float* tab = reinterpret_cast<float*>(img + C::XD + C::XC);
    if (m == 0 && lane >= C::COLS && lane < NG * 8) {
        tab[lane] = 0.0f;  // columns that hold no activation row
    }
    float xv[8];
    if (xb != nullptr) {
        const float4* xp = reinterpret_cast<const float4*>(xb) + 2 * lane;
        const float4 lo = xp[0], hi = xp[1];
        xv[0] = lo.x; xv[1] = lo.y; xv[2] = lo.z; xv[3] = lo.w;
        xv[4] = hi.x; xv[5] = hi.y; xv[6] = hi.z; xv[7] = hi.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            xv[i] = 0.0f;
        }
    }
    float am = 0.0f;
    bool bad = false;  // a NaN or an Inf among the values: the column weights become NaN and with them every output of this row of x
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
    e = e < 0x0c000000u ? 0x0c000000u : (e > 0x7e800000u ? 0x7e800000u : e);  // keeps 2^21 / s and s * 2^-21 normal
    const float inv = __uint_as_float(0x7f000000u - e + (21u << 23));           // 2^21 / s: |X| <= 2^22
    int X[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        X[i] = __float2int_rn(xv[i] * inv);
    }
#pragma unroll
    for (int dgt = 0; dgt < 3; dgt++) {
        uint32_t w0 = 0, w1 = 0;
        int sum = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int d = dgt == 2 ? X[i] : (int)(int8_t)(X[i] & 0xff);  // signed low byte
            X[i] = (X[i] - d) >> 8;
            sum += d;
            if (i < 4) {
                w0 |= (uint32_t)(d & 0xff) << (8 * i);
            } else {
                w1 |= (uint32_t)(d & 0xff) << (8 * (i - 4));
            }
        }
        const int col = 3 * m + dgt;
        // lane slots 2 half and 2 half + 1 of this group's B fragment
        uint32_t* cell = xd + ((((size_t)(grp >> 2) * NG + (col >> 3)) * NCOL + (col & 7)) * 16) + (grp & 3);
        cell[(2 * half) * 4] = w0;
        cell[(2 * half + 1) * 4] = w1;
        // -32 * (digit sum of the group's 16 elements): the row-independent part of sum (q - 32) x, the MMA's C operand
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        if (half == 0) {
            xc[((((size_t)(grp >> 1) * NG + (col >> 3)) * 4 + ((col & 7) >> 1)) * 2 + (grp & 1)) * 2 + (col & 1)] = -32 * sum;
        }
        if (lane == 0) {
            tab[col] = xb == nullptr ? 0.0f : (bad ? __uint_as_float(0x7fc00000u) : __uint_as_float(e + ((uint32_t)(8 * dgt) << 23) - (21u << 23)));  // s * 2^(8 dgt - 21)
        }
    }
}

}  // namespace q6k
}  // namespace jq
