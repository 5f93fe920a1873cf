// The activation image of the Q4_K integer GEMV (jq_gemv_q4k_i8.cu): its layout and the warp-level routine that
// builds one (super-block, row of x) part of it. Kernels that produce activations (the decoder's norm, attention
// and SwiGLU kernels) include this to write the image directly instead of a float vector.
#pragma once

#include "jq_common.cuh"

namespace jq {
namespace q4k {

// Column layouts of the activation image. Up to two activation rows are "packed": one MMA column group holds column
// 3m + i for digit i of row m. More rows are "digit major": group i holds digit i, column m of it row m, so that a
// lane's accumulator columns 2t and 2t + 1 are all three digits of rows 2t and 2t + 1 and need no exchange with
// other lanes.
template <int MT>
struct Cfg {
    static constexpr bool DIGIT_MAJOR = MT > 2;
    static constexpr int COLS = 3 * MT;
    static constexpr int NG = DIGIT_MAJOR ? 3 : 1;                         // MMA column groups for the quants
    static constexpr int NCOL = DIGIT_MAJOR ? 8 : COLS;                    // columns stored per group
    // mins: two columns (low 7 bits / rest of the digit sums) per digit column. Packed: column 2 (3m + i) + part.
    // Digit major: group 2i + (m & 1), column 2 (m / 2) + part, which hands lane t the rows 2t and 2t + 1 again.
    static constexpr int NGM = DIGIT_MAJOR ? 6 : (2 * COLS + 7) / 8;
    static constexpr int NCOLM = NGM == 1 ? 2 * COLS : 8;
    // bytes of activation image per super-block: digit fragments, digit-sum fragments, column weights
    static constexpr size_t XD = (size_t)8 * NG * NCOL * 4 * 8;   // 8 sub-blocks x groups x columns x 4 lanes x 8 bytes
    static constexpr size_t XM = (size_t)NGM * NCOLM * 4 * 4;     // groups x columns x 4 lanes x 4 bytes (lanes 2, 3: zero)
    // one float per digit column: its weight s 2^(8 i - 21); packed layouts add a second table with the weights / 16
    static constexpr size_t TAB = (size_t)NG * 8 * 4 * (DIGIT_MAJOR ? 1 : 2);
    static constexpr size_t PB = XD + XM + TAB;
    static_assert(PB % 16 == 0, "the image is copied in 16-byte pieces");
    __host__ __device__ static constexpr int qcol(int m, int i) { return DIGIT_MAJOR ? 8 * i + m : 3 * m + i; }
    __host__ __device__ static constexpr int mcol(int m, int i, int part) {
        return DIGIT_MAJOR ? 8 * (2 * i + (m & 1)) + 2 * (m >> 1) + part : 2 * (3 * m + i) + part;
    }
};

// One warp turns the 256 values at xb (one super-block of k of row m of x; nullptr: a row beyond those of x, all zero)
// into its part of the super-block's image at `img` (global or shared memory);
// lane = octet: sub-block lane / 4, k-slots 8 (lane % 4) .. + 7 of that sub-block's MMA. Digit fragments are stored
// per pair of sub-blocks, so that the GEMV reads the B operands of two MMAs with one 16-byte load.
template <int MT>
__device__ __forceinline__ void build_image_from(const float (&xv)[8], bool present, int m, uint8_t* img, int lane) {
    // xv: this lane's eight values (lane = octet: sub-block lane / 4, elements 8 (lane % 4) .. + 7 of it); present = false:
    // a row beyond those of x, all zero
    using C = Cfg<MT>;
    constexpr int NG = C::NG, NCOL = C::NCOL, NCOLM = C::NCOLM;
    const int sub = lane >> 2, tt = lane & 3;
    uint2* xd = reinterpret_cast<uint2*>(img);
    uint8_t* xm = img + C::XD;
    float* tab = reinterpret_cast<float*>(img + C::XD + C::XM);
    if (!C::DIGIT_MAJOR && m == 0 && lane >= C::COLS && lane < NG * 8) {
        tab[lane] = 0.0f;  // columns that hold no activation row
        tab[NG * 8 + lane] = 0.0f;
    }
    // largest magnitude as an integer (NaN > Inf > every finite value in this order), so one comparison finds a value that is
    // not finite: the column weights then become NaN and with them every output of this row of x
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
    e = e < 0x0d000000u ? 0x0d000000u : (e > 0x7e800000u ? 0x7e800000u : e);  // keeps 2^21 / s and s * 2^-25 normal
    // 2^21 / s: |X| <= 2^22, so the top digit stays within a signed byte after the carries
    const float inv = __uint_as_float(0x7f000000u - e + (21u << 23));
    // X = rint(x * inv) lands in the mantissa of x * inv + 1.5 * 2^23 (the product is exact: inv is a power of two). With 128
    // added at every byte position the three low bytes of Y = X + 0x808080 are the signed base-256 digits plus 128 each
    // (X = d0 + 256 d1 + 65536 d2 with -128 <= d < 128 has exactly one such form), so digit = byte ^ 0x80.
    uint32_t Y[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        Y[i] = __float_as_uint(fmaf(xv[i], inv, 12582912.0f)) - 0x4b400000u + 0x00808080u;
    }
    // bytes of four values side by side: [Y0.b, Y1.b, Y2.b, Y3.b] for b = 0, 1, 2
    uint32_t dw[3][2];
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const uint32_t t01 = __byte_perm(Y[4 * h], Y[4 * h + 1], 0x5140), t23 = __byte_perm(Y[4 * h + 2], Y[4 * h + 3], 0x5140);
        const uint32_t h01 = __byte_perm(Y[4 * h], Y[4 * h + 1], 0x0062), h23 = __byte_perm(Y[4 * h + 2], Y[4 * h + 3], 0x0062);
        dw[0][h] = __byte_perm(t01, t23, 0x5410) ^ 0x80808080u;
        dw[1][h] = __byte_perm(t01, t23, 0x7632) ^ 0x80808080u;
        dw[2][h] = __byte_perm(h01, h23, 0x5410) ^ 0x80808080u;
    }
#pragma unroll
    for (int dgt = 0; dgt < 3; dgt++) {
        const uint32_t w0 = dw[dgt][0], w1 = dw[dgt][1];
        int sum = __dp4a((int)w0, 0x01010101, __dp4a((int)w1, 0x01010101, 0));  // the eight digits as signed bytes
        const int col = C::qcol(m, dgt);
        xd[((((size_t)(sub >> 1) * NG + (col >> 3)) * NCOL + (col & 7)) * 4 + tt) * 2 + (sub & 1)] = make_uint2(w0, w1);
        // digit sum of the sub-block (its 4 octets sit in 4 consecutive lanes): sum = 128 hi + lo7, both fit a signed byte.
        // The mins MMA has k = 16 and eight mins: lane slot sub / 4 holds the sums of sub-blocks 4 (sub / 4) .. + 3 as bytes,
        // lane slots 2 and 3 (k = 8 .. 15) are zero.
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (tt < 2) {
            const int lo7 = sum & 127, hi = (sum - lo7) >> 7;
#pragma unroll
            for (int p = 0; p < 2; p++) {
                const int mc = C::mcol(m, dgt, p);
                uint8_t* cell = xm + ((size_t)(mc >> 3) * NCOLM + (mc & 7)) * 16;
                cell[(tt == 0 ? (sub >> 2) : 2 + (sub >> 2)) * 4 + (sub & 3)] = tt == 0 ? (uint8_t)(p == 0 ? lo7 : hi) : (uint8_t)0;
            }
        }
        if (lane == 0) {
            tab[col] = !present ? 0.0f : (bad ? __uint_as_float(0x7fc00000u) : __uint_as_float(e + ((uint32_t)(8 * dgt) << 23) - (21u << 23)));  // s * 2^(8 dgt - 21)
            if (!C::DIGIT_MAJOR) {
                tab[NG * 8 + col] = !present ? 0.0f : (bad ? __uint_as_float(0x7fc00000u) : __uint_as_float(e + ((uint32_t)(8 * dgt) << 23) - (25u << 23)));  // ... / 16
            }
        }
    }
}

// This lane's eight values of the super-block at xb (nullptr: zeros).
__device__ __forceinline__ void load_image_values(const float* xb, int lane, float (&xv)[8]) {
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
}

template <int MT>
__device__ __forceinline__ void build_image(const float* xb, int m, uint8_t* img, int lane) {
    float xv[8];
    load_image_values(xb, lane, xv);
    build_image_from<MT>(xv, xb != nullptr, m, img, lane);
}

}  // namespace q4k
}  // namespace jq
