// Device-side decoders of the GGUF block formats on the linear path.
//
// Every format is described by a struct Fmt<TYPE> that splits a block into "units": the weights a
// single thread decodes from one or three 16-byte loads. A unit yields RUNS runs of 16 consecutive
// weights. decode() reproduces the reference's per-element arithmetic bit for bit
// (kernels/GgufKernels.java:85-140 and ops/Quant.java:137-144 of the reference): each multiply, add
// and subtract is a separately rounded float operation (__fmul_rn / __fadd_rn / __fsub_rn are never
// contracted into a fused multiply-add), in the reference's association order.
//
// Device layouts (what View::q and View::aux hold):
//   Q4_K  144-byte blocks as in GGUF (fp16 d, fp16 dmin, 12 scale bytes, 128 bytes of nibbles), stored tile by tile
//   Q5_K  176-byte blocks as in GGUF (fp16 d, fp16 dmin, 12 scale bytes, 32 bytes qh, 128 bytes qs), stored tile by tile
//         (tiles of 128 rows, the blocks of one super-block of k together: tiled_offset in jq_common.cuh)
//   Q6_K  q: 208 bytes per block (128 ql, 64 qh, 16 int8 scales); aux: fp16 d per block
//   Q8_0  q: 32 int8 per block; aux: fp16 d per block
//   Q4_0  q: 16 nibble bytes per block; aux: fp16 d per block
//   Q4_1  q: 16 nibble bytes per block; aux: fp16 d, fp16 m per block
#pragma once

#include <cuda_fp16.h>

#include "jq_common.cuh"

namespace jq {

__device__ __forceinline__ float half_bits_to_float(uint32_t bits16) {
    return __half2float(__ushort_as_half((unsigned short)(bits16 & 0xffffu)));
}

__device__ __forceinline__ uint4 ld16(const uint8_t* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

// Address of block number `block` (row-major numbering: row * blocks per row + b) of a tiled weight.
__device__ __forceinline__ const uint8_t* tiled_block(const View& v, int64_t block, int bytes) {
    const uint32_t kb = (uint32_t)(v.k >> 8);
    const uint32_t row = (uint32_t)block / kb, b = (uint32_t)block - row * kb;  // fewer than 2^23 blocks: weights have fewer than 2^31 elements
    return v.q + tiled_offset(row, b, kb, bytes);
}

__device__ __forceinline__ uint32_t byte_of(uint32_t w, int i) { return (w >> (8 * i)) & 0xffu; }

// Byte i (0..11) of the 12 scale bytes held in three words.
__device__ __forceinline__ uint32_t scale_byte(uint32_t s0, uint32_t s1, uint32_t s2, int i) {
    uint32_t w = i < 4 ? s0 : (i < 8 ? s1 : s2);
    return byte_of(w, i & 3);
}

// 6-bit scale and min of sub-block `sub` (GgufKernels.java:74-83).
__device__ __forceinline__ void k_scale_min(uint32_t s0, uint32_t s1, uint32_t s2, int sub, int& sc, int& mn) {
    if (sub < 4) {
        sc = scale_byte(s0, s1, s2, sub) & 63;
        mn = scale_byte(s0, s1, s2, sub + 4) & 63;
    } else {
        uint32_t b = scale_byte(s0, s1, s2, sub + 4);
        sc = (b & 15) | ((scale_byte(s0, s1, s2, sub - 4) >> 6) << 4);
        mn = (b >> 4) | ((scale_byte(s0, s1, s2, sub) >> 6) << 4);
    }
}

template <int TYPE>
struct Fmt;

// ---- Q8_0: w = d * q (ops/Quant.java:141-142) ---------------------------------------------------
template <>
struct Fmt<JQ_TYPE_Q8_0> {
    static constexpr int QK = 32, UNITS = 2, RUNS = 1;
    struct Raw {
        uint4 q;
        uint32_t d;
    };
    __device__ static void load(const View& v, int64_t block, int unit, Raw& r) {
        r.q = ld16(v.q + block * 32 + unit * 16);
        r.d = __ldg(reinterpret_cast<const unsigned short*>(v.aux) + block);
    }
    __device__ static void decode(const View& v, int64_t block, int unit, float (&out)[RUNS][16], int (&pos)[RUNS]) {
        Raw r;
        load(v, block, unit, r);
        convert(r, unit, out, pos);
    }
    __device__ static void convert(const Raw& r, int unit, float (&out)[RUNS][16], int (&pos)[RUNS]) {
        const uint4 q = r.q;
        float d = half_bits_to_float(r.d);
        uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 16; i++) {
            int s = (int)(int8_t)byte_of(w[i >> 2], i & 3);
            out[0][i] = __fmul_rn(d, (float)s);
        }
        pos[0] = unit * 16;
    }
};

// ---- Q4_0: w = (q - 8) * d (GgufKernels.java:85-91) ---------------------------------------------
template <>
struct Fmt<JQ_TYPE_Q4_0> {
    static constexpr int QK = 32, UNITS = 1, RUNS = 2;
    struct Raw {
        uint4 q;
        uint32_t d;
    };
    __device__ static void load(const View& v, int64_t block, int, Raw& r) {
        r.q = ld16(v.q + block * 16);
        r.d = __ldg(reinterpret_cast<const unsigned short*>(v.aux) + block);
    }
    __device__ static void decode(const View& v, int64_t block, int unit, float (&out)[RUNS][16], int (&pos)[RUNS]) {
        Raw r;
        load(v, block, unit, r);
        convert(r, unit, out, pos);
    }
    __device__ static void convert(const Raw& r, int, float (&out)[RUNS][16], int (&pos)[RUNS]) {
        const uint4 q = r.q;
        float d = half_bits_to_float(r.d);
        uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 16; i++) {
            uint32_t b = byte_of(w[i >> 2], i & 3);
            out[0][i] = __fmul_rn((float)((int)(b & 15) - 8), d);
            out[1][i] = __fmul_rn((float)((int)(b >> 4) - 8), d);
        }
        pos[0] = 0;
        pos[1] = 16;
    }
};

// ---- Q4_1: w = (q * d) + m (GgufKernels.java:93-99) ---------------------------------------------
template <>
struct Fmt<JQ_TYPE_Q4_1> {
    static constexpr int QK = 32, UNITS = 1, RUNS = 2;
    struct Raw {
        uint4 q;
        uint32_t dm;
    };
    __device__ static void load(const View& v, int64_t block, int, Raw& r) {
        r.q = ld16(v.q + block * 16);
        r.dm = __ldg(reinterpret_cast<const uint32_t*>(v.aux) + block);
    }
    __device__ static void decode(const View& v, int64_t block, int unit, float (&out)[RUNS][16], int (&pos)[RUNS]) {
        Raw r;
        load(v, block, unit, r);
        convert(r, unit, out, pos);
    }
    __device__ static void convert(const Raw& r, int, float (&out)[RUNS][16], int (&pos)[RUNS]) {
        const uint4 q = r.q;
        const uint32_t dm = r.dm;
        float d = half_bits_to_float(dm), m = half_bits_to_float(dm >> 16);
        uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 16; i++) {
            uint32_t b = byte_of(w[i >> 2], i & 3);
            out[0][i] = __fadd_rn(__fmul_rn((float)(b & 15), d), m);
            out[1][i] = __fadd_rn(__fmul_rn((float)(b >> 4), d), m);
        }
        pos[0] = 0;
        pos[1] = 16;
    }
};

// ---- Q4_K: w = ((d * sc) * q) - (dmin * m) (GgufKernels.java:101-111) ----------------------------
template <>
struct Fmt<JQ_TYPE_Q4_K> {
    static constexpr int QK = 256, UNITS = 8, RUNS = 2;
    struct Raw {
        uint4 h, q;
    };
    __device__ static void load(const View& v, int64_t block, int unit, Raw& r) {
        const uint8_t* b = tiled_block(v, block, 144);
        r.h = ld16(b);
        r.q = ld16(b + 16 + unit * 16);
    }
    __device__ static void decode(const View& v, int64_t block, int unit, float (&out)[RUNS][16], int (&pos)[RUNS]) {
        Raw r;
        load(v, block, unit, r);
        convert(r, unit, out, pos);
    }
    __device__ static void convert(const Raw& r, int unit, float (&out)[RUNS][16], int (&pos)[RUNS]) {
        const uint4 h = r.h, q = r.q;
        float d = half_bits_to_float(h.x), dmin = half_bits_to_float(h.x >> 16);
        int j = unit >> 1, hf = unit & 1;
        int sc0, mn0, sc1, mn1;
        k_scale_min(h.y, h.z, h.w, 2 * j, sc0, mn0);
        k_scale_min(h.y, h.z, h.w, 2 * j + 1, sc1, mn1);
        float a0 = __fmul_rn(d, (float)sc0), m0 = __fmul_rn(dmin, (float)mn0);
        float a1 = __fmul_rn(d, (float)sc1), m1 = __fmul_rn(dmin, (float)mn1);
        uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 16; i++) {
            uint32_t by = byte_of(w[i >> 2], i & 3);
            out[0][i] = __fsub_rn(__fmul_rn(a0, (float)(by & 15)), m0);
            out[1][i] = __fsub_rn(__fmul_rn(a1, (float)(by >> 4)), m1);
        }
        pos[0] = 64 * j + 16 * hf;
        pos[1] = pos[0] + 32;
    }
};

// ---- Q5_K: as Q4_K with a fifth bit from qh (GgufKernels.java:113-125) ---------------------------
template <>
struct Fmt<JQ_TYPE_Q5_K> {
    static constexpr int QK = 256, UNITS = 8, RUNS = 2;
    struct Raw {
        uint4 h, hi, q;
    };
    __device__ static void load(const View& v, int64_t block, int unit, Raw& r) {
        const uint8_t* b = tiled_block(v, block, 176);
        r.h = ld16(b);
        r.hi = ld16(b + 16 + (unit & 1) * 16);
        r.q = ld16(b + 48 + unit * 16);
    }
    __device__ static void decode(const View& v, int64_t block, int unit, float (&out)[RUNS][16], int (&pos)[RUNS]) {
        Raw r;
        load(v, block, unit, r);
        convert(r, unit, out, pos);
    }
    __device__ static void convert(const Raw& r, int unit, float (&out)[RUNS][16], int (&pos)[RUNS]) {
        const uint4 h = r.h, hi = r.hi, q = r.q;
        int j = unit >> 1, hf = unit & 1;
        float d = half_bits_to_float(h.x), dmin = half_bits_to_float(h.x >> 16);
        int sc0, mn0, sc1, mn1;
        k_scale_min(h.y, h.z, h.w, 2 * j, sc0, mn0);
        k_scale_min(h.y, h.z, h.w, 2 * j + 1, sc1, mn1);
        float a0 = __fmul_rn(d, (float)sc0), m0 = __fmul_rn(dmin, (float)mn0);
        float a1 = __fmul_rn(d, (float)sc1), m1 = __fmul_rn(dmin, (float)mn1);
        uint32_t w[4] = {q.x, q.y, q.z, q.w};
        uint32_t g[4] = {hi.x, hi.y, hi.z, hi.w};
#pragma unroll
        for (int i = 0; i < 16; i++) {
            uint32_t by = byte_of(w[i >> 2], i & 3);
            uint32_t hb = byte_of(g[i >> 2], i & 3);
            uint32_t q0 = (by & 15) + 16 * ((hb >> (2 * j)) & 1);
            uint32_t q1 = (by >> 4) + 16 * ((hb >> (2 * j + 1)) & 1);
            out[0][i] = __fsub_rn(__fmul_rn(a0, (float)q0), m0);
            out[1][i] = __fsub_rn(__fmul_rn(a1, (float)q1), m1);
        }
        pos[0] = 64 * j + 16 * hf;
        pos[1] = pos[0] + 32;
    }
};

// ---- Q6_K: w = (d * sc) * q, q in [-32, 31] (GgufKernels.java:127-140) ---------------------------
template <>
struct Fmt<JQ_TYPE_Q6_K> {
    static constexpr int QK = 256, UNITS = 4, RUNS = 4;
    struct Raw {
        uint4 la, lb, hq, sv;
        uint32_t d;
    };
    __device__ static void load(const View& v, int64_t block, int unit, Raw& r) {
        const uint32_t kb = (uint32_t)(v.k >> 8);
        const uint32_t row = (uint32_t)block / kb;
        const int64_t at = tiled_index(row, (uint32_t)block - row * kb, kb);  // the planes hold their blocks in tiled order
        const uint8_t* b = v.q + at * 208;
        const int n = unit >> 1, c = unit & 1;
        r.la = ld16(b + 64 * n + 16 * c);
        r.lb = ld16(b + 64 * n + 32 + 16 * c);
        r.hq = ld16(b + 128 + 32 * n + 16 * c);
        r.sv = ld16(b + 192);
        r.d = __ldg(reinterpret_cast<const unsigned short*>(v.aux) + at);
    }
    __device__ static void decode(const View& v, int64_t block, int unit, float (&out)[RUNS][16], int (&pos)[RUNS]) {
        Raw r;
        load(v, block, unit, r);
        convert(r, unit, out, pos);
    }
    __device__ static void convert(const Raw& r, int unit, float (&out)[RUNS][16], int (&pos)[RUNS]) {
        const uint4 la = r.la, lb = r.lb, hq = r.hq, sv = r.sv;
        int n = unit >> 1, c = unit & 1;
        float d = half_bits_to_float(r.d);
        uint32_t sw0 = n == 0 ? sv.x : sv.z, sw1 = n == 0 ? sv.y : sv.w;  // scale bytes 8n .. 8n+7
        float a[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            int idx = c + 2 * k;  // 0..7 within this half
            int s = (int)(int8_t)byte_of(idx < 4 ? sw0 : sw1, idx & 3);
            a[k] = __fmul_rn(d, (float)s);
        }
        uint32_t wa[4] = {la.x, la.y, la.z, la.w}, wb[4] = {lb.x, lb.y, lb.z, lb.w}, wh[4] = {hq.x, hq.y, hq.z, hq.w};
#pragma unroll
        for (int i = 0; i < 16; i++) {
            uint32_t ba = byte_of(wa[i >> 2], i & 3), bb = byte_of(wb[i >> 2], i & 3), bh = byte_of(wh[i >> 2], i & 3);
            int q0 = (int)((ba & 15) | ((bh & 3) << 4)) - 32;
            int q1 = (int)((bb & 15) | (((bh >> 2) & 3) << 4)) - 32;
            int q2 = (int)((ba >> 4) | (((bh >> 4) & 3) << 4)) - 32;
            int q3 = (int)((bb >> 4) | (((bh >> 6) & 3) << 4)) - 32;
            out[0][i] = __fmul_rn(a[0], (float)q0);
            out[1][i] = __fmul_rn(a[1], (float)q1);
            out[2][i] = __fmul_rn(a[2], (float)q2);
            out[3][i] = __fmul_rn(a[3], (float)q3);
        }
#pragma unroll
        for (int k = 0; k < 4; k++) {
            pos[k] = 128 * n + 32 * k + 16 * c;
        }
    }
};

}  // namespace jq
