// Decode GEMV for Q4_K on the tensor cores: y[m, n] = x[m, k] . W[n, k]^T for 1 <= m <= 16.
//
// Why tensor cores for a matrix-vector product: at HBM speed a B200 SM has to consume about 40
// four-bit weights per clock. Unpacking a nibble, converting it to float and issuing one FMA per
// activation row costs three or more instructions per weight on the CUDA cores, which is more than the
// SM can issue. Here two nibbles become an fp16 pair with one logic operation (the bits are OR-ed into
// the mantissa of 1024.0) and one half2 FMA that also folds in the 6-bit sub-block scale (scale * q is
// an integer below 2048, exact in fp16); mma.sync.m16n8k16 then does the multiply-accumulate for up to
// four activation rows at once with FP32 accumulation.
//
// Numerics: activations stay FP32-accurate. Each x is scaled by a power of two (per row of x) and split
// into an fp16 head and an fp16 remainder, x = s * (hi + lo), which occupy two columns of the B operand.
// Products sc*q*hi and sc*q*lo are exact in the FP32 accumulator; per super-block the accumulator is
// scaled by fp16 d in FP32. The "min" part of Q4_K, -dmin * m_sub * sum(x over the sub-block), goes
// through one more MMA whose A operand holds the eight 6-bit mins and whose B operand holds the
// sub-block sums of x. The reduction order depends only on k, never on n, so a row shard of a weight
// yields bitwise the same outputs as the whole weight.
//
// Work split: a CTA (8 warps) owns 16 output rows at a time and walks the tiles blockIdx.x,
// blockIdx.x + gridDim.x, ...; warp p takes the super-blocks b = p (mod 8) of those rows. Lane (g, t)
// (g = lane / 4, t = lane % 4) loads for rows g and g + 8 the 16-byte header and the 32 bytes of nibbles
// of group t (sub-blocks 2t and 2t+1) with 128-bit loads, one super-block ahead of the arithmetic.
// The activations are converted once per CTA into MMA B-fragment order in shared memory.
#include <cuda_fp16.h>

#include "jq_formats.cuh"

namespace jq {

namespace {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int FRAGS = 17;  // 16 MMAs of quants + 1 MMA of mins per super-block

__device__ __forceinline__ __half2 u2h(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint32_t h2u(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) { return h2u(__floats2half2_rn(lo, hi)); }

// What one lane holds of one super-block of two rows: header and its group's nibbles.
struct Raw {
    uint4 h0, h1;    // headers of rows g and g + 8
    uint4 a0, a1;    // row g: bytes [32t, 32t+32) of qs
    uint4 b0, b1;    // row g + 8
};

// Per row: fp16 pairs used by the conversion of this lane's two sub-blocks, and d / dmin.
struct RowScales {
    __half2 s_lo, c_lo;  // (sc, sc) and -1024 * sc for sub-block 2t (low nibbles)
    __half2 s_hi, c_hi;  // (sc / 16, sc / 16) and -64 * sc for sub-block 2t + 1 (high nibbles)
    uint32_t mins;       // half2 (m[2t], m[2t+1])
    float d, dmin;
};

__device__ __forceinline__ RowScales decode_scales(const uint4& h, int t) {
    // 12 packed bytes: bytes 0-3 low 6 bits sc[0..3], bytes 4-7 low 6 bits m[0..3]; bytes 8-11 low/high
    // nibbles sc[4..7]/m[4..7] whose top two bits sit in the top two bits of bytes 0-3 / 4-7.
    uint32_t sc = t < 2 ? (h.y & 0x3f3f3f3fu) : ((h.w & 0x0f0f0f0fu) | ((h.y >> 2) & 0x30303030u));
    uint32_t mn = t < 2 ? (h.z & 0x3f3f3f3fu) : (((h.w >> 4) & 0x0f0f0f0fu) | ((h.z >> 2) & 0x30303030u));
    const uint32_t bi = (2u * (uint32_t)t) & 3u;
    const uint32_t magic = 0x64646464u;  // byte 0x64 = high byte of fp16 1024.0
    uint32_t lo = __byte_perm(sc, magic, (4u << 12) | (bi << 8) | (4u << 4) | bi);
    uint32_t hi = __byte_perm(sc, magic, (4u << 12) | ((bi + 1) << 8) | (4u << 4) | (bi + 1));
    uint32_t mm = __byte_perm(mn, magic, (4u << 12) | ((bi + 1) << 8) | (4u << 4) | bi);
    RowScales r;
    const __half2 k1024 = u2h(0x64006400u), kneg1024 = u2h(0xE400E400u), k16th = u2h(0x2C002C00u), kneg64 = u2h(0xD400D400u);
    r.s_lo = __hsub2(u2h(lo), k1024);
    r.c_lo = __hmul2(r.s_lo, kneg1024);
    r.s_hi = __hfma2(u2h(hi), k16th, kneg64);
    r.c_hi = __hmul2(r.s_hi, kneg1024);
    r.mins = h2u(__hsub2(u2h(mm), k1024));
    r.d = half_bits_to_float(h.x);
    r.dmin = half_bits_to_float(h.x >> 16);
    return r;
}

template <int MT>
struct Cfg {
    static constexpr int NG = MT <= 4 ? 1 : MT / 4;      // column groups of four activation rows
    static constexpr int NCOL = MT <= 4 ? 2 * MT : 8;    // B columns stored per group (hi, lo per row)
    static constexpr int MP = NG * 4;                    // activation rows padded to the groups
};

template <int MT>
__host__ __device__ constexpr size_t frag_bytes_per_block() {
    return (size_t)FRAGS * Cfg<MT>::NG * Cfg<MT>::NCOL * 4 * 8;
}

template <int MT>
__global__ void __launch_bounds__(THREADS, 2) gemv_q4k_mma_kernel(View v, const float* __restrict__ x, int rows,
                                                                 const float* __restrict__ bias, float* __restrict__ y, int tiles) {
    using C = Cfg<MT>;
    constexpr int NG = C::NG, NCOL = C::NCOL, MP = C::MP;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int KB = (int)(v.k >> 8);
    uint2* xf = reinterpret_cast<uint2*>(smem_raw);                                   // [KB][FRAGS][NG][NCOL][4]
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)KB * frag_bytes_per_block<MT>());  // [2][WARPS][16][MP]
    float* amax_s = red + 2 * WARPS * 16 * MP;                                         // [WARPS][MT]
    float* scale_s = amax_s + WARPS * MT;                                              // [MT]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int64_t n = v.n;
    const int64_t row_bytes = (int64_t)KB * 144;

    auto load_raw = [&](Raw& r, int tile, int b) {
        int64_t r0 = (int64_t)tile * 16 + g, r1 = r0 + 8;
        r0 = r0 < n ? r0 : n - 1;
        r1 = r1 < n ? r1 : n - 1;
        const uint8_t* p0 = v.q + r0 * row_bytes + (int64_t)b * 144;
        const uint8_t* p1 = v.q + r1 * row_bytes + (int64_t)b * 144;
        r.h0 = ld16(p0);
        r.h1 = ld16(p1);
        r.a0 = ld16(p0 + 16 + 32 * t);
        r.a1 = ld16(p0 + 32 + 32 * t);
        r.b0 = ld16(p1 + 16 + 32 * t);
        r.b1 = ld16(p1 + 32 + 32 * t);
    };

    // The first weights are requested before the activations are prepared: they do not depend on x.
    int tile = blockIdx.x, b = warp;
    // advance (tile, b) to this warp's first valid step
    auto valid = [&]() { return tile < tiles; };
    if (b >= KB) {
        tile = tiles;  // a warp without super-blocks only helps with the activations and the reduction
    }
    Raw cur;
    if (valid()) {
        load_raw(cur, tile, b);
    }

    // ---- activations -> B fragments in shared memory ------------------------------------------------------
    const int quads = (int)(v.k >> 2);
    {
        float am[MT];
#pragma unroll
        for (int m = 0; m < MT; m++) {
            am[m] = 0.0f;
        }
        for (int q = tid; q < quads; q += THREADS) {
#pragma unroll
            for (int m = 0; m < MT; m++) {
                if (m < rows) {
                    float4 xv = __ldg(reinterpret_cast<const float4*>(x + (int64_t)m * v.k) + q);
                    am[m] = fmaxf(am[m], fmaxf(fmaxf(fabsf(xv.x), fabsf(xv.y)), fmaxf(fabsf(xv.z), fabsf(xv.w))));
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MT; m++) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                am[m] = fmaxf(am[m], __shfl_xor_sync(0xffffffffu, am[m], o));
            }
            if (lane == 0) {
                amax_s[warp * MT + m] = am[m];
            }
        }
        __syncthreads();
        if (tid < MT) {
            float a = 0.0f;
            for (int w = 0; w < WARPS; w++) {
                a = fmaxf(a, amax_s[w * MT + tid]);
            }
            // s = 2^floor(log2(amax)) so that the largest |x| / s lies in [1, 2)
            uint32_t e = __float_as_uint(a) & 0x7f800000u;
            e = e < 0x00800000u ? 0x00800000u : (e > 0x7e800000u ? 0x7e800000u : e);
            scale_s[tid] = __uint_as_float(e);
        }
        __syncthreads();
        for (int q = tid; q < quads; q += THREADS) {
            const int blk = q >> 6, eb = (q & 63) << 2;        // element offset inside the super-block
            const int j = eb >> 6, hf = (eb >> 5) & 1, w = (eb & 31) >> 2;
            uint2* frag = xf + ((size_t)(blk * FRAGS + 2 * w + hf) * NG) * NCOL * 4;
            uint2* fmin = xf + ((size_t)(blk * FRAGS + 16) * NG) * NCOL * 4;
#pragma unroll
            for (int m = 0; m < (MT <= 4 ? MT : MP); m++) {
                float4 xv = make_float4(0.f, 0.f, 0.f, 0.f);
                if (m < rows) {
                    xv = __ldg(reinterpret_cast<const float4*>(x + (int64_t)m * v.k) + q);
                    const float inv = __uint_as_float(0x7f000000u - __float_as_uint(scale_s[m]));
                    xv.x *= inv; xv.y *= inv; xv.z *= inv; xv.w *= inv;
                }
                __half2 h02 = __floats2half2_rn(xv.x, xv.z), h13 = __floats2half2_rn(xv.y, xv.w);
                float2 f02 = __half22float2(h02), f13 = __half22float2(h13);
                uint32_t l02 = pack_half2(xv.x - f02.x, xv.z - f02.y), l13 = pack_half2(xv.y - f13.x, xv.w - f13.y);
                const int grp = m >> 2, col = (m & 3) * 2;
                uint2* dst = frag + ((size_t)grp * NCOL + col) * 4 + j;
                dst[0] = make_uint2(h2u(h02), h2u(h13));
                dst[4] = make_uint2(l02, l13);
                // sub-block sum of x for the mins: 8 consecutive quads = 8 consecutive lanes
                float s = (xv.x + xv.y) + (xv.z + xv.w);
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                s += __shfl_xor_sync(0xffffffffu, s, 4);
                if ((lane & 7) == 0) {
                    __half sh = __float2half_rn(s);
                    __half sl = __float2half_rn(s - __half2float(sh));
                    uint2* md = fmin + ((size_t)grp * NCOL + col) * 4 + j;
                    reinterpret_cast<__half*>(md)[hf] = sh;
                    reinterpret_cast<__half*>(md + 4)[hf] = sl;
                    if (hf == 0) {
                        md[0].y = 0u;
                        md[4].y = 0u;
                    }
                }
            }
        }
        __syncthreads();
    }

    // ---- main loop -------------------------------------------------------------------------------------------
    float acc[NG][2];
#pragma unroll
    for (int i = 0; i < NG; i++) {
        acc[i][0] = acc[i][1] = 0.0f;
    }
    int parity = 0;
    for (int my_tile = blockIdx.x; my_tile < tiles; my_tile += gridDim.x) {
        // every warp takes part in every tile's reduction, with or without super-blocks of its own
        while (valid() && tile == my_tile) {
            // prefetch the next step of this warp
            int nt = tile, nb = b + WARPS;
            if (nb >= KB) {
                nb = warp;
                nt = tile + gridDim.x;
            }
            Raw nxt;
            const bool more = nt < tiles;
            if (more) {
                load_raw(nxt, nt, nb);
            }

            RowScales s0 = decode_scales(cur.h0, t), s1 = decode_scales(cur.h1, t);
            float D[NG][4], E[NG][4];
#pragma unroll
            for (int i = 0; i < NG; i++) {
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    D[i][c] = 0.0f;
                    E[i][c] = 0.0f;
                }
            }
            const uint2* fb = xf + ((size_t)b * FRAGS * NG) * NCOL * 4 + (size_t)g * 4 + t;
            const uint32_t wa[8] = {cur.a0.x, cur.a0.y, cur.a0.z, cur.a0.w, cur.a1.x, cur.a1.y, cur.a1.z, cur.a1.w};
            const uint32_t wb[8] = {cur.b0.x, cur.b0.y, cur.b0.z, cur.b0.w, cur.b1.x, cur.b1.y, cur.b1.z, cur.b1.w};
#pragma unroll
            for (int w = 0; w < 8; w++) {
                const uint32_t va = wa[w], vb = wb[w], va8 = va >> 8, vb8 = vb >> 8;
                // low nibbles: sub-block 2t, elements 4w + {0, 2} and 4w + {1, 3}
                uint32_t a0 = h2u(__hfma2(u2h((va & 0x000F000Fu) | 0x64006400u), s0.s_lo, s0.c_lo));
                uint32_t a2 = h2u(__hfma2(u2h((va8 & 0x000F000Fu) | 0x64006400u), s0.s_lo, s0.c_lo));
                uint32_t a1 = h2u(__hfma2(u2h((vb & 0x000F000Fu) | 0x64006400u), s1.s_lo, s1.c_lo));
                uint32_t a3 = h2u(__hfma2(u2h((vb8 & 0x000F000Fu) | 0x64006400u), s1.s_lo, s1.c_lo));
#pragma unroll
                for (int i = 0; i < NG; i++) {
                    uint2 bf = make_uint2(0u, 0u);
                    if (NCOL == 8 || g < NCOL) {
                        bf = fb[((size_t)(2 * w) * NG + i) * NCOL * 4];
                    }
                    mma16816(D[i], a0, a1, a2, a3, bf.x, bf.y);
                }
                // high nibbles: sub-block 2t + 1
                a0 = h2u(__hfma2(u2h((va & 0x00F000F0u) | 0x64006400u), s0.s_hi, s0.c_hi));
                a2 = h2u(__hfma2(u2h((va8 & 0x00F000F0u) | 0x64006400u), s0.s_hi, s0.c_hi));
                a1 = h2u(__hfma2(u2h((vb & 0x00F000F0u) | 0x64006400u), s1.s_hi, s1.c_hi));
                a3 = h2u(__hfma2(u2h((vb8 & 0x00F000F0u) | 0x64006400u), s1.s_hi, s1.c_hi));
#pragma unroll
                for (int i = 0; i < NG; i++) {
                    uint2 bf = make_uint2(0u, 0u);
                    if (NCOL == 8 || g < NCOL) {
                        bf = fb[((size_t)(2 * w + 1) * NG + i) * NCOL * 4];
                    }
                    mma16816(D[i], a0, a1, a2, a3, bf.x, bf.y);
                }
            }
#pragma unroll
            for (int i = 0; i < NG; i++) {
                uint2 bf = make_uint2(0u, 0u);
                if (NCOL == 8 || g < NCOL) {
                    bf = fb[((size_t)16 * NG + i) * NCOL * 4];
                }
                mma16816(E[i], s0.mins, s1.mins, 0u, 0u, bf.x, bf.y);
                acc[i][0] += s0.d * (D[i][0] + D[i][1]) - s0.dmin * (E[i][0] + E[i][1]);
                acc[i][1] += s1.d * (D[i][2] + D[i][3]) - s1.dmin * (E[i][2] + E[i][3]);
            }

            tile = nt;
            b = nb;
            if (more) {
                cur = nxt;
            }
        }
        // ---- reduce the 8 warps' partial sums of this tile in a fixed order ---------------------------------
        float* rd = red + (size_t)parity * WARPS * 16 * MP;
#pragma unroll
        for (int i = 0; i < NG; i++) {
            rd[(warp * 16 + g) * MP + i * 4 + t] = acc[i][0];
            rd[(warp * 16 + g + 8) * MP + i * 4 + t] = acc[i][1];
            acc[i][0] = acc[i][1] = 0.0f;
        }
        __syncthreads();
        for (int o = tid; o < 16 * MP; o += THREADS) {
            const int r = o / MP, m = o % MP;
            const int64_t row = (int64_t)my_tile * 16 + r;
            if (m < rows && row < n) {
                const float* p = rd + r * MP + m;
                float s = ((p[0] + p[16 * MP]) + (p[2 * 16 * MP] + p[3 * 16 * MP])) +
                          ((p[4 * 16 * MP] + p[5 * 16 * MP]) + (p[6 * 16 * MP] + p[7 * 16 * MP]));
                y[(int64_t)m * n + row] = s * scale_s[m] + (bias != nullptr ? bias[row] : 0.0f);
            }
        }
        parity ^= 1;
    }
}

int g_sms = 0;
int sm_count() {
    if (g_sms == 0) {
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0) {
            g_sms = sms;
        } else {
            g_sms = 148;
        }
    }
    return g_sms;
}

template <int MT>
int run_q4k(const View& v, const float* x, int rows, const float* bias, float* y, cudaStream_t s, bool* handled) {
    using C = Cfg<MT>;
    const int KB = (int)(v.k / 256);
    size_t smem = (size_t)KB * frag_bytes_per_block<MT>() + (size_t)(2 * WARPS * 16 * C::MP + WARPS * MT + MT) * sizeof(float);
    if (smem > 200 * 1024) {
        *handled = false;  // the activations do not fit in shared memory in fragment form
        return JQ_OK;
    }
    // the opt-in for more than 48 KB of dynamic shared memory is per device
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    JQ_CUDA(cudaGetDevice(&dev));
    if ((configured.load() >> (dev & 63) & 1) == 0) {
        JQ_CUDA(cudaFuncSetAttribute(gemv_q4k_mma_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured.fetch_or((uint64_t)1 << (dev & 63));
    }
    const int tiles = (int)((v.n + 15) / 16);
    int per_sm = smem > 100 * 1024 ? 1 : 2;
    int grid = tiles < sm_count() * per_sm ? tiles : sm_count() * per_sm;
    gemv_q4k_mma_kernel<MT><<<grid, THREADS, smem, s>>>(v, x, rows, bias, y, tiles);
    count_launch();
    *handled = true;
    return check_launch("gemv_q4k_mma_kernel");
}

}  // namespace

// Q4_K with rows in [1, 16]. *handled = false means the shape is left to the generic kernel.
int launch_gemv_q4k_mma(const View& v, const float* x, int rows, const float* bias, float* y, cudaStream_t s, bool* handled) {
    *handled = false;
    if (v.type != JQ_TYPE_Q4_K || v.n == 0 || v.k == 0) {
        return JQ_OK;
    }
    if (rows == 1) return run_q4k<1>(v, x, rows, bias, y, s, handled);
    if (rows == 2) return run_q4k<2>(v, x, rows, bias, y, s, handled);
    if (rows <= 4) return run_q4k<4>(v, x, rows, bias, y, s, handled);
    if (rows <= 8) return run_q4k<8>(v, x, rows, bias, y, s, handled);
    return run_q4k<16>(v, x, rows, bias, y, s, handled);
}

}  // namespace jq
