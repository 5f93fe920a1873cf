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
// of group t (sub-blocks 2t and 2t+1). The weights travel HBM -> shared memory with 16-byte cp.async
// copies into a private ring of STAGES super-block slots per warp, so each warp keeps STAGES - 1
// super-blocks (2304 bytes each) in flight without holding registers for them.
// The activations are converted once per CTA into MMA B-fragment order in shared memory.
#include <cuda_fp16.h>

#include "jq_formats.cuh"

namespace jq {

namespace {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int FRAGS = 17;  // 16 MMAs of quants + 1 MMA of mins per super-block
constexpr int SLOT_BYTES = 16 * 144;      // one super-block of 16 rows

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint4 lds16(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }

__device__ __forceinline__ __half2 u2h(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint32_t h2u(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The first MMA of an accumulator chain: C = 0 (the zero register), so no accumulator needs clearing.
__device__ __forceinline__ void mma16816_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

// (a & b) | c in one logic instruction.
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Two nibbles (selected by mask) placed in the mantissas of a pair of fp16 1024.0: (1024 + q, 1024 + q').
__device__ __forceinline__ __half2 magic_pair(uint32_t v, uint32_t mask) { return u2h(and_or(v, mask, 0x64006400u)); }

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) { return h2u(__floats2half2_rn(lo, hi)); }

// Per row: fp16 pairs used by the conversion of this lane's two sub-blocks, and d / dmin.
struct RowScales {
    __half2 s_lo, c_lo;  // (sc, sc) and -1024 * sc for sub-block 2t (low nibbles)
    __half2 s_hi, c_hi;  // (sc / 16, sc / 16) and -64 * sc for sub-block 2t + 1 (high nibbles)
    uint32_t mins;       // half2 (m[2t], m[2t+1])
    float d, dmin;
};

// Lane constants of the 6-bit scale unpacking. The 12 packed bytes (three words y, z, w of the header):
// bytes 0-3 hold sc[0..3] in their low 6 bits, bytes 4-7 hold m[0..3]; bytes 8-11 hold the low nibbles of
// sc[4..7] (low half) and m[4..7] (high half), whose top two bits are the top two bits of bytes 0-3 / 4-7.
// Lanes t < 2 need sub-blocks 0..3, lanes t >= 2 sub-blocks 4..7; both cases are written as
// ((y >> sh) & ma) | (w & mb) so that no lane takes a branch.
struct LaneConsts {
    uint32_t sh, ma, mb;            // shift and masks, see above
    uint32_t sel_lo, sel_hi, sel_m; // byte_perm selectors building fp16 1024+value pairs
};

__device__ __forceinline__ LaneConsts lane_consts(int t) {
    LaneConsts c;
    c.sh = t < 2 ? 0u : 2u;
    c.ma = t < 2 ? 0x3f3f3f3fu : 0x30303030u;
    c.mb = t < 2 ? 0u : 0x0f0f0f0fu;
    const uint32_t bi = (2u * (uint32_t)t) & 3u;
    c.sel_lo = (4u << 12) | (bi << 8) | (4u << 4) | bi;
    c.sel_hi = (4u << 12) | ((bi + 1) << 8) | (4u << 4) | (bi + 1);
    c.sel_m = (4u << 12) | ((bi + 1) << 8) | (4u << 4) | bi;
    return c;
}

__device__ __forceinline__ RowScales decode_scales(const uint4& h, const LaneConsts& c) {
    const uint32_t sc = and_or(h.y >> c.sh, c.ma, h.w & c.mb);
    const uint32_t mn = and_or(h.z >> c.sh, c.ma, (h.w >> 4) & c.mb);
    const uint32_t magic = 0x64646464u;  // byte 0x64 = high byte of fp16 1024.0
    const uint32_t lo = __byte_perm(sc, magic, c.sel_lo);
    const uint32_t hi = __byte_perm(sc, magic, c.sel_hi);
    const uint32_t mm = __byte_perm(mn, magic, c.sel_m);
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

template <int MT, int STAGES>
__global__ void __launch_bounds__(THREADS, MT <= 2 ? 3 : 2) gemv_q4k_mma_kernel(View v, const float* __restrict__ x, int rows,
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

    const LaneConsts lc = lane_consts(t);
    uint8_t* ring = reinterpret_cast<uint8_t*>(scale_s + MT + (4 - MT % 4) % 4) + (size_t)warp * STAGES * SLOT_BYTES;
    const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring);

    // This warp's steps: super-blocks b = warp, warp + 8, ... of every tile of the CTA, in order.
    const int nb_w = warp < KB ? (KB - warp + WARPS - 1) / WARPS : 0;
    const int my_tiles = (int)blockIdx.x < tiles ? (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int steps = nb_w * my_tiles;

    // Requests step s into ring slot s % STAGES: lane (g, t) copies its 32 bytes of nibbles of rows g and
    // g + 8, lanes t = 0 / t = 1 also the 16-byte header of row g / g + 8. Rows past n repeat row n - 1.
    int iss_tile = blockIdx.x, iss_j = 0;  // tile and block counter of the next step to request
    auto issue = [&](int s) {
        if (s < steps) {
            int64_t r0 = (int64_t)iss_tile * 16 + g, r1 = r0 + 8;
            r0 = r0 < n ? r0 : n - 1;
            r1 = r1 < n ? r1 : n - 1;
            const uint32_t boff = (uint32_t)(warp + WARPS * iss_j) * 144u;
            const uint8_t* p0 = v.q + r0 * row_bytes + boff;
            const uint8_t* p1 = v.q + r1 * row_bytes + boff;
            const uint32_t slot = ring_s + (uint32_t)(s % STAGES) * SLOT_BYTES;
            const uint32_t d0 = slot + (uint32_t)g * 144u, d1 = d0 + 8u * 144u;
            const uint32_t lo = 16u + 32u * (uint32_t)t;
            cp_async16(d0 + lo, p0 + lo);
            cp_async16(d0 + lo + 16, p0 + lo + 16);
            cp_async16(d1 + lo, p1 + lo);
            cp_async16(d1 + lo + 16, p1 + lo + 16);
            if (t < 2) {
                cp_async16(t == 0 ? d0 : d1, t == 0 ? p0 : p1);
            }
            if (++iss_j == nb_w) {
                iss_j = 0;
                iss_tile += gridDim.x;
            }
        }
        cp_async_commit();
    };

    // The first weights are requested before the activations are prepared: they do not depend on x.
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
        issue(s);
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
    // Lanes whose column g is not stored (g >= NCOL) read another lane's fragment: their accumulator columns
    // belong to activation rows that do not exist and are never written out.
    const uint2* fb_lane = xf + (size_t)(NCOL == 8 ? g : g % NCOL) * 4 + t;

    auto compute = [&](const uint8_t* slot, int b) {
        const uint8_t* q0 = slot + g * 144;
        const uint8_t* q1 = q0 + 8 * 144;
        const uint4 h0 = lds16(q0), h1 = lds16(q1);
        const uint4 qa0 = lds16(q0 + 16 + 32 * t), qa1 = lds16(q0 + 32 + 32 * t);
        const uint4 qb0 = lds16(q1 + 16 + 32 * t), qb1 = lds16(q1 + 32 + 32 * t);
        const RowScales s0 = decode_scales(h0, lc), s1 = decode_scales(h1, lc);
        // CH independent accumulator chains per column group keep the tensor pipe from waiting on itself
        constexpr int CH = NG == 1 ? 4 : 2;
        float D[NG][CH][4], E[NG][4];
        const uint2* fb = fb_lane + (size_t)b * (FRAGS * NG * NCOL * 4);
        const uint32_t wa[8] = {qa0.x, qa0.y, qa0.z, qa0.w, qa1.x, qa1.y, qa1.z, qa1.w};
        const uint32_t wb[8] = {qb0.x, qb0.y, qb0.z, qb0.w, qb1.x, qb1.y, qb1.z, qb1.w};
#pragma unroll
        for (int w = 0; w < 8; w++) {
            const uint32_t va = wa[w], vb = wb[w], va8 = va >> 8, vb8 = vb >> 8;
#pragma unroll
            for (int hf = 0; hf < 2; hf++) {
                // hf = 0: low nibbles, sub-block 2t; hf = 1: high nibbles, sub-block 2t + 1.
                // Elements 4w + {0, 2} come from va, 4w + {1, 3} from va >> 8.
                const uint32_t mask = hf == 0 ? 0x000F000Fu : 0x00F000F0u;
                const __half2 sa = hf == 0 ? s0.s_lo : s0.s_hi, ca = hf == 0 ? s0.c_lo : s0.c_hi;
                const __half2 sb = hf == 0 ? s1.s_lo : s1.s_hi, cb = hf == 0 ? s1.c_lo : s1.c_hi;
                const uint32_t a0 = h2u(__hfma2(magic_pair(va, mask), sa, ca));
                const uint32_t a2 = h2u(__hfma2(magic_pair(va8, mask), sa, ca));
                const uint32_t a1 = h2u(__hfma2(magic_pair(vb, mask), sb, cb));
                const uint32_t a3 = h2u(__hfma2(magic_pair(vb8, mask), sb, cb));
                const int f = 2 * w + hf;
#pragma unroll
                for (int i = 0; i < NG; i++) {
                    const uint2 bf = fb[(f * NG + i) * NCOL * 4];
                    if (f < CH) {
                        mma16816_first(D[i][f % CH], a0, a1, a2, a3, bf.x, bf.y);
                    } else {
                        mma16816(D[i][f % CH], a0, a1, a2, a3, bf.x, bf.y);
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < NG; i++) {
            const uint2 bf = fb[(16 * NG + i) * NCOL * 4];
            mma16816_first(E[i], s0.mins, s1.mins, 0u, 0u, bf.x, bf.y);
            float d01, d23;
            if (CH == 4) {
                d01 = ((D[i][0][0] + D[i][1][0]) + (D[i][2][0] + D[i][3][0])) + ((D[i][0][1] + D[i][1][1]) + (D[i][2][1] + D[i][3][1]));
                d23 = ((D[i][0][2] + D[i][1][2]) + (D[i][2][2] + D[i][3][2])) + ((D[i][0][3] + D[i][1][3]) + (D[i][2][3] + D[i][3][3]));
            } else {
                d01 = (D[i][0][0] + D[i][1][0]) + (D[i][0][1] + D[i][1][1]);
                d23 = (D[i][0][2] + D[i][1][2]) + (D[i][0][3] + D[i][1][3]);
            }
            acc[i][0] += s0.d * d01 - s0.dmin * (E[i][0] + E[i][1]);
            acc[i][1] += s1.d * d23 - s1.dmin * (E[i][2] + E[i][3]);
        }
    };

    int parity = 0;
    int step = 0;
    for (int my_tile = blockIdx.x; my_tile < tiles; my_tile += gridDim.x) {
        for (int b = warp; b < KB; b += WARPS) {
            __syncwarp();                 // every lane is done reading the slot that is requested next
            issue(step + STAGES - 1);
            cp_async_wait<STAGES - 1>();  // this lane's copies of `step` have landed
            __syncwarp();                 // ... and so have the other lanes'
            compute(ring + (size_t)(step % STAGES) * SLOT_BYTES, b);
            step++;
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

constexpr size_t SMEM_MAX = 227 * 1024;

template <int MT, int STAGES>
size_t smem_bytes(int KB) {
    using C = Cfg<MT>;
    return (size_t)KB * frag_bytes_per_block<MT>() + (size_t)(2 * WARPS * 16 * C::MP + WARPS * MT + (MT + 3) / 4 * 4) * sizeof(float) +
           (size_t)WARPS * STAGES * SLOT_BYTES;
}

template <int MT, int STAGES>
int launch_q4k(const View& v, const float* x, int rows, const float* bias, float* y, cudaStream_t s) {
    const size_t smem = smem_bytes<MT, STAGES>((int)(v.k / 256));
    // the opt-in for more than 48 KB of dynamic shared memory is per device
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    JQ_CUDA(cudaGetDevice(&dev));
    if ((configured.load() >> (dev & 63) & 1) == 0) {
        JQ_CUDA(cudaFuncSetAttribute(gemv_q4k_mma_kernel<MT, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX));
        configured.fetch_or((uint64_t)1 << (dev & 63));
    }
    const int tiles = (int)((v.n + 15) / 16);
    const int per_sm = smem > SMEM_MAX / 2 - 1024 ? 1 : (MT <= 2 && smem <= SMEM_MAX / 3 - 1024 ? 3 : 2);
    const int grid = tiles < sm_count() * per_sm ? tiles : sm_count() * per_sm;
    gemv_q4k_mma_kernel<MT, STAGES><<<grid, THREADS, smem, s>>>(v, x, rows, bias, y, tiles);
    count_launch();
    return check_launch("gemv_q4k_mma_kernel");
}

template <int MT>
int run_q4k(const View& v, const float* x, int rows, const float* bias, float* y, cudaStream_t s, bool* handled) {
    const int KB = (int)(v.k / 256);
    const size_t half = SMEM_MAX / 2 - 1024;  // two CTAs per SM (1 KB each is reserved by the system)
    *handled = true;
    if (MT <= 2 && smem_bytes<MT, 2>(KB) <= SMEM_MAX / 3 - 1024) return launch_q4k<MT, 2>(v, x, rows, bias, y, s);
    if (smem_bytes<MT, 4>(KB) <= half) return launch_q4k<MT, 4>(v, x, rows, bias, y, s);
    if (smem_bytes<MT, 3>(KB) <= half) return launch_q4k<MT, 3>(v, x, rows, bias, y, s);
    if (smem_bytes<MT, 4>(KB) <= SMEM_MAX) return launch_q4k<MT, 4>(v, x, rows, bias, y, s);
    if (smem_bytes<MT, 2>(KB) <= SMEM_MAX) return launch_q4k<MT, 2>(v, x, rows, bias, y, s);
    *handled = false;  // the activations do not fit in shared memory in fragment form
    return JQ_OK;
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
