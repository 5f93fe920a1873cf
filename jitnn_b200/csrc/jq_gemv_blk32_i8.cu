// Decode GEMV for the formats with 32-element blocks and fp16 scales (Q8_0, Q4_0, Q4_1) on the integer tensor cores:
// y[m, n] = x[m, k] . W[n, k]^T (+ bias), m <= 2, k a multiple of 256.
//
// The scheme of the Q4_K kernel (jq_gemv_q4k_i8.cu) with what these formats need. The activations become an image
// first: per 256 values of k a power-of-two scale, 22-bit fixed point, three signed base-256 digits laid out as B
// fragments of mma.sync.m16n8k32, column 3m + i = digit i of row m of x (one warp per 256 values, image_kernel).
// The GEMV kernel streams 16 rows x 256 k at a time (8 blocks per row) through a per-warp cp.async ring:
//   Q8_0  the int8 quants are the A operand as they are (s8 x s8 -> s32), read with one ldmatrix per block;
//   Q4_0  one AND / one shift + AND per four weights widen the nibbles (u8 x s8); the offset, -8 * sum(x over the block),
//         is the same for every weight row, so the image carries the digit sums and it costs one FMA per value;
//   Q4_1  the same with + m * sum(x over the block) instead.
// One MMA multiplies one block of 16 weight rows with every digit column exactly; its four results per lane are
// converted to float and scaled by the block's fp16 d (the scale is a float, so it cannot be folded in integers as the
// K-quants' 6-bit scales are), summed over the 8 blocks and scaled once by the column weight s * 2^(8i - 21).
// Reference arithmetic: Quant.java:137-144,171-188 (Q8_0, bias inside the sum), GgufKernels.java:85-99 (Q4_0, Q4_1);
// results agree with it to FP32 accumulation accuracy (x keeps 22 bits relative to the largest of its 256 neighbours).
//
// Work split as in the Q4_K kernel: a CTA of 8 warps owns 16 output rows at a time, warp p takes the 256-blocks of k
// with index p (mod 8); per tile the warps' partial sums meet in shared memory in a fixed order that depends on k only
// (row shards are bitwise equal to the whole weight). Quant and scale planes are separate on the device
// (jq_formats.cuh); both are padded by 16 rows. Shared-memory rows are swizzled by (row & 7) so that ldmatrix's eight
// row reads fall into different banks.
#include "jq_formats.cuh"

namespace jq {

namespace {

constexpr int NW = 8;
constexpr int THREADS = NW * 32;
constexpr size_t SMEM_MAX = 227 * 1024;

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16_if(uint32_t dst_smem, const void* src, int on) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %2, 0;\n"
        "@p cp.async.cg.shared.global [%0], [%1], 16;\n"
        "}\n" ::"r"(dst_smem),
        "l"(src), "r"(on)
        : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <bool SIGNED_A>
__device__ __forceinline__ void imma_k32(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    if constexpr (SIGNED_A) {
        asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
    } else {
        asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
    }
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}

// Per format: bytes of quants and of scales per row of a 256-wide step, and the layout of a ring slot.
template <int TYPE>
struct Geo {
    static constexpr int QROW = TYPE == JQ_TYPE_Q8_0 ? 256 : 128;  // quant bytes per row and step (8 blocks)
    static constexpr int AROW = TYPE == JQ_TYPE_Q4_1 ? 32 : 16;    // scale bytes per row and step
    static constexpr int QC = QROW / 16, AC = AROW / 16;           // 16-byte chunks per row
    static constexpr int AUX_OFF = 16 * QROW;
    static constexpr int SLOT = 16 * (QROW + AROW);
    static constexpr int CHUNKS = 16 * (QC + AC);
    static constexpr int PER_LANE = (CHUNKS + 31) / 32;
};

// Image of one row group of x per 256 values of k: digit fragments of the 8 blocks (two blocks side by side per
// 16-byte cell), the sums of x over each block as floats (digit-weighted, per column), the column weights.
template <int MT>
struct Img {
    static constexpr int COLS = 3 * MT;
    static constexpr size_t XD = (size_t)4 * COLS * 4 * 16;  // 4 block pairs x columns x 4 lanes x 16 bytes
    static constexpr size_t XS = (size_t)8 * 8 * 4;          // 8 blocks x 8 columns x float (unused columns: 0)
    static constexpr size_t TAB = 8 * 4;
    static constexpr size_t PB = XD + XS + TAB;
    static_assert(PB % 16 == 0, "the image is copied in 16-byte pieces");
};

// One warp per (256 values of k, row of x). Lane = (block lane / 4, tt = lane % 4): the values 4tt..4tt+3 and
// 16+4tt..16+4tt+3 of the block, which are the k-slots of that lane in the MMA's B fragment when the A fragment holds
// the block's 32 quants in their natural order.
constexpr int PREP_WARPS = 4;
template <int MT>
__global__ void __launch_bounds__(PREP_WARPS * 32) blk32_image_kernel(const float* __restrict__ x, int rows, int64_t k, uint8_t* __restrict__ image) {
    using I = Img<MT>;
    asm volatile("griddepcontrol.launch_dependents;");  // the GEMV kernel may start requesting weights now
    asm volatile("griddepcontrol.wait;" ::: "memory");  // x is complete, and the GEMV before this one is done with the scratch image
    const int lane = threadIdx.x & 31;
    const int pair = blockIdx.x * PREP_WARPS + (threadIdx.x >> 5);
    const int b = pair / MT, m = pair % MT;
    if (b >= (int)(k >> 8)) {
        return;
    }
    const int blk = lane >> 2, tt = lane & 3;
    uint8_t* img = image + (size_t)b * I::PB;
    uint2* xd = reinterpret_cast<uint2*>(img);
    float* xs = reinterpret_cast<float*>(img + I::XD);
    float* tab = reinterpret_cast<float*>(img + I::XD + I::XS);
    if (m == 0 && lane >= I::COLS && lane < 8) {
        tab[lane] = 0.0f;  // columns that hold no row of x
#pragma unroll
        for (int j = 0; j < 8; j++) {
            xs[j * 8 + lane] = 0.0f;
        }
    }
    float xv[8];
    if (m < rows) {
        const float* xb = x + (int64_t)m * k + (int64_t)b * 256 + blk * 32 + 4 * tt;
        const float4 lo = __ldg(reinterpret_cast<const float4*>(xb)), hi = __ldg(reinterpret_cast<const float4*>(xb + 16));
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
    // s = 2^floor(log2(amax)): the largest |x| / s of the 256 values lies in [1, 2)
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
        xd[((((size_t)(blk >> 1)) * I::COLS + col) * 4 + tt) * 2 + (blk & 1)] = make_uint2(w0, w1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if (tt == 0) {
            xs[blk * 8 + col] = (float)sum;  // |sum| <= 32 * 128: exact
        }
        if (lane == 0) {
            tab[col] = m >= rows ? 0.0f : (bad ? __uint_as_float(0x7fc00000u) : __uint_as_float(e + ((uint32_t)(8 * dgt) << 23) - (21u << 23)));  // s * 2^(8 dgt - 21)
        }
    }
}

template <int TYPE, int MT, int STAGES>
__global__ void __launch_bounds__(THREADS, 2) gemv_blk32_i8_kernel(View v, const uint8_t* __restrict__ image, int rows, const float* __restrict__ bias,
                                                                   float* __restrict__ y, int tiles) {
    using G = Geo<TYPE>;
    using I = Img<MT>;
    constexpr int COLS = I::COLS;
    constexpr uint32_t RING_BYTES = STAGES * G::SLOT;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int KB = (int)(v.k >> 8);
    uint8_t* img = smem_raw;                                              // [KB][PB]
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)KB * I::PB);  // [2][NW][16][MT]
    uint8_t* ring = reinterpret_cast<uint8_t*>(red + 2 * NW * 16 * MT) + (size_t)warp * RING_BYTES;
    const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring);
    const int64_t qrow = (int64_t)KB * G::QROW, arow = (int64_t)KB * G::AROW;  // plane bytes per weight row

    // ---- weight stream: chunk c = lane + 32 i of a slot's chunks (quant chunks of the 16 rows, then their scale chunks) ----
    uint32_t src_off[G::PER_LANE], dst_off[G::PER_LANE];
    bool is_aux[G::PER_LANE], live[G::PER_LANE];
#pragma unroll
    for (int i = 0; i < G::PER_LANE; i++) {
        const int c = lane + 32 * i;
        live[i] = c < G::CHUNKS;
        is_aux[i] = c >= 16 * G::QC;
        if (!is_aux[i]) {
            const int r = c / G::QC, ch = c % G::QC;
            src_off[i] = (uint32_t)(r * (int)qrow + ch * 16);
            dst_off[i] = (uint32_t)(r * G::QROW + (((ch & 8) | ((ch & 7) ^ (r & 7))) << 4));
        } else {
            const int ca = c - 16 * G::QC, r = ca / G::AC, ch = ca % G::AC;
            src_off[i] = (uint32_t)(r * (int)arow + ch * 16);
            dst_off[i] = (uint32_t)(G::AUX_OFF + r * G::AROW + ch * 16);
        }
    }
    const int nb = warp < KB ? (KB - warp + NW - 1) / NW : 0;
    const int my_tiles = (int)blockIdx.x < tiles ? (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    int iss_left = nb * my_tiles, iss_ti = 0, iss_j = 0;
    uint32_t iss_slot = 0;
    auto issue = [&]() {
        if (iss_left > 0) {
            iss_left--;
            const int tile = (int)blockIdx.x + iss_ti * (int)gridDim.x;
            const int sb = warp + NW * iss_j;
            const uint8_t* qb = v.q + (int64_t)tile * 16 * qrow + (int64_t)sb * G::QROW;
            const uint8_t* ab = v.aux + (int64_t)tile * 16 * arow + (int64_t)sb * G::AROW;
            const uint32_t slot = ring_s + iss_slot;
#pragma unroll
            for (int i = 0; i < G::PER_LANE; i++) {
                cp_async16_if(slot + dst_off[i], (is_aux[i] ? ab : qb) + src_off[i], live[i]);
            }
            if (++iss_j == nb) {
                iss_j = 0;
                iss_ti++;
            }
        }
        iss_slot = iss_slot + G::SLOT == RING_BYTES ? 0u : iss_slot + G::SLOT;
        cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
        issue();  // the first weights are on their way before the activation image is complete
    }

    asm volatile("griddepcontrol.wait;" ::: "memory");  // the image kernel has finished
    {
        const uint32_t img_s = (uint32_t)__cvta_generic_to_shared(img);
        const int chunks = (int)((size_t)KB * I::PB / 16);
        for (int c = tid; c < chunks; c += THREADS) {
            cp_async16(img_s + (uint32_t)c * 16u, image + (size_t)c * 16);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
    }

    // Lanes whose column is not stored read another lane's fragment; those columns have weight zero.
    const uint8_t* xd_lane = img + ((size_t)(g % COLS) * 4 + t) * 16;
    const uint8_t* xs_lane = img + I::XD + (size_t)(2 * t) * 4;
    const uint8_t* tab_lane = img + I::XD + I::XS + (size_t)(2 * t) * 4;
    // ldmatrix row addresses inside a slot. Q8_0 (x4): matrices = (rows 0-7 | 8-15) x (bytes 0-15 | 16-31) of a block;
    // Q4_0 / Q4_1 (x2): matrices = rows 0-7 | 8-15 of the block's 16 bytes. Chunks are swizzled by (row & 7).
    const int lrow = TYPE == JQ_TYPE_Q8_0 ? (lane & 7) + 8 * ((lane >> 3) & 1) : (lane & 15);
    const uint32_t lrow_off = (uint32_t)(lrow * G::QROW);
    float acc[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};  // [row g / g + 8][column 2t / 2t + 1]

    auto compute = [&](uint32_t slot_s, const uint8_t* slot, const uint8_t* blk) {
        // fp16 scales of the 8 blocks of rows g and g + 8
        uint32_t d0w[8], d1w[8];  // Q8_0 / Q4_0: word j = blocks 2j, 2j+1 (d); Q4_1: word j = block j (d, m)
        {
            const uint4 a = *reinterpret_cast<const uint4*>(slot + G::AUX_OFF + g * G::AROW);
            const uint4 b = *reinterpret_cast<const uint4*>(slot + G::AUX_OFF + (g + 8) * G::AROW);
            d0w[0] = a.x; d0w[1] = a.y; d0w[2] = a.z; d0w[3] = a.w;
            d1w[0] = b.x; d1w[1] = b.y; d1w[2] = b.z; d1w[3] = b.w;
            if constexpr (TYPE == JQ_TYPE_Q4_1) {
                const uint4 a2 = *reinterpret_cast<const uint4*>(slot + G::AUX_OFF + g * G::AROW + 16);
                const uint4 b2 = *reinterpret_cast<const uint4*>(slot + G::AUX_OFF + (g + 8) * G::AROW + 16);
                d0w[4] = a2.x; d0w[5] = a2.y; d0w[6] = a2.z; d0w[7] = a2.w;
                d1w[4] = b2.x; d1w[5] = b2.y; d1w[6] = b2.z; d1w[7] = b2.w;
            }
        }
        float f[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};
#pragma unroll
        for (int p = 0; p < 4; p++) {
            const uint4 bf = *reinterpret_cast<const uint4*>(blk + (size_t)p * COLS * 64);  // B operands of blocks 2p and 2p + 1
#pragma unroll
            for (int hf = 0; hf < 2; hf++) {
                const int j = 2 * p + hf;
                uint32_t a0, a1, a2, a3;
                if constexpr (TYPE == JQ_TYPE_Q8_0) {
                    uint32_t r[4];
                    const int ch = 2 * j + (lane >> 4);
                    ldmatrix_x4(r, slot_s + lrow_off + (uint32_t)(((ch & 8) | ((ch & 7) ^ (lrow & 7))) << 4));
                    a0 = r[0]; a1 = r[1]; a2 = r[2]; a3 = r[3];
                } else {
                    uint32_t r[2];
                    ldmatrix_x2(r, slot_s + lrow_off + (uint32_t)((j ^ (lrow & 7)) << 4));
                    a0 = r[0] & 0x0f0f0f0fu; a2 = (r[0] >> 4) & 0x0f0f0f0fu;  // elements 4t.. (low nibbles), 16 + 4t.. (high nibbles)
                    a1 = r[1] & 0x0f0f0f0fu; a3 = (r[1] >> 4) & 0x0f0f0f0fu;
                }
                int D[4];
                imma_k32<TYPE == JQ_TYPE_Q8_0>(D, a0, a1, a2, a3, hf == 0 ? bf.x : bf.z, hf == 0 ? bf.y : bf.w);
                float dd0, dd1;
                if constexpr (TYPE == JQ_TYPE_Q4_1) {
                    dd0 = half_bits_to_float(d0w[j]);
                    dd1 = half_bits_to_float(d1w[j]);
                } else {
                    dd0 = half_bits_to_float(d0w[j >> 1] >> (16 * (j & 1)));
                    dd1 = half_bits_to_float(d1w[j >> 1] >> (16 * (j & 1)));
                }
                float v0 = (float)D[0], v1 = (float)D[1], v2 = (float)D[2], v3 = (float)D[3];
                if constexpr (TYPE == JQ_TYPE_Q4_0) {
                    const float2 sx = *reinterpret_cast<const float2*>(xs_lane + (size_t)(blk - xd_lane) + j * 32);  // sums of x, columns 2t, 2t+1
                    v0 = fmaf(-8.0f, sx.x, v0); v1 = fmaf(-8.0f, sx.y, v1);  // exact: small integers
                    v2 = fmaf(-8.0f, sx.x, v2); v3 = fmaf(-8.0f, sx.y, v3);
                }
                f[0][0] = fmaf(dd0, v0, f[0][0]); f[0][1] = fmaf(dd0, v1, f[0][1]);
                f[1][0] = fmaf(dd1, v2, f[1][0]); f[1][1] = fmaf(dd1, v3, f[1][1]);
                if constexpr (TYPE == JQ_TYPE_Q4_1) {
                    const float2 sx = *reinterpret_cast<const float2*>(xs_lane + (size_t)(blk - xd_lane) + j * 32);
                    const float m0 = half_bits_to_float(d0w[j] >> 16), m1 = half_bits_to_float(d1w[j] >> 16);
                    f[0][0] = fmaf(m0, sx.x, f[0][0]); f[0][1] = fmaf(m0, sx.y, f[0][1]);
                    f[1][0] = fmaf(m1, sx.x, f[1][0]); f[1][1] = fmaf(m1, sx.y, f[1][1]);
                }
            }
        }
        const float2 w = *reinterpret_cast<const float2*>(tab_lane + (size_t)(blk - xd_lane));  // weights of columns 2t, 2t+1
        acc[0][0] = fmaf(w.x, f[0][0], acc[0][0]); acc[0][1] = fmaf(w.y, f[0][1], acc[0][1]);
        acc[1][0] = fmaf(w.x, f[1][0], acc[1][0]); acc[1][1] = fmaf(w.y, f[1][1], acc[1][1]);
    };

    int parity = 0;
    uint32_t cmp_slot = 0;
    for (int ti = 0; ti < my_tiles; ti++) {
        const int my_tile = (int)blockIdx.x + ti * (int)gridDim.x;
        const uint8_t* blk = xd_lane + (size_t)warp * I::PB;
        for (int j = 0; j < nb; j++) {
            __syncwarp();                 // every lane is done reading the slot that is requested next
            issue();
            cp_async_wait<STAGES - 1>();  // this lane's copies of this step have landed
            __syncwarp();                 // ... and so have the other lanes'
            compute(ring_s + cmp_slot, ring + cmp_slot, blk);
            cmp_slot = cmp_slot + G::SLOT == RING_BYTES ? 0u : cmp_slot + G::SLOT;
            blk += (size_t)NW * I::PB;
        }
        // combine the digit columns of a row of x, which sit in the 4 lanes of a quad
        float* rd = red + (size_t)parity * NW * 16 * MT;
#pragma unroll
        for (int m = 0; m < MT; m++) {
            float p0 = 0.0f, p1 = 0.0f;
#pragma unroll
            for (int c = 0; c < 2; c++) {
                const int col = 2 * t + c;
                const bool mine = col < COLS && col / 3 == m;
                p0 += mine ? acc[0][c] : 0.0f;
                p1 += mine ? acc[1][c] : 0.0f;
            }
            p0 += __shfl_xor_sync(0xffffffffu, p0, 1);
            p1 += __shfl_xor_sync(0xffffffffu, p1, 1);
            p0 += __shfl_xor_sync(0xffffffffu, p0, 2);
            p1 += __shfl_xor_sync(0xffffffffu, p1, 2);
            if (t == 0) {
                rd[(warp * 16 + g) * MT + m] = p0;
                rd[(warp * 16 + g + 8) * MT + m] = p1;
            }
        }
        acc[0][0] = acc[0][1] = acc[1][0] = acc[1][1] = 0.0f;
        __syncthreads();
        for (int o = tid; o < 16 * MT; o += THREADS) {
            const int r = o / MT, m = o % MT;
            const int64_t row = (int64_t)my_tile * 16 + r;
            const float* p = rd + o;
            constexpr int W = 16 * MT;
            const float sum = ((p[0] + p[W]) + (p[2 * W] + p[3 * W])) + ((p[4 * W] + p[5 * W]) + (p[6 * W] + p[7 * W]));
            if (m < rows && row < v.n) {
                y[(int64_t)m * v.n + row] = sum + (bias != nullptr ? bias[row] : 0.0f);
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

template <int TYPE, int MT>
int run(const View& v, const float* x, int rows, const float* bias, float* y, cudaStream_t s, uint8_t* image, bool* handled) {
    constexpr int STAGES = TYPE == JQ_TYPE_Q8_0 ? 2 : 3;
    const int KB = (int)(v.k / 256);
    const int tiles = (int)((v.n + 15) / 16);
    const size_t smem = (size_t)KB * Img<MT>::PB + (size_t)(2 * NW * 16 * MT) * sizeof(float) + (size_t)NW * STAGES * Geo<TYPE>::SLOT;
    if (smem > SMEM_MAX / 2 - 1024) {
        *handled = false;  // the image of the whole k does not fit beside the ring
        return JQ_OK;
    }
    *handled = true;
    static std::atomic<uint64_t> configured{0};  // the opt-in for large dynamic shared memory is per device
    int dev = 0;
    JQ_CUDA(cudaGetDevice(&dev));
    if ((configured.load() >> (dev & 63) & 1) == 0) {
        JQ_CUDA(cudaFuncSetAttribute(gemv_blk32_i8_kernel<TYPE, MT, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX));
        configured.fetch_or((uint64_t)1 << (dev & 63));
    }
    // launched programmatically as well: it is scheduled while the kernel before it still runs (it waits for that kernel
    // before touching memory) and lets the GEMV behind it be scheduled at once
    cudaLaunchConfig_t icfg = {};
    cudaLaunchAttribute iattr[1];
    iattr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    iattr[0].val.programmaticStreamSerializationAllowed = 1;
    icfg.attrs = iattr;
    icfg.numAttrs = 1;
    icfg.stream = s;
    icfg.gridDim = dim3((unsigned)((KB * MT + PREP_WARPS - 1) / PREP_WARPS));
    icfg.blockDim = dim3(PREP_WARPS * 32);
    JQ_CUDA(cudaLaunchKernelEx(&icfg, blk32_image_kernel<MT>, x, rows, (int64_t)v.k, image));
    count_launch();
    const int grid = tiles < sm_count() * 2 ? tiles : sm_count() * 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // may start while the image kernel runs
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    JQ_CUDA(cudaLaunchKernelEx(&cfg, gemv_blk32_i8_kernel<TYPE, MT, STAGES>, v, (const uint8_t*)image, rows, bias, y, tiles));
    count_launch();
    return JQ_OK;
}

template <int TYPE>
int by_rows(const View& v, const float* x, int rows, const float* bias, float* y, cudaStream_t s, uint8_t* image, bool* handled) {
    if (rows == 1) return run<TYPE, 1>(v, x, rows, bias, y, s, image, handled);
    return run<TYPE, 2>(v, x, rows, bias, y, s, image, handled);
}

}  // namespace

// Bytes of scratch (activation image) the kernel needs; 0 if the shape is not handled.
size_t gemv_blk32_i8_scratch_bytes(int type, int64_t k, int rows) {
    if ((type != JQ_TYPE_Q8_0 && type != JQ_TYPE_Q4_0 && type != JQ_TYPE_Q4_1) || rows < 1 || rows > 2 || k <= 0 || k % 256 != 0) {
        return 0;
    }
    return (size_t)(k / 256) * (rows == 1 ? Img<1>::PB : Img<2>::PB);
}

// Q8_0, Q4_0, Q4_1 with rows in [1, 2] and k a multiple of 256, on a weight whose planes are padded by 16 rows.
// *handled = false leaves the call to another kernel.
int launch_gemv_blk32_i8(const View& v, const float* x, int rows, const float* bias, float* y, cudaStream_t s, uint8_t* image, bool* handled) {
    *handled = false;
    if (gemv_blk32_i8_scratch_bytes(v.type, v.k, rows) == 0 || v.n == 0 || v.aux == nullptr || image == nullptr ||
        (int64_t)16 * (v.k / 256) * 256 >= ((int64_t)1 << 31)) {
        return JQ_OK;
    }
    switch (v.type) {
        case JQ_TYPE_Q8_0: return by_rows<JQ_TYPE_Q8_0>(v, x, rows, bias, y, s, image, handled);
        case JQ_TYPE_Q4_0: return by_rows<JQ_TYPE_Q4_0>(v, x, rows, bias, y, s, image, handled);
        default: return by_rows<JQ_TYPE_Q4_1>(v, x, rows, bias, y, s, image, handled);
    }
}

}  // namespace jq
