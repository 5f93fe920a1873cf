// Decode GEMV for Q6_K with integer tensor-core arithmetic: y[m, n] = x[m, k] . W[n, k]^T, m <= 4 per pass.
//
// Same scheme as the Q4_K kernel (jq_gemv_q4k_i8.cu): a first kernel turns the activations into an "activation image"
// (per 256-element super-block of k and row of x: power-of-two scale, 22-bit fixed point, three signed base-256 digits
// laid out as MMA B fragments), the GEMV kernel streams the weights through a per-warp cp.async ring and multiplies with
// mma.sync on the integer tensor cores, exactly, converting to float once per super-block.
// What differs for Q6_K (device layout: 208 bytes per super-block = 128 bytes of low nibbles ql, 64 bytes of high bit
// pairs qh, 16 signed 8-bit scales; fp16 d in a separate plane):
//   * a scale covers 16 elements, so one mma.sync.m16n8k16 (u8 x s8 -> s32) handles one scale group of 16 weight rows;
//     its A operand is (ql nibble) | (qh bit pair << 4), built per four weights with two or three logic operations;
//   * the quants are unsigned 0..63 with an offset of 32: the term -32 * sum(x digits of the group) does not depend on
//     the weight row, so the image carries it as the C operand of the MMA;
//   * group results are combined with the int8 scales by integer multiply-add (the sum over 16 groups stays below
//     2^31), converted to float once per super-block and scaled by fp16 d and the column weight;
//   * the A fragments are read with ldmatrix: lane (g, t) needs word t of a 16-byte chunk of rows g and g + 8, which
//     is exactly ldmatrix's distribution, and the 208-byte row pitch makes those reads conflict free.
// The summation order depends on k only: a row shard of a weight gives bitwise the same outputs as the whole weight.
#include <mutex>

#include "jq_formats.cuh"
#include "jq_q6k_image.cuh"
#include "jq_tc.cuh"

namespace jq {

using q6k::Cfg;
using q6k::build_image;

namespace {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int ROW_BYTES = 208;                       // one super-block of one row in the quant plane
constexpr int SLOT_D = 16 * ROW_BYTES;               // behind the 16 rows: their 16 fp16 d
constexpr int SLOT_BYTES = SLOT_D + 16 * 2;
static_assert(SLOT_BYTES % 16 == 0 && SLOT_D % 16 == 0, "bulk copies move multiples of 16 bytes to 16-byte aligned addresses");
constexpr size_t SMEM_MAX = 227 * 1024;

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Byte i (0..3) of a word as a sign-extended integer.
__device__ __forceinline__ int signed_byte(uint32_t w, int i) {
    // one byte permute: byte i below three copies of its sign (a selector digit of 8 + i replicates the byte's top bit)
    // (prmt in PTX: the __byte_perm intrinsic only honours the three low bits of a selector digit)
    const uint32_t s = (uint32_t)(8 + i);
    int r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(0u), "r"((uint32_t)i | (s << 4) | (s << 8) | (s << 12)));
    return r;
}

// The same copies under a predicate, without a branch around them.
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
__device__ __forceinline__ void cp_async4_if(uint32_t dst_smem, const void* src, int on) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %2, 0;\n"
        "@p cp.async.ca.shared.global [%0], [%1], 4;\n"
        "}\n" ::"r"(dst_smem),
        "l"(src), "r"(on)
        : "memory");
}

// D = A(16x16 u8) * B(16x8 s8) + C, C given per column pair (the same for rows g and g + 8).
__device__ __forceinline__ void imma_k16(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0, int c0, int c1) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%7,%8};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(c0), "r"(c1));
}

// Four 8x8 matrices of 16-bit elements: register i of lane (g, t) = the 4 bytes at byte offset 4t of row g of matrix i,
// whose 8 row addresses come from lanes 8i .. 8i + 7.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// ---- activations -> image (scratch buffer in global memory) ---------------------------------------------------
// One warp per (super-block of k, row of x).
constexpr int PREP_WARPS = 4;
__device__ int g_q6k_status;  // 0, or 25 once a wait for the weight ring has given up

template <int MT>
__global__ void __launch_bounds__(PREP_WARPS * 32) q6k_activation_image_kernel(const float* __restrict__ x, int rows, int64_t k,
                                                                             uint8_t* __restrict__ image) {
    asm volatile("griddepcontrol.launch_dependents;");  // the GEMV kernel may start requesting weights now
    asm volatile("griddepcontrol.wait;" ::: "memory");  // x is complete, and the GEMV before this one is done with the scratch image
    const int pair = blockIdx.x * PREP_WARPS + (threadIdx.x >> 5);
    const int b = pair / MT, m = pair % MT;
    if (b < (int)(k >> 8)) {
        build_image<MT>(m < rows ? x + (int64_t)m * k + (int64_t)b * 256 : nullptr, m, image + (size_t)b * Cfg<MT>::PB, threadIdx.x & 31);
    }
}

// ---- the GEMV ---------------------------------------------------------------------------------------------------
template <int MT, int STAGES, int OCC>
__global__ void __launch_bounds__(THREADS, OCC) gemv_q6k_i8_kernel(View v, const uint8_t* __restrict__ image, int rows,
                                                                  const float* __restrict__ bias, float* __restrict__ y, int tiles,
                                                                  int KS, int max_tiles, long long wait_clocks) {
    // KS = super-blocks of k per slice: the activation image of one slice is resident in shared memory at a time;
    // with more than one slice the per-tile sums are carried in shared memory (max_tiles tiles per CTA).
    using C = Cfg<MT>;
    constexpr int NG = C::NG, NCOL = C::NCOL;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    asm volatile("griddepcontrol.launch_dependents;");  // the kernel after this one may be scheduled as room becomes free
    const int KB = (int)(v.k >> 8);
    const int nslices = (KB + KS - 1) / KS;
    constexpr int BAR_BYTES = WARPS * STAGES * 8;                                    // one mbarrier per slot
    static_assert(BAR_BYTES % 16 == 0, "what follows the barriers stays 16-byte aligned");
    uint8_t* img = smem_raw + BAR_BYTES;                                             // [KS][PB]
    float* red = reinterpret_cast<float*>(img + (size_t)KS * C::PB);                 // [2][WARPS][16][MT]
    float* carry = red + 2 * WARPS * 16 * MT;                                        // [max_tiles][16][MT], only if nslices > 1
    uint8_t* ring = reinterpret_cast<uint8_t*>(carry + (nslices > 1 ? (size_t)max_tiles * 16 * MT : 0)) +
                    (size_t)(threadIdx.x >> 5) * STAGES * SLOT_BYTES;
    const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int64_t n = v.n;
    const uint32_t bars_s = tc::smem_u32(smem_raw) + (uint32_t)(warp * STAGES * 8);  // this warp's barriers

    // ---- weight stream: the planes hold their blocks tile by tile (jq_common.cuh), so the 16 rows of a tile of this kernel and
    // one super-block are 16 x 208 contiguous bytes of the quant plane and 32 of the d plane: two bulk copies per step,
    // requested by lane 0, complete when the slot's barrier says so. A slot holds the rows at their pitch of 208 bytes.
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) {
            tc::mbar_init(bars_s + 8 * s, 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");  // the copy engine sees initialised barriers
    }
    __syncwarp();
    // This warp's steps, in order: for every slice, for every tile of the CTA, the super-blocks b = slice start + warp + 8 i.
    const int len_last = KB - (nslices - 1) * KS;
    const int nb_full = nslices > 1 ? (warp < KS ? (KS - warp + WARPS - 1) / WARPS : 0) : 0;
    const int nb_last = warp < len_last ? (len_last - warp + WARPS - 1) / WARPS : 0;
    const int my_tiles = (int)blockIdx.x < tiles ? (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    int iss_left = ((nslices - 1) * nb_full + nb_last) * my_tiles;
    int iss_sl = 0, iss_ti = 0, iss_j = 0, iss_nb = nslices > 1 ? nb_full : nb_last;
    int iss_slot = 0;
    constexpr uint32_t RING_BYTES = STAGES * SLOT_BYTES;
    // position, among the blocks of a plane, of row 0 of the tile and the block that is requested next
    auto step_index = [&]() {
        const int tile = (int)blockIdx.x + iss_ti * (int)gridDim.x;
        return ((int64_t)(tile >> 3) * KB + (iss_sl * KS + warp + WARPS * iss_j)) * TILE_ROWS + (tile & 7) * 16;
    };
    auto issue = [&]() {  // every lane keeps the bookkeeping, lane 0 makes the requests
        if (iss_left > 0) {
            iss_left--;
            if (lane == 0) {
                const int64_t at = step_index();
                const uint32_t bar = bars_s + 8 * iss_slot, slot = ring_s + iss_slot * SLOT_BYTES;
                tc::mbar_expect_tx(bar, SLOT_BYTES);
                tc::bulk_load(slot, v.q + at * ROW_BYTES, SLOT_D, bar);
                tc::bulk_load(slot + SLOT_D, v.aux + at * 2, 32, bar);
            }
            if (++iss_j == iss_nb) {
                iss_j = 0;
                if (++iss_ti == my_tiles) {
                    iss_ti = 0;
                    iss_sl++;
                    iss_nb = iss_sl == nslices - 1 ? nb_last : nb_full;
                }
            }
        }
        iss_slot = iss_slot + 1 == STAGES ? 0 : iss_slot + 1;
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
        issue();  // the first weights are on their way before the activation image is complete
    }

    // ---- the activation image is complete once the kernel that writes it has finished ----------------------------
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t img_s = (uint32_t)__cvta_generic_to_shared(img);

    // ---- main loop ----------------------------------------------------------------------------------------------
    // Lanes whose column is not stored read another lane's fragment; those columns have weight zero.
    const uint8_t* xd_lane = img + ((size_t)(NCOL == 8 ? g : g % NCOL) * 4 + t) * 16;  // B operands of four groups per 16 bytes
    const uint8_t* xc_lane = img + C::XD + (size_t)t * 16;                              // C operands of two groups per 16 bytes
    const uint8_t* tab_lane = img + C::XD + C::XC;
    // ldmatrix row address of this lane inside a slot: matrix lane / 8 covers rows 8 (matrix % 2) .. + 7 and
    // chunk (matrix / 2) of a chunk pair
    const uint32_t ldm_off = (uint32_t)(((lane & 7) + 8 * ((lane >> 3) & 1)) * ROW_BYTES + (lane >> 4) * 16);
    float acc[NG][2][2];   // [group][row g / g + 8][column 2t / 2t + 1]
#pragma unroll
    for (int i = 0; i < NG; i++) {
        acc[i][0][0] = acc[i][0][1] = acc[i][1][0] = acc[i][1][1] = 0.0f;
    }

    auto compute = [&](const uint8_t* slot, uint32_t slot_s, int b, int tile, int blk) {  // b = index inside the resident slice
        int I[NG][4];
#pragma unroll
        for (int i = 0; i < NG; i++) {
            I[i][0] = I[i][1] = I[i][2] = I[i][3] = 0;
        }
        // the 16 signed scales of rows g and g + 8
        const uint4 sv0 = *reinterpret_cast<const uint4*>(slot + g * ROW_BYTES + 192);
        const uint4 sv1 = *reinterpret_cast<const uint4*>(slot + (g + 8) * ROW_BYTES + 192);
        const uint32_t sc0[4] = {sv0.x, sv0.y, sv0.z, sv0.w}, sc1[4] = {sv1.x, sv1.y, sv1.z, sv1.w};
        const uint8_t* bx = xd_lane + (size_t)b * C::PB;
        const uint8_t* bc = xc_lane + (size_t)b * C::PB;
#pragma unroll
        for (int n = 0; n < 2; n++) {
            // high bit pairs of half n: registers {row g, row g+8} x {elements 0-15, 16-31}
            uint32_t qh[4];
            ldmatrix_x4(qh, slot_s + ldm_off + (uint32_t)(8 + 2 * n) * 16u);
            // B operands of the half's eight groups: two 16-byte loads per column group
            uint32_t bq[NG][8];
#pragma unroll
            for (int i = 0; i < NG; i++) {
#pragma unroll
                for (int q = 0; q < 2; q++) {
                    const uint4 bw = *reinterpret_cast<const uint4*>(bx + (size_t)(((2 * n + q) * NG + i) * NCOL) * 64);
                    bq[i][4 * q] = bw.x; bq[i][4 * q + 1] = bw.y; bq[i][4 * q + 2] = bw.z; bq[i][4 * q + 3] = bw.w;
                }
            }
#pragma unroll
            for (int h = 0; h < 2; h++) {
                // low nibbles: bytes 64 n + 32 h + l; their low nibble is sub-block kk = h, their high nibble kk = h + 2
                uint32_t ql[4];
                ldmatrix_x4(ql, slot_s + ldm_off + (uint32_t)(4 * n + 2 * h) * 16u);
#pragma unroll
                for (int hi = 0; hi < 2; hi++) {
                    const int kk = h + 2 * hi;
                    // C operands of the pair of groups 8n + 2kk, + 1: one 16-byte load per column group
                    int4 cq[NG];
#pragma unroll
                    for (int i = 0; i < NG; i++) {
                        cq[i] = *reinterpret_cast<const int4*>(bc + (size_t)(((4 * n + kk) * NG + i) * 4) * 16);
                    }
#pragma unroll
                    for (int cp = 0; cp < 2; cp++) {
                        const int gi = 8 * n + 2 * kk + cp;  // scale group = elements 16 gi .. 16 gi + 15
                        const uint32_t la = hi == 0 ? ql[2 * cp] : ql[2 * cp] >> 4, lb = hi == 0 ? ql[2 * cp + 1] : ql[2 * cp + 1] >> 4;
                        const uint32_t ha = kk == 0 ? qh[2 * cp] << 4 : (kk == 1 ? qh[2 * cp] << 2 : (kk == 2 ? qh[2 * cp] : qh[2 * cp] >> 2));
                        const uint32_t hb = kk == 0 ? qh[2 * cp + 1] << 4
                                                    : (kk == 1 ? qh[2 * cp + 1] << 2 : (kk == 2 ? qh[2 * cp + 1] : qh[2 * cp + 1] >> 2));
                        const uint32_t a0 = and_or(ha, 0x30303030u, la & 0x0f0f0f0fu);
                        const uint32_t a1 = and_or(hb, 0x30303030u, lb & 0x0f0f0f0fu);
                        // sign-extended scale byte gi
                        const int s0 = signed_byte(sc0[gi >> 2], gi & 3);
                        const int s1 = signed_byte(sc1[gi >> 2], gi & 3);
#pragma unroll
                        for (int i = 0; i < NG; i++) {
                            int D[4];
                            imma_k16(D, a0, a1, bq[i][2 * kk + cp], cp == 0 ? cq[i].x : cq[i].z, cp == 0 ? cq[i].y : cq[i].w);
                            I[i][0] += s0 * D[0];
                            I[i][1] += s0 * D[1];
                            I[i][2] += s1 * D[2];
                            I[i][3] += s1 * D[3];
                        }
                    }
                }
            }
        }
        // fp16 d of rows g and g + 8
        const float d0 = half_bits_to_float(*reinterpret_cast<const uint16_t*>(slot + SLOT_D + 2 * g));
        const float d1 = half_bits_to_float(*reinterpret_cast<const uint16_t*>(slot + SLOT_D + 2 * (g + 8)));
        const uint8_t* tb = tab_lane + (size_t)b * C::PB;
#pragma unroll
        for (int i = 0; i < NG; i++) {
            const float2 w = *reinterpret_cast<const float2*>(tb + (8 * i + 2 * t) * 4);  // weights of columns 2t, 2t+1
            acc[i][0][0] = fmaf(d0 * w.x, (float)I[i][0], acc[i][0][0]);
            acc[i][0][1] = fmaf(d0 * w.y, (float)I[i][1], acc[i][0][1]);
            acc[i][1][0] = fmaf(d1 * w.x, (float)I[i][2], acc[i][1][0]);
            acc[i][1][1] = fmaf(d1 * w.y, (float)I[i][3], acc[i][1][1]);
        }
    };

    // activation row each accumulator column of this lane belongs to (-1: none)
    int mq[NG][2];
#pragma unroll
    for (int i = 0; i < NG; i++) {
#pragma unroll
        for (int c = 0; c < 2; c++) {
            const int col = 8 * i + 2 * t + c;
            mq[i][c] = col < C::COLS ? col / 3 : -1;
        }
    }

    int parity = 0;
    int cmp_slot = 0;
    uint32_t cmp_phase = 0;
    bool gave_up = false;  // a wait for weights ran out: the status word says so, the warp stops waiting and finishes with whatever is there
    for (int sl = 0; sl < nslices; sl++) {
        // ---- bring this slice of the activation image into shared memory ---------------------------------------------
        const int len = (KB - sl * KS) < KS ? (KB - sl * KS) : KS;
        if (sl > 0) {
            __syncthreads();  // every warp is done with the previous slice
        }
        if (nslices == 1) {
            // one slice: a warp only ever reads the image of its own super-blocks, so it fetches just those and waits for
            // nobody else (the wait also covers the weight stages requested so far, which it needs next anyway)
            constexpr int CH = (int)(C::PB / 16);
            for (int b = warp; b < KB; b += WARPS) {
                for (int c = lane; c < CH; c += 32) {
                    cp_async16(img_s + (uint32_t)(b * CH + c) * 16u, image + ((size_t)b * CH + c) * 16);
                }
            }
            cp_async_commit();
            cp_async_wait<0>();
            __syncwarp();
        } else {
            const uint8_t* src = image + (size_t)sl * KS * C::PB;
            const int chunks = (int)((size_t)len * C::PB / 16);
            for (int c = tid; c < chunks; c += THREADS) {
                cp_async16(img_s + (uint32_t)c * 16u, src + (size_t)c * 16);
            }
            cp_async_commit();
            cp_async_wait<0>();
            __syncthreads();
        }
        for (int ti = 0; ti < my_tiles; ti++) {
            const int my_tile = (int)blockIdx.x + ti * (int)gridDim.x;
            for (int b = warp; b < len; b += WARPS) {
                __syncwarp();  // every lane is done reading the slot that is requested next
                issue();
                if (!gave_up) {
                    // the copies of this step have landed (bounded: the clock, not the number of polls)
                    const uint32_t bar = bars_s + 8 * cmp_slot;
                    if (!tc::mbar_try(bar, cmp_phase)) {
                        const long long t0 = clock64();
                        while (!tc::mbar_try(bar, cmp_phase)) {
                            if (clock64() - t0 > wait_clocks) {
                                atomicCAS(&g_q6k_status, 0, 25);
                                gave_up = true;
                                break;
                            }
                        }
                    }
                }
                compute(ring + cmp_slot * SLOT_BYTES, ring_s + cmp_slot * SLOT_BYTES, b, my_tile, sl * KS + b);
                if (++cmp_slot == STAGES) {
                    cmp_slot = 0;
                    cmp_phase ^= 1u;
                }
            }
            // ---- this warp's partial sums per activation row: combine the digit columns, then the 4 lanes of a row ------
            float* rd = red + (size_t)parity * WARPS * 16 * MT;
#pragma unroll
            for (int m = 0; m < MT; m++) {
                float p0 = 0.0f, p1 = 0.0f;
#pragma unroll
                for (int i = 0; i < NG; i++) {
#pragma unroll
                    for (int c = 0; c < 2; c++) {
                        if (mq[i][c] == m) {
                            p0 += acc[i][0][c];
                            p1 += acc[i][1][c];
                        }
                    }
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
#pragma unroll
            for (int i = 0; i < NG; i++) {
                acc[i][0][0] = acc[i][0][1] = acc[i][1][0] = acc[i][1][1] = 0.0f;
            }
            __syncthreads();
            // ---- the 8 warps' partial sums in a fixed order, added to what earlier slices left ---------------------------------
            for (int o = tid; o < 16 * MT; o += THREADS) {
                const int r = o / MT, m = o % MT;
                const int64_t row = (int64_t)my_tile * 16 + r;
                const float* p = rd + r * MT + m;
                float sum = ((p[0] + p[16 * MT]) + (p[2 * 16 * MT] + p[3 * 16 * MT])) +
                            ((p[4 * 16 * MT] + p[5 * 16 * MT]) + (p[6 * 16 * MT] + p[7 * 16 * MT]));
                if (sl > 0) {
                    sum += carry[(size_t)ti * 16 * MT + o];
                }
                if (sl + 1 < nslices) {
                    carry[(size_t)ti * 16 * MT + o] = sum;
                } else if (m < rows && row < n) {
                    y[(int64_t)m * n + row] = sum + (bias != nullptr ? bias[row] : 0.0f);
                }
            }
            parity ^= 1;
        }
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

template <int MT, int STAGES, int OCC>
int launch(const View& v, const uint8_t* image, int rows, const float* bias, float* y, cudaStream_t s, int KS, int grid, int max_tiles, size_t smem) {
    static std::atomic<uint64_t> configured{0};  // the opt-in for large dynamic shared memory is per device
    int dev = 0;
    JQ_CUDA(cudaGetDevice(&dev));
    if ((configured.load() >> (dev & 63) & 1) == 0) {
        JQ_CUDA(cudaFuncSetAttribute(gemv_q6k_i8_kernel<MT, STAGES, OCC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX));
        configured.fetch_or((uint64_t)1 << (dev & 63));
    }
    const int tiles = (int)((v.n + 15) / 16);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // may start while the activation kernel runs
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const long long wait_clocks = (long long)g_opt_wait_limit_us.load(std::memory_order_relaxed) * 2000;  // about 2 GHz
    JQ_CUDA(cudaLaunchKernelEx(&cfg, gemv_q6k_i8_kernel<MT, STAGES, OCC>, v, image, rows, bias, y, tiles, KS, max_tiles, wait_clocks));
    count_launch();
    return JQ_OK;
}

// Shared memory of one CTA: image slice, cross-warp reduction, carried sums, weight ring.
template <int MT>
size_t smem_bytes(int KS, int stages, bool sliced, int max_tiles) {
    return (size_t)WARPS * stages * 8 + (size_t)KS * Cfg<MT>::PB + (size_t)(2 * WARPS * 16 * MT) * sizeof(float) + (sliced ? (size_t)max_tiles * 16 * MT * sizeof(float) : 0) +
           (size_t)WARPS * stages * SLOT_BYTES;
}

template <int MT>
int run(const View& v, const float* x, int rows, const float* bias, float* y, cudaStream_t s, uint8_t* image, bool* handled) {
    const int KB = (int)(v.k / 256);
    const int tiles = (int)((v.n + 15) / 16);
    // Candidate shapes, best first: (CTAs per SM, ring stages); two CTAs per SM with three stages measured best. The slice length KS is a function of MT and k only (so
    // that the summation order never depends on n): the whole k if its image fits beside the ring, else a multiple of 8.
    const int occ_of[3] = {2, 2, 2}, st_of[3] = {3, 3, 2};
    const size_t red_bytes = (size_t)(2 * WARPS * 16 * MT) * sizeof(float);
    const size_t fixed = red_bytes + 8 * 1024;  // sliced shapes: reduction buffer + room for carried sums
    int pick = -1, KS = KB;
    for (int c = 0; c < 3 && pick < 0; c++) {
        const size_t budget = SMEM_MAX / occ_of[c] - 1024;
        if ((size_t)KB * Cfg<MT>::PB + red_bytes + (size_t)WARPS * st_of[c] * (SLOT_BYTES + 8) <= budget) {
            pick = c;
        }
    }
    int stages = pick >= 0 ? st_of[pick] : 0;
    if (pick < 0) {
        // slices: two CTAs per SM, three ring stages, or two if a slice of 8 super-blocks needs the room
        pick = 2;
        for (stages = 3; stages >= 2; stages--) {
            const size_t budget = SMEM_MAX / 2 - 1024 - fixed - (size_t)WARPS * stages * (SLOT_BYTES + 8);
            KS = (int)(budget / Cfg<MT>::PB) / 8 * 8;
            if (KS >= 8) {
                break;
            }
        }
        if (KS < 8) {
            *handled = false;
            return JQ_OK;
        }
    }
    const int occ = occ_of[pick];
    const int grid = tiles < sm_count() * occ ? tiles : sm_count() * occ;
    const int max_tiles = (tiles + grid - 1) / grid;
    const bool sliced = KS < KB;
    const size_t smem = smem_bytes<MT>(KS, stages, sliced, max_tiles);
    if (smem > SMEM_MAX / occ - 1024) {
        *handled = false;  // more tiles per CTA than the carried sums have room for
        return JQ_OK;
    }
    *handled = true;
    if (x != nullptr) {  // else the image is already in `image` (written by a kernel earlier in the stream)
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
        JQ_CUDA(cudaLaunchKernelEx(&icfg, q6k_activation_image_kernel<MT>, x, rows, (int64_t)v.k, image));
        count_launch();
    }
    if (stages == 3) return launch<MT, 3, 2>(v, image, rows, bias, y, s, KS, grid, max_tiles, smem);
    return launch<MT, 2, 2>(v, image, rows, bias, y, s, KS, grid, max_tiles, smem);
}

}  // namespace

// Bytes of scratch (activation image) a Q6_K GEMV of `rows` activation rows over k inputs needs; 0 if the
// shape is not handled by the integer kernel.
size_t gemv_q6k_i8_scratch_bytes(int64_t k, int rows) {
    if (rows < 1 || rows > 4 || k <= 0) {
        return 0;
    }
    const size_t pb = rows == 1 ? Cfg<1>::PB : (rows == 2 ? Cfg<2>::PB : Cfg<4>::PB);
    return (size_t)(k / 256) * pb;
}

// Q6_K with rows in [1, 4] on a weight whose planes is padded by 16 rows. `image` is a scratch buffer of
// gemv_q6k_i8_scratch_bytes(k, rows) bytes, 16-byte aligned, private to `s` until the GEMV kernel has run.
// *handled = false leaves the call to another kernel.
int launch_gemv_q6k_i8(const View& v, const float* x, int rows, const float* bias, float* y, cudaStream_t s, uint8_t* image, bool* handled) {
    *handled = false;
    if (v.type != JQ_TYPE_Q6_K || v.n == 0 || v.k == 0 || rows > 4 || image == nullptr || (int64_t)16 * (v.k / 256) * 208 >= ((int64_t)1 << 31)) {
        return JQ_OK;
    }
    if (rows == 1) return run<1>(v, x, rows, bias, y, s, image, handled);
    if (rows == 2) return run<2>(v, x, rows, bias, y, s, image, handled);
    return run<4>(v, x, rows, bias, y, s, image, handled);
}

// Reads and clears the status of the weight-ring waits on the current device.
int gemv_q6k_status(int* status) {
    const int zero = 0;
    JQ_CUDA(cudaMemcpyFromSymbol(status, g_q6k_status, sizeof(int)));
    JQ_CUDA(cudaMemcpyToSymbol(g_q6k_status, &zero, sizeof(int)));
    return JQ_OK;
}

size_t q6k_image_bytes_one_row(int64_t k) { return (size_t)(k / 256) * Cfg<1>::PB; }

// One row of x whose image (q6k::build_image<1> per super-block) a kernel earlier in the stream has written to `image`;
// that kernel should execute griddepcontrol.launch_dependents so that this one can request weights meanwhile.
int launch_gemv_q6k_i8_imaged(const View& v, const uint8_t* image, const float* bias, float* y, cudaStream_t s, bool* handled) {
    *handled = false;
    if (v.type != JQ_TYPE_Q6_K || v.n == 0 || v.k == 0 || image == nullptr || (int64_t)16 * (v.k / 256) * 208 >= ((int64_t)1 << 31)) {
        return JQ_OK;
    }
    return run<1>(v, nullptr, 1, bias, y, s, const_cast<uint8_t*>(image), handled);
}

}  // namespace jq
