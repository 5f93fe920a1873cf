// Decode GEMV for Q4_K with integer tensor-core arithmetic: y[m, n] = x[m, k] . W[n, k]^T, m <= 8.
//
// The 4-bit quants never become floating point. A small first kernel turns the activations into an
// "activation image" in a scratch buffer: per 256-element super-block of k and per row of x, the values
// are scaled by a power of two s (from the block's largest magnitude), rounded to 22-bit fixed point,
// X = rint(x / s * 2^21), and split into three signed base-256 digits X = d2 * 65536 + d1 * 256 + d0.
// The digits are laid out as B fragments of mma.sync.m16n8k32 (u8 x s8 -> s32), one column per (row of x, digit);
// the fragments of two sub-blocks sit side by side, so one 16-byte load feeds two MMAs. The GEMV kernel widens four
// nibbles to four bytes with one AND and feeds them as the A operand, so one MMA multiplies one 32-element sub-block
// of 16 weight rows with every digit column exactly. Sub-block results are combined with the 6-bit scales in integer
// arithmetic (sum over 8 sub-blocks of sc * D stays below 2^31), converted to float once per super-block and scaled
// by fp16 d and the column weight s * 2^(8i - 21). The "min" part of Q4_K, dmin * sum_sub m_sub * sum(x over the
// sub-block), uses one m16n8k16 MMA whose A operand is the eight packed 6-bit mins and whose B operand holds the
// digit sums of every sub-block. Everything up to the per-super-block float conversion is exact and x keeps 22 bits
// relative to the largest magnitude of its super-block, so results match an FP32-accumulating kernel. The summation
// order depends on k and the number of rows of x only: a row shard of a weight gives bitwise the same outputs as the
// whole weight.
//
// Two column layouts (struct Cfg). One or two rows of x: column 3m + i of a single group; the three digit columns of
// a row sit in different lanes and are combined by shuffles once per tile; the high nibbles are masked in place
// (no shift) and their 16-fold products summed apart. Three to eight rows: digit i is column group i and row m its
// column m, which puts all digits of rows 2t and 2t + 1 into lane t: no exchange between lanes at all.
//
// Work split: a CTA of 8 warps (16 for three to eight rows of x, where one CTA per SM shares one copy of the large
// image) owns 16 output rows at a time (tiles blockIdx.x, blockIdx.x + gridDim.x, ...), warp p takes super-blocks
// b = p (mod warps). Weights stream HBM -> shared memory through a per-warp ring of slots: the 16 rows of a tile and one
// super-block are one contiguous run of bytes in the tiled device layout, which one lane requests with a single bulk copy
// (cp.async.bulk) that completes on the slot's mbarrier. A slot holds the rows as they are in global memory; lane group g
// works on rows 2 (g & 3) + (g >> 2) and eight further, which makes the 8-byte fragment reads conflict free (the row
// pitch of 144 or 176 bytes advances 4 or 12 banks per row). The tiled layout pads the last 128 rows with zeros, so the
// last tile needs no bounds check. The kernel is launched with programmatic stream serialization: it requests its first
// weights while the kernel before it is still running and waits for it (griddepcontrol.wait) only before it touches x or
// the image. With one or two rows of x that are given as floats the kernel builds the image itself: every warp makes
// exactly the super-blocks it consumes, straight from x, so there is no image kernel, no scratch round trip and no
// barrier between warps for it.
#include <mutex>

#include "jq_formats.cuh"
#include "jq_peer_device.cuh"
#include "jq_q4k_image.cuh"
#include "jq_tc.cuh"

namespace jq {

using q4k::Cfg;
using q4k::build_image;

namespace {

// One super-block of 16 rows in a ring slot, as in global memory: per row the 16-byte header, (Q5_K) 32 bytes of fifth
// bits, 128 bytes of nibbles. The kernel is written for Q4_K; Q5_K (template flag Q5) is the same format with one more
// bit per quant.
template <bool Q5>
struct Blk {
    static constexpr int BYTES = Q5 ? 176 : 144;  // bytes per super-block and row
    static constexpr int SLOT = 16 * BYTES;
    static constexpr int QH = 16;                  // offset of the fifth bits in a row (Q5_K)
    static constexpr int QS = Q5 ? 48 : 16;        // offset of the nibbles
};
constexpr size_t SMEM_MAX = 227 * 1024;

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// D = A(16x32 u8) * B(32x8 s8), accumulators start at zero.
__device__ __forceinline__ void imma_k32(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// D = A(16x16 u8) * B(16x8 s8), accumulators start at zero.
__device__ __forceinline__ void imma_k16(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// The image in a scratch buffer in global memory, for the GEMV shapes that do not build it themselves. The kernel is
// tiny and latency bound, so the work is spread over as many warps as possible.
constexpr int PREP_WARPS = 4;
__device__ int g_gemv_peer_status;  // 0, or 32 + rank once a GEMV's own wait for an exchange has given up

template <int MT>
__global__ void __launch_bounds__(PREP_WARPS * 32) q4k_activation_image_kernel(const float* __restrict__ x, int rows, int64_t k,
                                                                             uint8_t* __restrict__ image) {
    asm volatile("griddepcontrol.launch_dependents;");  // the GEMV kernel may start requesting weights now
    asm volatile("griddepcontrol.wait;" ::: "memory");  // x is complete, and the GEMV before this one is done with the scratch image
    const int pair = blockIdx.x * PREP_WARPS + (threadIdx.x >> 5);
    const int b = pair / MT, m = pair % MT;
    if (b < (int)(k >> 8)) {
        build_image<MT>(m < rows ? x + (int64_t)m * k + (int64_t)b * 256 : nullptr, m, image + (size_t)b * Cfg<MT>::PB, threadIdx.x & 31);
    }
}

// Development aid, compiled in with -DJQ_Q4K_TRACE: thread 0 of every CTA records %globaltimer at a few points of the kernel
// into the next free record; jq_debug_q4k_trace copies the records out.
#ifdef JQ_Q4K_TRACE
constexpr int TRACE_SLOTS = 16384;
__device__ long long g_q4k_tr[TRACE_SLOTS * 8];
__device__ int g_q4k_ticket;
__device__ __forceinline__ long long gtime() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define QT(k)                                        \
    do {                                             \
        if (threadIdx.x == 0) g_q4k_tr[tslot * 8 + (k)] = gtime(); \
    } while (0)
#else
#define QT(k) do { } while (0)
#endif

// ---- the GEMV ---------------------------------------------------------------------------------------------------
// A second and a third weight with the same k that are multiplied with the same x in the same launch (q = nullptr: none).
struct Second {
    const uint8_t* q;
    int64_t n;
    float* y;
    int first_tiles;   // tiles of the first weight
    const uint8_t* q3;
    int64_t n3;
    float* y3;
    int second_tiles;  // tiles of the first and the second weight
};

// PEER: the outputs go into every rank's y of a row-sharded linear (jq_peer.cu) instead of y. A template flag, not a
// run-time branch: the mere presence of the peer stores in the epilogue cost the ordinary kernel a fifth of its speed.
// FUSED: `xin` holds the rows of x as floats and every warp builds the image of its own super-blocks; otherwise `image`
// holds the image, written by a kernel earlier in the stream.
template <int MT, int STAGES, int NW, int OCC, bool Q5, bool PEER, bool FUSED>
__global__ void __launch_bounds__(NW * 32, OCC) gemv_q4k_i8_kernel(View v, Second w2, const PeerOut* __restrict__ peerp, const uint8_t* __restrict__ image,
                                                                  const float* __restrict__ xin, int rows, const float* __restrict__ bias, float* __restrict__ y,
                                                                  int tiles, int KS, int max_tiles, long long wait_clocks) {
    // Tiles 0 .. w2.first_tiles - 1 are rows of v, the tiles from w2.first_tiles on rows of the second weight w2 (same k,
    // same x, its own output), if there is one.
    // KS = super-blocks of k per slice: the activation image of one slice is resident in shared memory at a time;
    // with more than one slice the per-tile sums are carried in shared memory (max_tiles tiles per CTA).
    using C = Cfg<MT>;
    constexpr int NG = C::NG, NCOL = C::NCOL, NGM = C::NGM, NCOLM = C::NCOLM;
    constexpr int THREADS = NW * 32;
    using B = Blk<Q5>;
    constexpr int SLOT_BYTES = B::SLOT;
    constexpr uint32_t RING_BYTES = STAGES * SLOT_BYTES;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    asm volatile("griddepcontrol.launch_dependents;");  // the kernel after this one may be scheduled as room becomes free
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#ifdef JQ_Q4K_TRACE
    int tslot = 0;
    if (tid == 0) {
        tslot = atomicAdd(&g_q4k_ticket, 1) % TRACE_SLOTS;
        g_q4k_tr[tslot * 8 + 6] = (long long)v.q | (blockIdx.x == 0 ? 1 : 0);
        g_q4k_tr[tslot * 8 + 7] = 0;
    }
    QT(0);
#endif
    const int g = lane >> 2, t = lane & 3;
    const int R = 2 * (g & 3) + (g >> 2);  // this lane's rows of the tile: R and R + 8
    const int KB = (int)(v.k >> 8);
    const int nslices = (KB + KS - 1) / KS;
    constexpr int BAR_BYTES = NW * STAGES * 8;                                       // one mbarrier per slot
    static_assert(BAR_BYTES % 16 == 0, "what follows the barriers stays 16-byte aligned");
    uint8_t* img = smem_raw + BAR_BYTES;                                             // [KS][PB]
    float* red = reinterpret_cast<float*>(img + (size_t)KS * C::PB);                 // [2][NW][16][MT]
    float* carry = red + 2 * NW * 16 * MT;                                           // [max_tiles][16][MT], only if nslices > 1
    uint8_t* ring = reinterpret_cast<uint8_t*>(carry + (nslices > 1 ? (size_t)max_tiles * 16 * MT : 0)) + (size_t)warp * RING_BYTES;
    const uint32_t ring_s = tc::smem_u32(ring);
    const uint32_t bars_s = tc::smem_u32(smem_raw) + (uint32_t)(warp * STAGES * 8);  // this warp's barriers
    // The weight is stored tile by tile (jq_common.cuh): the 16 rows of a tile of this kernel and one super-block are 16 x BYTES
    // consecutive bytes inside a unit of 128 rows, and the units of consecutive super-blocks follow each other.
    constexpr int64_t UNIT = (int64_t)TILE_ROWS * B::BYTES;

    // ---- weight stream: one bulk copy per step, requested by lane 0, complete when the slot's barrier says so -----------
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) {
            tc::mbar_init(bars_s + 8 * s, 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");  // the copy engine sees initialised barriers
    }
    __syncwarp();
    // This warp's steps, in order: for every slice, for every tile of the CTA, the super-blocks b = slice start + warp + NW i.
    const int len_last = KB - (nslices - 1) * KS;
    const int nb_full = nslices > 1 ? (warp < KS ? (KS - warp + NW - 1) / NW : 0) : 0;
    const int nb_last = warp < len_last ? (len_last - warp + NW - 1) / NW : 0;
    const int my_tiles = (int)blockIdx.x < tiles ? (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    // the slot of tile number ti of the CTA, first block of this warp in slice sl
    auto step_ptr = [&](int ti, int sl) {
        const int tile = (int)blockIdx.x + ti * (int)gridDim.x;
        const int local = tile < w2.first_tiles ? tile : (tile < w2.second_tiles ? tile - w2.first_tiles : tile - w2.second_tiles);
        const uint8_t* base = tile < w2.first_tiles ? v.q : (tile < w2.second_tiles ? w2.q : w2.q3);
        return base + ((int64_t)(local >> 3) * KB + (sl * KS + warp)) * UNIT + (local & 7) * 16 * B::BYTES;
    };
    const uint8_t* gp = step_ptr(0, 0);
    int iss_left = ((nslices - 1) * nb_full + nb_last) * my_tiles;
    int iss_sl = 0, iss_ti = 0, iss_j = 0, iss_nb = nslices > 1 ? nb_full : nb_last;
    int iss_slot = 0;
    auto issue = [&]() {  // every lane keeps the bookkeeping, lane 0 makes the request
        if (iss_left > 0) {
            iss_left--;
            if (lane == 0) {
                tc::mbar_expect_tx(bars_s + 8 * iss_slot, SLOT_BYTES);
                tc::bulk_load(ring_s + iss_slot * SLOT_BYTES, gp, SLOT_BYTES, bars_s + 8 * iss_slot);
            }
            gp += NW * UNIT;
            if (++iss_j == iss_nb) {
                iss_j = 0;
                if (++iss_ti == my_tiles) {
                    iss_ti = 0;
                    iss_sl++;
                    iss_nb = iss_sl == nslices - 1 ? nb_last : nb_full;
                }
                gp = step_ptr(iss_ti, iss_sl);
            }
        }
        iss_slot = iss_slot + 1 == STAGES ? 0 : iss_slot + 1;
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
        issue();  // the first weights are on their way before x or the activation image is complete
    }

    // ---- x (or the image made from it) is complete once the kernel before this one has finished --------------------------
    asm volatile("griddepcontrol.wait;" ::: "memory");
    QT(1);
    const uint32_t img_s = tc::smem_u32(img);
    bool peer_marks = false;  // the outputs travel as marked words (jq_peer_device.cuh) rather than behind a release
    uint32_t peer_seq = 0;
    if constexpr (PEER) {
        peer_marks = peerp->stage[0] != nullptr;
        if (peer_marks) {
            peer_seq = peer_marks_seq(peerp);
        }
        if (peerp->wait_first) {
            // the image is what the ranks' latest exchange delivered: complete once all their flags are up
            if (warp == 0) {
                peer_wait_inline(peerp->flags[peerp->rank], peerp->world, lane, &g_gemv_peer_status);
            }
            __syncthreads();
        }
    }

    // ---- main loop ----------------------------------------------------------------------------------------------
    // Lanes whose column is not stored read another lane's fragment; those columns have weight zero.
    const uint8_t* xd_lane = img + ((size_t)(NCOL == 8 ? g : g % NCOL) * 4 + t) * 16;
    const uint8_t* xm_lane = img + C::XD + ((size_t)(NCOLM == 8 ? g : g % NCOLM) * 4 + t) * 4;
    const uint8_t* tab_lane = img + C::XD + C::XM;
    const int row_off = R * B::BYTES;  // this lane's first row inside a slot
    const bool mins_low = (t & 1) == 0;  // lanes t = 0, 2 feed mins 0..3, lanes 1, 3 mins 4..7 (slots 2, 3 meet zeros)
    // Packed: acc[group][row R / R + 8][column 2t / 2t + 1] and accm[mins group][row]. Digit major: acc[0][row][row of x].
    constexpr int NACC = C::DIGIT_MAJOR ? 1 : NG, NACCM = C::DIGIT_MAJOR ? 1 : NGM;
    float acc[NACC][2][2];
    float accm[NACCM][2];
#pragma unroll
    for (int i = 0; i < NACC; i++) {
        acc[i][0][0] = acc[i][0][1] = acc[i][1][0] = acc[i][1][1] = 0.0f;
    }
#pragma unroll
    for (int i = 0; i < NACCM; i++) {
        accm[i][0] = accm[i][1] = 0.0f;
    }

    auto compute = [&](const uint8_t* slot, const uint8_t* blk) {  // blk = this lane's view of the super-block's image
        const uint8_t* r0 = slot + row_off;     // row R of the tile: header, (fifth bits,) nibbles
        const uint8_t* r1 = r0 + 8 * B::BYTES;  // row R + 8
        const uint8_t* q0 = r0 + B::QS + 8 * t;
        const uint8_t* q1 = r1 + B::QS + 8 * t;
        const uint4 h0 = *reinterpret_cast<const uint4*>(r0);
        const uint4 h1 = *reinterpret_cast<const uint4*>(r1);
        // 6-bit scales and mins of the 8 sub-blocks as packed bytes: [0..3] and [4..7]
        const uint32_t sc0a = h0.y & 0x3f3f3f3fu, sc0b = and_or(h0.y >> 2, 0x30303030u, h0.w & 0x0f0f0f0fu);
        const uint32_t sc1a = h1.y & 0x3f3f3f3fu, sc1b = and_or(h1.y >> 2, 0x30303030u, h1.w & 0x0f0f0f0fu);
        const uint32_t mn0 = mins_low ? (h0.z & 0x3f3f3f3fu) : and_or(h0.z >> 2, 0x30303030u, (h0.w >> 4) & 0x0f0f0f0fu);
        const uint32_t mn1 = mins_low ? (h1.z & 0x3f3f3f3fu) : and_or(h1.z >> 2, 0x30303030u, (h1.w >> 4) & 0x0f0f0f0fu);
        // Packed layouts keep the high nibbles in place (one AND, no shift): the odd sub-blocks' products come out 16 times
        // too large, are summed apart from the even ones' and meet them as 16 even + odd; the column weights carry the 1 / 16.
        constexpr bool SPLIT = !C::DIGIT_MAJOR && !Q5;
        // Q5_K: the fifth bits of this lane's elements 8t .. 8t+7 of every sub-block, rows R and R + 8 (bit `sub` of each byte)
        uint2 qh0 = make_uint2(0u, 0u), qh1 = make_uint2(0u, 0u);
        if constexpr (Q5) {
            qh0 = *reinterpret_cast<const uint2*>(r0 + B::QH + 8 * t);
            qh1 = *reinterpret_cast<const uint2*>(r1 + B::QH + 8 * t);
        }
        int I[NG][4], IO[SPLIT ? NG : 1][4];
#pragma unroll
        for (int i = 0; i < NG; i++) {
            I[i][0] = I[i][1] = I[i][2] = I[i][3] = 0;
        }
#pragma unroll
        for (int i = 0; i < (SPLIT ? NG : 1); i++) {
            IO[i][0] = IO[i][1] = IO[i][2] = IO[i][3] = 0;
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            // this lane's 8 bytes of group j for rows R and R + 8: elements 8t .. 8t+7 of sub-blocks 2j (low) and 2j+1 (high)
            const uint2 wa = *reinterpret_cast<const uint2*>(q0 + 32 * j);
            const uint2 wb = *reinterpret_cast<const uint2*>(q1 + 32 * j);
            uint4 bfp[NG];  // B operands of sub-blocks 2j (x, y) and 2j + 1 (z, w)
#pragma unroll
            for (int i = 0; i < NG; i++) {
                bfp[i] = *reinterpret_cast<const uint4*>(blk + (size_t)((j * NG + i) * NCOL) * 64);
            }
#pragma unroll
            for (int hf = 0; hf < 2; hf++) {
                const int sub = 2 * j + hf;
                const bool keep = SPLIT && hf == 1;  // high nibbles stay where they are
                uint32_t a0 = keep ? wa.x & 0xf0f0f0f0u : (hf == 0 ? wa.x : wa.x >> 4) & 0x0f0f0f0fu;
                uint32_t a2 = keep ? wa.y & 0xf0f0f0f0u : (hf == 0 ? wa.y : wa.y >> 4) & 0x0f0f0f0fu;
                uint32_t a1 = keep ? wb.x & 0xf0f0f0f0u : (hf == 0 ? wb.x : wb.x >> 4) & 0x0f0f0f0fu;
                uint32_t a3 = keep ? wb.y & 0xf0f0f0f0u : (hf == 0 ? wb.y : wb.y >> 4) & 0x0f0f0f0fu;
                if constexpr (Q5) {
                    auto fifth = [&](uint32_t hw) { return sub < 4 ? hw << (4 - sub) : hw >> (sub - 4); };  // bit `sub` -> bit 4
                    a0 = and_or(fifth(qh0.x), 0x10101010u, a0);
                    a2 = and_or(fifth(qh0.y), 0x10101010u, a2);
                    a1 = and_or(fifth(qh1.x), 0x10101010u, a1);
                    a3 = and_or(fifth(qh1.y), 0x10101010u, a3);
                }
                const int s0 = (int)__byte_perm(sub < 4 ? sc0a : sc0b, 0u, 0x4440u + (sub & 3));
                const int s1 = (int)__byte_perm(sub < 4 ? sc1a : sc1b, 0u, 0x4440u + (sub & 3));
#pragma unroll
                for (int i = 0; i < NG; i++) {
                    int D[4];
                    imma_k32(D, a0, a1, a2, a3, hf == 0 ? bfp[i].x : bfp[i].z, hf == 0 ? bfp[i].y : bfp[i].w);
                    int(&S)[4] = keep ? IO[i] : I[i];
                    S[0] += s0 * D[0];
                    S[1] += s0 * D[1];
                    S[2] += s1 * D[2];
                    S[3] += s1 * D[3];
                }
            }
        }
        const float d0 = half_bits_to_float(h0.x), d1 = half_bits_to_float(h1.x);
        const float dm0 = half_bits_to_float(h0.x >> 16), dm1 = half_bits_to_float(h1.x >> 16);
        const uint8_t* tb = blk + (tab_lane - xd_lane);
        const uint8_t* fm = blk + (xm_lane - xd_lane);
        if constexpr (C::DIGIT_MAJOR) {
            float qf[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}}, mf[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};  // [row][row of x 2t + c]
#pragma unroll
            for (int i = 0; i < 3; i++) {
                const float2 w = *reinterpret_cast<const float2*>(tb + (8 * i + 2 * t) * 4);  // digit i of rows 2t, 2t + 1 of x
                qf[0][0] = fmaf(w.x, (float)I[i][0], qf[0][0]);
                qf[0][1] = fmaf(w.y, (float)I[i][1], qf[0][1]);
                qf[1][0] = fmaf(w.x, (float)I[i][2], qf[1][0]);
                qf[1][1] = fmaf(w.y, (float)I[i][3], qf[1][1]);
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    int E[4];
                    imma_k16(E, mn0, mn1, *reinterpret_cast<const uint32_t*>(fm + (size_t)(2 * i + c) * NCOLM * 16));
                    const float wc = c == 0 ? w.x : w.y;
                    mf[0][c] = fmaf(wc, (float)(E[1] * 128 + E[0]), mf[0][c]);
                    mf[1][c] = fmaf(wc, (float)(E[3] * 128 + E[2]), mf[1][c]);
                }
            }
#pragma unroll
            for (int c = 0; c < 2; c++) {
                acc[0][0][c] = fmaf(-dm0, mf[0][c], fmaf(d0, qf[0][c], acc[0][0][c]));
                acc[0][1][c] = fmaf(-dm1, mf[1][c], fmaf(d1, qf[1][c], acc[0][1][c]));
            }
        } else {
#pragma unroll
            for (int i = 0; i < NG; i++) {
                const float2 w = *reinterpret_cast<const float2*>(tb + (NG * 8 + 8 * i + 2 * t) * 4);  // weights / 16 of columns 2t, 2t+1
                acc[i][0][0] = fmaf(d0 * w.x, (float)(16 * I[i][0] + IO[i][0]), acc[i][0][0]);
                acc[i][0][1] = fmaf(d0 * w.y, (float)(16 * I[i][1] + IO[i][1]), acc[i][0][1]);
                acc[i][1][0] = fmaf(d1 * w.x, (float)(16 * I[i][2] + IO[i][2]), acc[i][1][0]);
                acc[i][1][1] = fmaf(d1 * w.y, (float)(16 * I[i][3] + IO[i][3]), acc[i][1][1]);
            }
#pragma unroll
            for (int i = 0; i < NGM; i++) {
                int E[4];
                imma_k16(E, mn0, mn1, *reinterpret_cast<const uint32_t*>(fm + (size_t)i * NCOLM * 16));
                const float w = *reinterpret_cast<const float*>(tb + (4 * i + t) * 4);  // weight of digit column 4i + t
                accm[i][0] = fmaf(dm0 * w, (float)(E[1] * 128 + E[0]), accm[i][0]);
                accm[i][1] = fmaf(dm1 * w, (float)(E[3] * 128 + E[2]), accm[i][1]);
            }
        }
    };

    int parity = 0;
    int cmp_slot = 0;
    uint32_t cmp_phase = 0;
    bool gave_up = false;  // a wait for weights ran out: the status word says so, the warp stops waiting and finishes with whatever is there
    for (int sl = 0; sl < nslices; sl++) {
        // ---- this slice of the activation image in shared memory ---------------------------------------------------------
        const int len = sl == nslices - 1 ? len_last : KS;
        const int nb = sl == nslices - 1 ? nb_last : nb_full;
        if constexpr (FUSED) {
            // a warp only ever reads the image of its own super-blocks, so it makes just those and waits for nobody
            __syncwarp();  // the warp's lanes are done with the previous slice
            // two (super-block, row) parts at a time, so that the loads of the second are in flight while the first is made
            const int parts = nb * MT;  // part p: block warp + NW (p / MT) of the slice, row p % MT of x
            for (int p = 0; p < parts; p += 2) {
                float xa[8], xb[8];
                const int bl0 = warp + NW * (p / MT), m0 = p % MT;
                const int bl1 = warp + NW * ((p + 1) / MT), m1 = (p + 1) % MT;
                const bool two = p + 1 < parts;
                const bool have0 = m0 < rows, have1 = two && m1 < rows;
                q4k::load_image_values(have0 ? xin + (int64_t)m0 * v.k + (int64_t)(sl * KS + bl0) * 256 : nullptr, lane, xa);
                q4k::load_image_values(have1 ? xin + (int64_t)m1 * v.k + (int64_t)(sl * KS + bl1) * 256 : nullptr, lane, xb);
                q4k::build_image_from<MT>(xa, have0, m0, img + (size_t)bl0 * C::PB, lane);
                if (two) {
                    q4k::build_image_from<MT>(xb, have1, m1, img + (size_t)bl1 * C::PB, lane);
                }
            }
            __syncwarp();
        } else if (nslices == 1) {
            // one slice: a warp fetches the image of its own super-blocks and waits for nobody else
            constexpr int CH = (int)(C::PB / 16);
            for (int b = warp; b < KB; b += NW) {
                for (int c = lane; c < CH; c += 32) {
                    cp_async16(img_s + (uint32_t)(b * CH + c) * 16u, image + ((size_t)b * CH + c) * 16);
                }
            }
            cp_async_commit();
            cp_async_wait<0>();
            __syncwarp();
        } else {
            if (sl > 0) {
                __syncthreads();  // every warp is done with the previous slice
            }
            const uint8_t* src = image + (size_t)sl * KS * C::PB;
            const int chunks = (int)((size_t)len * C::PB / 16);
            for (int c = tid; c < chunks; c += THREADS) {
                cp_async16(img_s + (uint32_t)c * 16u, src + (size_t)c * 16);
            }
            cp_async_commit();
            cp_async_wait<0>();
            __syncthreads();
        }
        if (sl == 0) {
            QT(2);
        }
        for (int ti = 0; ti < my_tiles; ti++) {
            const int my_tile = (int)blockIdx.x + ti * (int)gridDim.x;
            const uint8_t* blk = xd_lane + (size_t)warp * C::PB;
            for (int j = 0; j < nb; j++) {
                __syncwarp();  // every lane is done reading the slot that is requested next
                issue();
                if (!gave_up) {
                    // the copy of this step has landed (bounded: the clock, not the number of polls)
                    const uint32_t bar = bars_s + 8 * cmp_slot;
                    if (!tc::mbar_try(bar, cmp_phase)) {
                        const long long t0 = clock64();
                        while (!tc::mbar_try(bar, cmp_phase)) {
                            if (clock64() - t0 > wait_clocks) {
                                atomicCAS(&g_gemv_peer_status, 0, 24);
                                gave_up = true;
                                break;
                            }
                        }
                    }
                }
                if (sl == 0 && ti == 0 && j == 0) {
                    QT(3);
                }
                compute(ring + cmp_slot * SLOT_BYTES, blk);
                if (++cmp_slot == STAGES) {
                    cmp_slot = 0;
                    cmp_phase ^= 1u;
                }
                blk += (size_t)NW * C::PB;
            }
            if (sl == nslices - 1 && ti == my_tiles - 1) {
                QT(4);
            }
            // ---- this warp's partial sums per output row and row of x ---------------------------------------------------
            float* rd = red + (size_t)parity * NW * 16 * MT;
            if constexpr (C::DIGIT_MAJOR) {
                // the lane holds rows R, R + 8 for rows 2t, 2t + 1 of x (MT = 8: two floats side by side)
                *reinterpret_cast<float2*>(rd + (warp * 16 + R) * MT + 2 * t) = make_float2(acc[0][0][0], acc[0][0][1]);
                *reinterpret_cast<float2*>(rd + (warp * 16 + R + 8) * MT + 2 * t) = make_float2(acc[0][1][0], acc[0][1][1]);
                acc[0][0][0] = acc[0][0][1] = acc[0][1][0] = acc[0][1][1] = 0.0f;
            } else {
                // combine the digit columns of a row of x, which sit in the 4 lanes of a quad
#pragma unroll
                for (int m = 0; m < MT; m++) {
                    float p0 = 0.0f, p1 = 0.0f;
#pragma unroll
                    for (int c = 0; c < 2; c++) {
                        const int col = 2 * t + c;
                        const bool mine = col < C::COLS && col / 3 == m;
                        p0 += mine ? acc[0][0][c] : 0.0f;
                        p1 += mine ? acc[0][1][c] : 0.0f;
                    }
#pragma unroll
                    for (int i = 0; i < NGM; i++) {
                        const int col = 4 * i + t;  // digit column whose two sum parts this lane holds
                        const bool mine = col < C::COLS && col / 3 == m;
                        p0 -= mine ? accm[i][0] : 0.0f;
                        p1 -= mine ? accm[i][1] : 0.0f;
                    }
                    p0 += __shfl_xor_sync(0xffffffffu, p0, 1);
                    p1 += __shfl_xor_sync(0xffffffffu, p1, 1);
                    p0 += __shfl_xor_sync(0xffffffffu, p0, 2);
                    p1 += __shfl_xor_sync(0xffffffffu, p1, 2);
                    if (t == 0) {
                        rd[(warp * 16 + R) * MT + m] = p0;
                        rd[(warp * 16 + R + 8) * MT + m] = p1;
                    }
                }
                acc[0][0][0] = acc[0][0][1] = acc[0][1][0] = acc[0][1][1] = 0.0f;
#pragma unroll
                for (int i = 0; i < NGM; i++) {
                    accm[i][0] = accm[i][1] = 0.0f;
                }
            }
            __syncthreads();
            // ---- the warps' partial sums in a fixed order, added to what earlier slices left ---------------------------------
            const bool second = my_tile >= w2.first_tiles, third = my_tile >= w2.second_tiles;
            const int64_t n = third ? w2.n3 : (second ? w2.n : v.n);
            float* const yo = third ? w2.y3 : (second ? w2.y : y);
            for (int o = tid; o < 16 * MT; o += THREADS) {
                const int r = o / MT, m = o % MT;
                const int64_t row = (int64_t)(third ? my_tile - w2.second_tiles : (second ? my_tile - w2.first_tiles : my_tile)) * 16 + r;
                const float* p = rd + o;
                constexpr int W = 16 * MT;  // floats per warp
                float sum = ((p[0] + p[W]) + (p[2 * W] + p[3 * W])) + ((p[4 * W] + p[5 * W]) + (p[6 * W] + p[7 * W]));
                if constexpr (NW == 16) {
                    sum += ((p[8 * W] + p[9 * W]) + (p[10 * W] + p[11 * W])) + ((p[12 * W] + p[13 * W]) + (p[14 * W] + p[15 * W]));
                }
                if (sl > 0) {
                    sum += carry[(size_t)ti * 16 * MT + o];
                }
                if (sl + 1 < nslices) {
                    carry[(size_t)ti * 16 * MT + o] = sum;
                } else if (m < rows && row < n) {
                    const float val = sum + (bias != nullptr && !second ? bias[row] : 0.0f);
                    if constexpr (!PEER) {
                        yo[(int64_t)m * n + row] = val;
                    } else {
                        // a row shard: the value goes into every rank's y [m, n_total] at this rank's columns
                        const int64_t idx = (int64_t)m * peerp->n_total + peerp->col0 + row;
                        if (peer_marks) {
                            peer_store_marked(peerp, idx, val, peer_seq);
                        } else {
                            for (int r = 0; r < peerp->world; r++) {
                                peerp->y[r][idx] = val;
                            }
                        }
                    }
                }
            }
            parity ^= 1;
        }
    }
    QT(5);
    if constexpr (PEER) {
        if (peer_marks) {
            peer_collect(peerp, rows, peer_seq, &g_gemv_peer_status);  // the other ranks' rows, from this rank's staging words into its y
        } else {
            peer_publish(peerp->flags, peerp->rank, peerp->world, peerp->wait_after != 0, &g_gemv_peer_status);  // every CTA adds its share to this rank's counter on every rank
        }
        QT(7);
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

template <int MT, int STAGES, int NW, int OCC, bool Q5, bool PEER, bool FUSED>
int launch(const View& v, const Second& w2, const PeerOut& peer, const uint8_t* image, const float* x, int rows, const float* bias, float* y, cudaStream_t s,
           int KS, int grid, int max_tiles, size_t smem) {
    static std::atomic<uint64_t> configured{0};  // the opt-in for large dynamic shared memory is per device
    int dev = 0;
    JQ_CUDA(cudaGetDevice(&dev));
    if ((configured.load() >> (dev & 63) & 1) == 0) {
        JQ_CUDA(cudaFuncSetAttribute(gemv_q4k_i8_kernel<MT, STAGES, NW, OCC, Q5, PEER, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX));
        configured.fetch_or((uint64_t)1 << (dev & 63));
    }
    const int tiles = (int)((v.n + 15) / 16) + (w2.q != nullptr ? (int)((w2.n + 15) / 16) : 0) + (w2.q3 != nullptr ? (int)((w2.n3 + 15) / 16) : 0);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(NW * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // may request weights while the activation kernel runs
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const long long wait_clocks = (long long)g_opt_wait_limit_us.load(std::memory_order_relaxed) * 2000;  // about 2 GHz
    JQ_CUDA(cudaLaunchKernelEx(&cfg, gemv_q4k_i8_kernel<MT, STAGES, NW, OCC, Q5, PEER, FUSED>, v, w2, (const PeerOut*)(PEER ? peer.table : nullptr), image, x, rows,
                               bias, y, tiles, KS, max_tiles, wait_clocks));
    count_launch();
    return JQ_OK;
}

// Shared memory of one CTA: the ring's barriers, image slice, cross-warp reduction, carried sums, weight ring.
template <int MT, bool Q5>
size_t smem_bytes(int nw, int KS, int stages, bool sliced, int max_tiles) {
    return (size_t)nw * stages * 8 + (size_t)KS * Cfg<MT>::PB + (size_t)(2 * nw * 16 * MT) * sizeof(float) + (sliced ? (size_t)max_tiles * 16 * MT * sizeof(float) : 0) +
           (size_t)nw * stages * Blk<Q5>::SLOT;
}

// A launch shape: warps per CTA, CTAs per SM, ring stages. KS (the slice length) is a function of MT and k only, so
// that the summation order never depends on n: the whole k if its image fits beside the ring, else a multiple of the
// warps per CTA.
struct Shape {
    int nw, occ, stages;
};

template <int MT, bool Q5>
int run(const View& v, const Second& w2, const PeerOut& peer, const float* x, int rows, const float* bias, float* y, cudaStream_t s, uint8_t* image,
        bool* handled, bool may_fuse) {
    // x == nullptr: the image is already in `image` (written by a kernel earlier in the stream)
    const int KB = (int)(v.k / 256);
    const int tiles = (int)((v.n + 15) / 16) + (w2.q != nullptr ? (int)((w2.n + 15) / 16) : 0) + (w2.q3 != nullptr ? (int)((w2.n3 + 15) / 16) : 0);
    // Candidates, best first. Many rows of x make the image large: one CTA of 16 warps per SM shares one copy of it.
    constexpr bool WIDE = MT > 2;
    // (Three CTAs of 8 warps per SM, which 80 registers per thread allow, measured no faster than two on any shape and
    // slower on the small ones: the kernel is not short of warps.)
    const Shape unsliced[3] = {WIDE ? Shape{16, 1, 3} : Shape{8, 2, 3}, WIDE ? Shape{16, 1, 2} : Shape{8, 2, 3}, Shape{8, 2, 2}};
    const Shape sliced[2] = {WIDE ? Shape{16, 1, 2} : Shape{8, 2, 3}, Shape{8, 2, 2}};
    Shape sh{0, 0, 0};
    int KS = KB;
    for (int c = 0; c < 3 && sh.nw == 0; c++) {
        if (smem_bytes<MT, Q5>(unsliced[c].nw, KB, unsliced[c].stages, false, 0) <= SMEM_MAX / unsliced[c].occ - 1024) {
            sh = unsliced[c];
        }
    }
    if (sh.nw == 0) {
        for (int c = 0; c < 2 && sh.nw == 0; c++) {
            const size_t room = SMEM_MAX / sliced[c].occ - 1024 - 8 * 1024;  // 8 KB set aside for the carried sums
            const size_t rest = smem_bytes<MT, Q5>(sliced[c].nw, 0, sliced[c].stages, false, 0);
            const int ks = rest < room ? (int)((room - rest) / Cfg<MT>::PB) / sliced[c].nw * sliced[c].nw : 0;
            if (ks >= sliced[c].nw) {
                sh = sliced[c];
                KS = ks;
            }
        }
        if (sh.nw == 0) {
            *handled = false;
            return JQ_OK;
        }
    }
    const int grid = tiles < sm_count() * sh.occ ? tiles : sm_count() * sh.occ;
    const int max_tiles = (tiles + grid - 1) / grid;
    const bool is_sliced = KS < KB;
    const size_t smem = smem_bytes<MT, Q5>(sh.nw, KS, sh.stages, is_sliced, max_tiles);
    if (smem > SMEM_MAX / sh.occ - 1024) {
        *handled = false;  // more tiles per CTA than the carried sums have room for
        return JQ_OK;
    }
    *handled = true;
    // One or two rows of x and k <= 8192: the GEMV builds the image itself (every CTA makes all of it, which is redundant work
    // that grows with k; up to four super-blocks per warp it costs less than a launch and the scratch round trip). Not when
    // x lies in host memory: the image kernel reads it once, the thread blocks of the GEMV would each read it across PCIe.
    // With three to eight rows a warp would build eight parts for k = 4096, each behind a load of x from L2 (about 0.7
    // microseconds, two in flight): measured 3 microseconds slower per launch than the image kernel, so those rows keep it.
    constexpr bool CAN_FUSE = !WIDE;
    const bool fuse = CAN_FUSE && may_fuse && x != nullptr && KB <= 4 * sh.nw;
    if (x != nullptr && !fuse) {
        // launched programmatically as well: it is scheduled while the kernel before it still runs (it waits for that kernel
        // before touching memory) and lets the GEMV behind it be scheduled at once
        cudaLaunchConfig_t icfg = {};
        cudaLaunchAttribute iattr[1];
        iattr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        iattr[0].val.programmaticStreamSerializationAllowed = 1;
        icfg.attrs = iattr;
        icfg.numAttrs = WIDE ? 0 : 1;  // the 16-warp kernel fills an SM's registers: an early-scheduled successor only gets in its way
        icfg.stream = s;
        icfg.gridDim = dim3((unsigned)((KB * MT + PREP_WARPS - 1) / PREP_WARPS));
        icfg.blockDim = dim3(PREP_WARPS * 32);
        JQ_CUDA(cudaLaunchKernelEx(&icfg, q4k_activation_image_kernel<MT>, x, rows, (int64_t)v.k, image));
        count_launch();
    }
#define JQ_VARIANT(NWV, OCCV, STV, PEERV)                                                                                               \
    if constexpr (CAN_FUSE) {                                                                                                            \
        if (fuse) {                                                                                                                      \
            return launch<MT, STV, NWV, OCCV, Q5, PEERV, true>(v, w2, peer, image, x, rows, bias, y, s, KS, grid, max_tiles, smem);      \
        }                                                                                                                                \
    }                                                                                                                                    \
    if constexpr (true) {                                                                                                                \
        return launch<MT, STV, NWV, OCCV, Q5, PEERV, false>(v, w2, peer, image, nullptr, rows, bias, y, s, KS, grid, max_tiles, smem);   \
    }
#define JQ_SHAPE(NWV, OCCV, STV)                                   \
    if (sh.nw == NWV && sh.occ == OCCV && sh.stages == STV) {       \
        if (peer.world != 0) {                                      \
            JQ_VARIANT(NWV, OCCV, STV, true)                        \
        } else {                                                    \
            JQ_VARIANT(NWV, OCCV, STV, false)                       \
        }                                                           \
        return fail(JQ_ERR_UNSUPPORTED, "gemv_q4k_i8: no ready-made image is taken for this format and row count"); \
    }
    if constexpr (WIDE) {
        JQ_SHAPE(16, 1, 3)
        JQ_SHAPE(16, 1, 2)
    } else {
        JQ_SHAPE(8, 2, 3)
    }
    JQ_SHAPE(8, 2, 2)
#undef JQ_VARIANT
#undef JQ_SHAPE
    return fail(JQ_ERR_UNSUPPORTED, "gemv_q4k_i8: no kernel for the chosen launch shape");
}

}  // namespace

// Bytes of scratch (activation image) a Q4_K GEMV of `rows` activation rows over k inputs needs; 0 if the
// shape is not handled by the integer kernel.
size_t gemv_q4k_i8_scratch_bytes(int64_t k, int rows) {
    if (rows < 1 || rows > 8 || k <= 0) {
        return 0;
    }
    const size_t pb = rows == 1 ? Cfg<1>::PB : (rows == 2 ? Cfg<2>::PB : Cfg<8>::PB);
    return (size_t)(k / 256) * pb;
}

// Q4_K or Q5_K with rows in [1, 8] on a weight whose buffer is padded by 16 rows. `image` is a scratch buffer of
// gemv_q4k_i8_scratch_bytes(k, rows) bytes, 16-byte aligned, private to `s` until the GEMV kernel has run.
// *handled = false leaves the call to another kernel.
int launch_gemv_q4k_i8(const View& v, const float* x, int rows, const float* bias, float* y, cudaStream_t s, uint8_t* image, bool* handled,
                       const PeerOut* peer, bool x_remote) {
    *handled = false;
    if ((v.type != JQ_TYPE_Q4_K && v.type != JQ_TYPE_Q5_K) || v.n == 0 || v.k == 0 || rows > 8 || image == nullptr ||
        v.k / 256 >= (1 << 20)) {
        return JQ_OK;
    }
    const Second none{nullptr, 0, nullptr, 0x7fffffff, nullptr, 0, nullptr, 0x7fffffff};
    PeerOut local{};  // world = 0: results go to y
    const PeerOut& po = peer != nullptr ? *peer : local;
    if (v.type == JQ_TYPE_Q5_K) {
        if (rows == 1) return run<1, true>(v, none, po, x, rows, bias, y, s, image, handled, !x_remote);
        if (rows == 2) return run<2, true>(v, none, po, x, rows, bias, y, s, image, handled, !x_remote);
        return run<8, true>(v, none, po, x, rows, bias, y, s, image, handled, !x_remote);
    }
    if (rows == 1) return run<1, false>(v, none, po, x, rows, bias, y, s, image, handled, !x_remote);
    if (rows == 2) return run<2, false>(v, none, po, x, rows, bias, y, s, image, handled, !x_remote);
    return run<8, false>(v, none, po, x, rows, bias, y, s, image, handled, !x_remote);
}

// The same for two or three weights of one type and k on the same x: their rows follow one another in one launch, on one
// activation image (results in ys[i], [rows, n_i]; no bias).
int launch_gemv_q4k_i8_multi(const View* vs, int count, const float* x, int rows, float* const* ys, cudaStream_t s, uint8_t* image, bool* handled) {
    *handled = false;
    if (count < 2 || count > 3 || rows < 1 || rows > 8 || image == nullptr) {
        return JQ_OK;
    }
    const View& v = vs[0];
    for (int i = 0; i < count; i++) {
        if ((vs[i].type != JQ_TYPE_Q4_K && vs[i].type != JQ_TYPE_Q5_K) || vs[i].type != v.type || vs[i].k != v.k || vs[i].n == 0 || v.k == 0 ||
            v.k / 256 >= (1 << 20) || ys[i] == nullptr) {
            return JQ_OK;
        }
    }
    const int t1 = (int)((v.n + 15) / 16), t2 = t1 + (int)((vs[1].n + 15) / 16);
    const Second w2{vs[1].q, vs[1].n, ys[1], t1, count == 3 ? vs[2].q : nullptr, count == 3 ? vs[2].n : 0, count == 3 ? ys[2] : nullptr,
                    count == 3 ? t2 : 0x7fffffff};
    const PeerOut local{};
    if (v.type == JQ_TYPE_Q5_K) {
        if (rows == 1) return run<1, true>(v, w2, local, x, rows, nullptr, ys[0], s, image, handled, true);
        if (rows == 2) return run<2, true>(v, w2, local, x, rows, nullptr, ys[0], s, image, handled, true);
        return run<8, true>(v, w2, local, x, rows, nullptr, ys[0], s, image, handled, true);
    }
    if (rows == 1) return run<1, false>(v, w2, local, x, rows, nullptr, ys[0], s, image, handled, true);
    if (rows == 2) return run<2, false>(v, w2, local, x, rows, nullptr, ys[0], s, image, handled, true);
    return run<8, false>(v, w2, local, x, rows, nullptr, ys[0], s, image, handled, true);
}

#ifdef JQ_Q4K_TRACE
}  // namespace jq
extern "C" JQ_API int jq_debug_q4k_trace(long long* out, int* tickets) {
    if (cudaMemcpyFromSymbol(tickets, jq::g_q4k_ticket, sizeof(int)) != cudaSuccess) return -3;
    return cudaMemcpyFromSymbol(out, jq::g_q4k_tr, sizeof(jq::g_q4k_tr)) == cudaSuccess ? 0 : -3;
}
namespace jq {
#endif
int gemv_peer_status(int* status) {
    const int zero = 0;
    JQ_CUDA(cudaMemcpyFromSymbol(status, g_gemv_peer_status, sizeof(int)));
    JQ_CUDA(cudaMemcpyToSymbol(g_gemv_peer_status, &zero, sizeof(int)));
    return JQ_OK;
}

size_t q4k_image_bytes_one_row(int64_t k) { return (size_t)(k / 256) * Cfg<1>::PB; }

// One row of x whose image (q4k::build_image<1> per super-block) a kernel earlier in the stream has written to `image`;
// that kernel should execute griddepcontrol.launch_dependents so that this one can request weights meanwhile. With
// v2 != nullptr the rows of a second Q4_K weight with the same k follow in the same launch, results in y2, and with
// v3 != nullptr (only together with v2) those of a third, results in y3.
int launch_gemv_q4k_i8_imaged(const View& v, const View* v2, const uint8_t* image, const float* bias, float* y, float* y2, cudaStream_t s, bool* handled,
                              const PeerOut* peer, const View* v3, float* y3) {
    *handled = false;
    if (v.type != JQ_TYPE_Q4_K || v.n == 0 || v.k == 0 || image == nullptr || v.k / 256 >= (1 << 20) ||
        (v2 != nullptr && (v2->type != JQ_TYPE_Q4_K || v2->k != v.k || v2->n == 0 || y2 == nullptr)) ||
        (v3 != nullptr && (v2 == nullptr || v3->type != JQ_TYPE_Q4_K || v3->k != v.k || v3->n == 0 || y3 == nullptr))) {
        return JQ_OK;
    }
    const int t1 = (int)((v.n + 15) / 16), t2 = v2 != nullptr ? t1 + (int)((v2->n + 15) / 16) : 0x7fffffff;
    const Second w2{v2 != nullptr ? v2->q : nullptr, v2 != nullptr ? v2->n : 0, y2, v2 != nullptr ? t1 : 0x7fffffff,
                    v3 != nullptr ? v3->q : nullptr, v3 != nullptr ? v3->n : 0, y3, v3 != nullptr ? t2 : 0x7fffffff};
    const PeerOut local{};  // world = 0: results go to y (and y2)
    if (peer != nullptr && v2 != nullptr) {
        return JQ_OK;  // a second weight has no place in a peer's y
    }
    return run<1, false>(v, w2, peer != nullptr ? *peer : local, nullptr, 1, bias, y, s, const_cast<uint8_t*>(image), handled, false);
}

}  // namespace jq

// ---- an entry point that allocates nothing -------------------------------------------------------------------------
// jq_linear_f32 keeps the activation image in a scratch buffer that the library allocates with cudaMalloc the
// first time a stream needs one. Some callers cannot have that: a serving process that has handed every byte
// of device memory to its own pools fails the allocation, and cudaMalloc also makes the whole device wait,
// which a latency-bound decode loop on another stream would feel. For them the image lives in the array below,
// which is part of the loaded library image: every GPU that loads the library holds these bytes until the
// process exits, whether or not the entry point is ever called.
constexpr size_t NOALLOC_SCRATCH_BYTES = (size_t)1 << 20;
static __device__ __align__(256) uint8_t g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

namespace {

constexpr int NOALLOC_MAX_DEVICES = 64;
std::mutex g_noalloc_mu;
uint8_t* g_noalloc_addr[NOALLOC_MAX_DEVICES] = {};  // device address of g_noalloc_scratch, per device

// In host code `g_noalloc_scratch` is only a handle for the runtime, not an address a kernel can use: the device
// address has to be asked for, once per device and with that device current.
int noalloc_scratch_address(int device, uint8_t** out) {
    if (device < 0 || device >= NOALLOC_MAX_DEVICES) {
        return jq::fail(JQ_ERR_INVALID, "jq_linear_q4k_f32_noalloc: device %d is beyond the %d this entry point keeps addresses for", device,
                        NOALLOC_MAX_DEVICES);
    }
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (g_noalloc_addr[device] == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr) {
            return jq::cuda_fail(e, "cudaGetSymbolAddress(g_noalloc_scratch)");
        }
        g_noalloc_addr[device] = static_cast<uint8_t*>(p);
    }
    *out = g_noalloc_addr[device];
    return JQ_OK;
}

}  // namespace

extern "C" JQ_API int jq_linear_q4k_f32_noalloc(const jq_weight* w, const float* x, int64_t m, const float* bias, float* y, void* stream) {
    if (w == nullptr || w->magic != JQ_WEIGHT_MAGIC) {
        return jq::fail(JQ_ERR_INVALID, "jq_linear_q4k_f32_noalloc: not a live weight handle");
    }
    if (w->type != JQ_TYPE_Q4_K) {
        return jq::fail(JQ_ERR_UNSUPPORTED, "jq_linear_q4k_f32_noalloc: the weight is not Q4_K (type id %d)", w->type);
    }
    if (m < 1 || m > 8) {
        return jq::fail(JQ_ERR_INVALID, "jq_linear_q4k_f32_noalloc: %lld activation rows, this entry point takes 1 to 8", (long long)m);
    }
    if (x == nullptr || y == nullptr || (((uintptr_t)x | (uintptr_t)y) & 15) != 0) {
        return jq::fail(JQ_ERR_INVALID, "jq_linear_q4k_f32_noalloc: x and y must be non-null, 16-byte aligned device pointers");
    }
    if (w->n == 0) {
        return JQ_OK;
    }
    const size_t need = jq::gemv_q4k_i8_scratch_bytes(w->k, (int)m);
    if (need == 0 || need > NOALLOC_SCRATCH_BYTES) {
        return jq::fail(JQ_ERR_INVALID,
                        "jq_linear_q4k_f32_noalloc: k = %lld with %lld rows needs %zu bytes of activation image, the built-in scratch holds %zu", (long long)w->k,
                        (long long)m, need, NOALLOC_SCRATCH_BYTES);
    }
    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess) {
        prev = -1;
    }
    if (prev != w->device && cudaSetDevice(w->device) != cudaSuccess) {
        return jq::fail(JQ_ERR_CUDA, "jq_linear_q4k_f32_noalloc: cannot select device %d", w->device);
    }
    uint8_t* image = nullptr;
    int rc = noalloc_scratch_address(w->device, &image);
    if (rc == JQ_OK) {
        bool handled = false;
        const jq::View v{w->q, w->aux, w->n, w->k, w->type};
        rc = jq::launch_gemv_q4k_i8(v, x, (int)m, bias, y, (cudaStream_t)stream, image, &handled);
        if (rc == JQ_OK && !handled) {
            rc = jq::fail(JQ_ERR_UNSUPPORTED, "jq_linear_q4k_f32_noalloc: shape [%lld, %lld] x %lld rows is outside what the tensor-core kernel takes",
                          (long long)w->n, (long long)w->k, (long long)m);
        }
    }
    if (prev >= 0 && prev != w->device) {
        cudaSetDevice(prev);
    }
    return rc;
}
