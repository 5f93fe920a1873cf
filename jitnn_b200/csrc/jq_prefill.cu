// Prefill GEMM: y[m, n] = x[m, k] . W[n, k]^T for many activation rows (m >= 128 is where it pays), x in bfloat16,
// W in a GGUF block format, FP32 accumulation on the 5th-generation tensor cores (tcgen05.mma, accumulator in TMEM).
//
// Replaces the reference's prefill composition (ops/Gguf.java:94-95: dequantise the whole weight to an FP32 [N, K]
// tensor, then an FP32 CUDA-core GEMM, ops/MatMul.java:488-554): the weight is never materialised. A CTA owns a tile
// of 128 output features x 128 or 256 tokens and walks k in stages of 64:
//   * one thread issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle, no multicast) of the activation tile
//     [tokens x 64 k] into shared memory;
//   * 256 dequantiser threads (two per output feature) decode their row's 64 weights of the stage with the bit-exact
//     per-format decoders, round them to bfloat16 and store them in the same 128-byte-swizzled K-major layout;
//   * one thread issues four tcgen05.mma (M = 128 features, N = 128 or 256 tokens, K = 16) per stage and commits the
//     stage's "empty" barrier; the accumulator D[feature][token] (128 lanes x N columns of FP32) lives in tensor memory;
//   * after the last stage the dequantiser warps read the accumulator with tcgen05.ld (32 lanes x 32 columns
//     at a time) and store y[token][feature] (32 consecutive features per warp store: coalesced), adding the bias.
// Every mbarrier wait is bounded: a wait that does not complete within its poll budget records a status code in
// g_prefill_status, raises the CTA's abort flag and all roles fall through to the common exit, where tensor memory
// is released. Nothing here waits on another CTA or another GPU.
#include <cuda.h>
#include <cuda_bf16.h>

#include <mutex>

#include "jq_formats.cuh"
#include "jq_tc.cuh"

namespace jq {

// 0 = fine; otherwise the code of the first wait that gave up (1 empty slot, 2 weights ready, 3 activations ready,
// 4 accumulator ready) since the status was last cleared.
static __device__ int g_prefill_status;

namespace {

constexpr int TILE_F = 128;    // output features per CTA (MMA M)
constexpr int STAGE_K = 64;    // k per stage: 64 bf16 = 128 bytes = one swizzle row
// Pipeline stages: 4 for the 256-token tile (one CTA per SM), 3 for the 128-token tile, whose 97 KB let two CTAs share an SM
// (one dequantises while the other's MMAs run).
__host__ __device__ constexpr int stages_of(int tile_t, int nf) { return nf == 2 ? (tile_t == 128 ? 4 : 3) : (tile_t == 128 ? 3 : 4); }
constexpr int A_BYTES = TILE_F * STAGE_K * 2;
constexpr int DQ_THREADS = 256;  // two dequantiser threads per output feature, 32 weights each per stage
constexpr int THREADS = 64 + DQ_THREADS;  // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-9: dequantise, then epilogue

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Waits for the phase with the given parity; gives up after WAIT_CLOCKS of the SM's clock (a poll may suspend the thread for
// a time the hardware chooses, so the bound counts time, not polls) or when another role aborted.
constexpr long long WAIT_CLOCKS = 4000000000ll;  // about two seconds
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    if (mbar_try(bar, parity)) {
        return true;
    }
    const long long t0 = clock64();
    for (uint32_t i = 0;; i++) {
        if (mbar_try(bar, parity)) {
            return true;
        }
        if ((i & 63u) == 63u) {
            if (*abort_flag != 0) {
                return false;
            }
            if (clock64() - t0 > WAIT_CLOCKS) {
                break;
            }
        }
    }
    atomicCAS(&g_prefill_status, 0, code);
    *abort_flag = 1;
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                 "l"(map), "r"(bar), "r"(c0), "r"(c1)
                 : "memory");
}

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128 bytes, 8-row atoms 1024 bytes
// apart (stride byte offset), leading byte offset 1 (unused with swizzled K-major tiles), descriptor version 1
// (sm_100), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

// Instruction descriptor of kind::f16: D = F32 (bits 4-5 = 1), A and B = BF16 (bits 7-9 and 10-12 = 1), both K-major,
// N >> 3 in bits 17-22, M >> 4 in bits 24-28.
constexpr uint32_t idesc_of(int tile_t) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(tile_t >> 3) << 17) | ((uint32_t)(TILE_F >> 4) << 24);
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// A dequantiser thread's share of the 64 weights k0 .. k0 + 63 of its row: TASKS (block, unit) pairs of the format's
// decoder. `part` (0 or 1) says which half of the chunk's units the thread takes.
template <int TYPE>
struct ChunkTasks {
    using F = Fmt<TYPE>;
    static constexpr int TASKS = TYPE == JQ_TYPE_Q8_0 ? 2 : 1;
    __device__ static void of(const View& v, int64_t row, int k0, int part, int64_t (&block)[TASKS], int (&unit)[TASKS], int (&base)[TASKS]) {
        const int blocks_per_row = (int)(v.k / F::QK);
        if (TYPE == JQ_TYPE_Q4_K || TYPE == JQ_TYPE_Q5_K) {
            block[0] = row * blocks_per_row + k0 / 256;
            unit[0] = 2 * ((k0 & 255) >> 6) + part;  // group j = chunk index inside the block, units 2j and 2j + 1
            base[0] = k0 & ~255;
        } else if (TYPE == JQ_TYPE_Q6_K) {
            block[0] = row * blocks_per_row + k0 / 256;
            unit[0] = 2 * ((k0 & 255) >> 7) + part;  // half n of the block, units 2n and 2n + 1 (two of their four runs are used)
            base[0] = k0 & ~255;
        } else if (TYPE == JQ_TYPE_Q8_0) {
#pragma unroll
            for (int i = 0; i < TASKS; i++) {        // two blocks of 32 per chunk, unit `part` (16 values) of each
                block[i] = row * blocks_per_row + k0 / 32 + i;
                unit[i] = part;
                base[i] = k0 + 32 * i;
            }
        } else {                                     // Q4_0, Q4_1: one unit per block of 32, block `part` of the chunk
            block[0] = row * blocks_per_row + k0 / 32 + part;
            unit[0] = 0;
            base[0] = k0 + 32 * part;
        }
    }
};

// Rounds a run of 16 consecutive weights to bfloat16 and writes it into a 128-byte row of the swizzled A tile:
// the run starts at 16-byte chunk c, and chunk c lands at position c ^ (row & 7).
__device__ __forceinline__ void store_run(const float (&w)[16], int c, uint8_t* a_row, int swz) {
    uint4 lo, hi;
    __nv_bfloat162 t;
    t = __floats2bfloat162_rn(w[0], w[1]);   lo.x = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(w[2], w[3]);   lo.y = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(w[4], w[5]);   lo.z = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(w[6], w[7]);   lo.w = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(w[8], w[9]);   hi.x = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(w[10], w[11]); hi.y = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(w[12], w[13]); hi.z = *reinterpret_cast<uint32_t*>(&t);
    t = __floats2bfloat162_rn(w[14], w[15]); hi.w = *reinterpret_cast<uint32_t*>(&t);
    *reinterpret_cast<uint4*>(a_row + ((c ^ swz) << 4)) = lo;
    *reinterpret_cast<uint4*>(a_row + (((c + 1) ^ swz) << 4)) = hi;
}

// Byte i of `packed` as the float 2^23 + byte: one byte permute builds the bit pattern 0x4B0000bb. The integer to
// float conversion instruction runs at a quarter of the rate of the floating-point pipe, this does not.
__device__ __forceinline__ float magic_byte(uint32_t packed, int i) {
    return __uint_as_float(__byte_perm(packed, 0x4B000000u, 0x7440u + (uint32_t)i));
}
constexpr float MAGIC = 8388608.0f;  // 2^23

// Converts loaded raw units, rounds to bfloat16 and writes them into the 128-byte row `a_row` of the swizzled A tile.
// Q4_K and Q6_K take a route without integer to float conversions that gives the reference's values
// (GgufKernels.java:101-111, 127-140) bit for bit, except that a zero may come out as +0 where the reference has -0,
// which no product or sum can tell apart:
//   Q4_K  (d sc) q - dmin m:  fma(a, 2^23 + q, -(a 2^23)) rounds the exact product a q once, as the reference's multiply
//                             does (a 2^23 is exact), then the separately rounded subtraction follows;
//   Q6_K  (d sc) (q - 32):    (2^23 + q) - (2^23 + 32) is exact, then the same single multiply as the reference.
// The other formats go through the bit-exact decoder of jq_formats.cuh.
template <int TYPE>
__device__ __forceinline__ void convert_store(const typename Fmt<TYPE>::Raw (&raw)[ChunkTasks<TYPE>::TASKS], const int (&unit)[ChunkTasks<TYPE>::TASKS],
                                              const int (&base)[ChunkTasks<TYPE>::TASKS], int k0, uint8_t* a_row, int swz) {
    using F = Fmt<TYPE>;
    if constexpr (TYPE == JQ_TYPE_Q4_K) {
        const uint4 h = raw[0].h, q = raw[0].q;
        const int j = unit[0] >> 1, hf = unit[0] & 1;
        const float d = half_bits_to_float(h.x), dmin = half_bits_to_float(h.x >> 16);
        int sc0, mn0, sc1, mn1;
        k_scale_min(h.y, h.z, h.w, 2 * j, sc0, mn0);
        k_scale_min(h.y, h.z, h.w, 2 * j + 1, sc1, mn1);
        const float a0 = __fmul_rn(d, (float)sc0), m0 = __fmul_rn(dmin, (float)mn0);
        const float a1 = __fmul_rn(d, (float)sc1), m1 = __fmul_rn(dmin, (float)mn1);
        const float c0 = -__fmul_rn(a0, MAGIC), c1 = -__fmul_rn(a1, MAGIC);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        float lo[16], hi[16];
#pragma unroll
        for (int x = 0; x < 4; x++) {
            const uint32_t ln = w[x] & 0x0f0f0f0fu, hn = (w[x] >> 4) & 0x0f0f0f0fu;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                lo[4 * x + i] = __fsub_rn(__fmaf_rn(a0, magic_byte(ln, i), c0), m0);
                hi[4 * x + i] = __fsub_rn(__fmaf_rn(a1, magic_byte(hn, i), c1), m1);
            }
        }
        store_run(lo, 2 * hf, a_row, swz);      // elements 16 hf .. of sub-block 2j
        store_run(hi, 4 + 2 * hf, a_row, swz);  // and of sub-block 2j + 1
    } else if constexpr (TYPE == JQ_TYPE_Q6_K) {
        // unit (n, c) holds four runs; this 64-wide chunk is pair p of half n: runs 2p and 2p + 1
        const int c = unit[0] & 1, p = (k0 & 127) >> 6;
        const uint4 la = raw[0].la, lb = raw[0].lb, hq = raw[0].hq, sv = raw[0].sv;
        const float d = half_bits_to_float(raw[0].d);
        const uint32_t sw = (unit[0] >> 1) == 0 ? (p == 0 ? sv.x : sv.y) : (p == 0 ? sv.z : sv.w);  // scales 8n + 4p .. + 3
        const float a0 = __fmul_rn(d, (float)(int)(int8_t)byte_of(sw, c));
        const float a1 = __fmul_rn(d, (float)(int)(int8_t)byte_of(sw, c + 2));
        const uint32_t wa[4] = {la.x, la.y, la.z, la.w}, wb[4] = {lb.x, lb.y, lb.z, lb.w}, wh[4] = {hq.x, hq.y, hq.z, hq.w};
        float r0[16], r1[16];
#pragma unroll
        for (int x = 0; x < 4; x++) {
            const uint32_t hx = wh[x] >> (4 * p);
            const uint32_t qa = ((wa[x] >> (4 * p)) & 0x0f0f0f0fu) | ((hx & 0x03030303u) << 4);
            const uint32_t qb = ((wb[x] >> (4 * p)) & 0x0f0f0f0fu) | ((hx & 0x0c0c0c0cu) << 2);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                r0[4 * x + i] = __fmul_rn(a0, __fsub_rn(magic_byte(qa, i), MAGIC + 32.0f));
                r1[4 * x + i] = __fmul_rn(a1, __fsub_rn(magic_byte(qb, i), MAGIC + 32.0f));
            }
        }
        store_run(r0, 2 * c, a_row, swz);
        store_run(r1, 4 + 2 * c, a_row, swz);
    } else {
#pragma unroll
        for (int i = 0; i < ChunkTasks<TYPE>::TASKS; i++) {
            float w[F::RUNS][16];
            int pos[F::RUNS];
            F::convert(raw[i], unit[i], w, pos);
#pragma unroll
            for (int r = 0; r < F::RUNS; r++) {
                const int rel = base[i] + pos[r] - k0;  // position of the run inside the chunk
                if (rel >= 0 && rel < STAGE_K) {
                    store_run(w[r], rel >> 3, a_row, swz);
                }
            }
        }
    }
}

// NF = 1 or 2 feature tiles of 128 rows per CTA. With two, every activation tile that the TMA brings in from L2 feeds two
// accumulators (TMEM columns [0, TILE_T) and [TILE_T, 2 TILE_T)), which halves the L2-to-SM traffic per flop; the CTA then
// has 16 dequantiser warps.
// SPLIT: gridDim.z = 2 CTAs share a tile, each takes half of k and adds its result into a zeroed y.
template <int TYPE, int TILE_T, int NF, bool SPLIT>
__global__ void __launch_bounds__(64 + NF * DQ_THREADS, (TILE_T == 128 && NF == 1) ? 2 : 1)
    prefill_tcgen05_kernel(View v, const __grid_constant__ CUtensorMap xmap, int m, const float* __restrict__ bias, float* __restrict__ y) {
    constexpr int B_BYTES = TILE_T * STAGE_K * 2;
    constexpr int STAGES = stages_of(TILE_T, NF);
    constexpr uint32_t IDESC = idesc_of(TILE_T);
    extern __shared__ uint8_t smem_unaligned[];
    // the swizzled tiles must start on 1024-byte boundaries of the shared address space
    uint8_t* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    // [STAGES][NF][A_BYTES] weights, [STAGES][B_BYTES] activations (1024-byte aligned tiles), then barriers
    uint8_t* a_tiles = smem;
    uint8_t* b_tiles = smem + STAGES * NF * A_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * (NF * A_BYTES + B_BYTES));
    // bars: full_a[S], full_b[S], empty[S], accum
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * STAGES + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f0 = blockIdx.x * (NF * TILE_F), t0 = blockIdx.y * TILE_T;
    const int KT_all = (int)(v.k / STAGE_K);
    // SPLIT: k is cut into gridDim.z ranges, CTA z takes stages [z KT_all / S, (z + 1) KT_all / S) and leaves its partial
    // sums in part z of the buffer at y ([S][m][n]); split_sum_kernel adds the parts in order afterwards.
    const int it0 = SPLIT ? (int)(((int64_t)blockIdx.z * KT_all) / (int)gridDim.z) : 0;  // first 64-wide stage of k of this CTA
    const int KT = SPLIT ? (int)(((int64_t)(blockIdx.z + 1) * KT_all) / (int)gridDim.z) - it0 : KT_all;  // and their number
    const uint32_t bar0 = smem_u32(bars);
    auto full_a = [&](int s) { return bar0 + 8u * (uint32_t)s; };
    auto full_b = [&](int s) { return bar0 + 8u * (uint32_t)(STAGES + s); };
    auto empty = [&](int s) { return bar0 + 8u * (uint32_t)(2 * STAGES + s); };
    const uint32_t accum = bar0 + 8u * (uint32_t)(3 * STAGES);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full_a(s), NF * DQ_THREADS);
            mbar_init(full_b(s), 1);
            mbar_init(empty(s), 1);
        }
        mbar_init(accum, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(NF * TILE_T) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        // ---- activation tiles by TMA ------------------------------------------------------------------------------
        if (lane == 0) {
            for (int it = 0; it < KT; it++) {
                const int s = it % STAGES;
                const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                if (!mbar_wait(empty(s), ph ^ 1u, abort_flag, 1)) {
                    break;
                }
                mbar_expect_tx(full_b(s), B_BYTES);
                tma_load_2d(smem_u32(b_tiles + s * B_BYTES), &xmap, full_b(s), (it0 + it) * STAGE_K, t0);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issue ---------------------------------------------------------------------------------------------
        if (lane == 0) {
            bool ok = true;
            for (int it = 0; it < KT && ok; it++) {
                const int s = it % STAGES;
                const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
                ok = mbar_wait(full_a(s), ph, abort_flag, 2) && mbar_wait(full_b(s), ph, abort_flag, 3);
                if (!ok) {
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t bd = smem_desc(smem_u32(b_tiles + s * B_BYTES));
#pragma unroll
                for (int f = 0; f < NF; f++) {
                    const uint64_t ad = smem_desc(smem_u32(a_tiles + (s * NF + f) * A_BYTES));
#pragma unroll
                    for (int ks = 0; ks < STAGE_K / 16; ks++) {
                        // 16 k = 32 bytes further inside the swizzle row: +2 in the (address >> 4) field
                        umma(tmem + (uint32_t)(f * TILE_T), ad + 2u * ks, bd + 2u * ks, IDESC, (it | ks) != 0 ? 1u : 0u);
                    }
                }
                umma_commit(empty(s));  // arrives when the MMAs that read this stage have finished
            }
            if (ok) {
                umma_commit(accum);
            }
        }
    } else {
        // ---- dequantise: threads i and 128 + i own feature row f0 + i (rows past n repeat the last row; never stored); the
        // two halves of a row's chunk go to different warps so that no warp diverges
        const int i = (threadIdx.x - 64) & 127, part = ((threadIdx.x - 64) >> 7) & 1, sub = (threadIdx.x - 64) >> 8;  // sub: feature tile
        int64_t row = (int64_t)f0 + sub * TILE_F + i;
        row = row < v.n ? row : v.n - 1;
        const uint32_t row_off = (uint32_t)((i >> 3) * 1024 + (i & 7) * 128);
        bool ok = true;
        // the raw blocks of the next stage are requested before the current stage is converted
        using CT = ChunkTasks<TYPE>;
        typename Fmt<TYPE>::Raw cur[CT::TASKS], nxt[CT::TASKS];
        int64_t blk[CT::TASKS];
        int unit[CT::TASKS], base[CT::TASKS], unit_n[CT::TASKS], base_n[CT::TASKS];
        CT::of(v, row, it0 * STAGE_K, part, blk, unit, base);
#pragma unroll
        for (int q = 0; q < CT::TASKS; q++) {
            Fmt<TYPE>::load(v, blk[q], unit[q], cur[q]);
        }
        for (int it = 0; it < KT; it++) {
            const int s = it % STAGES;
            const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
            if (it + 1 < KT) {
                CT::of(v, row, (it0 + it + 1) * STAGE_K, part, blk, unit_n, base_n);
                if (TYPE == JQ_TYPE_Q6_K && ((it0 + it + 1) & 1)) {
                    nxt[0] = cur[0];  // the second 64 weights of a half come from the unit that is already loaded
                } else {
#pragma unroll
                    for (int q = 0; q < CT::TASKS; q++) {
                        Fmt<TYPE>::load(v, blk[q], unit_n[q], nxt[q]);
                    }
                }
            }
            if (!mbar_wait(empty(s), ph ^ 1u, abort_flag, 1)) {
                ok = false;
                break;
            }
            convert_store<TYPE>(cur, unit, base, (it0 + it) * STAGE_K, a_tiles + (s * NF + sub) * A_BYTES + row_off, i & 7);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> visible to the tensor core
            mbar_arrive(full_a(s));
#pragma unroll
            for (int q = 0; q < CT::TASKS; q++) {
                cur[q] = nxt[q];
                unit[q] = unit_n[q];
                base[q] = base_n[q];
            }
        }
        // ---- epilogue: accumulator -> y --------------------------------------------------------------------------------
        if (ok && mbar_wait(accum, 0, abort_flag, 4)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int lane_group = warp & 3;  // a warp may only read TMEM lanes 32 (warp % 4) .. + 31
            const int col_half = ((warp - 2) >> 2) & 1;  // the two warps of a lane group and feature tile split the token columns
            const int feature = f0 + sub * TILE_F + lane_group * 32 + lane;
            const float b = (bias != nullptr && feature < v.n && !SPLIT) ? bias[feature] : 0.0f;
            float* const out = SPLIT ? y + (int64_t)blockIdx.z * m * v.n : y;
#pragma unroll 1
            for (int c = col_half * (TILE_T / 64); c < (col_half + 1) * (TILE_T / 64); c++) {
                uint32_t r[32];
                const uint32_t taddr = tmem + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(sub * TILE_T + c * 32);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                      "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
                      "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
                      "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (feature < v.n) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int token = t0 + c * 32 + j;
                        if (token < m) {
                            out[(int64_t)token * v.n + feature] = __uint_as_float(r[j]) + b;
                        }
                    }
                }
            }
        }
    }
    // ---- common exit: everyone arrives, then the owning warp releases tensor memory -------------------------------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0 && lane == 0 && *abort_flag != 0) {
        // after an abort, give activation copies that may still be in flight a bounded time to land
        for (int s = 0; s < STAGES; s++) {
            for (uint32_t p = 0; p < (1u << 16); p++) {
                if (mbar_try(full_b(s), 0) || mbar_try(full_b(s), 1)) {
                    break;
                }
            }
        }
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(NF * TILE_T) : "memory");
    }
}

// y = parts[0] + parts[1] + ... (in that order) + bias: the second stage of a linear whose k was cut into ranges.
// Four elements per thread where the row length allows 16-byte accesses.
template <bool VEC>
__global__ void split_sum_kernel(const float* __restrict__ parts, int nparts, int64_t count, int64_t n, const float* __restrict__ bias,
                                 float* __restrict__ y) {
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * (VEC ? 4 : 1);
    if (i >= count) {
        return;
    }
    if constexpr (VEC) {
        float4 sum = *reinterpret_cast<const float4*>(parts + i);
        for (int p = 1; p < nparts; p++) {
            const float4 a = *reinterpret_cast<const float4*>(parts + (int64_t)p * count + i);
            sum.x += a.x; sum.y += a.y; sum.z += a.z; sum.w += a.w;
        }
        if (bias != nullptr) {
            const float4 b = *reinterpret_cast<const float4*>(bias + i % n);
            sum.x += b.x; sum.y += b.y; sum.z += b.z; sum.w += b.w;
        }
        *reinterpret_cast<float4*>(y + i) = sum;
    } else {
        float sum = parts[i];
        for (int p = 1; p < nparts; p++) {
            sum += parts[(int64_t)p * count + i];
        }
        y[i] = bias != nullptr ? sum + bias[i % n] : sum;
    }
}

// fp32 -> bf16 (round to nearest even, as the reference's LowPrecision.java:36-46), for jq_linear_f32's prefill option
__global__ void f32_to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out, int64_t count) {
    int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < count) {
        const float4 v = *reinterpret_cast<const float4*>(x + i);
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<uint2*>(out + i) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
    } else {
        for (; i < count; i++) {
            out[i] = __float2bfloat16_rn(x[i]);
        }
    }
}

template <int TYPE, int TILE_T, int NF, bool SPLIT>
int launch_typed(const View& v, const CUtensorMap& xmap, int m, const float* bias, float* y, cudaStream_t s, int ksplit) {
    constexpr int B_BYTES = TILE_T * STAGE_K * 2;
    constexpr int STAGES = stages_of(TILE_T, NF);
    const size_t smem = (size_t)STAGES * (NF * A_BYTES + B_BYTES) + 256 + 1024;  // tiles + barriers + slack for the 1024-byte alignment
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    JQ_CUDA(cudaGetDevice(&dev));
    if ((configured.load() >> (dev & 63) & 1) == 0) {
        JQ_CUDA(cudaFuncSetAttribute(prefill_tcgen05_kernel<TYPE, TILE_T, NF, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured.fetch_or((uint64_t)1 << (dev & 63));
    }
    float* out = y;
    if (SPLIT) {
        uint8_t* parts = nullptr;
        int rc = scratch_for_slot(s, 3, (size_t)ksplit * m * v.n * sizeof(float), &parts);
        if (rc != JQ_OK) {
            return rc;
        }
        out = reinterpret_cast<float*>(parts);
    }
    dim3 grid((unsigned)((v.n + NF * TILE_F - 1) / (NF * TILE_F)), (unsigned)((m + TILE_T - 1) / TILE_T), SPLIT ? (unsigned)ksplit : 1u);
    prefill_tcgen05_kernel<TYPE, TILE_T, NF, SPLIT><<<grid, 64 + NF * DQ_THREADS, smem, s>>>(v, xmap, m, bias, out);
    count_launch();
    int rc = check_launch("prefill_tcgen05_kernel");
    if (rc == JQ_OK && SPLIT) {
        const int64_t count = (int64_t)m * v.n;
        if (v.n % 4 == 0 && (((uintptr_t)y | (uintptr_t)bias) & 15) == 0) {
            split_sum_kernel<true><<<(unsigned)((count / 4 + 255) / 256), 256, 0, s>>>(out, ksplit, count, v.n, bias, y);
        } else {
            split_sum_kernel<false><<<(unsigned)((count + 255) / 256), 256, 0, s>>>(out, ksplit, count, v.n, bias, y);
        }
        count_launch();
        rc = check_launch("split_sum_kernel");
    }
    return rc;
}

}  // namespace

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(p);
        }
    });
    return fn;
}

bool prefill_supported(const View& v) {
    return has_linear_kernel(v.type) && v.k % STAGE_K == 0 && v.n > 0 && v.k > 0;
}

// y[m, n] = x_bf16[m, k] . W^T (+ bias); x 16-byte aligned device memory.
int launch_prefill_bf16(const View& v, const uint16_t* x_bf16, int64_t m, const float* bias, float* y, cudaStream_t s) {
    if (!prefill_supported(v)) {
        return fail(JQ_ERR_UNSUPPORTED, "prefill: the tensor-core kernel needs k to be a multiple of 64 (k = %lld)", (long long)v.k);
    }
    EncodeTiledFn enc = encode_tiled();
    if (enc == nullptr) {
        return fail(JQ_ERR_CUDA, "prefill: cuTensorMapEncodeTiled is not available from this driver");
    }
    CUtensorMap xmap;
    const cuuint64_t dims[2] = {(cuuint64_t)v.k, (cuuint64_t)m};
    const cuuint64_t strides[1] = {(cuuint64_t)v.k * 2};
    // Tile shape: 128 or 256 tokens x 128 or 256 features per CTA. More tokens per CTA spread the dequantisation of a weight
    // tile over more tensor work, two feature tiles halve the activation traffic from L2, but both leave fewer CTAs for
    // the 148 SMs. Chosen by a small cost model: waves of CTAs x the measured time of one wave (microseconds at k = 4096,
    // the same for every k up to a common factor).
    int tile_t = 128, nf = 1, ksplit = 1;
    {
        const int ts[4] = {128, 256, 128, 256}, nfs[4] = {1, 1, 2, 2};
        const double wave_us[4] = {44.0, 49.0, 67.0, 78.0};
        double best = 0.0;
        for (int c = 0; c < 4; c++) {
            if (ts[c] == 256 && m <= 128) {
                continue;
            }
            const int64_t ctas = ((v.n + 128 * nfs[c] - 1) / (128 * nfs[c])) * ((m + ts[c] - 1) / ts[c]);
            // Any shape can also take k in 2 to 4 ranges: the CTAs of a tile leave partial sums in a scratch buffer and a
            // second small kernel adds them in order (the same result whoever finishes first). That fills SMs which few
            // tiles leave idle and evens out the last wave. A part-k CTA costs a little more than its share, and the
            // second kernel reads every part once (from L2, mostly).
            const double kf = (double)v.k / 4096.0;
            const int max_split = v.k / STAGE_K >= 32 ? 4 : 1;
            for (int ks = 1; ks <= max_split; ks++) {
                const double part_bytes = (double)ks * m * v.n * 4.0;
                if (ks > 1 && part_bytes > 192e6) {
                    break;  // the parts stay in a scratch buffer for good: not for very long prompts
                }
                // (measured: with a smaller fixed cost the model cuts 11008 x 4096 in three and loses 20 microseconds)
                const double cost = (double)((ctas * ks + 147) / 148) * wave_us[c] * kf / ks * (ks > 1 ? 1.1 : 1.0) +
                                    (ks > 1 ? 8.0 + part_bytes / 5e6 : 0.0);  // microseconds
                if ((c == 0 && ks == 1) || cost < best) {
                    best = cost;
                    tile_t = ts[c];
                    nf = nfs[c];
                    ksplit = ks;
                }
            }
        }
    }
    const cuuint32_t box[2] = {STAGE_K, (cuuint32_t)tile_t};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t*>(x_bf16), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return fail(JQ_ERR_CUDA, "prefill: cuTensorMapEncodeTiled failed with code %d", (int)r);
    }
#define JQ_PREFILL_CASE(T)                                                                         \
    case T:                                                                                          \
        if (ksplit > 1) {                                                                            \
            return nf == 2 ? (tile_t == 256 ? launch_typed<T, 256, 2, true>(v, xmap, (int)m, bias, y, s, ksplit) : launch_typed<T, 128, 2, true>(v, xmap, (int)m, bias, y, s, ksplit)) \
                           : (tile_t == 256 ? launch_typed<T, 256, 1, true>(v, xmap, (int)m, bias, y, s, ksplit) : launch_typed<T, 128, 1, true>(v, xmap, (int)m, bias, y, s, ksplit)); \
        }                                                                                            \
        return nf == 2 ? (tile_t == 256 ? launch_typed<T, 256, 2, false>(v, xmap, (int)m, bias, y, s, 1) : launch_typed<T, 128, 2, false>(v, xmap, (int)m, bias, y, s, 1)) \
                       : (tile_t == 256 ? launch_typed<T, 256, 1, false>(v, xmap, (int)m, bias, y, s, 1) : launch_typed<T, 128, 1, false>(v, xmap, (int)m, bias, y, s, 1));
    switch (v.type) {
        JQ_PREFILL_CASE(JQ_TYPE_Q8_0)
        JQ_PREFILL_CASE(JQ_TYPE_Q4_0)
        JQ_PREFILL_CASE(JQ_TYPE_Q4_1)
        JQ_PREFILL_CASE(JQ_TYPE_Q4_K)
        JQ_PREFILL_CASE(JQ_TYPE_Q5_K)
        JQ_PREFILL_CASE(JQ_TYPE_Q6_K)
        default:
            return fail(JQ_ERR_UNSUPPORTED, "prefill: type %d has no tensor-core kernel", v.type);
    }
#undef JQ_PREFILL_CASE
}

int launch_f32_to_bf16(const float* x, uint16_t* out, int64_t count, cudaStream_t s) {
    if (count == 0) {
        return JQ_OK;
    }
    const int64_t threads = (count + 3) / 4;
    f32_to_bf16_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, s>>>(x, reinterpret_cast<__nv_bfloat16*>(out), count);
    count_launch();
    return check_launch("f32_to_bf16_kernel");
}

// Reads and clears the status word of the prefill kernel on the current device (0 = no wait ever gave up).
int prefill_status(int* status) {
    int zero = 0;
    JQ_CUDA(cudaMemcpyFromSymbol(status, g_prefill_status, sizeof(int)));
    JQ_CUDA(cudaMemcpyToSymbol(g_prefill_status, &zero, sizeof(int)));
    return JQ_OK;
}

}  // namespace jq
