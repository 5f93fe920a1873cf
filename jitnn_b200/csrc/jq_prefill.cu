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

namespace jq {

// 0 = fine; otherwise the code of the first wait that gave up (1 empty slot, 2 weights ready, 3 activations ready,
// 4 accumulator ready) since the status was last cleared.
static __device__ int g_prefill_status;

__host__ __device__ constexpr int plane_q_bytes_dev(int type) {
    return type == JQ_TYPE_Q8_0 ? 32 : 16;  // Q8_0, Q4_0, Q4_1 quant planes
}

namespace {

constexpr int TILE_F = 128;    // output features per CTA (MMA M)
constexpr int STAGE_K = 64;    // k per stage: 64 bf16 = 128 bytes = one swizzle row
constexpr int STAGES = 4;
constexpr int A_BYTES = TILE_F * STAGE_K * 2;
constexpr int DQ_THREADS = 256;  // two dequantiser threads per output feature, 32 weights each per stage
constexpr int THREADS = 64 + DQ_THREADS;  // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-9: dequantise, then epilogue
constexpr uint32_t POLL_LIMIT = 1u << 24;

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

// Waits for the phase with the given parity; gives up after POLL_LIMIT polls or when another role aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    for (uint32_t i = 0; i < POLL_LIMIT; i++) {
        if (mbar_try(bar, parity)) {
            return true;
        }
        if ((i & 1023u) == 1023u && *abort_flag != 0) {
            return false;
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

// Pulls the bytes that dequant_row_chunk will read for [k0, k0 + 64) of `row` towards the SM ahead of time.
template <int TYPE>
__device__ __forceinline__ void prefetch_row_chunk(const View& v, int64_t row, int k0) {
    using F = Fmt<TYPE>;
    const int blocks_per_row = (int)(v.k / F::QK);
    const int64_t block = row * blocks_per_row + k0 / F::QK;
    const int o = k0 % F::QK;
    const uint8_t* p;
    if (TYPE == JQ_TYPE_Q4_K) {
        p = v.q + block * 144 + 16 + (o >> 6) * 32;
    } else if (TYPE == JQ_TYPE_Q5_K) {
        p = v.q + block * 176 + 48 + (o >> 6) * 32;
    } else if (TYPE == JQ_TYPE_Q6_K) {
        p = v.q + block * 208 + (o >> 7) * 64;
        asm volatile("prefetch.global.L1 [%0];" ::"l"(p + 128 + (o >> 7) * 32 - (o >> 7) * 64));
    } else {
        p = v.q + block * plane_q_bytes_dev(TYPE);
    }
    asm volatile("prefetch.global.L1 [%0];" ::"l"(p));
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// The 64 weights k0 .. k0 + 63 of one row, decoded bit-exactly (jq_formats.cuh) and rounded to bfloat16, written as
// one 128-byte row of the swizzled A tile: 16-byte chunk c lands at position c ^ (row & 7).
template <int TYPE>
__device__ __forceinline__ void dequant_row_chunk(const View& v, int64_t row, int k0, uint8_t* a_row, int swz, int part) {
    // `part` (0 or 1) selects this thread's half of the units that cover the chunk
    using F = Fmt<TYPE>;
    const int blocks_per_row = (int)(v.k / F::QK);
    // units whose runs cover [k0, k0 + 64)
    constexpr int SPAN_BLOCKS = F::QK >= 64 ? 1 : 64 / F::QK;
#pragma unroll
    for (int bb = 0; bb < SPAN_BLOCKS; bb++) {
        const int kb = k0 + bb * F::QK;  // start of this block's part
        const int64_t block = row * blocks_per_row + kb / F::QK;
        const int base = (kb / F::QK) * F::QK;  // first k of the block
#pragma unroll
        for (int u = 0; u < F::UNITS; u++) {
            // skip units entirely outside the chunk (compile-time layouts: see Fmt<>::decode positions)
            bool any = false;
            if (TYPE == JQ_TYPE_Q4_K || TYPE == JQ_TYPE_Q5_K) {
                any = (u >> 1) == ((k0 - base) >> 6) && (u & 1) == part;
            } else if (TYPE == JQ_TYPE_Q6_K) {
                any = (u >> 1) == ((k0 - base) >> 7) && (u & 1) == part;
            } else if (TYPE == JQ_TYPE_Q8_0) {
                any = u == part;   // two units of 16 per block, two blocks per chunk
            } else {
                any = bb == part;  // Q4_0, Q4_1: one unit per block, two blocks per chunk
            }
            if (!any) {
                continue;
            }
            float w[F::RUNS][16];
            int pos[F::RUNS];
            F::decode(v, block, u, w, pos);
#pragma unroll
            for (int r = 0; r < F::RUNS; r++) {
                const int rel = base + pos[r] - k0;  // position of the run inside the chunk
                if (rel >= 0 && rel < STAGE_K) {
                    const int c = rel >> 3;  // 16-byte chunk index (two per run)
                    uint4 lo, hi;
                    __nv_bfloat162 t;
                    t = __floats2bfloat162_rn(w[r][0], w[r][1]);   lo.x = *reinterpret_cast<uint32_t*>(&t);
                    t = __floats2bfloat162_rn(w[r][2], w[r][3]);   lo.y = *reinterpret_cast<uint32_t*>(&t);
                    t = __floats2bfloat162_rn(w[r][4], w[r][5]);   lo.z = *reinterpret_cast<uint32_t*>(&t);
                    t = __floats2bfloat162_rn(w[r][6], w[r][7]);   lo.w = *reinterpret_cast<uint32_t*>(&t);
                    t = __floats2bfloat162_rn(w[r][8], w[r][9]);   hi.x = *reinterpret_cast<uint32_t*>(&t);
                    t = __floats2bfloat162_rn(w[r][10], w[r][11]); hi.y = *reinterpret_cast<uint32_t*>(&t);
                    t = __floats2bfloat162_rn(w[r][12], w[r][13]); hi.z = *reinterpret_cast<uint32_t*>(&t);
                    t = __floats2bfloat162_rn(w[r][14], w[r][15]); hi.w = *reinterpret_cast<uint32_t*>(&t);
                    *reinterpret_cast<uint4*>(a_row + ((c ^ swz) << 4)) = lo;
                    *reinterpret_cast<uint4*>(a_row + (((c + 1) ^ swz) << 4)) = hi;
                }
            }
        }
    }
}

template <int TYPE, int TILE_T>
__global__ void __launch_bounds__(THREADS, 1) prefill_tcgen05_kernel(View v, const __grid_constant__ CUtensorMap xmap, int m,
                                                                    const float* __restrict__ bias, float* __restrict__ y) {
    constexpr int B_BYTES = TILE_T * STAGE_K * 2;
    constexpr uint32_t IDESC = idesc_of(TILE_T);
    extern __shared__ uint8_t smem_unaligned[];
    // the swizzled tiles must start on 1024-byte boundaries of the shared address space
    uint8_t* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    // [STAGES][A_BYTES] weights, [STAGES][B_BYTES] activations (1024-byte aligned tiles), then barriers
    uint8_t* a_tiles = smem;
    uint8_t* b_tiles = smem + STAGES * A_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * (A_BYTES + B_BYTES));
    // bars: full_a[S], full_b[S], empty[S], accum
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * STAGES + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int f0 = blockIdx.x * TILE_F, t0 = blockIdx.y * TILE_T;
    const int KT = (int)(v.k / STAGE_K);
    const uint32_t bar0 = smem_u32(bars);
    auto full_a = [&](int s) { return bar0 + 8u * (uint32_t)s; };
    auto full_b = [&](int s) { return bar0 + 8u * (uint32_t)(STAGES + s); };
    auto empty = [&](int s) { return bar0 + 8u * (uint32_t)(2 * STAGES + s); };
    const uint32_t accum = bar0 + 8u * (uint32_t)(3 * STAGES);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full_a(s), DQ_THREADS);
            mbar_init(full_b(s), 1);
            mbar_init(empty(s), 1);
        }
        mbar_init(accum, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TILE_T) : "memory");
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
                tma_load_2d(smem_u32(b_tiles + s * B_BYTES), &xmap, full_b(s), it * STAGE_K, t0);
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
                const uint64_t ad = smem_desc(smem_u32(a_tiles + s * A_BYTES)), bd = smem_desc(smem_u32(b_tiles + s * B_BYTES));
#pragma unroll
                for (int ks = 0; ks < STAGE_K / 16; ks++) {
                    // 16 k = 32 bytes further inside the swizzle row: +2 in the (address >> 4) field
                    umma(tmem, ad + 2u * ks, bd + 2u * ks, IDESC, (it | ks) != 0 ? 1u : 0u);
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
        const int i = (threadIdx.x - 64) & 127, part = (threadIdx.x - 64) >> 7;
        int64_t row = (int64_t)f0 + i;
        row = row < v.n ? row : v.n - 1;
        const uint32_t row_off = (uint32_t)((i >> 3) * 1024 + (i & 7) * 128);
        bool ok = true;
        for (int it = 0; it < KT; it++) {
            const int s = it % STAGES;
            const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
            if (!mbar_wait(empty(s), ph ^ 1u, abort_flag, 1)) {
                ok = false;
                break;
            }
            if (it + 2 < KT) {
                prefetch_row_chunk<TYPE>(v, row, (it + 2) * STAGE_K);
            }
            dequant_row_chunk<TYPE>(v, row, it * STAGE_K, a_tiles + s * A_BYTES + row_off, i & 7, part);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> visible to the tensor core
            mbar_arrive(full_a(s));
        }
        // ---- epilogue: accumulator -> y --------------------------------------------------------------------------------
        if (ok && mbar_wait(accum, 0, abort_flag, 4)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int lane_group = warp & 3;  // a warp may only read TMEM lanes 32 (warp % 4) .. + 31
            const int col_half = (warp - 2) >> 2;  // the two warps of a lane group split the token columns
            const int feature = f0 + lane_group * 32 + lane;
            const float b = (bias != nullptr && feature < v.n) ? bias[feature] : 0.0f;
#pragma unroll 1
            for (int c = col_half * (TILE_T / 64); c < (col_half + 1) * (TILE_T / 64); c++) {
                uint32_t r[32];
                const uint32_t taddr = tmem + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(c * 32);
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
                            y[(int64_t)token * v.n + feature] = __uint_as_float(r[j]) + b;
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TILE_T) : "memory");
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

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

template <int TYPE, int TILE_T>
int launch_typed(const View& v, const CUtensorMap& xmap, int m, const float* bias, float* y, cudaStream_t s) {
    constexpr int B_BYTES = TILE_T * STAGE_K * 2;
    const size_t smem = (size_t)STAGES * (A_BYTES + B_BYTES) + 256 + 1024;  // tiles + barriers + slack for the 1024-byte alignment
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    JQ_CUDA(cudaGetDevice(&dev));
    if ((configured.load() >> (dev & 63) & 1) == 0) {
        JQ_CUDA(cudaFuncSetAttribute(prefill_tcgen05_kernel<TYPE, TILE_T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured.fetch_or((uint64_t)1 << (dev & 63));
    }
    dim3 grid((unsigned)((v.n + TILE_F - 1) / TILE_F), (unsigned)((m + TILE_T - 1) / TILE_T));
    prefill_tcgen05_kernel<TYPE, TILE_T><<<grid, THREADS, smem, s>>>(v, xmap, m, bias, y);
    count_launch();
    return check_launch("prefill_tcgen05_kernel");
}

}  // namespace

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
    // 256 tokens per CTA when there are enough of them: every dequantised weight tile then feeds twice the tensor work
    const int64_t ctas256 = ((v.n + TILE_F - 1) / TILE_F) * ((m + 255) / 256);
    const int tile_t = (m > 128 && ctas256 >= 140) ? 256 : 128;  // not at the price of leaving SMs without a CTA
    const cuuint32_t box[2] = {STAGE_K, (cuuint32_t)tile_t};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<uint16_t*>(x_bf16), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        return fail(JQ_ERR_CUDA, "prefill: cuTensorMapEncodeTiled failed with code %d", (int)r);
    }
#define JQ_PREFILL_CASE(T)                                                                         \
    case T:                                                                                          \
        return tile_t == 256 ? launch_typed<T, 256>(v, xmap, (int)m, bias, y, s) : launch_typed<T, 128>(v, xmap, (int)m, bias, y, s);
    switch (v.type) {
        JQ_PREFILL_CASE(JQ_TYPE_Q8_0)
        JQ_PREFILL_CASE(JQ_TYPE_Q4_0)
        JQ_PREFILL_CASE(JQ_TYPE_Q4_1)
        JQ_PREFILL_CASE(JQ_TYPE_Q4_K)
        JQ_PREFILL_CASE(JQ_TYPE_Q5_K)
        default:
            return tile_t == 256 ? launch_typed<JQ_TYPE_Q6_K, 256>(v, xmap, (int)m, bias, y, s) : launch_typed<JQ_TYPE_Q6_K, 128>(v, xmap, (int)m, bias, y, s);
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
