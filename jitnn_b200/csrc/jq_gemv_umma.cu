// Decode GEMV on the 5th-generation tensor cores: y[m, n] = x[m, k] . W[n, k]^T for 1 <= m <= 16 rows of x, W in Q4_K or
// Q5_K, one pass over the weights for every m.
//
// Replaces the reference's matrix-vector kernels (kernels/jitllm/TransformerComputeKernelsQ4_K.java:130-215,
// ...Q5_K.java:422-532, dispatch ops/Gguf.java:170-183).
//   * the activations are turned into an "image" of half-precision digits (jq_umma_image.cuh: 22-bit fixed point per
//     super-block of k, two signed 11-bit digits per value, one MMA column per (row of x, digit));
//   * a persistent CTA per SM walks units of 128 weight rows x one 256-element super-block of k. Per unit
//       - one thread asks the copy engine for the unit's weights (one cp.async.bulk of 128 x 144 contiguous bytes: the
//         weight is stored tile by tile for exactly this, jq_common.cuh) and for the super-block's image (another
//         cp.async.bulk), both into shared-memory rings that complete on mbarriers;
//       - 128 "unpack" threads, one per weight row, turn the row's quants into quant x 6-bit scale (an integer below
//         2048, exact in half precision: one byte permute per two quants and one fused multiply-add per pair) and store
//         them into tensor memory as the A operand (tcgen05.st); the row's mins, d and dmin go into a small
//         shared-memory ring;
//       - one thread issues sixteen tcgen05.mma.cta_group::1.kind::f16 (M = 128 rows, N = 16 or 32 digit columns, K = 16,
//         A from tensor memory, B = the image in shared memory) that accumulate the whole super-block into one FP32
//         accumulator: the scales are already in the operand;
//       - 128 "epilogue" threads, one per weight row, read the accumulators (tcgen05.ld), weigh the two digits, and
//         apply fp16 d, dmin and the mins (through the sub-blocks' sums of x).
//   * a row's result is the sum of its super-blocks' contributions in k order, each contribution rounded to FP32
//     first. Units are dealt to the CTAs in contiguous runs, so a run can start or end inside a tile; such
//     pieces are written to a scratch buffer (the first piece as a running sum, later pieces contribution by
//     contribution) and the CTA that finishes a tile's last piece adds them in k order. The result therefore does not
//     depend on how many CTAs or rows there are: a row shard of a weight gives bitwise the outputs of the whole weight.
// The products are exact; a super-block's 256 of them per digit are summed in FP32 by the tensor core. x keeps 22 bits
// relative to the largest magnitude of its super-block.
//
// Every wait (mbarrier phases) is bounded: a wait that runs out records 64 + its role in a status word, raises the
// CTA's abort flag, all roles fall through to the common exit and tensor memory is released. No CTA waits for another.
#include <mutex>

#include "jq_formats.cuh"
#include "jq_peer_device.cuh"
#include "jq_tc.cuh"
#include "jq_umma_image.cuh"

namespace jq {

// 0, or 64 + the role whose wait gave up first (1 copy issue, 2 MMA issue, 3 unpack, 4 epilogue) since the last read.
static __device__ int g_umma_status;
static __device__ int g_umma_peer_status;

// Development aid, compiled in with -DJQ_UMMA_TRACE: CTA 0 records clock64() at the hand-over points of every role for
// its first 64 units; jq_debug_umma_trace copies the record out.
#ifdef JQ_UMMA_TRACE
__device__ long long g_umma_cta[160 * 8];  // per CTA: %globaltimer at start, after the wait for the kernel before, image built, first unit's inputs ready, last unit done
__device__ __forceinline__ long long gtime() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define CT(k)                                                                  \
    do {                                                                       \
        if (blockIdx.x < 160) g_umma_cta[blockIdx.x * 8 + (k)] = gtime();      \
    } while (0)
__device__ long long g_umma_trace[5 * 64 * 4];
#define TR(role, i, k)                                                                       \
    do {                                                                                     \
        if (blockIdx.x == 0 && lane == 0 && (i) < 64) g_umma_trace[((role) * 64 + (i)) * 4 + (k)] = clock64(); \
    } while (0)
#else
#define TR(role, i, k) \
    do {               \
    } while (0)
#define CT(k) \
    do {      \
    } while (0)
#endif

std::atomic<int64_t> g_opt_gemv_umma{0};
std::atomic<int64_t> g_opt_wait_limit_us{2000000};

namespace {

constexpr int ROWS = 128;        // weight rows per unit (MMA M)
constexpr int SP = 4;            // stages of the row-parameter ring
constexpr int P_BYTES = ROWS * 16;
constexpr int MAX_SX = 8;        // stages of the image ring: enough of them in flight to cover the latency of a copy from L2
constexpr int MAX_SW = 12;       // stages of the weight ring (as many as fit)
constexpr size_t SMEM_MAX = 227 * 1024;
constexpr int UMMA_AUTO_MIN_ROWS = 11;  // rows of x from which the kernel is chosen without being asked for
constexpr size_t RESIDENT_MAX = 96 * 1024;  // largest activation image that stays in shared memory for the whole kernel

template <int TYPE>
struct UFmt;
template <>
struct UFmt<JQ_TYPE_Q4_K> {
    static constexpr int BYTES = 144;
    static constexpr int QS = 16;             // offset of the nibbles
    static constexpr bool IN_PLACE = true;    // high nibbles stay where they are (16 q): the odd sub-blocks' scales are divided by 16 instead
};
template <>
struct UFmt<JQ_TYPE_Q5_K> {
    static constexpr int BYTES = 176;
    static constexpr int QS = 48;
    static constexpr bool IN_PLACE = false;
};

struct UArgs {
    const uint8_t* q[3];    // blocks of up to three weights of one type and k (unused entries: those of the first)
    const uint8_t* image;   // [KB][image block], unless the kernel builds the image itself ...
    const float* x;         // ... from x [rows, k]
    const float* bias;
    float* y[3];
    int64_t n[3];           // rows of the weights (0: none)
    int64_t col0[3], n_sum; // NC > 1: where a weight's rows start in a row of `parts`, and the length of such a row
    int KB;                 // super-blocks per tile: those of a weight row, or (NC > 1) of one of the NC equal ranges a row's k is cut into
    int NC;                 // ranges of k: each (tile, range) is a tile of its own whose sums go to `parts` instead of y
    float* parts;           // NC > 1: [NC][rows][n_sum] sums per range, added in range order by umma_parts_sum_kernel
    int tile_end[3], tiles; // 128-row tiles (times NC) up to and including each weight; of all
    int rows;               // rows of x
    int SW;                 // stages of the weight ring
    int SX;                 // stages of the image ring
    unsigned long long* partial;  // per CTA [max_pieces][rows][128] marked floats: what the CTA has of a tile it does not finish (all zero between launches)
    float* aside;           // per CTA [max_pieces][rows][128] floats, private to the CTA
    int max_pieces;
    int whole_tiles;        // non-zero: every CTA's run is whole tiles (partial is not used)
    long long wait_clocks;  // clocks after which a bounded wait gives up
    uint32_t lbo, sbo;      // byte offsets of the image's shared-memory descriptor
    const PeerOut* peer;
};

template <int NREG>
__device__ __forceinline__ void tmem_ld(uint32_t (&r)[NREG], uint32_t taddr);
template <>
__device__ __forceinline__ void tmem_ld<4>(uint32_t (&r)[4], uint32_t taddr) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr) : "memory");
}
template <>
__device__ __forceinline__ void tmem_ld<8>(uint32_t (&r)[8], uint32_t taddr) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
template <>
__device__ __forceinline__ void tmem_ld<16>(uint32_t (&r)[16], uint32_t taddr) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
                   "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
}
template <>
__device__ __forceinline__ void tmem_ld<32>(uint32_t (&r)[32], uint32_t taddr) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]),
                 "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[128 x N] (tensor memory, f32) (+)= A[128 x 16] (tensor memory, f16) . B[16 x N] (shared memory, f16)
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d), "r"(tmem_a),
        "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Instruction descriptor of kind::f16: D = F32 (bits 4-5 = 1), A and B half precision (bits 7-9 and 10-12 = 0), both K-major,
// N >> 3 in bits 17-22, M >> 4 in bits 24-28.
constexpr uint32_t idesc_of(int n_cols) { return (1u << 4) | ((uint32_t)(n_cols >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24); }

// Shared-memory descriptor of a K-major operand without swizzle: 8 rows x 16 bytes per core matrix, `lbo` bytes between the
// core matrices of consecutive 16-byte steps of k, `sbo` bytes between those of consecutive groups of 8 rows; descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc_plain(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | ((uint64_t)1 << 46);
}

// A poll of an mbarrier takes well over a hundred clocks to come back from the shared-memory unit even when the phase is
// already complete, so a role polls everything a unit needs at once (the round trips overlap) and only then waits, bounded,
// for what was not complete.
struct Phase {
    uint32_t bar, parity;
};
__device__ __forceinline__ bool wait_phases(const Phase& p0, const Phase& p1, const Phase& p2, bool use2, volatile int* abort_flag, int code, long long limit) {
    const bool r0 = tc::mbar_try(p0.bar, p0.parity);
    const bool r1 = tc::mbar_try(p1.bar, p1.parity);
    const bool r2 = use2 ? tc::mbar_try(p2.bar, p2.parity) : true;
    if (r0 && r1 && r2) {
        return true;
    }
    return (r0 || tc::mbar_wait(p0.bar, p0.parity, abort_flag, &g_umma_status, code, limit)) &&
           (r1 || tc::mbar_wait(p1.bar, p1.parity, abort_flag, &g_umma_status, code, limit)) &&
           (r2 || tc::mbar_wait(p2.bar, p2.parity, abort_flag, &g_umma_status, code, limit));
}
// The same on behalf of a whole warp: lane 0 polls (32 lanes polling one word would serialise), the outcome goes to the other
// lanes, and __shfl_sync orders their later reads behind lane 0's acquire.
__device__ __forceinline__ bool warp_wait_phases(const Phase& p0, const Phase& p1, const Phase& p2, bool use2, volatile int* abort_flag, int code,
                                                 long long limit, int lane) {
    int ok = 1;
    if (lane == 0) {
        ok = wait_phases(p0, p1, p2, use2, abort_flag, code, limit) ? 1 : 0;
    }
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
// The order in which a CTA visits the units [u0, u1) of its run: tile after tile from the last tile of the run to the first,
// the super-blocks of a tile in ascending order. The tile in which the run ends (of which the CTA has the first super-blocks)
// is visited first, so that its running sums are known to the CTA that continues the tile long before that CTA gets there:
// the tile in which a run begins is visited last.
struct Walk {
    int t, b, e;        // tile, super-block, end of the tile's super-blocks that belong to the run
    int t_first, b0;    // the run's first tile and its first super-block in it
    int kb;
    __device__ __forceinline__ void start(int64_t u0, int64_t u1, int kb_) {
        kb = kb_;
        t_first = (int)(u0 / kb);
        b0 = (int)(u0 - (int64_t)t_first * kb);
        t = (int)((u1 - 1) / kb);
        e = (int)(u1 - (int64_t)t * kb);
        b = t == t_first ? b0 : 0;
    }
    __device__ __forceinline__ void next() {
        if (++b == e) {
            t--;
            b = t == t_first ? b0 : 0;
            e = kb;
        }
    }
};

// What one CTA hands to another through the scratch buffer: a float and, in the same naturally aligned 8-byte word, a mark that
// says the float has been written. An 8-byte store is seen whole or not at all, so the reader needs no flag and the writer no
// fence: the reader polls the word until the mark is there, takes the float and clears the word for the next launch.
__device__ __forceinline__ void handoff_store(unsigned long long* p, float v) {
    const unsigned long long w = (unsigned long long)__float_as_uint(v) | (1ull << 32);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long handoff_load(const unsigned long long* p) {
    unsigned long long w;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}
__device__ __forceinline__ void handoff_clear(unsigned long long* p) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(0ull) : "memory");
}

// A ring position: stage and the parity of the phase in which the stage gets filled.
struct Ring {
    int s = 0;
    uint32_t ph = 0;
    __device__ __forceinline__ void next(int stages) {
        if (++s == stages) {
            s = 0;
            ph ^= 1u;
        }
    }
};
// One arrival per warp, after all of its lanes have got here (their shared-memory writes come before lane 0's release).
__device__ __forceinline__ void warp_arrive(uint32_t bar, int lane) {
    __syncwarp();
    if (lane == 0) {
        tc::mbar_arrive(bar);
    }
}

__device__ __forceinline__ void epilogue_barrier(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }

__device__ __forceinline__ __half2 u32_as_half2(uint32_t v) { return *reinterpret_cast<const __half2*>(&v); }
__device__ __forceinline__ uint32_t half2_as_u32(__half2 v) { return *reinterpret_cast<const uint32_t*>(&v); }

__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

template <int N>
__global__ void __launch_bounds__(128) umma_activation_image_kernel(const float* __restrict__ x, int rows, int64_t k, uint8_t* __restrict__ image) {
    asm volatile("griddepcontrol.launch_dependents;");  // the GEMV may start asking for weights
    asm volatile("griddepcontrol.wait;" ::: "memory");  // x is complete, and the GEMV before this one is done with the image
    const int pair = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int b = pair / rows, m = pair % rows;
    if (b < (int)(k >> 8)) {
        umma::build_image<N>(x + (int64_t)m * k + (int64_t)b * 256, m, rows, image + (size_t)b * umma::ImageCfg<N>::BYTES, threadIdx.x & 31);
    }
}

// Where the outputs of up to three weights go: weight w owns columns [col0[w], col0[w] + n[w]) of a row of `parts`.
struct PartsOut {
    float* y[3];
    int64_t n[3], col0[3];
    int64_t n_sum;
};
// y_w [rows, n_w] = (bias +) the sums of the NC ranges of k, added in range order (one thread per output).
__global__ void __launch_bounds__(256) umma_parts_sum_kernel(const float* __restrict__ parts, int nc, int rows, PartsOut po, const float* __restrict__ bias) {
    const int64_t outputs = (int64_t)rows * po.n_sum;
    const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (i < outputs) {
        float v[8];
#pragma unroll
        for (int c = 0; c < 8; c++) {
            v[c] = c < nc ? __ldcg(parts + (size_t)c * outputs + i) : 0.0f;
        }
        float sum = v[0];
#pragma unroll
        for (int c = 1; c < 8; c++) {
            if (c < nc) {
                sum += v[c];
            }
        }
        const int64_t m = i / po.n_sum, col = i - m * po.n_sum;
        const int wi = col < po.col0[1] ? 0 : (col < po.col0[2] ? 1 : 2);
        const int64_t row = col - (wi == 0 ? 0 : (wi == 1 ? po.col0[1] : po.col0[2]));
        const int64_t n = wi == 0 ? po.n[0] : (wi == 1 ? po.n[1] : po.n[2]);
        float* y = wi == 0 ? po.y[0] : (wi == 1 ? po.y[1] : po.y[2]);
        y[m * n + row] = sum + ((bias != nullptr && wi == 0) ? bias[row] : 0.0f);
    }
}

// MR = rows of x the kernel computes (8 or 16; a call with fewer rows leaves the others unused). Two sets of epilogue warps
// share the rows of x. RES: the image of the whole k is built by this kernel into shared memory and
// stays there (small k x rows).
template <int MR>
struct Roles {
    static constexpr int ES = MR >= 8 ? 2 : 1;     // sets of four epilogue warps
    static constexpr int HM = MR / ES;             // rows of x per epilogue thread
    static constexpr int THREADS = 192 + 128 * ES + 32;  // warp 0: copies, warp 1: MMA issue and tensor-memory owner, warps 2-5: unpack, then epilogue, last warp: MMA issue
};

template <int TYPE, int MR, bool PEER, bool RES>
__global__ void __launch_bounds__(Roles<MR>::THREADS, 1) gemv_umma_kernel(const UArgs a) {
    constexpr int N = umma::columns_for_rows(MR);
    using IC = umma::ImageCfg<N>;
    using F = UFmt<TYPE>;
    constexpr int ES = Roles<MR>::ES, HM = Roles<MR>::HM;
    constexpr int MMA2_WARP = 6 + 4 * ES;       // the second MMA issuer
    constexpr int NGROUPS = 1;                  // one accumulator stage per unit: the scales are in the A operand
    // (A unit's MMAs taking turns on two accumulators, so that none waits for the one before it, measured no faster: the
    // sixteen MMAs of a unit take 1500 (N = 16) to 2100 (N = 32) clocks to issue either way.)
    constexpr int ACC = 1;
    constexpr int D_COLS = ACC * N;             // tensor-memory columns of an accumulator stage
    constexpr int A_COLS = 128;                 // of an A stage: 256 half-precision values of k per row
    constexpr int NA = 3;                       // A stages
    constexpr int ND = 128 / D_COLS < 4 ? 128 / D_COLS : 4;  // accumulator stages
    constexpr int D_BASE = NA * A_COLS;
    constexpr uint32_t TMEM_COLS = 512u;
    static_assert(D_BASE + ND * D_COLS <= 512, "tensor memory has 512 columns");
    constexpr int WB = ROWS * F::BYTES;
    constexpr int XB = (IC::BYTES + 127) & ~127;
    constexpr uint32_t IDESC = idesc_of(N);
    constexpr int LDW = 2 * HM;  // accumulator columns an epilogue thread reads per unit: two digits per row of x
    static_assert(LDW == 8 || LDW == 16, "tcgen05.ld shapes of the epilogue");

    extern __shared__ uint8_t smem_unaligned[];
    uint8_t* smem = smem_unaligned + ((128u - (tc::smem_u32(smem_unaligned) & 127u)) & 127u);
    const int SW = a.SW, SX = a.SX;
    const int KB = a.KB;
    uint8_t* w_ring = smem;
    uint8_t* x_ring = w_ring + (size_t)SW * WB;  // RES: the KB blocks of the image; else SX stages
    uint8_t* p_ring = x_ring + (size_t)(RES ? KB : SX) * XB;
    uint64_t* bars = reinterpret_cast<uint64_t*>(p_ring + SP * P_BYTES);
    const uint32_t bar0 = tc::smem_u32(bars);
    auto full_w = [&](int s) { return bar0 + 8u * (uint32_t)s; };
    auto empty_w = [&](int s) { return bar0 + 8u * (uint32_t)(MAX_SW + s); };
    auto full_x = [&](int s) { return bar0 + 8u * (uint32_t)(2 * MAX_SW + s); };
    auto empty_x = [&](int s) { return bar0 + 8u * (uint32_t)(2 * MAX_SW + MAX_SX + s); };
    auto full_p = [&](int s) { return bar0 + 8u * (uint32_t)(2 * MAX_SW + 2 * MAX_SX + s); };
    auto empty_p = [&](int s) { return bar0 + 8u * (uint32_t)(2 * MAX_SW + 2 * MAX_SX + SP + s); };
    constexpr int B2 = 2 * MAX_SW + 2 * MAX_SX + 2 * SP;
    auto full_a = [&](int s) { return bar0 + 8u * (uint32_t)(B2 + s); };
    auto empty_a = [&](int s) { return bar0 + 8u * (uint32_t)(B2 + 4 + s); };
    auto full_d = [&](int s) { return bar0 + 8u * (uint32_t)(B2 + 8 + s); };
    auto empty_d = [&](int s) { return bar0 + 8u * (uint32_t)(B2 + 12 + s); };
    constexpr int NBARS = B2 + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBARS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* d_issued = reinterpret_cast<volatile int*>(tmem_slot + 2);  // per accumulator stage: fillings whose wait for the stage has passed
    volatile int* fin_all = reinterpret_cast<volatile int*>(tmem_slot + 6);  // per epilogue set: [0] this CTA adds the tile up, [1], [2] first and last CTA of the tile

    asm volatile("griddepcontrol.launch_dependents;");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t U = (int64_t)a.tiles * KB;
    const int64_t G = gridDim.x;
    // This CTA's run of units: an even share of all units, or (no scratch for pieces of tiles) an even share of the tiles.
    const int64_t u0 = a.whole_tiles ? (int64_t)blockIdx.x * a.tiles / G * KB : (int64_t)blockIdx.x * U / G;
    const int units = (int)((a.whole_tiles ? ((int64_t)blockIdx.x + 1) * a.tiles / G * KB : ((int64_t)blockIdx.x + 1) * U / G) - u0);
    const int64_t u1 = u0 + units;
    const long long limit = a.wait_clocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < MAX_SW; s++) {
            tc::mbar_init(full_w(s), 1);
            tc::mbar_init(empty_w(s), 4);  // one arrival per unpack warp
        }
        for (int s = 0; s < MAX_SX; s++) {
            tc::mbar_init(full_x(s), 1);
            tc::mbar_init(empty_x(s), 1 + 4 * ES);  // the MMAs that read the digits, and one lane of each epilogue warp
        }
        for (int s = 0; s < SP; s++) {
            tc::mbar_init(full_p(s), 4);
            tc::mbar_init(empty_p(s), 4 * ES);
        }
        for (int s = 0; s < 4; s++) {
            tc::mbar_init(full_a(s), 4);
            tc::mbar_init(empty_a(s), 1);
            tc::mbar_init(full_d(s), 1);
            tc::mbar_init(empty_d(s), 4 * ES);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        for (int s = 0; s < 4; s++) {
            d_issued[s] = 0;
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    // Weights depend on nothing that runs before this kernel: the first ring-full of them is requested at once.
    auto issue_w = [&](int i, int s, int t, int b) {
        const int wi = t < a.tile_end[0] ? 0 : (t < a.tile_end[1] ? 1 : 2);
        const int t_in = t - (wi == 0 ? 0 : (wi == 1 ? a.tile_end[0] : a.tile_end[1]));
        const uint8_t* src = (wi == 0 ? a.q[0] : (wi == 1 ? a.q[1] : a.q[2])) + ((int64_t)t_in * KB + b) * WB;
        tc::mbar_expect_tx(full_w(s), WB);
        tc::bulk_load(tc::smem_u32(w_ring + (size_t)s * WB), src, WB, full_w(s));
        TR(0, i, 0);
    };
    const int w_prologue = units < SW ? units : SW;
    Walk ww;  // thread 0: the unit whose weights are requested next
    ww.start(u0, u1, KB);
    if (threadIdx.x == 0) {
        for (int i = 0; i < w_prologue; i++) {
            issue_w(i, i, ww.t, ww.b);
            ww.next();
        }
    }
    if constexpr (RES) {
        // The activation image of the whole k, built here from x by the warps that have nothing to do yet: one warp per
        // (super-block, row of x). x is complete once the kernel before this one has finished.
        if (warp >= 2) {
            if (warp == 2 && lane == 0) CT(0);
            asm volatile("griddepcontrol.wait;" ::: "memory");
            if (warp == 2 && lane == 0) CT(1);
            const int workers = Roles<MR>::THREADS / 32 - 2;  // every warp but the copy and the first MMA warp
            // the values of a warp's next part are requested before its current part is worked on
            const int tasks = KB * a.rows;
            auto src_of = [&](int task) { return a.x + (int64_t)(task % a.rows) * KB * 256 + (int64_t)(task / a.rows) * 256; };
            float4 lo, hi, lo_next = make_float4(0.f, 0.f, 0.f, 0.f), hi_next = lo_next;
            int task = warp - 2;
            if (task < tasks) {
                umma::load_lane_values(src_of(task), lane, lo_next, hi_next);
            }
            for (; task < tasks; task += workers) {
                lo = lo_next;
                hi = hi_next;
                if (task + workers < tasks) {
                    umma::load_lane_values(src_of(task + workers), lane, lo_next, hi_next);
                }
                umma::build_image_from<N>(lo, hi, task % a.rows, a.rows, x_ring + (size_t)(task / a.rows) * XB, lane);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor core reads the digits through the async proxy
            if (warp == 2 && lane == 0) CT(2);
        }
        __syncthreads();
    }

    if (warp == 0) {
        // ---- copies: one thread asks the copy engine for a unit's weights (one contiguous run of the tiled layout) and, unless
        // the image is resident, for its super-block's image, which is complete only when the kernel before this one has finished.
        auto issue_x = [&](int i, int s, int t, int b_in_tile) {
            const int b = a.NC > 1 ? (t % a.NC) * KB + b_in_tile : b_in_tile;  // the range's first super-block of k + the position in it
            tc::mbar_expect_tx(full_x(s), IC::BYTES);
            tc::bulk_load(tc::smem_u32(x_ring + s * XB), a.image + (size_t)b * IC::BYTES, IC::BYTES, full_x(s));
            TR(0, i, 1);
        };
        if constexpr (!RES) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            if constexpr (PEER) {
                if (a.peer->wait_first) {
                    // the image is what the ranks' latest exchange delivered: complete once all their flags are up
                    peer_wait_inline(a.peer->flags[a.peer->rank], a.peer->world, lane, &g_umma_peer_status);
                }
            }
        }
        if (lane == 0) {
            int iw = w_prologue;
            int ix = RES ? units : (units < SX ? units : SX);
            Walk wx;
            wx.start(u0, u1, KB);
            if constexpr (!RES) {
                for (int i = 0; i < ix; i++) {
                    issue_x(i, i, wx.t, wx.b);
                    wx.next();
                }
            }
            Ring wr, xr;  // the next slot to fill, and the parity of the phase in which its last filling was consumed
            wr.s = iw == SW ? 0 : iw;
            xr.s = ix == SX ? 0 : ix;
            long long idle_since = 0;
            while (iw < units || ix < units) {
                // both rings polled together and without suspending: a slot of either may come free first
                const bool wfree = iw < units && tc::mbar_test(empty_w(wr.s), wr.ph);
                const bool xfree = ix < units && tc::mbar_test(empty_x(xr.s), xr.ph);
                if (wfree) {
                    issue_w(iw++, wr.s, ww.t, ww.b);
                    ww.next();
                    wr.next(SW);
                }
                if (xfree) {
                    issue_x(ix++, xr.s, wx.t, wx.b);
                    wx.next();
                    xr.next(SX);
                }
                if (wfree || xfree) {
                    idle_since = 0;
                } else if (*abort_flag != 0) {
                    break;
                } else if (idle_since == 0) {
                    idle_since = clock64();
                } else if (clock64() - idle_since > limit) {
                    atomicCAS(&g_umma_status, 0, 64 + 1);
                    *abort_flag = 1;
                    break;
                }
            }
        }
    } else if (warp == 1 || warp == MMA2_WARP) {
        // ---- MMA issue: one thread of warp 1 takes the even units of the run, one thread of the last warp the odd ones. An
        // MMA of this shape keeps the tensor core busy for about a hundred clocks whatever N is, and issuing stalls while the
        // tensor core's queue is full; with two issuers one waits for its unit's inputs (a poll of an mbarrier takes a few
        // hundred clocks to come back) while the other's MMAs run.
        if (lane == 0) {
            const int first = warp == 1 ? 0 : 1;
            bool ok = true;
            Ring xr, ar, dr;
            for (int k = 0; k < first; k++) {
                xr.next(SX);
                ar.next(NA);
                for (int g = 0; g < NGROUPS; g++) {
                    dr.next(ND);
                }
            }
            Walk wk;
            wk.start(u0, u1, KB);
            if (first == 1 && units > 1) {
                wk.next();
            }
            // descriptor of sub-block 0 of image block 0; blocks and sub-blocks only move the 14-bit address field (16-byte units)
            const uint64_t desc0 = smem_desc_plain(tc::smem_u32(x_ring), a.lbo, a.sbo);
            // Both issuers fill the same accumulator stages in turn. A wait for "the stage's previous filling has been read" may only
            // be made once that filling's own wait has passed (an mbarrier tells two phases apart, not three), so the issuers
            // count per stage the fillings that have got that far.
            auto my_turn = [&](int stage, int filling) {
                if (d_issued[stage] >= filling) {
                    return true;
                }
                const long long t0 = clock64();
                while (d_issued[stage] < filling) {
                    if (*abort_flag != 0) {
                        return false;
                    }
                    if (clock64() - t0 > limit) {
                        atomicCAS(&g_umma_status, 0, 64 + 2);
                        *abort_flag = 1;
                        return false;
                    }
                }
                return true;
            };
            int filling[4] = {0, 0, 0, 0};  // per stage: the number of the next filling by this issuer
            {
                // where the first unit of this issuer stands
                int q = 0;
                for (int k = 0; k < first; k++) {
                    q += NGROUPS;
                }
                for (int st = 0; st < ND; st++) {
                    filling[st] = (q + ND - 1 - st) / ND;  // groups before q that fell on stage st
                }
            }
            for (int i = first; i < units && ok; i += 2) {
                ok = my_turn(dr.s, filling[dr.s]) &&
                     wait_phases(Phase{full_a(ar.s), ar.ph}, Phase{empty_d(dr.s), dr.ph ^ 1u}, Phase{full_x(xr.s), xr.ph}, !RES, abort_flag, 64 + 2, limit);
                if (!ok) {
                    break;
                }
                d_issued[dr.s] = filling[dr.s] + 1;
                tc::fence_after_sync();
                TR(1, i, 0);
                if (i == 0) CT(3);
                const uint64_t xdesc = desc0 + (uint64_t)((uint32_t)((RES ? wk.b : xr.s) * XB) >> 4);
                const uint32_t abase = tmem + (uint32_t)(ar.s * A_COLS);
                const uint32_t dbase = tmem + (uint32_t)D_BASE + (uint32_t)(dr.s * D_COLS);
                // sixteen steps of 16 values of k: 8 tensor-memory columns of A and one 16-row slab of the image each
#pragma unroll
                for (int st = 0; st < IC::STEPS; st++) {
                    umma_f16_ts(dbase + (uint32_t)((st % ACC) * N), abase + (uint32_t)(st * 8), xdesc + (uint64_t)((st * IC::SUB_BYTES) >> 4), IDESC,
                                st >= ACC ? 1u : 0u);
                }
                tc::umma_commit(full_d(dr.s));
                TR(1, i, 1);
                dr.next(ND);
                if (!ok) {
                    break;
                }
                // the other issuer's unit takes the next NGROUPS fillings, this issuer's next unit the NGROUPS after them
                for (int st = 0; st < ND; st++) {
                    filling[st] = ((i + 2) * NGROUPS + ND - 1 - st) / ND;
                }
                tc::umma_commit(empty_a(ar.s));
                if constexpr (!RES) {
                    tc::umma_commit(empty_x(xr.s));
                }
                TR(1, i, 3);
                // on to the unit after the other issuer's
                for (int k = 0; k < 2; k++) {
                    xr.next(SX);
                    ar.next(NA);
                    if (i + 1 + k < units) {
                        wk.next();
                    }
                }
                for (int g = 0; g < NGROUPS; g++) {
                    dr.next(ND);
                }
            }
        }
    } else if (warp < 6) {
        // ---- unpack: thread = weight row; a warp may only touch the tensor-memory lanes 32 (warp % 4) .. + 31 --------------------
        const int r = (warp & 3) * 32 + lane;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        Ring wr, ar, pr;
        for (int i = 0; i < units; i++) {
            const int ws = wr.s, as = ar.s, ps = pr.s;
            // the weights have landed, the MMAs that read the A stage before have finished, the epilogue has read the parameter slot
            if (!warp_wait_phases(Phase{full_w(ws), wr.ph}, Phase{empty_a(as), ar.ph ^ 1u}, Phase{empty_p(ps), pr.ph ^ 1u}, true, abort_flag, 64 + 3, limit,
                                  lane)) {
                break;
            }
            tc::fence_after_sync();
            if (warp == 2) TR(2, i, 0);
            const uint8_t* wrow = w_ring + (size_t)ws * WB + r * F::BYTES;
            const uint4 h = *reinterpret_cast<const uint4*>(wrow);  // fp16 d, fp16 dmin, 12 bytes of 6-bit scales and mins
            const uint32_t sca = h.y & 0x3f3f3f3fu, scb = and_or(h.y >> 2, 0x30303030u, h.w & 0x0f0f0f0fu);            // scales 0..3, 4..7
            const uint32_t mna = h.z & 0x3f3f3f3fu, mnb = and_or(h.z >> 2, 0x30303030u, (h.w >> 4) & 0x0f0f0f0fu);     // mins 0..3, 4..7
            uint4* prow = reinterpret_cast<uint4*>(p_ring + ps * P_BYTES) + r;
            prow[0] = make_uint4(mna, mnb, h.x, 0u);
            warp_arrive(full_p(ps), lane);
            if (warp == 2) TR(2, i, 1);
            uint4 qh0 = make_uint4(0u, 0u, 0u, 0u), qh1 = qh0;
            if constexpr (TYPE == JQ_TYPE_Q5_K) {
                qh0 = *reinterpret_cast<const uint4*>(wrow + 16);
                qh1 = *reinterpret_cast<const uint4*>(wrow + 32);
            }
            const uint32_t hw[8] = {qh0.x, qh0.y, qh0.z, qh0.w, qh1.x, qh1.y, qh1.z, qh1.w};
            // A byte b under the exponent byte 0x64 is the half-precision number 1024 + b. The operand is quant x scale, an
            // integer below 2048 and therefore exact in half precision: (1024 + q) sc - 1024 sc in one fused multiply-add per
            // pair. Q4_K's high nibbles stay where they are: (1024 + 16 q) (sc / 16) - 64 sc.
            const __half2 k1024 = u32_as_half2(0x64006400u);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint4 qa = *reinterpret_cast<const uint4*>(wrow + F::QS + 32 * j);
                const uint4 qb = *reinterpret_cast<const uint4*>(wrow + F::QS + 32 * j + 16);
                const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                const uint32_t scw = j < 2 ? sca : scb;
                const __half2 sce = __hsub2(u32_as_half2(__byte_perm(scw, 0x64646464u, 0x4040u + (uint32_t)(2 * (j & 1)) * 0x0101u)), k1024);
                const __half2 sco = __hsub2(u32_as_half2(__byte_perm(scw, 0x64646464u, 0x4141u + (uint32_t)(2 * (j & 1)) * 0x0101u)), k1024);
                const __half2 mule = sce, adde = __hmul2(sce, u32_as_half2(0xe400e400u));                                   // -1024 sc
                const __half2 mulo = F::IN_PLACE ? __hmul2(sco, u32_as_half2(0x2c002c00u)) : sco;                           // sc / 16
                const __half2 addo = __hmul2(sco, F::IN_PLACE ? u32_as_half2(0xd400d400u) : u32_as_half2(0xe400e400u));    // -64 sc
                uint32_t lo[16], hi[16];  // sub-block 2j and sub-block 2j + 1: 32 values each, two to a register
#pragma unroll
                for (int c = 0; c < 8; c++) {
                    uint32_t te, to;
                    if constexpr (TYPE == JQ_TYPE_Q5_K) {
                        // bit 2j (2j + 1) of the fifth-bit bytes goes to bit 4 of the low (high) nibbles' bytes
                        const uint32_t e = 2 * j <= 4 ? hw[c] << (4 - 2 * j) : hw[c] >> (2 * j - 4);
                        const uint32_t o = 2 * j + 1 <= 4 ? hw[c] << (3 - 2 * j) : hw[c] >> (2 * j - 3);
                        te = and_or(e, 0x10101010u, w[c] & 0x0f0f0f0fu);
                        to = and_or(o, 0x10101010u, (w[c] >> 4) & 0x0f0f0f0fu);
                    } else {
                        te = w[c] & 0x0f0f0f0fu;
                        to = w[c] & 0xf0f0f0f0u;
                    }
                    lo[2 * c] = half2_as_u32(__hfma2(u32_as_half2(__byte_perm(te, 0x64646464u, 0x4140u)), mule, adde));
                    lo[2 * c + 1] = half2_as_u32(__hfma2(u32_as_half2(__byte_perm(te, 0x64646464u, 0x4342u)), mule, adde));
                    hi[2 * c] = half2_as_u32(__hfma2(u32_as_half2(__byte_perm(to, 0x64646464u, 0x4140u)), mulo, addo));
                    hi[2 * c + 1] = half2_as_u32(__hfma2(u32_as_half2(__byte_perm(to, 0x64646464u, 0x4342u)), mulo, addo));
                }
                tmem_st16(tmem + lane_base + (uint32_t)(as * A_COLS + 32 * j), lo);
                tmem_st16(tmem + lane_base + (uint32_t)(as * A_COLS + 32 * j + 16), hi);
            }
            tmem_st_wait();
            if (warp == 2) TR(2, i, 2);
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                tc::mbar_arrive(empty_w(ws));  // the warp's rows of the slot are in registers or tensor memory
                tc::mbar_arrive(full_a(as));
            }
            if (warp == 2) TR(2, i, 3);
            wr.next(SW);
            ar.next(NA);
            pr.next(SP);
        }
    } else {
        // ---- epilogue: thread = weight row; set `eset` of four warps takes rows m0 .. m0 + HM - 1 of x ------------------------------
        const int r = (warp & 3) * 32 + lane;
        const int eset = (warp - 6) >> 2;
        const int m0 = eset * HM;
        const bool et0 = ((threadIdx.x - 192) & 127) == 0;
        volatile int* fin = fin_all + 4 * eset;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        asm volatile("griddepcontrol.wait;" ::: "memory");  // y and the scratch are no longer in use by the kernel before
        float acc[HM];
#pragma unroll
        for (int m = 0; m < HM; m++) {
            acc[m] = 0.0f;
        }
        Walk we;
        we.start(u0, u1, KB);
        int part_b0 = we.b;  // first super-block of the part of a tile that is being visited
        Ring xr, pr, dr;
        const size_t slot_words = (size_t)a.max_pieces * a.rows * ROWS;
        unsigned long long* const my_slot = a.partial + (size_t)blockIdx.x * slot_words;
        float* const my_aside = a.aside + (size_t)blockIdx.x * slot_words;  // this CTA's own contributions to a tile it finishes after its run
        int late_tile = -1, late_len = 0;
        bool ok = true;
        if (et0) {
            fin[0] = 1;  // cleared by a thread of the set whose wait for another CTA's sums has run out
        }
        epilogue_barrier(1 + eset);
        // y (or every rank's y) for this thread's row of tile `tile`
        auto write_tile = [&](int tile, const float (&sum)[HM]) {
            const int wi = tile < a.tile_end[0] ? 0 : (tile < a.tile_end[1] ? 1 : 2);
            const int t_in = tile - (wi == 0 ? 0 : (wi == 1 ? a.tile_end[0] : a.tile_end[1]));
            const int64_t n = wi == 0 ? a.n[0] : (wi == 1 ? a.n[1] : a.n[2]);
            if (a.NC > 1) {
                // a range of k of tile `t_in / NC` of its weight: its sums wait in `parts` for the kernel that adds the ranges in order
                const int t = t_in / a.NC, c = t_in - t * a.NC;
                const int64_t row = (int64_t)t * ROWS + r;
                if (row < n) {
                    float* dst = a.parts + ((size_t)c * a.rows + m0) * a.n_sum + (wi == 0 ? a.col0[0] : (wi == 1 ? a.col0[1] : a.col0[2])) + row;
#pragma unroll
                    for (int m = 0; m < HM; m++) {
                        if (m0 + m < a.rows) {
                            dst[(size_t)m * a.n_sum] = sum[m];
                        }
                    }
                }
                return;
            }
            const bool second = wi != 0;
            const int64_t row = (int64_t)t_in * ROWS + r;
            float* const yo = wi == 0 ? a.y[0] : (wi == 1 ? a.y[1] : a.y[2]);
            if (row < n) {
                const float bv = (a.bias != nullptr && !second) ? a.bias[row] : 0.0f;
#pragma unroll
                for (int m = 0; m < HM; m++) {
                    if (m0 + m < a.rows) {
                        const float val = sum[m] + bv;
                        if constexpr (!PEER) {
                            yo[(int64_t)(m0 + m) * n + row] = val;
                        } else {
                            // a row shard: the value goes into every rank's y [m, n_total] at this rank's columns
                            const int64_t idx = (int64_t)(m0 + m) * a.peer->n_total + a.peer->col0 + row;
                            if (a.peer->stage[0] != nullptr) {
                                peer_store_marked(a.peer, idx, val, peer_marks_seq(a.peer));  // this kernel's number: read after the wait for the kernel before
                            } else {
                                for (int rk = 0; rk < a.peer->world; rk++) {
                                    a.peer->y[rk][idx] = val;
                                }
                            }
                        }
                    }
                }
            }
        };
        // The sum of the super-blocks of `tile` that the CTAs before this one hold: the first of them its running sum, the ones
        // between it and this CTA (few output rows: a tile is then shared by several CTAs) their contributions one by one. Every
        // float is polled, bounded, until its mark is there; with many output rows the one running sum was written at the start of
        // the other CTA's run. Eight words are requested together (a load from L2 takes the better part of a microsecond).
        auto gather = [&](int tile, float (&sum)[HM]) {
            const int c_first = (int)((((int64_t)tile * KB + 1) * G - 1) / U);
            const int64_t tb = (int64_t)tile * KB;
            bool good = true;
            // the words in k order: the first CTA's running sum, then every contribution of the CTAs between it and this one
            int cta = c_first, q = 0, len = 1;
            bool more = cta < (int)blockIdx.x;
            while (more && good) {
                constexpr int CH = 16;  // words requested together, and asked for again together until every one has its mark
                unsigned long long* ptr[CH];
                int count = 0;
                while (count < CH && more) {
                    ptr[count++] = a.partial + (size_t)cta * slot_words + ((size_t)q * a.rows + m0) * ROWS + r;
                    if (++q == len) {
                        cta++;
                        q = 0;
                        more = cta < (int)blockIdx.x;
                        len = (int)(((int64_t)cta + 1) * U / G - (int64_t)cta * U / G);  // a CTA between the first and this one: its whole run
                    }
                }
                const bool starts = ptr[0] == a.partial + (size_t)c_first * slot_words + (size_t)m0 * ROWS + r;
#pragma unroll
                for (int m = 0; m < HM; m++) {
                    if (m0 + m < a.rows && good) {
                        unsigned long long w[CH];
                        long long t0 = 0;
                        for (;;) {
                            bool all = true;
#pragma unroll
                            for (int c = 0; c < CH; c++) {
                                w[c] = c < count ? handoff_load(ptr[c] + (size_t)m * ROWS) : (1ull << 32);
                            }
#pragma unroll
                            for (int c = 0; c < CH; c++) {
                                all = all && (w[c] >> 32) != 0;
                            }
                            if (all) {
                                break;
                            }
                            if (t0 == 0) {
                                t0 = clock64();
                            } else if (*abort_flag != 0 || clock64() - t0 > limit) {
                                atomicCAS(&g_umma_status, 0, 64 + 5);
                                *abort_flag = 1;
                                good = false;
                                break;
                            }
                        }
                        if (good) {
#pragma unroll
                            for (int c = 0; c < CH; c++) {
                                if (c < count) {
                                    handoff_clear(ptr[c] + (size_t)m * ROWS);
                                    const float v = __uint_as_float((uint32_t)w[c]);
                                    sum[m] = (starts && c == 0) ? v : sum[m] + v;
                                }
                            }
                        }
                    }
                }
            }
            // every thread of the set continues only if all of them got what they waited for
            if (!good) {
                fin[0] = 0;
            }
            epilogue_barrier(1 + eset);
            const bool all_good = fin[0] != 0;
            epilogue_barrier(1 + eset);
            return all_good;
        };
        for (int i = 0; i < units && ok; i++) {
            const int ps = pr.s, xs = xr.s;
            const int t = we.t, b = we.b;
            // What this CTA has of tile t: [part_b0, we.e). Starting at 0 it holds the running sum (written out at KB, handed on as
            // it stands before); starting later it continues a sum that the CTAs before it hold, if it reaches KB, or stores its
            // contributions one by one for the CTA that does.
            const bool stores_each = part_b0 > 0 && we.e < KB;
            // The end of a tile whose beginning other CTAs hold. If only one does (many output rows), it wrote its running sum at the
            // start of its run, long ago: fetch it now and carry on from it. If several do (few output rows), they are still at
            // work: keep this CTA's contributions aside and put everything together when the run is over.
            const bool continues = part_b0 > 0 && we.e == KB;
            const bool aside = continues && (int)blockIdx.x - (int)((((int64_t)t * KB + 1) * G - 1) / U) > 1;
            if (b == part_b0 && continues && !aside) {
                ok = gather(t, acc);
                if (!ok) {
                    break;
                }
            }
            if (!warp_wait_phases(Phase{full_p(ps), pr.ph}, Phase{full_d(dr.s), dr.ph}, Phase{full_x(xs), xr.ph}, !RES, abort_flag, 64 + 4, limit, lane)) {
                ok = false;
                break;
            }
            tc::fence_after_sync();
            if (warp == 6) TR(3, i, 0);
            const uint4 pb = *(reinterpret_cast<const uint4*>(p_ring + ps * P_BYTES) + r);
            warp_arrive(empty_p(ps), lane);
            // the accumulators of this thread's rows of x: for row m the sum over the super-block of quant x scale x high digit, then x low digit
            uint32_t dv[ACC][LDW];
            {
                const uint32_t ds = (uint32_t)dr.s;
#pragma unroll
                for (int j = 0; j < ACC; j++) {
                    tmem_ld<LDW>(dv[j], tmem + lane_base + (uint32_t)(D_BASE + ds * D_COLS + j * N + 2 * m0));
                }
                tmem_ld_wait();
                tc::fence_before_sync();
                warp_arrive(empty_d(ds), lane);
                if (warp == 6) TR(3, i, 1);
                dr.next(ND);
            }
            // ---- this super-block's contribution: d (sum over the two digits of weight x accumulator) - dmin (sum over sub-blocks of min x sum of x) ----
            const float* aux = reinterpret_cast<const float*>(x_ring + (size_t)(RES ? b : xs) * XB + IC::XD) + m0;
            const float d = half_bits_to_float(pb.z), dmin = half_bits_to_float(pb.z >> 16);
            float msum[HM];
#pragma unroll
            for (int m = 0; m < HM; m++) {
                msum[m] = 0.0f;
            }
#pragma unroll
            for (int s = 0; s < 8; s++) {
                const float mn = (float)(((s < 4 ? pb.x : pb.y) >> (8 * (s & 3))) & 0xffu);
#pragma unroll
                for (int m = 0; m < HM; m++) {
                    msum[m] = fmaf(mn, aux[s * IC::MPAD + m], msum[m]);
                }
            }
            float c[HM];
#pragma unroll
            for (int m = 0; m < HM; m++) {
                const float w0 = aux[8 * IC::MPAD + m];
                float dh = __uint_as_float(dv[0][2 * m]), dl = __uint_as_float(dv[0][2 * m + 1]);
#pragma unroll
                for (int j = 1; j < ACC; j++) {
                    dh += __uint_as_float(dv[j][2 * m]);
                    dl += __uint_as_float(dv[j][2 * m + 1]);
                }
                const float q = fmaf(w0 * 2048.0f, dh, w0 * dl);
                c[m] = fmaf(d, q, -(dmin * msum[m]));
            }
            if constexpr (!RES) {
                __syncwarp();
                if (lane == 0) {
                    tc::mbar_arrive(empty_x(xs));
                }
            }
            if (stores_each) {
                unsigned long long* dst = my_slot + ((size_t)(b - part_b0) * a.rows + m0) * ROWS + r;
#pragma unroll
                for (int m = 0; m < HM; m++) {
                    if (m0 + m < a.rows) {
                        handoff_store(dst + m * ROWS, c[m]);
                    }
                }
            } else if (aside) {
                float* dst = my_aside + ((size_t)(b - part_b0) * a.rows + m0) * ROWS + r;
#pragma unroll
                for (int m = 0; m < HM; m++) {
                    if (m0 + m < a.rows) {
                        __stcg(dst + m * ROWS, c[m]);
                    }
                }
                late_tile = t;
                late_len = b - part_b0 + 1;
            } else {
#pragma unroll
                for (int m = 0; m < HM; m++) {
                    acc[m] += c[m];
                }
            }
            if (b == we.e - 1) {
                // the CTA's part of the tile is done
                if (we.e == KB) {
                    if (!aside) {
                        write_tile(t, acc);
                    }
                } else {
                    if (part_b0 == 0) {
                        unsigned long long* dst = my_slot + (size_t)m0 * ROWS + r;  // the running sum of the tile's first super-blocks
#pragma unroll
                        for (int m = 0; m < HM; m++) {
                            if (m0 + m < a.rows) {
                                handoff_store(dst + m * ROWS, acc[m]);
                            }
                        }
                    }
                }
#pragma unroll
                for (int m = 0; m < HM; m++) {
                    acc[m] = 0.0f;
                }
            }
            if (warp == 6) TR(3, i, 3);
            xr.next(SX);
            pr.next(SP);
            we.next();
            if (we.t != t) {
                part_b0 = we.b;
            }
        }
        if (ok && late_tile >= 0) {
            // the tile whose end this CTA computed and kept aside: the other CTAs' sums first, then its own contributions, in k order
            ok = gather(late_tile, acc);
            if (ok) {
                const float* own = my_aside + (size_t)m0 * ROWS + r;
                for (int q0 = 0; q0 < late_len; q0 += 8) {
#pragma unroll
                    for (int m = 0; m < HM; m++) {
                        if (m0 + m < a.rows) {
                            float v[8];
#pragma unroll
                            for (int q = 0; q < 8; q++) {
                                v[q] = q0 + q < late_len ? __ldcg(own + ((size_t)(q0 + q) * a.rows + m) * ROWS) : 0.0f;
                            }
#pragma unroll
                            for (int q = 0; q < 8; q++) {
                                if (q0 + q < late_len) {
                                    acc[m] += v[q];
                                }
                            }
                        }
                    }
                }
                write_tile(late_tile, acc);
            }
        }
    }
    if (warp == 6 && lane == 0) CT(4);
    // ---- common exit: everyone arrives, copies in flight get a bounded time to land after an abort, tensor memory is released ----
    tc::fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag != 0) {
        for (int s = 0; s < SW + (RES ? 0 : SX); s++) {
            const uint32_t bar = s < SW ? full_w(s) : full_x(s - SW);
            for (uint32_t p = 0; p < (1u << 14); p++) {
                if (tc::mbar_try(bar, 0) || tc::mbar_try(bar, 1)) {
                    break;
                }
            }
        }
    }
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
    if constexpr (PEER) {
        if (a.peer->stage[0] != nullptr) {
            __syncthreads();  // no thread of the CTA reads the exchange number after this
            peer_collect(a.peer, a.rows, peer_marks_seq(a.peer), &g_umma_peer_status);  // the other ranks' rows, from this rank's staging words into its y
        } else {
            peer_publish(a.peer->flags, a.peer->rank, a.peer->world, a.peer->wait_after != 0, &g_umma_peer_status);  // every CTA adds its share to this rank's counter on every rank
        }
    }
}

int sm_count_of_current_device() {
    static std::atomic<int> cached{0};
    int v = cached.load();
    if (v == 0) {
        int dev = 0, sms = 0;
        v = (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0) ? sms : 148;
        cached.store(v);
    }
    return v;
}

template <int TYPE, int MR, bool PEER, bool RES>
int launch_typed(const UArgs& a, int grid, size_t smem, cudaStream_t s) {
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    JQ_CUDA(cudaGetDevice(&dev));
    if ((configured.load() >> (dev & 63) & 1) == 0) {
        JQ_CUDA(cudaFuncSetAttribute(gemv_umma_kernel<TYPE, MR, PEER, RES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX));
        configured.fetch_or((uint64_t)1 << (dev & 63));
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(Roles<MR>::THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // may ask for weights while the kernel before it still runs
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    JQ_CUDA(cudaLaunchKernelEx(&cfg, gemv_umma_kernel<TYPE, MR, PEER, RES>, a));
    count_launch();
    return JQ_OK;
}

template <int TYPE, bool PEER>
int by_rows(int mr, bool resident, const UArgs& a, int grid, size_t smem, cudaStream_t s) {
    if (resident) {
        return launch_typed<TYPE, 8, PEER, true>(a, grid, smem, s);
    }
    return mr == 8 ? launch_typed<TYPE, 8, PEER, false>(a, grid, smem, s) : launch_typed<TYPE, 16, PEER, false>(a, grid, smem, s);
}

template <int N>
int launch_image(const float* x, int rows, int64_t k, uint8_t* image, cudaStream_t s) {
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.stream = s;
    cfg.gridDim = dim3((unsigned)(((k / 256) * rows + 3) / 4));
    cfg.blockDim = dim3(128);
    JQ_CUDA(cudaLaunchKernelEx(&cfg, umma_activation_image_kernel<N>, x, rows, k, image));
    count_launch();
    return JQ_OK;
}

int rows_bucket(int rows) { return rows <= 8 ? 8 : 16; }

}  // namespace

size_t gemv_umma_image_bytes(int64_t k, int rows) {
    if (rows < 1 || rows > 16 || k <= 0 || k % 256 != 0) {
        return 0;
    }
    return (size_t)(k / 256) * umma::image_block_bytes(umma::columns_for_rows(rows_bucket(rows)));
}

static bool shape_ok(int type, int64_t k, int rows) {
    return (type == JQ_TYPE_Q4_K || type == JQ_TYPE_Q5_K) && rows >= 1 && rows <= 16 && k > 0 && k % 256 == 0;
}

// Option gemv_tcgen05 = 1: every shape the kernel takes. 0 (the default): where it is measured faster than the mma.sync kernel's
// two passes, which is 11 or more rows of x on a weight with at least one 128-row tile per SM (a CTA's run then spans whole
// tiles and only running sums change hands). 2: never. n = 0: the caller does not know the weight's rows (only option 1 counts).
// Into how many equal ranges the k of a weight with few tiles is cut so that every CTA's run spans at least one (tile, range):
// such a pair is then shared by at most two CTAs and only running sums change hands. 1: no cut needed; 0: no cut of at most 8
// ranges of at least 4 super-blocks does it.
static int ranges_of_k(int type, int kb, int64_t tiles, int sms) {
    if (tiles >= sms) {
        return 1;
    }
    if (type == JQ_TYPE_Q5_K && tiles * kb < 12 * (int64_t)sms) {
        return 0;  // measured: with fewer than 12 units per CTA the Q5_K kernel does not make up for its start and the extra launch
    }
    for (int nc = 2; nc <= 8; nc++) {
        if (kb % nc == 0 && kb / nc >= 4 && tiles * nc >= sms) {
            return nc;
        }
    }
    return 0;
}

bool gemv_umma_takes(int type, int64_t k, int rows, int64_t n) {
    if (!shape_ok(type, k, rows) || g_opt_gemv_generic.load(std::memory_order_relaxed) != 0) {
        return false;
    }
    const int64_t opt = g_opt_gemv_umma.load(std::memory_order_relaxed);
    if (opt != 0) {
        return opt == 1;
    }
    return rows >= UMMA_AUTO_MIN_ROWS && n > 0 && ranges_of_k(type, (int)(k / 256), (n + ROWS - 1) / ROWS, sm_count_of_current_device()) > 0;
}

bool gemv_umma_fallback(int type, int64_t k, int rows) {
    return shape_ok(type, k, rows) && g_opt_gemv_umma.load(std::memory_order_relaxed) != 2 && g_opt_gemv_generic.load(std::memory_order_relaxed) == 0;
}

// Writes the activation image of x [rows, k] for gemv_umma (rows in [1, 16]) into `image` (gemv_umma_image_bytes bytes).
int launch_gemv_umma_image(const float* x, int rows, int64_t k, uint8_t* image, cudaStream_t s) {
    switch (umma::columns_for_rows(rows_bucket(rows))) {
        case 16: return launch_image<16>(x, rows, k, image, s);
        default: return launch_image<32>(x, rows, k, image, s);
    }
}

// y_w [rows, n_w] = x . W_w^T (+ bias for the first) for one to three Q4_K or Q5_K weights of one type and k, and 1 to 16 rows of x:
// the rows of the weights follow one another in the same launch. Either x is given (FP32 [rows, k]; `image` is then scratch of
// gemv_umma_image_bytes(k, rows) bytes that is used unless the kernel can keep the whole image in shared memory), or x is
// nullptr and `image` already holds the activation image, written earlier in the stream.
// `peer` (one weight only): the outputs go into every rank's y of a row-sharded linear instead.
// no_scratch: deal whole tiles to the CTAs, which needs no scratch buffers (and balances the load worse).
int launch_gemv_umma_multi(const View* vs, int count, const float* x, uint8_t* image, int rows, const float* bias, float* const* ys, cudaStream_t s,
                           const PeerOut* peer, bool no_scratch) {
    if (count < 1 || count > 3 || vs == nullptr || ys == nullptr) {
        return fail(JQ_ERR_INVALID, "decode GEMV: %d weights in one launch (1 to 3)", count);
    }
    const View& v = vs[0];
    bool ok = shape_ok(v.type, v.k, rows) && (x != nullptr || image != nullptr) && (count == 1 || peer == nullptr);
    for (int i = 0; i < count && ok; i++) {
        ok = vs[i].type == v.type && vs[i].k == v.k && vs[i].n > 0;
    }
    if (!ok) {
        return fail(JQ_ERR_UNSUPPORTED, "decode GEMV: type %d, k = %lld, %d rows is outside what the tcgen05 kernel takes", v.type, (long long)v.k, rows);
    }
    const int bb = v.type == JQ_TYPE_Q4_K ? 144 : 176;
    const int mr = rows_bucket(rows);
    const int ncols = umma::columns_for_rows(mr);
    int rc = JQ_OK;
    UArgs a = {};
    a.image = image;
    a.bias = bias;
    const int sms = sm_count_of_current_device();
    int64_t tiles_all = 0;
    for (int i = 0; i < count; i++) {
        tiles_all += (vs[i].n + ROWS - 1) / ROWS;
    }
    // Chosen by the default rule for many rows of x on weights of few tiles: the k of every tile in NC ranges (see ranges_of_k).
    // The results then depend on NC, that is on the number of weight rows; asked for by the option, the kernel never cuts k.
    int nc = 1;
    if (g_opt_gemv_umma.load(std::memory_order_relaxed) == 0 && rows >= UMMA_AUTO_MIN_ROWS && peer == nullptr && !no_scratch) {
        nc = ranges_of_k(v.type, (int)(v.k / 256), tiles_all, sms);
        nc = nc < 1 ? 1 : nc;
    }
    a.NC = nc;
    a.KB = (int)(v.k / 256) / nc;
    PartsOut po = {};
    int tile_end = 0;
    int64_t col = 0;
    for (int i = 0; i < 3; i++) {
        const bool live = i < count;
        a.q[i] = live ? vs[i].q : v.q;
        a.y[i] = po.y[i] = live ? ys[i] : ys[0];
        a.n[i] = po.n[i] = live ? vs[i].n : 0;
        a.col0[i] = po.col0[i] = col;  // a weight that is not there starts where the rows end: no column is its
        if (live) {
            tile_end += (int)((vs[i].n + ROWS - 1) / ROWS) * nc;
            col += vs[i].n;
        }
        a.tile_end[i] = tile_end;
    }
    a.n_sum = po.n_sum = col;
    a.tiles = tile_end;
    a.rows = rows;
    const int64_t U = no_scratch ? a.tiles : (int64_t)a.tiles * a.KB;
    const int grid = (int)(U < sms ? U : sms);
    a.whole_tiles = no_scratch ? 1 : 0;
    const int64_t per_cta = (U + grid - 1) / grid;
    a.max_pieces = (int)(per_cta < a.KB - 1 ? per_cta : a.KB - 1);
    if (a.max_pieces < 1) {
        a.max_pieces = 1;
    }
    const size_t xb = (umma::image_block_bytes(ncols) + 127) & ~(size_t)127;
    a.SX = ncols == 16 ? 6 : 4;
    // Few rows of x and a k whose whole image fits beside the weight ring: the kernel builds the image itself in shared memory
    // (no image kernel, no trip of the image through global memory).
    const bool resident = x != nullptr && nc == 1 && ncols <= 16 && (size_t)a.KB * xb <= RESIDENT_MAX;
    if (x != nullptr && !resident) {
        if (image == nullptr) {
            return fail(JQ_ERR_INVALID, "decode GEMV: no scratch for the activation image");
        }
        rc = launch_gemv_umma_image(x, rows, v.k, image, s);
        if (rc != JQ_OK) {
            return rc;
        }
    }
    a.x = x;
    const size_t fixed = 128 + (resident ? (size_t)a.KB : (size_t)a.SX) * xb + SP * P_BYTES + 1024;
    int sw = (int)((SMEM_MAX - fixed) / ((size_t)ROWS * bb));
    a.SW = sw > MAX_SW ? MAX_SW : sw;
    const size_t smem = fixed + (size_t)a.SW * ROWS * bb;
    a.wait_clocks = g_opt_wait_limit_us.load(std::memory_order_relaxed) * 2000;  // about 2 GHz
    a.lbo = (uint32_t)(ncols / 8) * 128u;
    a.sbo = 128u;
    a.peer = peer != nullptr ? peer->table : nullptr;
    // Two scratch areas. The hand-off words are all zero between launches (every word a CTA writes is cleared by the CTA that
    // reads it), whatever the launches' shapes; the floats a CTA keeps aside for itself are never cleared, so they live in an
    // area of their own, where no launch looks for marks.
    uint8_t* partial = nullptr;
    uint8_t* aside = nullptr;
    if (!no_scratch) {
        const size_t words = (size_t)grid * a.max_pieces * rows * ROWS;
        rc = scratch_zeroed_for_slot(s, 2, words * sizeof(unsigned long long), &partial);
        if (rc == JQ_OK) {
            rc = scratch_for_slot(s, 5, words * sizeof(float), &aside);
        }
        if (rc != JQ_OK) {
            return rc;
        }
    }
    a.partial = reinterpret_cast<unsigned long long*>(partial);
    a.aside = reinterpret_cast<float*>(aside);
    if (nc > 1) {
        uint8_t* parts = nullptr;
        rc = scratch_for_slot(s, 4, (size_t)nc * rows * a.n_sum * sizeof(float), &parts);
        if (rc != JQ_OK) {
            return rc;
        }
        a.parts = reinterpret_cast<float*>(parts);
    }
    if (v.type == JQ_TYPE_Q4_K) {
        rc = peer != nullptr ? by_rows<JQ_TYPE_Q4_K, true>(mr, resident, a, grid, smem, s) : by_rows<JQ_TYPE_Q4_K, false>(mr, resident, a, grid, smem, s);
    } else {
        rc = peer != nullptr ? by_rows<JQ_TYPE_Q5_K, true>(mr, resident, a, grid, smem, s) : by_rows<JQ_TYPE_Q5_K, false>(mr, resident, a, grid, smem, s);
    }
    if (rc == JQ_OK && nc > 1) {
        const int64_t outputs = (int64_t)rows * a.n_sum;
        umma_parts_sum_kernel<<<(unsigned)((outputs + 255) / 256), 256, 0, s>>>(a.parts, nc, rows, po, bias);
        count_launch();
        rc = check_launch("umma_parts_sum_kernel");
    }
    return rc;
}

int launch_gemv_umma(const View& v, const View* v2, const float* x, uint8_t* image, int rows, const float* bias, float* y, float* y2, cudaStream_t s,
                     const PeerOut* peer, bool no_scratch) {
    const View vs[2] = {v, v2 != nullptr ? *v2 : v};
    float* const ys[2] = {y, y2};
    return launch_gemv_umma_multi(vs, v2 != nullptr ? 2 : 1, x, image, rows, bias, ys, s, peer, no_scratch);
}

#ifdef JQ_UMMA_TRACE
}  // namespace jq
extern "C" JQ_API int jq_debug_umma_trace(long long* out) {
    return cudaMemcpyFromSymbol(out, jq::g_umma_trace, sizeof(jq::g_umma_trace)) == cudaSuccess ? 0 : -3;
}
extern "C" JQ_API int jq_debug_umma_cta(long long* out) {
    return cudaMemcpyFromSymbol(out, jq::g_umma_cta, sizeof(jq::g_umma_cta)) == cudaSuccess ? 0 : -3;
}
namespace jq {
#endif
// Reads and clears the status words of the tcgen05 GEMV on the current device (0 = no wait ever gave up).
int gemv_umma_status(int* status) {
    const int zero = 0;
    int peer = 0;
    JQ_CUDA(cudaMemcpyFromSymbol(status, g_umma_status, sizeof(int)));
    JQ_CUDA(cudaMemcpyToSymbol(g_umma_status, &zero, sizeof(int)));
    JQ_CUDA(cudaMemcpyFromSymbol(&peer, g_umma_peer_status, sizeof(int)));
    JQ_CUDA(cudaMemcpyToSymbol(g_umma_peer_status, &zero, sizeof(int)));
    if (*status == 0) {
        *status = peer;
    }
    return JQ_OK;
}

}  // namespace jq
