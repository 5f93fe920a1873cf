// Input gradient of the quantised linear: gx[m, k] = sum_n g[m, n] * dequant(W)[n, k]
// (ops/Gguf.java:208-212 and ops/Quant.java:191-197 of the reference: gx = g . dequant(W), no weight gradient; the
// bias gradient is a plain column sum that the caller's framework already has).
//
// The weight is streamed once per tile of g rows, in its quantised form: a thread owns one unit of a block column
// (16 to 64 consecutive weights of every row, decoded with the format's bit-exact decoder), walks down the rows of its
// slab and accumulates g[m, n] * w[n, k] in FP32 for its rows of g. Slabs of rows keep enough CTAs in flight; their
// partial sums are added in slab order by a second kernel, so results do not depend on scheduling.
#include "jq_formats.cuh"

namespace jq {

namespace {

constexpr int BWD_THREADS = 128;

// MT rows of g per pass, chosen so that a thread holds 64 accumulators whatever the format's unit size.
template <int TYPE>
struct BwdTile {
    static constexpr int MT = 4 / Fmt<TYPE>::RUNS;
};

// grid (ceil(units per row / 128), slabs, ceil(m / MT)); out = partial sums [slab][m][k] (or gx itself with one slab)
template <int TYPE>
__global__ void __launch_bounds__(BWD_THREADS) linear_backward_kernel(View v, const float* __restrict__ g, int64_t m, float* __restrict__ out,
                                                                      int64_t rows_per_slab) {
    using F = Fmt<TYPE>;
    constexpr int MT = BwdTile<TYPE>::MT;
    const int64_t blocks_per_row = v.k / F::QK, units_per_row = blocks_per_row * F::UNITS;
    const int64_t u = (int64_t)blockIdx.x * BWD_THREADS + threadIdx.x;
    if (u >= units_per_row) {
        return;
    }
    const int64_t kb = u / F::UNITS;
    const int unit = (int)(u % F::UNITS);
    const int64_t n0 = (int64_t)blockIdx.y * rows_per_slab;
    const int64_t n1 = n0 + rows_per_slab < v.n ? n0 + rows_per_slab : v.n;
    const int64_t m0 = (int64_t)blockIdx.z * MT;
    float acc[MT][F::RUNS][16];
#pragma unroll
    for (int a = 0; a < MT; a++) {
#pragma unroll
        for (int r = 0; r < F::RUNS; r++) {
#pragma unroll
            for (int i = 0; i < 16; i++) {
                acc[a][r][i] = 0.0f;
            }
        }
    }
    int pos[F::RUNS];
    for (int64_t n = n0; n < n1; n++) {
        float w[F::RUNS][16];
        F::decode(v, n * blocks_per_row + kb, unit, w, pos);
#pragma unroll
        for (int a = 0; a < MT; a++) {
            const float gv = m0 + a < m ? __ldg(g + (m0 + a) * v.n + n) : 0.0f;
#pragma unroll
            for (int r = 0; r < F::RUNS; r++) {
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    acc[a][r][i] = fmaf(gv, w[r][i], acc[a][r][i]);
                }
            }
        }
    }
    if (n1 <= n0) {
        return;  // an empty slab cannot happen with the launcher's slab count; nothing to write
    }
    float* base = out + (int64_t)blockIdx.y * m * v.k;
#pragma unroll
    for (int a = 0; a < MT; a++) {
        if (m0 + a < m) {
#pragma unroll
            for (int r = 0; r < F::RUNS; r++) {
                float4* p = reinterpret_cast<float4*>(base + (m0 + a) * v.k + kb * F::QK + pos[r]);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    p[i] = make_float4(acc[a][r][4 * i], acc[a][r][4 * i + 1], acc[a][r][4 * i + 2], acc[a][r][4 * i + 3]);
                }
            }
        }
    }
}

// gx[i] = partial[0][i] + partial[1][i] + ... in slab order
__global__ void __launch_bounds__(256) backward_reduce_kernel(const float* __restrict__ partial, int slabs, int64_t count, float* __restrict__ gx) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) {
        return;
    }
    float s = partial[i];
    for (int sl = 1; sl < slabs; sl++) {
        s += partial[(int64_t)sl * count + i];
    }
    gx[i] = s;
}

template <int TYPE>
int run(const View& v, const float* g, int64_t m, float* gx, cudaStream_t s) {
    using F = Fmt<TYPE>;
    constexpr int MT = BwdTile<TYPE>::MT;
    const int64_t units_per_row = v.k / F::QK * F::UNITS;
    const unsigned gx_ctas = (unsigned)((units_per_row + BWD_THREADS - 1) / BWD_THREADS);
    const unsigned gz = (unsigned)((m + MT - 1) / MT);
    // about eight CTAs per SM over the whole grid, at least 64 rows per slab, at most 64 slabs
    int64_t slabs = (148 * 8 + (int64_t)gx_ctas * gz - 1) / ((int64_t)gx_ctas * gz);
    const int64_t max_slabs = (v.n + 63) / 64;
    slabs = slabs > max_slabs ? max_slabs : slabs;
    slabs = slabs > 64 ? 64 : (slabs < 1 ? 1 : slabs);
    int64_t rows_per_slab = (v.n + slabs - 1) / slabs;
    slabs = (v.n + rows_per_slab - 1) / rows_per_slab;  // no empty slab
    float* out = gx;
    if (slabs > 1) {
        uint8_t* scratch = nullptr;
        int rc = scratch_for(s, (size_t)slabs * m * v.k * sizeof(float), &scratch);
        if (rc != JQ_OK) {
            return rc;
        }
        out = reinterpret_cast<float*>(scratch);
    }
    linear_backward_kernel<TYPE><<<dim3(gx_ctas, (unsigned)slabs, gz), BWD_THREADS, 0, s>>>(v, g, m, out, rows_per_slab);
    count_launch();
    int rc = check_launch("linear_backward_kernel");
    if (rc == JQ_OK && slabs > 1) {
        const int64_t count = m * v.k;
        backward_reduce_kernel<<<(unsigned)((count + 255) / 256), 256, 0, s>>>(out, (int)slabs, count, gx);
        count_launch();
        rc = check_launch("backward_reduce_kernel");
    }
    return rc;
}

}  // namespace

// gx [m, k] = g [m, n] . dequant(W); device pointers, gx 16-byte aligned; n >= 1, m >= 1.
int launch_linear_backward(const View& v, const float* g, int64_t m, float* gx, cudaStream_t s) {
    switch (v.type) {
        case JQ_TYPE_Q8_0: return run<JQ_TYPE_Q8_0>(v, g, m, gx, s);
        case JQ_TYPE_Q4_0: return run<JQ_TYPE_Q4_0>(v, g, m, gx, s);
        case JQ_TYPE_Q4_1: return run<JQ_TYPE_Q4_1>(v, g, m, gx, s);
        case JQ_TYPE_Q4_K: return run<JQ_TYPE_Q4_K>(v, g, m, gx, s);
        case JQ_TYPE_Q5_K: return run<JQ_TYPE_Q5_K>(v, g, m, gx, s);
        case JQ_TYPE_Q6_K: return run<JQ_TYPE_Q6_K>(v, g, m, gx, s);
        default: return fail(JQ_ERR_UNSUPPORTED, "linear backward: type %d is dequantise-only", v.type);
    }
}

}  // namespace jq
