// Fused dequantise-GEMV for decode: y[m, n] = x[m, k] . W[n, k]^T (+ bias), 1 <= m <= 16.
//
// Replaces the reference's matrix-vector kernels (kernels/jitllm/TransformerComputeKernelsQ4_K.java:130-215
// and siblings, kernels/Q8Kernels.java:102-155), which read weights byte by byte and decode the block
// scales again for every element. Here a weight is read from HBM exactly once with 128-bit loads,
// decoded once per unit and used for all m activation rows; accumulation is FP32 in a fixed order
// that depends only on k (so a row-sharded weight gives bitwise the same outputs as the whole one).
#include "jq_formats.cuh"

namespace jq {

constexpr int GEMV_WARPS = 4;

// One warp per output row; lanes stride over the row's units. MT = activation rows held in registers.
template <int TYPE, int MT>
__global__ void __launch_bounds__(GEMV_WARPS * 32) gemv_rows_kernel(View v, const float* __restrict__ x, int rows,
                                                                   const float* __restrict__ bias, float* __restrict__ y) {
    using F = Fmt<TYPE>;
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * GEMV_WARPS + (threadIdx.x >> 5);
    if (row >= v.n) {
        return;
    }
    const int blocks_per_row = (int)(v.k / F::QK);
    const int units = blocks_per_row * F::UNITS;
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) {
        acc[m] = 0.0f;
    }
    for (int u = lane; u < units; u += 32) {
        const int b = u / F::UNITS;
        float w[F::RUNS][16];
        int pos[F::RUNS];
        F::decode(v, row * blocks_per_row + b, u % F::UNITS, w, pos);
#pragma unroll
        for (int r = 0; r < F::RUNS; r++) {
            const float* xp = x + (int64_t)b * F::QK + pos[r];
#pragma unroll
            for (int m = 0; m < MT; m++) {
                if (m < rows) {
                    const float4* x4 = reinterpret_cast<const float4*>(xp + (int64_t)m * v.k);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        float4 t = __ldg(x4 + i);
                        acc[m] = fmaf(w[r][4 * i], t.x, acc[m]);
                        acc[m] = fmaf(w[r][4 * i + 1], t.y, acc[m]);
                        acc[m] = fmaf(w[r][4 * i + 2], t.z, acc[m]);
                        acc[m] = fmaf(w[r][4 * i + 3], t.w, acc[m]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MT; m++) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
        }
    }
    if (lane == 0) {
        const float b = bias != nullptr ? bias[row] : 0.0f;
#pragma unroll
        for (int m = 0; m < MT; m++) {
            if (m < rows) {
                y[(int64_t)m * v.n + row] = acc[m] + b;
            }
        }
    }
}

template <int TYPE, int MT>
static int run(const View& v, const float* x, int rows, const float* bias, float* y, cudaStream_t s) {
    unsigned grid = (unsigned)((v.n + GEMV_WARPS - 1) / GEMV_WARPS);
    gemv_rows_kernel<TYPE, MT><<<grid, GEMV_WARPS * 32, 0, s>>>(v, x, rows, bias, y);
    count_launch();
    return check_launch("gemv_rows_kernel");
}

template <int TYPE>
static int by_rows(const View& v, const float* x, int rows, const float* bias, float* y, cudaStream_t s) {
    if (rows == 1) return run<TYPE, 1>(v, x, rows, bias, y, s);
    if (rows == 2) return run<TYPE, 2>(v, x, rows, bias, y, s);
    if (rows <= 4) return run<TYPE, 4>(v, x, rows, bias, y, s);
    if (rows <= 8) return run<TYPE, 8>(v, x, rows, bias, y, s);
    return run<TYPE, 16>(v, x, rows, bias, y, s);
}

// rows in [1, 16].
int launch_gemv(const View& v, const float* x, int rows, const float* bias, float* y, cudaStream_t s, bool x_remote) {
    if (v.n == 0) {
        return JQ_OK;
    }
    if (gemv_umma_takes(v.type, v.k, rows, v.n)) {
        // Q4_K, Q5_K: the tcgen05 kernel, one pass over the weights for up to 16 rows
        uint8_t* image = nullptr;
        int rc = scratch_for(s, gemv_umma_image_bytes(v.k, rows), &image);
        return rc == JQ_OK ? launch_gemv_umma(v, nullptr, x, image, rows, bias, y, nullptr, s) : rc;
    }
    if ((v.type == JQ_TYPE_Q4_K || v.type == JQ_TYPE_Q5_K) && rows <= 8 && g_opt_gemv_generic.load(std::memory_order_relaxed) == 0) {
        bool handled = false;
        const size_t need = gemv_q4k_i8_scratch_bytes(v.k, rows);
        uint8_t* image = nullptr;
        int rc = need > 0 ? scratch_for(s, need, &image) : JQ_OK;
        if (rc == JQ_OK) {
            rc = launch_gemv_q4k_i8(v, x, rows, bias, y, s, image, &handled, nullptr, x_remote);
        }
        if (rc != JQ_OK || handled) {
            return rc;
        }
        if (gemv_umma_fallback(v.type, v.k, rows)) {
            // a shape that kernel declines (a large k whose image does not fit beside the sums of many tiles per CTA):
            // the tcgen05 kernel streams the image and is many times faster than the CUDA-core kernel below
            rc = scratch_for(s, gemv_umma_image_bytes(v.k, rows), &image);
            return rc == JQ_OK ? launch_gemv_umma(v, nullptr, x, image, rows, bias, y, nullptr, s) : rc;
        }
    }
    if (v.type == JQ_TYPE_Q6_K && rows <= 4 && g_opt_gemv_generic.load(std::memory_order_relaxed) == 0) {
        bool handled = false;
        const size_t need = gemv_q6k_i8_scratch_bytes(v.k, rows);
        uint8_t* image = nullptr;
        int rc = need > 0 ? scratch_for(s, need, &image) : JQ_OK;
        if (rc == JQ_OK) {
            rc = launch_gemv_q6k_i8(v, x, rows, bias, y, s, image, &handled);
        }
        if (rc != JQ_OK || handled) {
            return rc;
        }
    }
    if (rows <= 2 && g_opt_gemv_generic.load(std::memory_order_relaxed) == 0) {
        const size_t need = gemv_blk32_i8_scratch_bytes(v.type, v.k, rows);  // 0 unless Q8_0, Q4_0, Q4_1 with k a multiple of 256
        if (need > 0) {
            bool handled = false;
            uint8_t* image = nullptr;
            int rc = scratch_for(s, need, &image);
            if (rc == JQ_OK) {
                rc = launch_gemv_blk32_i8(v, x, rows, bias, y, s, image, &handled);
            }
            if (rc != JQ_OK || handled) {
                return rc;
            }
        }
    }
    switch (v.type) {
        case JQ_TYPE_Q8_0: return by_rows<JQ_TYPE_Q8_0>(v, x, rows, bias, y, s);
        case JQ_TYPE_Q4_0: return by_rows<JQ_TYPE_Q4_0>(v, x, rows, bias, y, s);
        case JQ_TYPE_Q4_1: return by_rows<JQ_TYPE_Q4_1>(v, x, rows, bias, y, s);
        case JQ_TYPE_Q4_K: return by_rows<JQ_TYPE_Q4_K>(v, x, rows, bias, y, s);
        case JQ_TYPE_Q5_K: return by_rows<JQ_TYPE_Q5_K>(v, x, rows, bias, y, s);
        case JQ_TYPE_Q6_K: return by_rows<JQ_TYPE_Q6_K>(v, x, rows, bias, y, s);
        default: return fail(JQ_ERR_UNSUPPORTED, "linear: type %d has no matrix-vector kernel", v.type);
    }
}

}  // namespace jq
