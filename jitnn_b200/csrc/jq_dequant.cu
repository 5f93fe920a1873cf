// Bit-exact dequantisation of an uploaded weight to float32 (Gguf.dequantize / Quant.dequantize of
// the reference: ops/Gguf.java:68-73,127-133, ops/Quant.java:52-60,137-144).
#include "jq_formats.cuh"

namespace jq {

// One thread per unit of a block; each run of 16 weights leaves as four 128-bit stores.
template <int TYPE>
__global__ void __launch_bounds__(256) dequantize_kernel(View v, float* __restrict__ dst, int64_t units) {
    using F = Fmt<TYPE>;
    int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (u >= units) {
        return;
    }
    int64_t block = u / F::UNITS;
    int unit = (int)(u % F::UNITS);
    float out[F::RUNS][16];
    int pos[F::RUNS];
    F::decode(v, block, unit, out, pos);
#pragma unroll
    for (int r = 0; r < F::RUNS; r++) {
        float4* p = reinterpret_cast<float4*>(dst + block * F::QK + pos[r]);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            p[i] = make_float4(out[r][4 * i], out[r][4 * i + 1], out[r][4 * i + 2], out[r][4 * i + 3]);
        }
    }
}

// ---- formats that are dequantised only (no linear kernel): verbatim bytes, one thread per value ----
__device__ __forceinline__ int u8(const uint8_t* w, int64_t at) { return w[at]; }
__device__ __forceinline__ float f16(const uint8_t* w, int64_t at) {
    return __half2float(__ushort_as_half((unsigned short)(w[at] | (w[at + 1] << 8))));
}
__device__ __forceinline__ int bit32(const uint8_t* w, int64_t at, int bit) { return (u8(w, at + bit / 8) >> (bit % 8)) & 1; }

// kernels/GgufKernels.java:147-198 of the reference (Q5_0, Q5_1, Q2_K, Q3_K), one rounded float
// operation per arithmetic step.
__device__ float extra_value(int type, const uint8_t* w, int64_t i) {
    if (type == JQ_TYPE_Q5_0) {
        int64_t base = (i / 32) * 22;
        int e = (int)(i % 32);
        int b = u8(w, base + 6 + e % 16);
        int q = (e < 16 ? b & 15 : b >> 4) + 16 * bit32(w, base + 2, e);
        return __fmul_rn((float)(q - 16), f16(w, base));
    }
    if (type == JQ_TYPE_Q5_1) {
        int64_t base = (i / 32) * 24;
        int e = (int)(i % 32);
        int b = u8(w, base + 8 + e % 16);
        int q = (e < 16 ? b & 15 : b >> 4) + 16 * bit32(w, base + 4, e);
        return __fadd_rn(__fmul_rn((float)q, f16(w, base)), f16(w, base + 2));
    }
    if (type == JQ_TYPE_Q2_K) {
        int64_t base = (i / 256) * 84;
        int e = (int)(i % 256);
        int n = e / 128, j = (e % 128) / 32, l = e % 32;
        int sc = u8(w, base + n * 8 + j * 2 + l / 16);
        int q = (u8(w, base + 16 + n * 32 + l) >> (2 * j)) & 3;
        float a = __fmul_rn(__fmul_rn(f16(w, base + 80), (float)(sc & 15)), (float)q);
        return __fsub_rn(a, __fmul_rn(f16(w, base + 82), (float)(sc >> 4)));
    }
    // Q3_K
    int64_t base = (i / 256) * 110;
    int e = (int)(i % 256);
    int n = e / 128, j = (e % 128) / 32, l = e % 32;
    int is = n * 8 + j * 2 + l / 16;
    int q = (u8(w, base + 32 + n * 32 + l) >> (2 * j)) & 3;
    int high = (u8(w, base + l) >> (4 * n + j)) & 1;
    int64_t s = base + 96;
    int low = is < 8 ? u8(w, s + is) & 15 : u8(w, s + is - 8) >> 4;
    int hi2 = (u8(w, s + 8 + is % 4) >> (2 * (is / 4))) & 3;
    int scale = low + 16 * hi2 - 32;
    return __fmul_rn(__fmul_rn(f16(w, base + 108), (float)scale), (float)(q - (high == 1 ? 0 : 4)));
}

__global__ void dequantize_extra_kernel(int type, const uint8_t* __restrict__ w, float* __restrict__ dst, int64_t count) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) {
        dst[i] = extra_value(type, w, i);
    }
}

template <int TYPE>
static int run(const View& v, float* dst, cudaStream_t s) {
    int64_t units = v.n * (v.k / Fmt<TYPE>::QK) * Fmt<TYPE>::UNITS;
    if (units == 0) {
        return JQ_OK;
    }
    dequantize_kernel<TYPE><<<(unsigned)((units + 255) / 256), 256, 0, s>>>(v, dst, units);
    count_launch();
    return check_launch("dequantize_kernel");
}

int launch_dequantize(const View& v, float* dst, cudaStream_t s) {
    switch (v.type) {
        case JQ_TYPE_Q8_0: return run<JQ_TYPE_Q8_0>(v, dst, s);
        case JQ_TYPE_Q4_0: return run<JQ_TYPE_Q4_0>(v, dst, s);
        case JQ_TYPE_Q4_1: return run<JQ_TYPE_Q4_1>(v, dst, s);
        case JQ_TYPE_Q4_K: return run<JQ_TYPE_Q4_K>(v, dst, s);
        case JQ_TYPE_Q5_K: return run<JQ_TYPE_Q5_K>(v, dst, s);
        case JQ_TYPE_Q6_K: return run<JQ_TYPE_Q6_K>(v, dst, s);
        case JQ_TYPE_Q5_0: case JQ_TYPE_Q5_1: case JQ_TYPE_Q2_K: case JQ_TYPE_Q3_K: {
            int64_t count = v.n * v.k;
            if (count == 0) {
                return JQ_OK;
            }
            dequantize_extra_kernel<<<(unsigned)((count + 255) / 256), 256, 0, s>>>(v.type, v.q, dst, count);
            count_launch();
            return check_launch("dequantize_extra_kernel");
        }
        default: return fail(JQ_ERR_UNSUPPORTED, "dequantize: unknown type %d", v.type);
    }
}

}  // namespace jq
