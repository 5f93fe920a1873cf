// FP32 -> Q8_0 quantiser (F.quantizeQ8 of the reference), following the host form
// ops/Quant.java:102-118: the scale and the rounding are computed in double so that the blocks equal
// the reference's bit for bit.
#include <cuda_fp16.h>

#include "jq_common.cuh"

namespace jq {

// One warp per block of 32 values; output verbatim GGUF Q8_0 blocks (34 bytes, 2-byte aligned).
__global__ void __launch_bounds__(256) quantize_q8_0_kernel(const float* __restrict__ x, uint8_t* __restrict__ out, int64_t blocks) {
    int64_t b = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int lane = threadIdx.x & 31;
    if (b >= blocks) {
        return;
    }
    float v = x[b * 32 + lane];
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    }
    float d = (float)((double)amax / 127.0);
    double s = d > 0.0f ? (double)v / (double)d : 0.0;
    long long q = s >= 0 ? (long long)(s + 0.5) : -(long long)(-s + 0.5);
    q = q > 127 ? 127 : q;
    q = q < -127 ? -127 : q;
    uint8_t* blk = out + b * 34;
    if (lane == 0) {
        *reinterpret_cast<unsigned short*>(blk) = __half_as_ushort(__float2half_rn(d));
    }
    blk[2 + lane] = (uint8_t)(int8_t)q;
}

int launch_quantize_q8_0(const float* x, int64_t blocks, uint8_t* out, cudaStream_t s) {
    if (blocks == 0) {
        return JQ_OK;
    }
    quantize_q8_0_kernel<<<(unsigned)((blocks + 7) / 8), 256, 0, s>>>(x, out, blocks);
    count_launch();
    return check_launch("quantize_q8_0_kernel");
}

}  // namespace jq
