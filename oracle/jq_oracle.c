/*
 * CPU oracle for jitNN's quantised linear operator over GGUF block formats.
 *
 * TEST INFRASTRUCTURE ONLY. This file restates, in plain C, the host ("reference()") arithmetic of
 * the reference operator so that the CUDA library can be checked against it. Nothing in the product
 * path links or calls it: only the test-suite, the smoke check and the CPU-baseline leg of the
 * benchmark do. It is compiled with -ffp-contract=off so that no fused multiply-add is introduced:
 * the reference is Java, which rounds after every float operation.
 *
 * Parity status: pinned for dequantisation and for the linear product by the reference's own
 * fixtures (jitnn-gguf/src/test/resources/gguf/fixture.gguf and the gguf_* cases of
 * jitnn-core/src/test/resources/golden/{manifest.txt,data.bin}); the float -> half rounding inside
 * jqo_quantize_q8_0 follows round-to-nearest-even, which the reference takes from a third-party
 * class (tornado-api 8.1.0 HalfFloat, not in the reference tree): that one conversion is
 * "parity unpinned".
 *
 * Each function cites the reference file:line it follows (paths relative to
 * jitnn-core/src/main/java/ai/beestream/jitnn/ unless stated otherwise).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ggml type ids, jitnn-gguf/src/main/java/ai/beestream/jitnn/gguf/GgmlType.java:27-51 */
enum {
    JQO_Q4_0 = 2,
    JQO_Q4_1 = 3,
    JQO_Q5_0 = 6,
    JQO_Q5_1 = 7,
    JQO_Q8_0 = 8,
    JQO_Q2_K = 10,
    JQO_Q3_K = 11,
    JQO_Q4_K = 12,
    JQO_Q5_K = 13,
    JQO_Q6_K = 14
};

/* DType.java:75-98: values per block and bytes per block. */
int jqo_block_values(int type) {
    switch (type) {
        case JQO_Q8_0: case JQO_Q4_0: case JQO_Q4_1: case JQO_Q5_0: case JQO_Q5_1: return 32;
        case JQO_Q4_K: case JQO_Q5_K: case JQO_Q6_K: case JQO_Q2_K: case JQO_Q3_K: return 256;
        default: return 0;
    }
}

int jqo_block_bytes(int type) {
    switch (type) {
        case JQO_Q8_0: return 34;
        case JQO_Q4_0: return 18;
        case JQO_Q4_1: return 20;
        case JQO_Q4_K: return 144;
        case JQO_Q5_K: return 176;
        case JQO_Q6_K: return 210;
        case JQO_Q5_0: return 22;
        case JQO_Q5_1: return 24;
        case JQO_Q2_K: return 84;
        case JQO_Q3_K: return 110;
        default: return 0;
    }
}

/* IEEE binary16 -> binary32, exact (ByteArray.getHalfFloat(i).getFloat32(), GgufKernels.java:69-71). */
float jqo_half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int shift = 0;
            while ((man & 0x400u) == 0) {
                man <<= 1;
                shift++;
            }
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(113 - shift) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* binary32 -> binary16, round to nearest even (stand-in for tornado-api's `new HalfFloat(float)`,
 * Quant.java:111; rounding mode unpinned). */
uint16_t jqo_float_to_half(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) {
        return (uint16_t)(sign | 0x7c00u | ((absx > 0x7f800000u) ? 0x200u : 0));
    }
    if (absx >= 0x477ff000u) { /* >= 65520 rounds to infinity */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (absx < 0x33000001u) { /* <= 2^-25 rounds to zero */
        return (uint16_t)sign;
    }
    int e = (int)(absx >> 23) - 127;
    uint32_t m = (absx & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { /* subnormal half */
        shift = 13 + (-14 - e);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        m &= 0x7fffffu;
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) {
        q++;
    }
    return (uint16_t)(sign | (base + q));
}

static inline int u8(const uint8_t* w, int64_t at) { return w[at]; }
static inline int i8(const uint8_t* w, int64_t at) { return (int8_t)w[at]; }
static inline float f16(const uint8_t* w, int64_t at) {
    return jqo_half_to_float((uint16_t)(w[at] | (w[at + 1] << 8)));
}

/* GgufKernels.java:74-83: 6-bit scale (part 0) or min (part 1) of sub-block j from 12 bytes at s. */
static int scale_min(const uint8_t* w, int64_t s, int j, int part) {
    if (j < 4) {
        return u8(w, s + j + 4 * part) % 64;
    }
    int low = part == 0 ? u8(w, s + j + 4) % 16 : u8(w, s + j + 4) / 16;
    return low + (u8(w, s + j - 4 + 4 * part) / 64) * 16;
}

/* Quant.java:137-144, Tensor.java:547-554 */
static float q8_0(const uint8_t* w, int64_t i) {
    int64_t base = (i / 32) * 34;
    return f16(w, base) * (float)i8(w, base + 2 + i % 32);
}

/* GgufKernels.java:85-91 */
static float q4_0(const uint8_t* w, int64_t i) {
    int64_t base = (i / 32) * 18;
    int e = (int)(i % 32);
    int b = u8(w, base + 2 + e % 16);
    int q = e < 16 ? b % 16 : b / 16;
    return (float)(q - 8) * f16(w, base);
}

/* GgufKernels.java:93-99: float multiply, then float add (two roundings). */
static float q4_1(const uint8_t* w, int64_t i) {
    int64_t base = (i / 32) * 20;
    int e = (int)(i % 32);
    int b = u8(w, base + 4 + e % 16);
    int q = e < 16 ? b % 16 : b / 16;
    float p = (float)q * f16(w, base);
    return p + f16(w, base + 2);
}

/* GgufKernels.java:101-111: ((d*sc)*q) - (dmin*m), every operation rounded to float. */
static float q4_k(const uint8_t* w, int64_t i) {
    int64_t base = (i / 256) * 144;
    int e = (int)(i % 256);
    int j = e / 64;
    int half = (e % 64) / 32;
    int l = e % 32;
    int sub = 2 * j + half;
    int b = u8(w, base + 16 + 32 * j + l);
    int q = half == 0 ? b % 16 : b / 16;
    float a = f16(w, base) * (float)scale_min(w, base + 4, sub, 0);
    a = a * (float)q;
    float m = f16(w, base + 2) * (float)scale_min(w, base + 4, sub, 1);
    return a - m;
}

/* GgufKernels.java:113-125 */
static float q5_k(const uint8_t* w, int64_t i) {
    int64_t base = (i / 256) * 176;
    int e = (int)(i % 256);
    int j = e / 64;
    int half = (e % 64) / 32;
    int l = e % 32;
    int sub = 2 * j + half;
    int b = u8(w, base + 48 + 32 * j + l);
    int q = half == 0 ? b % 16 : b / 16;
    int hbit = (u8(w, base + 16 + l) / (1 << sub)) % 2;
    q = q + 16 * hbit;
    float a = f16(w, base) * (float)scale_min(w, base + 4, sub, 0);
    a = a * (float)q;
    float m = f16(w, base + 2) * (float)scale_min(w, base + 4, sub, 1);
    return a - m;
}

/* GgufKernels.java:127-140: (d*sc)*q */
static float q6_k(const uint8_t* w, int64_t i) {
    int64_t base = (i / 256) * 210;
    int e = (int)(i % 256);
    int n = e / 128;
    int r = e % 128;
    int k = r / 32;
    int l = r % 32;
    int lb = u8(w, base + 64 * n + l + (k % 2) * 32);
    int low = k < 2 ? lb % 16 : lb / 16;
    int hb = (u8(w, base + 128 + 32 * n + l) / (1 << (2 * k))) % 4;
    int q = low + 16 * hb - 32;
    int sc = i8(w, base + 192 + 8 * n + l / 16 + 2 * k);
    float a = f16(w, base + 208) * (float)sc;
    return a * (float)q;
}

/* GgufKernels.java:142-145 */
static int bit32(const uint8_t* w, int64_t at, int bit) {
    return (u8(w, at + bit / 8) / (1 << (bit % 8))) % 2;
}

/* GgufKernels.java:147-154 */
static float q5_0(const uint8_t* w, int64_t i) {
    int64_t base = (i / 32) * 22;
    int e = (int)(i % 32);
    int b = u8(w, base + 6 + e % 16);
    int q = (e < 16 ? b % 16 : b / 16) + 16 * bit32(w, base + 2, e);
    return (float)(q - 16) * f16(w, base);
}

/* GgufKernels.java:156-163 */
static float q5_1(const uint8_t* w, int64_t i) {
    int64_t base = (i / 32) * 24;
    int e = (int)(i % 32);
    int b = u8(w, base + 8 + e % 16);
    int q = (e < 16 ? b % 16 : b / 16) + 16 * bit32(w, base + 4, e);
    float p = (float)q * f16(w, base);
    return p + f16(w, base + 2);
}

/* GgufKernels.java:165-175 */
static float q2_k(const uint8_t* w, int64_t i) {
    int64_t base = (i / 256) * 84;
    int e = (int)(i % 256);
    int n = e / 128;
    int j = (e % 128) / 32;
    int l = e % 32;
    int sc = u8(w, base + n * 8 + j * 2 + l / 16);
    int q = (u8(w, base + 16 + n * 32 + l) / (1 << (2 * j))) % 4;
    float a = f16(w, base + 80) * (float)(sc % 16);
    a = a * (float)q;
    float m = f16(w, base + 82) * (float)(sc / 16);
    return a - m;
}

/* GgufKernels.java:181-185 */
static int scale3(const uint8_t* w, int64_t s, int is) {
    int low = is < 8 ? u8(w, s + is) % 16 : u8(w, s + is - 8) / 16;
    int high = (u8(w, s + 8 + is % 4) / (1 << (2 * (is / 4)))) % 4;
    return low + 16 * high;
}

/* GgufKernels.java:188-198 */
static float q3_k(const uint8_t* w, int64_t i) {
    int64_t base = (i / 256) * 110;
    int e = (int)(i % 256);
    int n = e / 128;
    int j = (e % 128) / 32;
    int l = e % 32;
    int is = n * 8 + j * 2 + l / 16;
    int q = (u8(w, base + 32 + n * 32 + l) / (1 << (2 * j))) % 4;
    int high = (u8(w, base + l) / (1 << (4 * n + j))) % 2;
    float a = f16(w, base + 108) * (float)(scale3(w, base + 96, is) - 32);
    return a * (float)(q - (high == 1 ? 0 : 4));
}

/* GgufKernels.java:201-223 (`value`), plus Q8_0 from Quant.java:137-144. */
float jqo_value(int type, const uint8_t* w, int64_t i) {
    switch (type) {
        case JQO_Q8_0: return q8_0(w, i);
        case JQO_Q4_0: return q4_0(w, i);
        case JQO_Q4_1: return q4_1(w, i);
        case JQO_Q4_K: return q4_k(w, i);
        case JQO_Q5_K: return q5_k(w, i);
        case JQO_Q6_K: return q6_k(w, i);
        case JQO_Q5_0: return q5_0(w, i);
        case JQO_Q5_1: return q5_1(w, i);
        case JQO_Q2_K: return q2_k(w, i);
        case JQO_Q3_K: return q3_k(w, i);
        default: return NAN;
    }
}

/* ops/Gguf.java:127-133 (Dequantize.reference) and ops/Quant.java:137-144. */
int jqo_dequantize(int type, const uint8_t* w, int64_t count, float* out) {
    if (jqo_block_values(type) == 0) {
        return -1;
    }
    for (int64_t i = 0; i < count; i++) {
        out[i] = jqo_value(type, w, i);
    }
    return 0;
}

/*
 * ops/Gguf.java:187-205 (MatVec.reference): the row of W is dequantised to float and widened to
 * double, the dot product is accumulated in double in index order, the result is cast to float.
 * The prefill composition dequantize + matmul (ops/Gguf.java:94-95, ops/MatMul.java:597-625) has the
 * same arithmetic, so this one routine is the oracle for every row count.
 * threads > 1 splits the output rows over OpenMP threads (something the reference never does; each
 * output keeps its own sequential sum, so results do not depend on the thread count).
 */
int jqo_matvec(int type, const uint8_t* w, const float* x, int64_t rows, int64_t n, int64_t k, float* y, int threads) {
    if (jqo_block_values(type) == 0 || k % jqo_block_values(type) != 0) {
        return -1;
    }
    if (threads < 1) {
        threads = 1;
    }
#pragma omp parallel num_threads(threads)
    {
        double* wr = (double*)malloc(sizeof(double) * (size_t)k);
#pragma omp for schedule(static)
        for (int64_t c = 0; c < n; c++) {
            for (int64_t j = 0; j < k; j++) {
                wr[j] = (double)jqo_value(type, w, c * k + j);
            }
            for (int64_t r = 0; r < rows; r++) {
                double acc = 0;
                for (int64_t j = 0; j < k; j++) {
                    acc += wr[j] * (double)x[r * k + j];
                }
                y[r * n + c] = (float)acc;
            }
        }
        free(wr);
    }
    return 0;
}

/*
 * ops/Quant.java:171-188 (LinearQ8.reference): the accumulator starts at the bias, every product
 * (double)d * q * x is formed in double.
 */
int jqo_linear_q8_0(const uint8_t* w, const float* x, const float* bias, int64_t m, int64_t n, int64_t k, float* y, int threads) {
    if (k % 32 != 0) {
        return -1;
    }
    if (threads < 1) {
        threads = 1;
    }
    int64_t blocks = k / 32;
#pragma omp parallel for schedule(static) num_threads(threads)
    for (int64_t r = 0; r < n; r++) {
        for (int64_t i = 0; i < m; i++) {
            double acc = bias == NULL ? 0 : (double)bias[r];
            for (int64_t j = 0; j < k; j++) {
                int64_t off = (r * blocks + j / 32) * 34;
                acc += (double)f16(w, off) * (double)i8(w, off + 2 + j % 32) * (double)x[i * k + j];
            }
            y[i * n + r] = (float)acc;
        }
    }
    return 0;
}

/*
 * ops/Gguf.java:76-98 (Gguf.linear): Q8_0 goes to Quant.linear (bias inside the sum); every other
 * format is the product followed by a separate float add of the bias.
 */
int jqo_linear(int type, const uint8_t* w, const float* x, const float* bias, int64_t m, int64_t n, int64_t k, float* y, int threads) {
    if (type == JQO_Q8_0) {
        return jqo_linear_q8_0(w, x, bias, m, n, k, y, threads);
    }
    int rc = jqo_matvec(type, w, x, m, n, k, y, threads);
    if (rc != 0) {
        return rc;
    }
    if (bias != NULL) {
        for (int64_t r = 0; r < m; r++) {
            for (int64_t c = 0; c < n; c++) {
                y[r * n + c] = y[r * n + c] + bias[c];
            }
        }
    }
    return 0;
}

/*
 * ops/Quant.java:102-118 (Quantize.reference): amax in double, d = (float)(amax / 127.0), the stored
 * scale is half(d) but the division uses the unrounded float d; halves round away from zero.
 */
int jqo_quantize_q8_0(const float* x, int64_t count, uint8_t* out) {
    if (count % 32 != 0) {
        return -1;
    }
    for (int64_t b = 0; b < count / 32; b++) {
        double amax = 0;
        for (int l = 0; l < 32; l++) {
            double a = fabs((double)x[b * 32 + l]);
            amax = a > amax ? a : amax;
        }
        float d = (float)(amax / 127.0);
        uint16_t h = jqo_float_to_half(d);
        out[b * 34] = (uint8_t)(h & 0xff);
        out[b * 34 + 1] = (uint8_t)(h >> 8);
        for (int l = 0; l < 32; l++) {
            double s = d > 0 ? (double)x[b * 32 + l] / (double)d : 0;
            long long v = s >= 0 ? (long long)(s + 0.5) : -(long long)(-s + 0.5);
            v = v > 127 ? 127 : v;
            v = v < -127 ? -127 : v;
            out[b * 34 + 2 + l] = (uint8_t)(int8_t)v;
        }
    }
    return 0;
}

int jqo_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
