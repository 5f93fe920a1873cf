// Llama-style decoder around the quantised linears: the glue kernels (embedding, RMSNorm, RoPE, attention over a
// key/value cache, SwiGLU, residual adds, greedy argmax) and the host loop that strings them together.
//
// The block math is the reference's (jitnn-nn/.../nn/models/Llama.java:209-222; ops/RowNorm.java:266-306;
// ops/Rope.java:84-149; ops/FlashAttention.java:538-626; F.java:588-599,1158-1161; ops/Reduce.java:201) with each
// nn.Linear replaced by jq_linear_f32 on a quantised weight. The reference recomputes all positions on every call and
// has no generation loop; here keys and values are kept in a cache [layer][position][kv_head * head_dim], which
// computes the same function. All arithmetic is FP32 in a fixed order (the reference's host path uses double).
#include <cooperative_groups.h>

#include <cmath>
#include <cstring>
#include <vector>

#include "jq_common.cuh"
#include "jq_q4k_image.cuh"
#include "jq_q6k_image.cuh"
#include "jq_peer_device.cuh"

namespace jq {

int linear_device(const jq_weight* w, const float* x, int64_t m, const float* bias, float* y, cudaStream_t s, bool x_remote = false);
int linear_device_multi(const jq_weight* const* ws, int count, const float* x, int64_t m, float* const* ys, cudaStream_t s);

namespace {

constexpr int MAX_TOKENS = 16;  // activation rows per forward call

__device__ __forceinline__ float block_sum(float v, float* scratch) {
    // fixed-order sum over a CTA of up to 1024 threads
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, o);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) {
        scratch[warp] = v;
    }
    __syncthreads();
    float t = 0.0f;
    for (int i = 0; i < nw; i++) {
        t += scratch[i];
    }
    return t;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) {
        scratch[warp] = v;
    }
    __syncthreads();
    float t = scratch[0];
    for (int i = 1; i < nw; i++) {
        t = fmaxf(t, scratch[i]);
    }
    return t;
}

struct TokenArgs {
    int tokens[MAX_TOKENS];
    int pos0;
};

// Tokens and start position travel as kernel arguments: no host buffer has to stay valid after the call returns.
__global__ void set_tokens_kernel(TokenArgs a, int* __restrict__ tokens, int* __restrict__ pos) {
    if (threadIdx.x < MAX_TOKENS) {
        tokens[threadIdx.x] = a.tokens[threadIdx.x];
    }
    if (threadIdx.x == 0) {
        *pos = a.pos0;
    }
}

// x[t, :] = table[token[t], :]
__global__ void embed_kernel(const int* __restrict__ tokens, const float* __restrict__ table, float* __restrict__ x, int dim, int vocab) {
    asm volatile("griddepcontrol.launch_dependents;");  // launched programmatically, the kernel behind this one may be scheduled now ...
    asm volatile("griddepcontrol.wait;" ::: "memory");  // ... and this one touches memory only when the kernel before it has finished
    int tok = tokens[blockIdx.x];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    const float4* src = reinterpret_cast<const float4*>(table + (int64_t)tok * dim);
    float4* dst = reinterpret_cast<float4*>(x + (int64_t)blockIdx.x * dim);
    for (int i = threadIdx.x; i < dim / 4; i += blockDim.x) {
        dst[i] = src[i];
    }
}

// If delta != nullptr: x += delta (the residual add). Then out = x * rsqrt(mean(x^2) + eps) * w (RMSNorm).
// One CTA of NORM_THREADS threads per row: with few rows the kernel is bound by the latency of its loads, so every thread has
// all of its row's values in flight at once (128-bit loads) and keeps up to 16 of them in registers for the second pass.
constexpr int NORM_THREADS = 1024;
__global__ void __launch_bounds__(NORM_THREADS) add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta, const float* __restrict__ w,
                                                                   float eps, float* __restrict__ out, int dim) {
    asm volatile("griddepcontrol.launch_dependents;");  // launched programmatically, the kernel behind this one may be scheduled now ...
    asm volatile("griddepcontrol.wait;" ::: "memory");  // ... and this one touches memory only when the kernel before it has finished
    __shared__ float scratch[32];
    float* xr = x + (int64_t)blockIdx.x * dim;
    const float* dr = delta != nullptr ? delta + (int64_t)blockIdx.x * dim : nullptr;
    float* o = out + (int64_t)blockIdx.x * dim;
    constexpr int HOLD = 4;
    const int nv = (dim & 3) == 0 ? dim >> 2 : 0;  // 128-bit pieces; a dim that is no multiple of 4 takes the scalar loops below
    float4 held[HOLD];
    float sq = 0.0f;
#pragma unroll
    for (int h = 0; h < HOLD; h++) {
        const int i = threadIdx.x + h * NORM_THREADS;
        held[h] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (i < nv) {
            float4 v = reinterpret_cast<const float4*>(xr)[i];
            if (dr != nullptr) {
                const float4 dv = reinterpret_cast<const float4*>(dr)[i];
                v.x += dv.x; v.y += dv.y; v.z += dv.z; v.w += dv.w;
                reinterpret_cast<float4*>(xr)[i] = v;
            }
            held[h] = v;
            sq = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, sq))));
        }
    }
    const int rest = nv > 0 ? (nv > HOLD * NORM_THREADS ? 4 * HOLD * NORM_THREADS : dim) : 0;  // first element the loops below handle
    for (int i = rest + threadIdx.x; i < dim; i += NORM_THREADS) {
        float v = xr[i];
        if (dr != nullptr) {
            v += dr[i];
            xr[i] = v;
        }
        sq = fmaf(v, v, sq);
    }
    const float total = block_sum(sq, scratch);
    const float inv = 1.0f / sqrtf(total / (float)dim + eps);
#pragma unroll
    for (int h = 0; h < HOLD; h++) {
        const int i = threadIdx.x + h * NORM_THREADS;
        if (i < nv) {
            const float4 wv = reinterpret_cast<const float4*>(w)[i];
            reinterpret_cast<float4*>(o)[i] = make_float4(held[h].x * inv * wv.x, held[h].y * inv * wv.y, held[h].z * inv * wv.z, held[h].w * inv * wv.w);
        }
    }
    for (int i = rest + threadIdx.x; i < dim; i += NORM_THREADS) {
        o[i] = xr[i] * inv * w[i];
    }
}

// x += delta (the last residual add of a block)
__global__ void add_kernel(float* __restrict__ x, const float* __restrict__ delta, int64_t count) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) {
        x[i] += delta[i];
    }
}

// Rotate-half RoPE on the query heads (in place) and key heads, and the append of key and value to the cache.
// grid (tokens, heads + 2 * kv_heads), head_dim / 2 threads.
__global__ void rope_store_kernel(float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, float* __restrict__ k_cache,
                                  float* __restrict__ v_cache, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                  const int* __restrict__ pos0, int heads, int kv_heads, int head_dim, int pos_step, int64_t tok_stride) {
    asm volatile("griddepcontrol.launch_dependents;");  // launched programmatically, the kernel behind this one may be scheduled now ...
    asm volatile("griddepcontrol.wait;" ::: "memory");  // ... and this one touches memory only when the kernel before it has finished
    // consecutive tokens of one sequence: pos_step 1, tok_stride 0; one token each of several sequences at the same
    // position: pos_step 0, tok_stride = elements between two sequences' caches
    const int t = blockIdx.x, h = blockIdx.y, p = threadIdx.x, half = head_dim / 2;
    const int pos = *pos0 + t * pos_step;
    const int kv_dim = kv_heads * head_dim;
    k_cache += t * tok_stride;
    v_cache += t * tok_stride;
    if (h < heads) {
        float* qh = q + ((int64_t)t * heads + h) * head_dim;
        const float c = cos_t[pos * half + p], s = sin_t[pos * half + p];
        const float a = qh[p], b = qh[p + half];
        qh[p] = a * c - b * s;
        qh[p + half] = a * s + b * c;
    } else if (h < heads + kv_heads) {
        const int kh = h - heads;
        const float* src = k + (int64_t)t * kv_dim + kh * head_dim;
        float* dst = k_cache + (int64_t)pos * kv_dim + kh * head_dim;
        const float c = cos_t[pos * half + p], s = sin_t[pos * half + p];
        const float a = src[p], b = src[p + half];
        dst[p] = a * c - b * s;
        dst[p + half] = a * s + b * c;
    } else {
        const int kh = h - heads - kv_heads;
        const float* src = v + (int64_t)t * kv_dim + kh * head_dim;
        float* dst = v_cache + (int64_t)pos * kv_dim + kh * head_dim;
        dst[p] = src[p];
        dst[p + half] = src[p + half];
    }
}

// Causal attention of query (token t, head h) over cache positions 0 .. pos0 + t, split over the keys so that enough CTAs
// are in flight to stream the cache at memory speed: CTA (h, split, t) handles keys [split * ATT_CHUNK, + ATT_CHUNK) and
// writes an unnormalised partial result (running maximum m, sum of exponentials l, sum of exp(score - m) * v); the
// combine kernel merges the partials of a (token, head) in split order. 128 threads; thread d owns output dimension d.
constexpr int ATT_CHUNK = 64;
constexpr int ATT_THREADS = 128;

__global__ void __launch_bounds__(ATT_THREADS) attention_partial_kernel(const float* __restrict__ q, const float* __restrict__ k_cache,
                                                                        const float* __restrict__ v_cache, float* __restrict__ part,
                                                                        const int* __restrict__ pos0, int heads, int kv_heads, int head_dim,
                                                                        int splits, float scale, int pos_step, int64_t tok_stride) {
    asm volatile("griddepcontrol.launch_dependents;");  // launched programmatically, the kernel behind this one may be scheduled now ...
    asm volatile("griddepcontrol.wait;" ::: "memory");  // ... and this one touches memory only when the kernel before it has finished
    __shared__ float qs[256];
    __shared__ float sc[ATT_CHUNK];
    __shared__ float scratch[32];
    const int h = blockIdx.x, sp = blockIdx.y, t = blockIdx.z;
    const int keys = *pos0 + t * pos_step + 1;
    k_cache += t * tok_stride;
    v_cache += t * tok_stride;
    const int k0 = sp * ATT_CHUNK;
    float* out = part + (((int64_t)t * heads + h) * splits + sp) * (head_dim + 2);
    if (k0 >= keys) {
        if (threadIdx.x == 0) {
            out[head_dim] = -INFINITY;  // m
            out[head_dim + 1] = 0.0f;   // l
        }
        return;
    }
    const int cnt = keys - k0 < ATT_CHUNK ? keys - k0 : ATT_CHUNK;
    const int kv_dim = kv_heads * head_dim;
    const int kvh = h / (heads / kv_heads);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* qh = q + ((int64_t)t * heads + h) * head_dim;
    for (int i = threadIdx.x; i < head_dim; i += ATT_THREADS) {
        qs[i] = qh[i];
    }
    __syncthreads();
    // scores: one warp per key, four keys in flight per warp
    const float* kbase = k_cache + (int64_t)k0 * kv_dim + kvh * head_dim;
    for (int j0 = warp * 4; j0 < cnt; j0 += 16) {
        float dot[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int u = 0; u < 4; u++) {
            if (j0 + u < cnt) {
                const float* kr = kbase + (int64_t)(j0 + u) * kv_dim;
                for (int d = lane; d < head_dim; d += 32) {
                    dot[u] = fmaf(qs[d], kr[d], dot[u]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                dot[u] += __shfl_xor_sync(0xffffffffu, dot[u], o);
            }
            if (lane == 0 && j0 + u < cnt) {
                sc[j0 + u] = dot[u] * scale;
            }
        }
    }
    __syncthreads();
    float mx = threadIdx.x < cnt ? sc[threadIdx.x] : -INFINITY;
    mx = block_max(mx, scratch);
    float e = 0.0f;
    if (threadIdx.x < cnt) {
        e = expf(sc[threadIdx.x] - mx);
        sc[threadIdx.x] = e;
    }
    const float l = block_sum(e, scratch);
    __syncthreads();
    // partial output: thread d (and d + 128 for wide heads) sums over the chunk's keys, four at a time
    const float* vbase = v_cache + (int64_t)k0 * kv_dim + kvh * head_dim;
    for (int d = threadIdx.x; d < head_dim; d += ATT_THREADS) {
        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
        int j = 0;
        for (; j + 3 < cnt; j += 4) {
            a0 = fmaf(sc[j], vbase[(int64_t)j * kv_dim + d], a0);
            a1 = fmaf(sc[j + 1], vbase[(int64_t)(j + 1) * kv_dim + d], a1);
            a2 = fmaf(sc[j + 2], vbase[(int64_t)(j + 2) * kv_dim + d], a2);
            a3 = fmaf(sc[j + 3], vbase[(int64_t)(j + 3) * kv_dim + d], a3);
        }
        for (; j < cnt; j++) {
            a0 = fmaf(sc[j], vbase[(int64_t)j * kv_dim + d], a0);
        }
        out[d] = (a0 + a1) + (a2 + a3);
    }
    if (threadIdx.x == 0) {
        out[head_dim] = mx;
        out[head_dim + 1] = l;
    }
}

// out[t, h, :] = sum_s exp(m_s - M) acc_s / sum_s exp(m_s - M) l_s over the splits of (t, h), in split order.
__global__ void attention_combine_kernel(const float* __restrict__ part, float* __restrict__ out, int heads, int head_dim, int stride_splits,
                                         int splits) {
    asm volatile("griddepcontrol.launch_dependents;");  // launched programmatically, the kernel behind this one may be scheduled now ...
    asm volatile("griddepcontrol.wait;" ::: "memory");  // ... and this one touches memory only when the kernel before it has finished
    // stride_splits = chunks the partial buffer was laid out for, splits = chunks written by this call
    const int h = blockIdx.x, t = blockIdx.y;
    const float* p = part + ((int64_t)t * heads + h) * stride_splits * (head_dim + 2);
    float M = -INFINITY;
    for (int s = 0; s < splits; s++) {
        M = fmaxf(M, p[(int64_t)s * (head_dim + 2) + head_dim]);
    }
    float L = 0.0f;
    for (int s = 0; s < splits; s++) {
        const float m = p[(int64_t)s * (head_dim + 2) + head_dim];
        if (m != -INFINITY) {
            L = fmaf(expf(m - M), p[(int64_t)s * (head_dim + 2) + head_dim + 1], L);
        }
    }
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < splits; s++) {
            const float m = p[(int64_t)s * (head_dim + 2) + head_dim];
            if (m != -INFINITY) {
                acc = fmaf(expf(m - M), p[(int64_t)s * (head_dim + 2) + d], acc);
            }
        }
        out[((int64_t)t * heads + h) * head_dim + d] = acc / L;
    }
}

// Causal attention for a long run of consecutive tokens (the prompt path): CTA (head h, group of PA_Q queries) walks the keys
// 0 .. (its last query's position) in tiles of PA_KEYS. A tile of keys and values is loaded into shared memory once and
// serves all PA_Q queries; per query a running maximum m, a running sum l and the output row are carried from tile to
// tile (the usual streaming softmax: out = sum_j exp(s_j - m) v_j / sum_j exp(s_j - m)). Thread (query, key) pairs compute
// the scores, two queries per warp the softmax statistics, thread d the output dimension d of every query.
constexpr int PA_Q = 8;
constexpr int PA_KEYS = 64;
constexpr int PA_THREADS = 128;

template <int HD>
constexpr size_t prompt_attention_smem() {
    return (size_t)(PA_Q * HD + PA_KEYS * (HD + 4) + PA_KEYS * HD + PA_Q * PA_KEYS + 3 * PA_Q) * sizeof(float);
}

template <int HD>
__global__ void __launch_bounds__(PA_THREADS) attention_prompt_kernel(const float* __restrict__ q, const float* __restrict__ k_cache,
                                                                       const float* __restrict__ v_cache, float* __restrict__ out,
                                                                       const int* __restrict__ pos0p, int heads, int kv_heads, int T, float scale) {
    static_assert(HD == 64 || HD == 128, "head sizes of the prompt path");
    extern __shared__ __align__(16) float pa_smem[];
    float* qs = pa_smem;                          // [PA_Q][HD]
    float* ks = qs + PA_Q * HD;                   // [PA_KEYS][HD + 4]: the pad spreads a key's 16-byte pieces over the banks
    float* vs = ks + PA_KEYS * (HD + 4);          // [PA_KEYS][HD]
    float* ps = vs + PA_KEYS * HD;                // [PA_Q][PA_KEYS] scores, then exp(score - m)
    float* m_s = ps + PA_Q * PA_KEYS;             // [PA_Q] running maximum
    float* l_s = m_s + PA_Q;                      // [PA_Q] running sum
    float* a_s = l_s + PA_Q;                      // [PA_Q] exp(m before - m after) of the tile
    const int h = blockIdx.x, t0 = blockIdx.y * PA_Q, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nq = T - t0 < PA_Q ? T - t0 : PA_Q;
    const int pos0 = *pos0p;
    const int kv_dim = kv_heads * HD;
    const int kvh = h / (heads / kv_heads);
    const int keys_all = pos0 + t0 + nq;  // keys the last query of the group sees
    for (int i = tid; i < PA_Q * HD; i += PA_THREADS) {
        const int qi = i / HD, d = i % HD;
        qs[i] = qi < nq ? q[((int64_t)(t0 + qi) * heads + h) * HD + d] : 0.0f;
    }
    if (tid < PA_Q) {
        m_s[tid] = -INFINITY;
        l_s[tid] = 0.0f;
    }
    float acc[PA_Q];
#pragma unroll
    for (int i = 0; i < PA_Q; i++) {
        acc[i] = 0.0f;
    }
    for (int kc = 0; kc < keys_all; kc += PA_KEYS) {
        const int cnt = keys_all - kc < PA_KEYS ? keys_all - kc : PA_KEYS;
        __syncthreads();  // the tile before is used up (first pass: qs, m_s, l_s are written)
        // ---- the tile's keys and values
        constexpr int V4 = HD / 4;
        for (int i = tid; i < PA_KEYS * V4; i += PA_THREADS) {
            const int r = i / V4, c = i % V4;
            float4 kv4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f), vv4 = kv4;
            if (r < cnt) {
                const int64_t off = (int64_t)(kc + r) * kv_dim + kvh * HD + 4 * c;
                kv4 = *reinterpret_cast<const float4*>(k_cache + off);
                vv4 = *reinterpret_cast<const float4*>(v_cache + off);
            }
            *reinterpret_cast<float4*>(ks + r * (HD + 4) + 4 * c) = kv4;
            *reinterpret_cast<float4*>(vs + r * HD + 4 * c) = vv4;
        }
        __syncthreads();
        // ---- scores: pair p = (query p / PA_KEYS, key p % PA_KEYS)
        for (int p = tid; p < PA_Q * PA_KEYS; p += PA_THREADS) {
            const int qi = p / PA_KEYS, j = p % PA_KEYS;
            const float4* kr = reinterpret_cast<const float4*>(ks + j * (HD + 4));
            const float4* qr = reinterpret_cast<const float4*>(qs + qi * HD);
            float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
#pragma unroll 8
            for (int c = 0; c < V4; c++) {
                const float4 a = qr[c], b = kr[c];
                d0 = fmaf(a.x, b.x, d0);
                d1 = fmaf(a.y, b.y, d1);
                d2 = fmaf(a.z, b.z, d2);
                d3 = fmaf(a.w, b.w, d3);
            }
            const bool seen = qi < nq && j < cnt && kc + j <= pos0 + t0 + qi;
            ps[p] = seen ? ((d0 + d1) + (d2 + d3)) * scale : -INFINITY;
        }
        __syncthreads();
        // ---- statistics: warp w takes queries w and w + 4
#pragma unroll
        for (int u = 0; u < PA_Q / 4; u++) {
            const int qi = warp + 4 * u;
            const float s0 = ps[qi * PA_KEYS + lane], s1 = ps[qi * PA_KEYS + lane + 32];
            float mx = fmaxf(s0, s1);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            }
            const float m_old = m_s[qi];
            const float m_new = fmaxf(m_old, mx);
            const float e0 = s0 == -INFINITY ? 0.0f : expf(s0 - m_new), e1 = s1 == -INFINITY ? 0.0f : expf(s1 - m_new);
            float sum = e0 + e1;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                sum += __shfl_xor_sync(0xffffffffu, sum, o);
            }
            ps[qi * PA_KEYS + lane] = e0;
            ps[qi * PA_KEYS + lane + 32] = e1;
            __syncwarp();
            if (lane == 0) {
                const float alpha = m_old == -INFINITY ? 0.0f : expf(m_old - m_new);  // no key seen so far: nothing to carry
                a_s[qi] = alpha;
                l_s[qi] = fmaf(l_s[qi], alpha, sum);
                m_s[qi] = m_new;
            }
        }
        __syncthreads();
        // ---- weighted values: thread d, every query
        if (tid < HD) {
#pragma unroll
            for (int qi = 0; qi < PA_Q; qi++) {
                acc[qi] *= a_s[qi];
            }
            for (int j = 0; j < PA_KEYS; j += 4) {
                const float v0 = vs[j * HD + tid], v1 = vs[(j + 1) * HD + tid], v2 = vs[(j + 2) * HD + tid], v3 = vs[(j + 3) * HD + tid];
#pragma unroll
                for (int qi = 0; qi < PA_Q; qi++) {
                    const float4 pr = *reinterpret_cast<const float4*>(ps + qi * PA_KEYS + j);
                    acc[qi] = fmaf(pr.w, v3, fmaf(pr.z, v2, fmaf(pr.y, v1, fmaf(pr.x, v0, acc[qi]))));
                }
            }
        }
    }
    if (tid < HD) {
#pragma unroll
        for (int qi = 0; qi < PA_Q; qi++) {
            if (qi < nq) {
                out[((int64_t)(t0 + qi) * heads + h) * HD + tid] = acc[qi] / l_s[qi];
            }
        }
    }
}

__global__ void set_pos_kernel(int pos0, int* __restrict__ pos) { *pos = pos0; }

// act = silu(gate) * up
__global__ void swiglu_kernel(const float* __restrict__ gate, const float* __restrict__ up, float* __restrict__ act, int64_t count) {
    asm volatile("griddepcontrol.launch_dependents;");  // launched programmatically, the kernel behind this one may be scheduled now ...
    asm volatile("griddepcontrol.wait;" ::: "memory");  // ... and this one touches memory only when the kernel before it has finished
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) {
        const float g = gate[i];
        act[i] = (g / (1.0f + expf(-g))) * up[i];
    }
}

// First index of the maximum of each row (ops/Reduce.java:201). grid = rows, 1024 threads.
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab) {
    asm volatile("griddepcontrol.launch_dependents;");  // launched programmatically, the kernel behind this one may be scheduled now ...
    asm volatile("griddepcontrol.wait;" ::: "memory");  // ... and this one touches memory only when the kernel before it has finished
    __shared__ float bv[32];
    __shared__ int bi[32];
    const float* row = logits + (int64_t)blockIdx.x * vocab;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (v > best || (v == best && i < idx)) {
            best = v;
            idx = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) {
            best = ov;
            idx = oi;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        bv[threadIdx.x >> 5] = best;
        bi[threadIdx.x >> 5] = idx;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); w++) {
            if (bv[w] > best || (bv[w] == best && bi[w] < idx)) {
                best = bv[w];
                idx = bi[w];
            }
        }
        out[blockIdx.x] = idx;
    }
}


// ---- the single-token step with fewer, fused kernels --------------------------------------------------------------
// For one token and Q4_K / Q6_K linears the kernels that produce an activation vector (norm, attention, SwiGLU) write
// it straight as the activation image the integer GEMV kernels read (jq_q4k_image.cuh, jq_q6k_image.cuh): no float
// vector and no separate image kernel in between. Every kernel of the step starts with griddepcontrol.wait (all that
// the kernel before it wrote is visible from there on) followed by griddepcontrol.launch_dependents (the next kernel
// may be scheduled and, if it is a GEMV, start requesting its weights), and does not touch global memory before.
__device__ __forceinline__ void pdl_enter() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
}

__device__ int g_decoder_peer_status;  // 0, or 32 + rank once a wait of peer_wait_inline in this file has given up

struct Images {
    uint8_t* q4k;  // destination of the Q4_K image, or nullptr if no consumer is Q4_K
    uint8_t* q6k;
};

__device__ __forceinline__ void write_images(const float* block, int b, const Images& im, int lane) {
    if (im.q4k != nullptr) {
        q4k::build_image<1>(block, 0, im.q4k + (size_t)b * q4k::Cfg<1>::PB, lane);
    }
    if (im.q6k != nullptr) {
        q6k::build_image<1>(block, 0, im.q6k + (size_t)b * q6k::Cfg<1>::PB, lane);
    }
}

// x = embedding row of the token (table != nullptr), or x += delta (delta != nullptr), or x as it is; then RMSNorm
// (ops/RowNorm.java:266-306) and from there the images. A thread-block cluster of up to 8 CTAs shares the vector: every
// CTA takes dim / CTAs elements (whole super-blocks of 256), the sums of squares meet through distributed shared
// memory (each CTA adds the partial sums of all CTAs in rank order, so all get the same total), and every CTA writes
// the images of its own super-blocks. blockDim.x = elements per CTA / 4.
__global__ void __launch_bounds__(1024) norm_image_kernel(float* __restrict__ x, const float* __restrict__ delta, const float* __restrict__ table,
                                                          const int* __restrict__ token, int vocab, const float* __restrict__ w, float eps, int dim,
                                                          Images im, const uint32_t* wait_flags, int wait_world) {
    namespace cg = cooperative_groups;
    extern __shared__ __align__(16) float norm_xs[];  // this CTA's normalised elements
    __shared__ float scratch[32];
    __shared__ float partial;
    cg::cluster_group cluster = cg::this_cluster();
    // the norm weights never change: requested before the wait for the kernel in front
    const float4 ww = reinterpret_cast<const float4*>(w + (int)blockIdx.x * (dim / (int)gridDim.x))[threadIdx.x];
    pdl_enter();
    if (wait_flags != nullptr) {
        // delta is what the ranks' latest exchange delivered (row-sharded decoder): complete once all their flags are up
        if (threadIdx.x < 32) {
            peer_wait_inline(wait_flags, wait_world, threadIdx.x, &g_decoder_peer_status);
        }
        __syncthreads();
    }
    const int per_cta = dim / (int)gridDim.x, first = (int)blockIdx.x * per_cta;
    const float4* src = reinterpret_cast<const float4*>(x + first);
    if (table != nullptr) {
        int tok = token[0];
        tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
        src = reinterpret_cast<const float4*>(table + (int64_t)tok * dim + first);
    }
    const int i = (int)threadIdx.x;
    float4 a = src[i];
    if (delta != nullptr) {
        const float4 b = reinterpret_cast<const float4*>(delta + first)[i];
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    }
    if (delta != nullptr || table != nullptr) {
        reinterpret_cast<float4*>(x + first)[i] = a;
    }
    const float sq = fmaf(a.w, a.w, fmaf(a.z, a.z, fmaf(a.y, a.y, a.x * a.x)));
    const float mine = block_sum(sq, scratch);
    if (threadIdx.x == 0) {
        partial = mine;
    }
    cluster.sync();
    float total = 0.0f;
    for (unsigned r = 0; r < cluster.num_blocks(); r++) {
        total += *cluster.map_shared_rank(&partial, r);
    }
    const float inv = 1.0f / sqrtf(total / (float)dim + eps);
    reinterpret_cast<float4*>(norm_xs)[i] = make_float4(a.x * inv * ww.x, a.y * inv * ww.y, a.z * inv * ww.z, a.w * inv * ww.w);
    __syncthreads();
    const int blocks = per_cta >> 8, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (int task = warp; task < 2 * blocks; task += warps) {
        const int b = task < blocks ? task : task - blocks;
        Images one{task < blocks ? im.q4k : nullptr, task < blocks ? nullptr : im.q6k};
        write_images(norm_xs + (size_t)b * 256, (first >> 8) + b, one, lane);
    }
    cluster.sync();  // no CTA leaves (and frees its shared memory) while another may still read its partial sum
}

// Attention of the one new token (head_dim 128): RoPE of its query and key (ops/Rope.java:125-149), the append of key
// and value to the cache, the scores against one chunk of ATT_CHUNK cached keys, and the partial softmax-weighted sum
// of their values, per CTA (head, chunk) of 256 threads. The CTA that finishes last among those of a pair of heads
// (256 outputs = one super-block of the next linear's k) merges the chunks' partial results in chunk order and writes
// them as that linear's activation image.
constexpr int ATTF_THREADS = 256;
// PEER (a rank of the row-sharded decoder): heads are this rank's, the image block goes to the same place of every
// rank's image area, and the CTA that finishes last of the whole grid raises this rank's flag on every rank.
template <bool PEER>
__global__ void __launch_bounds__(ATTF_THREADS) attention_image_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                                                                       float* __restrict__ k_cache, float* __restrict__ v_cache,
                                                                       const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                                       const int* __restrict__ pos0, int heads, int kv_heads, int stride_splits, float scale,
                                                                       float* __restrict__ part, int* __restrict__ counters, Images im, PeerImage pi) {
    constexpr int HD = 128, HALF = 64;
    __shared__ __align__(16) float qs[HD];
    __shared__ __align__(16) float knew[HD];
    __shared__ __align__(16) float vnew[HD];
    __shared__ float sc[ATT_CHUNK];
    __shared__ __align__(16) float red[8][HD];
    __shared__ __align__(16) float outs[256];
    __shared__ int last_flag;
    // The position was set before the first kernel of this step started, and the cached keys and values of earlier
    // positions by earlier steps: both are read before the wait for the kernel in front, so that a CTA scheduled while that
    // kernel still runs has its cache lines on the way.
    const int h = blockIdx.x, sp = blockIdx.y, splits = gridDim.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pos = *pos0, keys = pos + 1, k0 = sp * ATT_CHUNK;
    const int kv_dim = kv_heads * HD, group = heads / kv_heads, kvh = h / group;
    float* out = part + ((int64_t)h * stride_splits + sp) * (HD + 2);
    const int cnt = keys - k0 < ATT_CHUNK ? keys - k0 : ATT_CHUNK;
    // Warp w owns keys 8w .. 8w + 7 of the chunk, a lane four consecutive dimensions of each.
    float4 kreg[8], vreg[8];
#pragma unroll
    for (int u = 0; u < 8; u++) {
        const int j = warp * 8 + u;
        kreg[u] = vreg[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (j < cnt && k0 + j != pos) {
            kreg[u] = __ldg(reinterpret_cast<const float4*>(k_cache + (int64_t)(k0 + j) * kv_dim + kvh * HD) + lane);
            vreg[u] = __ldg(reinterpret_cast<const float4*>(v_cache + (int64_t)(k0 + j) * kv_dim + kvh * HD) + lane);
        }
    }
    pdl_enter();
    if (k0 < keys) {
        const bool has_new = pos < k0 + ATT_CHUNK;  // the new token's key and value belong to this chunk
        if (tid < HALF) {
            const float c = cos_t[pos * HALF + tid], s = sin_t[pos * HALF + tid];
            const float a = q[h * HD + tid], b = q[h * HD + tid + HALF];
            qs[tid] = a * c - b * s;
            qs[tid + HALF] = a * s + b * c;
        } else if (tid < 2 * HALF && has_new) {
            const int p = tid - HALF;
            const float c = cos_t[pos * HALF + p], s = sin_t[pos * HALF + p];
            const float a = k[kvh * HD + p], b = k[kvh * HD + p + HALF];
            const float r0 = a * c - b * s, r1 = a * s + b * c;
            knew[p] = r0;
            knew[p + HALF] = r1;
            if (h % group == 0) {
                k_cache[(int64_t)pos * kv_dim + kvh * HD + p] = r0;
                k_cache[(int64_t)pos * kv_dim + kvh * HD + p + HALF] = r1;
            }
        } else if (tid >= 2 * HALF && has_new) {
            const int p = tid - 2 * HALF;
            const float val = v[kvh * HD + p];
            vnew[p] = val;
            if (h % group == 0) {
                v_cache[(int64_t)pos * kv_dim + kvh * HD + p] = val;
            }
        }
        __syncthreads();
        // this warp's scores, its own running maximum and sum of exponentials, and its weighted sum of values
        const float4 qv = reinterpret_cast<const float4*>(qs)[lane];
        float sco[8], mw = -INFINITY;
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int j = warp * 8 + u;
            if (k0 + j == pos) {
                kreg[u] = reinterpret_cast<const float4*>(knew)[lane];
                vreg[u] = reinterpret_cast<const float4*>(vnew)[lane];
            }
            float dot = fmaf(qv.x, kreg[u].x, fmaf(qv.y, kreg[u].y, fmaf(qv.z, kreg[u].z, qv.w * kreg[u].w)));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                dot += __shfl_xor_sync(0xffffffffu, dot, o);
            }
            sco[u] = j < cnt ? dot * scale : -INFINITY;
            mw = fmaxf(mw, sco[u]);
        }
        float lw = 0.0f;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (mw != -INFINITY) {
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const float pj = expf(sco[u] - mw);  // 0 for the keys beyond the chunk's count
                lw += pj;
                acc.x = fmaf(pj, vreg[u].x, acc.x); acc.y = fmaf(pj, vreg[u].y, acc.y); acc.z = fmaf(pj, vreg[u].z, acc.z); acc.w = fmaf(pj, vreg[u].w, acc.w);
            }
        }
        reinterpret_cast<float4*>(red[warp])[lane] = acc;
        if (lane == 0) {
            sc[warp] = mw;
            sc[8 + warp] = lw;
        }
        __syncthreads();
        // the 8 warps' results in warp order
        if (tid <= HD) {
            float M = sc[0];  // warp 0 always has a key
#pragma unroll
            for (int wv = 1; wv < 8; wv++) {
                M = fmaxf(M, sc[wv]);
            }
            float sum = 0.0f, l = 0.0f;
#pragma unroll
            for (int wv = 0; wv < 8; wv++) {
                const float wgt = expf(sc[wv] - M);  // 0 for a warp without keys
                l = fmaf(wgt, sc[8 + wv], l);
                sum = fmaf(wgt, red[wv][tid & 127], sum);
            }
            if (tid < HD) {
                out[tid] = sum;
            } else {
                out[HD] = M;
                out[HD + 1] = l;
            }
        }
    } else if (tid == 0) {
        out[HD] = -INFINITY;  // no key of this chunk is visible yet
        out[HD + 1] = 0.0f;
    }
    // ---- the last CTA of this pair of heads merges the chunks ---------------------------------------------------------------
    __threadfence();
    __syncthreads();
    const int sb = h >> 1;  // 2 heads of 128 = one super-block of 256
    if (tid == 0) {
        const int done = atomicAdd(&counters[sb], 1);
        last_flag = done == 2 * splits - 1;
        if (last_flag) {
            counters[sb] = 0;  // every CTA of the pair has counted: ready for the next launch
        }
    }
    __syncthreads();
    if (!last_flag) {
        if constexpr (PEER) {
            peer_publish(pi.flags, pi.rank, pi.world, false, nullptr, false);  // this CTA stored nothing to a peer
        }
        return;
    }
    __threadfence();
    {
        // Chunk maxima and sums first, then the weights exp(m - M), then the weighted sums with every load independent of
        // the others (chunks without a visible key have weight zero and their partial sums are never used).
        float* wm = red[0];  // [2 heads][splits <= 128]: m, later the weight
        float* wl = red[2];  // [2 heads][splits]: l
        for (int i = tid; i < 2 * splits; i += ATTF_THREADS) {
            const float* cell = part + ((int64_t)(2 * sb + i / splits) * stride_splits + i % splits) * (HD + 2) + HD;
            wm[(i / splits) * 128 + i % splits] = __ldcg(cell);
            wl[(i / splits) * 128 + i % splits] = __ldcg(cell + 1);
        }
        __syncthreads();
        if (warp < 2) {
            float M = -INFINITY;
            for (int sidx = lane; sidx < splits; sidx += 32) {
                M = fmaxf(M, wm[warp * 128 + sidx]);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
            }
            for (int sidx = lane; sidx < splits; sidx += 32) {
                const float m = wm[warp * 128 + sidx];
                wm[warp * 128 + sidx] = m == -INFINITY ? 0.0f : expf(m - M);
            }
        }
        __syncthreads();
        const int hsel = tid >> 7, d = tid & 127;
        const float* p = part + (int64_t)(2 * sb + hsel) * stride_splits * (HD + 2) + d;
        float L = 0.0f, acc = 0.0f;
#pragma unroll 4
        for (int sidx = 0; sidx < splits; sidx++) {
            const float wgt = wm[hsel * 128 + sidx];
            const float val = __ldcg(p + (int64_t)sidx * (HD + 2));
            L = fmaf(wgt, wl[hsel * 128 + sidx], L);
            acc = fmaf(wgt, wgt != 0.0f ? val : 0.0f, acc);
        }
        outs[tid] = acc / L;
    }
    __syncthreads();
    if (warp == 0) {
        if constexpr (PEER) {
            write_images(outs, pi.first_block + sb, im, lane);
            peer_copy_block(pi, (size_t)(pi.first_block + sb) * q4k::Cfg<1>::PB, (int)q4k::Cfg<1>::PB, lane);
        } else {
            write_images(outs, sb, im, lane);
        }
    }
    if constexpr (PEER) {
        peer_publish(pi.flags, pi.rank, pi.world);
    }
}

// act = silu(gate) * up (F.java:1158-1161) for one super-block of 256 per CTA, written as the next linear's image.
// The sharded form takes SWIGLU_PEER_BLOCKS super-blocks per CTA (one warp each), so that fewer CTAs have to announce
// their stores to the other ranks (each announcement is a release at system scope).
constexpr int SWIGLU_PEER_BLOCKS = 4;
template <bool PEER>
__global__ void __launch_bounds__(256) swiglu_image_kernel(const float* __restrict__ gate, const float* __restrict__ up, Images im, PeerImage pi, int blocks) {
    constexpr int PER_CTA = PEER ? SWIGLU_PEER_BLOCKS : 1;
    __shared__ __align__(16) float xs[PER_CTA][256];
    pdl_enter();
    const int b0 = (int)blockIdx.x * PER_CTA;
    const int nb = blocks - b0 < PER_CTA ? blocks - b0 : PER_CTA;
#pragma unroll
    for (int j = 0; j < PER_CTA; j++) {
        if (j < nb) {
            const int64_t i = (int64_t)(b0 + j) * 256 + threadIdx.x;
            const float g = gate[i];
            xs[j][threadIdx.x] = (g / (1.0f + expf(-g))) * up[i];
        }
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp < nb) {
        if constexpr (PEER) {
            write_images(xs[warp], pi.first_block + b0 + warp, im, lane);
            peer_copy_block(pi, (size_t)(pi.first_block + b0 + warp) * q4k::Cfg<1>::PB, (int)q4k::Cfg<1>::PB, lane);
        } else {
            write_images(xs[warp], b0 + warp, im, lane);
        }
    }
    if constexpr (PEER) {
        peer_publish(pi.flags, pi.rank, pi.world);
    }
}

// First index of the maximum (ops/Reduce.java:201) of one row, over ARGMAX_CTAS CTAs: each leaves its best (value,
// index), the CTA that finishes last picks among them.
constexpr int ARGMAX_CTAS = 64;
__global__ void __launch_bounds__(256) argmax_split_kernel(const float* __restrict__ logits, int vocab, float* __restrict__ best_v, int* __restrict__ best_i,
                                                           int* __restrict__ counter, int* __restrict__ out) {
    __shared__ float bv[8];
    __shared__ int bi[8];
    __shared__ int last_flag;
    pdl_enter();
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = blockIdx.x * 256 + threadIdx.x; i < vocab; i += ARGMAX_CTAS * 256) {
        const float val = logits[i];
        if (val > best || (val == best && i < idx)) {
            best = val;
            idx = i;
        }
    }
    auto better = [](float v1, int i1, float v2, int i2) { return v1 > v2 || (v1 == v2 && i1 < i2); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (better(ov, oi, best, idx)) {
            best = ov;
            idx = oi;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        bv[threadIdx.x >> 5] = best;
        bi[threadIdx.x >> 5] = idx;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int wv = 1; wv < 8; wv++) {
            if (better(bv[wv], bi[wv], best, idx)) {
                best = bv[wv];
                idx = bi[wv];
            }
        }
        best_v[blockIdx.x] = best;
        best_i[blockIdx.x] = idx;
        __threadfence();
        const int done = atomicAdd(counter, 1);
        last_flag = done == ARGMAX_CTAS - 1;
        if (last_flag) {
            *counter = 0;
        }
    }
    __syncthreads();
    if (!last_flag || threadIdx.x >= 32) {
        return;
    }
    __threadfence();
    best = -INFINITY;
    idx = 0x7fffffff;
    for (int c = threadIdx.x; c < ARGMAX_CTAS; c += 32) {
        const float ov = __ldcg(best_v + c);
        const int oi = __ldcg(best_i + c);
        if (better(ov, oi, best, idx)) {
            best = ov;
            idx = oi;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (better(ov, oi, best, idx)) {
            best = ov;
            idx = oi;
        }
    }
    if (threadIdx.x == 0) {
        out[0] = idx == 0x7fffffff ? 0 : idx;
    }
}

// Launch with programmatic stream serialization: the kernel may be scheduled while the one before it still runs
// (it starts with griddepcontrol.wait).
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, bool programmatic, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same for a kernel whose whole grid is one thread-block cluster.
template <typename... KArgs, typename... Args>
cudaError_t launch_cluster_pdl(void (*kernel)(KArgs...), int ctas, dim3 block, size_t smem, cudaStream_t s, bool programmatic, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)ctas;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace

// Reads and clears the status of the exchange waits made by kernels of this file.
int decoder_peer_status(int* status) {
    const int zero = 0;
    JQ_CUDA(cudaMemcpyFromSymbol(status, g_decoder_peer_status, sizeof(int)));
    JQ_CUDA(cudaMemcpyToSymbol(g_decoder_peer_status, &zero, sizeof(int)));
    return JQ_OK;
}

}  // namespace jq

#define JQ_DECODER_MAGIC 0x4a514443u

struct jq_decoder {
    uint32_t magic;
    int device;
    int layers, dim, heads, kv_heads, hidden, vocab, max_seq, head_dim;
    float eps, rope_base;
    std::vector<const jq_weight*> lin;  // [layers][7]: wq, wk, wv, wo, w1 (gate), w3 (up), w2 (down)
    const jq_weight* output;
    float* norms;        // [layers][2][dim] then final [dim]
    float* embed;        // [vocab][dim]
    float *cos_t, *sin_t;
    float *k_cache, *v_cache;  // [sequences][layers][max_seq][kv_dim]
    float *x, *xn, *q, *k, *v, *att, *proj, *gate, *up, *act, *logits;
    float* att_part;     // [tokens][heads][splits][head_dim + 2] partial attention results
    int splits;          // key chunks of ATT_CHUNK positions covering max_seq
    int *tokens, *pos, *argmax;
    uint8_t *img_q4k, *img_q6k;  // activation images of the fused single-token step
    int* counters;               // [dim / 256 attention merge counters][1 argmax counter], zero between launches
    float* argmax_v;             // [ARGMAX_CTAS] per-CTA best value
    int* argmax_i;               // [ARGMAX_CTAS] per-CTA best index
    int* host_stage;     // pinned: [0..7] tokens in, [8] position in, [9..16] argmax out
    int sequences;       // key/value caches held (jq_decoder_set_sequences)
    int cur_seq;         // the sequence the call being enqueued works on
    bool cur_batch;      // the call being enqueued runs one token of each of the first T sequences
    int graph_T, graph_seq;  // what the captured step was captured for (batch: graph_seq = -1)
    int warm_calls;      // decode steps of that kind issued so far
    cudaGraphExec_t graph;  // the decode step, captured on its second call
    cudaStream_t own_stream;  // used when the caller passes no stream (the legacy default stream cannot be captured)
    // Row-sharded form (jq_decoder_set_shard): this rank holds rows [rank * n / world, (rank + 1) * n / world) of every
    // linear, that is heads / world query heads, kv_heads / world key/value heads and hidden / world feed-forward
    // features; the five gathered activations live in the ranks' peer buffers (jq_peer_alloc).
    int world, rank;
    void* peer_buf[8];
    int64_t area[8];  // payload offsets: attention output, wo output, SwiGLU output, w2 output, logits; the Q4_K activation
                      // images of the attention output and of the SwiGLU output; [7] = the end of those
    int64_t stage[6]; // payload offsets of the staging words (8 bytes per element) of the five gathered activations; [5] = the end
    // Workspace of the prompt path (jq_decoder_prompt), allocated by its first call and grown when a longer run arrives:
    // one float buffer cut into the activations of `prompt_rows` tokens, a bfloat16 copy of a linear's input, the tokens.
    float* prompt_buf;
    uint16_t* prompt_bf16;
    int* prompt_tokens;
    int prompt_rows;
};

using namespace jq;

static int check_decoder(const jq_decoder* d, const char* who) {
    if (d == nullptr || d->magic != JQ_DECODER_MAGIC) {
        return fail(JQ_ERR_INVALID, "%s: not a live decoder handle", who);
    }
    return JQ_OK;
}

extern "C" {

JQ_API int jq_decoder_destroy(jq_decoder* d) {
    if (d == nullptr) {
        return JQ_OK;
    }
    int rc = check_decoder(d, "jq_decoder_destroy");
    if (rc != JQ_OK) {
        return rc;
    }
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(d->device);
    float* bufs[] = {d->norms, d->embed, d->cos_t, d->sin_t, d->k_cache, d->v_cache, d->x, d->xn, d->q, d->k, d->v, d->att, d->proj, d->gate, d->up,
                     d->act, d->logits, d->att_part};
    for (float* p : bufs) {
        cudaFree(p);
    }
    cudaFree(d->tokens);
    cudaFree(d->pos);
    cudaFree(d->argmax);
    cudaFree(d->img_q4k);
    cudaFree(d->img_q6k);
    cudaFree(d->counters);
    cudaFree(d->argmax_v);
    cudaFree(d->argmax_i);
    cudaFreeHost(d->host_stage);
    cudaFree(d->prompt_buf);
    cudaFree(d->prompt_bf16);
    cudaFree(d->prompt_tokens);
    if (d->graph != nullptr) {
        cudaGraphExecDestroy(d->graph);
    }
    if (d->own_stream != nullptr) {
        cudaStreamSynchronize(d->own_stream);
        cudaStreamDestroy(d->own_stream);
    }

    if (prev >= 0) {
        cudaSetDevice(prev);
    }
    d->magic = 0;
    delete d;
    return JQ_OK;
}

JQ_API int jq_decoder_create(int device, int layers, int dim, int heads, int kv_heads, int hidden, int vocab, int max_seq, float eps, float rope_base,
                             jq_decoder** out) {
    if (out == nullptr) {
        return fail(JQ_ERR_INVALID, "jq_decoder_create: null result pointer");
    }
    *out = nullptr;
    if (layers < 1 || dim < 1 || heads < 1 || kv_heads < 1 || hidden < 1 || vocab < 1 || max_seq < 1 || dim % heads != 0 || heads % kv_heads != 0) {
        return fail(JQ_ERR_INVALID, "jq_decoder_create: inconsistent sizes (dim %d, heads %d, kv heads %d)", dim, heads, kv_heads);
    }
    const int head_dim = dim / heads;
    if (head_dim % 2 != 0 || head_dim > 256 || dim % 4 != 0 || max_seq > 8192) {
        return fail(JQ_ERR_INVALID, "jq_decoder_create: head_dim %d must be even and at most 256, dim a multiple of 4, max_seq at most 8192", head_dim);
    }
    int count = 0;
    JQ_CUDA(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count) {
        return fail(JQ_ERR_INVALID, "jq_decoder_create: device %d of %d", device, count);
    }
    int prev = -1;
    cudaGetDevice(&prev);
    JQ_CUDA(cudaSetDevice(device));
    jq_decoder* d = new (std::nothrow) jq_decoder();
    if (d == nullptr) {
        return fail(JQ_ERR_OOM, "jq_decoder_create: out of host memory");
    }
    d->magic = JQ_DECODER_MAGIC;
    d->device = device;
    d->layers = layers; d->dim = dim; d->heads = heads; d->kv_heads = kv_heads; d->hidden = hidden; d->vocab = vocab; d->max_seq = max_seq;
    d->head_dim = head_dim; d->eps = eps; d->rope_base = rope_base;
    d->lin.assign((size_t)layers * 7, nullptr);
    d->output = nullptr;
    d->warm_calls = 0;
    d->graph = nullptr;
    d->sequences = 1;
    d->cur_seq = 0;
    d->cur_batch = false;
    d->graph_T = 0;
    d->graph_seq = 0;
    d->own_stream = nullptr;
    d->prompt_buf = nullptr;
    d->prompt_bf16 = nullptr;
    d->prompt_tokens = nullptr;
    d->prompt_rows = 0;
    d->world = 1;
    d->rank = 0;
    for (int r = 0; r < 8; r++) {
        d->peer_buf[r] = nullptr;
    }
    {
        // areas of the peer payload, each for MAX_TOKENS rows and a multiple of 256 bytes
        const int64_t widths[5] = {dim, dim, hidden, dim, vocab};
        int64_t off = 0;
        for (int i = 0; i < 5; i++) {
            d->area[i] = off;
            off += ((int64_t)MAX_TOKENS * widths[i] * (int64_t)sizeof(float) + 255) / 256 * 256;
        }
        d->area[5] = off;
        off += ((int64_t)q4k_image_bytes_one_row(dim) + 511) / 256 * 256;
        d->area[6] = off;
        off += ((int64_t)q4k_image_bytes_one_row(hidden) + 511) / 256 * 256;
        d->area[7] = off;
        for (int i = 0; i < 5; i++) {
            d->stage[i] = off;
            off += ((int64_t)MAX_TOKENS * widths[i] * 8 + 255) / 256 * 256;
        }
        d->stage[5] = off;
    }
    const size_t kv_dim = (size_t)kv_heads * head_dim, T = MAX_TOKENS;
    d->splits = (max_seq + ATT_CHUNK - 1) / ATT_CHUNK;
    struct { float** p; size_t n; } allocs[] = {
        {&d->norms, ((size_t)layers * 2 + 1) * dim}, {&d->embed, (size_t)vocab * dim}, {&d->cos_t, (size_t)max_seq * head_dim / 2},
        {&d->sin_t, (size_t)max_seq * head_dim / 2}, {&d->k_cache, (size_t)layers * max_seq * kv_dim}, {&d->v_cache, (size_t)layers * max_seq * kv_dim},
        {&d->x, T * dim}, {&d->xn, T * dim}, {&d->q, T * dim}, {&d->k, T * kv_dim}, {&d->v, T * kv_dim}, {&d->att, T * dim}, {&d->proj, T * dim},
        {&d->gate, T * hidden}, {&d->up, T * hidden}, {&d->act, T * hidden}, {&d->logits, T * vocab},
        {&d->att_part, T * (size_t)heads * d->splits * (head_dim + 2)}};
    cudaError_t e = cudaSuccess;
    for (auto& a : allocs) {
        *a.p = nullptr;
    }
    d->tokens = d->pos = d->argmax = nullptr;
    d->host_stage = nullptr;
    d->img_q4k = d->img_q6k = nullptr;
    d->counters = nullptr;
    d->argmax_v = nullptr;
    d->argmax_i = nullptr;
    for (auto& a : allocs) {
        if (e == cudaSuccess) {
            e = cudaMalloc(a.p, a.n * sizeof(float));
        }
    }
    if (e == cudaSuccess) e = cudaMalloc(&d->tokens, T * sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&d->pos, sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(&d->argmax, T * sizeof(int));
    if (e == cudaSuccess) e = cudaMallocHost(&d->host_stage, (2 * T + 1) * sizeof(int));
    {
        const int64_t kmax = dim > hidden ? dim : hidden;
        const size_t ncount = (size_t)(dim / 256 + 2);
        if (e == cudaSuccess) e = cudaMalloc(&d->img_q4k, q4k_image_bytes_one_row(kmax) + 256);
        if (e == cudaSuccess) e = cudaMalloc(&d->img_q6k, q6k_image_bytes_one_row(kmax) + 256);
        if (e == cudaSuccess) e = cudaMalloc(&d->counters, ncount * sizeof(int));
        if (e == cudaSuccess) e = cudaMemset(d->counters, 0, ncount * sizeof(int));
        if (e == cudaSuccess) e = cudaMalloc(&d->argmax_v, ARGMAX_CTAS * sizeof(float));
        if (e == cudaSuccess) e = cudaMalloc(&d->argmax_i, ARGMAX_CTAS * sizeof(int));
    }
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&d->own_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) {
        // cos / sin tables in double, stored as float (ops/Rope.java:84-101)
        const int half = head_dim / 2;
        std::vector<float> c((size_t)max_seq * half), s((size_t)max_seq * half);
        for (int t = 0; t < max_seq; t++) {
            for (int i = 0; i < half; i++) {
                const double freq = std::pow((double)rope_base, -2.0 * i / head_dim);
                c[(size_t)t * half + i] = (float)std::cos(t * freq);
                s[(size_t)t * half + i] = (float)std::sin(t * freq);
            }
        }
        e = cudaMemcpy(d->cos_t, c.data(), c.size() * sizeof(float), cudaMemcpyHostToDevice);
        if (e == cudaSuccess) e = cudaMemcpy(d->sin_t, s.data(), s.size() * sizeof(float), cudaMemcpyHostToDevice);
    }
    if (prev >= 0) {
        cudaSetDevice(prev);
    }
    if (e != cudaSuccess) {
        int rc = cuda_fail(e, "jq_decoder_create");
        jq_decoder_destroy(d);
        return rc;
    }
    *out = d;
    return JQ_OK;
}

JQ_API int jq_decoder_peer_bytes(const jq_decoder* d, int64_t* payload_bytes) {
    int rc = check_decoder(d, "jq_decoder_peer_bytes");
    if (rc != JQ_OK) {
        return rc;
    }
    if (payload_bytes == nullptr) {
        return fail(JQ_ERR_INVALID, "jq_decoder_peer_bytes: null result pointer");
    }
    *payload_bytes = d->stage[5];
    return JQ_OK;
}

JQ_API int jq_decoder_set_shard(jq_decoder* d, int rank, int world, void* const* peer_buffers) {
    int rc = check_decoder(d, "jq_decoder_set_shard");
    if (rc != JQ_OK) {
        return rc;
    }
    if (world < 1 || world > 8 || rank < 0 || rank >= world || (world > 1 && peer_buffers == nullptr)) {
        return fail(JQ_ERR_INVALID, "jq_decoder_set_shard: rank %d of %d (at most 8)", rank, world);
    }
    if (d->heads % world != 0 || d->kv_heads % world != 0 || d->hidden % (4 * world) != 0 || d->vocab % (4 * world) != 0) {
        return fail(JQ_ERR_INVALID, "jq_decoder_set_shard: %d ranks do not divide %d heads, %d key/value heads, %d / 4 hidden features and %d / 4 tokens",
                    world, d->heads, d->kv_heads, d->hidden, d->vocab);
    }
    if (d->output != nullptr) {
        return fail(JQ_ERR_INVALID, "jq_decoder_set_shard: call it before the linears are set");
    }
    for (const jq_weight* w : d->lin) {
        if (w != nullptr) {
            return fail(JQ_ERR_INVALID, "jq_decoder_set_shard: call it before the linears are set");
        }
    }
    for (int r = 0; r < world && world > 1; r++) {
        if (peer_buffers[r] == nullptr) {
            return fail(JQ_ERR_INVALID, "jq_decoder_set_shard: the buffer of rank %d is null", r);
        }
    }
    if (d->graph != nullptr) {
        cudaGraphExecDestroy(d->graph);
        d->graph = nullptr;
    }
    d->world = world;
    d->rank = rank;
    for (int r = 0; r < 8; r++) {
        d->peer_buf[r] = world > 1 && r < world ? peer_buffers[r] : nullptr;
    }
    return JQ_OK;
}

JQ_API int jq_decoder_set_linear(jq_decoder* d, int layer, int which, const jq_weight* w) {
    int rc = check_decoder(d, "jq_decoder_set_linear");
    if (rc != JQ_OK) {
        return rc;
    }
    if (w == nullptr || w->magic != JQ_WEIGHT_MAGIC || w->device != d->device) {
        return fail(JQ_ERR_INVALID, "jq_decoder_set_linear: not a live weight on device %d", d->device);
    }
    const int64_t kv_dim = (int64_t)d->kv_heads * d->head_dim;
    int64_t n = 0, k = 0;
    if (layer == -1 && which == 7) {
        n = d->vocab / d->world; k = d->dim;
    } else if (layer >= 0 && layer < d->layers && which >= 0 && which < 7) {
        const int64_t ns[7] = {d->dim, kv_dim, kv_dim, d->dim, d->hidden, d->hidden, d->dim};
        const int64_t ks[7] = {d->dim, d->dim, d->dim, d->dim, d->dim, d->dim, d->hidden};
        n = ns[which] / d->world; k = ks[which];  // a rank of a sharded decoder holds its rows of every weight
    } else {
        return fail(JQ_ERR_INVALID, "jq_decoder_set_linear: layer %d, slot %d", layer, which);
    }
    if (w->n != n || w->k != k) {
        return fail(JQ_ERR_INVALID, "jq_decoder_set_linear: layer %d slot %d needs a [%lld, %lld] weight, got [%lld, %lld]", layer, which, (long long)n,
                    (long long)k, (long long)w->n, (long long)w->k);
    }
    if (d->graph != nullptr) {
        cudaGraphExecDestroy(d->graph);  // the captured forward holds the old weight
        d->graph = nullptr;
    }
    if (layer == -1) {
        d->output = w;
    } else {
        d->lin[(size_t)layer * 7 + which] = w;
    }
    return JQ_OK;
}

JQ_API int jq_decoder_set_norm(jq_decoder* d, int layer, int which, const float* host_weights) {
    int rc = check_decoder(d, "jq_decoder_set_norm");
    if (rc != JQ_OK) {
        return rc;
    }
    size_t slot;
    if (layer == -1) {
        slot = (size_t)d->layers * 2;
    } else if (layer >= 0 && layer < d->layers && (which == 0 || which == 1)) {
        slot = (size_t)layer * 2 + which;
    } else {
        return fail(JQ_ERR_INVALID, "jq_decoder_set_norm: layer %d, slot %d", layer, which);
    }
    if (host_weights == nullptr) {
        return fail(JQ_ERR_INVALID, "jq_decoder_set_norm: null weights");
    }
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(d->device);
    cudaError_t e = cudaMemcpy(d->norms + slot * d->dim, host_weights, (size_t)d->dim * sizeof(float), cudaMemcpyHostToDevice);
    if (prev >= 0) cudaSetDevice(prev);
    return e == cudaSuccess ? JQ_OK : cuda_fail(e, "jq_decoder_set_norm");
}

JQ_API int jq_decoder_set_embedding(jq_decoder* d, const float* host_table) {
    int rc = check_decoder(d, "jq_decoder_set_embedding");
    if (rc != JQ_OK) {
        return rc;
    }
    if (host_table == nullptr) {
        return fail(JQ_ERR_INVALID, "jq_decoder_set_embedding: null table");
    }
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(d->device);
    cudaError_t e = cudaMemcpy(d->embed, host_table, (size_t)d->vocab * d->dim * sizeof(float), cudaMemcpyHostToDevice);
    if (prev >= 0) cudaSetDevice(prev);
    return e == cudaSuccess ? JQ_OK : cuda_fail(e, "jq_decoder_set_embedding");
}

// Whether the single-token step can take the fused kernels: Q4_K / Q6_K linears, head_dim 128, sizes in whole super-blocks.
static bool fused_step_possible(const jq_decoder* d) {
    if (g_opt_decoder_fused.load() == 0 || d->world != 1 || d->head_dim != 128 || d->dim % 256 != 0 || d->hidden % 256 != 0 || d->dim > 32768) {
        return false;
    }
    for (const jq_weight* w : d->lin) {
        if (w == nullptr || (w->type != JQ_TYPE_Q4_K && w->type != JQ_TYPE_Q6_K)) {
            return false;
        }
    }
    return d->output != nullptr && (d->output->type == JQ_TYPE_Q4_K || d->output->type == JQ_TYPE_Q6_K);
}

// The image buffers the kernels in front of the given linears have to fill.
static Images decoder_images_for(const jq_decoder* d, std::initializer_list<const jq_weight*> consumers) {
    Images im{nullptr, nullptr};
    for (const jq_weight* w : consumers) {
        if (w->type == JQ_TYPE_Q4_K) im.q4k = d->img_q4k;
        if (w->type == JQ_TYPE_Q6_K) im.q6k = d->img_q6k;
    }
    return im;
}

// y = W x (and y2 = W2 x in the same launch when both are Q4_K), x being the image written just before
static int decoder_gemv_imaged(jq_decoder* d, const jq_weight* w, float* y, const jq_weight* w2, float* y2, cudaStream_t gs);

// The same for three weights (wq, wk, wv): one launch when all are Q4_K, else the first two together and the third alone.
static int decoder_gemv_imaged3(jq_decoder* d, const jq_weight* w, float* y, const jq_weight* w2, float* y2, const jq_weight* w3, float* y3,
                                cudaStream_t gs) {
    if (w->type == JQ_TYPE_Q4_K && w2->type == JQ_TYPE_Q4_K && w3->type == JQ_TYPE_Q4_K) {
        const View v{w->q, w->aux, w->n, w->k, w->type}, v2{w2->q, w2->aux, w2->n, w2->k, w2->type}, v3{w3->q, w3->aux, w3->n, w3->k, w3->type};
        bool handled = false;
        int rc = launch_gemv_q4k_i8_imaged(v, &v2, d->img_q4k, nullptr, y, y2, gs, &handled, nullptr, &v3, y3);
        if (rc != JQ_OK || handled) {
            return rc;
        }
    }
    int rc = decoder_gemv_imaged(d, w, y, w2, y2, gs);
    return rc == JQ_OK ? decoder_gemv_imaged(d, w3, y3, nullptr, nullptr, gs) : rc;
}

static int decoder_gemv_imaged(jq_decoder* d, const jq_weight* w, float* y, const jq_weight* w2, float* y2, cudaStream_t gs) {
    int rc = JQ_OK;
    for (int pass = 0; pass < 2 && rc == JQ_OK; pass++) {
        const jq_weight* cur = pass == 0 ? w : w2;
        float* out_ = pass == 0 ? y : y2;
        if (cur == nullptr) {
            break;
        }
        const View v{cur->q, cur->aux, cur->n, cur->k, cur->type};
        bool handled = false;
        if (cur->type == JQ_TYPE_Q4_K) {
            if (pass == 0 && w2 != nullptr && w2->type == JQ_TYPE_Q4_K) {
                const View v2{w2->q, w2->aux, w2->n, w2->k, w2->type};
                rc = launch_gemv_q4k_i8_imaged(v, &v2, d->img_q4k, nullptr, y, y2, gs, &handled);
                pass = 1;  // both done
            } else {
                rc = launch_gemv_q4k_i8_imaged(v, nullptr, d->img_q4k, nullptr, out_, nullptr, gs, &handled);
            }
        } else {
            rc = launch_gemv_q6k_i8_imaged(v, d->img_q6k, nullptr, out_, gs, &handled);
        }
        if (rc == JQ_OK && !handled) {
            rc = fail(JQ_ERR_UNSUPPORTED, "decoder: a [%lld, %lld] linear is outside what the tensor-core GEMV takes (set option decoder_fused to 0)",
                      (long long)cur->n, (long long)cur->k);
        }
    }
    return rc;
}

// The forward of one token with the fused kernels (see pdl_enter above). `first_programmatic` is false when the
// operation before the first kernel in the stream is not a kernel (the token copy of the captured graph).
static int enqueue_forward_fused(jq_decoder* d, int max_keys, const TokenArgs* ta, cudaStream_t s) {
    const int dim = d->dim;
    const int64_t kv_dim = (int64_t)d->kv_heads * d->head_dim;
    int rc = JQ_OK;
    auto CKL = [&](cudaError_t e, const char* name) {
        count_launch(1);
        if (rc == JQ_OK && e != cudaSuccess) {
            rc = cuda_fail(e, name);
        }
    };
    auto images_for = [&](std::initializer_list<const jq_weight*> consumers) { return decoder_images_for(d, consumers); };
    auto GEMV = [&](const jq_weight* w, float* y, const jq_weight* w2, float* y2, cudaStream_t gs) {
        if (rc == JQ_OK) {
            rc = decoder_gemv_imaged(d, w, y, w2, y2, gs);
        }
    };
    bool first_programmatic = true;
    if (ta != nullptr) {
        set_tokens_kernel<<<1, 32, 0, s>>>(*ta, d->tokens, d->pos);
        CKL(cudaGetLastError(), "set_tokens_kernel");
    } else {
        cudaError_t e = cudaMemcpyAsync(d->tokens, d->host_stage, MAX_TOKENS * sizeof(int), cudaMemcpyHostToDevice, s);
        if (e == cudaSuccess) {
            e = cudaMemcpyAsync(d->pos, d->host_stage + MAX_TOKENS, sizeof(int), cudaMemcpyHostToDevice, s);
        }
        if (e != cudaSuccess) {
            return cuda_fail(e, "decoder inputs");
        }
        first_programmatic = false;
    }
    const float scale = (float)(1.0 / std::sqrt((double)d->head_dim));
    // caches are [sequence][layer][position][kv_dim]; a call works on one sequence, or on one token of each of the first T
    const size_t seq_elems = (size_t)d->layers * d->max_seq * kv_dim, seq_base = (size_t)d->cur_seq * seq_elems;
    const int pos_step = d->cur_batch ? 0 : 1;
    const int64_t tok_stride = d->cur_batch ? (int64_t)seq_elems : 0;
    (void)pos_step;
    (void)tok_stride;  // one token of one sequence here
    // the norm kernel's cluster: the most CTAs (up to 8) that still get whole super-blocks each
    int norm_ctas = 8;
    while (norm_ctas > 1 && dim % (256 * norm_ctas) != 0) {
        norm_ctas /= 2;
    }
    const size_t norm_smem = (size_t)(dim / norm_ctas) * sizeof(float);
    const dim3 norm_block((unsigned)(dim / norm_ctas / 4));
    const int splits_now = (max_keys + ATT_CHUNK - 1) / ATT_CHUNK;
    for (int l = 0; l < d->layers && rc == JQ_OK; l++) {
        const jq_weight* const* L = &d->lin[(size_t)l * 7];
        float* kc = d->k_cache + seq_base + (size_t)l * d->max_seq * kv_dim;
        float* vc = d->v_cache + seq_base + (size_t)l * d->max_seq * kv_dim;
        // attention block: x = embedding (first layer) or x += feed-forward output of the layer before; norm -> images
        CKL(launch_cluster_pdl(norm_image_kernel, norm_ctas, norm_block, norm_smem, s, l > 0 || first_programmatic, d->x, l == 0 ? nullptr : d->proj,
                       l == 0 ? d->embed : nullptr, d->tokens, d->vocab, d->norms + (size_t)(2 * l) * dim, d->eps, dim, images_for({L[0], L[1], L[2]}), (const uint32_t*)nullptr, 0),
            "norm_image_kernel");
        if (rc == JQ_OK) {
            rc = decoder_gemv_imaged3(d, L[0], d->q, L[1], d->k, L[2], d->v, s);
        }
        if (rc != JQ_OK) break;
        CKL(launch_pdl(attention_image_kernel<false>, dim3(d->heads, splits_now), dim3(ATTF_THREADS), 0, s, true, d->q, d->k, d->v, kc, vc, d->cos_t, d->sin_t, d->pos,
                       d->heads, d->kv_heads, d->splits, scale, d->att_part, d->counters, images_for({L[3]}), PeerImage{}),
            "attention_image_kernel");
        GEMV(L[3], d->proj, nullptr, nullptr, s);
        if (rc != JQ_OK) break;
        // feed-forward block
        CKL(launch_cluster_pdl(norm_image_kernel, norm_ctas, norm_block, norm_smem, s, true, d->x, d->proj, nullptr, d->tokens, d->vocab,
                       d->norms + (size_t)(2 * l + 1) * dim, d->eps, dim, images_for({L[4], L[5]}), (const uint32_t*)nullptr, 0),
            "norm_image_kernel");
        GEMV(L[4], d->gate, L[5], d->up, s);
        if (rc != JQ_OK) break;
        CKL(launch_pdl(swiglu_image_kernel<false>, dim3(d->hidden / 256), dim3(256), 0, s, true, d->gate, d->up, images_for({L[6]}), PeerImage{}, d->hidden / 256), "swiglu_image_kernel");
        GEMV(L[6], d->proj, nullptr, nullptr, s);
    }
    if (rc == JQ_OK) {
        CKL(launch_cluster_pdl(norm_image_kernel, norm_ctas, norm_block, norm_smem, s, true, d->x, d->proj, nullptr, d->tokens, d->vocab,
                       d->norms + (size_t)(2 * d->layers) * dim, d->eps, dim, images_for({d->output}), (const uint32_t*)nullptr, 0),
            "norm_image_kernel");
        GEMV(d->output, d->logits, nullptr, nullptr, s);
    }
    if (rc == JQ_OK) {
        CKL(launch_pdl(argmax_split_kernel, dim3(ARGMAX_CTAS), dim3(256), 0, s, true, d->logits, d->vocab, d->argmax_v, d->argmax_i,
                       d->counters + d->dim / 256 + 1, d->argmax),
            "argmax_split_kernel");
    }
    return rc;
}

static int enqueue_forward_sharded(jq_decoder* d, int T, int max_keys, const TokenArgs* ta, cudaStream_t s);

// Enqueues the forward of T tokens on s. Tokens and position come either from kernel arguments (ta != nullptr) or, for
// the captured single-token graph, from the pinned staging words through a host-to-device copy.
static int enqueue_forward(jq_decoder* d, int T, int max_keys, const TokenArgs* ta, cudaStream_t s) {
    if (d->world > 1) {
        return enqueue_forward_sharded(d, T, max_keys, ta, s);
    }
    if (T == 1 && fused_step_possible(d)) {
        return enqueue_forward_fused(d, max_keys, ta, s);
    }
    const int dim = d->dim, hd = d->head_dim;
    const int64_t kv_dim = (int64_t)d->kv_heads * hd;
    int rc = JQ_OK;
    auto LIN = [&](const jq_weight* w, const float* in, float* out_) {
        if (rc == JQ_OK) {
            rc = linear_device(w, in, T, nullptr, out_, s);
        }
    };
    cudaError_t pdl_err = cudaSuccess;  // what the latest programmatic launch returned
    auto LAUNCHED = [&](const char* name) {
        count_launch(1);
        if (rc == JQ_OK && pdl_err != cudaSuccess) {
            rc = cuda_fail(pdl_err, name);
        }
        pdl_err = cudaSuccess;
        if (rc == JQ_OK) {
            rc = check_launch(name);
        }
    };
    if (ta != nullptr) {
        set_tokens_kernel<<<1, 32, 0, s>>>(*ta, d->tokens, d->pos);
        LAUNCHED("set_tokens_kernel");
    } else {
        cudaError_t e = cudaMemcpyAsync(d->tokens, d->host_stage, MAX_TOKENS * sizeof(int), cudaMemcpyHostToDevice, s);
        if (e == cudaSuccess) {
            e = cudaMemcpyAsync(d->pos, d->host_stage + MAX_TOKENS, sizeof(int), cudaMemcpyHostToDevice, s);
        }
        if (e != cudaSuccess) {
            return cuda_fail(e, "decoder inputs");
        }
    }
    if (rc == JQ_OK) {
        if (rc == JQ_OK) pdl_err = launch_pdl(embed_kernel, dim3(T), dim3(256), 0, s, true, d->tokens, d->embed, d->x, dim, d->vocab);
        LAUNCHED("embed_kernel");
    }
    const float scale = (float)(1.0 / std::sqrt((double)hd));
    // caches are [sequence][layer][position][kv_dim]; a call works on one sequence, or on one token of each of the first T
    const size_t seq_elems = (size_t)d->layers * d->max_seq * kv_dim, seq_base = (size_t)d->cur_seq * seq_elems;
    const int pos_step = d->cur_batch ? 0 : 1;
    const int64_t tok_stride = d->cur_batch ? (int64_t)seq_elems : 0;
    for (int l = 0; l < d->layers && rc == JQ_OK; l++) {
        const jq_weight* const* L = &d->lin[(size_t)l * 7];
        float* kc = d->k_cache + seq_base + (size_t)l * d->max_seq * kv_dim;
        float* vc = d->v_cache + seq_base + (size_t)l * d->max_seq * kv_dim;
        // attention block; the residual add of the previous block's feed-forward output is fused into this norm
        if (rc == JQ_OK) pdl_err = launch_pdl(add_rmsnorm_kernel, dim3(T), dim3(NORM_THREADS), 0, s, true, d->x, l == 0 ? nullptr : d->proj, d->norms + (size_t)(2 * l) * dim, d->eps, d->xn, dim);
        LAUNCHED("add_rmsnorm_kernel");
        {
            float* const qkv[3] = {d->q, d->k, d->v};
            if (rc == JQ_OK) rc = linear_device_multi(L, 3, d->xn, T, qkv, s);
        }
        if (rc != JQ_OK) break;
        if (rc == JQ_OK) pdl_err = launch_pdl(rope_store_kernel, dim3(T, d->heads + 2 * d->kv_heads), dim3(hd / 2), 0, s, true, d->q, d->k, d->v, kc, vc, d->cos_t, d->sin_t, d->pos, d->heads, d->kv_heads, hd, pos_step, tok_stride);
        LAUNCHED("rope_store_kernel");
        // only the key chunks that can hold a position of this call are launched (all of them inside the captured graph)
        const int splits_now = (max_keys + ATT_CHUNK - 1) / ATT_CHUNK;
        if (rc == JQ_OK) pdl_err = launch_pdl(attention_partial_kernel, dim3(d->heads, splits_now, T), dim3(ATT_THREADS), 0, s, true, d->q, kc, vc, d->att_part, d->pos, d->heads, d->kv_heads, hd,
                                                                                 d->splits, scale, pos_step, tok_stride);
        LAUNCHED("attention_partial_kernel");
        if (rc == JQ_OK) pdl_err = launch_pdl(attention_combine_kernel, dim3(d->heads, T), dim3(hd < 128 ? hd : 128), 0, s, true, d->att_part, d->att, d->heads, hd, d->splits, splits_now);
        LAUNCHED("attention_combine_kernel");
        LIN(L[3], d->att, d->proj);
        if (rc != JQ_OK) break;
        // feed-forward block
        if (rc == JQ_OK) pdl_err = launch_pdl(add_rmsnorm_kernel, dim3(T), dim3(NORM_THREADS), 0, s, true, d->x, d->proj, d->norms + (size_t)(2 * l + 1) * dim, d->eps, d->xn, dim);
        LAUNCHED("add_rmsnorm_kernel");
        {
            float* const gu[2] = {d->gate, d->up};
            if (rc == JQ_OK) rc = linear_device_multi(L + 4, 2, d->xn, T, gu, s);
        }
        if (rc != JQ_OK) break;
        const int64_t cnt = (int64_t)T * d->hidden;
        if (rc == JQ_OK) pdl_err = launch_pdl(swiglu_kernel, dim3((unsigned)((cnt + 255) / 256)), dim3(256), 0, s, true, d->gate, d->up, d->act, cnt);
        LAUNCHED("swiglu_kernel");
        LIN(L[6], d->act, d->proj);
    }
    if (rc == JQ_OK) {
        if (rc == JQ_OK) pdl_err = launch_pdl(add_rmsnorm_kernel, dim3(T), dim3(NORM_THREADS), 0, s, true, d->x, d->proj, d->norms + (size_t)(2 * d->layers) * dim, d->eps, d->xn, dim);
        LAUNCHED("add_rmsnorm_kernel");
        LIN(d->output, d->xn, d->logits);
    }
    if (rc == JQ_OK) {
        if (rc == JQ_OK) pdl_err = launch_pdl(argmax_kernel, dim3(T), dim3(1024), 0, s, true, d->logits, d->argmax, d->vocab);
        LAUNCHED("argmax_kernel");
    }
    return rc;
}

// This rank's area `i` of gathered activations.
static float* shard_area(const jq_decoder* d, int i) {
    return reinterpret_cast<float*>(static_cast<uint8_t*>(d->peer_buf[d->rank]) + jq_peer_payload_offset() + d->area[i]);
}

// This rank's image area `i` (5 or 6), and the same area of every rank for the kernels that write an image into all of them.
static uint8_t* shard_image(const jq_decoder* d, int i) {
    return static_cast<uint8_t*>(d->peer_buf[d->rank]) + jq_peer_payload_offset() + d->area[i];
}

static PeerImage peer_image(const jq_decoder* d, int i, int blocks_per_rank) {
    PeerImage pi;
    memset(&pi, 0, sizeof(pi));
    for (int r = 0; r < d->world; r++) {
        pi.q4k[r] = static_cast<uint8_t*>(d->peer_buf[r]) + jq_peer_payload_offset() + d->area[i];
        pi.flags[r] = static_cast<uint32_t*>(d->peer_buf[r]);
    }
    pi.world = d->world;
    pi.rank = d->rank;
    pi.first_block = d->rank * blocks_per_rank;
    return pi;
}

// The forward of a rank of a row-sharded decoder. Every rank runs the replicated parts (embedding, norms, residual
// adds, argmax) on the whole vectors and its own rows of every linear: wq / wk / wv give this rank's heads, whose
// attention needs nothing from the other ranks; the attention output and the SwiGLU output are exchanged (each rank
// stores its columns into every rank's copy, jq_peer_gather) because wo and w2 read all of them; wo, w2 and the output
// projection store their rows into every rank's copy from the GEMV's epilogue (jq_linear_f32_peer). Five areas of the
// peer buffer are used in turn, so that no area is the target of two exchanges in a row. Per row the arithmetic is the
// unsharded decoder's (general kernels), so logits and tokens are bitwise those of one GPU.
static int enqueue_forward_sharded(jq_decoder* d, int T, int max_keys, const TokenArgs* ta, cudaStream_t s) {
    const int G = d->world, dim = d->dim, hd = d->head_dim;
    const int heads = d->heads / G, kv_heads = d->kv_heads / G;
    const int64_t kv_dim = (int64_t)kv_heads * hd, dim_l = dim / G, hidden_l = d->hidden / G, vocab_l = d->vocab / G;
    float *A = shard_area(d, 0), *B = shard_area(d, 1), *C = shard_area(d, 2), *D = shard_area(d, 3), *E = shard_area(d, 4);
    int rc = JQ_OK;
    // One token, Q4_K / Q6_K weights: the two norms write the activation images of the linears behind them (the fused
    // step's norm kernel), and wq|wk and w1|w3 are one launch each: 19 launches per layer instead of 26. The norm's
    // sum of squares is then added in another order than the general kernel's, so results agree with the unsharded
    // decoder within rounding instead of bit for bit; option decoder_fused = 0 keeps the general kernels.
    bool fused_in = T == 1 && g_opt_decoder_fused.load() != 0 && dim % 256 == 0 && dim <= 32768;
    for (size_t i = 0; i < d->lin.size() && fused_in; i++) {
        const int slot = (int)(i % 7);
        if (slot != 3 && slot != 6 && d->lin[i]->type != JQ_TYPE_Q4_K && d->lin[i]->type != JQ_TYPE_Q6_K) {
            fused_in = false;
        }
    }
    int norm_ctas = 8;
    while (norm_ctas > 1 && dim % (256 * norm_ctas) != 0) {
        norm_ctas /= 2;
    }
    const size_t norm_smem = (size_t)(dim / norm_ctas) * sizeof(float);
    const dim3 norm_block((unsigned)(dim / norm_ctas / 4));
    // A peer linear whose flag wait has not been enqueued as a kernel: the norm that reads its output waits itself.
    bool pending_wait = false;
    auto NORM_IMAGE = [&](const float* delta, const float* w, std::initializer_list<const jq_weight*> consumers) {
        count_launch(1);
        const cudaError_t e = launch_cluster_pdl(norm_image_kernel, norm_ctas, norm_block, norm_smem, s, true, d->x, delta, (const float*)nullptr,
                                                 (const int*)d->tokens, d->vocab, w, d->eps, dim, decoder_images_for(d, consumers),
                                                 pending_wait ? (const uint32_t*)d->peer_buf[d->rank] : (const uint32_t*)nullptr, G);
        pending_wait = false;
        if (rc == JQ_OK && e != cudaSuccess) {
            rc = cuda_fail(e, "norm_image_kernel");
        }
    };
    auto GEMV_IMAGED = [&](const jq_weight* w, float* y, const jq_weight* w2, float* y2) {
        if (rc == JQ_OK) {
            rc = decoder_gemv_imaged(d, w, y, w2, y2, s);
        }
    };
    auto LIN = [&](const jq_weight* w, const float* in, float* out_) {
        if (rc == JQ_OK) {
            rc = linear_device(w, in, T, nullptr, out_, s);
        }
    };
    auto PEER_LIN = [&](const jq_weight* w, const float* in, int64_t n_total, int64_t n_local, int area) {
        if (rc == JQ_OK) {
            rc = jq_linear_f32_peer(w, in, T, nullptr, n_total, d->rank * n_local, d->peer_buf, d->area[area], d->stage[area], d->rank, G, s);
        }
    };
    auto GATHER = [&](const float* slice, int64_t n_total, int64_t n_local, int area) {
        if (rc == JQ_OK) {
            rc = jq_peer_gather(slice, T, n_local, n_total, d->rank * n_local, d->peer_buf, d->area[area], d->stage[area], d->rank, G, s);
        }
    };
    auto LAUNCHED = [&](const char* name) {
        count_launch(1);
        if (rc == JQ_OK) {
            rc = check_launch(name);
        }
    };
    if (ta != nullptr) {
        set_tokens_kernel<<<1, 32, 0, s>>>(*ta, d->tokens, d->pos);
        LAUNCHED("set_tokens_kernel");
    } else {
        cudaError_t e = cudaMemcpyAsync(d->tokens, d->host_stage, MAX_TOKENS * sizeof(int), cudaMemcpyHostToDevice, s);
        if (e == cudaSuccess) {
            e = cudaMemcpyAsync(d->pos, d->host_stage + MAX_TOKENS, sizeof(int), cudaMemcpyHostToDevice, s);
        }
        if (e != cudaSuccess) {
            return cuda_fail(e, "decoder inputs");
        }
    }
    if (rc == JQ_OK) {
        embed_kernel<<<T, 256, 0, s>>>(d->tokens, d->embed, d->x, dim, d->vocab);
        LAUNCHED("embed_kernel");
    }
    const float scale = (float)(1.0 / std::sqrt((double)hd));
    // caches are [sequence][layer][position][kv_dim]; a call works on one sequence, or on one token of each of the first T
    const size_t seq_elems = (size_t)d->layers * d->max_seq * kv_dim, seq_base = (size_t)d->cur_seq * seq_elems;
    const int pos_step = d->cur_batch ? 0 : 1;
    const int64_t tok_stride = d->cur_batch ? (int64_t)seq_elems : 0;
    for (int l = 0; l < d->layers && rc == JQ_OK; l++) {
        const jq_weight* const* L = &d->lin[(size_t)l * 7];
        float* kc = d->k_cache + seq_base + (size_t)l * d->max_seq * kv_dim;
        float* vc = d->v_cache + seq_base + (size_t)l * d->max_seq * kv_dim;
        if (fused_in) {
            NORM_IMAGE(l == 0 ? nullptr : D, d->norms + (size_t)(2 * l) * dim, {L[0], L[1], L[2]});
            if (rc == JQ_OK) {
                rc = decoder_gemv_imaged3(d, L[0], d->q, L[1], d->k, L[2], d->v, s);
            }
        } else {
            add_rmsnorm_kernel<<<T, NORM_THREADS, 0, s>>>(d->x, l == 0 ? nullptr : D, d->norms + (size_t)(2 * l) * dim, d->eps, d->xn, dim);
            LAUNCHED("add_rmsnorm_kernel");
            float* const qkv[3] = {d->q, d->k, d->v};
            if (rc == JQ_OK) rc = linear_device_multi(L, 3, d->xn, T, qkv, s);
        }
        if (rc != JQ_OK) break;
        const int splits_now = (max_keys + ATT_CHUNK - 1) / ATT_CHUNK;
        if (fused_in && hd == 128 && heads % 2 == 0 && L[3]->type == JQ_TYPE_Q4_K) {
            // the fused attention kernel on this rank's heads; its merging CTAs store their super-block of wo's activation
            // image into every rank's image area, the last CTA raises the flags; wo then reads the image all ranks wrote
            count_launch(1);
            const cudaError_t e = launch_pdl(attention_image_kernel<true>, dim3(heads, splits_now), dim3(ATTF_THREADS), 0, s, true, (const float*)d->q,
                                             (const float*)d->k, (const float*)d->v, kc, vc, (const float*)d->cos_t, (const float*)d->sin_t,
                                             (const int*)d->pos, heads, kv_heads, d->splits, scale, d->att_part, d->counters,
                                             Images{shard_image(d, 5), nullptr}, peer_image(d, 5, (int)(dim_l / 256)));
            if (rc == JQ_OK && e != cudaSuccess) {
                rc = cuda_fail(e, "attention_image_kernel");
            }
            // wo waits for the image's counters itself; its outputs travel as marked words that its own threads collect, so
            // the norm behind it finds the vector complete
            if (rc == JQ_OK) rc = peer_linear_q4k_imaged(L[3], shard_image(d, 5), dim, d->rank * dim_l, d->peer_buf, d->area[1], d->stage[1], d->rank, G, s, true, false);
        } else {
            rope_store_kernel<<<dim3(T, heads + 2 * kv_heads), hd / 2, 0, s>>>(d->q, d->k, d->v, kc, vc, d->cos_t, d->sin_t, d->pos, heads, kv_heads, hd, pos_step,
                                                                               tok_stride);
            LAUNCHED("rope_store_kernel");
            attention_partial_kernel<<<dim3(heads, splits_now, T), ATT_THREADS, 0, s>>>(d->q, kc, vc, d->att_part, d->pos, heads, kv_heads, hd, d->splits,
                                                                                  scale, pos_step, tok_stride);
            LAUNCHED("attention_partial_kernel");
            attention_combine_kernel<<<dim3(heads, T), hd < 128 ? hd : 128, 0, s>>>(d->att_part, d->att, heads, hd, d->splits, splits_now);
            LAUNCHED("attention_combine_kernel");
            GATHER(d->att, dim, dim_l, 0);
            PEER_LIN(L[3], A, dim, dim_l, 1);
        }
        if (rc != JQ_OK) break;
        if (fused_in) {
            NORM_IMAGE(B, d->norms + (size_t)(2 * l + 1) * dim, {L[4], L[5]});
            GEMV_IMAGED(L[4], d->gate, L[5], d->up);
        } else {
            add_rmsnorm_kernel<<<T, NORM_THREADS, 0, s>>>(d->x, B, d->norms + (size_t)(2 * l + 1) * dim, d->eps, d->xn, dim);
            LAUNCHED("add_rmsnorm_kernel");
            float* const gu[2] = {d->gate, d->up};
            if (rc == JQ_OK) rc = linear_device_multi(L + 4, 2, d->xn, T, gu, s);
        }
        if (rc != JQ_OK) break;
        if (fused_in && hidden_l % 256 == 0 && L[6]->type == JQ_TYPE_Q4_K) {
            count_launch(1);
            const int blocks = (int)(hidden_l / 256);
            const cudaError_t e = launch_pdl(swiglu_image_kernel<true>, dim3((unsigned)((blocks + SWIGLU_PEER_BLOCKS - 1) / SWIGLU_PEER_BLOCKS)), dim3(256), 0, s, true,
                                             (const float*)d->gate, (const float*)d->up, Images{shard_image(d, 6), nullptr}, peer_image(d, 6, blocks), blocks);
            if (rc == JQ_OK && e != cudaSuccess) {
                rc = cuda_fail(e, "swiglu_image_kernel");
            }
            if (rc == JQ_OK) rc = peer_linear_q4k_imaged(L[6], shard_image(d, 6), dim, d->rank * dim_l, d->peer_buf, d->area[3], d->stage[3], d->rank, G, s, true, false);
        } else {
            const int64_t cnt = (int64_t)T * hidden_l;
            swiglu_kernel<<<(unsigned)((cnt + 255) / 256), 256, 0, s>>>(d->gate, d->up, d->act, cnt);
            LAUNCHED("swiglu_kernel");
            GATHER(d->act, d->hidden, hidden_l, 2);
            PEER_LIN(L[6], C, dim, dim_l, 3);
        }
    }
    if (rc == JQ_OK) {
        add_rmsnorm_kernel<<<T, NORM_THREADS, 0, s>>>(d->x, D, d->norms + (size_t)(2 * d->layers) * dim, d->eps, d->xn, dim);
        LAUNCHED("add_rmsnorm_kernel");
        PEER_LIN(d->output, d->xn, d->vocab, vocab_l, 4);
    }
    if (rc == JQ_OK) {
        argmax_kernel<<<T, 1024, 0, s>>>(E, d->argmax, d->vocab);
        LAUNCHED("argmax_kernel");
    }
    return rc;
}

// Runs n_tokens consecutive tokens of sequence `seq` at positions pos0 .. pos0 + n_tokens - 1 (batch false), or one token of
// each of the sequences 0 .. n_tokens - 1, all at position pos0 (batch true), and appends their keys and values to the
// caches. logits_host (may be NULL) receives [n_tokens, vocab], next_host (may be NULL) the greedy next token after each
// of them. Synchronises `stream` before returning when either output is requested.
// A call that asks for the next token of a single token, or of a batch, is a decode step: the second step of the same
// kind (same sequence, or same batch size) is captured into a CUDA graph (all launches of the step read tokens and
// position from memory), later ones replay the graph.
static int decoder_forward(jq_decoder* d, int seq, bool batch, const int32_t* tokens_host, int n_tokens, int pos0, float* logits_host, int32_t* next_host,
                           void* stream) {
    int rc = check_decoder(d, "jq_decoder_forward");
    if (rc != JQ_OK) {
        return rc;
    }
    if (tokens_host == nullptr || n_tokens < 1 || n_tokens > MAX_TOKENS || pos0 < 0 || pos0 + (batch ? 1 : n_tokens) > d->max_seq) {
        return fail(JQ_ERR_INVALID, "jq_decoder_forward: %d tokens at position %d (at most %d per call, %d positions)", n_tokens, pos0, MAX_TOKENS,
                    d->max_seq);
    }
    if (seq < 0 || seq >= d->sequences || (batch && n_tokens > d->sequences)) {
        return fail(JQ_ERR_INVALID, "jq_decoder_forward: sequence %d, batch of %d: the decoder holds %d sequence(s) (jq_decoder_set_sequences)", seq,
                    batch ? n_tokens : 1, d->sequences);
    }
    if (d->output == nullptr) {
        return fail(JQ_ERR_INVALID, "jq_decoder_forward: the output projection is not set");
    }
    for (size_t i = 0; i < d->lin.size(); i++) {
        if (d->lin[i] == nullptr) {
            return fail(JQ_ERR_INVALID, "jq_decoder_forward: layer %d linear %d is not set", (int)(i / 7), (int)(i % 7));
        }
    }
    int prev = -1;
    cudaGetDevice(&prev);
    if (prev != d->device) {
        JQ_CUDA(cudaSetDevice(d->device));
    }
    // all state of a decoder is private to it and its inputs come from the host, so its own stream is as good as any
    cudaStream_t s = stream != nullptr ? (cudaStream_t)stream : d->own_stream;
    const int T = n_tokens;
    const bool decode_step = (T == 1 || batch) && next_host != nullptr && g_opt_decoder_graph.load() != 0;
    d->cur_seq = batch ? 0 : seq;
    d->cur_batch = batch && T > 1;  // a batch of one is the single-token step of sequence 0
    if (decode_step && (d->graph_T != T || d->graph_seq != (d->cur_batch ? -1 : d->cur_seq))) {
        // another kind of step than the one counted (and perhaps captured) so far
        if (d->graph != nullptr) {
            cudaGraphExecDestroy(d->graph);
            d->graph = nullptr;
        }
        d->warm_calls = 0;
        d->graph_T = T;
        d->graph_seq = d->cur_batch ? -1 : d->cur_seq;
    }
    auto CK = [&](cudaError_t e, const char* what) {
        if (rc == JQ_OK && e != cudaSuccess) {
            rc = cuda_fail(e, what);
        }
    };
    if (decode_step && d->warm_calls >= 1) {
        // the staging words are free again: every decode step ends with a wait for the stream
        for (int i = 0; i < T; i++) {
            d->host_stage[i] = tokens_host[i];
        }
        d->host_stage[MAX_TOKENS] = pos0;
        if (d->graph == nullptr) {
            cudaGraph_t g = nullptr;
            CK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
            if (rc == JQ_OK) {
                rc = enqueue_forward(d, T, d->max_seq, nullptr, s);
                cudaError_t e = cudaMemcpyAsync(d->host_stage + MAX_TOKENS + 1, d->argmax, T * sizeof(int), cudaMemcpyDeviceToHost, s);
                cudaError_t e2 = cudaStreamEndCapture(s, &g);
                CK(e, "argmax copy");
                CK(e2, "cudaStreamEndCapture");
            }
            if (rc == JQ_OK) {
                CK(cudaGraphInstantiate(&d->graph, g, 0), "cudaGraphInstantiate");
            }
            if (g != nullptr) {
                cudaGraphDestroy(g);
            }
        }
        if (rc == JQ_OK) {
            CK(cudaGraphLaunch(d->graph, s), "cudaGraphLaunch");
        }
    } else {
        TokenArgs ta;
        for (int i = 0; i < MAX_TOKENS; i++) {
            ta.tokens[i] = i < T ? tokens_host[i] : 0;
        }
        ta.pos0 = pos0;
        rc = enqueue_forward(d, T, pos0 + (batch ? 1 : T), &ta, s);
        if (rc == JQ_OK && next_host != nullptr) {
            CK(cudaMemcpyAsync(d->host_stage + MAX_TOKENS + 1, d->argmax, T * sizeof(int), cudaMemcpyDeviceToHost, s), "argmax");
        }
        if (decode_step) {
            d->warm_calls++;
        }
    }
    if (rc == JQ_OK && (logits_host != nullptr || next_host != nullptr)) {
        if (logits_host != nullptr) {
            const float* src = d->world > 1 ? shard_area(d, 4) : d->logits;
            CK(cudaMemcpyAsync(logits_host, src, (size_t)T * d->vocab * sizeof(float), cudaMemcpyDeviceToHost, s), "logits");
        }
        CK(cudaStreamSynchronize(s), "jq_decoder_forward");
        if (rc == JQ_OK && d->world > 1) {
            int status = 0, part = 0;
            rc = peer_status(&status);
            if (rc == JQ_OK) rc = gemv_peer_status(&part);
            status = status != 0 ? status : part;
            if (rc == JQ_OK) rc = decoder_peer_status(&part);
            status = status != 0 ? status : part;
            if (rc == JQ_OK && status != 0) {
                rc = fail(JQ_ERR_TIMEOUT, "jq_decoder_forward: the slice of rank %d did not arrive (bounded wait gave up)", status - 32);
            }
        }
        if (rc == JQ_OK && next_host != nullptr) {
            for (int i = 0; i < T; i++) {
                next_host[i] = d->host_stage[MAX_TOKENS + 1 + i];
            }
        }
    }
    if (prev >= 0 && prev != d->device) {
        cudaSetDevice(prev);
    }
    return rc;
}

JQ_API int jq_decoder_forward(jq_decoder* d, const int32_t* tokens_host, int n_tokens, int pos0, float* logits_host, int32_t* next_host, void* stream) {
    return decoder_forward(d, 0, false, tokens_host, n_tokens, pos0, logits_host, next_host, stream);
}

JQ_API int jq_decoder_forward_seq(jq_decoder* d, int seq, const int32_t* tokens_host, int n_tokens, int pos0, float* logits_host, int32_t* next_host,
                                  void* stream) {
    return decoder_forward(d, seq, false, tokens_host, n_tokens, pos0, logits_host, next_host, stream);
}

JQ_API int jq_decoder_forward_batch(jq_decoder* d, const int32_t* tokens_host, int n_seqs, int pos, float* logits_host, int32_t* next_host, void* stream) {
    return decoder_forward(d, 0, true, tokens_host, n_seqs, pos, logits_host, next_host, stream);
}

// ---- the prompt path ---------------------------------------------------------------------------------------------------------
// A long run of consecutive tokens in one pass over the weights: the general path's operators on T rows, with every linear
// on the tensor-core prefill kernel (its input rounded to bfloat16, FP32 accumulation) and the attention of all T queries by
// attention_prompt_kernel. Only the last token's logits are computed.
constexpr int PROMPT_MAX_TOKENS = 4096;

static int ensure_prompt_workspace(jq_decoder* d, int rows) {
    if (rows <= d->prompt_rows) {
        return JQ_OK;
    }
    cudaFree(d->prompt_buf);
    cudaFree(d->prompt_bf16);
    cudaFree(d->prompt_tokens);
    d->prompt_buf = nullptr;
    d->prompt_bf16 = nullptr;
    d->prompt_tokens = nullptr;
    d->prompt_rows = 0;
    const size_t kv_dim = (size_t)d->kv_heads * d->head_dim;
    const size_t per_row = (size_t)5 * d->dim + 2 * kv_dim + 3 * (size_t)d->hidden;  // x, xn, q, att, proj; k, v; gate, up, act
    const size_t widest = (size_t)(d->dim > d->hidden ? d->dim : d->hidden);
    cudaError_t e = cudaMalloc(&d->prompt_buf, (size_t)rows * per_row * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&d->prompt_bf16, (size_t)rows * widest * sizeof(uint16_t));
    if (e == cudaSuccess) e = cudaMalloc(&d->prompt_tokens, (size_t)rows * sizeof(int));
    if (e != cudaSuccess) {
        cudaFree(d->prompt_buf);
        cudaFree(d->prompt_bf16);
        cudaFree(d->prompt_tokens);
        d->prompt_buf = nullptr;
        d->prompt_bf16 = nullptr;
        d->prompt_tokens = nullptr;
        return e == cudaErrorMemoryAllocation ? fail(JQ_ERR_OOM, "jq_decoder_prompt: workspace for %d tokens", rows) : cuda_fail(e, "jq_decoder_prompt workspace");
    }
    d->prompt_rows = rows;
    return JQ_OK;
}

JQ_API int jq_decoder_prompt(jq_decoder* d, int seq, const int32_t* tokens_host, int n_tokens, int pos0, float* logits_host, int32_t* next_host,
                             void* stream) {
    int rc = check_decoder(d, "jq_decoder_prompt");
    if (rc != JQ_OK) {
        return rc;
    }
    if (tokens_host == nullptr || n_tokens < 1 || n_tokens > PROMPT_MAX_TOKENS || pos0 < 0 || pos0 + n_tokens > d->max_seq) {
        return fail(JQ_ERR_INVALID, "jq_decoder_prompt: %d tokens at position %d (at most %d per call, %d positions)", n_tokens, pos0, PROMPT_MAX_TOKENS,
                    d->max_seq);
    }
    if (seq < 0 || seq >= d->sequences) {
        return fail(JQ_ERR_INVALID, "jq_decoder_prompt: sequence %d of %d", seq, d->sequences);
    }
    if (d->world > 1) {
        return fail(JQ_ERR_UNSUPPORTED, "jq_decoder_prompt: the row-sharded decoder takes its prompt through jq_decoder_forward");
    }
    if (d->head_dim != 64 && d->head_dim != 128) {
        return fail(JQ_ERR_UNSUPPORTED, "jq_decoder_prompt: head size %d (64 or 128)", d->head_dim);
    }
    if (d->output == nullptr) {
        return fail(JQ_ERR_INVALID, "jq_decoder_prompt: the output projection is not set");
    }
    for (size_t i = 0; i < d->lin.size(); i++) {
        if (d->lin[i] == nullptr) {
            return fail(JQ_ERR_INVALID, "jq_decoder_prompt: layer %d linear %d is not set", (int)(i / 7), (int)(i % 7));
        }
        if (!prefill_supported(View{d->lin[i]->q, d->lin[i]->aux, d->lin[i]->n, d->lin[i]->k, d->lin[i]->type})) {
            return fail(JQ_ERR_UNSUPPORTED, "jq_decoder_prompt: layer %d linear %d has a format or shape the tensor-core kernel does not take", (int)(i / 7),
                        (int)(i % 7));
        }
    }
    int prev = -1;
    cudaGetDevice(&prev);
    if (prev != d->device) {
        JQ_CUDA(cudaSetDevice(d->device));
    }
    cudaStream_t s = stream != nullptr ? (cudaStream_t)stream : d->own_stream;
    const int T = n_tokens, dim = d->dim, hd = d->head_dim, hidden = d->hidden;
    const int64_t kv_dim = (int64_t)d->kv_heads * hd;
    rc = ensure_prompt_workspace(d, T);
    auto CK = [&](cudaError_t e, const char* what) {
        if (rc == JQ_OK && e != cudaSuccess) {
            rc = cuda_fail(e, what);
        }
    };
    auto LAUNCHED = [&](const char* name) {
        count_launch(1);
        if (rc == JQ_OK) {
            rc = check_launch(name);
        }
    };
    if (rc == JQ_OK) {
        float* p = d->prompt_buf;
        float* x = p; p += (size_t)T * dim;
        float* xn = p; p += (size_t)T * dim;
        float* q = p; p += (size_t)T * dim;
        float* att = p; p += (size_t)T * dim;
        float* proj = p; p += (size_t)T * dim;
        float* k = p; p += (size_t)T * kv_dim;
        float* v = p; p += (size_t)T * kv_dim;
        float* gate = p; p += (size_t)T * hidden;
        float* up = p; p += (size_t)T * hidden;
        float* act = p;
        uint16_t* xb = d->prompt_bf16;
        // a linear on all T rows: the input rounded to bfloat16 once (`fresh`), then the tensor-core kernel
        auto LIN = [&](const jq_weight* w, const float* in, float* out_, bool fresh) {
            if (rc == JQ_OK && fresh) {
                rc = launch_f32_to_bf16(in, xb, (int64_t)T * w->k, s);
            }
            if (rc == JQ_OK) {
                rc = launch_prefill_bf16(View{w->q, w->aux, w->n, w->k, w->type}, xb, T, nullptr, out_, s);
            }
        };
        // the copy out of pageable host memory is staged before the call returns: the caller's buffer is free afterwards
        CK(cudaMemcpyAsync(d->prompt_tokens, tokens_host, (size_t)T * sizeof(int), cudaMemcpyHostToDevice, s), "prompt tokens");
        if (rc == JQ_OK) {
            set_pos_kernel<<<1, 1, 0, s>>>(pos0, d->pos);
            LAUNCHED("set_pos_kernel");
        }
        if (rc == JQ_OK) {
            embed_kernel<<<T, 256, 0, s>>>(d->prompt_tokens, d->embed, x, dim, d->vocab);
            LAUNCHED("embed_kernel");
        }
        const float scale = (float)(1.0 / std::sqrt((double)hd));
        const size_t seq_elems = (size_t)d->layers * d->max_seq * kv_dim, seq_base = (size_t)seq * seq_elems;
        static std::atomic<uint64_t> configured{0};  // the opt-in for large dynamic shared memory is per device
        if (rc == JQ_OK && (configured.load() >> (d->device & 63) & 1) == 0) {
            CK(cudaFuncSetAttribute(attention_prompt_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)prompt_attention_smem<64>()), "attention_prompt_kernel");
            CK(cudaFuncSetAttribute(attention_prompt_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)prompt_attention_smem<128>()), "attention_prompt_kernel");
            configured.fetch_or((uint64_t)1 << (d->device & 63));
        }
        for (int l = 0; l < d->layers && rc == JQ_OK; l++) {
            const jq_weight* const* L = &d->lin[(size_t)l * 7];
            float* kc = d->k_cache + seq_base + (size_t)l * d->max_seq * kv_dim;
            float* vc = d->v_cache + seq_base + (size_t)l * d->max_seq * kv_dim;
            add_rmsnorm_kernel<<<T, NORM_THREADS, 0, s>>>(x, l == 0 ? nullptr : proj, d->norms + (size_t)(2 * l) * dim, d->eps, xn, dim);
            LAUNCHED("add_rmsnorm_kernel");
            LIN(L[0], xn, q, true);
            LIN(L[1], xn, k, false);
            LIN(L[2], xn, v, false);
            if (rc != JQ_OK) break;
            rope_store_kernel<<<dim3(T, d->heads + 2 * d->kv_heads), hd / 2, 0, s>>>(q, k, v, kc, vc, d->cos_t, d->sin_t, d->pos, d->heads, d->kv_heads, hd, 1, 0);
            LAUNCHED("rope_store_kernel");
            const dim3 agrid((unsigned)d->heads, (unsigned)((T + PA_Q - 1) / PA_Q));
            if (hd == 128) {
                attention_prompt_kernel<128><<<agrid, PA_THREADS, prompt_attention_smem<128>(), s>>>(q, kc, vc, att, d->pos, d->heads, d->kv_heads, T, scale);
            } else {
                attention_prompt_kernel<64><<<agrid, PA_THREADS, prompt_attention_smem<64>(), s>>>(q, kc, vc, att, d->pos, d->heads, d->kv_heads, T, scale);
            }
            LAUNCHED("attention_prompt_kernel");
            LIN(L[3], att, proj, true);
            if (rc != JQ_OK) break;
            add_rmsnorm_kernel<<<T, NORM_THREADS, 0, s>>>(x, proj, d->norms + (size_t)(2 * l + 1) * dim, d->eps, xn, dim);
            LAUNCHED("add_rmsnorm_kernel");
            LIN(L[4], xn, gate, true);
            LIN(L[5], xn, up, false);
            if (rc != JQ_OK) break;
            const int64_t cnt = (int64_t)T * hidden;
            swiglu_kernel<<<(unsigned)((cnt + 255) / 256), 256, 0, s>>>(gate, up, act, cnt);
            LAUNCHED("swiglu_kernel");
            LIN(L[6], act, proj, true);
        }
        if (rc == JQ_OK) {
            // the last token alone goes on: final residual add and norm, output projection (FP32 path), first index of the maximum
            const size_t last = (size_t)(T - 1) * dim;
            add_rmsnorm_kernel<<<1, NORM_THREADS, 0, s>>>(x + last, proj + last, d->norms + (size_t)(2 * d->layers) * dim, d->eps, d->xn, dim);
            LAUNCHED("add_rmsnorm_kernel");
            if (rc == JQ_OK) rc = linear_device(d->output, d->xn, 1, nullptr, d->logits, s);
        }
        if (rc == JQ_OK) {
            argmax_kernel<<<1, 1024, 0, s>>>(d->logits, d->argmax, d->vocab);
            LAUNCHED("argmax_kernel");
        }
    }
    if (rc == JQ_OK && (logits_host != nullptr || next_host != nullptr)) {
        if (logits_host != nullptr) {
            CK(cudaMemcpyAsync(logits_host, d->logits, (size_t)d->vocab * sizeof(float), cudaMemcpyDeviceToHost, s), "logits");
        }
        if (next_host != nullptr) {
            CK(cudaMemcpyAsync(d->host_stage + MAX_TOKENS + 1, d->argmax, sizeof(int), cudaMemcpyDeviceToHost, s), "argmax");
        }
        CK(cudaStreamSynchronize(s), "jq_decoder_prompt");
        if (rc == JQ_OK) {
            int status = 0;
            rc = prefill_status(&status);
            if (rc == JQ_OK && status != 0) {
                rc = fail(JQ_ERR_TIMEOUT, "jq_decoder_prompt: a bounded wait of the tensor-core kernel gave up (code %d)", status);
            }
        }
        if (rc == JQ_OK && next_host != nullptr) {
            next_host[0] = d->host_stage[MAX_TOKENS + 1];
        }
    }
    if (prev >= 0 && prev != d->device) {
        cudaSetDevice(prev);
    }
    return rc;
}

// Key/value caches for `sequences` (1..16) independent sequences; what the caches held is lost.
JQ_API int jq_decoder_set_sequences(jq_decoder* d, int sequences) {
    int rc = check_decoder(d, "jq_decoder_set_sequences");
    if (rc != JQ_OK) {
        return rc;
    }
    if (sequences < 1 || sequences > MAX_TOKENS) {
        return fail(JQ_ERR_INVALID, "jq_decoder_set_sequences: %d sequences (1 to %d)", sequences, MAX_TOKENS);
    }
    int prev = -1;
    cudaGetDevice(&prev);
    JQ_CUDA(cudaSetDevice(d->device));
    JQ_CUDA(cudaDeviceSynchronize());
    if (d->graph != nullptr) {
        cudaGraphExecDestroy(d->graph);  // the captured step holds the old cache addresses
        d->graph = nullptr;
    }
    d->warm_calls = 0;
    d->graph_T = 0;
    const size_t elems = (size_t)sequences * d->layers * d->max_seq * d->kv_heads * d->head_dim;
    float *kc = nullptr, *vc = nullptr;
    cudaError_t e = cudaMalloc(&kc, elems * sizeof(float));
    if (e == cudaSuccess) {
        e = cudaMalloc(&vc, elems * sizeof(float));
    }
    if (e != cudaSuccess) {
        cudaFree(kc);
        if (prev >= 0) cudaSetDevice(prev);
        return cuda_fail(e, "jq_decoder_set_sequences");
    }
    cudaFree(d->k_cache);
    cudaFree(d->v_cache);
    d->k_cache = kc;
    d->v_cache = vc;
    d->sequences = sequences;
    if (prev >= 0) cudaSetDevice(prev);
    return JQ_OK;
}

}  // extern "C"
