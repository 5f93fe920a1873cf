// The C ABI (include/jitnn_b200.h): argument validation, weight upload, dispatch, host staging.
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "jq_common.cuh"

namespace jq {

std::atomic<int64_t> g_launches{0};
static thread_local std::string t_error;

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    t_error = buf;
    return code;
}

int cuda_fail(cudaError_t e, const char* what) {
    int code = e == cudaErrorMemoryAllocation ? JQ_ERR_OOM : JQ_ERR_CUDA;
    return fail(code, "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
}

int check_launch(const char* kernel) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        return fail(JQ_ERR_CUDA, "launch of %s failed: %s", kernel, cudaGetErrorString(e));
    }
    return JQ_OK;
}

// Makes `device` current for the scope and restores the caller's device afterwards.
struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int device) {
        if (cudaGetDevice(&prev) != cudaSuccess) {
            prev = -1;
        }
        if (prev != device) {
            ok = cudaSetDevice(device) == cudaSuccess;
        } else {
            prev = -1;
        }
    }
    ~DeviceGuard() {
        if (prev >= 0) {
            cudaSetDevice(prev);
        }
    }
};

// Per-thread, per-device staging for calls whose data lives on the host: a device buffer that grows on
// demand and a private stream, so that concurrent callers never share scratch.
struct Staging {
    uint8_t* dev = nullptr;
    size_t bytes = 0;
    cudaStream_t stream = nullptr;
};

static thread_local std::vector<Staging> t_staging;

static int staging_for(int device, size_t bytes, Staging** out) {
    if ((size_t)device >= t_staging.size()) {
        t_staging.resize(device + 1);
    }
    Staging& st = t_staging[device];
    if (st.stream == nullptr) {
        JQ_CUDA(cudaStreamCreateWithFlags(&st.stream, cudaStreamNonBlocking));
    }
    if (st.bytes < bytes) {
        if (st.dev != nullptr) {
            JQ_CUDA(cudaStreamSynchronize(st.stream));
            JQ_CUDA(cudaFree(st.dev));
            st.dev = nullptr;
            st.bytes = 0;
        }
        size_t want = bytes + bytes / 4 + 4096;
        JQ_CUDA(cudaMalloc(&st.dev, want));
        st.bytes = want;
    }
    *out = &st;
    return JQ_OK;
}

// ---- per (device, stream) scratch ------------------------------------------------------------------
// A buffer that has been handed out may be baked into a captured CUDA graph (the decoder's step, a caller's own capture
// of jq_linear_*), so it is never freed or moved: a request that outgrows it gets a new allocation and the old one stays
// where it is until the process ends.
struct Scratch {
    int device;
    cudaStream_t stream;
    int slot;
    uint8_t* buf;
    size_t bytes;
};
static std::mutex g_scratch_mu;
static std::vector<Scratch> g_scratch;
static std::vector<uint8_t*> g_scratch_retired;

int scratch_for(cudaStream_t s, size_t bytes, uint8_t** out) { return scratch_for_slot(s, 0, bytes, out); }

static int scratch_impl(cudaStream_t s, int slot, size_t bytes, bool zeroed, uint8_t** out) {
    int dev = 0;
    JQ_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    Scratch* hit = nullptr;
    for (Scratch& sc : g_scratch) {
        if (sc.device == dev && sc.stream == s && sc.slot == slot) {
            hit = &sc;
            break;
        }
    }
    if (hit == nullptr) {
        g_scratch.push_back(Scratch{dev, s, slot, nullptr, 0});
        hit = &g_scratch.back();
    }
    if (hit->bytes < bytes) {
        const size_t floor_bytes = zeroed ? ((size_t)64 << 10) : ((size_t)1 << 20);
        const size_t want = bytes < floor_bytes ? floor_bytes : bytes + bytes / 2;
        uint8_t* fresh = nullptr;
        JQ_CUDA(cudaMalloc(&fresh, want));
        if (zeroed) {
            JQ_CUDA(cudaMemsetAsync(fresh, 0, want, s));  // in stream order before the first kernel that uses it
        }
        if (hit->buf != nullptr) {
            g_scratch_retired.push_back(hit->buf);
        }
        hit->buf = fresh;
        hit->bytes = want;
    }
    *out = hit->buf;
    return JQ_OK;
}

int scratch_for_slot(cudaStream_t s, int slot, size_t bytes, uint8_t** out) { return scratch_impl(s, slot, bytes, false, out); }

// The same, for words that kernels use as counters and leave at zero: a new allocation starts out zeroed.
int scratch_zeroed_for_slot(cudaStream_t s, int slot, size_t bytes, uint8_t** out) { return scratch_impl(s, slot, bytes, true, out); }

static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

// The device-side address of a host buffer that kernels may use directly: page-locked, 16-byte aligned, at most `limit`
// bytes. nullptr otherwise (pageable memory, or a driver that cannot say).
static const float* pinned_device_pointer(const void* host, size_t bytes, size_t limit) {
    if (bytes > limit || ((uintptr_t)host & 15) != 0) {
        return nullptr;
    }
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, host) != cudaSuccess) {
        cudaGetLastError();  // an unregistered pointer is not an error of this call
        return nullptr;
    }
    return attr.type == cudaMemoryTypeHost ? static_cast<const float*>(attr.devicePointer) : nullptr;
}

static int check_weight(const jq_weight* w, const char* who) {
    if (w == nullptr || w->magic != JQ_WEIGHT_MAGIC) {
        return fail(JQ_ERR_INVALID, "%s: not a live weight handle", who);
    }
    return JQ_OK;
}

static View view_of(const jq_weight* w) { return View{w->q, w->aux, w->n, w->k, w->type}; }

static const char* type_name(int type) {
    switch (type) {
        case JQ_TYPE_Q8_0: return "Q8_0";
        case JQ_TYPE_Q4_0: return "Q4_0";
        case JQ_TYPE_Q4_1: return "Q4_1";
        case JQ_TYPE_Q4_K: return "Q4_K";
        case JQ_TYPE_Q5_K: return "Q5_K";
        case JQ_TYPE_Q6_K: return "Q6_K";
        case JQ_TYPE_Q5_0: return "Q5_0";
        case JQ_TYPE_Q5_1: return "Q5_1";
        case JQ_TYPE_Q2_K: return "Q2_K";
        case JQ_TYPE_Q3_K: return "Q3_K";
        default: return "?";
    }
}

// ---- options ------------------------------------------------------------------------------------
static std::atomic<int64_t> g_prefill_min_rows{0};
std::atomic<int64_t> g_opt_gemv_generic{0};
std::atomic<int64_t> g_opt_decoder_graph{1};
std::atomic<int64_t> g_opt_decoder_fused{1};

// ---- linear on device pointers --------------------------------------------------------------------
int linear_device(const jq_weight* w, const float* x, int64_t m, const float* bias, float* y, cudaStream_t s, bool x_remote) {
    View v = view_of(w);
    const int64_t min_rows = g_prefill_min_rows.load();
    if (min_rows > 0 && m >= min_rows && prefill_supported(v)) {
        // the caller opted in to bfloat16 operand precision for large row counts: round x, then the tensor-core kernel
        uint8_t* xb = nullptr;
        int rc = scratch_for(s, (size_t)m * w->k * 2, &xb);
        if (rc == JQ_OK) {
            rc = launch_f32_to_bf16(x, (uint16_t*)xb, m * w->k, s);
        }
        if (rc == JQ_OK) {
            rc = launch_prefill_bf16(v, (const uint16_t*)xb, m, bias, y, s);
        }
        return rc;
    }
    // The integer tensor-core kernel of Q4_K and Q5_K takes up to 8 activation rows per pass (the tcgen05 one, where it is chosen, 16),
    // Q6_K's 4, the generic kernel 16.
    const bool tc = g_opt_gemv_generic.load() == 0;
    // Q8_0, Q4_0 and Q4_1 (k a multiple of 256) go two rows at a time through their tensor-core kernel: re-reading the weights
    // (mostly from L2) per pair of rows is far cheaper than the generic kernel's arithmetic.
    const bool blk32 = tc && gemv_blk32_i8_scratch_bytes(w->type, w->k, 2) > 0;
    const int64_t group = (tc && (w->type == JQ_TYPE_Q4_K || w->type == JQ_TYPE_Q5_K)) ? 8 : ((tc && w->type == JQ_TYPE_Q6_K) ? 4 : (blk32 ? 2 : 16));
    for (int64_t m0 = 0; m0 < m;) {
        const int left = (int)(m - m0 < 16 ? m - m0 : 16);
        const int rows = gemv_umma_takes(w->type, w->k, left, w->n) ? left : (int)(left < group ? left : group);
        int rc = launch_gemv(v, x + m0 * w->k, rows, bias, y + m0 * w->n, s, x_remote);
        if (rc != JQ_OK) {
            return rc;
        }
        m0 += rows;
    }
    return JQ_OK;
}

// Up to three linears on the same x [m, k] (the decoder's wq / wk / wv, and w1 / w3). Weights of one K-quant type and k whose
// rows together are a shape the tcgen05 kernel is chosen for go through it in one launch, sharing one activation image;
// anything else is one linear after the other.
int linear_device_multi(const jq_weight* const* ws, int count, const float* x, int64_t m, float* const* ys, cudaStream_t s) {
    if (count <= 0) {
        return JQ_OK;
    }
    const int64_t min_rows = g_prefill_min_rows.load();
    bool same = count >= 1;
    int64_t n_all = 0;
    for (int i = 0; i < count && same; i++) {
        same = ws[i]->type == ws[0]->type && ws[i]->k == ws[0]->k && ws[i]->n > 0;
        n_all += ws[i]->n;
    }
    if (!same && count >= 2 && count <= 3) {
        // mixed formats (a Q6_K wv beside Q4_K wq and wk): those like the first go together, the others alone
        const jq_weight* like[3];
        float* like_y[3];
        int n_like = 0;
        for (int i = 0; i < count; i++) {
            if (ws[i]->type == ws[0]->type && ws[i]->k == ws[0]->k && ws[i]->n > 0) {
                like[n_like] = ws[i];
                like_y[n_like++] = ys[i];
            } else {
                int rc = linear_device(ws[i], x, m, nullptr, ys[i], s, false);
                if (rc != JQ_OK) {
                    return rc;
                }
            }
        }
        return n_like > 0 ? linear_device_multi(like, n_like, x, m, like_y, s) : JQ_OK;
    }
    const bool together = same && count >= 2 && count <= 3 && m >= 1 && m <= 16 && !(min_rows > 0 && m >= min_rows);
    if (together && gemv_umma_takes(ws[0]->type, ws[0]->k, (int)m, n_all)) {
        View vs[3];
        for (int i = 0; i < count; i++) {
            vs[i] = view_of(ws[i]);
        }
        uint8_t* image = nullptr;
        int rc = scratch_for(s, gemv_umma_image_bytes(ws[0]->k, (int)m), &image);
        return rc == JQ_OK ? launch_gemv_umma_multi(vs, count, x, image, (int)m, nullptr, ys, s) : rc;
    }
    const bool k_quant = ws[0]->type == JQ_TYPE_Q4_K || ws[0]->type == JQ_TYPE_Q5_K;
    if (count >= 2 && count <= 3 && same && k_quant && g_opt_gemv_generic.load() == 0 && !(min_rows > 0 && m >= min_rows)) {
        // the mma.sync kernel: up to 8 rows of x per pass, the weights' rows one after the other in one launch on one image
        View vs[3];
        for (int i = 0; i < count; i++) {
            vs[i] = view_of(ws[i]);
        }
        bool all = true;
        for (int64_t m0 = 0; m0 < m && all; m0 += 8) {
            const int rows = (int)(m - m0 < 8 ? m - m0 : 8);
            float* out[3];
            for (int i = 0; i < count; i++) {
                out[i] = ys[i] + m0 * ws[i]->n;
            }
            uint8_t* image = nullptr;
            bool handled = false;
            int rc = scratch_for(s, gemv_q4k_i8_scratch_bytes(ws[0]->k, rows), &image);
            if (rc == JQ_OK) {
                rc = launch_gemv_q4k_i8_multi(vs, count, x + m0 * ws[0]->k, rows, out, s, image, &handled);
            }
            if (rc != JQ_OK) {
                return rc;
            }
            all = handled;  // a shape that kernel declines (nothing has been launched for this group): one linear after the other
        }
        if (all) {
            return JQ_OK;
        }
    }
    for (int i = 0; i < count; i++) {
        int rc = linear_device(ws[i], x, m, nullptr, ys[i], s, false);
        if (rc != JQ_OK) {
            return rc;
        }
    }
    return JQ_OK;
}

}  // namespace jq

using namespace jq;

extern "C" {

int jq_version(void) { return 100; }

const char* jq_last_error(void) { return t_error.c_str(); }

int jq_block_values(int type) { return block_values(type); }

int jq_block_bytes(int type) { return block_bytes(type); }

int jq_device_count(int* count) {
    if (count == nullptr) {
        return fail(JQ_ERR_INVALID, "jq_device_count: null result pointer");
    }
    JQ_CUDA(cudaGetDeviceCount(count));
    return JQ_OK;
}

int64_t jq_launch_count(void) { return g_launches.load(); }

int jq_weight_upload_rows(int device, int type, const void* host_blocks, int64_t nbytes, int64_t n, int64_t k, int64_t row_begin,
                          int64_t row_end, int layout, jq_weight** out) {
    if (out == nullptr) {
        return fail(JQ_ERR_INVALID, "weight upload: null result pointer");
    }
    *out = nullptr;
    int qk = block_values(type), bb = block_bytes(type);
    if (qk == 0) {
        return fail(JQ_ERR_INVALID, "weight upload: type id %d is not a GGUF block format this library loads", type);
    }
    if (n < 0 || k < 0 || k % qk != 0) {
        return fail(JQ_ERR_INVALID, "%s weight of shape [%lld, %lld]: last axis not a multiple of its block of %d", type_name(type),
                    (long long)n, (long long)k, qk);
    }
    if (n * k >= ((int64_t)1 << 31)) {
        return fail(JQ_ERR_INVALID, "%s weight of shape [%lld, %lld]: more than 2^31-1 elements", type_name(type), (long long)n, (long long)k);
    }
    int64_t row_bytes = k / qk * bb;
    if (nbytes != n * row_bytes) {
        return fail(JQ_ERR_INVALID, "%s tensor of shape [%lld, %lld] needs %lld bytes, got %lld", type_name(type), (long long)n, (long long)k,
                    (long long)(n * row_bytes), (long long)nbytes);
    }
    if (row_begin < 0 || row_end < row_begin || row_end > n) {
        return fail(JQ_ERR_INVALID, "weight upload: rows [%lld, %lld) outside [0, %lld)", (long long)row_begin, (long long)row_end, (long long)n);
    }
    if (layout != JQ_LAYOUT_AUTO) {
        return fail(JQ_ERR_INVALID, "weight upload: unknown layout %d", layout);
    }
    if (host_blocks == nullptr && nbytes > 0) {
        return fail(JQ_ERR_INVALID, "weight upload: null blocks");
    }
    int count = 0;
    JQ_CUDA(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count) {
        return fail(JQ_ERR_INVALID, "weight upload: device %d of %d", device, count);
    }
    DeviceGuard guard(device);
    if (!guard.ok) {
        return fail(JQ_ERR_CUDA, "weight upload: cannot select device %d", device);
    }
    int64_t rows = row_end - row_begin;
    int64_t blocks = rows * (k / qk);
    const uint8_t* src = (const uint8_t*)host_blocks + row_begin * row_bytes;
    int64_t src_bytes = rows * row_bytes;

    jq_weight* w = new (std::nothrow) jq_weight();
    if (w == nullptr) {
        return fail(JQ_ERR_OOM, "weight upload: out of host memory");
    }
    w->magic = JQ_WEIGHT_MAGIC;
    w->device = device;
    w->type = type;
    w->layout = layout;
    w->n = rows;
    w->k = k;
    const bool tiled = tiled_layout(type) || tiled_planes(type);
    w->q_bytes = tiled ? tiled_rows(rows) * (k / qk) * plane_q_bytes(type) : blocks * plane_q_bytes(type);
    w->aux_bytes = (tiled_planes(type) ? tiled_rows(rows) * (k / qk) : blocks) * plane_aux_bytes(type);
    w->q = nullptr;
    w->aux = nullptr;

    int rc = JQ_OK;
    uint8_t* tmp = nullptr;
    // PAD_ROWS rows of zeros follow each plane, so that 16-row tiles may read past the last row
    const int64_t pad_q = (int64_t)PAD_ROWS * (k / qk) * plane_q_bytes(type), pad_aux = (int64_t)PAD_ROWS * (k / qk) * plane_aux_bytes(type);
    cudaError_t e = cudaMalloc(&w->q, (size_t)(w->q_bytes + pad_q + 16));
    if (e == cudaSuccess) {
        // a tiled weight is zeroed as a whole (the rows that pad its last tile), the others behind their last row
        e = tiled ? cudaMemset(w->q, 0, (size_t)(w->q_bytes + pad_q + 16)) : cudaMemset(w->q + w->q_bytes, 0, (size_t)(pad_q + 16));
    }
    if (e == cudaSuccess && w->aux_bytes > 0) {
        e = cudaMalloc(&w->aux, (size_t)(w->aux_bytes + pad_aux));
        if (e == cudaSuccess) {
            e = tiled ? cudaMemset(w->aux, 0, (size_t)(w->aux_bytes + pad_aux)) : cudaMemset(w->aux + w->aux_bytes, 0, (size_t)pad_aux);
        }
    }
    if (e != cudaSuccess) {
        rc = cuda_fail(e, "cudaMalloc(weight)");
    }
    if (rc == JQ_OK && src_bytes > 0) {
        if (plane_aux_bytes(type) == 0 && !tiled_layout(type)) {
            e = cudaMemcpy(w->q, src, (size_t)src_bytes, cudaMemcpyHostToDevice);
            if (e != cudaSuccess) {
                rc = cuda_fail(e, "cudaMemcpy(weight)");
            }
        } else {
            e = cudaMalloc(&tmp, (size_t)src_bytes);
            if (e == cudaSuccess) {
                e = cudaMemcpy(tmp, src, (size_t)src_bytes, cudaMemcpyHostToDevice);
            }
            if (e != cudaSuccess) {
                rc = cuda_fail(e, "staging the verbatim blocks");
            } else {
                rc = tiled_layout(type) ? launch_tile(type, tmp, w->q, rows, k / qk, false, nullptr) : launch_repack(type, tmp, w->q, w->aux, blocks, k / qk, nullptr);
                if (rc == JQ_OK) {
                    e = cudaDeviceSynchronize();
                    if (e != cudaSuccess) {
                        rc = cuda_fail(e, "repack");
                    }
                }
            }
        }
    }
    if (tmp != nullptr) {
        cudaFree(tmp);
    }
    if (rc != JQ_OK) {
        cudaFree(w->q);
        cudaFree(w->aux);
        w->magic = 0;
        delete w;
        return rc;
    }
    *out = w;
    return JQ_OK;
}

int jq_weight_upload(int device, int type, const void* host_blocks, int64_t nbytes, int64_t n, int64_t k, int layout, jq_weight** out) {
    return jq_weight_upload_rows(device, type, host_blocks, nbytes, n, k, 0, n < 0 ? 0 : n, layout, out);
}

int jq_weight_free(jq_weight* w) {
    if (w == nullptr) {
        return JQ_OK;
    }
    int rc = check_weight(w, "jq_weight_free");
    if (rc != JQ_OK) {
        return rc;
    }
    DeviceGuard guard(w->device);
    cudaFree(w->q);
    cudaFree(w->aux);
    w->magic = 0;
    delete w;
    return JQ_OK;
}

int jq_weight_info(const jq_weight* w, int64_t info[8]) {
    int rc = check_weight(w, "jq_weight_info");
    if (rc != JQ_OK) {
        return rc;
    }
    if (info == nullptr) {
        return fail(JQ_ERR_INVALID, "jq_weight_info: null result pointer");
    }
    info[0] = w->n;
    info[1] = w->k;
    info[2] = w->type;
    info[3] = w->layout;
    info[4] = w->device;
    info[5] = w->q_bytes + w->aux_bytes;
    info[6] = block_values(w->type);
    info[7] = block_bytes(w->type);
    return JQ_OK;
}

int jq_weight_download(const jq_weight* w, void* host_blocks, int64_t nbytes) {
    int rc = check_weight(w, "jq_weight_download");
    if (rc != JQ_OK) {
        return rc;
    }
    int64_t blocks = w->n * (w->k / block_values(w->type));
    int64_t want = blocks * block_bytes(w->type);
    if (nbytes != want || (host_blocks == nullptr && want > 0)) {
        return fail(JQ_ERR_INVALID, "jq_weight_download: needs a buffer of %lld bytes, got %lld", (long long)want, (long long)nbytes);
    }
    if (want == 0) {
        return JQ_OK;
    }
    DeviceGuard guard(w->device);
    if (plane_aux_bytes(w->type) == 0 && !tiled_layout(w->type)) {
        JQ_CUDA(cudaMemcpy(host_blocks, w->q, (size_t)want, cudaMemcpyDeviceToHost));
        return JQ_OK;
    }
    uint8_t* tmp = nullptr;
    JQ_CUDA(cudaMalloc(&tmp, (size_t)want));
    rc = tiled_layout(w->type) ? launch_tile(w->type, tmp, w->q, w->n, w->k / block_values(w->type), true, nullptr)
                               : launch_unpack(w->type, w->q, w->aux, tmp, blocks, w->k / block_values(w->type), nullptr);
    if (rc == JQ_OK) {
        cudaError_t e = cudaMemcpy(host_blocks, tmp, (size_t)want, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) {
            rc = cuda_fail(e, "cudaMemcpy(download)");
        }
    }
    cudaFree(tmp);
    return rc;
}

int jq_dequantize(const jq_weight* w, float* dst, int dst_mem, void* stream) {
    int rc = check_weight(w, "jq_dequantize");
    if (rc != JQ_OK) {
        return rc;
    }
    int64_t count = w->n * w->k;
    if (count == 0) {
        return JQ_OK;
    }
    if (dst == nullptr) {
        return fail(JQ_ERR_INVALID, "jq_dequantize: null destination");
    }
    DeviceGuard guard(w->device);
    if (dst_mem == JQ_MEM_DEVICE) {
        if (((uintptr_t)dst & 15) != 0) {
            return fail(JQ_ERR_INVALID, "jq_dequantize: device destination must be 16-byte aligned");
        }
        return launch_dequantize(view_of(w), dst, (cudaStream_t)stream);
    }
    if (dst_mem != JQ_MEM_HOST) {
        return fail(JQ_ERR_INVALID, "jq_dequantize: unknown memory kind %d", dst_mem);
    }
    Staging* st;
    rc = staging_for(w->device, (size_t)count * 4, &st);
    if (rc != JQ_OK) {
        return rc;
    }
    rc = launch_dequantize(view_of(w), (float*)st->dev, st->stream);
    if (rc != JQ_OK) {
        return rc;
    }
    JQ_CUDA(cudaMemcpyAsync(dst, st->dev, (size_t)count * 4, cudaMemcpyDeviceToHost, st->stream));
    JQ_CUDA(cudaStreamSynchronize(st->stream));
    return JQ_OK;
}

int jq_linear_f32(const jq_weight* w, const float* x, int64_t m, const float* bias, float* y, int mem, void* stream) {
    int rc = check_weight(w, "jq_linear_f32");
    if (rc != JQ_OK) {
        return rc;
    }
    if (!has_linear_kernel(w->type)) {
        return fail(JQ_ERR_UNSUPPORTED, "%s linear: the format is dequantise-only", type_name(w->type));
    }
    if (m < 0) {
        return fail(JQ_ERR_INVALID, "%s linear: input of %lld rows and weight [%lld, %lld]", type_name(w->type), (long long)m, (long long)w->n,
                    (long long)w->k);
    }
    if (m == 0 || w->n == 0) {
        return JQ_OK;
    }
    if (x == nullptr || y == nullptr) {
        return fail(JQ_ERR_INVALID, "%s linear: null input or output", type_name(w->type));
    }
    DeviceGuard guard(w->device);
    if (mem == JQ_MEM_DEVICE) {
        if ((((uintptr_t)x | (uintptr_t)y) & 15) != 0) {
            return fail(JQ_ERR_INVALID, "%s linear: device pointers must be 16-byte aligned", type_name(w->type));
        }
        return linear_device(w, x, m, bias, y, (cudaStream_t)stream, false);
    }
    if (mem != JQ_MEM_HOST) {
        return fail(JQ_ERR_INVALID, "%s linear: unknown memory kind %d", type_name(w->type), mem);
    }
    size_t xb = align256((size_t)m * w->k * 4), bb = align256((size_t)w->n * 4), yb = align256((size_t)m * w->n * 4);
    Staging* st;
    rc = staging_for(w->device, xb + bb + yb, &st);
    if (rc != JQ_OK) {
        return rc;
    }
    // Page-locked host buffers (jq_host_alloc, cudaHostAlloc, cudaHostRegister) are addressable from the GPU: small inputs
    // and outputs are then read and written by the kernels themselves across PCIe, which saves the set-up latency of two
    // copy-engine transfers per call. Pageable memory, and outputs too large for scattered stores, go through copies.
    const size_t direct_limit = (size_t)256 << 10;
    const float* dx = pinned_device_pointer(x, (size_t)m * w->k * 4, direct_limit << 2);
    const float* db = bias != nullptr ? pinned_device_pointer(bias, (size_t)w->n * 4, direct_limit) : nullptr;
    float* dy = const_cast<float*>(pinned_device_pointer(y, (size_t)m * w->n * 4, direct_limit));
    const bool copy_y = dy == nullptr;
    if (dx == nullptr) {
        JQ_CUDA(cudaMemcpyAsync(st->dev, x, (size_t)m * w->k * 4, cudaMemcpyHostToDevice, st->stream));
        dx = (const float*)st->dev;
    }
    if (bias != nullptr && db == nullptr) {
        JQ_CUDA(cudaMemcpyAsync(st->dev + xb, bias, (size_t)w->n * 4, cudaMemcpyHostToDevice, st->stream));
        db = (const float*)(st->dev + xb);
    }
    if (copy_y) {
        dy = (float*)(st->dev + xb + bb);
    }
    rc = linear_device(w, dx, m, db, dy, st->stream, dx == x);  // x in host memory: read it once, not once per thread block
    if (rc != JQ_OK) {
        return rc;
    }
    if (copy_y) {
        JQ_CUDA(cudaMemcpyAsync(y, dy, (size_t)m * w->n * 4, cudaMemcpyDeviceToHost, st->stream));
    }
    JQ_CUDA(cudaStreamSynchronize(st->stream));
    return JQ_OK;
}

int jq_linear_backward_f32(const jq_weight* w, const float* g, int64_t m, float* gx, int mem, void* stream) {
    int rc = check_weight(w, "jq_linear_backward_f32");
    if (rc != JQ_OK) {
        return rc;
    }
    if (!has_linear_kernel(w->type)) {
        return fail(JQ_ERR_UNSUPPORTED, "%s linear backward: the format is dequantise-only", type_name(w->type));
    }
    if (m < 0) {
        return fail(JQ_ERR_INVALID, "%s linear backward: gradient of %lld rows and weight [%lld, %lld]", type_name(w->type), (long long)m,
                    (long long)w->n, (long long)w->k);
    }
    if (m == 0 || w->k == 0) {
        return JQ_OK;
    }
    if (gx == nullptr || (g == nullptr && w->n > 0)) {
        return fail(JQ_ERR_INVALID, "%s linear backward: null gradient", type_name(w->type));
    }
    DeviceGuard guard(w->device);
    const size_t gb = align256((size_t)m * w->n * 4), xb = (size_t)m * w->k * 4;
    if (mem == JQ_MEM_DEVICE) {
        if (((uintptr_t)gx & 15) != 0) {
            return fail(JQ_ERR_INVALID, "%s linear backward: device pointers must be 16-byte aligned", type_name(w->type));
        }
        if (w->n == 0) {
            JQ_CUDA(cudaMemsetAsync(gx, 0, xb, (cudaStream_t)stream));
            return JQ_OK;
        }
        return launch_linear_backward(view_of(w), g, m, gx, (cudaStream_t)stream);
    }
    if (mem != JQ_MEM_HOST) {
        return fail(JQ_ERR_INVALID, "%s linear backward: unknown memory kind %d", type_name(w->type), mem);
    }
    Staging* st;
    rc = staging_for(w->device, gb + xb, &st);
    if (rc != JQ_OK) {
        return rc;
    }
    float* dgx = (float*)(st->dev + gb);
    if (w->n == 0) {
        JQ_CUDA(cudaMemsetAsync(dgx, 0, xb, st->stream));
    } else {
        JQ_CUDA(cudaMemcpyAsync(st->dev, g, (size_t)m * w->n * 4, cudaMemcpyHostToDevice, st->stream));
        rc = launch_linear_backward(view_of(w), (const float*)st->dev, m, dgx, st->stream);
        if (rc != JQ_OK) {
            return rc;
        }
    }
    JQ_CUDA(cudaMemcpyAsync(gx, dgx, xb, cudaMemcpyDeviceToHost, st->stream));
    JQ_CUDA(cudaStreamSynchronize(st->stream));
    return JQ_OK;
}

int jq_linear_bf16(const jq_weight* w, const uint16_t* x, int64_t m, const float* bias, float* y, int mem, void* stream) {
    int rc = check_weight(w, "jq_linear_bf16");
    if (rc != JQ_OK) {
        return rc;
    }
    if (!has_linear_kernel(w->type)) {
        return fail(JQ_ERR_UNSUPPORTED, "%s linear: the format is dequantise-only", type_name(w->type));
    }
    if (m < 0 || m >= ((int64_t)1 << 31)) {
        return fail(JQ_ERR_INVALID, "%s linear: input of %lld rows and weight [%lld, %lld]", type_name(w->type), (long long)m, (long long)w->n,
                    (long long)w->k);
    }
    if (m == 0 || w->n == 0) {
        return JQ_OK;
    }
    if (x == nullptr || y == nullptr) {
        return fail(JQ_ERR_INVALID, "%s linear: null input or output", type_name(w->type));
    }
    DeviceGuard guard(w->device);
    View v = view_of(w);
    if (mem == JQ_MEM_DEVICE) {
        if ((((uintptr_t)x | (uintptr_t)y) & 15) != 0) {
            return fail(JQ_ERR_INVALID, "%s linear: device pointers must be 16-byte aligned", type_name(w->type));
        }
        return launch_prefill_bf16(v, x, m, bias, y, (cudaStream_t)stream);
    }
    if (mem != JQ_MEM_HOST) {
        return fail(JQ_ERR_INVALID, "%s linear: unknown memory kind %d", type_name(w->type), mem);
    }
    size_t xb = align256((size_t)m * w->k * 2), bb = align256((size_t)w->n * 4), yb = align256((size_t)m * w->n * 4);
    Staging* st;
    rc = staging_for(w->device, xb + bb + yb, &st);
    if (rc != JQ_OK) {
        return rc;
    }
    uint16_t* dx = (uint16_t*)st->dev;
    float* db = (float*)(st->dev + xb);
    float* dy = (float*)(st->dev + xb + bb);
    JQ_CUDA(cudaMemcpyAsync(dx, x, (size_t)m * w->k * 2, cudaMemcpyHostToDevice, st->stream));
    if (bias != nullptr) {
        JQ_CUDA(cudaMemcpyAsync(db, bias, (size_t)w->n * 4, cudaMemcpyHostToDevice, st->stream));
    }
    rc = launch_prefill_bf16(v, dx, m, bias != nullptr ? db : nullptr, dy, st->stream);
    if (rc != JQ_OK) {
        return rc;
    }
    JQ_CUDA(cudaMemcpyAsync(y, dy, (size_t)m * w->n * 4, cudaMemcpyDeviceToHost, st->stream));
    JQ_CUDA(cudaStreamSynchronize(st->stream));
    int status = 0;
    rc = prefill_status(&status);
    if (rc == JQ_OK && status != 0) {
        rc = fail(JQ_ERR_TIMEOUT, "prefill kernel: a bounded wait gave up (code %d)", status);
    }
    return rc;
}

int jq_device_status(int device, int* status) {
    if (status == nullptr) {
        return fail(JQ_ERR_INVALID, "jq_device_status: null result pointer");
    }
    int count = 0;
    JQ_CUDA(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count) {
        return fail(JQ_ERR_INVALID, "jq_device_status: device %d of %d", device, count);
    }
    DeviceGuard guard(device);
    JQ_CUDA(cudaDeviceSynchronize());
    int rc = prefill_status(status);
    int peer = 0;
    if (rc == JQ_OK) {
        rc = peer_status(&peer);
    }
    if (rc == JQ_OK && *status == 0) {
        *status = peer;
    }
    for (int part = 0; part < 4 && rc == JQ_OK; part++) {
        int other = 0;
        rc = part == 0 ? gemv_peer_status(&other) : (part == 1 ? decoder_peer_status(&other) : (part == 2 ? gemv_umma_status(&other) : gemv_q6k_status(&other)));
        if (rc == JQ_OK && *status == 0) {
            *status = other;
        }
    }
    return rc;
}

int jq_quantize_q8_0(int device, const float* x, int64_t count, void* blocks_out, int mem, void* stream) {
    if (count < 0 || count % 32 != 0) {
        return fail(JQ_ERR_INVALID, "Q8_0 needs a last axis that is a multiple of 32, got %lld values", (long long)count);
    }
    if (count == 0) {
        return JQ_OK;
    }
    if (x == nullptr || blocks_out == nullptr) {
        return fail(JQ_ERR_INVALID, "jq_quantize_q8_0: null input or output");
    }
    int devices = 0;
    JQ_CUDA(cudaGetDeviceCount(&devices));
    if (device < 0 || device >= devices) {
        return fail(JQ_ERR_INVALID, "jq_quantize_q8_0: device %d of %d", device, devices);
    }
    DeviceGuard guard(device);
    int64_t blocks = count / 32;
    if (mem == JQ_MEM_DEVICE) {
        return launch_quantize_q8_0(x, blocks, (uint8_t*)blocks_out, (cudaStream_t)stream);
    }
    if (mem != JQ_MEM_HOST) {
        return fail(JQ_ERR_INVALID, "jq_quantize_q8_0: unknown memory kind %d", mem);
    }
    size_t xb = align256((size_t)count * 4), ob = (size_t)blocks * 34;
    Staging* st;
    int rc = staging_for(device, xb + ob, &st);
    if (rc != JQ_OK) {
        return rc;
    }
    JQ_CUDA(cudaMemcpyAsync(st->dev, x, (size_t)count * 4, cudaMemcpyHostToDevice, st->stream));
    rc = launch_quantize_q8_0((const float*)st->dev, blocks, st->dev + xb, st->stream);
    if (rc != JQ_OK) {
        return rc;
    }
    JQ_CUDA(cudaMemcpyAsync(blocks_out, st->dev + xb, ob, cudaMemcpyDeviceToHost, st->stream));
    JQ_CUDA(cudaStreamSynchronize(st->stream));
    return JQ_OK;
}

int jq_set_option(const char* name, int64_t value) {
    if (name != nullptr && strcmp(name, "prefill_min_rows") == 0) {
        if (value < 0) {
            return fail(JQ_ERR_INVALID, "option prefill_min_rows: %lld is negative", (long long)value);
        }
        g_prefill_min_rows.store(value);
        return JQ_OK;
    }
    if (name != nullptr && strcmp(name, "gemv_generic") == 0) {
        g_opt_gemv_generic.store(value != 0);
        return JQ_OK;
    }
    if (name != nullptr && strcmp(name, "decoder_fused") == 0) {
        g_opt_decoder_fused.store(value != 0);
        return JQ_OK;
    }
    if (name != nullptr && strcmp(name, "gemv_tcgen05") == 0) {
        if (value < 0 || value > 2) {
            return fail(JQ_ERR_INVALID, "option gemv_tcgen05: %lld is not 0 (where faster), 1 (always) or 2 (never)", (long long)value);
        }
        g_opt_gemv_umma.store(value);
        return JQ_OK;
    }
    if (name != nullptr && strcmp(name, "wait_limit_us") == 0) {
        if (value < 1 || value > 60000000) {
            return fail(JQ_ERR_INVALID, "option wait_limit_us: %lld is outside [1, 60000000]", (long long)value);
        }
        g_opt_wait_limit_us.store(value);
        return JQ_OK;
    }
    if (name != nullptr && strcmp(name, "peer_wait_us") == 0) {
        if (value < 1 || value > 60000000) {
            return fail(JQ_ERR_INVALID, "option peer_wait_us: %lld is outside [1, 60000000]", (long long)value);
        }
        g_opt_peer_wait_us.store(value);
        return JQ_OK;
    }
    if (name != nullptr && strcmp(name, "decoder_graph") == 0) {
        g_opt_decoder_graph.store(value != 0);
        return JQ_OK;
    }
    return fail(JQ_ERR_INVALID, "unknown option '%s'", name == nullptr ? "(null)" : name);
}

int jq_get_option(const char* name, int64_t* value) {
    if (name != nullptr && value != nullptr && strcmp(name, "prefill_min_rows") == 0) {
        *value = g_prefill_min_rows.load();
        return JQ_OK;
    }
    if (name != nullptr && value != nullptr && strcmp(name, "gemv_generic") == 0) {
        *value = g_opt_gemv_generic.load();
        return JQ_OK;
    }
    if (name != nullptr && value != nullptr && strcmp(name, "decoder_fused") == 0) {
        *value = g_opt_decoder_fused.load();
        return JQ_OK;
    }
    if (name != nullptr && value != nullptr && strcmp(name, "gemv_tcgen05") == 0) {
        *value = g_opt_gemv_umma.load();
        return JQ_OK;
    }
    if (name != nullptr && value != nullptr && strcmp(name, "wait_limit_us") == 0) {
        *value = g_opt_wait_limit_us.load();
        return JQ_OK;
    }
    if (name != nullptr && value != nullptr && strcmp(name, "peer_wait_us") == 0) {
        *value = g_opt_peer_wait_us.load();
        return JQ_OK;
    }
    if (name != nullptr && value != nullptr && strcmp(name, "decoder_graph") == 0) {
        *value = g_opt_decoder_graph.load();
        return JQ_OK;
    }
    return fail(JQ_ERR_INVALID, "unknown option '%s'", name == nullptr ? "(null)" : name);
}

int jq_host_alloc(void** ptr, int64_t nbytes) {
    if (ptr == nullptr || nbytes < 0) {
        return fail(JQ_ERR_INVALID, "jq_host_alloc: bad arguments");
    }
    *ptr = nullptr;
    cudaError_t e = cudaMallocHost(ptr, (size_t)(nbytes > 0 ? nbytes : 1));
    if (e != cudaSuccess) {
        return fail(JQ_ERR_OOM, "jq_host_alloc(%lld): %s", (long long)nbytes, cudaGetErrorString(e));
    }
    return JQ_OK;
}

int jq_host_free(void* ptr) {
    if (ptr != nullptr) {
        JQ_CUDA(cudaFreeHost(ptr));
    }
    return JQ_OK;
}

}  // extern "C"
