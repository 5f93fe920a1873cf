// Row-sharded linears over the GPUs of one box without a collective library in the data path: every rank stores its
// slice of y straight into every rank's copy of the full y over NVLink (plain peer stores into memory mapped with CUDA
// IPC), then raises a flag on every rank; a rank's next kernels start after a bounded wait on its own flags.
//
//   rank g:   GEMV over its rows  ->  peer_scatter_kernel: every value of the slice goes into y_g and, as an 8-byte word
//                                     {value, number of the exchange}, into every other rank's staging area; then the
//                                     kernel's threads collect what the other ranks own: each polls a staging word until it
//                                     carries this exchange's number (bounded) and moves the value into y_g
//             (for Q4_K and Q5_K decode shapes the GEMV's own epilogue does what the scatter kernel does)
// Nothing in this path needs a fence or an atomic between GPUs (a system-wide release costs a thread block 2.5 to 8
// microseconds when every block of a grid makes one). The decoder's activation images, which cannot carry marks, use
// the other form (jq_peer_device.cuh): release-ordered remote adds to arrival counters.
//
// The reference gathers with Collective.allGather (dist/Collective.java:64-65, NCCL form dist/NcclOp.java:184-198); for
// the 4 KB - 128 KB slices of a decode step that call costs more than the GEMV it follows.
//
// A peer buffer is one cudaMalloc'd allocation: 4096 bytes of flags (uint32 [world] arrival counters, counter r added
// to by rank r; word 17, never written by peers: the number of exchanges this rank has made on the
// buffer; from byte 128 on up to eight copies of the target table PeerOut that the fused GEMV epilogue reads), then the
// payload. Every exchange adds 2^16 to a counter, so a counter says which exchange has completely arrived. The number
// lives in device memory and grows by one per exchange, so a captured CUDA graph can be replayed; all ranks make the
// same exchanges on a buffer in the same order, which keeps their numbers in step. A rank can run one exchange ahead of another:
// a payload area must not be the target of two consecutive exchanges (use two areas in turn, or other buffers in
// between).
// No load ever targets a peer's memory, nothing here uses multicast, and the only wait is bounded: when it gives up
// it records status 32 + (rank it waited for), readable through jq_device_status, and the kernel returns.
#include <cstring>
#include <map>
#include <mutex>

#include "jq_common.cuh"
#include "jq_peer_device.cuh"

namespace jq {

static __device__ int g_peer_status;
std::atomic<int64_t> g_opt_peer_wait_us{400000};

int linear_device(const jq_weight* w, const float* x, int64_t m, const float* bias, float* y, cudaStream_t s, bool x_remote = false);

namespace {


struct PeerTargets {
    float* y[PEER_MAX_WORLD];                   // every rank's full y [m, n_total] (own included)
    uint32_t* flags[PEER_MAX_WORLD];            // every rank's flag words
    unsigned long long* stage[PEER_MAX_WORLD];  // every rank's staging words [m, n_total]
};

// slice [m, n_slice] -> columns col0 .. of this rank's y [m, n_total] and, marked, of every other rank's staging area;
// then the other ranks' columns from this rank's staging area into its y.
__global__ void __launch_bounds__(256) peer_scatter_kernel(const float* __restrict__ slice, int64_t m, PeerOut po) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t seq = peer_marks_seq(&po);
    const int64_t count = m * po.n_own;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / po.n_own, col = i % po.n_own;
        peer_store_marked(&po, row * po.n_total + po.col0 + col, slice[i], seq);
    }
    peer_collect(&po, (int)m, seq, &g_peer_status);
}

// Writes a target table into this rank's flag area (one thread).
__global__ void peer_table_kernel(PeerOut table, PeerOut* dst) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 0) {
        *dst = table;
    }
}

}  // namespace

// Reads and clears the status of the peer waits of the current device.
int peer_status(int* status) {
    const int zero = 0;
    JQ_CUDA(cudaMemcpyFromSymbol(status, g_peer_status, sizeof(int)));
    JQ_CUDA(cudaMemcpyToSymbol(g_peer_status, &zero, sizeof(int)));
    return JQ_OK;
}

}  // namespace jq

using namespace jq;

extern "C" {

static void forget_tables(const void* buffer);

JQ_API int jq_peer_alloc(int device, int64_t payload_bytes, void** ptr, void* handle_out) {
    if (ptr == nullptr || handle_out == nullptr || payload_bytes < 0) {
        return fail(JQ_ERR_INVALID, "jq_peer_alloc: null result pointer or negative size");
    }
    *ptr = nullptr;
    int prev = -1;
    cudaGetDevice(&prev);
    JQ_CUDA(cudaSetDevice(device));
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, (size_t)payload_bytes + PEER_FLAG_BYTES);
    if (e == cudaSuccess) e = cudaMemset(p, 0, (size_t)payload_bytes + PEER_FLAG_BYTES);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (prev >= 0) cudaSetDevice(prev);
    if (e != cudaSuccess) {
        if (p != nullptr) cudaFree(p);
        return e == cudaErrorMemoryAllocation ? fail(JQ_ERR_OOM, "jq_peer_alloc: %lld bytes on device %d", (long long)payload_bytes, device)
                                              : cuda_fail(e, "jq_peer_alloc");
    }
    forget_tables(p);
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
    memcpy(handle_out, &h, sizeof(h));
    *ptr = p;
    return JQ_OK;
}

JQ_API int jq_peer_open(int device, const void* handle, void** ptr) {
    if (ptr == nullptr || handle == nullptr) {
        return fail(JQ_ERR_INVALID, "jq_peer_open: null handle or result pointer");
    }
    *ptr = nullptr;
    int prev = -1;
    cudaGetDevice(&prev);
    JQ_CUDA(cudaSetDevice(device));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (prev >= 0) cudaSetDevice(prev);
    if (e != cudaSuccess) {
        return cuda_fail(e, "jq_peer_open (is peer access between the two GPUs possible?)");
    }
    *ptr = p;
    return JQ_OK;
}

JQ_API int jq_peer_close(void* ptr) {
    if (ptr == nullptr) {
        return JQ_OK;
    }
    cudaError_t e = cudaIpcCloseMemHandle(ptr);
    return e == cudaSuccess ? JQ_OK : cuda_fail(e, "jq_peer_close");
}

JQ_API int jq_peer_free(void* ptr) {
    if (ptr == nullptr) {
        return JQ_OK;
    }
    forget_tables(ptr);
    cudaError_t e = cudaFree(ptr);
    return e == cudaSuccess ? JQ_OK : cuda_fail(e, "jq_peer_free");
}

JQ_API int64_t jq_peer_payload_offset(void) { return PEER_FLAG_BYTES; }

static int fill_targets(void* const* peer_buffers, int64_t payload_offset, int64_t staging_offset, int rank, int world, PeerTargets* tg, const char* who) {
    // staging_offset < 0: an exchange that does not use staging words (the decoder's)
    if (peer_buffers == nullptr || world < 1 || world > PEER_MAX_WORLD || rank < 0 || rank >= world || payload_offset < 0 || payload_offset % 16 != 0 ||
        staging_offset % 16 != 0) {
        return fail(JQ_ERR_INVALID, "%s: rank %d of %d (at most %d), payload offset %lld, staging offset %lld (multiples of 16)", who, rank, world, PEER_MAX_WORLD,
                    (long long)payload_offset, (long long)staging_offset);
    }
    for (int r = 0; r < PEER_MAX_WORLD; r++) {
        uint8_t* base = r < world ? static_cast<uint8_t*>(peer_buffers[r]) : nullptr;
        if (r < world && base == nullptr) {
            return fail(JQ_ERR_INVALID, "%s: the buffer of rank %d is null", who, r);
        }
        tg->flags[r] = reinterpret_cast<uint32_t*>(base);
        tg->y[r] = base != nullptr ? reinterpret_cast<float*>(base + PEER_FLAG_BYTES + payload_offset) : nullptr;
        tg->stage[r] = base != nullptr && staging_offset >= 0 ? reinterpret_cast<unsigned long long*>(base + PEER_FLAG_BYTES + staging_offset) : nullptr;
    }
    return JQ_OK;
}

static cudaLaunchConfig_t pdl_config(cudaLaunchAttribute* attr, unsigned grid, unsigned block, cudaStream_t s) {
    cudaLaunchConfig_t cfg = {};
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.stream = s;
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    return cfg;
}

// The device copy of `po` in the flag area of this rank's buffer: found in a small host-side cache of what the area's
// table slots hold, or written (by a one-thread kernel on `s`) into the next slot in turn.
struct TableSlots {
    PeerOut held[PEER_TABLES];
    int used;
};
static std::mutex g_table_mu;
static std::map<const void*, TableSlots> g_table_cache;  // by this rank's buffer; forgotten when the buffer is freed

static void forget_tables(const void* buffer) {
    std::lock_guard<std::mutex> lock(g_table_mu);
    g_table_cache.erase(buffer);
}

static int device_table(const PeerOut& po, cudaStream_t s, const PeerOut** out) {
    uint8_t* own = reinterpret_cast<uint8_t*>(po.flags[po.rank]);
    std::lock_guard<std::mutex> lock(g_table_mu);
    TableSlots& sl = g_table_cache[own];
    for (int i = 0; i < sl.used; i++) {
        if (memcmp(&sl.held[i], &po, sizeof(PeerOut)) == 0) {
            *out = reinterpret_cast<const PeerOut*>(own + PEER_TABLE_OFFSET + i * PEER_TABLE_STRIDE);
            return JQ_OK;
        }
    }
    if (sl.used == PEER_TABLES) {
        // a slot that has been handed out may be baked into a captured graph: it is never overwritten
        return fail(JQ_ERR_INVALID, "peer exchange: this buffer already serves %d distinct (area, shard) targets, the most it has room for; "
                                    "use another buffer (jq_peer_alloc) for more", PEER_TABLES);
    }
    const int slot = sl.used;
    PeerOut* dst = reinterpret_cast<PeerOut*>(own + PEER_TABLE_OFFSET + slot * PEER_TABLE_STRIDE);
    cudaLaunchAttribute attr[1];
    cudaLaunchConfig_t cfg = pdl_config(attr, 1, 32, s);
    JQ_CUDA(cudaLaunchKernelEx(&cfg, peer_table_kernel, po, dst));
    count_launch(1);
    sl.held[slot] = po;
    sl.used++;
    *out = dst;
    return JQ_OK;
}

static long long wait_clocks() { return (long long)g_opt_peer_wait_us.load(std::memory_order_relaxed) * 2000; }  // about 2 GHz

static PeerOut peer_out(const PeerTargets& tg, int64_t n_own, int64_t n_total, int64_t col0, int rank, int world) {
    PeerOut po;
    memset(&po, 0, sizeof(po));
    for (int r = 0; r < PEER_MAX_WORLD; r++) {
        po.y[r] = tg.y[r];
        po.flags[r] = tg.flags[r];
        po.stage[r] = tg.stage[r];
    }
    po.world = world; po.rank = rank; po.n_total = n_total; po.col0 = col0; po.n_own = n_own;
    po.wait_clocks = wait_clocks();
    return po;
}

static int enqueue_scatter(const float* slice, int64_t m, int64_t n_slice, int64_t n_total, int64_t col0, const PeerTargets& tg, int rank, int world,
                           cudaStream_t s) {
    // the grid also collects the other ranks' columns: sized for all of y
    const int64_t count = m * n_total;
    int grid = (int)((count + 255) / 256);
    grid = grid < 1 ? 1 : (grid > 148 ? 148 : grid);
    cudaLaunchAttribute attr[1];
    cudaLaunchConfig_t cfg = pdl_config(attr, (unsigned)grid, 256, s);
    JQ_CUDA(cudaLaunchKernelEx(&cfg, peer_scatter_kernel, slice, m, peer_out(tg, n_slice, n_total, col0, rank, world)));
    count_launch(1);
    return JQ_OK;
}

}  // extern "C"

namespace jq {

int peer_linear_q4k_imaged(const jq_weight* w, const uint8_t* image, int64_t n_total, int64_t col0, void* const* peer_buffers, int64_t payload_offset,
                           int64_t staging_offset, int rank, int world, cudaStream_t s, bool wait_first, bool wait_after) {
    PeerTargets tg;
    int rc = fill_targets(peer_buffers, payload_offset, staging_offset < 0 ? -16 : staging_offset, rank, world, &tg, "peer linear");
    if (rc != JQ_OK) {
        return rc;
    }
    PeerOut po = peer_out(tg, w->n, n_total, col0, rank, world);
    po.wait_first = wait_first ? 1 : 0;
    po.wait_after = wait_after ? 1 : 0;
    rc = device_table(po, s, &po.table);
    bool handled = false;
    if (rc == JQ_OK) {
        const View v{w->q, w->aux, w->n, w->k, w->type};
        rc = launch_gemv_q4k_i8_imaged(v, nullptr, image, nullptr, nullptr, nullptr, s, &handled, &po);
    }
    if (rc == JQ_OK && !handled) {
        rc = fail(JQ_ERR_UNSUPPORTED, "peer linear: a [%lld, %lld] shard is outside what the tensor-core GEMV takes", (long long)w->n, (long long)w->k);
    }
    return rc;
}

}  // namespace jq

extern "C" {

JQ_API int jq_peer_gather(const float* slice, int64_t m, int64_t n_slice, int64_t n_total, int64_t col0, void* const* peer_buffers, int64_t payload_offset,
                          int64_t staging_offset, int rank, int world, void* stream) {
    if (slice == nullptr || m < 1 || n_slice < 0 || col0 < 0 || col0 + n_slice > n_total) {
        return fail(JQ_ERR_INVALID, "jq_peer_gather: slice [%lld, %lld] at column %lld of %lld", (long long)m, (long long)n_slice, (long long)col0,
                    (long long)n_total);
    }
    PeerTargets tg;
    int rc = staging_offset < 0 ? fail(JQ_ERR_INVALID, "jq_peer_gather: negative staging offset")
                                : fill_targets(peer_buffers, payload_offset, staging_offset, rank, world, &tg, "jq_peer_gather");
    if (rc == JQ_OK) rc = enqueue_scatter(slice, m, n_slice, n_total, col0, tg, rank, world, (cudaStream_t)stream);  // waits itself
    return rc;
}

JQ_API int jq_linear_f32_peer(const jq_weight* w, const float* x, int64_t m, const float* bias, int64_t n_total, int64_t col0, void* const* peer_buffers,
                              int64_t payload_offset, int64_t staging_offset, int rank, int world, void* stream) {
    if (w == nullptr || w->magic != JQ_WEIGHT_MAGIC || x == nullptr || m < 1 || col0 < 0 || col0 + w->n > n_total) {
        return fail(JQ_ERR_INVALID, "jq_linear_f32_peer: not a live weight, null x, or rows [%lld, +%lld) outside %lld", (long long)col0,
                    (long long)(w != nullptr ? w->n : 0), (long long)n_total);
    }
    PeerTargets tg;
    int rc = staging_offset < 0 ? fail(JQ_ERR_INVALID, "jq_linear_f32_peer: negative staging offset")
                                : fill_targets(peer_buffers, payload_offset, staging_offset, rank, world, &tg, "jq_linear_f32_peer");
    if (rc != JQ_OK) {
        return rc;
    }
    int prev = -1;
    cudaGetDevice(&prev);
    if (prev != w->device) {
        JQ_CUDA(cudaSetDevice(w->device));
    }
    cudaStream_t s = (cudaStream_t)stream;
    const View v{w->q, w->aux, w->n, w->k, w->type};
    bool fused = false;
    if (w->n > 0 && gemv_umma_takes(w->type, w->k, (int)m)) {
        // the tcgen05 GEMV stores into every rank's y and publishes the exchange itself
        PeerOut po = peer_out(tg, w->n, n_total, col0, rank, world);
        rc = device_table(po, s, &po.table);
        uint8_t* image = nullptr;
        if (rc == JQ_OK) rc = scratch_for(s, gemv_umma_image_bytes(w->k, (int)m), &image);
        if (rc == JQ_OK) rc = launch_gemv_umma(v, nullptr, x, image, (int)m, bias, nullptr, nullptr, s, &po);
        fused = rc == JQ_OK;
    } else if ((w->type == JQ_TYPE_Q4_K || w->type == JQ_TYPE_Q5_K) && m <= 8 && w->n > 0 && g_opt_gemv_generic.load() == 0) {
        // the GEMV kernel itself stores into every rank's y and publishes the exchange; it reads the targets from a table
        // in this rank's flag area, which is written once per distinct (buffers, area, shard) and then found again
        PeerOut po = peer_out(tg, w->n, n_total, col0, rank, world);
        rc = device_table(po, s, &po.table);
        uint8_t* image = nullptr;
        if (rc == JQ_OK) rc = scratch_for(s, gemv_q4k_i8_scratch_bytes(w->k, (int)m), &image);
        if (rc == JQ_OK) {
            rc = launch_gemv_q4k_i8(v, x, (int)m, bias, nullptr, s, image, &fused, &po);
        }
    }
    if (rc == JQ_OK && !fused) {
        // any other format or row count: the ordinary kernels into a slice, then the scatter kernel
        uint8_t* slice = nullptr;
        rc = scratch_for_slot(s, 1, (size_t)m * w->n * sizeof(float), &slice);
        if (rc == JQ_OK) rc = linear_device(w, x, m, bias, reinterpret_cast<float*>(slice), s);
        if (rc == JQ_OK) rc = enqueue_scatter(reinterpret_cast<const float*>(slice), m, w->n, n_total, col0, tg, rank, world, s);
    }
    if (prev >= 0 && prev != w->device) {
        cudaSetDevice(prev);
    }
    return rc;
}

}  // extern "C"
