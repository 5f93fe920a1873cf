// Row-sharded linears over the GPUs of one box without a collective library in the data path: every rank stores its
// slice of y straight into every rank's copy of the full y over NVLink (plain peer stores into memory mapped with CUDA
// IPC), then raises a flag on every rank; a rank's next kernels start after a bounded wait on its own flags.
//
//   rank g:   GEMV over its rows  ->  peer_scatter_kernel: y_r[:, col0 .. col0 + n_g) = slice for every rank r,
//                                     __threadfence_system, last CTA: flags_r[g] = seq for every rank r
//             peer_wait_kernel: until flags_g[r] >= seq for every r (bounded)  ->  consumers of y_g
//
// The reference gathers with Collective.allGather (dist/Collective.java:64-65, NCCL form dist/NcclOp.java:184-198); for
// the 4 KB - 128 KB slices of a decode step that call costs more than the GEMV it follows.
//
// A peer buffer is one cudaMalloc'd allocation: 256 bytes of flags (uint32 [world] arrival flags written by the peers;
// words 16 and 17, never written by peers: a CTA counter and the number of exchanges this rank has made on the
// buffer), then the payload. A flag carries the number of the exchange it announces. The number lives in device
// memory and grows by one per exchange, so a captured CUDA graph can be replayed; all ranks make the same exchanges
// on a buffer in the same order, which keeps their numbers in step. A rank can run one exchange ahead of another:
// a payload area must not be the target of two consecutive exchanges (use two areas in turn, or other buffers in
// between).
// No load ever targets a peer's memory, nothing here uses multicast, and the only wait is bounded: when it gives up
// it records status 32 + (rank it waited for), readable through jq_device_status, and the kernel returns.
#include <cstring>

#include "jq_common.cuh"

namespace jq {

static __device__ int g_peer_status;

namespace {

constexpr int PEER_MAX_WORLD = 8;
constexpr int PEER_FLAG_BYTES = 256;
constexpr int PEER_COUNTER_WORD = 16;
constexpr int PEER_SEQ_WORD = 17;
constexpr unsigned PEER_POLL_LIMIT = 1u << 22;  // polls of about 100 ns each: gives up after roughly half a second

struct PeerTargets {
    float* y[PEER_MAX_WORLD];         // every rank's full y [m, n_total] (own included)
    uint32_t* flags[PEER_MAX_WORLD];  // every rank's flag words
};

// slice [m, n_slice] -> columns col0 .. of every rank's y [m, n_total]; the CTA that finishes last raises the flags.
__global__ void __launch_bounds__(256) peer_scatter_kernel(const float* __restrict__ slice, int64_t m, int64_t n_slice, int64_t n_total, int64_t col0,
                                                           PeerTargets tg, int rank, int world) {
    __shared__ int last_flag;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int64_t count = m * n_slice;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / n_slice, col = i % n_slice;
        const float val = slice[i];
        for (int r = 0; r < world; r++) {
            tg.y[r][row * n_total + col0 + col] = val;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* counter = reinterpret_cast<int*>(tg.flags[rank] + PEER_COUNTER_WORD);
        const int done = atomicAdd(counter, 1);
        last_flag = done == (int)gridDim.x - 1;
        if (last_flag) {
            *counter = 0;
        }
    }
    __syncthreads();
    if (last_flag && (int)threadIdx.x < world) {
        const uint32_t seq = tg.flags[rank][PEER_SEQ_WORD] + 1u;  // this exchange's number
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(tg.flags[threadIdx.x] + rank), "r"(seq) : "memory");
        __syncwarp();
        if (threadIdx.x == 0) {
            tg.flags[rank][PEER_SEQ_WORD] = seq;
        }
    }
}

// Thread r waits until rank r's slice of this rank's latest exchange has arrived in this rank's y.
__global__ void peer_wait_kernel(const uint32_t* flags, int world) {
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the scatter kernel before this one has advanced the number
    const int r = threadIdx.x;
    if (r >= world) {
        return;
    }
    const uint32_t seq = *reinterpret_cast<const volatile uint32_t*>(flags + PEER_SEQ_WORD);
    for (unsigned poll = 0; poll < PEER_POLL_LIMIT; poll++) {
        uint32_t seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flags + r) : "memory");
        if ((int32_t)(seen - seq) >= 0) {
            return;
        }
        __nanosleep(100);
    }
    atomicCAS(&g_peer_status, 0, 32 + r);
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
    cudaError_t e = cudaFree(ptr);
    return e == cudaSuccess ? JQ_OK : cuda_fail(e, "jq_peer_free");
}

JQ_API int64_t jq_peer_payload_offset(void) { return PEER_FLAG_BYTES; }

JQ_API int jq_peer_gather(const float* slice, int64_t m, int64_t n_slice, int64_t n_total, int64_t col0, void* const* peer_buffers, int64_t payload_offset,
                          int rank, int world, void* stream) {
    if (slice == nullptr || peer_buffers == nullptr || world < 1 || world > PEER_MAX_WORLD || rank < 0 || rank >= world || m < 1 || n_slice < 0 ||
        col0 < 0 || col0 + n_slice > n_total || payload_offset < 0 || payload_offset % 16 != 0) {
        return fail(JQ_ERR_INVALID, "jq_peer_gather: rank %d of %d, slice [%lld, %lld] at column %lld of %lld", rank, world, (long long)m, (long long)n_slice,
                    (long long)col0, (long long)n_total);
    }
    PeerTargets tg;
    for (int r = 0; r < PEER_MAX_WORLD; r++) {
        uint8_t* base = r < world ? static_cast<uint8_t*>(peer_buffers[r]) : nullptr;
        if (r < world && base == nullptr) {
            return fail(JQ_ERR_INVALID, "jq_peer_gather: the buffer of rank %d is null", r);
        }
        tg.flags[r] = reinterpret_cast<uint32_t*>(base);
        tg.y[r] = base != nullptr ? reinterpret_cast<float*>(base + PEER_FLAG_BYTES + payload_offset) : nullptr;
    }
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t count = m * n_slice;
    int grid = (int)((count + 255) / 256);
    grid = grid < 1 ? 1 : (grid > 148 ? 148 : grid);
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.stream = s;
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(256);
    JQ_CUDA(cudaLaunchKernelEx(&cfg, peer_scatter_kernel, slice, m, n_slice, n_total, col0, tg, rank, world));
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    JQ_CUDA(cudaLaunchKernelEx(&cfg, peer_wait_kernel, (const uint32_t*)tg.flags[rank], world));
    count_launch(2);
    return JQ_OK;
}

}  // extern "C"
