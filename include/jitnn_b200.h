/*
 * jitnn_b200 — C ABI of the B200 (sm_100a) quantised linear operator for GGUF block formats.
 *
 * This is the boundary a jitNN backend binds through the Panama FFM API (java.lang.foreign), in the
 * style of the reference's own native binding jitnn-core/.../cpu/Blas.java:85-104,177-201: plain C
 * symbols, scalars and pointers only, no callbacks, no structs by value. Every function returns
 * JQ_OK (0) or a negative JQ_ERR_* code; the message of the last failure on the calling thread is
 * available from jq_last_error(). Nothing here aborts the process or throws.
 *
 * Citations name the reference interface each entry point stands in for; paths are relative to
 * jitnn-core/src/main/java/ai/beestream/jitnn/ unless they start with another module's name.
 */
#ifndef JITNN_B200_H
#define JITNN_B200_H

#include <stdint.h>

#if defined(__GNUC__)
#define JQ_API __attribute__((visibility("default")))
#else
#define JQ_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------------- */
#define JQ_OK 0
#define JQ_ERR_INVALID (-1)     /* shape, type, alignment or handle misuse (Java: IllegalArgumentException) */
#define JQ_ERR_OOM (-2)         /* device or pinned-host allocation failed */
#define JQ_ERR_CUDA (-3)        /* a CUDA runtime call or kernel launch failed (Java: JitnnException) */
#define JQ_ERR_NCCL (-4)        /* reserved for collective failures reported by the host side */
#define JQ_ERR_TIMEOUT (-5)     /* a bounded device-side wait gave up */
#define JQ_ERR_UNSUPPORTED (-6) /* the format has no kernel for this operation */

/* ---- weight element types: ggml type ids (jitnn-gguf/.../gguf/GgmlType.java:27-51) ---------- */
#define JQ_TYPE_Q4_0 2
#define JQ_TYPE_Q4_1 3
#define JQ_TYPE_Q5_0 6
#define JQ_TYPE_Q5_1 7
#define JQ_TYPE_Q8_0 8
#define JQ_TYPE_Q2_K 10
#define JQ_TYPE_Q3_K 11
#define JQ_TYPE_Q4_K 12
#define JQ_TYPE_Q5_K 13
#define JQ_TYPE_Q6_K 14

/* ---- where a data pointer lives ------------------------------------------------------------ */
#define JQ_MEM_HOST 0   /* host memory (pageable or pinned); the call copies in, computes, copies out and
                           returns when y is complete */
#define JQ_MEM_DEVICE 1 /* device memory of the weight's GPU; the call only enqueues work on `stream` */

/* ---- device layouts of an uploaded weight --------------------------------------------------- */
#define JQ_LAYOUT_AUTO 0 /* the library's layout for the format: Q4_K and Q5_K blocks stay verbatim (their
                            144/176-byte blocks are 16-byte multiples); Q8_0, Q4_0, Q4_1 and Q6_K are split
                            into a 16-byte aligned plane of quants and a plane of fp16 scales */

typedef struct jq_weight jq_weight; /* opaque; immutable after upload, safe to share between threads */

/* Library version: major * 10000 + minor * 100 + patch. */
JQ_API int jq_version(void);

/* Message of the last error on the calling thread ("" if none). The pointer stays valid until the
 * next failing call on the same thread. (Java side: the message of the exception to throw.) */
JQ_API const char* jq_last_error(void);

/* Values per block and bytes per block of a format, 0 for an unknown type (DType.java:75-98). */
JQ_API int jq_block_values(int type);
JQ_API int jq_block_bytes(int type);

/* Number of CUDA devices visible to the process. */
JQ_API int jq_device_count(int* count);

/*
 * Uploads the raw blocks of a [n, k] weight (row r occupies bytes [r*k/QK*B, (r+1)*k/QK*B), exactly
 * as a GGUF file stores it) to `device`. Stands in for Tensor.quantized(DType, byte[], dims...)
 * (Tensor.java:249-278) plus the first-use upload of a persistent tensor
 * (engine/PlanCompiler.java:209,240). Validates k % QK == 0 and nbytes == n*k/QK*B as
 * Tensor.persistent does. The blocks are copied during the call; the caller's buffer (for example a
 * memory-mapped GGUF region, jitnn-gguf/.../GgufFile.java:382-402) is not retained.
 */
JQ_API int jq_weight_upload(int device, int type, const void* host_blocks, int64_t nbytes, int64_t n, int64_t k,
                     int layout, jq_weight** out);

/*
 * As jq_weight_upload for the output rows [row_begin, row_end) only: the shard one GPU holds when a
 * linear is split by output rows. `host_blocks`/`nbytes` still describe the whole [n, k] weight. The
 * resulting handle is a [row_end - row_begin, k] weight. (No counterpart in the reference, which
 * never shards a linear; the collective that completes it mirrors dist/Collective.java:64-65.)
 */
JQ_API int jq_weight_upload_rows(int device, int type, const void* host_blocks, int64_t nbytes, int64_t n, int64_t k,
                          int64_t row_begin, int64_t row_end, int layout, jq_weight** out);

/* Releases the device memory of a weight (Tensor.release/close, Tensor.java:362-370). NULL is a no-op. */
JQ_API int jq_weight_free(jq_weight* w);

/* info[0..7] = n, k, type, layout, device, bytes held on the device, QK, block bytes. */
JQ_API int jq_weight_info(const jq_weight* w, int64_t info[8]);

/* Copies the weight back to the host in its original GGUF block bytes (n*k/QK*B of them): undoes any
 * device repacking. For tests and for saving what was loaded. */
JQ_API int jq_weight_download(const jq_weight* w, void* host_blocks, int64_t nbytes);

/*
 * dst[n*k] = dequantised weight in float32, bit-exact with the reference's per-element decode
 * (kernels/GgufKernels.java:85-223 `value`; Q8_0: ops/Quant.java:137-144). Stands in for
 * Gguf.dequantize / Quant.dequantize (ops/Gguf.java:68-73, ops/Quant.java:52-60).
 */
JQ_API int jq_dequantize(const jq_weight* w, float* dst, int dst_mem, void* stream);

/*
 * y[m, n] = x[m, k] * W^T (+ bias[n]), float32 activations and outputs. The reference never quantises
 * activations to a block format and neither does this: the decode kernels of the K-quant and 32-block formats
 * multiply the integer quants exactly with x held as 22-bit fixed point per 256-element super-block of k (relative
 * to the super-block's largest magnitude: a rounding of at most 2^-22 of that magnitude per element, the order of
 * FP32's own), and add the super-blocks' results up in FP32 in k order; measured against the double-precision
 * reference arithmetic the error stays below 1e-6 of the largest output. An x that holds a NaN or an Inf gives
 * non-finite outputs (Q4_K, Q5_K: NaN in every output of that row of x). Stands in for Gguf.linear(x, w, bias) (ops/Gguf.java:76-98) and
 * Quant.linear / F.linearQ8 (ops/Quant.java:66-80): any m >= 0 (leading axes of x flattened by the
 * caller as ops/Gguf.java:86-93 does), bias may be NULL. Rows are dispatched like the reference
 * dispatches them (ops/Gguf.java:90): m <= 16 to the fused dequantise-GEMV kernels, larger m in
 * groups of up to 16 rows through the same kernels unless the tensor-core prefill path is selected with
 * jq_set_option. `mem` says where x, bias and y live (all three alike); with JQ_MEM_DEVICE they must
 * be 16-byte aligned and `stream` is the CUDA stream (cudaStream_t, NULL = default stream).
 */
JQ_API int jq_linear_f32(const jq_weight* w, const float* x, int64_t m, const float* bias, float* y, int mem,
                  void* stream);

/*
 * Prefill form: x is bfloat16 [m, k] (raw 16-bit patterns), y float32 [m, n]; dequantised weights are
 * rounded to bfloat16 and multiplied on the tensor cores (tcgen05) with FP32 accumulation. Semantics of the
 * reference's prefill composition dequantize + matmul (ops/Gguf.java:94-95,
 * ops/MatMul.java:597-625) at bfloat16 operand precision. k must be a multiple of 64; any m works, the
 * kernel is built for m >= 128.
 */
JQ_API int jq_linear_bf16(const jq_weight* w, const uint16_t* x_bf16, int64_t m, const float* bias, float* y, int mem,
                   void* stream);

/*
 * Input gradient of the linear: gx[m, k] = g[m, n] . dequant(W), float32 (the backward of Gguf.linear and Quant.linear,
 * ops/Gguf.java:208-212 and ops/Quant.java:191-197: the quantised weight gets no gradient, the bias gradient is the
 * column sum of g and needs no weight). The weight is read once per four (Q6_K: one, 4-bit formats: two) rows of g, in
 * its quantised form, with FP32 accumulation (the reference accumulates in double; results agree within 1e-3 relative).
 * `mem` as for jq_linear_f32; device pointers must be 16-byte aligned.
 */
JQ_API int jq_linear_backward_f32(const jq_weight* w, const float* g, int64_t m, float* gx, int mem, void* stream);

/*
 * Waits for the work enqueued on `device` and reports, then clears, the status word of its kernels: 0, or the code of
 * the first bounded device-side wait that gave up (the prefill kernel's barrier waits are bounded instead of being
 * able to hang). Calls with host memory check this themselves and return JQ_ERR_TIMEOUT; callers that enqueue with
 * device memory can poll it at a synchronisation point of their own. (No counterpart in the reference.)
 */
JQ_API int jq_device_status(int device, int* status);

/*
 * Row-sharded linears over the GPUs of one box (one process per GPU): instead of Collective.allGather
 * (dist/Collective.java:64-65, NCCL form dist/NcclOp.java:184-198) every rank stores its slice of y directly into every
 * rank's buffer over NVLink, each value as one 8-byte word {value, number of the exchange} in the rank's staging area; the
 * same kernel then collects the other ranks' slices from its own staging area into its y, polling each word (bounded)
 * until it carries the number of this exchange. No fence and no atomic crosses NVLink, and the call's kernel ends when this
 * rank's y is complete. (No counterpart in the reference, which never shards a linear.)
 *
 * jq_peer_alloc    a buffer on `device` for `payload_bytes` of gathered outputs (plus 4096 bytes of flags in front, at
 *                  jq_peer_payload_offset() the payload starts) and its 64-byte CUDA IPC handle, which the caller sends
 *                  to the other ranks' processes by whatever channel it has.
 * jq_peer_open     maps another rank's buffer into this process (peer access is enabled on first use); jq_peer_close
 *                  unmaps it; jq_peer_free releases a buffer made by jq_peer_alloc, after every rank has closed it.
 * jq_peer_gather   enqueues on `stream`: y_r[0..m, col0 .. col0 + n_slice) = slice [m, n_slice] for every rank r, where
 *                  y_r [m, n_total] FP32 starts `payload_offset` bytes (a multiple of 16) into the payload of
 *                  peer_buffers[r] (entry `rank` is this rank's own buffer, the others come from jq_peer_open, all in
 *                  rank order) and the staging words [m, n_total] x 8 bytes start `staging_offset` bytes (a multiple of 16)
 *                  into it, overlapping no y; the kernel ends when the slices of all `world` (at most 8) ranks have arrived
 *                  in this rank's y. All ranks must make the same exchanges on a buffer in the same order, and the same
 *                  (y, staging) area must not be the target of two exchanges in a row (alternate two areas, or use other
 *                  buffers in between): a rank may run one exchange ahead of another. A thread that has waited
 *                  "peer_wait_us" (option, default 400 000) in all leaves status 32 + r for jq_device_status, r being the
 *                  rank that owns the missing column when the n_total columns are split evenly, and the kernel returns
 *                  with that part of y unwritten. After such a timeout the ranks' exchange numbers on the buffers are out
 *                  of step: the buffers are to be released (jq_peer_close / jq_peer_free) and allocated anew before the
 *                  ranks exchange again. Works inside a captured CUDA graph (a captured call pins the library's per-stream
 *                  scratch buffers and the buffer's target-table slot it uses: neither is ever freed or reused).
 */
JQ_API int jq_peer_alloc(int device, int64_t payload_bytes, void** ptr, void* handle_out);
JQ_API int jq_peer_open(int device, const void* handle, void** ptr);
JQ_API int jq_peer_close(void* ptr);
JQ_API int jq_peer_free(void* ptr);
JQ_API int64_t jq_peer_payload_offset(void);
JQ_API int jq_peer_gather(const float* slice, int64_t m, int64_t n_slice, int64_t n_total, int64_t col0, void* const* peer_buffers,
                          int64_t payload_offset, int64_t staging_offset, int rank, int world, void* stream);
/*
 * The sharded linear in one call: y_r[0..m, col0 .. col0 + n_w) = x W_shard^T (+ bias) for every rank r, complete on
 * this rank when the call's last kernel ends, with w this rank's row shard (n_w rows, uploaded with
 * jq_weight_upload_rows), x [m, k] and bias [n_w] device pointers, and the buffers and offsets as for jq_peer_gather.
 * For Q4_K and Q5_K with m <= 8 the GEMV kernel itself stores into every rank's buffer and collects the other ranks'
 * rows (no slice buffer, no copy kernel); other formats and row counts run the ordinary kernels into a scratch slice
 * followed by the copy kernel.
 */
JQ_API int jq_linear_f32_peer(const jq_weight* w, const float* x, int64_t m, const float* bias, int64_t n_total, int64_t col0,
                              void* const* peer_buffers, int64_t payload_offset, int64_t staging_offset, int rank, int world, void* stream);

/*
 * blocks_out[count/32*34] = Q8_0 blocks of x[count] (count % 32 == 0), following the reference's host
 * quantiser ops/Quant.java:102-118 (F.quantizeQ8): d = (float)(max|x| / 127.0) stored as fp16, q =
 * x / d rounded half away from zero using the unrounded float d, clamped to [-127, 127].
 */
JQ_API int jq_quantize_q8_0(int device, const float* x, int64_t count, void* blocks_out, int mem, void* stream);

/*
 * Named integer options, the counterpart of the reference's jitnn.* configuration keys
 * (JitnnConfig.java:423-424 for this path). Known names:
 *   "prefill_min_rows"  rows of x from which jq_linear_f32 rounds x to bfloat16 and uses the
 *                       tensor-core prefill kernel (default 0 = never: FP32 results for every m).
 *   "gemv_generic"      non-zero: every decode GEMV runs on the generic CUDA-core kernel (for comparisons).
 *   "decoder_graph"     zero: the decoder issues its single-token step kernel by kernel instead of replaying a CUDA graph.
 *   "decoder_fused"     zero: the decoder's single-token step uses the general kernels (one per operator) instead of the
 *                       fused ones that hand activations to the next linear as its activation image.
 *   "gemv_tcgen05"      which Q4_K and Q5_K decode GEMVs run on the tcgen05 kernel (1 to 16 rows of x in one pass over the weights)
 *                       instead of the mma.sync one (up to 8 rows per pass). 0 (default): those where it is the faster of the
 *                       two, 11 or more rows of x on a weight of at least one 128-row tile per SM, and the shapes the mma.sync
 *                       kernel declines; 1: all; 2: none.
 *   "wait_limit_us"     microseconds after which a bounded device-side wait of the tcgen05 GEMV gives up (default 2 000 000; a
 *                       wait that gives up makes jq_device_status report 64 + the waiting role, and the outputs of that call
 *                       are undefined).
 */
JQ_API int jq_set_option(const char* name, int64_t value);
JQ_API int jq_get_option(const char* name, int64_t* value);

/*
 * y[m, n] = x[m, k] * W^T (+ bias[n]) for a Q4_K weight, 1 <= m <= 8, device pointers only (16-byte aligned),
 * enqueued on `stream`: the same kernels and bit for bit the same results as jq_linear_f32, but the call allocates
 * no memory. It has no counterpart in the reference. jq_linear_f32 keeps its intermediate "activation image" in a
 * buffer it allocates with cudaMalloc when a stream first needs one; this entry point is for callers that
 * cannot have that happen: a process that has already given all device memory to its own pools (the allocation
 * would fail), or a latency-bound loop that must not meet cudaMalloc's device-wide wait. Here the image lives
 * in a 1 MiB array that is part of the library itself, so every GPU that loads the library holds that 1 MiB
 * until the process exits. Limits: the image, (k / 256) * 928 bytes for one row, 1856 for two and 7008 for three to
 * eight rows, must fit 1 MiB (for example k <= 38144 at eight rows); anything larger and any other row count is
 * refused with JQ_ERR_INVALID, any other format, and a shape whose carried sums do not fit the kernel's shared
 * memory (which jq_linear_f32 would hand to its generic kernel), with JQ_ERR_UNSUPPORTED, all with a message.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device
 * current); make that first call before starting any stream capture. All calls share the one array, which keeps
 * whatever the last call left in it; every call rewrites the part it reads, nothing has to start at zero.
 * Two calls that overlap on the GPU (different streams, or different host threads without ordering) race on it:
 * serialise them.
 */
JQ_API int jq_linear_q4k_f32_noalloc(const jq_weight* w, const float* x, int64_t m, const float* bias, float* y, void* stream);

/*
 * ---- Llama-style decoder over quantised linears -----------------------------------------------------------------
 * The block math of jitnn-nn/.../nn/models/Llama.java:167-222 (RMSNorm, rotate-half RoPE with base `rope_base`,
 * causal grouped-query attention with scale 1/sqrt(head_dim), SwiGLU, residual adds, final norm, output projection,
 * greedy argmax = first index of the maximum, ops/Reduce.java:201) with every nn.Linear replaced by jq_linear_f32 on
 * a quantised weight. The reference recomputes every position on each call and has no generation loop; the decoder
 * here keeps keys and values in a cache of `max_seq` positions, which computes the same function.
 * Linear slots of a layer: 0 wq, 1 wk, 2 wv, 3 wo, 4 w1 (gate), 5 w3 (up), 6 w2 (down); layer -1 slot 7 is the output
 * projection. Norm slots: 0 attention norm, 1 feed-forward norm; layer -1 is the final norm. Weights set with
 * jq_decoder_set_linear are borrowed: they must outlive the decoder. One forward call at a time per decoder.
 */
typedef struct jq_decoder jq_decoder;
JQ_API int jq_decoder_create(int device, int layers, int dim, int heads, int kv_heads, int hidden, int vocab, int max_seq, float eps,
                      float rope_base, jq_decoder** out);
JQ_API int jq_decoder_destroy(jq_decoder* d);
JQ_API int jq_decoder_set_linear(jq_decoder* d, int layer, int which, const jq_weight* w);
JQ_API int jq_decoder_set_norm(jq_decoder* d, int layer, int which, const float* host_weights);
JQ_API int jq_decoder_set_embedding(jq_decoder* d, const float* host_table);
/*
 * The decoder split over the GPUs of one box by output rows of every linear (one process and one decoder per GPU; the
 * reference never shards a model). jq_decoder_peer_bytes gives the payload size of the peer buffer a rank needs
 * (jq_peer_alloc); jq_decoder_set_shard, called before any linear is set, makes the decoder rank `rank` of `world`
 * (at most 8, dividing heads, kv_heads, hidden / 4 and vocab / 4) with peer_buffers[r] rank r's buffer (own at `rank`,
 * the others from jq_peer_open). From then on jq_decoder_set_linear expects this rank's rows of each weight (n / world
 * rows: whole heads of wq / wk / wv), norms and the embedding stay whole, and jq_decoder_forward must be called by all
 * ranks with the same tokens and positions. Every rank gets the full logits and the next token, bitwise those of the
 * unsharded decoder on its general kernels. A rank that stops calling makes the others' bounded waits give up:
 * their forward returns JQ_ERR_TIMEOUT when it next waits for the stream.
 */
JQ_API int jq_decoder_peer_bytes(const jq_decoder* d, int64_t* payload_bytes);
JQ_API int jq_decoder_set_shard(jq_decoder* d, int rank, int world, void* const* peer_buffers);
/* Runs n_tokens (1..16) consecutive tokens at positions pos0 .. pos0 + n_tokens - 1 and appends their keys and values to
 * the cache. logits_host (or NULL) receives float32 [n_tokens, vocab], next_host (or NULL) the greedy next token after
 * each of them; the call waits for `stream` when either is requested, otherwise it only enqueues work. With a NULL
 * stream the decoder uses a stream of its own. Single-token calls that ask for the next token (the decode step) are
 * captured into a CUDA graph on their second occurrence and replayed afterwards. */
JQ_API int jq_decoder_forward(jq_decoder* d, const int32_t* tokens_host, int n_tokens, int pos0, float* logits_host, int32_t* next_host,
                       void* stream);
/*
 * Several independent sequences in one decoder (batched decode; the reference has no generation loop):
 * jq_decoder_set_sequences gives the decoder key/value caches for `sequences` (1..16) sequences (what the caches held is
 * lost); jq_decoder_forward_seq is jq_decoder_forward on sequence `seq` (jq_decoder_forward works on sequence 0);
 * jq_decoder_forward_batch runs one token of each of the sequences 0 .. n_seqs - 1, all at position `pos`, as one pass
 * over the weights: logits_host [n_seqs, vocab], next_host [n_seqs]. Repeated batch steps of one size that ask for the
 * next tokens are captured into a CUDA graph like the single-token step.
 */
JQ_API int jq_decoder_set_sequences(jq_decoder* d, int sequences);
JQ_API int jq_decoder_forward_seq(jq_decoder* d, int seq, const int32_t* tokens_host, int n_tokens, int pos0, float* logits_host,
                                  int32_t* next_host, void* stream);
JQ_API int jq_decoder_forward_batch(jq_decoder* d, const int32_t* tokens_host, int n_seqs, int pos, float* logits_host, int32_t* next_host,
                                    void* stream);
/*
 * The prompt path: n_tokens (1..4096) consecutive tokens of sequence `seq` at positions pos0 .. in one pass over the
 * weights, their keys and values appended to the cache. Every linear runs on the tensor-core prefill kernel, which rounds
 * its input to bfloat16 (what jq_linear_bf16 computes; FP32 accumulation, everything else in FP32), so the results
 * agree with jq_decoder_forward's to about 1e-2 of the largest logit, not to FP32 precision: the caller chooses this
 * path, jq_decoder_forward never takes it by itself. Only the last token's logits are computed: logits_host (or NULL)
 * receives float32 [vocab], next_host (or NULL) the greedy token after the last one; the call waits for `stream` when
 * either is requested. Head sizes 64 and 128; not for the row-sharded decoder (JQ_ERR_UNSUPPORTED). The workspace
 * (activations of n_tokens rows) is allocated by the first call and grows with the longest run seen.
 * (The reference has no generation loop; the operators are those of models/Llama.java:192-222 on T rows.)
 */
JQ_API int jq_decoder_prompt(jq_decoder* d, int seq, const int32_t* tokens_host, int n_tokens, int pos0, float* logits_host, int32_t* next_host,
                             void* stream);

/*
 * GGUF file -> device weights (the reference's jitnn-gguf/.../GgufFile.java:100-175,329-418, whose GgufFile.tensor(name)
 * hands a tensor's block bytes to Tensor.persistent): the file is mapped read-only, header, metadata and tensor table are
 * parsed with every access bounds-checked, and a tensor's blocks go to the GPU straight from the mapping. GGUF versions 2
 * and 3, little-endian. Hostile input is an error (JQ_ERR_INVALID with a message naming the file), never a read past
 * the mapping: wrong magic, truncation, dimensions or offsets beyond 2^63, sizes that overflow, data outside the file or
 * off the general.alignment grid, arrays nested more than 8 deep (GgufFileTest.java:115-155).
 *
 * jq_gguf_tensor       name (valid until close), ggml type id, dimensions outermost first (dims[8], unused = 1), absolute
 *                      file offset and byte size (-1 for a type id whose block geometry is unknown) of tensor `index`.
 * jq_gguf_tensor_data  pointer to the tensor's bytes inside the mapping (valid until close).
 * jq_gguf_meta_*       metadata by key: value type (GGUF ids 0..12; arrays report length and element type), numbers as
 *                      double and exact int64, strings as pointer + length into the mapping (not NUL-terminated).
 * jq_gguf_upload       rows [row_begin, row_end) (row_end -1: all) of the 2-D tensor `index` as a jq_weight on `device`.
 */
typedef struct jq_gguf jq_gguf;
JQ_API int jq_gguf_open(const char* path, jq_gguf** out);
JQ_API int jq_gguf_close(jq_gguf* f);
JQ_API int jq_gguf_info(const jq_gguf* f, int* version, int64_t* alignment, int64_t* data_offset, int64_t* n_tensors, int64_t* n_meta);
JQ_API int jq_gguf_tensor(const jq_gguf* f, int64_t index, const char** name, int* ggml_type, int* n_dims, int64_t* dims, int64_t* offset,
                          int64_t* nbytes);
JQ_API int jq_gguf_find_tensor(const jq_gguf* f, const char* name, int64_t* index);
JQ_API int jq_gguf_tensor_data(const jq_gguf* f, int64_t index, const void** data);
JQ_API int jq_gguf_meta_find(const jq_gguf* f, const char* key, int* value_type, int64_t* array_len, int* elem_type);
JQ_API int jq_gguf_meta_number(const jq_gguf* f, const char* key, double* value, int64_t* integer);
JQ_API int jq_gguf_meta_string(const jq_gguf* f, const char* key, const char** bytes, int64_t* length);
JQ_API int jq_gguf_upload(const jq_gguf* f, int64_t index, int device, int64_t row_begin, int64_t row_end, jq_weight** out);

/* Pinned host memory for activations and results (faster and truly asynchronous copies). */
JQ_API int jq_host_alloc(void** ptr, int64_t nbytes);
JQ_API int jq_host_free(void* ptr);

/* Number of kernels this library has launched from the calling process since load (all threads). */
JQ_API int64_t jq_launch_count(void);

#ifdef __cplusplus
}
#endif

#endif /* JITNN_B200_H */
