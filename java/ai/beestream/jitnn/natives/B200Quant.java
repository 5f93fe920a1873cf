// NOT COMPILED: no JDK exists in the environment this library was built in. Source for a jitNN maintainer, written
// against the exports of include/jitnn_b200.h; the style (one static downcall handle per symbol, plain pointers and
// scalars) follows jitNN's own cpu/Blas.java:85-104,177-201.
package ai.beestream.jitnn.natives;

import java.lang.foreign.Arena;
import java.lang.foreign.FunctionDescriptor;
import java.lang.foreign.Linker;
import java.lang.foreign.MemorySegment;
import java.lang.foreign.SymbolLookup;
import java.lang.invoke.MethodHandle;

import static java.lang.foreign.ValueLayout.ADDRESS;
import static java.lang.foreign.ValueLayout.JAVA_FLOAT;
import static java.lang.foreign.ValueLayout.JAVA_INT;
import static java.lang.foreign.ValueLayout.JAVA_LONG;

/** Downcall handles for libjitnn_b200.so: weights, the quantised linear and its gradient, the decoder, the GGUF reader. */
public final class B200Quant {
    public static final int MEM_HOST = 0, MEM_DEVICE = 1;
    public static final int OK = 0, ERR_INVALID = -1, ERR_OOM = -2, ERR_CUDA = -3, ERR_TIMEOUT = -5, ERR_UNSUPPORTED = -6;

    private static final Linker LINKER = Linker.nativeLinker();
    private static SymbolLookup lib;

    /** Loads the library named by -Djitnn.b200.lib (default: libjitnn_b200.so on the loader's path). Throws if it is absent. */
    static synchronized SymbolLookup lib() {
        if (lib == null) {
            lib = SymbolLookup.libraryLookup(System.getProperty("jitnn.b200.lib", "libjitnn_b200.so"), Arena.global());
        }
        return lib;
    }

    private static MethodHandle h(String name, FunctionDescriptor fd) {
        return LINKER.downcallHandle(lib().find(name).orElseThrow(() -> new UnsatisfiedLinkError(name)), fd);
    }

    // ---- lazily bound handles: nothing is looked up before the gate (B200Gate) has decided to use the library
    private static final class H {
        static final MethodHandle LAST_ERROR = h("jq_last_error", FunctionDescriptor.of(ADDRESS));
        static final MethodHandle DEVICE_COUNT = h("jq_device_count", FunctionDescriptor.of(JAVA_INT, ADDRESS));
        static final MethodHandle DEVICE_STATUS = h("jq_device_status", FunctionDescriptor.of(JAVA_INT, JAVA_INT, ADDRESS));
        static final MethodHandle UPLOAD = h("jq_weight_upload",
            FunctionDescriptor.of(JAVA_INT, JAVA_INT, JAVA_INT, ADDRESS, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_INT, ADDRESS));
        static final MethodHandle UPLOAD_ROWS = h("jq_weight_upload_rows",
            FunctionDescriptor.of(JAVA_INT, JAVA_INT, JAVA_INT, ADDRESS, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_LONG, JAVA_INT, ADDRESS));
        static final MethodHandle FREE = h("jq_weight_free", FunctionDescriptor.of(JAVA_INT, ADDRESS));
        static final MethodHandle DEQUANTIZE = h("jq_dequantize", FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS, JAVA_INT, ADDRESS));
        static final MethodHandle LINEAR = h("jq_linear_f32",
            FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS, JAVA_LONG, ADDRESS, ADDRESS, JAVA_INT, ADDRESS));
        static final MethodHandle LINEAR_BF16 = h("jq_linear_bf16",
            FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS, JAVA_LONG, ADDRESS, ADDRESS, JAVA_INT, ADDRESS));
        static final MethodHandle LINEAR_BACKWARD = h("jq_linear_backward_f32",
            FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS, JAVA_LONG, ADDRESS, JAVA_INT, ADDRESS));
        static final MethodHandle QUANTIZE_Q8 = h("jq_quantize_q8_0",
            FunctionDescriptor.of(JAVA_INT, JAVA_INT, ADDRESS, JAVA_LONG, ADDRESS, JAVA_INT, ADDRESS));
        static final MethodHandle SET_OPTION = h("jq_set_option", FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_LONG));
        // decoder
        static final MethodHandle DEC_CREATE = h("jq_decoder_create",
            FunctionDescriptor.of(JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_FLOAT, JAVA_FLOAT, ADDRESS));
        static final MethodHandle DEC_SET_LINEAR = h("jq_decoder_set_linear", FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, JAVA_INT, ADDRESS));
        static final MethodHandle DEC_SET_NORM = h("jq_decoder_set_norm", FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, JAVA_INT, ADDRESS));
        static final MethodHandle DEC_SET_EMBEDDING = h("jq_decoder_set_embedding", FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS));
        static final MethodHandle DEC_FORWARD = h("jq_decoder_forward",
            FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS, ADDRESS));
        static final MethodHandle DEC_PROMPT = h("jq_decoder_prompt",
            FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, ADDRESS, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS, ADDRESS));
        static final MethodHandle DEC_DESTROY = h("jq_decoder_destroy", FunctionDescriptor.of(JAVA_INT, ADDRESS));
        // GGUF reader
        static final MethodHandle GGUF_OPEN = h("jq_gguf_open", FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS));
        static final MethodHandle GGUF_FIND = h("jq_gguf_find_tensor", FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS, ADDRESS));
        static final MethodHandle GGUF_UPLOAD = h("jq_gguf_upload",
            FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_LONG, JAVA_INT, JAVA_LONG, JAVA_LONG, ADDRESS));
        static final MethodHandle GGUF_CLOSE = h("jq_gguf_close", FunctionDescriptor.of(JAVA_INT, ADDRESS));
    }

    private B200Quant() {
    }

    /** Turns a status code into the exception the reference's operators throw for the same mistake. */
    static void check(int rc) {
        if (rc == OK) {
            return;
        }
        String msg;
        try {
            msg = ((MemorySegment) H.LAST_ERROR.invokeExact()).reinterpret(1024).getString(0);
        } catch (Throwable t) {
            msg = "libjitnn_b200 status " + rc;
        }
        if (rc == ERR_INVALID || rc == ERR_UNSUPPORTED) {
            throw new IllegalArgumentException(msg);  // Gguf.linear / Quant.linear throw this for shape and format errors
        }
        throw new IllegalStateException(msg);
    }

    private static int call(MethodHandle mh, Object... args) {
        try {
            return (int) mh.invokeWithArguments(args);
        } catch (RuntimeException | Error e) {
            throw e;
        } catch (Throwable t) {
            throw new IllegalStateException(t);
        }
    }

    /** GPUs the library sees; 0 without a driver. The gate's probe. */
    public static int deviceCount() {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment out = a.allocate(JAVA_INT);
            return call(H.DEVICE_COUNT, out) == OK ? out.get(JAVA_INT, 0) : 0;
        }
    }

    /** Tensor.quantized / first-use upload of a persistent tensor; `blocks` may be a mapped region of a GGUF file. */
    public static MemorySegment upload(int device, int ggmlType, MemorySegment blocks, long n, long k) {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment out = a.allocate(ADDRESS);
            check(call(H.UPLOAD, device, ggmlType, blocks, blocks.byteSize(), n, k, 0, out));
            return out.get(ADDRESS, 0);
        }
    }

    /** Rows [rowBegin, rowEnd) of the tensor only: one rank's shard of a linear split over several GPUs. */
    public static MemorySegment uploadRows(int device, int ggmlType, MemorySegment blocks, long n, long k, long rowBegin, long rowEnd) {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment out = a.allocate(ADDRESS);
            check(call(H.UPLOAD_ROWS, device, ggmlType, blocks, blocks.byteSize(), n, k, rowBegin, rowEnd, 0, out));
            return out.get(ADDRESS, 0);
        }
    }

    public static void free(MemorySegment weight) {
        check(call(H.FREE, weight));
    }

    /** Gguf.dequantize / Quant.dequantize into host floats [n * k]. */
    public static void dequantize(MemorySegment weight, MemorySegment out) {
        check(call(H.DEQUANTIZE, weight, out, MEM_HOST, MemorySegment.NULL));
    }

    /** Gguf.linear / Quant.linear on host arrays: x [m, k], bias [n] or NULL, y [m, n]; FP32 operands. */
    public static void linear(MemorySegment weight, MemorySegment x, long m, MemorySegment biasOrNull, MemorySegment y) {
        check(call(H.LINEAR, weight, x, m, biasOrNull, y, MEM_HOST, MemorySegment.NULL));
    }

    /** The same with bfloat16 activations (the GEMM composition for many rows, ops/Gguf.java:90-95). */
    public static void linearBf16(MemorySegment weight, MemorySegment xBf16, long m, MemorySegment biasOrNull, MemorySegment y) {
        check(call(H.LINEAR_BF16, weight, xBf16, m, biasOrNull, y, MEM_HOST, MemorySegment.NULL));
    }

    /** gx [m, k] = g [m, n] . dequant(W): the input gradient of Gguf.MatVec / Quant.LinearQ8. */
    public static void linearBackward(MemorySegment weight, MemorySegment g, long m, MemorySegment gx) {
        check(call(H.LINEAR_BACKWARD, weight, g, m, gx, MEM_HOST, MemorySegment.NULL));
    }

    /** F.quantizeQ8: Q8_0 blocks of x [count], count a multiple of 32. */
    public static void quantizeQ8(int device, MemorySegment x, long count, MemorySegment blocksOut) {
        check(call(H.QUANTIZE_Q8, device, x, count, blocksOut, MEM_HOST, MemorySegment.NULL));
    }

    public static void setOption(String name, long value) {
        try (Arena a = Arena.ofConfined()) {
            check(call(H.SET_OPTION, a.allocateFrom(name), value));
        }
    }

    // ---- decoder (jq_decoder_*): the block math of jitnn-nn's models/Llama.java:192-222 with a key/value cache
    public static MemorySegment decoderCreate(int device, int layers, int dim, int heads, int kvHeads, int hidden, int vocab, int maxSeq, float eps,
                                              float ropeBase) {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment out = a.allocate(ADDRESS);
            check(call(H.DEC_CREATE, device, layers, dim, heads, kvHeads, hidden, vocab, maxSeq, eps, ropeBase, out));
            return out.get(ADDRESS, 0);
        }
    }

    /** slot: 0 wq, 1 wk, 2 wv, 3 wo, 4 w1 (gate), 5 w3 (up), 6 w2 (down); layer -1 = the output projection. */
    public static void decoderSetLinear(MemorySegment dec, int layer, int slot, MemorySegment weight) {
        check(call(H.DEC_SET_LINEAR, dec, layer, slot, weight));
    }

    public static void decoderSetNorm(MemorySegment dec, int layer, int which, MemorySegment weights) {
        check(call(H.DEC_SET_NORM, dec, layer, which, weights));
    }

    public static void decoderSetEmbedding(MemorySegment dec, MemorySegment table) {
        check(call(H.DEC_SET_EMBEDDING, dec, table));
    }

    /** Up to 16 tokens at positions pos0..; logits [n, vocab] and / or the greedy next tokens [n] (either may be NULL). */
    public static void decoderForward(MemorySegment dec, MemorySegment tokens, int n, int pos0, MemorySegment logitsOrNull, MemorySegment nextOrNull) {
        check(call(H.DEC_FORWARD, dec, tokens, n, pos0, logitsOrNull, nextOrNull, MemorySegment.NULL));
    }

    /** A long prompt in one pass over the weights (bfloat16 operands); logits of the last token only. */
    public static void decoderPrompt(MemorySegment dec, int seq, MemorySegment tokens, int n, int pos0, MemorySegment lastLogitsOrNull,
                                     MemorySegment nextOrNull) {
        check(call(H.DEC_PROMPT, dec, seq, tokens, n, pos0, lastLogitsOrNull, nextOrNull, MemorySegment.NULL));
    }

    public static void decoderDestroy(MemorySegment dec) {
        check(call(H.DEC_DESTROY, dec));
    }

    // ---- the library's own GGUF reader, for hosts that do not go through jitnn-gguf's GgufFile
    public static MemorySegment ggufOpen(String path) {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment out = a.allocate(ADDRESS);
            check(call(H.GGUF_OPEN, a.allocateFrom(path), out));
            return out.get(ADDRESS, 0);
        }
    }

    public static long ggufFindTensor(MemorySegment file, String name) {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment out = a.allocate(JAVA_LONG);
            check(call(H.GGUF_FIND, file, a.allocateFrom(name), out));
            return out.get(JAVA_LONG, 0);
        }
    }

    /** Rows [rowBegin, rowEnd) of tensor `index` (rowEnd = -1: all) straight from the file mapping to the GPU. */
    public static MemorySegment ggufUpload(MemorySegment file, long index, int device, long rowBegin, long rowEnd) {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment out = a.allocate(ADDRESS);
            check(call(H.GGUF_UPLOAD, file, index, device, rowBegin, rowEnd, out));
            return out.get(ADDRESS, 0);
        }
    }

    public static void ggufClose(MemorySegment file) {
        check(call(H.GGUF_CLOSE, file));
    }
}
