// NOT COMPILED: no JDK exists in the environment this library was built in. Source for a jitNN maintainer.
package ai.beestream.jitnn.natives;

import java.util.Map;
import java.util.Set;
import java.util.TreeSet;
import java.util.concurrent.ConcurrentHashMap;

/**
 * Decides, once per process and function, whether an operator of the quantised-linear path calls libjitnn_b200 or keeps
 * jitNN's own kernels: the same contract as engine/Native.java:129-153 (requested, probed once, a failure falls back to
 * jitNN's kernels with one line on stderr) and engine/Native.java:208-216 (a function that fails on first use is disabled
 * unless it has already run successfully).
 *
 * Switch: -Djitnn.b200=true (off by default); library path: -Djitnn.b200.lib=/path/to/libjitnn_b200.so.
 */
public final class B200Gate {
    /** The functions an operator can route to the library. */
    public enum Function { LINEAR, LINEAR_BF16, DEQUANTIZE, QUANTIZE_Q8, LINEAR_BACKWARD, DECODER }

    private static final boolean REQUESTED = Boolean.getBoolean("jitnn.b200");
    private static final Map<Function, Boolean> AVAILABLE = new ConcurrentHashMap<>();
    private static final Set<Function> DISABLED = ConcurrentHashMap.newKeySet();
    private static final Set<Function> PROVEN = ConcurrentHashMap.newKeySet();
    private static volatile Boolean library;  // null: not probed yet

    private B200Gate() {
    }

    public static boolean requested() {
        return REQUESTED;
    }

    /** True when `fn` should run on the library: requested, the library loads, a GPU answers, and fn has not been disabled. */
    public static boolean use(Function fn) {
        if (!REQUESTED || DISABLED.contains(fn)) {
            return false;
        }
        return AVAILABLE.computeIfAbsent(fn, f -> probeLibrary());
    }

    private static synchronized boolean probeLibrary() {
        if (library == null) {
            String why = null;
            try {
                if (B200Quant.deviceCount() < 1) {
                    why = "no CUDA device";
                }
            } catch (LinkageError | RuntimeException ex) {
                why = ex.getClass().getSimpleName() + ": " + ex.getMessage();
            }
            library = why == null;
            if (why != null) {
                System.err.printf("[jitnn] native b200: not available (%s); using jitNN kernels%n", why);
            }
        }
        return library;
    }

    /** An operator's first call through `features` failed: stop using those that have not run successfully elsewhere. */
    public static void disable(Set<Function> features, Throwable cause) {
        Set<Function> suspects = new TreeSet<>(features);
        suspects.removeAll(PROVEN);
        if (suspects.isEmpty()) {
            suspects.addAll(features);
        }
        DISABLED.addAll(suspects);
        System.err.printf("[jitnn] native b200 %s failed (%s); using jitNN kernels instead%n", suspects, cause.getMessage());
    }

    /** A call through `features` ran: they work on this machine. */
    public static void proven(Set<Function> features) {
        PROVEN.addAll(features);
    }

    /**
     * The body of an operator's {@code cpu(Node)} hook (engine/Op.java:46-55): runs `call` if the gate is open and reports
     * whether the outputs were written. A failure disables the function and returns false before anything was written by
     * the caller's contract (the library writes y only on success), so the CPU backend runs the operator's reference().
     */
    public static boolean run(Function fn, Runnable call) {
        if (!use(fn)) {
            return false;
        }
        try {
            call.run();
            proven(Set.of(fn));
            return true;
        } catch (IllegalArgumentException ex) {
            throw ex;  // a shape or format error is the caller's, with the reference's wording: not a reason to fall back
        } catch (RuntimeException | LinkageError ex) {
            disable(Set.of(fn), ex);
            return false;
        }
    }
}
