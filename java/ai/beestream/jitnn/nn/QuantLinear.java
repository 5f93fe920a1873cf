// NOT COMPILED: no JDK exists in the environment this library was built in. Source for a jitNN maintainer.
package ai.beestream.jitnn.nn;

import ai.beestream.jitnn.F;
import ai.beestream.jitnn.Tensor;

/**
 * A linear layer whose weight stays in its GGUF block format: the counterpart of nn/Linear.java:56-58 (forward =
 * F.linear(x, weight, bias)) for a quantised weight, so that a Llama built from jitnn-nn's modules can hold the tensors of
 * a GGUF file as they are. forward goes through Gguf.linear (ops/Gguf.java:76-98), whose MatVec / LinearQ8 operators
 * carry a cpu(Node) hook (engine/Op.java:46-55) that asks B200Gate; with -Djitnn.b200=true that hook runs libjitnn_b200, otherwise
 * jitNN's own kernels, with the same results within the operator's tolerance.
 *
 * The weight takes no gradient (a quantised tensor is a constant of the graph, ops/Gguf.java:208-212); the input does.
 */
public final class QuantLinear extends Module {
    private final Tensor weight;  // Tensor.quantized(type, blocks, out, in), persistent
    private final Tensor bias;    // FP32 [out] or null

    /** weight: a quantised tensor [out, in] (Tensor.quantized, Tensor.java:249-278); bias: FP32 [out] or null. */
    public QuantLinear(Tensor weight, Tensor bias) {
        if (!weight.dtype().isQuantized() || weight.rank() != 2) {
            throw new IllegalArgumentException("QuantLinear needs a quantised [out, in] weight, got " + weight);
        }
        if (bias != null && (bias.rank() != 1 || bias.dim(0) != weight.dim(0))) {
            throw new IllegalArgumentException("QuantLinear bias " + bias + " does not match weight " + weight);
        }
        this.weight = weight;
        this.bias = bias == null ? null : parameter(bias);
    }

    public Tensor weight() {
        return weight;
    }

    public Tensor bias() {
        return bias;
    }

    @Override
    public Tensor forward(Tensor x) {
        return F.linear(x, weight, bias);  // F.linear sends a quantised weight to Gguf.linear / Quant.linear (F.java:1048-1051)
    }
}
