package com.omega.engine.nn.layer.llama;

import com.omega.engine.nn.layer.FullyLayer;
import com.omega.engine.nn.layer.Layer;
import com.omega.engine.nn.layer.LayerType;
import com.omega.engine.nn.network.Network;
import com.omega.engine.tensor.Tensor;
import jcuda.Pointer;
import jcuda.Sizeof;
import jcuda.runtime.JCuda;
import jcuda.runtime.cudaMemcpyKind;

import java.io.IOException;
import java.io.RandomAccessFile;

/**
 * Mixture-of-experts feed-forward layer: router -> top-k -> dispatch -> grouped
 * SwiGLU experts -> gate-weighted combine, executed by libomoe.so on sm_100a.
 *
 * Takes the slot of LlamaMLPLayer in LlamaTransformerBlock (constructed at
 * LlamaTransformerBlock.java:97, called at :135) and keeps its surface:
 * forward(Tensor) = setInput; init(); output(), result via getOutput().
 *
 * Weights live in FullyLayer objects so the engine's bookkeeping (paramLayers,
 * updaters, save/load, gradient clipping) keeps working: router [E,d] and per
 * expert gate=linear1 [dff,d], up=linear3 [dff,d], down=linear2 [d,dff], the
 * [out,in] layout of FullyLayer.  The native library keeps its own bf16 copies;
 * call syncWeights() after the weights change.
 *
 * Training: setTraining(true) once, then back(delta) runs the native backward and
 * hands every FullyLayer its diffW; update() lets their updaters change the weights
 * and re-syncs the native copies.  Not compiled in the repository that ships it (no
 * JDK in that build image).
 */
public class MoELayer extends Layer {

    private final int embedDim;
    private final int dff;
    private final int numExperts;
    private final int topK;
    private final boolean bias;
    private final int tMax;
    private final int computeDtype;

    private FullyLayer router;
    private FullyLayer[] gate;   // linear1 of each expert
    private FullyLayer[] up;     // linear3
    private FullyLayer[] down;   // linear2

    private long handle;
    // experts packed contiguously for omoe_set_weights: [E,dff,d], [E,dff,d], [E,d,dff]
    private Tensor packedGate, packedUp, packedDown;
    // network.train_time at the last syncWeights(): an optimizer that walks the network's parameter list
    // (putParamters below) changes the FullyLayer weights without calling update() here, so the native copies
    // are refreshed at the start of the first forward after the network's step counter has moved
    private int syncedTrainTime = -1;

    public MoELayer(int embedDim, int dff, int numExperts, int topK, boolean bias, Network network) {
        this(embedDim, dff, numExperts, topK, bias, network, 16384, OmoeNative.BF16);
    }

    public MoELayer(int embedDim, int dff, int numExperts, int topK, boolean bias, Network network, int tMax,
                    int computeDtype) {
        this.network = network;
        this.embedDim = embedDim;
        this.dff = dff;
        this.numExperts = numExperts;
        this.topK = topK;
        this.bias = bias;
        this.tMax = tMax;
        this.computeDtype = computeDtype;
        this.oChannel = 1;
        this.oHeight = 1;
        this.oWidth = embedDim;
        this.router = new FullyLayer(embedDim, numExperts, bias, network);
        this.gate = new FullyLayer[numExperts];
        this.up = new FullyLayer[numExperts];
        this.down = new FullyLayer[numExperts];
        for (int e = 0; e < numExperts; e++) {
            gate[e] = new FullyLayer(embedDim, dff, false, network);
            up[e] = new FullyLayer(embedDim, dff, false, network);
            down[e] = new FullyLayer(dff, embedDim, false, network);
        }
        this.handle = OmoeNative.create(tMax, embedDim, dff, numExperts, topK, computeDtype, 1, bias ? 1 : 0, 1, 0, 0);
        if (handle == 0) {
            throw new RuntimeException("omoe_create: " + OmoeNative.lastError(0));
        }
        this.packedGate = new Tensor(numExperts, 1, dff, embedDim, true, true);
        this.packedUp = new Tensor(numExperts, 1, dff, embedDim, true, true);
        this.packedDown = new Tensor(numExperts, 1, embedDim, dff, true, true);
        syncWeights();
    }

    /** Exposes the raw device address of a JCuda pointer (getNativePointer is protected), the way the
     *  engine's own SerializablePointer does (parallel/ddp/distributed/SerializablePointer.java:26-28). */
    private static final class RawPointer extends Pointer {
        RawPointer(Pointer p) {
            super(p);
        }

        long address() {
            return getNativePointer();
        }
    }

    private static long addr(Pointer p) {
        return new RawPointer(p).address();
    }

    private static void copyInto(Tensor dst, long floatOffset, Tensor src) {
        JCuda.cudaMemcpy(dst.getGpuData().withByteOffset(floatOffset * Sizeof.FLOAT), src.getGpuData(),
                (long) src.dataLength * Sizeof.FLOAT, cudaMemcpyKind.cudaMemcpyDeviceToDevice);
    }

    /** Packs the experts' FullyLayer weights and hands them to the native library. */
    public void syncWeights() {
        for (int e = 0; e < numExperts; e++) {
            copyInto(packedGate, (long) e * dff * embedDim, gate[e].weight);
            copyInto(packedUp, (long) e * dff * embedDim, up[e].weight);
            copyInto(packedDown, (long) e * embedDim * dff, down[e].weight);
        }
        check(OmoeNative.setWeights(handle, addr(router.weight.getGpuData()),
                bias ? addr(router.bias.getGpuData()) : 0L, addr(packedGate.getGpuData()),
                addr(packedUp.getGpuData()), addr(packedDown.getGpuData()), OmoeNative.F32));
        syncedTrainTime = network != null ? network.train_time : 0;
    }

    /** Re-syncs the native weight copies when the network has taken a training step since the last sync. */
    private void syncWeightsIfStale() {
        if (network != null && network.train_time != syncedTrainTime) {
            syncWeights();
        }
    }

    /** Registers every weight with the network's parameter list, as LlamaMLPLayer.putParamters() does for its
     *  three linears (LlamaMLPLayer.java:285-289; FullyLayer.java:868-873); LlamaTransformerBlock.putParamters()
     *  calls this on its mlp (LlamaTransformerBlock.java:281). */
    public void putParamters() {
        router.putParamters();
        for (int e = 0; e < numExperts; e++) {
            gate[e].putParamters();
            up[e].putParamters();
            down[e].putParamters();
        }
    }

    /** The gradients in the same order (LlamaMLPLayer.java:291-295; FullyLayer.java:875-880). */
    public void putParamterGrads() {
        router.putParamterGrads();
        for (int e = 0; e < numExperts; e++) {
            gate[e].putParamterGrads();
            up[e].putParamterGrads();
            down[e].putParamterGrads();
        }
    }

    private void check(int rc) {
        if (rc != 0) {
            throw new RuntimeException("libomoe: " + OmoeNative.lastError(handle));
        }
    }

    @Override
    public void init() {
        this.number = this.input.number;
        if (this.output == null || this.number != this.output.number) {
            this.output = Tensor.createGPUTensor(this.output, number, oChannel, oHeight, oWidth, true);
        }
    }

    @Override
    public void output() {
        syncWeightsIfStale();
        // one native call; it enqueues on the legacy default stream and does not synchronise
        check(OmoeNative.forward(handle, addr(input.getGpuData()), addr(output.getGpuData()), number, OmoeNative.F32));
    }

    @Override
    public void forward(Tensor input) {
        this.setInput(input);
        this.init();
        this.output();
    }

    @Override
    public void forward() {
        this.setInput();
        this.init();
        this.output();
    }

    @Override
    public Tensor getOutput() {
        return output;
    }

    @Override
    public LayerType getLayerType() {
        return LayerType.feed_forward;
    }

    public void saveModel(RandomAccessFile outputStream) throws IOException {
        // router first, then per expert gate, up, down — the order LlamaMLPLayer uses for linear1, linear3, linear2
        router.saveModel(outputStream);
        for (int e = 0; e < numExperts; e++) {
            gate[e].saveModel(outputStream);
            up[e].saveModel(outputStream);
            down[e].saveModel(outputStream);
        }
    }

    public void loadModel(RandomAccessFile inputStream) throws IOException {
        router.loadModel(inputStream);
        for (int e = 0; e < numExperts; e++) {
            gate[e].loadModel(inputStream);
            up[e].loadModel(inputStream);
            down[e].loadModel(inputStream);
        }
        syncWeights();
    }

    public void close() {
        if (handle != 0) {
            OmoeNative.destroy(handle);
            handle = 0;
        }
    }

    // ---- training surface (LlamaMLPLayer.java:139-158, 182-237 is the pattern) ----
    private Tensor packedDGate, packedDUp, packedDDown;
    private boolean training;

    /** Switches the native layer to training mode (forwards keep g, u, h and the routing). */
    public void setTraining(boolean on) {
        check(OmoeNative.setTraining(handle, on ? 1 : 0));
        training = on;
    }

    @Override
    public void initBack() {
        if (this.diff == null || this.number != this.diff.number) {
            this.diff = new Tensor(number, 1, 1, embedDim, true, true);
        }
        if (packedDGate == null) {
            packedDGate = new Tensor(numExperts, 1, dff, embedDim, true, true);
            packedDUp = new Tensor(numExperts, 1, dff, embedDim, true, true);
            packedDDown = new Tensor(numExperts, 1, embedDim, dff, true, true);
            router.initBack();
            for (int e = 0; e < numExperts; e++) {
                gate[e].initBack();
                up[e].initBack();
                down[e].initBack();
            }
        }
    }

    @Override
    public void initParam() {
    }

    private static void copyFrom(Tensor dst, Tensor src, long floatOffset) {
        JCuda.cudaMemcpy(dst.getGpuData(), src.getGpuData().withByteOffset(floatOffset * Sizeof.FLOAT),
                (long) dst.dataLength * Sizeof.FLOAT, cudaMemcpyKind.cudaMemcpyDeviceToDevice);
    }

    /** One native call computes diff and every diffW; the packed gradients are then handed to the FullyLayers
     *  whose updaters the network already walks (FullyLayer.java:57-70, 292-301). */
    @Override
    public void diff() {
        if (!training) {
            throw new IllegalStateException("MoELayer: call setTraining(true) before the forward of a training step");
        }
        check(OmoeNative.backward(handle, addr(input.getGpuData()), addr(delta.getGpuData()), addr(diff.getGpuData()),
                number, OmoeNative.F32));
        check(OmoeNative.getWeightGrads(handle, addr(router.diffW.getGpuData()),
                bias ? addr(router.diffB.getGpuData()) : 0L, addr(packedDGate.getGpuData()),
                addr(packedDUp.getGpuData()), addr(packedDDown.getGpuData())));
        for (int e = 0; e < numExperts; e++) {
            copyFrom(gate[e].diffW, packedDGate, (long) e * dff * embedDim);
            copyFrom(up[e].diffW, packedDUp, (long) e * dff * embedDim);
            copyFrom(down[e].diffW, packedDDown, (long) e * embedDim * dff);
        }
    }

    @Override
    public void back() {
        this.initBack();
        this.setDelta();
        this.diff();
    }

    @Override
    public void back(Tensor delta) {
        this.initBack();
        this.setDelta(delta);
        this.diff();
    }

    @Override
    public void backTemp() {
    }

    /** The FullyLayers' own updaters change the weights; the native copies follow. */
    @Override
    public void update() {
        router.update();
        for (int e = 0; e < numExperts; e++) {
            gate[e].update();
            up[e].update();
            down[e].update();
        }
        syncWeights();
    }

    @Override
    public void accGrad(float scale) {
        router.accGrad(scale);
        for (int e = 0; e < numExperts; e++) {
            gate[e].accGrad(scale);
            up[e].accGrad(scale);
            down[e].accGrad(scale);
        }
    }

    @Override
    public void showDiff() {
    }

    @Override
    public float[][][][] output(float[][][][] input) {
        return null;
    }

    @Override
    public void initCache() {
    }
}
