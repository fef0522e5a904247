package com.omega.engine.nn.layer.llama;

import com.omega.common.lib.LibPaths;

/**
 * JNI binding of libomoe.so (C ABI in include/omoe.h).  Device buffers cross the
 * boundary as raw 64-bit addresses; every call returns 0 or a negative
 * OMOE_ERR_* code.  The shim library (jni/omoe_jni.c) only forwards to the C ABI.
 *
 * Not compiled in the repository that ships it: that build image has no JDK.
 */
public final class OmoeNative {

    public static final int F32 = 0;
    public static final int BF16 = 1;

    static {
        // same loading idiom as com.omega.engine.gpu.JNITest: an absolute path next to the kernels
        System.load(LibPaths.getLibPath() + "libomoe_jni.so");
    }

    private OmoeNative() {
    }

    /** @return handle, or 0 on failure (see lastError(0)) */
    public static native long create(int tMax, int dModel, int dFf, int nExperts, int topK, int computeDtype,
                                     int renormalize, int hasRouterBias, int world, int rank, int recvRowsMax);

    public static native int destroy(long handle);

    public static native String lastError(long handle);

    /** All pointers are device addresses; routerBias may be 0. */
    public static native int setWeights(long handle, long wRouter, long routerBias, long wGate, long wUp,
                                        long wDown, int srcDtype);

    /** Enqueues on the legacy default stream, like every kernel launch of the engine. */
    public static native int forward(long handle, long xDev, long yDev, int tokens, int ioDtype);

    /** Host arrays in and out: H2D, forward, D2H, synchronise. */
    public static native int forwardHost(long handle, float[] x, float[] y, int tokens);

    /** omoe_forward_host_async: the same without the final synchronise; the arrays are pinned by the JVM until
     *  waitDone() has returned, so they must stay reachable and untouched until then. */
    public static native int forwardHostAsync(long handle, float[] x, float[] y, int tokens);

    /** omoe_wait: host waits for everything enqueued on the handle; reports a device-side failure. */
    public static native int waitDone(long handle);

    /** omoe_forward_block: y = x + MoE(rmsnorm(x) * gamma); gammaDev is the fp32 device address of RMSLayer's gamma. */
    public static native int forwardBlock(long handle, long xDev, long gammaDev, float eps, long yDev, int tokens,
                                          int ioDtype);

    public static native int getRouting(long handle, int[] topkIdx, float[] topkW, int[] counts, int[] offsets,
                                        int[] perm);

    /** omoe_set_training: forwards keep what the backward pass needs. */
    public static native int setTraining(long handle, int on);

    /** omoe_backward: device addresses of the forward's input, of delta and of diff (all [tokens, d_model]). */
    public static native int backward(long handle, long xDev, long dyDev, long dxDev, int tokens, int ioDtype);

    /** omoe_get_weight_grads: fp32 device addresses (0 = skip): router [E,d], bias [E], gate/up [E,dff,d], down [E,d,dff]. */
    public static native int getWeightGrads(long handle, long dRouter, long dBias, long dGate, long dUp, long dDown);

    /** omoe_ep_connect_local: all ranks' handles of this JVM, in rank order (one per device, DP.java:68-94). */
    public static native int epConnectLocal(long[] handles);

    public static native int epExport(long handle, byte[] blob320);

    public static native int epImport(long handle, byte[] allBlobs);
}
