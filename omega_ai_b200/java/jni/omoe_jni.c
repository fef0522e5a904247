/*
 * JNI shim for com.omega.engine.nn.layer.llama.OmoeNative: forwards each native
 * method to the C ABI of libomoe.so.  Naming follows the engine's own JNI
 * precedent (jni/com_omega_engine_gpu_JNITest.h: Java_<package>_<Class>_<method>).
 *
 * Build where a JDK exists:
 *   gcc -shared -fPIC -I"$JAVA_HOME/include" -I"$JAVA_HOME/include/linux" -I../../../include \
 *       omoe_jni.c -o libomoe_jni.so -L.. -lomoe -Wl,-rpath,'$ORIGIN'
 */
#if defined(__has_include)
#if __has_include(<jni.h>)
#define OMOE_HAVE_JNI 1
#endif
#endif

#ifdef OMOE_HAVE_JNI
#include <jni.h>
#include <string.h>

#include "omoe.h"

#define JFN(ret, name) JNIEXPORT ret JNICALL Java_com_omega_engine_nn_layer_llama_OmoeNative_##name

JFN(jlong, create)(JNIEnv *env, jclass c, jint tMax, jint d, jint dff, jint E, jint k, jint cdt, jint renorm,
                   jint hasBias, jint world, jint rank, jint recvRows) {
    omoe_config cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.t_max = tMax; cfg.d_model = d; cfg.d_ff = dff; cfg.n_experts = E; cfg.top_k = k;
    cfg.compute_dtype = cdt; cfg.renormalize = renorm; cfg.has_router_bias = hasBias;
    cfg.world = world; cfg.rank = rank; cfg.recv_rows_max = recvRows;
    omoe_handle *h = NULL;
    return omoe_create(&cfg, &h) == OMOE_OK ? (jlong)(intptr_t)h : 0;
}

JFN(jint, destroy)(JNIEnv *env, jclass c, jlong h) { return omoe_destroy((omoe_handle *)(intptr_t)h); }

JFN(jstring, lastError)(JNIEnv *env, jclass c, jlong h) {
    return (*env)->NewStringUTF(env, omoe_last_error((omoe_handle *)(intptr_t)h));
}

JFN(jint, setWeights)(JNIEnv *env, jclass c, jlong h, jlong wr, jlong rb, jlong wg, jlong wu, jlong wd, jint dt) {
    return omoe_set_weights((omoe_handle *)(intptr_t)h, (const void *)(intptr_t)wr, (const void *)(intptr_t)rb,
                            (const void *)(intptr_t)wg, (const void *)(intptr_t)wu, (const void *)(intptr_t)wd, dt,
                            NULL /* legacy default stream */);
}

JFN(jint, forward)(JNIEnv *env, jclass c, jlong h, jlong x, jlong y, jint T, jint io) {
    return omoe_forward((omoe_handle *)(intptr_t)h, (const void *)(intptr_t)x, (void *)(intptr_t)y, T, io, NULL);
}

JFN(jint, forwardHost)(JNIEnv *env, jclass c, jlong h, jfloatArray x, jfloatArray y, jint T) {
    jfloat *xp = (*env)->GetFloatArrayElements(env, x, NULL);
    jfloat *yp = (*env)->GetFloatArrayElements(env, y, NULL);
    int rc = omoe_forward_host((omoe_handle *)(intptr_t)h, xp, yp, T, OMOE_F32, NULL);
    (*env)->ReleaseFloatArrayElements(env, x, xp, JNI_ABORT);
    (*env)->ReleaseFloatArrayElements(env, y, yp, 0);
    return rc;
}

/* The arrays of an asynchronous call stay pinned (GetFloatArrayElements) until waitDone releases them. */
static jfloatArray g_async_x, g_async_y;
static jfloat *g_async_xp, *g_async_yp;

static void release_async(JNIEnv *env) {
    if (g_async_x) {
        (*env)->ReleaseFloatArrayElements(env, g_async_x, g_async_xp, JNI_ABORT);
        (*env)->ReleaseFloatArrayElements(env, g_async_y, g_async_yp, 0);
        (*env)->DeleteGlobalRef(env, g_async_x);
        (*env)->DeleteGlobalRef(env, g_async_y);
        g_async_x = g_async_y = NULL;
    }
}

JFN(jint, forwardHostAsync)(JNIEnv *env, jclass c, jlong h, jfloatArray x, jfloatArray y, jint T) {
    if (g_async_x) {  /* one call in flight per process through this shim: finish the previous one first */
        int rc0 = omoe_wait((omoe_handle *)(intptr_t)h);
        release_async(env);
        if (rc0 != OMOE_OK) return rc0;
    }
    g_async_x = (jfloatArray)(*env)->NewGlobalRef(env, x);
    g_async_y = (jfloatArray)(*env)->NewGlobalRef(env, y);
    g_async_xp = (*env)->GetFloatArrayElements(env, g_async_x, NULL);
    g_async_yp = (*env)->GetFloatArrayElements(env, g_async_y, NULL);
    int rc = omoe_forward_host_async((omoe_handle *)(intptr_t)h, g_async_xp, g_async_yp, T, OMOE_F32, NULL);
    if (rc != OMOE_OK) release_async(env);
    return rc;
}

JFN(jint, waitDone)(JNIEnv *env, jclass c, jlong h) {
    int rc = omoe_wait((omoe_handle *)(intptr_t)h);
    release_async(env);
    return rc;
}

JFN(jint, forwardBlock)(JNIEnv *env, jclass c, jlong h, jlong x, jlong gamma, jfloat eps, jlong y, jint T, jint io) {
    return omoe_forward_block((omoe_handle *)(intptr_t)h, (const void *)(intptr_t)x, (const float *)(intptr_t)gamma, eps,
                              (void *)(intptr_t)y, T, io, NULL);
}

JFN(jint, getRouting)(JNIEnv *env, jclass c, jlong h, jintArray idx, jfloatArray w, jintArray counts,
                      jintArray offsets, jintArray perm) {
    jint *pi = idx ? (*env)->GetIntArrayElements(env, idx, NULL) : NULL;
    jfloat *pw = w ? (*env)->GetFloatArrayElements(env, w, NULL) : NULL;
    jint *pc = counts ? (*env)->GetIntArrayElements(env, counts, NULL) : NULL;
    jint *po = offsets ? (*env)->GetIntArrayElements(env, offsets, NULL) : NULL;
    jint *pp = perm ? (*env)->GetIntArrayElements(env, perm, NULL) : NULL;
    int rc = omoe_get_routing((omoe_handle *)(intptr_t)h, (int32_t *)pi, pw, (int32_t *)pc, (int32_t *)po, (int32_t *)pp);
    if (pi) (*env)->ReleaseIntArrayElements(env, idx, pi, 0);
    if (pw) (*env)->ReleaseFloatArrayElements(env, w, pw, 0);
    if (pc) (*env)->ReleaseIntArrayElements(env, counts, pc, 0);
    if (po) (*env)->ReleaseIntArrayElements(env, offsets, po, 0);
    if (pp) (*env)->ReleaseIntArrayElements(env, perm, pp, 0);
    return rc;
}

JFN(jint, setTraining)(JNIEnv *env, jclass c, jlong h, jint on) {
    return omoe_set_training((omoe_handle *)(intptr_t)h, on);
}

JFN(jint, backward)(JNIEnv *env, jclass c, jlong h, jlong x, jlong dy, jlong dx, jint T, jint io) {
    return omoe_backward((omoe_handle *)(intptr_t)h, (const void *)(intptr_t)x, (const void *)(intptr_t)dy,
                         (void *)(intptr_t)dx, T, io, NULL);
}

JFN(jint, getWeightGrads)(JNIEnv *env, jclass c, jlong h, jlong dr, jlong db, jlong dg, jlong du, jlong dd) {
    return omoe_get_weight_grads((omoe_handle *)(intptr_t)h, (float *)(intptr_t)dr, (float *)(intptr_t)db,
                                 (float *)(intptr_t)dg, (float *)(intptr_t)du, (float *)(intptr_t)dd, NULL);
}

JFN(jint, epConnectLocal)(JNIEnv *env, jclass c, jlongArray hs) {
    jsize n = (*env)->GetArrayLength(env, hs);
    jlong *p = (*env)->GetLongArrayElements(env, hs, NULL);
    omoe_handle *arr[8];
    if (n > 8) n = 8;
    for (jsize i = 0; i < n; i++) arr[i] = (omoe_handle *)(intptr_t)p[i];
    int rc = omoe_ep_connect_local(arr, (int32_t)n);
    (*env)->ReleaseLongArrayElements(env, hs, p, JNI_ABORT);
    return rc;
}

JFN(jint, epExport)(JNIEnv *env, jclass c, jlong h, jbyteArray blob) {
    jbyte *p = (*env)->GetByteArrayElements(env, blob, NULL);
    int rc = omoe_ep_export((omoe_handle *)(intptr_t)h, p);
    (*env)->ReleaseByteArrayElements(env, blob, p, 0);
    return rc;
}

JFN(jint, epImport)(JNIEnv *env, jclass c, jlong h, jbyteArray blobs) {
    jbyte *p = (*env)->GetByteArrayElements(env, blobs, NULL);
    int rc = omoe_ep_import((omoe_handle *)(intptr_t)h, p);
    (*env)->ReleaseByteArrayElements(env, blobs, p, JNI_ABORT);
    return rc;
}
#else
/* No JDK headers on this machine: nothing to compile. */
typedef int omoe_jni_unavailable;
#endif
