// Test infrastructure, never linked into the product: a host driver that runs the REFERENCE's own CUDA
// kernels (compiled from the reference's .cu files into oracle/_ref/*.cubin by oracle/Makefile, never
// copied) together with cuBLAS SGEMM, in the order and with the launch shapes the reference's Java
// wrappers use.  It stands where the JVM + JCuda would stand: the reference loads each kernel by name
// from a module and starts it with cuLaunchKernel on the null stream
// (src/main/java/com/omega/engine/gpu/BaseKernel.java:66-72).  The checker and the "reference kernels
// on this GPU" baseline call it; the product never does.
//
//   softmax       SoftmaxKernel.cu:5 `softmax`, launched as SoftmaxKernel.java:169-184
//                 (grid ceil(rows/1024), block 1024: one thread per row)
//   SiLU          activeFunction.cu:173 `silu_forward`, launched as
//                 nn/layer/active/gpu/SiLUKernel.java:125-146 (grid ceil(n/1024), block 1024)
//   backward      activeFunction.cu:182 `silu_backward`, SoftmaxKernel.cu:101 `softmax_back` (same launch shapes)
//   product       OPKernel.cu:1040 `mul_kernel`, launched as ad/op/gpu/OPKernel.java:742-758
//   RMSNorm       RMSKernel.cu:185 `rmsnorm_forward_kernel2`, launched as
//                 nn/layer/normalization/gpu/RMSKernel.java:232-249 (grid ceil((B*32+1023)/1024), block 1024)
//   linear        FullyLayer.output() (nn/layer/FullyLayer.java:235) -> GPUOP.multiplyFloat
//                 (gpu/GPUOP.java:405-417): cublasSgemm(handle, OP_T, OP_N, out, rows, in, 1, W, in, X, in, 0, Y, out)
//                 on a handle with default math mode and no stream set
//   dense MLP     LlamaMLPLayer.output() (nn/layer/llama/LlamaMLPLayer.java:117-123):
//                 linear1 -> SiLU -> linear3 -> product -> linear2
#include <cublas_v2.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

namespace {

char g_err[1280] = "";
CUmodule g_mod[4];
CUfunction g_softmax, g_silu, g_mul, g_rms, g_silu_back, g_softmax_back;
cublasHandle_t g_blas = nullptr;
bool g_ready = false;
constexpr int kThreads = 1024;  // CAFFE_CUDA_NUM_THREADS in every wrapper class

int fail(const char *what, int code) {
    snprintf(g_err, sizeof(g_err), "%s failed (%d)", what, code);
    return -1;
}

int blocks(long n) { return (int)((n + kThreads - 1) / kThreads); }

int launch(CUfunction f, int grid, void **params) {
    CUresult r = cuLaunchKernel(f, grid, 1, 1, kThreads, 1, 1, 0, nullptr, params, nullptr);
    return r == CUDA_SUCCESS ? 0 : fail("cuLaunchKernel", (int)r);
}

}  // namespace

extern "C" {

const char *refk_error() { return g_err; }

// dir: folder holding SoftmaxKernel.cubin, activeFunction.cubin, OPKernel.cubin, RMSKernel.cubin
int refk_init(const char *dir) {
    if (g_ready) return 0;
    cudaError_t ce = cudaFree(0);  // the runtime's context becomes current, as torch's is
    if (ce != cudaSuccess) return fail("cudaFree(0)", (int)ce);
    const char *files[4] = {"SoftmaxKernel.cubin", "activeFunction.cubin", "OPKernel.cubin", "RMSKernel.cubin"};
    for (int i = 0; i < 4; i++) {
        char path[1024];
        snprintf(path, sizeof(path), "%s/%s", dir, files[i]);
        CUresult r = cuModuleLoad(&g_mod[i], path);
        if (r != CUDA_SUCCESS) {
            snprintf(g_err, sizeof(g_err), "cuModuleLoad(%s) failed (%d)", path, (int)r);
            return -1;
        }
    }
    CUresult r;
    if ((r = cuModuleGetFunction(&g_softmax, g_mod[0], "softmax")) != CUDA_SUCCESS) return fail("softmax", (int)r);
    if ((r = cuModuleGetFunction(&g_silu, g_mod[1], "silu_forward")) != CUDA_SUCCESS) return fail("silu_forward", (int)r);
    if ((r = cuModuleGetFunction(&g_mul, g_mod[2], "mul_kernel")) != CUDA_SUCCESS) return fail("mul_kernel", (int)r);
    if ((r = cuModuleGetFunction(&g_rms, g_mod[3], "rmsnorm_forward_kernel2")) != CUDA_SUCCESS)
        return fail("rmsnorm_forward_kernel2", (int)r);
    if ((r = cuModuleGetFunction(&g_silu_back, g_mod[1], "silu_backward")) != CUDA_SUCCESS)
        return fail("silu_backward", (int)r);
    if ((r = cuModuleGetFunction(&g_softmax_back, g_mod[0], "softmax_back")) != CUDA_SUCCESS)
        return fail("softmax_back", (int)r);
    cublasStatus_t bs = cublasCreate(&g_blas);
    if (bs != CUBLAS_STATUS_SUCCESS) return fail("cublasCreate", (int)bs);
    g_ready = true;
    return 0;
}

int refk_softmax(float *in, float *out, int rows, int n) {
    void *p[] = {&in, &out, &rows, &n};
    return launch(g_softmax, blocks(rows), p);
}

int refk_silu(float *x, float *out, int n) {
    void *p[] = {&x, &out, &n};
    return launch(g_silu, blocks(n), p);
}

// silu_backward(x, output, delta, diff, n): activeFunction.cu:182, launched as SiLUKernel.backward does
// (grid ceil(n/1024), block 1024); `output` is not read by the kernel.
int refk_silu_backward(float *x, float *out, float *delta, float *diff, int n) {
    void *p[] = {&x, &out, &delta, &diff, &n};
    return launch(g_silu_back, blocks(n), p);
}

// softmax_back(output, delta, diff, batch, n): SoftmaxKernel.cu:101, one thread per row.
int refk_softmax_back(float *out, float *delta, float *diff, int rows, int n) {
    void *p[] = {&out, &delta, &diff, &rows, &n};
    return launch(g_softmax_back, blocks(rows), p);
}

int refk_mul(float *a, float *b, float *r, int n) {
    void *p[] = {&n, &a, &b, &r};
    return launch(g_mul, blocks(n), p);
}

int refk_rmsnorm(float *out, float *inp, float *gamma, int rows, int width) {
    void *p[] = {&out, &inp, &gamma, &rows, &width};
    return launch(g_rms, blocks((long)rows * 32), p);
}

// y[rows, n_out] = x[rows, n_in] * w[n_out, n_in]^T
int refk_linear(const float *x, const float *w, float *y, int rows, int n_in, int n_out) {
    const float one = 1.0f, zero = 0.0f;
    cublasStatus_t s = cublasSgemm(g_blas, CUBLAS_OP_T, CUBLAS_OP_N, n_out, rows, n_in, &one, w, n_in, x, n_in, &zero,
                                   y, n_out);
    return s == CUBLAS_STATUS_SUCCESS ? 0 : fail("cublasSgemm", (int)s);
}

// The reference's dense SwiGLU MLP on `rows` rows; g, a, u, tmp: [rows, dff] scratch, all kept as the
// reference keeps them (linear1 output, SiLU output, linear3 output, product).
int refk_mlp(const float *x, const float *w1, const float *w3, const float *w2, float *g, float *a, float *u,
             float *tmp, float *y, int rows, int d, int dff) {
    if (rows == 0) return 0;
    const long n = (long)rows * dff;
    if (n > 0x7fffffffL) return fail("rows*dff beyond the kernels' int index", 0);
    if (refk_linear(x, w1, g, rows, d, dff)) return -1;
    if (refk_silu(g, a, (int)n)) return -1;
    if (refk_linear(x, w3, u, rows, d, dff)) return -1;
    if (refk_mul(a, u, tmp, (int)n)) return -1;
    return refk_linear(tmp, w2, y, rows, dff, d);
}

}  // extern "C"
