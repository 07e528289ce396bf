// runtime.cu — device probe, error text, and the small synchronous memory helpers
// that let a C host drive the library without linking the CUDA runtime itself.
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "common.cuh"

static thread_local char g_cuda_err[512];

extern "C" void ornith_set_error(const char *fmt, ...);

void orn_record_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_cuda_err, sizeof(g_cuda_err), fmt, ap);
    va_end(ap);
    ornith_set_error("%s", g_cuda_err);
}

ornith_status orn_check(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return ORNITH_OK;
    orn_record_error("%s: %s", what, cudaGetErrorString(e));
    return e == cudaErrorMemoryAllocation ? ORNITH_ERR_OOM : (ornith_status)ORNITH_ERR_BACKEND;
}

ornith_status orn_check_launch(const char *what) { return orn_check(cudaGetLastError(), what); }

// 1 = usable sm_10x device, 0 = none; probed once.
static int probe_device() {
    static int cached = -1;
    if (cached >= 0) return cached;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();
        return cached = 0;
    }
    int dev = 0, major = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
        (void)cudaGetLastError();
        return cached = 0;
    }
    return cached = (major == 10) ? 1 : 0;
}

ornith_status orn_require_device() {
    if (probe_device()) return ORNITH_OK;
    orn_record_error("no usable CUDA device (needs compute capability 10.x); there is no CPU fallback");
    return (ornith_status)ORNITH_ERR_BACKEND;
}

extern "C" {

int ornith_backend_cuda_available(void) { return probe_device(); }

const char *ornith_cuda_last_error(void) { return g_cuda_err[0] ? g_cuda_err : "(no detail)"; }

ornith_status ornith_cuda_set_device(int device) {
    ORN_TRY(orn_require_device());
    return orn_check(cudaSetDevice(device), "cudaSetDevice");
}

ornith_status ornith_cuda_malloc(void **dev_ptr, size_t bytes) {
    ORN_TRY(orn_require_device());
    *dev_ptr = nullptr;
    if (bytes == 0) bytes = 16;
    ORN_TRY(orn_check(cudaMalloc(dev_ptr, bytes), "cudaMalloc"));
    return orn_check(cudaMemset(*dev_ptr, 0, bytes), "cudaMemset");
}

ornith_status ornith_cuda_free(void *dev_ptr) {
    if (!dev_ptr) return ORNITH_OK;
    return orn_check(cudaFree(dev_ptr), "cudaFree");
}

ornith_status ornith_cuda_memset(void *dev_ptr, int value, size_t bytes) {
    ORN_TRY(orn_require_device());
    return orn_check(cudaMemset(dev_ptr, value, bytes), "cudaMemset");
}

ornith_status ornith_cuda_h2d(void *dev_dst, const void *host_src, size_t bytes) {
    ORN_TRY(orn_require_device());
    if (!bytes) return ORNITH_OK;
    return orn_check(cudaMemcpy(dev_dst, host_src, bytes, cudaMemcpyHostToDevice), "h2d copy");
}

ornith_status ornith_cuda_d2h(void *host_dst, const void *dev_src, size_t bytes) {
    ORN_TRY(orn_require_device());
    if (!bytes) return ORNITH_OK;
    return orn_check(cudaMemcpy(host_dst, dev_src, bytes, cudaMemcpyDeviceToHost), "d2h copy");
}

ornith_status ornith_cuda_sync(void *stream) {
    ORN_TRY(orn_require_device());
    return orn_check(cudaStreamSynchronize(as_stream(stream)), "stream sync");
}

// theta^(-2i/rot) with the host libm, the same expression the engine evaluates
// per call (reference: src/ornith_tensor.c:171); doing it here keeps the angle
// pos*freq bit-identical to the CPU path.
void ornith_cuda_rope_inv_freq(float theta, int rotary_dim, float *host_out) {
    int half = rotary_dim / 2;
    for (int i = 0; i < half; i++)
        host_out[i] = powf(theta, -2.0f * (float)i / (float)rotary_dim);
}

// ---- counters ------------------------------------------------------------------
__global__ void k_advance(int32_t *c, int n, int delta) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) c[i] += delta;
}

ornith_status ornith_cuda_advance(int32_t *counters, int n, int delta, void *stream) {
    ORN_TRY(orn_require_device());
    if (n <= 0) return ORNITH_OK;
    k_advance<<<(n + 255) / 256, 256, 0, as_stream(stream)>>>(counters, n, delta);
    return orn_check_launch("k_advance");
}

}  // extern "C"
