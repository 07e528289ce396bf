// runtime.cu — device probe, error text, and the small synchronous memory helpers
// that let a C host drive the library without linking the CUDA runtime itself.
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "common.cuh"
#include "tcgen05.cuh"

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

int orn_device_index() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess) { (void)cudaGetLastError(); return 0; }
    return d < 0 ? 0 : (d >= ORN_MAX_DEVICES ? ORN_MAX_DEVICES - 1 : d);
}

// ---- allocation hook ---------------------------------------------------------------
static std::mutex g_hook_mu;
static ornith_cuda_alloc_hook g_alloc_hook = nullptr;
static void *g_alloc_hook_user = nullptr;

// 0 = go ahead, else the allocation is refused (host-side failure injection)
static ornith_status alloc_hook_check(size_t bytes, const char *what) {
    ornith_cuda_alloc_hook hook;
    void *user;
    {
        std::lock_guard<std::mutex> lock(g_hook_mu);
        hook = g_alloc_hook; user = g_alloc_hook_user;
    }
    if (hook && hook(bytes, user) != 0) {
        orn_record_error("%s: allocation of %zu bytes refused by the allocation hook", what, bytes);
        return ORNITH_ERR_OOM;
    }
    return ORNITH_OK;
}

ornith_status orn_device_alloc(void **p, size_t bytes, const char *what) {
    *p = nullptr;
    ORN_TRY(alloc_hook_check(bytes, what));
    return orn_check(cudaMalloc(p, bytes), what);
}

// ---- status word ---------------------------------------------------------------------
static unsigned int *g_status_host[ORN_MAX_DEVICES] = {};
static unsigned int *g_status_dev[ORN_MAX_DEVICES] = {};
static bool g_status_tried[ORN_MAX_DEVICES] = {};

unsigned int *orn_status_word() {
    const int d = orn_device_index();
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (!g_status_tried[d]) {
        g_status_tried[d] = true;
        void *h = nullptr, *dv = nullptr;
        if (cudaHostAlloc(&h, 64, cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess &&
            cudaHostGetDevicePointer(&dv, h, 0) == cudaSuccess) {
            memset(h, 0, 64);
            g_status_host[d] = (unsigned int *)h;
            g_status_dev[d] = (unsigned int *)dv;
        } else {
            (void)cudaGetLastError();
        }
    }
    return g_status_dev[d];
}

// non-zero status word of the current device -> error text + ORNITH_ERR_BACKEND, word cleared
static ornith_status take_status_word() {
    const int d = orn_device_index();
    volatile unsigned int *w = g_status_host[d];
    if (!w || !*w) return ORNITH_OK;
    const unsigned int code = *w;
    *w = 0;
    orn_record_error("a kernel gave up a bounded wait (status 0x%x:%s%s%s%s): its outputs are not valid", code,
                     (code & ORN_WAIT_GQA_PREFILL) ? " full-attention prefill" : "",
                     (code & ORN_WAIT_DELTA_SCAN) ? " delta-net prefill scan" : "",
                     (code & ORN_WAIT_DECODE) ? " decode" : "", (code & ORN_WAIT_SELFTEST) ? " self-test" : "");
    return (ornith_status)ORNITH_ERR_BACKEND;
}

OrnTensorMapEncodeFn orn_tensor_map_encoder() {
    static OrnTensorMapEncodeFn fn = nullptr;
    if (!fn) {
        cudaDriverEntryPointQueryResult q;
        void *p = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (OrnTensorMapEncodeFn)p;
        else
            (void)cudaGetLastError();
    }
    return fn;
}

// A kernel whose only job is to wait, a few polls long, on an mbarrier nobody arrives on: the wait
// helper of the tensor-core kernels must come back, report through the status word, and leave the
// context usable.  Nothing is in flight when it gives up.
__global__ void k_wait_selftest(unsigned int *status, int polls, int *gave_up) {
    __shared__ unsigned long long bar;
    if (threadIdx.x == 0) {
        tc5::mbar_init(tc5::su32(&bar), 1);
        tc5::mbar_init_fence();
        const bool ok = tc5::mbar_wait(tc5::su32(&bar), 0, polls);
        if (!ok) tc5::report_timeout(status, ORN_WAIT_SELFTEST);
        *gave_up = ok ? 0 : 1;
    }
}

ornith_status release_linear_decode_buffers(cudaStream_t s, bool all);   // linear_decode_ring.cu
ornith_status release_delta_slab_pipe();                                  // delta_scan_tc5.cu

extern "C" {

int ornith_backend_cuda_available(void) { return probe_device(); }

void ornith_cuda_set_alloc_hook(ornith_cuda_alloc_hook hook, void *user) {
    std::lock_guard<std::mutex> lock(g_hook_mu);
    g_alloc_hook = hook;
    g_alloc_hook_user = user;
}

ornith_status ornith_cuda_poll_status(void) {
    ORN_TRY(orn_require_device());
    return take_status_word();
}

ornith_status ornith_cuda_stream_release(void *stream, int all_streams) {
    ORN_TRY(orn_require_device());
    if (all_streams) ORN_TRY(orn_check(cudaDeviceSynchronize(), "device sync"));
    else ORN_TRY(orn_check(cudaStreamSynchronize(as_stream(stream)), "stream sync"));
    if (all_streams) ORN_TRY(release_delta_slab_pipe());       // the prefill's second stream and its events (this device)
    return release_linear_decode_buffers(as_stream(stream), all_streams != 0);
}

ornith_status ornith_cuda_selftest_wait_timeout(int polls) {
    ORN_TRY(orn_require_device());
    if (polls < 1) polls = 1;
    if (polls > (1 << 16)) polls = 1 << 16;
    unsigned int *status = orn_status_word();
    int *flag = nullptr;
    ORN_TRY(orn_check(cudaMalloc((void **)&flag, sizeof(int)), "selftest flag"));
    int gave_up = -1;
    k_wait_selftest<<<1, 32>>>(status, polls, flag);
    ornith_status st = orn_check_launch("k_wait_selftest");
    if (st == ORNITH_OK) st = orn_check(cudaMemcpy(&gave_up, flag, sizeof(int), cudaMemcpyDeviceToHost), "selftest read-back");
    (void)cudaFree(flag);
    if (st != ORNITH_OK) return st;
    if (gave_up != 1) { orn_record_error("wait self-test: the wait did not give up (%d)", gave_up); return ORNITH_ERR_FORMAT; }
    st = take_status_word();                       // must report the give-up
    if (st == ORNITH_OK && status) { orn_record_error("wait self-test: the status word stayed clear"); return ORNITH_ERR_FORMAT; }
    return st == ORNITH_OK ? (ornith_status)ORNITH_ERR_BACKEND : st;   // the expected outcome is ORNITH_ERR_BACKEND
}

const char *ornith_cuda_last_error(void) { return g_cuda_err[0] ? g_cuda_err : "(no detail)"; }

ornith_status ornith_cuda_set_device(int device) {
    ORN_TRY(orn_require_device());
    return orn_check(cudaSetDevice(device), "cudaSetDevice");
}

ornith_status ornith_cuda_malloc(void **dev_ptr, size_t bytes) {
    *dev_ptr = nullptr;
    if (bytes == 0) bytes = 16;
    ORN_TRY(alloc_hook_check(bytes, "ornith_cuda_malloc"));      // before the device is touched: a host can test its OOM paths without a GPU
    ORN_TRY(orn_require_device());
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
    ORN_TRY(orn_check(cudaStreamSynchronize(as_stream(stream)), "stream sync"));
    return take_status_word();
}

// theta^(-2i/rot) with the host libm, the same expression the engine evaluates
// per call (reference: src/ornith_tensor.c:171); doing it here keeps the angle
// pos*freq bit-identical to the CPU path.
void ornith_cuda_rope_inv_freq(float theta, int rotary_dim, float *host_out) {
    int half = rotary_dim / 2;
    for (int i = 0; i < half; i++)
        host_out[i] = powf(theta, -2.0f * (float)i / (float)rotary_dim);
}

// ---- multi-GPU plan -------------------------------------------------------------
ornith_status ornith_cuda_head_shard(int nk, int nv, int nh, int nkv, int rank, int world, ornith_cuda_shard *out) {
    if (!out || nk <= 0 || nv <= 0 || nh <= 0 || nkv <= 0 || world <= 0 || rank < 0 || rank >= world) {
        orn_record_error("head_shard: bad arguments");
        return ORNITH_ERR_FORMAT;
    }
    if (nv % world || nh % world || nh % nkv) {
        orn_record_error("head_shard: %d ranks do not divide %d value heads / %d query heads", world, nv, nh);
        return ORNITH_ERR_UNSUPPORTED;
    }
    const int pv = nv / world, ph = nh / world, v0 = rank * pv;
    int k0, n_k;
    if (pv >= nk) {
        if (pv % nk) { orn_record_error("head_shard: value heads per rank must be a multiple of the key heads"); return ORNITH_ERR_UNSUPPORTED; }
        k0 = 0; n_k = nk;
    } else {
        if (nk % pv) { orn_record_error("head_shard: key heads must be a multiple of the value heads per rank"); return ORNITH_ERR_UNSUPPORTED; }
        k0 = v0 % nk; n_k = pv;
    }
    const int group = nh / nkv, kv_lo = (rank * ph) / group, kv_hi = (rank * ph + ph - 1) / group;
    out->rank = rank; out->world = world;
    out->v_head0 = v0; out->n_v_heads = pv;
    out->k_head0 = k0; out->n_k_heads = n_k;
    out->q_head0 = rank * ph; out->n_q_heads = ph;
    out->kv_head0 = kv_lo; out->n_kv_heads = kv_hi - kv_lo + 1;
    return ORNITH_OK;
}

// gathered [world][rows][w16] -> full [rows][world][w16], 16-byte pieces
__global__ void k_gather_layout(const uint4 *gathered, uint4 *full, int world, size_t rows, int w16) {
    const size_t n = (size_t)world * rows * w16;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(e % w16);
        const size_t t = e / w16;
        const int r = (int)(t % world);
        const size_t row = t / world;
        full[e] = gathered[((size_t)r * rows + row) * w16 + c];
    }
}

ornith_status ornith_cuda_gather_layout(const void *gathered, void *full, int world, size_t rows, int width,
                                        int elem_bytes, void *stream) {
    ORN_TRY(orn_require_device());
    if (!gathered || !full || world <= 0 || width <= 0 || (elem_bytes != 2 && elem_bytes != 4) ||
        ((size_t)width * elem_bytes) % 16 || ((uintptr_t)gathered % 16) || ((uintptr_t)full % 16)) {
        orn_record_error("gather_layout: bad arguments (rows of a multiple of 16 bytes, 16-byte aligned buffers)");
        return ORNITH_ERR_FORMAT;
    }
    if (rows == 0) return ORNITH_OK;
    const int w16 = (int)((size_t)width * elem_bytes / 16);
    const size_t n = (size_t)world * rows * w16;
    const unsigned blocks = (unsigned)((n + 255) / 256 < 148u * 16u ? (n + 255) / 256 : 148u * 16u);
    k_gather_layout<<<blocks, 256, 0, as_stream(stream)>>>((const uint4 *)gathered, (uint4 *)full, world, rows, w16);
    return orn_check_launch("k_gather_layout");
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
