// common.cuh — shared device helpers and host-side error plumbing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ornith_cuda.h"

// ---- host side -------------------------------------------------------------
void orn_record_error(const char *fmt, ...);          // fills both last-error buffers
ornith_status orn_check(cudaError_t e, const char *what);
ornith_status orn_check_launch(const char *what);     // cudaGetLastError after a launch
ornith_status orn_require_device();                    // ORNITH_ERR_BACKEND when no usable GPU

// Per-device bookkeeping.  Attributes such as the dynamic shared-memory opt-in of a kernel and
// the SM count belong to a device, not to the process: one process may drive several GPUs
// (ornith_cuda_set_device), so "done once" flags are arrays indexed by the current device.
#define ORN_MAX_DEVICES 64
int orn_device_index();                                // current device, clamped to [0, ORN_MAX_DEVICES)
// cudaMalloc through the allocation hook (ornith_cuda_set_alloc_hook): every device allocation the
// library makes on its own goes through here, so a host can make the N-th one fail.
ornith_status orn_device_alloc(void **p, size_t bytes, const char *what);
// Status word of the current device: host memory the kernels can write.  A bounded wait that gives
// up ORs a code into it; ornith_cuda_sync / ornith_cuda_poll_status turn it into ORNITH_ERR_BACKEND.
// nullptr when the word could not be set up (the kernels then only poison their outputs).
unsigned int *orn_status_word();
#define ORN_WAIT_GQA_PREFILL 0x1u
#define ORN_WAIT_DELTA_SCAN  0x2u
#define ORN_WAIT_SELFTEST    0x4u
#define ORN_WAIT_DECODE      0x8u

#define ORN_TRY(expr)                                   \
    do {                                                \
        ornith_status _s = (expr);                      \
        if (_s != ORNITH_OK) return _s;                 \
    } while (0)

static inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }
static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// ---- activation I/O ----------------------------------------------------------
template <typename T> __device__ __forceinline__ float act_ld(const T *p, size_t i);
template <> __device__ __forceinline__ float act_ld<float>(const float *p, size_t i) { return p[i]; }
template <> __device__ __forceinline__ float act_ld<__nv_bfloat16>(const __nv_bfloat16 *p, size_t i) {
    return __bfloat162float(p[i]);
}
template <typename T> __device__ __forceinline__ void act_st(T *p, size_t i, float v);
template <> __device__ __forceinline__ void act_st<float>(float *p, size_t i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void act_st<__nv_bfloat16>(__nv_bfloat16 *p, size_t i, float v) {
    p[i] = __float2bfloat16_rn(v);
}

// four adjacent activations (16-byte / 8-byte aligned)
__device__ __forceinline__ float4 act_ld4(const float *p, size_t i) { return *reinterpret_cast<const float4 *>(p + i); }
__device__ __forceinline__ float4 act_ld4(const __nv_bfloat16 *p, size_t i) {
    const uint2 u = *reinterpret_cast<const uint2 *>(p + i);
    return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u),
                       __uint_as_float(u.y << 16), __uint_as_float(u.y & 0xffff0000u));
}
__device__ __forceinline__ void act_st4(float *p, size_t i, float4 v) { *reinterpret_cast<float4 *>(p + i) = v; }
__device__ __forceinline__ void act_st4(__nv_bfloat16 *p, size_t i, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2 *>(p + i) = make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
}

// ---- scalar math in the engine's form (reference: src/ornith_tensor.c:117-119)
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x * sigmoid_f(x); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
// SiLU with the hardware exponential and reciprocal (a few ulp); for the tensor-core
// prefill paths, whose products are already rounded to tf32 / f16
// (the .ftz forms: without them the compiler wraps each special-function instruction in a denormal fix-up)
__device__ __forceinline__ float ex2_fast(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float rcp_fast(float x) { float y; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float silu_fast(float x) { return x * rcp_fast(1.0f + ex2_fast(-1.4426950408889634f * x)); }

// Launch `kernel` as a programmatic dependent of the kernel in front of it on the stream: its CTAs may become resident
// while that kernel still runs.  The kernel must execute griddepcontrol.wait in every CTA before it touches anything a
// kernel in front of it may write or read, and before it exits.
template <typename... KArgs, typename... Args>
static inline cudaError_t orn_launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---- reductions ---------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide reductions over up to 32 warps. `red` is shared scratch of at least
// 32 elements; every thread of the block must call. Result is returned to all.
template <typename T>
__device__ __forceinline__ T block_sum(T v, T *red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                       // protects `red` from the previous use
    if (lane == 0) red[w] = v;
    __syncthreads();
    T r = (lane < nw) ? red[lane] : T(0);
    return warp_sum(r);
}
__device__ __forceinline__ float block_max(float v, float *red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : -INFINITY;
    return warp_max(r);
}
