// linear_attn.cuh — argument block shared by the gated delta-net kernels.
#pragma once
#include <functional>

#include "common.cuh"

struct LinArgs {
    int nk, nv, dk, dv, conv_k, head_map;
    float out_scale, eps;
    const float *conv_w, *conv_b, *a_coef, *dt_bias, *norm_w;
    float *S, *conv;
    int64_t S_stride, conv_stride;
    const int32_t *pos;
    const void *qkv, *a, *b, *z;
    void *out;
    int T;                               // tokens per sequence (prefill kernels)
};

__device__ __forceinline__ int key_head_of(const LinArgs &a, int hv) {
    return a.head_map == ORNITH_HEADMAP_GROUPED ? hv / (a.nv / a.nk) : hv % a.nk;
}
// exactly one value head per key head stores that key head's q/k conv inputs
__device__ __forceinline__ bool owns_key_head(const LinArgs &a, int hv) {
    return a.head_map == ORNITH_HEADMAP_GROUPED ? (hv % (a.nv / a.nk)) == 0 : hv < a.nk;
}

// Tensor-core chunked scan for dk = dv = 128 (delta_prefill_tc.cu).  Y holds the
// conv + SiLU image of qkv, rq / rk the
// per-(token, key head) inverse norms, la / be the per-(token, value head) log-decay
// and write gate, blocks a work area of linear_prefill_tc_blocks_bytes() bytes.
size_t linear_prefill_tc_blocks_bytes(int nk, int nv, int n_seq, int T);
ornith_status launch_linear_prefill_tc(const LinArgs &x, int n_seq, int act_dtype, float *Y, const float *rq,
                                       const float *rk, const float *la, const float *be, float *blocks,
                                       cudaStream_t s);

// The same scan on the 5th-generation tensor cores (delta_scan_tc5.cu): tcgen05.mma in tf32 with the
// state in tensor memory, operands staged by TMA, 64-token chunks.  Y must hold the q and k channels
// rounded to tf32 (k_conv4_silu_prefill does that); work = linear_prefill_tc5_work_bytes() bytes;
// la = be = nullptr: the gates are computed from the layer's a / b inputs.
//
// With a front (the causal conv of a token range and the refresh of the conv history, as launches the caller
// provides) and one wave of heads or less, the prompt is cut into slabs and pipelined: conv + chunk preparation
// of slab k + 1 run on the caller's stream while slab k is scanned on a second, high-priority stream, so the
// SMs the scan leaves idle (one CTA per head) do the memory-bound passes.  Events order the slabs; the caller's
// stream waits for the last scan before the call returns.  front = nullptr: Y, rq and rk are complete already.
struct TC5Front {
    std::function<ornith_status(int t_begin, int t_end, cudaStream_t)> conv;
    std::function<ornith_status(cudaStream_t)> ring_refresh;
};
// conv_prefill_tma.cu: the conv + SiLU front of that path fed by tensor copies (see there)
ornith_status launch_conv4_silu_prefill_tma(const LinArgs &x, int n_seq, int act_dtype, float *Y, float *rq, float *rk,
                                            int t_begin, int t_end, cudaStream_t s, bool *handled);
size_t linear_prefill_tc5_work_bytes(int nk, int nv, int n_seq, int T);
ornith_status release_delta_slab_pipe();
ornith_status launch_linear_prefill_tc5(const LinArgs &x, int n_seq, int act_dtype, const float *Y, const float *rq,
                                        const float *rk, const float *la, const float *be, const TC5Front *front,
                                        float *work, float *dbg, cudaStream_t s);

__device__ __forceinline__ float4 lds128(const float *p) {        // not hoisted: keeps k/q out of registers
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];\n"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"((uint32_t)__cvta_generic_to_shared(p)));
    return v;
}

// conv of one channel from its four ring slots (slot of token t' is t' & 3); taps are the
// tokens t-3, t-2, t-1 = slots sb, sb+1, sb+2 with sb = (t + 1) & 3.  Same operation order
// and rounding as the engine (reference: src/ornith_attn.c:373-381), then SiLU.
__device__ __forceinline__ float conv4_silu(const float (&h)[4], float xin, float4 w, float bias, int sb) {
    float t0, t1, t2;
    switch (sb) {                                                  // uniform over the CTA
    case 0:  t0 = h[0]; t1 = h[1]; t2 = h[2]; break;
    case 1:  t0 = h[1]; t1 = h[2]; t2 = h[3]; break;
    case 2:  t0 = h[2]; t1 = h[3]; t2 = h[0]; break;
    default: t0 = h[3]; t1 = h[0]; t2 = h[1]; break;
    }
    float acc = bias;
    acc = __fadd_rn(acc, __fmul_rn(w.x, t0));
    acc = __fadd_rn(acc, __fmul_rn(w.y, t1));
    acc = __fadd_rn(acc, __fmul_rn(w.z, t2));
    acc = __fadd_rn(acc, __fmul_rn(w.w, xin));
    return silu_f(acc);
}

// Persistent variant of the dk = dv = 128 decode step (linear_decode_ring.cu): the state is
// streamed through a ring of bulk copies in shared memory.
ornith_status launch_linear_decode_ring(const LinArgs &x, int n_seq, int act_dtype, cudaStream_t s);
