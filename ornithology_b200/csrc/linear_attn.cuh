// linear_attn.cuh — argument block shared by the gated delta-net kernels.
#pragma once
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
// conv + SiLU image of qkv (its q / k parts are normalised in place), rq / rk the
// per-(token, key head) inverse norms, la / be the per-(token, value head) log-decay
// and write gate, blocks a work area of linear_prefill_tc_blocks_bytes() bytes.
size_t linear_prefill_tc_blocks_bytes(int nv, int n_seq, int T);
ornith_status launch_linear_prefill_tc(const LinArgs &x, int n_seq, int act_dtype, float *Y, const float *rq,
                                       const float *rk, const float *la, const float *be, float *blocks,
                                       cudaStream_t s);
