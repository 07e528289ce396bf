// kv_rows.cuh — the three KV row formats: addressing, encode, decode.
//
//   F32        head_dim floats
//   INT8_HEAD  head_dim int8 codes + one f32 scale per (position, head)
//              (engine's own quantised cache, reference: src/ornith_attn.c:65-85)
//   Q8_0       head_dim/32 blocks of {f16 scale, 32 int8}, 34 bytes each
//              (reference: src/ornith_quant.c:155-184)
//
// The encoders reproduce the engine's arithmetic operation by operation with
// explicitly rounded intrinsics so no multiply-add is contracted: the stored
// bytes are identical to the CPU codec's for identical f32 inputs.
#pragma once
#include "common.cuh"

struct KvView {
    int mode, nkv, hd;
    uint8_t *K, *V;          // row pools
    float *Ks, *Vs;          // INT8_HEAD scales
    const int64_t *seq_off;  // [n_seq + 1] positions
};

static inline KvView make_view(const ornith_cuda_kv *kv) {
    KvView v;
    v.mode = kv->mode; v.nkv = kv->n_kv_heads; v.hd = kv->head_dim;
    v.K = (uint8_t *)kv->K; v.V = (uint8_t *)kv->V; v.Ks = kv->Ks; v.Vs = kv->Vs;
    v.seq_off = kv->seq_off;
    return v;
}

__host__ __device__ __forceinline__ size_t kv_row_bytes(int mode, int hd) {
    return mode == ORNITH_KV_F32 ? (size_t)hd * 4 : mode == ORNITH_KV_Q8_0 ? (size_t)(hd / 32) * 34 : (size_t)hd;
}

__device__ __forceinline__ float q8_0_block_scale(const uint8_t *blk) {
    return __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(blk)));
}

// ---- encoders: one CTA encodes one row held as f32 in shared memory ---------

// Q8_0: each warp takes blocks warp, warp+nwarps, ...; lane = element in block.
__device__ __forceinline__ void encode_row_q8_0(const float *row, int hd, uint8_t *dst) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int blk = w; blk < hd / 32; blk += nw) {
        float x = row[blk * 32 + lane];
        float amax = warp_max(fabsf(x));
        float d = __fdiv_rn(amax, 127.0f);
        float id = (d != 0.0f) ? __fdiv_rn(1.0f, d) : 0.0f;
        int q = (int)roundf(__fmul_rn(x, id));          // lroundf: ties away from zero
        q = max(-127, min(127, q));
        uint8_t *o = dst + (size_t)blk * 34;
        if (lane == 0) *reinterpret_cast<unsigned short *>(o) = __half_as_ushort(__float2half_rn(d));
        o[2 + lane] = (uint8_t)(int8_t)q;
    }
}

// INT8_HEAD: one scale for the whole row; lrintf = round half to even.
__device__ __forceinline__ void encode_row_int8(const float *row, int hd, int8_t *codes, float *scale,
                                                float *red) {
    float m = 0.0f;
    for (int i = threadIdx.x; i < hd; i += blockDim.x) m = fmaxf(m, fabsf(row[i]));
    float amax = block_max(m, red);
    if (amax == 0.0f) {
        for (int i = threadIdx.x; i < hd; i += blockDim.x) codes[i] = 0;
        if (threadIdx.x == 0) *scale = 0.0f;
        return;
    }
    float inv = __fdiv_rn(127.0f, amax);
    for (int i = threadIdx.x; i < hd; i += blockDim.x) {
        int q = __float2int_rn(__fmul_rn(row[i], inv));
        codes[i] = (int8_t)max(-127, min(127, q));
    }
    if (threadIdx.x == 0) *scale = __fdiv_rn(amax, 127.0f);
}

// ---- element decode (generic paths) -------------------------------------------
// Value of element d of a stored row, exactly what the CPU path attends over:
// Q8_0 -> (float)code * f16_to_f32(scale); INT8_HEAD -> the raw code (the scale
// is applied once per dot product, as the engine does).
template <int MODE>
__device__ __forceinline__ float kv_elem(const uint8_t *row, int d) {
    if (MODE == ORNITH_KV_F32) return reinterpret_cast<const float *>(row)[d];
    if (MODE == ORNITH_KV_INT8_HEAD) return (float)reinterpret_cast<const int8_t *>(row)[d];
    const uint8_t *blk = row + (size_t)(d >> 5) * 34;
    return __fmul_rn((float)(int8_t)blk[2 + (d & 31)], q8_0_block_scale(blk));
}
