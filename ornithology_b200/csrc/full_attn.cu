// full_attn.cu — GQA full-attention layers: q/k preparation + KV append/encode,
// split-K decode over f32 / Q8_0 / int8-per-head rows, causal prefill.
//
// Reference behaviour being replaced:
//   full_attn()          src/ornith_rforward.c:419-455
//   full_attn_prefill()  src/ornith_rforward.c:513-556
//   ornith_gqa_step()    src/ornith_attn.c:87-149
#include <math.h>
#include <stdlib.h>

#include "common.cuh"
#include "full_attn.cuh"
#include "kv_rows.cuh"

// =============================================================================
// q/k preparation and KV append  (one CTA per (token, head-row))
// =============================================================================

struct PrepArgs {
    KvView kv;
    const int32_t *kv_len, *rope_pos;
    const void *qproj, *k, *v;
    float *q_prep;                       // [n_tok][nh][hd] f32
    __half *Qh;                          // if set: query rows as f16 [n_seq*nh*T][hd], each scaled by 2^-e, instead of q_prep
    float *rs;                           //         and scale * 2^e * log2(e) per row
    float scale;
    const float *q_norm_w, *k_norm_w, *inv_freq;
    int nh, rope_dim, gated, T;
    int row0;                            // first row handled (nh skips the query heads)
    float eps;
    int *group_ctr;                      // if set: n_ctr arrival counters of the decode kernel's fused merge, zeroed here
    int n_ctr;
};

// Row j of token tt: j < nh is a query head (normalise, rotate, write f32 to the
// scratch the attention kernels read); the next nkv rows are key heads
// (normalise, rotate, encode into the cache); the last nkv rows are value heads
// (encode as they are).  Reference: src/ornith_rforward.c:432-447 and the append
// half of ornith_gqa_step (src/ornith_attn.c:94-110).
template <typename ACT>
__global__ void __launch_bounds__(128) k_full_prep(PrepArgs a) {
    extern __shared__ float row[];
    __shared__ double redd[32];
    __shared__ float redf[32];
    const int hd = a.kv.hd, nkv = a.kv.nkv, nh = a.nh;
    // Launched as a programmatic dependent of the kernel in front of it (the layer before): resident when that kernel
    // ends, and waiting for its end before anything else.  After that a decode kernel launched behind this one may
    // begin its prologue (it streams cache rows early, and waits for this grid before it reads its output).
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    if (a.group_ctr)
        for (int i = (blockIdx.y * gridDim.x + blockIdx.x) * 128 + threadIdx.x; i < a.n_ctr; i += gridDim.x * gridDim.y * 128)
            a.group_ctr[i] = 0;
    const int j = blockIdx.y + a.row0, tt = blockIdx.x, b = tt / a.T, t = tt % a.T;
    const int64_t base = a.kv.seq_off[b];
    const int cap = (int)(a.kv.seq_off[b + 1] - base);
    const int slot = a.kv_len[b] + t;
    if (slot >= cap) return;                              // full cache: silent no-op
    const int pos = (a.rope_pos ? a.rope_pos[b] : a.kv_len[b]) + t;

    int kind, h;
    const ACT *src;
    const float *w;
    if (j < nh) {
        kind = 0; h = j; w = a.q_norm_w;
        size_t per_tok = (size_t)nh * hd * (a.gated ? 2 : 1);
        src = (const ACT *)a.qproj + (size_t)tt * per_tok + (size_t)h * hd * (a.gated ? 2 : 1);
    } else if (j < nh + nkv) {
        kind = 1; h = j - nh; w = a.k_norm_w;
        src = (const ACT *)a.k + ((size_t)tt * nkv + h) * hd;
    } else {
        kind = 2; h = j - nh - nkv; w = nullptr;
        src = (const ACT *)a.v + ((size_t)tt * nkv + h) * hd;
    }
    for (int i = threadIdx.x; i < hd; i += blockDim.x) row[i] = act_ld(src, i);
    __syncthreads();

    if (w) {                                              // RMSNorm, f64 sum like the engine
        double ss = 0.0;
        for (int i = threadIdx.x; i < hd; i += blockDim.x) ss += (double)row[i] * (double)row[i];
        ss = block_sum(ss, redd);
        float inv = (float)(1.0 / sqrt(ss / (double)hd + (double)a.eps));
        for (int i = threadIdx.x; i < hd; i += blockDim.x)
            row[i] = __fmul_rn(__fmul_rn(row[i], inv), w[i]);
        __syncthreads();
    }
    if (kind != 2 && a.rope_dim > 0) {                    // partial RoPE, rotate-half pairs
        const int half = a.rope_dim / 2;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            float ang = __fmul_rn((float)pos, a.inv_freq[i]);
            float c = cosf(ang), s = sinf(ang);
            float lo = row[i], hi = row[i + half];
            row[i]        = __fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, s));
            row[i + half] = __fadd_rn(__fmul_rn(lo, s), __fmul_rn(hi, c));
        }
        __syncthreads();
    }

    if (kind == 0) {
        float *dst = a.q_prep + ((size_t)tt * nh + h) * hd;
        for (int i = threadIdx.x; i < hd; i += blockDim.x) dst[i] = row[i];
        return;
    }
    const size_t r = (size_t)(base + slot) * nkv + h;
    uint8_t *pool = (kind == 1) ? a.kv.K : a.kv.V;
    if (a.kv.mode == ORNITH_KV_F32) {
        float *dst = reinterpret_cast<float *>(pool) + r * hd;
        for (int i = threadIdx.x; i < hd; i += blockDim.x) dst[i] = row[i];
    } else if (a.kv.mode == ORNITH_KV_Q8_0) {
        encode_row_q8_0(row, hd, pool + r * kv_row_bytes(ORNITH_KV_Q8_0, hd));
    } else {
        float *sc = ((kind == 1) ? a.kv.Ks : a.kv.Vs) + r;
        encode_row_int8(row, hd, reinterpret_cast<int8_t *>(pool) + r * hd, sc, redf);
    }
}

// The same work with one warp per row and four rows per CTA, for prefill, where the
// rows number in the millions and a CTA with block barriers per row is launch-bound.
// Same products, sums (f64 sum of squares) and rounding as k_full_prep.
template <typename ACT>
__global__ void __launch_bounds__(128) k_full_prep_warp(PrepArgs a, long long n_rows, int rows_per_tok) {
    extern __shared__ float rowbuf[];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int hd = a.kv.hd, nkv = a.kv.nkv, nh = a.nh;
    if (a.group_ctr)
        for (long long i = (long long)blockIdx.x * 128 + threadIdx.x; i < a.n_ctr; i += (long long)gridDim.x * 128)
            a.group_ctr[i] = 0;
    const long long R = (long long)blockIdx.x * 4 + wid;
    if (R >= n_rows) return;
    const int tt = (int)(R / rows_per_tok), j = (int)(R % rows_per_tok) + a.row0, b = tt / a.T, t = tt % a.T;
    const int64_t base = a.kv.seq_off[b];
    const int cap = (int)(a.kv.seq_off[b + 1] - base);
    const int slot = a.kv_len[b] + t;
    if (slot >= cap) return;                              // full cache: silent no-op
    const int pos = (a.rope_pos ? a.rope_pos[b] : a.kv_len[b]) + t;
    float *row = rowbuf + wid * hd;

    int kind, h;
    const ACT *src;
    const float *w;
    if (j < nh) {
        kind = 0; h = j; w = a.q_norm_w;
        size_t per_tok = (size_t)nh * hd * (a.gated ? 2 : 1);
        src = (const ACT *)a.qproj + (size_t)tt * per_tok + (size_t)h * hd * (a.gated ? 2 : 1);
    } else if (j < nh + nkv) {
        kind = 1; h = j - nh; w = a.k_norm_w;
        src = (const ACT *)a.k + ((size_t)tt * nkv + h) * hd;
    } else {
        kind = 2; h = j - nh - nkv; w = nullptr;
        src = (const ACT *)a.v + ((size_t)tt * nkv + h) * hd;
    }
    for (int i = lane; i < hd; i += 32) row[i] = act_ld(src, i);
    __syncwarp();
    if (w) {
        double ss = 0.0;
        for (int i = lane; i < hd; i += 32) ss += (double)row[i] * (double)row[i];
        ss = warp_sum(ss);
        const float inv = (float)(1.0 / sqrt(ss / (double)hd + (double)a.eps));
        for (int i = lane; i < hd; i += 32) row[i] = __fmul_rn(__fmul_rn(row[i], inv), w[i]);
        __syncwarp();
    }
    if (kind != 2 && a.rope_dim > 0) {
        const int half = a.rope_dim / 2;
        for (int i = lane; i < half; i += 32) {
            float ang = __fmul_rn((float)pos, a.inv_freq[i]);
            float c = cosf(ang), s = sinf(ang);
            float lo = row[i], hi = row[i + half];
            row[i]        = __fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, s));
            row[i + half] = __fadd_rn(__fmul_rn(lo, s), __fmul_rn(hi, c));
        }
        __syncwarp();
    }
    if (kind == 0) {
        if (a.Qh) {                                       // f16 image for the tensor-core kernel (hd = 256)
            float mx = 0.0f;
            for (int i = lane; i < hd; i += 32) mx = fmaxf(mx, fabsf(row[i]));
            mx = warp_max(mx);
            int e = 0;
            if (mx > 0.0f && mx < INFINITY) (void)frexpf(mx, &e);
            const float down = exp2f((float)-e);
            const size_t orow = ((size_t)b * nh + h) * a.T + t;
            const float *src8 = row + lane * 8;           // hd = 256: eight values per lane
            __half2 p0 = __floats2half2_rn(src8[0] * down, src8[1] * down), p1 = __floats2half2_rn(src8[2] * down, src8[3] * down);
            __half2 p2 = __floats2half2_rn(src8[4] * down, src8[5] * down), p3 = __floats2half2_rn(src8[6] * down, src8[7] * down);
            *reinterpret_cast<uint4 *>(a.Qh + orow * hd + lane * 8) =
                make_uint4(*reinterpret_cast<uint32_t *>(&p0), *reinterpret_cast<uint32_t *>(&p1),
                           *reinterpret_cast<uint32_t *>(&p2), *reinterpret_cast<uint32_t *>(&p3));
            if (lane == 0) a.rs[orow] = a.scale * exp2f((float)e) * 1.4426950408889634f;
            return;
        }
        float *dst = a.q_prep + ((size_t)tt * nh + h) * hd;
        for (int i = lane; i < hd; i += 32) dst[i] = row[i];
        return;
    }
    const size_t r = (size_t)(base + slot) * nkv + h;
    uint8_t *pool = (kind == 1) ? a.kv.K : a.kv.V;
    if (a.kv.mode == ORNITH_KV_F32) {
        float *dst = reinterpret_cast<float *>(pool) + r * hd;
        for (int i = lane; i < hd; i += 32) dst[i] = row[i];
    } else if (a.kv.mode == ORNITH_KV_Q8_0) {
        uint8_t *dst = pool + r * kv_row_bytes(ORNITH_KV_Q8_0, hd);
        for (int blk = 0; blk < hd / 32; blk++) {         // as encode_row_q8_0, all blocks by this warp
            const float x = row[blk * 32 + lane];
            const float amax = warp_max(fabsf(x));
            const float d = __fdiv_rn(amax, 127.0f);
            const float id = (d != 0.0f) ? __fdiv_rn(1.0f, d) : 0.0f;
            int q = (int)roundf(__fmul_rn(x, id));
            q = max(-127, min(127, q));
            uint8_t *o = dst + (size_t)blk * 34;
            if (lane == 0) *reinterpret_cast<unsigned short *>(o) = __half_as_ushort(__float2half_rn(d));
            o[2 + lane] = (uint8_t)(int8_t)q;
        }
    } else {                                              // as encode_row_int8
        int8_t *codes = reinterpret_cast<int8_t *>(pool) + r * hd;
        float *sc = ((kind == 1) ? a.kv.Ks : a.kv.Vs) + r;
        float m = 0.0f;
        for (int i = lane; i < hd; i += 32) m = fmaxf(m, fabsf(row[i]));
        const float amax = warp_max(m);
        if (amax == 0.0f) {
            for (int i = lane; i < hd; i += 32) codes[i] = 0;
            if (lane == 0) *sc = 0.0f;
            return;
        }
        const float inv = __fdiv_rn(127.0f, amax);
        for (int i = lane; i < hd; i += 32) {
            const int q = __float2int_rn(__fmul_rn(row[i], inv));
            codes[i] = (int8_t)max(-127, min(127, q));
        }
        if (lane == 0) *sc = __fdiv_rn(amax, 127.0f);
    }
}

// head_dim = 256, one warp per row, a lane owns 8 adjacent elements: one 16-byte (bf16) or two (f32) loads per lane
// instead of eight 2-byte ones, everything but the rotation in registers, and a Q8_0 row leaves as 17 chunks of 16
// bytes.  Same products and rounding as k_full_prep_warp; the f64 sum of squares adds a lane's 8 squares first.
__device__ __forceinline__ void ld_row8(const __nv_bfloat16 *src, int lane, float (&v)[8]) {
    const uint4 u = *reinterpret_cast<const uint4 *>(src + lane * 8);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; i++) { v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
}
__device__ __forceinline__ void ld_row8(const float *src, int lane, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4 *>(src + lane * 8), b = *reinterpret_cast<const float4 *>(src + lane * 8 + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

template <typename ACT>
__global__ void __launch_bounds__(128) k_full_prep_row8(PrepArgs a, long long n_rows, int rows_per_tok) {
    constexpr int hd = 256;
    __shared__ __align__(16) float rowbuf[4][hd];          // the rotation's exchange; then the encoded Q8_0 row (272 bytes)
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int nkv = a.kv.nkv, nh = a.nh;
    // Launched as a programmatic dependent of the kernel in front of it (in a decode step: the layer before): resident
    // when that kernel ends, and waiting for its end before anything else.  After that a decode kernel launched behind
    // this one may begin its prologue (it streams cache rows early, and waits for this grid before it reads its output).
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    if (a.group_ctr)
        for (long long i = (long long)blockIdx.x * 128 + threadIdx.x; i < a.n_ctr; i += (long long)gridDim.x * 128)
            a.group_ctr[i] = 0;
    const long long R = (long long)blockIdx.x * 4 + wid;
    if (R >= n_rows) return;
    const int tt = (int)(R / rows_per_tok), j = (int)(R % rows_per_tok) + a.row0, b = tt / a.T, t = tt % a.T;
    const int64_t base = a.kv.seq_off[b];
    const int cap = (int)(a.kv.seq_off[b + 1] - base);
    const int slot = a.kv_len[b] + t;
    if (slot >= cap) return;                              // full cache: silent no-op
    const int pos = (a.rope_pos ? a.rope_pos[b] : a.kv_len[b]) + t;
    float *row = rowbuf[wid];

    int kind, h;
    const ACT *src;
    const float *w;
    if (j < nh) {
        kind = 0; h = j; w = a.q_norm_w;
        const size_t per_tok = (size_t)nh * hd * (a.gated ? 2 : 1);
        src = (const ACT *)a.qproj + (size_t)tt * per_tok + (size_t)h * hd * (a.gated ? 2 : 1);
    } else if (j < nh + nkv) {
        kind = 1; h = j - nh; w = a.k_norm_w;
        src = (const ACT *)a.k + ((size_t)tt * nkv + h) * hd;
    } else {
        kind = 2; h = j - nh - nkv; w = nullptr;
        src = (const ACT *)a.v + ((size_t)tt * nkv + h) * hd;
    }
    float v[8];
    ld_row8(src, lane, v);
    if (w) {
        double ss = 0.0;
#pragma unroll
        for (int i = 0; i < 8; i++) ss += (double)v[i] * (double)v[i];
        ss = warp_sum(ss);
        const float inv = (float)(1.0 / sqrt(ss / (double)hd + (double)a.eps));
        float wv[8];
        ld_row8(w, lane, wv);
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = __fmul_rn(__fmul_rn(v[i], inv), wv[i]);
    }
    if (kind != 2 && a.rope_dim > 0) {                    // pairs (i, i + half) sit in different lanes: through shared memory
        const int half = a.rope_dim / 2;
        if (lane * 8 < a.rope_dim) {
            *reinterpret_cast<float4 *>(row + lane * 8) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4 *>(row + lane * 8 + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
        __syncwarp();
        for (int i = lane; i < half; i += 32) {
            const float ang = __fmul_rn((float)pos, a.inv_freq[i]);
            const float c = cosf(ang), sn = sinf(ang);
            const float lo = row[i], hi = row[i + half];
            row[i]        = __fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, sn));
            row[i + half] = __fadd_rn(__fmul_rn(lo, sn), __fmul_rn(hi, c));
        }
        __syncwarp();
        if (lane * 8 < a.rope_dim) {
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = (lane * 8 + i < a.rope_dim) ? row[lane * 8 + i] : v[i];
        }
        __syncwarp();
    }
    if (kind == 0) {
        if (a.Qh) {                                       // f16 image for the tensor-core kernel
            float mx = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; i++) mx = fmaxf(mx, fabsf(v[i]));
            mx = warp_max(mx);
            int e = 0;
            if (mx > 0.0f && mx < INFINITY) (void)frexpf(mx, &e);
            const float down = exp2f((float)-e);
            const size_t orow = ((size_t)b * nh + h) * a.T + t;
            __half2 p0 = __floats2half2_rn(v[0] * down, v[1] * down), p1 = __floats2half2_rn(v[2] * down, v[3] * down);
            __half2 p2 = __floats2half2_rn(v[4] * down, v[5] * down), p3 = __floats2half2_rn(v[6] * down, v[7] * down);
            *reinterpret_cast<uint4 *>(a.Qh + orow * hd + lane * 8) =
                make_uint4(*reinterpret_cast<uint32_t *>(&p0), *reinterpret_cast<uint32_t *>(&p1),
                           *reinterpret_cast<uint32_t *>(&p2), *reinterpret_cast<uint32_t *>(&p3));
            if (lane == 0) a.rs[orow] = a.scale * exp2f((float)e) * 1.4426950408889634f;
            return;
        }
        float *dst = a.q_prep + ((size_t)tt * nh + h) * hd + lane * 8;
        *reinterpret_cast<float4 *>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
        return;
    }
    const size_t r = (size_t)(base + slot) * nkv + h;
    uint8_t *pool = (kind == 1) ? a.kv.K : a.kv.V;
    if (a.kv.mode == ORNITH_KV_F32) {
        float *dst = reinterpret_cast<float *>(pool) + r * hd + lane * 8;
        *reinterpret_cast<float4 *>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
    } else if (a.kv.mode == ORNITH_KV_Q8_0) {
        // as encode_row_q8_0: a block of 32 = 4 lanes
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[i]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const float d = __fdiv_rn(amax, 127.0f);
        const float id = (d != 0.0f) ? __fdiv_rn(1.0f, d) : 0.0f;
        uint8_t *enc = reinterpret_cast<uint8_t *>(row);   // 272 bytes of this warp's buffer
        uint8_t *o = enc + (lane >> 2) * 34;
        if ((lane & 3) == 0) *reinterpret_cast<unsigned short *>(o) = __half_as_ushort(__float2half_rn(d));
#pragma unroll
        for (int i = 0; i < 8; i += 2) {                  // code pairs: the block's codes start 2 bytes into it
            int q0 = (int)roundf(__fmul_rn(v[i], id)), q1 = (int)roundf(__fmul_rn(v[i + 1], id));
            q0 = max(-127, min(127, q0)); q1 = max(-127, min(127, q1));
            *reinterpret_cast<unsigned short *>(o + 2 + 8 * (lane & 3) + i) = (unsigned short)((q0 & 255) | ((q1 & 255) << 8));
        }
        __syncwarp();
        if (lane < 17)
            reinterpret_cast<uint4 *>(pool + r * kv_row_bytes(ORNITH_KV_Q8_0, hd))[lane] = reinterpret_cast<const uint4 *>(enc)[lane];
    } else {                                              // as encode_row_int8
        int8_t *codes = reinterpret_cast<int8_t *>(pool) + r * hd;
        float *sc = ((kind == 1) ? a.kv.Ks : a.kv.Vs) + r;
        float m = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) m = fmaxf(m, fabsf(v[i]));
        const float amax = warp_max(m);
        uint2 packed = make_uint2(0u, 0u);
        if (amax != 0.0f) {
            const float inv = __fdiv_rn(127.0f, amax);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int q = max(-127, min(127, __float2int_rn(__fmul_rn(v[i], inv))));
                if (i < 4) packed.x |= (uint32_t)(q & 255) << (8 * i);
                else packed.y |= (uint32_t)(q & 255) << (8 * (i - 4));
            }
        }
        *reinterpret_cast<uint2 *>(codes + lane * 8) = packed;
        if (lane == 0) *sc = amax != 0.0f ? __fdiv_rn(amax, 127.0f) : 0.0f;
    }
}

// =============================================================================
// split-K decode, generic in head_dim and group size
// =============================================================================

// One CTA = one (split, query head, sequence).  Scores are one thread per token
// with the engine's element order; the value pass is one thread per dimension.
// Partial (m, l, o) go to scratch for k_gqa_combine.
template <int MODE>
__global__ void __launch_bounds__(128) k_gqa_decode_generic(DecodeArgs a) {
    extern __shared__ float sm[];
    const int hd = a.kv.hd, nkv = a.kv.nkv;
    float *q_s = sm, *p_s = sm + hd;                      // [hd], [128]
    __shared__ float red[32];
    const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z, tid = threadIdx.x;
    const int64_t base = a.kv.seq_off[b];
    const int cap = (int)(a.kv.seq_off[b + 1] - base);
    const int len0 = a.kv_len[b];
    if (len0 >= cap) return;
    const int L = len0 + 1;
    float *part = a.part + (((size_t)b * a.nh + h) * a.nsplit + split) * (hd + 2);
    const int t0 = split * a.tokens_per_split, t1 = min(L, t0 + a.tokens_per_split);
    if (t0 >= L) {
        if (tid == 0) { part[0] = -INFINITY; part[1] = 0.0f; }
        return;
    }
    const int kvh = h / (a.nh / nkv);
    const size_t rb = kv_row_bytes(MODE, hd);
    for (int i = tid; i < hd; i += 128) q_s[i] = a.q_prep[((size_t)b * a.nh + h) * hd + i];
    __syncthreads();

    float m_run = -INFINITY, l_run = 0.0f, acc[8];
#pragma unroll
    for (int i = 0; i < 8; i++) acc[i] = 0.0f;

    for (int tb = t0; tb < t1; tb += 128) {
        const int tok = tb + tid;
        const bool valid = tok < t1;
        float s = -INFINITY, vscale = 1.0f;
        if (valid) {
            const size_t r = (size_t)(base + tok) * nkv + kvh;
            const uint8_t *krow = a.kv.K + r * rb;
            float dot = 0.0f;
            for (int d = 0; d < hd; d++) dot += q_s[d] * kv_elem<MODE>(krow, d);
            if (MODE == ORNITH_KV_INT8_HEAD) {
                float ks = a.kv.Ks[r];
                dot = (ks == 0.0f) ? 0.0f : dot * ks;
                vscale = a.kv.Vs[r];
            }
            s = dot * a.scale;
        }
        const float m_new = fmaxf(m_run, block_max(s, red));
        const float p = valid ? expf(s - m_new) : 0.0f;
        const float corr = expf(m_run - m_new);           // 0 on the first tile
        l_run = l_run * corr + block_sum(p, red);
        m_run = m_new;
        p_s[tid] = p * vscale;
        __syncthreads();
        const int n = min(128, t1 - tb);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int d = tid + i * 128;
            if (d < hd) {
                float o = acc[i] * corr;
                for (int tt = 0; tt < n; tt++) {
                    const uint8_t *vrow = a.kv.V + ((size_t)(base + tb + tt) * nkv + kvh) * rb;
                    o += p_s[tt] * kv_elem<MODE>(vrow, d);
                }
                acc[i] = o;
            }
        }
        __syncthreads();
    }
    if (tid == 0) { part[0] = m_run; part[1] = l_run; }
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int d = tid + i * 128;
        if (d < hd) part[2 + d] = acc[i];
    }
}

struct CombineArgs {
    KvView kv;
    const int32_t *kv_len;
    const float *part;
    const void *qproj;                   // for the gate half, when gated
    void *out;
    int nh, nsplit, gated;
    int tokens_per_split;                // splits past the sequence's context hold nothing
};

// Merge the split partials of one (head, sequence), normalise, apply the sigmoid
// output gate (reference: src/ornith_rforward.c:450) and store.
template <typename ACT>
__global__ void __launch_bounds__(128) k_gqa_combine(CombineArgs a) {
    extern __shared__ float w_s[];                       // [nsplit]
    __shared__ float red[32];
    const int hd = a.kv.hd, h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
    const int cap = (int)(a.kv.seq_off[b + 1] - a.kv.seq_off[b]);
    const int len0 = a.kv_len[b];
    if (len0 >= cap) return;
    const float *part = a.part + ((size_t)b * a.nh + h) * a.nsplit * (hd + 2);
    const int nlive = min(a.nsplit, (len0 + a.tokens_per_split) / a.tokens_per_split);   // ceil((len0+1)/tps)
    float m = -INFINITY;
    for (int s = tid; s < nlive; s += 128)
        if (part[(size_t)s * (hd + 2) + 1] > 0.0f) m = fmaxf(m, part[(size_t)s * (hd + 2)]);
    const float M = block_max(m, red);
    float lsum = 0.0f;
    for (int s = tid; s < nlive; s += 128) {
        const float l = part[(size_t)s * (hd + 2) + 1];
        const float w = (l > 0.0f) ? expf(part[(size_t)s * (hd + 2)] - M) : 0.0f;
        w_s[s] = w;
        lsum += l * w;
    }
    const float Lsum = block_sum(lsum, red);              // also orders the w_s writes
    const float inv = 1.0f / Lsum;
    const ACT *gate = nullptr;
    if (a.gated) gate = (const ACT *)a.qproj + (size_t)b * a.nh * hd * 2 + (size_t)h * hd * 2 + hd;
    ACT *out = (ACT *)a.out + ((size_t)b * a.nh + h) * hd;
    for (int d = tid; d < hd; d += 128) {
        float o = 0.0f;
        for (int s = 0; s < nlive; s++)
            if (w_s[s] != 0.0f) o += part[(size_t)s * (hd + 2) + 2 + d] * w_s[s];
        o *= inv;
        if (gate) o *= sigmoid_f(act_ld(gate, d));
        act_st(out, d, o);
    }
}

// =============================================================================
// causal prefill (f32 accumulate, online softmax), generic in head_dim
// =============================================================================

struct PrefillArgs {
    KvView kv;
    const int32_t *kv_len;
    const float *q_prep;                 // [n_seq*T][nh][hd]
    const void *qproj;
    void *out;
    int nh, T, gated, hpb, tpb;          // heads / tokens per block, hpb*tpb == 8
    float scale;
};

constexpr int PF_KT = 32;                // keys per shared-memory tile

// One CTA = 8 (token, head) pairs that share a kv head: warp w owns pair w.
// K and V tiles are decoded to f32 in shared memory once per CTA.  Score phase:
// lane = key; value phase: lane = dimension slice.
template <int MODE, typename ACT>
__global__ void __launch_bounds__(256) k_gqa_prefill(PrefillArgs a) {
    extern __shared__ float sm[];
    const int hd = a.kv.hd, nkv = a.kv.nkv, ldk = hd + 1;   // odd stride: lane = key reads are conflict-free
    float *K_s = sm;                                      // [PF_KT][hd + 1]
    float *V_s = K_s + PF_KT * ldk;                       // [PF_KT][hd]
    float *q_s = V_s + PF_KT * hd;                        // [8][hd]
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int b = blockIdx.z;
    const int groups_per_kv = (a.nh / nkv) / a.hpb;       // head sub-groups per kv head
    const int kvh = blockIdx.y / groups_per_kv;
    const int h = kvh * (a.nh / nkv) + (blockIdx.y % groups_per_kv) * a.hpb + (w % a.hpb);
    const int t = blockIdx.x * a.tpb + (w / a.hpb);       // token of this warp
    const int64_t base = a.kv.seq_off[b];
    const int cap = (int)(a.kv.seq_off[b + 1] - base);
    const int len0 = a.kv_len[b];
    const bool live = (t < a.T) && (len0 + t < cap);      // appended tokens only
    const int qpos = len0 + t;                            // attends keys 0..qpos
    const int t_last = min(a.T - 1, blockIdx.x * a.tpb + a.tpb - 1);
    const int kmax = min(len0 + t_last, cap - 1);         // last key any warp needs
    const size_t rb = kv_row_bytes(MODE, hd);
    const int ndim = (hd + 31) / 32;                      // dims per lane (<= 8 for hd <= 256), strided

    const size_t tok = (size_t)b * a.T + min(t, a.T - 1);
    for (int i = lane; i < hd; i += 32) q_s[w * hd + i] = a.q_prep[(tok * a.nh + h) * hd + i];

    float m_run = -INFINITY, l_run = 0.0f, acc[8];
#pragma unroll
    for (int i = 0; i < 8; i++) acc[i] = 0.0f;

    for (int kb = 0; kb <= kmax; kb += PF_KT) {
        __syncthreads();                                  // previous tile fully consumed
        for (int e = tid; e < PF_KT * hd; e += 256) {
            const int kk = e / hd, d = e % hd, kp = kb + kk;
            float kvv = 0.0f, vv = 0.0f;
            if (kp <= kmax) {
                const size_t r = (size_t)(base + kp) * nkv + kvh;
                kvv = kv_elem<MODE>(a.kv.K + r * rb, d);
                vv = kv_elem<MODE>(a.kv.V + r * rb, d);
                if (MODE == ORNITH_KV_INT8_HEAD) vv *= a.kv.Vs[r];
            }
            K_s[kk * ldk + d] = kvv;
            V_s[kk * hd + d] = vv;
        }
        __syncthreads();
        if (!live) continue;
        const int kp = kb + lane;
        float s = -INFINITY;
        if (kp <= qpos) {
            float dot = 0.0f;
            const float *kr = K_s + lane * ldk, *qr = q_s + w * hd;
            for (int d = 0; d < hd; d++) dot += qr[d] * kr[d];
            if (MODE == ORNITH_KV_INT8_HEAD) {
                float ks = a.kv.Ks[(size_t)(base + kp) * nkv + kvh];
                dot = (ks == 0.0f) ? 0.0f : dot * ks;
            }
            s = dot * a.scale;
        }
        const float tile_max = warp_max(s);
        if (tile_max == -INFINITY) continue;              // whole tile is in the future
        const float m_new = fmaxf(m_run, tile_max);
        const float p = (kp <= qpos) ? expf(s - m_new) : 0.0f;
        const float corr = expf(m_run - m_new);
        l_run = l_run * corr + warp_sum(p);
        m_run = m_new;
#pragma unroll
        for (int i = 0; i < 8; i++) acc[i] *= corr;
        for (int kk = 0; kk < PF_KT; kk++) {
            const float pk = __shfl_sync(0xffffffffu, p, kk);
            if (pk == 0.0f) continue;
#pragma unroll
            for (int i = 0; i < 8; i++)
                if (i < ndim) {
                    const int d = lane + i * 32;
                    if (d < hd) acc[i] += pk * V_s[kk * hd + d];
                }
        }
    }
    if (!live) return;
    const float inv = 1.0f / l_run;
    const ACT *gate = nullptr;
    const size_t otok = (size_t)b * a.T + t;
    if (a.gated) gate = (const ACT *)a.qproj + otok * a.nh * hd * 2 + (size_t)h * hd * 2 + hd;
    ACT *out = (ACT *)a.out + (otok * a.nh + h) * hd;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int d = lane + i * 32;
        if (i < ndim && d < hd) {
            float o = acc[i] * inv;
            if (gate) o *= sigmoid_f(act_ld(gate, d));
            act_st(out, d, o);
        }
    }
}

// =============================================================================
// host entry points
// =============================================================================

static float attn_scale(const ornith_cuda_full_layer *l) {
    return l->scale > 0.0f ? l->scale : 1.0f / sqrtf((float)l->head_dim);
}

static ornith_status check_full(const ornith_cuda_full_layer *l, const ornith_cuda_kv *kv) {
    if (!l || !kv || l->n_heads <= 0 || l->n_kv_heads <= 0 || l->head_dim <= 0 ||
        l->n_heads % l->n_kv_heads || kv->n_kv_heads != l->n_kv_heads || kv->head_dim != l->head_dim) {
        orn_record_error("full attention: inconsistent layer / cache geometry");
        return ORNITH_ERR_FORMAT;
    }
    if (l->head_dim > 1024) { orn_record_error("full attention: head_dim > 1024 unsupported"); return ORNITH_ERR_UNSUPPORTED; }
    if (kv->mode == ORNITH_KV_Q8_0 && l->head_dim % 32) {
        orn_record_error("Q8_0 KV rows need head_dim to be a multiple of 32");
        return ORNITH_ERR_FORMAT;
    }
    if (kv->mode < 0 || kv->mode > 2) { orn_record_error("unknown KV mode %d", kv->mode); return ORNITH_ERR_FORMAT; }
    if (l->rope_dim > 0 && (!l->rope_inv_freq || l->rope_dim > l->head_dim || (l->rope_dim & 1))) {
        orn_record_error("full attention: bad rope_dim %d or missing inverse-frequency table", l->rope_dim);
        return ORNITH_ERR_FORMAT;
    }
    return ORNITH_OK;
}

// ORNITH_CUDA_GENERIC_DECODE=1 routes Q8_0 decode through the generic CUDA-core
// kernel (A/B comparison of the two device paths; both run on the GPU).
static bool force_generic_decode() {
    static int v = -1;
    if (v < 0) { const char *e = getenv("ORNITH_CUDA_GENERIC_DECODE"); v = (e && e[0] == '1') ? 1 : 0; }
    return v == 1;
}

static int split_tokens(int max_len) {
    // tokens per split: long contexts use 512-token splits; short ones fewer CTAs
    return max_len <= 512 ? 128 : 512;
}
// Split length of the tensor-core decode kernels.
// coarse: by context alone, the fewest partials (what the smallest accepted scratch holds).
static int split_tokens_coarse(int max_len) {
    return max_len > 16384 ? 2048 : (max_len > 8192 ? 1024 : (max_len > 1024 ? 512 : 256));
}
// fine: for batches too small to fill the GPU with coarse splits.  A CTA walks one split of one head group and
// 4 CTAs are resident per SM; if even at max_len the coarse splits give less than one wave (592 CTAs on 148
// SMs), the splits are shortened towards one wave, but never to more than about 32 per sequence: the last CTA
// of a group merges the group's partials alone, and past that its work outweighs the gain.  Batches that
// fill the GPU keep the coarse length (their CTA count depends on the actual contexts, which the host does
// not know).
static int split_tokens_fine(int max_len, long long n_groups) {
    const int coarse = split_tokens_coarse(max_len);
    if (n_groups * ((max_len + coarse - 1) / coarse) >= 592) return coarse;
    long long t = (n_groups * (long long)max_len / 592 + 63) / 64 * 64;
    const long long floor_t = ((max_len / 32 > 256 ? max_len / 32 : 256) + 63) / 64 * 64;
    if (t < floor_t) t = floor_t;
    return (int)(t < coarse ? t : coarse);
}
static long long head_groups(const ornith_cuda_full_layer *l, int n_seq) {
    const int g = l->n_heads / l->n_kv_heads;
    return (long long)n_seq * l->n_kv_heads * ((g + 7) / 8);
}
// Scratch of one decode step: query rows, one arrival counter per (sequence, head), then the partials.
//   SPLIT_TC  a tensor-core kernel with splits of tps_mma tokens serves the cache;
//   BALANCED  the Q8_0 raw-fragment kernel with its own schedule: a fixed number of partial slots per head;
//   ANY       the size query, which does not see the cache: the larger of the two, with the CUDA-core kernel's
//             fixed 512- or 128-token splits covered as well.  A step served by the CUDA-core kernel needs this too.
enum DecodePath { PATH_ANY, PATH_SPLIT_TC, PATH_BALANCED };
static size_t step_need(const ornith_cuda_full_layer *l, int n_seq, int max_len, int tps_mma, DecodePath path) {
    const int ta = split_tokens(max_len), t = path == PATH_ANY ? (ta < tps_mma ? ta : tps_mma) : tps_mma,
              nsplit = (max_len + t - 1) / t;
    size_t rows = (size_t)n_seq * l->n_heads * nsplit;
    if (path != PATH_SPLIT_TC && l->n_kv_heads > 0 && l->n_heads % l->n_kv_heads == 0) {
        const size_t bal = (size_t)l->n_heads * gqa_decode_q8_raw_slots(l->n_kv_heads, l->n_heads, n_seq, max_len);
        rows = path == PATH_BALANCED ? bal : (bal > rows ? bal : rows);
    }
    return align_up((size_t)n_seq * l->n_heads * l->head_dim * sizeof(float), 256) +
           align_up((size_t)n_seq * l->n_heads * sizeof(int), 256) +
           align_up(rows * (l->head_dim + 2) * sizeof(float), 256);
}

// Whether a decode step over this cache runs on one of the tensor-core kernels (the dispatch of
// ornith_cuda_full_attn_step below follows the same order).
static DecodePath decode_path(const ornith_cuda_full_layer *l, const ornith_cuda_kv *kv) {
    if (force_generic_decode()) return PATH_ANY;
    const KvView v = make_view(kv);
    if (gqa_decode_q8_raw_balanced(v, l->n_heads)) return PATH_BALANCED;
    return (gqa_decode_q8_mma_supported(v, l->n_heads) || gqa_decode_f32_tc_supported(v, l->n_heads) ||
            gqa_decode_i8_raw_supported(v, l->n_heads)) ? PATH_SPLIT_TC : PATH_ANY;
}

template <typename ACT>
static ornith_status launch_prep(const ornith_cuda_full_layer *l, const ornith_cuda_kv *kv,
                                 const int32_t *kv_len, const int32_t *rope_pos, const void *qproj,
                                 const void *k, const void *v, float *q_prep, int n_tok, int T,
                                 cudaStream_t st, bool kv_only = false, __half *Qh = nullptr, float *rs = nullptr,
                                 int *group_ctr = nullptr, int n_ctr = 0) {
    PrepArgs a;
    a.group_ctr = group_ctr; a.n_ctr = n_ctr;
    a.Qh = Qh; a.rs = rs; a.scale = attn_scale(l);
    a.kv = make_view(kv); a.kv_len = kv_len; a.rope_pos = rope_pos;
    a.qproj = qproj; a.k = k; a.v = v; a.q_prep = q_prep;
    a.q_norm_w = l->q_norm_w; a.k_norm_w = l->k_norm_w; a.inv_freq = l->rope_inv_freq;
    a.nh = l->n_heads; a.rope_dim = l->rope_dim; a.gated = l->gated; a.T = T; a.eps = l->eps;
    a.row0 = kv_only ? l->n_heads : 0;
    const int rows_per_tok = (kv_only ? 0 : l->n_heads) + 2 * l->n_kv_heads;
    // prefill-sized batches of head_dim 256 with 16-byte-aligned rows: one warp per row, a lane owns 8 adjacent elements
    // (rows of a token are multiples of 256 elements apart).  For a decode step it measures no faster than the
    // one-CTA-per-row kernel below (3.796 against 3.785 ms per step: the front end hides behind the layer before it).
    const bool aligned = (((uintptr_t)qproj | (uintptr_t)k | (uintptr_t)v | (uintptr_t)kv->K | (uintptr_t)kv->V |
                           (uintptr_t)l->q_norm_w | (uintptr_t)l->k_norm_w) & 15) == 0 &&
                         (!Qh || ((uintptr_t)Qh & 15) == 0) && (!q_prep || ((uintptr_t)q_prep & 15) == 0);
    static int row8_ok = -1;
    if (row8_ok < 0) { const char *e = getenv("ORNITH_CUDA_PREP_ROW8"); row8_ok = e ? atoi(e) : 1; }   // =0: the older kernels
    if (row8_ok && n_tok >= 256 && l->head_dim == 256 && aligned && l->rope_dim % 2 == 0 && l->rope_dim <= 256) {
        const long long n_rows = (long long)n_tok * rows_per_tok;
        return orn_check(orn_launch_dependent(k_full_prep_row8<ACT>, dim3((unsigned)((n_rows + 3) / 4)), dim3(128), 0, st, a, n_rows,
                                              rows_per_tok), "k_full_prep_row8");
    }
    if (n_tok >= 256) {                                   // prefill-sized: one warp per row
        const long long n_rows = (long long)n_tok * rows_per_tok;
        k_full_prep_warp<ACT><<<(unsigned)((n_rows + 3) / 4), 128, 4 * l->head_dim * sizeof(float), st>>>(a, n_rows,
                                                                                                      rows_per_tok);
        return orn_check_launch("k_full_prep_warp");
    }
    dim3 grid(n_tok, rows_per_tok);
    return orn_check(orn_launch_dependent(k_full_prep<ACT>, grid, dim3(128), l->head_dim * sizeof(float), st, a), "k_full_prep");
}

extern "C" {

size_t ornith_cuda_full_attn_step_scratch(const ornith_cuda_full_layer *l, int n_seq, int max_len) {
    if (!l || n_seq <= 0 || l->n_kv_heads <= 0) return 0;
    if (max_len < 1) max_len = 1;
    return step_need(l, n_seq, max_len, split_tokens_fine(max_len, head_groups(l, n_seq)), PATH_ANY);
}

ornith_status ornith_cuda_full_attn_step(const ornith_cuda_full_layer *l, const ornith_cuda_kv *kv,
                                         const int32_t *kv_len, const int32_t *rope_pos,
                                         const void *qproj, const void *k, const void *v, void *out,
                                         int act_dtype, int max_len, void *scratch, size_t scratch_bytes,
                                         void *stream) {
    ORN_TRY(orn_require_device());
    ORN_TRY(check_full(l, kv));
    const int B = kv->n_seq;
    if (B <= 0) return ORNITH_OK;
    if (max_len < 1) max_len = 1;
    // Split length of the tensor-core kernels: the fine one if the scratch holds its partials, else doubled until
    // it fits, down to the coarse one (ornith_cuda_full_attn_step_scratch asks for the fine one; a caller with a
    // fixed budget may pass less).  ORNITH_CUDA_DECODE_SPLIT=<tokens> overrides it when that fits too.
    int tps_mma = split_tokens_fine(max_len, head_groups(l, B));
    const DecodePath path = decode_path(l, kv);
    {
        const int coarse = split_tokens_coarse(max_len), tps_max = tps_mma > coarse ? tps_mma : coarse;
        while (step_need(l, B, max_len, tps_mma, path) > scratch_bytes && tps_mma < tps_max)
            tps_mma = (2 * tps_mma < tps_max) ? 2 * tps_mma : tps_max;
        static int forced = -1;
        if (forced < 0) { const char *e = getenv("ORNITH_CUDA_DECODE_SPLIT"); forced = e ? atoi(e) : 0; }
        if (forced >= 64 && step_need(l, B, max_len, forced / 64 * 64, path) <= scratch_bytes) tps_mma = forced / 64 * 64;
    }
    if (!scratch || step_need(l, B, max_len, tps_mma, path) > scratch_bytes) {
        orn_record_error("full_attn_step: scratch too small (%zu bytes given)", scratch_bytes);
        return ORNITH_ERR_FORMAT;
    }
    cudaStream_t st = as_stream(stream);
    const int hd = l->head_dim, nh = l->n_heads;
    const int tps = split_tokens(max_len), nsplit = (max_len + tps - 1) / tps;
    float *q_prep = (float *)scratch;
    int *group_ctr = (int *)((char *)scratch + align_up((size_t)B * nh * hd * sizeof(float), 256));
    float *part = (float *)((char *)group_ctr + align_up((size_t)B * nh * sizeof(int), 256));

    if (act_dtype == ORNITH_ACT_BF16)
        ORN_TRY(launch_prep<__nv_bfloat16>(l, kv, kv_len, rope_pos, qproj, k, v, q_prep, B, 1, st, false, nullptr, nullptr,
                                           group_ctr, B * nh));
    else
        ORN_TRY(launch_prep<float>(l, kv, kv_len, rope_pos, qproj, k, v, q_prep, B, 1, st, false, nullptr, nullptr,
                                   group_ctr, B * nh));

    DecodeArgs d;
    d.kv = make_view(kv); d.kv_len = kv_len; d.q_prep = q_prep; d.part = part;
    d.nh = nh; d.scale = attn_scale(l);
    d.group_ctr = group_ctr; d.qproj = qproj; d.out = out; d.gated = l->gated; d.act_dtype = act_dtype;
    d.n_seq = B; d.max_len = max_len; d.status = nullptr; d.piece_cost = 0;
    bool merged = false;
    int nsplit_used;
    if (gqa_decode_q8_mma_supported(d.kv, nh) && !force_generic_decode()) {
        d.tokens_per_split = tps_mma; d.nsplit = nsplit_used = (max_len + tps_mma - 1) / tps_mma;
        if (path == PATH_BALANCED) d.nsplit = nsplit_used = gqa_decode_q8_raw_slots(l->n_kv_heads, nh, B, max_len);
        ORN_TRY(launch_gqa_decode_q8_mma(d, B, st, &merged));
    } else if (gqa_decode_f32_tc_supported(d.kv, nh) && !force_generic_decode()) {
        d.tokens_per_split = tps_mma; d.nsplit = nsplit_used = (max_len + tps_mma - 1) / tps_mma;
        ORN_TRY(launch_gqa_decode_f32_tc(d, B, st));
    } else if (gqa_decode_i8_raw_supported(d.kv, nh) && !force_generic_decode()) {
        d.tokens_per_split = tps_mma; d.nsplit = nsplit_used = (max_len + tps_mma - 1) / tps_mma;
        ORN_TRY(launch_gqa_decode_i8_raw(d, B, st));
    } else {
        d.tokens_per_split = tps; d.nsplit = nsplit_used = nsplit;
        dim3 grid(nsplit, nh, B);
        const size_t smem = (size_t)(hd + 128) * sizeof(float);
        switch (kv->mode) {
        case ORNITH_KV_F32:       k_gqa_decode_generic<ORNITH_KV_F32><<<grid, 128, smem, st>>>(d); break;
        case ORNITH_KV_INT8_HEAD: k_gqa_decode_generic<ORNITH_KV_INT8_HEAD><<<grid, 128, smem, st>>>(d); break;
        default:                  k_gqa_decode_generic<ORNITH_KV_Q8_0><<<grid, 128, smem, st>>>(d); break;
        }
        ORN_TRY(orn_check_launch("k_gqa_decode_generic"));
    }

    if (merged) return ORNITH_OK;
    CombineArgs c;
    c.kv = d.kv; c.kv_len = kv_len; c.part = part; c.qproj = qproj; c.out = out;
    c.nh = nh; c.nsplit = nsplit_used; c.gated = l->gated; c.tokens_per_split = d.tokens_per_split;
    dim3 cgrid(nh, B);
    if (act_dtype == ORNITH_ACT_BF16)
        k_gqa_combine<__nv_bfloat16><<<cgrid, 128, nsplit_used * sizeof(float), st>>>(c);
    else
        k_gqa_combine<float><<<cgrid, 128, nsplit_used * sizeof(float), st>>>(c);
    return orn_check_launch("k_gqa_combine");
}

// The f32 image of the prepared query rows is only read by the kernels other than the tcgen05 one: when that
// kernel will run (head_dim 256, at least 256 rows so that the warp-per-row front end writes the f16 image itself)
// it is not reserved.
static size_t prefill_q_f32_bytes(const ornith_cuda_full_layer *l, int n_seq, int T) {
    const bool f16_image_only = l->head_dim == 256 && !force_generic_decode() && (long long)n_seq * T >= 256 && gqa_prefill_tc_selected();
    return f16_image_only ? 0 : align_up((size_t)n_seq * T * l->n_heads * l->head_dim * sizeof(float), 256);
}

size_t ornith_cuda_full_attn_prefill_scratch(const ornith_cuda_full_layer *l, int n_seq, int T, int max_len) {
    if (!l || n_seq <= 0 || T <= 0) return 0;
    if (max_len < T) max_len = T;
    size_t q = prefill_q_f32_bytes(l, n_seq, T);
    // decoded f16 image of the visible cache rows and the f16 query image, used by the tensor-core path
    if (l->head_dim == 256) q += gqa_prefill_mma_scratch(n_seq, l->n_kv_heads, l->n_heads, T, max_len);
    return q;
}

}  // extern "C"

template <int MODE, typename ACT>
static ornith_status launch_prefill(const PrefillArgs &a, dim3 grid, size_t smem, cudaStream_t st) {
    static bool configured_dev[ORN_MAX_DEVICES] = {};
    bool &configured = configured_dev[orn_device_index()];                      // per instantiation
    if (!configured) {
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_gqa_prefill<MODE, ACT>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024),
                          "prefill smem opt-in"));
        configured = true;
    }
    k_gqa_prefill<MODE, ACT><<<grid, 256, smem, st>>>(a);
    return orn_check_launch("k_gqa_prefill");
}

extern "C" {

ornith_status ornith_cuda_full_attn_prefill(const ornith_cuda_full_layer *l, const ornith_cuda_kv *kv,
                                            const int32_t *kv_len, const int32_t *rope_pos,
                                            const void *qproj, const void *k, const void *v, void *out,
                                            int act_dtype, int T, int max_len, void *scratch,
                                            size_t scratch_bytes, void *stream) {
    ORN_TRY(orn_require_device());
    ORN_TRY(check_full(l, kv));
    const int B = kv->n_seq;
    if (B <= 0 || T <= 0) return ORNITH_OK;
    if (max_len < T) max_len = T;
    if (l->head_dim > 256) { orn_record_error("prefill: head_dim > 256 unsupported"); return ORNITH_ERR_UNSUPPORTED; }
    if (scratch_bytes < ornith_cuda_full_attn_prefill_scratch(l, B, T, max_len) || !scratch) {
        orn_record_error("full_attn_prefill: scratch too small (%zu bytes given)", scratch_bytes);
        return ORNITH_ERR_FORMAT;
    }
    cudaStream_t st = as_stream(stream);
    const int hd = l->head_dim, nh = l->n_heads, G = nh / l->n_kv_heads;
    const size_t q_f32 = prefill_q_f32_bytes(l, B, T);
    float *q_prep = q_f32 ? (float *)scratch : nullptr;
    const bool bf = act_dtype == ORNITH_ACT_BF16;
    const bool tensor_path = gqa_prefill_mma_supported(make_view(kv)) && !force_generic_decode();
    void *kvh = (char *)scratch + q_f32;
    __half *Qh = nullptr;
    float *rs = nullptr;
    // the warp-per-row front end (B * T >= 256) writes the f16 query image of the tcgen05 kernel itself
    const bool q_image = tensor_path && (long long)B * T >= 256 &&
                         gqa_prefill_q_image(kvh, B, l->n_kv_heads, nh, T, max_len, &Qh, &rs);
    if (!q_image) { Qh = nullptr; rs = nullptr; }
    if (!q_image && !q_prep) {
        orn_record_error("full_attn_prefill: the scratch must be 16-byte aligned");
        return ORNITH_ERR_FORMAT;
    }
    if (bf) ORN_TRY(launch_prep<__nv_bfloat16>(l, kv, kv_len, rope_pos, qproj, k, v, q_prep, B * T, T, st, false, Qh, rs));
    else    ORN_TRY(launch_prep<float>(l, kv, kv_len, rope_pos, qproj, k, v, q_prep, B * T, T, st, false, Qh, rs));

    if (tensor_path) {
        return launch_gqa_prefill_mma(make_view(kv), kv_len, q_image ? nullptr : q_prep, kvh, qproj, out, nh, T, max_len, l->gated,
                                      attn_scale(l), B, bf, st);
    }
    PrefillArgs a;
    a.kv = make_view(kv); a.kv_len = kv_len; a.q_prep = q_prep; a.qproj = qproj; a.out = out;
    a.nh = nh; a.T = T; a.gated = l->gated; a.scale = attn_scale(l);
    a.hpb = (G % 8 == 0) ? 8 : (8 % G == 0 ? G : 1);
    a.tpb = 8 / a.hpb;
    dim3 grid((T + a.tpb - 1) / a.tpb, nh / a.hpb, B);
    const size_t smem = ((size_t)PF_KT * (hd + 1) + (size_t)PF_KT * hd + 8 * (size_t)hd) * sizeof(float);
#define PF_LAUNCH(M)                                                                    \
    (bf ? launch_prefill<M, __nv_bfloat16>(a, grid, smem, st) : launch_prefill<M, float>(a, grid, smem, st))
    switch (kv->mode) {
    case ORNITH_KV_F32:       return PF_LAUNCH(ORNITH_KV_F32);
    case ORNITH_KV_INT8_HEAD: return PF_LAUNCH(ORNITH_KV_INT8_HEAD);
    default:                  return PF_LAUNCH(ORNITH_KV_Q8_0);
    }
#undef PF_LAUNCH
}

// K/V rows only: normalise + rotate k, encode k and v into the cache (no attention).
ornith_status ornith_cuda_kv_append(const ornith_cuda_full_layer *l, const ornith_cuda_kv *kv,
                                    const int32_t *kv_len, const int32_t *rope_pos, const void *k,
                                    const void *v, int act_dtype, int T, void *stream) {
    ORN_TRY(orn_require_device());
    ORN_TRY(check_full(l, kv));
    if (kv->n_seq <= 0 || T <= 0) return ORNITH_OK;
    cudaStream_t st = as_stream(stream);
    if (act_dtype == ORNITH_ACT_BF16)
        return launch_prep<__nv_bfloat16>(l, kv, kv_len, rope_pos, nullptr, k, v, nullptr, kv->n_seq * T, T, st, true);
    return launch_prep<float>(l, kv, kv_len, rope_pos, nullptr, k, v, nullptr, kv->n_seq * T, T, st, true);
}

// ---- decode step for hosts that must not allocate device memory -----------------------
//
// Some callers cannot call cudaMalloc on the token path: an engine whose device memory
// was carved up once at start-up and handed to other subsystems, a serving loop where an
// allocation (which synchronises the device and may fail) is not acceptable in the middle
// of a generation, or an embedding host that simply gives this library no allocator.  For
// them the split-K partials and the prepared query rows live in a fixed array that is part
// of the library image: every GPU that loads the library carries these 8 MiB until exit.
//
// In host code `g_static_scratch` is only a handle; the address kernels can use is looked
// up with cudaGetSymbolAddress the first time a device calls in, with that device current.
// That first call per device should therefore happen before any stream capture begins.
// All calls share the one array: it still holds what the previous call left (every word a
// step reads is rewritten by that step first, so nothing has to be cleared), and two calls
// whose kernels overlap on the GPU would race on it — issue them on one stream.
static __device__ __align__(256) unsigned char g_static_scratch[ORNITH_CUDA_STATIC_SCRATCH_BYTES];
static void *g_static_scratch_dev[64];                   // device address, per CUDA device

ornith_status ornith_cuda_full_attn_step_static(const ornith_cuda_full_layer *l, const ornith_cuda_kv *kv,
                                                const int32_t *kv_len, const int32_t *rope_pos,
                                                const void *qproj, const void *k, const void *v, void *out,
                                                int act_dtype, int max_len, void *stream) {
    ORN_TRY(orn_require_device());
    ORN_TRY(check_full(l, kv));
    if (kv->n_seq <= 0) return ORNITH_OK;
    // the step adapts its split length to the scratch it is given: what must fit is the coarse split's need
    const int mlen = max_len < 1 ? 1 : max_len, fine = split_tokens_fine(mlen, head_groups(l, kv->n_seq)), coarse = split_tokens_coarse(mlen);
    const size_t need = step_need(l, kv->n_seq, mlen, fine > coarse ? fine : coarse, decode_path(l, kv));
    if (need > (size_t)ORNITH_CUDA_STATIC_SCRATCH_BYTES) {
        orn_record_error("full_attn_step_static: %d sequences x context %d need %zu bytes of scratch, the built-in "
                         "array holds %u; use ornith_cuda_full_attn_step with caller scratch",
                         kv->n_seq, max_len, need, (unsigned)ORNITH_CUDA_STATIC_SCRATCH_BYTES);
        return ORNITH_ERR_UNSUPPORTED;
    }
    int dev = -1;
    ORN_TRY(orn_check(cudaGetDevice(&dev), "cudaGetDevice"));
    if (dev < 0 || dev >= 64) { orn_record_error("full_attn_step_static: device index %d out of range", dev); return ORNITH_ERR_UNSUPPORTED; }
    if (!g_static_scratch_dev[dev]) {
        void *p = nullptr;
        ORN_TRY(orn_check(cudaGetSymbolAddress(&p, g_static_scratch), "cudaGetSymbolAddress(static scratch)"));
        g_static_scratch_dev[dev] = p;
    }
    return ornith_cuda_full_attn_step(l, kv, kv_len, rope_pos, qproj, k, v, out, act_dtype, max_len,
                                      g_static_scratch_dev[dev], (size_t)ORNITH_CUDA_STATIC_SCRATCH_BYTES, stream);
}

// ---- standalone Q8_0 codec on flat arrays ---------------------------------------
__global__ void __launch_bounds__(128) k_q8_0_encode(const float *src, uint8_t *dst, size_t nblk) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const size_t blk = (size_t)blockIdx.x * 4 + w;
    if (blk >= nblk) return;                             // whole warp leaves together
    float x = src[blk * 32 + lane];
    float amax = warp_max(fabsf(x));
    float d = __fdiv_rn(amax, 127.0f);
    float id = (d != 0.0f) ? __fdiv_rn(1.0f, d) : 0.0f;
    int q = (int)roundf(__fmul_rn(x, id));
    q = max(-127, min(127, q));
    uint8_t *o = dst + blk * 34;
    if (lane == 0) *reinterpret_cast<unsigned short *>(o) = __half_as_ushort(__float2half_rn(d));
    o[2 + lane] = (uint8_t)(int8_t)q;
}

__global__ void k_q8_0_decode(const uint8_t *src, float *dst, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint8_t *blk = src + (i >> 5) * 34;
    dst[i] = __fmul_rn((float)(int8_t)blk[2 + (i & 31)], q8_0_block_scale(blk));
}

ornith_status ornith_cuda_q8_0_encode(const float *src, void *dst, size_t n, void *stream) {
    ORN_TRY(orn_require_device());
    if (n % 32) { orn_record_error("Q8_0 needs a multiple of 32 values"); return ORNITH_ERR_FORMAT; }
    if (!n) return ORNITH_OK;
    const size_t nblk = n / 32;
    k_q8_0_encode<<<(unsigned)((nblk + 3) / 4), 128, 0, as_stream(stream)>>>(src, (uint8_t *)dst, nblk);
    return orn_check_launch("k_q8_0_encode");
}

ornith_status ornith_cuda_q8_0_decode(const void *src, float *dst, size_t n, void *stream) {
    ORN_TRY(orn_require_device());
    if (n % 32) { orn_record_error("Q8_0 needs a multiple of 32 values"); return ORNITH_ERR_FORMAT; }
    if (!n) return ORNITH_OK;
    k_q8_0_decode<<<(unsigned)((n + 255) / 256), 256, 0, as_stream(stream)>>>((const uint8_t *)src, dst, n);
    return orn_check_launch("k_q8_0_decode");
}

}  // extern "C"
