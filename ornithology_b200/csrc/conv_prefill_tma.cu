// conv_prefill_tma.cu — the causal conv + SiLU front of the tensor-core delta-net prefill, fed by tensor copies.
//
// Replaces ornith_conv_prefill + ot_silu_ + the q/k part of ot_l2norm_eps for a whole prompt (reference:
// src/ornith_attn.c:369-397, src/ornith_tensor.c:117-123, :155-160; wiring src/ornith_rforward.c:571-601).
//
// The pass is a stream: read the projected activations once, write the f32 image Y once.  With plain loads a thread
// can keep about a hundred bytes in flight, and with the registers that takes the SM holds too few warps to cover the
// memory latency (the kernel sat at 0.56 of the HBM rate, waiting on its loads).  Here the loads are tensor copies
// into shared memory, three stages per CTA and four CTAs per SM, so an SM keeps about 200 KB in flight whatever the
// register count; the threads only read shared memory, compute and store.
//
// Tile: 32 tokens (+ the 3 tokens of history in front of them) x 512 bytes of channels (256 bf16 or 128 f32).  A warp
// owns 128 adjacent channels (one q or k head when the channel is a q/k channel, so the sums of squares of a head
// are warp sums) and a run of 16 (bf16) or 8 (f32) tokens, which it walks with a sliding window of 4 rows.  The
// first tile of a sequence takes its history from the conv ring instead.  Same arithmetic as k_conv4_silu_prefill's
// tensor-core form: fused multiply-adds in tap order, hardware-exponential SiLU, q/k rounded to tf32.
#include <cuda.h>
#include <cuda_bf16.h>

#include "linear_attn.cuh"
#include "tcgen05.cuh"          // the tensor-map encoder entry point, bounded mbarrier waits

namespace {

constexpr int CT_TOK = 32, CT_ROWS = CT_TOK + 3, CT_ROWB = 512, CT_STAGE = CT_ROWS * CT_ROWB, CT_NST = 3;
constexpr int CT_SMEM = CT_NST * CT_STAGE + 128;

__device__ __forceinline__ uint32_t su32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tile_copy(uint32_t dst, const CUtensorMap *map, int col, int row, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(col), "r"(row) : "memory");
}
__device__ __forceinline__ float tf32_round(float x) { return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u); }

__device__ __forceinline__ float4 ld_row4(const unsigned char *row, int ch_local, const __nv_bfloat16 *) {
    const uint2 u = *reinterpret_cast<const uint2 *>(row + ch_local * 2);
    return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xFFFF0000u), __uint_as_float(u.y << 16),
                       __uint_as_float(u.y & 0xFFFF0000u));
}
__device__ __forceinline__ float4 ld_row4(const unsigned char *row, int ch_local, const float *) {
    return *reinterpret_cast<const float4 *>(row + ch_local * 4);
}

struct ConvTmaArgs {
    float *Y, *rq, *rk;
    int t_begin, t_end, n_seq, n_cblk, n_ttile;
    unsigned int *status;
};

template <typename ACT>
__global__ void __launch_bounds__(128) k_conv4_silu_prefill_tma(LinArgs a, const __grid_constant__ CUtensorMap map_x, ConvTmaArgs c) {
    constexpr int CH = CT_ROWB / (int)sizeof(ACT);        // channels of a tile: 256 (bf16) or 128 (f32)
    constexpr int SPAN = CH / 128, GROUPS = 4 / SPAN, TPT = CT_TOK / GROUPS;   // warps across the channels; token runs; tokens per thread
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[CT_NST];
    __shared__ int failed;
    unsigned char *smem = smem_raw + ((128 - (su32(smem_raw) & 127)) & 127);
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, span = wid % SPAN, grp = wid / SPAN;
    const int qd = a.nk * a.dk, Cc = 2 * qd + a.nv * a.dv;
    const int tiles = c.n_cblk * c.n_ttile * c.n_seq;
    if (tid == 0) {
        failed = 0;
        for (int i = 0; i < CT_NST; i++) tc5::mbar_init(su32(&bars[i]), 1);
        tc5::mbar_init_fence();
    }
    __syncthreads();
    auto issue = [&](int tile, int stage) {               // rows before the tensor's first and past its last read as zeros
        const int cb = tile % c.n_cblk, tt = (tile / c.n_cblk) % c.n_ttile, b = tile / (c.n_cblk * c.n_ttile);
        tc5::mbar_expect_tx(su32(&bars[stage]), (uint32_t)CT_STAGE);
        tile_copy(su32(smem + stage * CT_STAGE), &map_x, cb * CH, b * a.T + c.t_begin + tt * CT_TOK - 3, su32(&bars[stage]));
    };
    if (tid == 0)
        for (int k = 0; k < CT_NST; k++) {
            const long long tile = (long long)blockIdx.x + (long long)k * gridDim.x;
            if (tile < tiles) issue((int)tile, k);
        }
    const int ch_local = span * 128 + lane * 4;
    bool ok = true;
    for (int k = 0;; k++) {
        const long long tile_l = (long long)blockIdx.x + (long long)k * gridDim.x;
        if (tile_l >= tiles) break;
        const int tile = (int)tile_l, stage = k % CT_NST;
        const int cb = tile % c.n_cblk, tt = (tile / c.n_cblk) % c.n_ttile, b = tile / (c.n_cblk * c.n_ttile);
        const int t0 = c.t_begin + tt * CT_TOK, ch = cb * CH + ch_local;
        if (ok && !tc5::mbar_wait(su32(&bars[stage]), (uint32_t)(k / CT_NST) & 1u)) { ok = false; failed = 1; }
        if (ok && ch < Cc) {
            const unsigned char *rows = smem + stage * CT_STAGE + (grp * TPT) * CT_ROWB;    // row i = token t0 + grp TPT - 3 + i
            float4 w[4];                                  // w[q] = taps of channel ch + q
#pragma unroll
            for (int q = 0; q < 4; q++) w[q] = *reinterpret_cast<const float4 *>(a.conv_w + (size_t)(ch + q) * 4);
            float4 bias = make_float4(0.f, 0.f, 0.f, 0.f);
            if (a.conv_b) bias = *reinterpret_cast<const float4 *>(a.conv_b + ch);
            float4 x0, x1, x2;
            const int tfirst = t0 + grp * TPT;            // this thread's first token
            if (tfirst >= 3) {
                x0 = ld_row4(rows, ch_local, (const ACT *)nullptr);
                x1 = ld_row4(rows + CT_ROWB, ch_local, (const ACT *)nullptr);
                x2 = ld_row4(rows + 2 * CT_ROWB, ch_local, (const ACT *)nullptr);
            } else {                                      // the start of the sequence: the history is the conv ring's
                const int pos0 = a.pos[b];
                const float *ring = a.conv + (size_t)b * a.conv_stride;
                float4 h[3];
#pragma unroll
                for (int i = 0; i < 3; i++) {
                    const int t = tfirst - 3 + i;
                    h[i] = t >= 0 ? ld_row4(rows + i * CT_ROWB, ch_local, (const ACT *)nullptr)
                                  : *reinterpret_cast<const float4 *>(ring + (size_t)(((pos0 + t) % 4 + 4) % 4) * Cc + ch);
                }
                x0 = h[0]; x1 = h[1]; x2 = h[2];
            }
            const bool qk = ch < 2 * qd;                  // warp-uniform: a warp covers 128 channels = one head
            float *Yp = c.Y + ((size_t)b * a.T + tfirst) * Cc + ch;
#pragma unroll
            for (int i8 = 0; i8 < TPT; i8 += 8) {
                float ss[8];
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float4 x3 = ld_row4(rows + (i8 + i + 3) * CT_ROWB, ch_local, (const ACT *)nullptr);
                    float4 y;
#define ORN_TAP(F, Q) y.F = silu_fast(fmaf(w[Q].w, x3.F, fmaf(w[Q].z, x2.F, fmaf(w[Q].y, x1.F, fmaf(w[Q].x, x0.F, bias.F)))))
                    ORN_TAP(x, 0); ORN_TAP(y, 1); ORN_TAP(z, 2); ORN_TAP(w, 3);
#undef ORN_TAP
                    if (qk) { y.x = tf32_round(y.x); y.y = tf32_round(y.y); y.z = tf32_round(y.z); y.w = tf32_round(y.w); }
                    if (tfirst + i8 + i < c.t_end) *reinterpret_cast<float4 *>(Yp + (size_t)(i8 + i) * Cc) = y;
                    ss[i] = (y.x * y.x + y.y * y.y) + (y.z * y.z + y.w * y.w);
                    x0 = x1; x1 = x2; x2 = x3;
                }
                if (qk) {
                    // sums over the 32 lanes for 8 tokens: token i ends up in lanes i, i + 8, i + 16, i + 24
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        ss[i] += __shfl_xor_sync(0xffffffffu, ss[i], 16);
                        ss[i] += __shfl_xor_sync(0xffffffffu, ss[i], 8);
                    }
#pragma unroll
                    for (int off = 4; off >= 1; off >>= 1) {
                        const bool up = (lane & off) != 0;
#pragma unroll
                        for (int i = 0; i < off; i++) {
                            const float send = up ? ss[i] : ss[i + off], keep = up ? ss[i + off] : ss[i];
                            ss[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                        }
                    }
                    const int t = tfirst + i8 + lane;
                    if (lane < 8 && t < c.t_end) {
                        const bool is_k = ch >= qd;
                        const int kh = (is_k ? ch - qd : ch) / 128;
                        (is_k ? c.rk : c.rq)[((size_t)b * a.T + t) * a.nk + kh] = 1.0f / sqrtf(ss[0] + 1e-6f);
                    }
                }
            }
        }
        __syncthreads();                                  // every warp is done with this stage
        if (tid == 0 && !failed) {
            const long long next = tile_l + (long long)CT_NST * gridDim.x;
            if (next < tiles) {
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                issue((int)next, stage);
            }
        }
        if (failed) ok = false;
    }
    if (!ok && tid == 0) tc5::report_timeout(c.status, ORN_WAIT_DELTA_SCAN);
}

template <typename ACT>
ornith_status launch_t(const LinArgs &x, int n_seq, float *Y, float *rq, float *rk, int t_begin, int t_end, cudaStream_t s, bool *handled) {
    constexpr int CH = CT_ROWB / (int)sizeof(ACT);
    const int Cc = 2 * x.nk * x.dk + x.nv * x.dv;
    OrnTensorMapEncodeFn enc = orn_tensor_map_encoder();
    const size_t row_bytes = (size_t)Cc * sizeof(ACT);
    if (!enc || ((uintptr_t)x.qkv & 15) != 0 || (row_bytes & 15) != 0 || (size_t)n_seq * x.T >= (1u << 31)) return ORNITH_OK;
    CUtensorMap map;
    cuuint64_t dims[2] = {(cuuint64_t)Cc, (cuuint64_t)n_seq * x.T};
    cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    cuuint32_t box[2] = {(cuuint32_t)CH, (cuuint32_t)CT_ROWS};
    cuuint32_t es[2] = {1, 1};
    const CUtensorMapDataType dt = sizeof(ACT) == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    if (enc(&map, dt, 2, const_cast<void *>(x.qkv), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return ORNITH_OK;                                 // not handled: the caller takes the plain kernel
    static int n_sm_dev[ORN_MAX_DEVICES] = {};
    int &n_sm = n_sm_dev[orn_device_index()];
    if (!n_sm) {
        int dev = 0, n = 0;
        ORN_TRY(orn_check(cudaGetDevice(&dev), "current device"));
        ORN_TRY(orn_check(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev), "SM count"));
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_conv4_silu_prefill_tma<ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, CT_SMEM), "conv smem opt-in"));
        n_sm = n;
    }
    ConvTmaArgs c;
    c.Y = Y; c.rq = rq; c.rk = rk; c.t_begin = t_begin; c.t_end = t_end; c.n_seq = n_seq;
    c.n_cblk = (Cc + CH - 1) / CH; c.n_ttile = (t_end - t_begin + CT_TOK - 1) / CT_TOK; c.status = orn_status_word();
    const long long tiles = (long long)c.n_cblk * c.n_ttile * n_seq;
    if (tiles >= (1ll << 31)) return ORNITH_OK;
    const int grid = (int)(tiles < 4ll * n_sm ? tiles : 4ll * n_sm);
    k_conv4_silu_prefill_tma<ACT><<<grid, 128, CT_SMEM, s>>>(x, map, c);
    *handled = true;
    return orn_check_launch("k_conv4_silu_prefill_tma");
}

}  // namespace

// conv + SiLU of tokens t_begin .. t_end - 1 of every sequence into Y, q/k rounded to tf32, inverse norms into rq / rk.
// *handled = false (and ORNITH_OK) when the shape cannot be addressed by a tensor copy: the caller takes the plain kernel.
ornith_status launch_conv4_silu_prefill_tma(const LinArgs &x, int n_seq, int act_dtype, float *Y, float *rq, float *rk,
                                            int t_begin, int t_end, cudaStream_t s, bool *handled) {
    *handled = false;
    const int Cc = 2 * x.nk * x.dk + x.nv * x.dv;
    if (x.conv_k != 4 || x.dk != 128 || Cc % 4 != 0 || t_end <= t_begin) return ORNITH_OK;
    if (act_dtype == ORNITH_ACT_BF16) return launch_t<__nv_bfloat16>(x, n_seq, Y, rq, rk, t_begin, t_end, s, handled);
    return launch_t<float>(x, n_seq, Y, rq, rk, t_begin, t_end, s, handled);
}
