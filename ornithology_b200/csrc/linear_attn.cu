// linear_attn.cu — gated delta-net (linear attention) layers: causal conv + SiLU,
// q/k L2-norm, decay / write gates, fp32 recurrent state, gated RMSNorm output.
//
// Reference behaviour being replaced:
//   linear_attn() + linear_finish()   src/ornith_rforward.c:457-503, :300-319
//   linear_attn_prefill()             src/ornith_rforward.c:563-618
//   ornith_delta_step / _prefill      src/ornith_attn.c:198-349
//   ornith_conv_step / _prefill       src/ornith_attn.c:370-397
#include <math.h>

#include <stdlib.h>

#include "linear_attn.cuh"

// One channel of the causal conv at token t, history in a ring of conv_k slots
// (token t' lives in slot t' % conv_k).  Sum order and rounding follow the
// engine: bias, taps oldest first, current input last, no fused multiply-add
// (reference: src/ornith_attn.c:373-381).  Returns SiLU(conv).
template <typename ACT>
__device__ __forceinline__ float conv_channel(const LinArgs &a, const float *ring, float *ring_w,
                                              const ACT *x, int Cc, int t, int ch, bool store) {
    const int K = a.conv_k;
    const float xin = act_ld(x, ch);
    float acc = a.conv_b ? a.conv_b[ch] : 0.0f;
    const float *wc = a.conv_w + (size_t)ch * K;
    for (int j = 0; j < K - 1; j++)
        acc = __fadd_rn(acc, __fmul_rn(wc[j], ring[(size_t)((t + 1 + j) % K) * Cc + ch]));
    acc = __fadd_rn(acc, __fmul_rn(wc[K - 1], xin));
    if (store) ring_w[(size_t)(t % K) * Cc + ch] = xin;
    return silu_f(acc);
}

// =============================================================================
// fused decode step, dk = dv = 128, conv_k = 4: one CTA per (value head, sequence)
// =============================================================================
//
// The 64 KiB state of the head is read once into registers (16 x float4 per
// thread) and written back once.  Every load the step needs is issued before the
// first dependent instruction: the state, and — independent of the token index —
// all four ring slots, the input and the taps of each conv channel, the gate
// inputs and the z / norm weights of the epilogue, so the step pays one memory
// latency.  Rows are split 16 per warp; within a warp 8 lanes share a row
// (4 x float4 each), so the two dot products per row reduce over 3 shuffles.
// Three block barriers in all.

template <typename ACT>
__global__ void __launch_bounds__(256, 2) k_linear_decode_128(LinArgs a) {
    __shared__ __align__(16) float q_s[128], k_s[128], v_s[128];
    __shared__ double redd[32];
    __shared__ float gates[2];
    const int hv = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int kh = key_head_of(a, hv), qd = a.nk * 128, vd = a.nv * 128, Cc = 2 * qd + vd;
    float *S = a.S + (size_t)b * a.S_stride + (size_t)hv * 128 * 128;
    const int sr = lane >> 3, cc = lane & 7;

    float4 s[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
            s[i][j] = __ldcs(reinterpret_cast<const float4 *>(S + (size_t)(w * 16 + i * 4 + sr) * 128) + cc + j * 8);

    // ---- all remaining loads, none of which depends on another ------------------------------
    float *ring = a.conv + (size_t)b * a.conv_stride;
    const ACT *x = (const ACT *)a.qkv + (size_t)b * Cc;
    const bool qk_thread = tid < 128;
    const int c0 = qk_thread ? kh * 128 + tid : 2 * qd + hv * 128 + (tid - 128);      // q channel | v channel
    const int c1 = qd + kh * 128 + (tid & 127);                                       // k channel (qk threads)
    float h0[4], h1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int sl = 0; sl < 4; sl++) h0[sl] = ring[(size_t)sl * Cc + c0];
    const float x0 = act_ld(x, c0);
    const float4 w0 = *reinterpret_cast<const float4 *>(a.conv_w + (size_t)c0 * 4);
    const float bias0 = a.conv_b ? a.conv_b[c0] : 0.0f;
    float x1 = 0.0f, bias1 = 0.0f;
    float4 w1 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (qk_thread) {
#pragma unroll
        for (int sl = 0; sl < 4; sl++) h1[sl] = ring[(size_t)sl * Cc + c1];
        x1 = act_ld(x, c1);
        w1 = *reinterpret_cast<const float4 *>(a.conv_w + (size_t)c1 * 4);
        bias1 = a.conv_b ? a.conv_b[c1] : 0.0f;
    }
    const int t = a.pos[b];
    const float ain = act_ld((const ACT *)a.a, (size_t)b * a.nv + hv);
    const float bin = act_ld((const ACT *)a.b, (size_t)b * a.nv + hv);
    const float acoef = a.a_coef[hv], dtb = a.dt_bias[hv];
    // epilogue operands of the rows whose result this lane will hold (lanes with cc == 0)
    const size_t out_base = (size_t)b * vd + (size_t)hv * 128;
    float zin[4], nw[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int r = w * 16 + i * 4 + sr;
        zin[i] = (cc == 0) ? act_ld((const ACT *)a.z, out_base + r) : 0.0f;
        nw[i] = (cc == 0) ? a.norm_w[r] : 0.0f;
    }

    // ---- conv + SiLU, q/k L2-norm (reference: src/ornith_tensor.c:155-160), gates ------------
    const int sb = (t + 1) & 3;
    const bool own = owns_key_head(a, hv);
    const float y0 = conv4_silu(h0, x0, w0, bias0, sb);
    float y1 = 0.0f;
    if (qk_thread) {
        y1 = conv4_silu(h1, x1, w1, bias1, sb);
        if (own) { ring[(size_t)(t & 3) * Cc + c0] = x0; ring[(size_t)(t & 3) * Cc + c1] = x1; }
    } else {
        ring[(size_t)(t & 3) * Cc + c0] = x0;
        v_s[tid - 128] = y0;
    }
    {
        double sq = qk_thread ? (double)y0 * (double)y0 : 0.0, sk = (double)y1 * (double)y1;
        sq = warp_sum(sq); sk = warp_sum(sk);
        if (lane == 0) { redd[w] = sq; redd[8 + w] = sk; }
    }
    __syncthreads();
    if (qk_thread) {
        const double ssq = redd[0] + redd[1] + redd[2] + redd[3], ssk = redd[8] + redd[9] + redd[10] + redd[11];
        q_s[tid] = y0 * (float)(1.0 / sqrt(ssq + (double)1e-6f));
        k_s[tid] = y1 * (float)(1.0 / sqrt(ssk + (double)1e-6f));
    }
    if (tid == 0) {   // decay and write gates (reference: src/ornith_rforward.c:282-284, :493-496)
        gates[0] = expf(acoef * softplus_f(ain + dtb));
        gates[1] = sigmoid_f(bin);
    }
    __syncthreads();

    // ---- S <- alpha S; u = beta (v - S k); S += u k^T; o = S q  (reference: src/ornith_attn.c:203-212)
    const float alpha = gates[0], beta = gates[1];
    float orow[4];
    double ss = 0.0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int r = w * 16 + i * 4 + sr;
        float recall = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float4 kr = lds128(k_s + (cc + j * 8) * 4);
            s[i][j].x *= alpha; s[i][j].y *= alpha; s[i][j].z *= alpha; s[i][j].w *= alpha;
            recall += s[i][j].x * kr.x + s[i][j].y * kr.y + s[i][j].z * kr.z + s[i][j].w * kr.w;
        }
        recall += __shfl_xor_sync(0xffffffffu, recall, 1);
        recall += __shfl_xor_sync(0xffffffffu, recall, 2);
        recall += __shfl_xor_sync(0xffffffffu, recall, 4);
        const float u = beta * (v_s[r] - recall);
        float read = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float4 kr = lds128(k_s + (cc + j * 8) * 4);
            const float4 qr = lds128(q_s + (cc + j * 8) * 4);
            s[i][j].x += u * kr.x; s[i][j].y += u * kr.y; s[i][j].z += u * kr.z; s[i][j].w += u * kr.w;
            read += s[i][j].x * qr.x + s[i][j].y * qr.y + s[i][j].z * qr.z + s[i][j].w * qr.w;
            __stcs(reinterpret_cast<float4 *>(S + (size_t)r * 128) + cc + j * 8, s[i][j]);
        }
        read += __shfl_xor_sync(0xffffffffu, read, 1);
        read += __shfl_xor_sync(0xffffffffu, read, 2);
        read += __shfl_xor_sync(0xffffffffu, read, 4);
        orow[i] = read * a.out_scale;                      // scaled head output of row r (all 8 lanes agree)
        if (cc == 0) ss += (double)orow[i] * (double)orow[i];
    }

    // ---- per-head RMSNorm and SiLU(z) gate (reference: src/ornith_rforward.c:305-314) ---------
    ss = warp_sum(ss);
    if (lane == 0) redd[16 + w] = ss;
    __syncthreads();
    if (cc == 0) {
        double tot = 0.0;
#pragma unroll
        for (int i = 0; i < 8; i++) tot += redd[16 + i];
        const float inv = (float)(1.0 / sqrt(tot / 128.0 + (double)a.eps));
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int r = w * 16 + i * 4 + sr;
            float y = orow[i] * inv * nw[i];
            y *= silu_f(zin[i]);
            act_st((ACT *)a.out, out_base + r, y);
        }
    }
}

// =============================================================================
// the same step for any dk, dv, conv_k (128 threads, one thread per state row)
// =============================================================================

// rows r = tid, tid+blockDim,...: S_r <- alpha S_r; u = beta (v_r - S_r.k);
// S_r += u k; o_r = S_r.q   (reference: src/ornith_attn.c:203-212)
__device__ __forceinline__ void delta_rows(float *S, int dk, int dv, const float *q_s, const float *k_s,
                                           const float *v_s, float alpha, float beta, float *o_s) {
    for (int r = threadIdx.x; r < dv; r += blockDim.x) {
        float *row = S + (size_t)r * dk;
        float recall = 0.0f;
        for (int c = 0; c < dk; c++) {
            const float sv = row[c] * alpha;
            row[c] = sv;
            recall += sv * k_s[c];
        }
        const float u = beta * (v_s[r] - recall);
        float read = 0.0f;
        for (int c = 0; c < dk; c++) {
            const float sv = row[c] + u * k_s[c];
            row[c] = sv;
            read += sv * q_s[c];
        }
        o_s[r] = read;
    }
}

// out_h = RMSNorm(scale * o_h; norm_w) * SiLU(z_h) for the dv values in o_s
template <typename ACT>
__device__ __forceinline__ void gated_norm_store(const LinArgs &a, const float *o_s, const ACT *z, ACT *out,
                                                 double *redd) {
    double ss = 0.0;
    for (int r = threadIdx.x; r < a.dv; r += blockDim.x) {
        const float o = o_s[r] * a.out_scale;
        ss += (double)o * (double)o;
    }
    ss = block_sum(ss, redd);
    const float inv = (float)(1.0 / sqrt(ss / (double)a.dv + (double)a.eps));
    for (int r = threadIdx.x; r < a.dv; r += blockDim.x) {
        float y = (o_s[r] * a.out_scale) * inv * a.norm_w[r];
        y *= silu_f(act_ld(z, r));
        act_st(out, r, y);
    }
}

template <typename ACT>
__global__ void __launch_bounds__(128) k_linear_decode_generic(LinArgs a) {
    extern __shared__ float sm[];
    __shared__ double redd[32];
    __shared__ float gates[2];
    const int dk = a.dk, dv = a.dv;
    float *q_s = sm, *k_s = q_s + dk, *v_s = k_s + dk, *o_s = v_s + dv;
    const int hv = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
    const int kh = key_head_of(a, hv), qd = a.nk * dk, vd = a.nv * dv, Cc = 2 * qd + vd;
    const int t = a.pos[b];
    float *ring = a.conv + (size_t)b * a.conv_stride;
    const ACT *x = (const ACT *)a.qkv + (size_t)b * Cc;
    const bool own = owns_key_head(a, hv);
    double sq = 0.0, sk = 0.0;
    for (int i = tid; i < dk; i += blockDim.x) {
        const float yq = conv_channel(a, ring, ring, x, Cc, t, kh * dk + i, own);
        const float yk = conv_channel(a, ring, ring, x, Cc, t, qd + kh * dk + i, own);
        q_s[i] = yq; k_s[i] = yk;
        sq += (double)yq * (double)yq; sk += (double)yk * (double)yk;
    }
    for (int i = tid; i < dv; i += blockDim.x)
        v_s[i] = conv_channel(a, ring, ring, x, Cc, t, 2 * qd + hv * dv + i, true);
    sq = block_sum(sq, redd);
    sk = block_sum(sk, redd);
    const float rq = (float)(1.0 / sqrt(sq + (double)1e-6f)), rk = (float)(1.0 / sqrt(sk + (double)1e-6f));
    for (int i = tid; i < dk; i += blockDim.x) { q_s[i] *= rq; k_s[i] *= rk; }
    if (tid == 0) {
        const float ain = act_ld((const ACT *)a.a, (size_t)b * a.nv + hv);
        const float bin = act_ld((const ACT *)a.b, (size_t)b * a.nv + hv);
        gates[0] = expf(a.a_coef[hv] * softplus_f(ain + a.dt_bias[hv]));
        gates[1] = sigmoid_f(bin);
    }
    __syncthreads();
    delta_rows(a.S + (size_t)b * a.S_stride + (size_t)hv * dv * dk, dk, dv, q_s, k_s, v_s, gates[0], gates[1], o_s);
    __syncthreads();
    const size_t off = (size_t)b * vd + (size_t)hv * dv;
    gated_norm_store(a, o_s, (const ACT *)a.z + off, (ACT *)a.out + off, redd);
}

// =============================================================================
// per-head primitives on raw pointers (tier 1 is built from these)
// =============================================================================

__global__ void __launch_bounds__(128) k_delta_step_raw(float *S, int dk, int dv, const float *q, const float *k,
                                                        const float *v, const float *alpha, const float *beta,
                                                        float *o) {
    extern __shared__ float sm[];
    float *q_s = sm, *k_s = q_s + dk, *v_s = k_s + dk, *o_s = v_s + dv;
    const int h = blockIdx.x;
    for (int i = threadIdx.x; i < dk; i += blockDim.x) { q_s[i] = q[(size_t)h * dk + i]; k_s[i] = k[(size_t)h * dk + i]; }
    for (int i = threadIdx.x; i < dv; i += blockDim.x) v_s[i] = v[(size_t)h * dv + i];
    __syncthreads();
    delta_rows(S + (size_t)h * dv * dk, dk, dv, q_s, k_s, v_s, alpha[h], beta[h], o_s);
    __syncthreads();
    for (int i = threadIdx.x; i < dv; i += blockDim.x) o[(size_t)h * dv + i] = o_s[i];
}

// T sequential steps of one head inside one CTA; each thread keeps its own rows,
// so only the per-token vectors need a barrier.
__global__ void __launch_bounds__(128) k_delta_prefill_seq_raw(float *S, int dk, int dv, const float *Q,
                                                               const float *K, const float *V,
                                                               const float *alpha, const float *beta, int T,
                                                               float *O) {
    extern __shared__ float sm[];
    float *q_s = sm, *k_s = q_s + dk, *v_s = k_s + dk, *o_s = v_s + dv;
    for (int t = 0; t < T; t++) {
        __syncthreads();
        for (int i = threadIdx.x; i < dk; i += blockDim.x) { q_s[i] = Q[(size_t)t * dk + i]; k_s[i] = K[(size_t)t * dk + i]; }
        for (int i = threadIdx.x; i < dv; i += blockDim.x) v_s[i] = V[(size_t)t * dv + i];
        __syncthreads();
        delta_rows(S, dk, dv, q_s, k_s, v_s, alpha[t], beta[t], o_s);
        for (int r = threadIdx.x; r < dv; r += blockDim.x) O[(size_t)t * dv + r] = o_s[r];
    }
}

// conv over the engine's history image [(K-1)][C] (oldest first): one thread per
// channel walks T tokens with the window in registers, then stores the new image.
__global__ void k_conv_image(float *image, int K, int C, const float *X, const float *w, const float *bias,
                             int T, float *OUT) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float win[8];                                         // K <= 9
    for (int j = 0; j < K - 1; j++) win[j] = image[(size_t)j * C + c];
    const float *wc = w + (size_t)c * K;
    for (int t = 0; t < T; t++) {
        const float xin = X[(size_t)t * C + c];
        float acc = bias ? bias[c] : 0.0f;
        for (int j = 0; j < K - 1; j++) acc = __fadd_rn(acc, __fmul_rn(wc[j], win[j]));
        acc = __fadd_rn(acc, __fmul_rn(wc[K - 1], xin));
        OUT[(size_t)t * C + c] = acc;
        for (int j = 0; j + 1 < K - 1; j++) win[j] = win[j + 1];
        if (K >= 2) win[K - 2] = xin;
    }
    for (int j = 0; j < K - 1; j++) image[(size_t)j * C + c] = win[j];
}

// ring <-> image.  Image row j holds token pos-(K-1)+j, which lives in ring slot
// (pos + 1 + j) % K.
__global__ void k_conv_ring_image(float *ring, float *image, int K, int C, int pos, int to_image) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    for (int j = 0; j < K - 1; j++) {
        float *r = ring + (size_t)((pos + 1 + j) % K) * C + c, *im = image + (size_t)j * C + c;
        if (to_image) *im = *r; else *r = *im;
    }
}

// =============================================================================
// prefill front end: conv + SiLU over T tokens, ring refresh, norms and gates
// =============================================================================

constexpr int CONV_TOK = 32;             // tokens walked by one thread

// Y[tok][ch] = SiLU(conv) as f32.  grid (Cc/128, T/CONV_TOK, n_seq).  The ring is
// only read here; k_conv_ring_refresh stores the new history afterwards.
template <typename ACT>
__global__ void __launch_bounds__(128) k_conv_silu_prefill(LinArgs a, float *Y) {
    const int qd = a.nk * a.dk, Cc = 2 * qd + a.nv * a.dv, K = a.conv_k;
    const int ch = blockIdx.x * 128 + threadIdx.x, b = blockIdx.z, t0 = blockIdx.y * CONV_TOK;
    if (ch >= Cc) return;
    const int pos0 = a.pos[b];
    const float *ring = a.conv + (size_t)b * a.conv_stride;
    const ACT *X = (const ACT *)a.qkv + (size_t)b * a.T * Cc;
    float win[8];
    for (int j = 0; j < K - 1; j++) {                     // token t0-(K-1)+j
        const int tj = t0 - (K - 1) + j;
        win[j] = tj >= 0 ? act_ld(X, (size_t)tj * Cc + ch)
                         : ring[(size_t)(((pos0 + tj) % K + K) % K) * Cc + ch];
    }
    const float *wc = a.conv_w + (size_t)ch * K;
    const float bias = a.conv_b ? a.conv_b[ch] : 0.0f;
    const int t1 = min(a.T, t0 + CONV_TOK);
    for (int t = t0; t < t1; t++) {
        const float xin = act_ld(X, (size_t)t * Cc + ch);
        float acc = bias;
        for (int j = 0; j < K - 1; j++) acc = __fadd_rn(acc, __fmul_rn(wc[j], win[j]));
        acc = __fadd_rn(acc, __fmul_rn(wc[K - 1], xin));
        Y[((size_t)b * a.T + t) * Cc + ch] = silu_f(acc);
        for (int j = 0; j + 1 < K - 1; j++) win[j] = win[j + 1];
        if (K >= 2) win[K - 2] = xin;
    }
}


// conv_k = 4, Cc a multiple of 4: one thread owns 4 adjacent channels over CONV4_TOK
// tokens and requests all its inputs before the first use.  Same products, sums and
// rounding as k_conv_silu_prefill.  grid (ceil(Cc/512), ceil(T/CONV4_TOK), n_seq).
#ifndef ORN_CONV4_TOK
#define ORN_CONV4_TOK 8
#endif
constexpr int CONV4_TOK = ORN_CONV4_TOK;      // 8 tokens (+ 3 of history) per thread: ~80 registers, 24 warps per SM; 16 tokens took 128
                                              // registers (16 warps per SM) and the kernel waited on its loads (200 us per 8192 tokens x 12288 channels)

// nearest tf32 value (ties away from zero, finite inputs), in integer arithmetic
__device__ __forceinline__ float tf32_rna(float x) { return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u); }
// NORMS (needs dk = 128, so that the 32 threads of a warp own exactly one q or k head): the kernel also leaves the
// inverse L2 norms 1/sqrt(sum x^2 + 1e-6) of the q and k rows it produces in rq / rk [token][key head], which saves
// the pass of k_linear_prep over the image (reference: ot_l2norm_eps, src/ornith_tensor.c:155-160).
template <typename ACT, bool FAST, bool NORMS>
__global__ void __launch_bounds__(128) k_conv4_silu_prefill(LinArgs a, float *Y, float *rq, float *rk, int t_begin, int t_end) {
    // tokens t_begin .. t_end - 1 of every sequence (the whole prompt, or one slab of it)
    const int qd = a.nk * a.dk, Cc = 2 * qd + a.nv * a.dv;
    const int ch = (blockIdx.x * 128 + threadIdx.x) * 4, b = blockIdx.z, t0 = t_begin + blockIdx.y * CONV4_TOK;
    if (ch >= Cc) return;
    const int pos0 = a.pos[b];
    const float *ring = a.conv + (size_t)b * a.conv_stride;
    const ACT *X = (const ACT *)a.qkv + (size_t)b * a.T * Cc;
    float4 x[CONV4_TOK + 3];
#pragma unroll
    for (int i = 0; i < CONV4_TOK + 3; i++) {             // token t0 - 3 + i
        const int t = t0 - 3 + i;
        if (t >= a.T) x[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        else if (t >= 0) x[i] = act_ld4(X, (size_t)t * Cc + ch);
        else x[i] = *reinterpret_cast<const float4 *>(ring + (size_t)(((pos0 + t) % 4 + 4) % 4) * Cc + ch);
    }
    float4 w[4];                                          // w[c] = taps of channel ch + c
#pragma unroll
    for (int c = 0; c < 4; c++) w[c] = *reinterpret_cast<const float4 *>(a.conv_w + (size_t)(ch + c) * 4);
    float4 bias = make_float4(0.f, 0.f, 0.f, 0.f);
    if (a.conv_b) bias = *reinterpret_cast<const float4 *>(a.conv_b + ch);
    float ss[CONV4_TOK];                                  // this thread's share of each token's sum of squares
#pragma unroll
    for (int i = 0; i < CONV4_TOK; i++) ss[i] = 0.0f;
#pragma unroll
    for (int i = 0; i < CONV4_TOK; i++) {
        if (t0 + i >= t_end) break;
        float4 y;
        // the tensor-core paths (FAST) round q, k to tf32 and take a hardware-exponential SiLU anyway: fused multiply-adds
#define ORN_CONV4(F, WC, B)                                                                               \
        y.F = FAST ? silu_fast(fmaf(WC.w, x[i + 3].F, fmaf(WC.z, x[i + 2].F, fmaf(WC.y, x[i + 1].F, fmaf(WC.x, x[i].F, B)))))  \
                   : silu_f(__fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(B, __fmul_rn(WC.x, x[i].F)),                  \
                                                             __fmul_rn(WC.y, x[i + 1].F)),                \
                                                   __fmul_rn(WC.z, x[i + 2].F)),                          \
                                         __fmul_rn(WC.w, x[i + 3].F)))
        ORN_CONV4(x, w[0], bias.x); ORN_CONV4(y, w[1], bias.y); ORN_CONV4(z, w[2], bias.z); ORN_CONV4(w, w[3], bias.w);
#undef ORN_CONV4
        if (FAST && ch < 2 * qd) {                        // q and k feed tf32 tensor-core products: round once, here
            y.x = tf32_rna(y.x); y.y = tf32_rna(y.y); y.z = tf32_rna(y.z); y.w = tf32_rna(y.w);
        }
        *reinterpret_cast<float4 *>(Y + ((size_t)b * a.T + t0 + i) * Cc + ch) = y;
        if (NORMS) ss[i] = (y.x * y.x + y.y * y.y) + (y.z * y.z + y.w * y.w);
    }
    if (NORMS && ch < 2 * qd) {                           // warp-uniform: a warp covers 128 channels = one head
        const int lane = threadIdx.x & 31;
        // sums over the 32 lanes for CONV4_TOK tokens: token t ends up in the lanes that are t modulo CONV4_TOK
#pragma unroll
        for (int i = 0; i < CONV4_TOK; i++)
#pragma unroll
            for (int off = 16; off >= CONV4_TOK; off >>= 1) ss[i] += __shfl_xor_sync(0xffffffffu, ss[i], off);
#pragma unroll
        for (int off = CONV4_TOK / 2; off >= 1; off >>= 1) {
            const bool up = (lane & off) != 0;
#pragma unroll
            for (int k = 0; k < off; k++) {
                const float send = up ? ss[k] : ss[k + off], keep = up ? ss[k + off] : ss[k];
                ss[k] = keep + __shfl_xor_sync(0xffffffffu, send, off);
            }
        }
        if (lane < CONV4_TOK && t0 + lane < t_end) {
            const bool is_k = ch >= qd;
            const int kh = (is_k ? ch - qd : ch) / 128;
            (is_k ? rk : rq)[((size_t)b * a.T + t0 + lane) * a.nk + kh] = 1.0f / sqrtf(ss[0] + 1e-6f);
        }
    }
}

// store the last min(T, conv_k) inputs of each sequence into their ring slots
template <typename ACT>
__global__ void k_conv_ring_refresh(LinArgs a) {
    const int qd = a.nk * a.dk, Cc = 2 * qd + a.nv * a.dv, K = a.conv_k;
    const int ch = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
    if (ch >= Cc) return;
    const int pos0 = a.pos[b];
    float *ring = a.conv + (size_t)b * a.conv_stride;
    const ACT *X = (const ACT *)a.qkv + (size_t)b * a.T * Cc;
    for (int t = max(0, a.T - K); t < a.T; t++)
        ring[(size_t)((pos0 + t) % K) * Cc + ch] = act_ld(X, (size_t)t * Cc + ch);
}

// per (token, key head): 1/sqrt(sum q^2 + eps), 1/sqrt(sum k^2 + eps);
// per (token, value head): log-decay a_coef*softplus(a+dt) and beta = sigmoid(b).
// One warp per (token, key head); grid (n_tok).
template <typename ACT>
__global__ void __launch_bounds__(128) k_linear_prep(LinArgs a, const float *Y, int n_tok, float *rq, float *rk,
                                                     float *la, float *be) {
    const int tok = blockIdx.x, lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int qd = a.nk * a.dk, Cc = 2 * qd + a.nv * a.dv;
    const float *y = Y + (size_t)tok * Cc;
    for (int kh = w; kh < a.nk; kh += nw) {
        double sq = 0.0, sk = 0.0;
        for (int i = lane; i < a.dk; i += 32) {
            const float vq = y[kh * a.dk + i], vk = y[qd + kh * a.dk + i];
            sq += (double)vq * (double)vq; sk += (double)vk * (double)vk;
        }
        sq = warp_sum(sq); sk = warp_sum(sk);
        if (lane == 0) {
            rq[(size_t)tok * a.nk + kh] = (float)(1.0 / sqrt(sq + (double)1e-6f));
            rk[(size_t)tok * a.nk + kh] = (float)(1.0 / sqrt(sk + (double)1e-6f));
        }
    }
    for (int hv = threadIdx.x; hv < a.nv; hv += blockDim.x) {
        const float ain = act_ld((const ACT *)a.a, (size_t)tok * a.nv + hv);
        const float bin = act_ld((const ACT *)a.b, (size_t)tok * a.nv + hv);
        la[(size_t)tok * a.nv + hv] = a.a_coef[hv] * softplus_f(ain + a.dt_bias[hv]);
        be[(size_t)tok * a.nv + hv] = sigmoid_f(bin);
    }
}

// =============================================================================
// prefill scan, any dk/dv: T sequential steps per (value head, sequence)
// =============================================================================
template <typename ACT>
__global__ void __launch_bounds__(128) k_linear_prefill_seq(LinArgs a, const float *Y, const float *rq,
                                                            const float *rk, const float *la, const float *be) {
    extern __shared__ float sm[];
    __shared__ double redd[32];
    const int dk = a.dk, dv = a.dv;
    float *q_s = sm, *k_s = q_s + dk, *v_s = k_s + dk, *o_s = v_s + dv;
    const int hv = blockIdx.x, b = blockIdx.y, kh = key_head_of(a, hv);
    const int qd = a.nk * dk, vd = a.nv * dv, Cc = 2 * qd + vd;
    float *S = a.S + (size_t)b * a.S_stride + (size_t)hv * dv * dk;
    for (int t = 0; t < a.T; t++) {
        const size_t tok = (size_t)b * a.T + t;
        const float *y = Y + tok * Cc;
        __syncthreads();
        const float sq = rq[tok * a.nk + kh], sk = rk[tok * a.nk + kh];
        for (int i = threadIdx.x; i < dk; i += blockDim.x) {
            q_s[i] = y[kh * dk + i] * sq;
            k_s[i] = y[qd + kh * dk + i] * sk;
        }
        for (int i = threadIdx.x; i < dv; i += blockDim.x) v_s[i] = y[2 * qd + hv * dv + i];
        __syncthreads();
        delta_rows(S, dk, dv, q_s, k_s, v_s, expf(la[tok * a.nv + hv]), be[tok * a.nv + hv], o_s);
        __syncthreads();
        const size_t off = tok * vd + (size_t)hv * dv;
        gated_norm_store(a, o_s, (const ACT *)a.z + off, (ACT *)a.out + off, redd);
    }
}

// =============================================================================
// prefill scan, dk = dv = 128: chunked (WY / UT-transform) form in fp32
// =============================================================================
//
// Per chunk of C tokens with incoming state S (reference derivation:
// src/ornith_attn.c:215-243), G_i = running sum of log-decay inside the chunk:
//   Gamma_ij = exp(G_i - G_j) (j <= i),  p_i = exp(G_i)
//   T = diag(beta) (V - diag(p) K S^T)
//   (I + diag(beta) strictLower(Gamma o K K^T)) U = T
//   O = diag(p) Q S^T + lower(Gamma o Q K^T) U
//   S <- p_{C-1} S + sum_j Gamma_{C-1,j} u_j k_j^T
// Decay ratios are exponentials of differences of the in-chunk log-decay sum,
// never quotients of cumulative products.  The state lives transposed in shared
// memory for the whole scan and is written back once.
template <int C>
struct ChunkSmem {
    float St[128 * 128];                 // St[c][r] = S[r][c]
    float Ks[C * 129];                   // normalised k rows, odd stride
    float Qs[C * 129];
    float Us[C * 128];                   // V -> T -> U, [token][r]
    float Ms[C * (C + 1)];               // beta_i Gamma_ij (k_i.k_j), j < i
    float Ps[C * (C + 1)];               // Gamma_ij (q_i.k_j), j <= i
    float G[C], beta[C], w_end[C];
};

template <int C, typename ACT>
__global__ void __launch_bounds__(256, 1) k_linear_prefill_chunk128(LinArgs a, const float *Y, const float *rq,
                                                                    const float *rk, const float *la,
                                                                    const float *be) {
    extern __shared__ __align__(16) unsigned char smraw[];
    ChunkSmem<C> &sm = *reinterpret_cast<ChunkSmem<C> *>(smraw);
    const int hv = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, tx = tid & 31, ty = tid >> 5;
    const int kh = key_head_of(a, hv), qd = a.nk * 128, vd = a.nv * 128, Cc = 2 * qd + vd;
    float *S = a.S + (size_t)b * a.S_stride + (size_t)hv * 128 * 128;
    constexpr int RI = C / 8;            // token rows per thread in the [C][128] tiles

    for (int e = tid; e < 128 * 128; e += 256) {          // S[r][c] -> St[c][r]
        const int r = e >> 7, c = e & 127;
        sm.St[c * 128 + r] = S[e];
    }

    for (int t0 = 0; t0 < a.T; t0 += C) {
        const int n = min(C, a.T - t0);
        const size_t tok0 = (size_t)b * a.T + t0;
        __syncthreads();
        // ---- load the chunk; rows past the end behave as alpha = 1, beta = 0, k = q = v = 0
        for (int e = tid; e < C * 128; e += 256) {
            const int i = e >> 7, c = e & 127;
            float kv = 0.0f, qv = 0.0f, vv = 0.0f;
            if (i < n) {
                const float *y = Y + (tok0 + i) * Cc;
                qv = y[kh * 128 + c] * rq[(tok0 + i) * a.nk + kh];
                kv = y[qd + kh * 128 + c] * rk[(tok0 + i) * a.nk + kh];
                vv = y[2 * qd + hv * 128 + c];
            }
            sm.Ks[i * 129 + c] = kv; sm.Qs[i * 129 + c] = qv; sm.Us[i * 128 + c] = vv;
        }
        if (tid < 32) {                                   // inclusive scan of the log-decay
            float g = 0.0f, bb = 0.0f;
            if (C == 32 || tid < C) {
                if (tid < n) { g = la[(tok0 + tid) * a.nv + hv]; bb = be[(tok0 + tid) * a.nv + hv]; }
            }
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float up = __shfl_up_sync(0xffffffffu, g, o);
                if (tx >= o) g += up;
            }
            if (tid < C) { sm.G[tid] = g; sm.beta[tid] = bb; }
        }
        __syncthreads();
        if (tid < C) sm.w_end[tid] = expf(sm.G[C - 1] - sm.G[tid]);

        // ---- S_in K^T and S_in Q^T: thread owns tokens ty*RI.., columns r = tx + 32m
        float sk[RI][4], sq[RI][4];
#pragma unroll
        for (int i = 0; i < RI; i++)
#pragma unroll
            for (int m = 0; m < 4; m++) { sk[i][m] = 0.0f; sq[i][m] = 0.0f; }
        for (int c = 0; c < 128; c++) {
            float sv[4];
#pragma unroll
            for (int m = 0; m < 4; m++) sv[m] = sm.St[c * 128 + tx + 32 * m];
#pragma unroll
            for (int i = 0; i < RI; i++) {
                const float kv = sm.Ks[(ty * RI + i) * 129 + c], qv = sm.Qs[(ty * RI + i) * 129 + c];
#pragma unroll
                for (int m = 0; m < 4; m++) { sk[i][m] += kv * sv[m]; sq[i][m] += qv * sv[m]; }
            }
        }
        // ---- Gram matrices: thread -> (i = e / C, j = e % C)
        for (int e = tid; e < C * C; e += 256) {
            const int i = e / C, j = e % C;
            float mk = 0.0f, pq = 0.0f;
            if (j <= i) {
                const float *ki = sm.Ks + i * 129, *kj = sm.Ks + j * 129, *qi = sm.Qs + i * 129;
                for (int c = 0; c < 128; c++) { mk += ki[c] * kj[c]; pq += qi[c] * kj[c]; }
                const float gam = expf(sm.G[i] - sm.G[j]);
                mk = (j < i) ? sm.beta[i] * gam * mk : 0.0f;
                pq = gam * pq;
            }
            sm.Ms[i * (C + 1) + j] = mk;
            sm.Ps[i * (C + 1) + j] = pq;
        }
        __syncthreads();                                  // everyone has read V from Us
        // ---- T = beta (V - p S K^T) in place of V
#pragma unroll
        for (int i = 0; i < RI; i++) {
            const int ti = ty * RI + i;
            const float bi = sm.beta[ti], pi = expf(sm.G[ti]);
#pragma unroll
            for (int m = 0; m < 4; m++) {
                const int r = tx + 32 * m;
                sm.Us[ti * 128 + r] = bi * sm.Us[ti * 128 + r] - bi * pi * sk[i][m];
            }
        }
        __syncthreads();
        // ---- forward substitution, one thread per column r
        if (tid < 128) {
            float u[C];
#pragma unroll
            for (int i = 0; i < C; i++) {
                float acc = sm.Us[i * 128 + tid];
#pragma unroll
                for (int j = 0; j < i; j++) acc -= sm.Ms[i * (C + 1) + j] * u[j];
                u[i] = acc;
            }
#pragma unroll
            for (int i = 0; i < C; i++) sm.Us[i * 128 + tid] = u[i];
        }
        __syncthreads();
        // ---- O = p S Q^T + P U, then scale / RMSNorm / SiLU(z) gate per token
#pragma unroll
        for (int i = 0; i < RI; i++) {
            const int ti = ty * RI + i;
            const float pi = expf(sm.G[ti]);
            float o[4];
#pragma unroll
            for (int m = 0; m < 4; m++) o[m] = pi * sq[i][m];
            for (int j = 0; j <= ti; j++) {
                const float pj = sm.Ps[ti * (C + 1) + j];
#pragma unroll
                for (int m = 0; m < 4; m++) o[m] += pj * sm.Us[j * 128 + tx + 32 * m];
            }
            double ss = 0.0;
#pragma unroll
            for (int m = 0; m < 4; m++) { o[m] *= a.out_scale; ss += (double)o[m] * (double)o[m]; }
            ss = warp_sum(ss);                            // the warp holds the whole head row
            if (ti < n) {
                const float inv = (float)(1.0 / sqrt(ss / 128.0 + (double)a.eps));
                const size_t off = (tok0 + ti) * vd + (size_t)hv * 128;
#pragma unroll
                for (int m = 0; m < 4; m++) {
                    const int r = tx + 32 * m;
                    float y = o[m] * inv * a.norm_w[r];
                    y *= silu_f(act_ld((const ACT *)a.z, off + r));
                    act_st((ACT *)a.out, off + r, y);
                }
            }
        }
        // ---- St[c][r] = p_end St[c][r] + sum_j (w_end_j U[j][r]) K[j][c]
        {
            const float pend = expf(sm.G[C - 1]);
            float acc[16][4];
#pragma unroll
            for (int cc = 0; cc < 16; cc++)
#pragma unroll
                for (int m = 0; m < 4; m++) acc[cc][m] = pend * sm.St[(ty * 16 + cc) * 128 + tx + 32 * m];
            for (int j = 0; j < C; j++) {
                const float wj = sm.w_end[j];
                float uw[4];
#pragma unroll
                for (int m = 0; m < 4; m++) uw[m] = wj * sm.Us[j * 128 + tx + 32 * m];
#pragma unroll
                for (int cc = 0; cc < 16; cc++) {
                    const float kv = sm.Ks[j * 129 + ty * 16 + cc];
#pragma unroll
                    for (int m = 0; m < 4; m++) acc[cc][m] += uw[m] * kv;
                }
            }
#pragma unroll
            for (int cc = 0; cc < 16; cc++)
#pragma unroll
                for (int m = 0; m < 4; m++) sm.St[(ty * 16 + cc) * 128 + tx + 32 * m] = acc[cc][m];
        }
    }
    __syncthreads();
    for (int e = tid; e < 128 * 128; e += 256) {
        const int r = e >> 7, c = e & 127;
        S[e] = sm.St[c * 128 + r];
    }
}

// =============================================================================
// host entry points
// =============================================================================

// Kernel bring-up aid, not part of the public interface: when set, the tcgen05 scan copies the first
// chunk's intermediate tiles (KS, U, QS, PU; [128][64] floats each per (sequence, head)) there.
static float *g_delta_scan_dump = nullptr;
extern "C" void ornith_cuda_debug_delta_scan_dump(float *dev) { g_delta_scan_dump = dev; }
long long *g_delta_scan_trace = nullptr;
extern "C" void ornith_cuda_debug_delta_scan_trace(long long *dev) { g_delta_scan_trace = dev; }

static ornith_status check_linear(const ornith_cuda_linear_layer *l, const ornith_cuda_linear_state *st) {
    if (!l || !st || l->nk <= 0 || l->nv <= 0 || l->dk <= 0 || l->dv <= 0 || l->nv % l->nk ||
        l->conv_k < 1 || l->conv_k > 9 || !l->conv_w || !l->a_coef || !l->dt_bias || !l->norm_w ||
        !st->S || !st->conv) {
        orn_record_error("linear attention: inconsistent layer / state description");
        return ORNITH_ERR_FORMAT;
    }
    if (l->dk > 1024 || l->dv > 1024) { orn_record_error("linear attention: head dim > 1024 unsupported"); return ORNITH_ERR_UNSUPPORTED; }
    return ORNITH_OK;
}

static LinArgs make_args(const ornith_cuda_linear_layer *l, const ornith_cuda_linear_state *st,
                         const int32_t *pos, const void *qkv, const void *a, const void *b, const void *z,
                         void *out, int T) {
    LinArgs x;
    x.nk = l->nk; x.nv = l->nv; x.dk = l->dk; x.dv = l->dv; x.conv_k = l->conv_k; x.head_map = l->head_map;
    x.out_scale = l->out_scale; x.eps = l->eps;
    x.conv_w = l->conv_w; x.conv_b = l->conv_b; x.a_coef = l->a_coef; x.dt_bias = l->dt_bias; x.norm_w = l->norm_w;
    x.S = st->S; x.conv = st->conv; x.S_stride = st->S_seq_stride; x.conv_stride = st->conv_seq_stride;
    x.pos = pos; x.qkv = qkv; x.a = a; x.b = b; x.z = z; x.out = out; x.T = T;
    return x;
}

extern "C" {

ornith_status ornith_cuda_linear_attn_step(const ornith_cuda_linear_layer *l, const ornith_cuda_linear_state *st,
                                           const int32_t *pos, const void *qkv, const void *a, const void *b,
                                           const void *z, void *out, int act_dtype, int n_seq, void *stream) {
    ORN_TRY(orn_require_device());
    ORN_TRY(check_linear(l, st));
    if (n_seq <= 0) return ORNITH_OK;
    LinArgs x = make_args(l, st, pos, qkv, a, b, z, out, 1);
    dim3 grid(l->nv, n_seq);
    cudaStream_t s = as_stream(stream);
    const bool bf = act_dtype == ORNITH_ACT_BF16;
    if (l->dk == 128 && l->dv == 128 && l->conv_k == 4 && (st->S_seq_stride % 4) == 0 &&
        ((uintptr_t)st->S % 16) == 0 && ((uintptr_t)l->conv_w % 16) == 0) {
        // Once there are more (sequence, head) units than the 2 x 148 CTAs the SMs hold, the persistent
        // kernel that streams the state through a bulk-copy ring is faster (59 vs 66 us at 2048 units).
        // ORNITH_CUDA_LINEAR_DECODE=ring | cta forces one of the two.
        const char *variant = getenv("ORNITH_CUDA_LINEAR_DECODE");
        const bool ring = variant ? variant[0] == 'r' : (long long)n_seq * l->nv > 296;
        if (ring) return launch_linear_decode_ring(x, n_seq, act_dtype, s);
        if (bf) k_linear_decode_128<__nv_bfloat16><<<grid, 256, 0, s>>>(x);
        else    k_linear_decode_128<float><<<grid, 256, 0, s>>>(x);
        return orn_check_launch("k_linear_decode_128");
    }
    const size_t smem = (size_t)(2 * l->dk + 2 * l->dv) * sizeof(float);
    if (bf) k_linear_decode_generic<__nv_bfloat16><<<grid, 128, smem, s>>>(x);
    else    k_linear_decode_generic<float><<<grid, 128, smem, s>>>(x);
    return orn_check_launch("k_linear_decode_generic");
}

size_t ornith_cuda_linear_attn_prefill_scratch(const ornith_cuda_linear_layer *l, int n_seq, int T) {
    if (!l || n_seq <= 0 || T <= 0) return 0;
    const size_t n_tok = (size_t)n_seq * T, Cc = 2 * (size_t)l->nk * l->dk + (size_t)l->nv * l->dv;
    size_t bytes = align_up(n_tok * Cc * 4, 256) + 2 * align_up(n_tok * l->nk * 4, 256) + 2 * align_up(n_tok * l->nv * 4, 256);
    if (l->dk == 128 && l->dv == 128) {                   // work area of whichever tensor-core scan is selected at run time
        const size_t w_mma = linear_prefill_tc_blocks_bytes(l->nk, l->nv, n_seq, T), w_tc5 = linear_prefill_tc5_work_bytes(l->nk, l->nv, n_seq, T);
        bytes += align_up(w_mma > w_tc5 ? w_mma : w_tc5, 256);
    }
    return bytes;
}

}  // extern "C"

template <int C, typename ACT>
static ornith_status launch_chunk(const LinArgs &x, dim3 grid, const float *Y, const float *rq, const float *rk,
                                  const float *la, const float *be, cudaStream_t s) {
    static bool configured_dev[ORN_MAX_DEVICES] = {};
    bool &configured = configured_dev[orn_device_index()];
    if (!configured) {
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_linear_prefill_chunk128<C, ACT>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)sizeof(ChunkSmem<C>)),
                          "chunk prefill smem opt-in"));
        configured = true;
    }
    k_linear_prefill_chunk128<C, ACT><<<grid, 256, sizeof(ChunkSmem<C>), s>>>(x, Y, rq, rk, la, be);
    return orn_check_launch("k_linear_prefill_chunk128");
}

extern "C" {

ornith_status ornith_cuda_linear_attn_prefill(const ornith_cuda_linear_layer *l, const ornith_cuda_linear_state *st,
                                              const int32_t *pos, const void *qkv, const void *a, const void *b,
                                              const void *z, void *out, int act_dtype, int n_seq, int T, int chunk,
                                              void *scratch, size_t scratch_bytes, void *stream) {
    ORN_TRY(orn_require_device());
    ORN_TRY(check_linear(l, st));
    if (n_seq <= 0 || T <= 0) return ORNITH_OK;
    if (!scratch || scratch_bytes < ornith_cuda_linear_attn_prefill_scratch(l, n_seq, T)) {
        orn_record_error("linear_attn_prefill: scratch too small (%zu bytes given)", scratch_bytes);
        return ORNITH_ERR_FORMAT;
    }
    cudaStream_t s = as_stream(stream);
    const bool bf = act_dtype == ORNITH_ACT_BF16;
    const size_t n_tok = (size_t)n_seq * T, Cc = 2 * (size_t)l->nk * l->dk + (size_t)l->nv * l->dv;
    char *p = (char *)scratch;
    float *Y = (float *)p;  p += align_up(n_tok * Cc * 4, 256);
    float *rq = (float *)p; p += align_up(n_tok * l->nk * 4, 256);
    float *rk = (float *)p; p += align_up(n_tok * l->nk * 4, 256);
    float *la = (float *)p; p += align_up(n_tok * l->nv * 4, 256);
    float *be = (float *)p; p += align_up(n_tok * l->nv * 4, 256);
    float *blocks = (float *)p;          // only the tensor-core scan uses this part
    if (((uintptr_t)scratch % 256) != 0) { orn_record_error("linear_attn_prefill: scratch must be 256-byte aligned"); return ORNITH_ERR_FORMAT; }
    LinArgs x = make_args(l, st, pos, qkv, a, b, z, out, T);

    // dk = dv = 128 scans on the tensor cores in tf32 unless ORNITH_CUDA_PREFILL_FP32=1 asks for fp32 products;
    // tcgen05 scan unless ORNITH_CUDA_DELTA_SCAN=mma asks for the mma.sync one (or the state is not 16-byte aligned)
    const char *exact = getenv("ORNITH_CUDA_PREFILL_FP32");
    const bool tc = l->dk == 128 && l->dv == 128 && !(exact && exact[0] == '1');
    const char *variant = getenv("ORNITH_CUDA_DELTA_SCAN");
    const bool tc5 = tc && ((uintptr_t)st->S % 16) == 0 && (st->S_seq_stride % 4) == 0 && !(variant && variant[0] == 'm');
    if (l->conv_k == 4 && Cc % 4 == 0 && st->conv_seq_stride % 4 == 0 && ((uintptr_t)qkv % 16) == 0 &&
        ((uintptr_t)st->conv % 16) == 0 && ((uintptr_t)l->conv_w % 16) == 0 && ((uintptr_t)l->conv_b % 16) == 0) {
        dim3 cgrid((unsigned)((Cc + 511) / 512), (T + CONV4_TOK - 1) / CONV4_TOK, n_seq);
        if (tc5) {
            // the tcgen05 path: conv, chunk preparation and scan, slab by slab (see launch_linear_prefill_tc5)
            TC5Front front;
            const char *plain_conv = getenv("ORNITH_CUDA_CONV_PLAIN");       // =1: the plain-load conv kernel
            const bool conv_tma = !(plain_conv && plain_conv[0] == '1');
            front.conv = [=](int t_begin, int t_end, cudaStream_t cs) -> ornith_status {
                if (conv_tma) {                                              // tensor-copy-fed kernel where the shape allows
                    bool handled = false;
                    ORN_TRY(launch_conv4_silu_prefill_tma(x, n_seq, act_dtype, Y, rq, rk, t_begin, t_end, cs, &handled));
                    if (handled) return ORNITH_OK;
                }
                dim3 g((unsigned)((Cc + 511) / 512), (unsigned)((t_end - t_begin + CONV4_TOK - 1) / CONV4_TOK), (unsigned)n_seq);
                if (bf) k_conv4_silu_prefill<__nv_bfloat16, true, true><<<g, 128, 0, cs>>>(x, Y, rq, rk, t_begin, t_end);
                else    k_conv4_silu_prefill<float, true, true><<<g, 128, 0, cs>>>(x, Y, rq, rk, t_begin, t_end);
                return orn_check_launch("k_conv4_silu_prefill");
            };
            front.ring_refresh = [=](cudaStream_t cs) {
                dim3 rg((unsigned)((Cc + 255) / 256), n_seq);
                if (bf) k_conv_ring_refresh<__nv_bfloat16><<<rg, 256, 0, cs>>>(x);
                else    k_conv_ring_refresh<float><<<rg, 256, 0, cs>>>(x);
                return orn_check_launch("k_conv_ring_refresh");
            };
            return launch_linear_prefill_tc5(x, n_seq, act_dtype, Y, rq, rk, nullptr, nullptr, &front, blocks, g_delta_scan_dump, s);
        }
        else if (bf && tc)  k_conv4_silu_prefill<__nv_bfloat16, true, false><<<cgrid, 128, 0, s>>>(x, Y, nullptr, nullptr, 0, T);
        else if (bf)   k_conv4_silu_prefill<__nv_bfloat16, false, false><<<cgrid, 128, 0, s>>>(x, Y, nullptr, nullptr, 0, T);
        else if (tc)   k_conv4_silu_prefill<float, true, false><<<cgrid, 128, 0, s>>>(x, Y, nullptr, nullptr, 0, T);
        else           k_conv4_silu_prefill<float, false, false><<<cgrid, 128, 0, s>>>(x, Y, nullptr, nullptr, 0, T);
        ORN_TRY(orn_check_launch("k_conv4_silu_prefill"));
    } else {
        dim3 cgrid((unsigned)((Cc + 127) / 128), (T + CONV_TOK - 1) / CONV_TOK, n_seq);
        if (bf) k_conv_silu_prefill<__nv_bfloat16><<<cgrid, 128, 0, s>>>(x, Y);
        else    k_conv_silu_prefill<float><<<cgrid, 128, 0, s>>>(x, Y);
        ORN_TRY(orn_check_launch("k_conv_silu_prefill"));
    }
    dim3 rgrid((unsigned)((Cc + 255) / 256), n_seq);
    if (bf) k_conv_ring_refresh<__nv_bfloat16><<<rgrid, 256, 0, s>>>(x);
    else    k_conv_ring_refresh<float><<<rgrid, 256, 0, s>>>(x);
    ORN_TRY(orn_check_launch("k_conv_ring_refresh"));
    if (bf) k_linear_prep<__nv_bfloat16><<<(unsigned)n_tok, 128, 0, s>>>(x, Y, (int)n_tok, rq, rk, la, be);
    else    k_linear_prep<float><<<(unsigned)n_tok, 128, 0, s>>>(x, Y, (int)n_tok, rq, rk, la, be);
    ORN_TRY(orn_check_launch("k_linear_prep"));

    dim3 grid(l->nv, n_seq);
    if (l->dk == 128 && l->dv == 128) {
        // default: tf32 tensor-core scan; ORNITH_CUDA_PREFILL_FP32=1 keeps every product in fp32
        if (tc5) return launch_linear_prefill_tc5(x, n_seq, act_dtype, Y, rq, rk, la, be, nullptr, blocks, g_delta_scan_dump, s);
        if (tc) return launch_linear_prefill_tc(x, n_seq, act_dtype, Y, rq, rk, la, be, blocks, s);
        if (chunk >= 32) return bf ? launch_chunk<32, __nv_bfloat16>(x, grid, Y, rq, rk, la, be, s)
                                   : launch_chunk<32, float>(x, grid, Y, rq, rk, la, be, s);
        return bf ? launch_chunk<16, __nv_bfloat16>(x, grid, Y, rq, rk, la, be, s)
                  : launch_chunk<16, float>(x, grid, Y, rq, rk, la, be, s);
    }
    const size_t smem = (size_t)(2 * l->dk + 2 * l->dv) * sizeof(float);
    if (bf) k_linear_prefill_seq<__nv_bfloat16><<<grid, 128, smem, s>>>(x, Y, rq, rk, la, be);
    else    k_linear_prefill_seq<float><<<grid, 128, smem, s>>>(x, Y, rq, rk, la, be);
    return orn_check_launch("k_linear_prefill_seq");
}

ornith_status ornith_cuda_conv_export(const float *ring, int conv_k, int Cc, int pos, float *image, void *stream) {
    ORN_TRY(orn_require_device());
    if (conv_k < 1 || Cc <= 0 || pos < 0) { orn_record_error("conv_export: bad arguments"); return ORNITH_ERR_FORMAT; }
    k_conv_ring_image<<<(Cc + 255) / 256, 256, 0, as_stream(stream)>>>((float *)ring, image, conv_k, Cc, pos, 1);
    return orn_check_launch("k_conv_ring_image");
}

ornith_status ornith_cuda_conv_import(float *ring, int conv_k, int Cc, int pos, const float *image, void *stream) {
    ORN_TRY(orn_require_device());
    if (conv_k < 1 || Cc <= 0 || pos < 0) { orn_record_error("conv_import: bad arguments"); return ORNITH_ERR_FORMAT; }
    k_conv_ring_image<<<(Cc + 255) / 256, 256, 0, as_stream(stream)>>>(ring, (float *)image, conv_k, Cc, pos, 0);
    return orn_check_launch("k_conv_ring_image");
}

ornith_status ornith_cuda_delta_step(float *S, int n_heads, int dk, int dv, const float *q, const float *k,
                                     const float *v, const float *alpha, const float *beta, float *o, void *stream) {
    ORN_TRY(orn_require_device());
    if (n_heads <= 0) return ORNITH_OK;
    if (dk <= 0 || dv <= 0 || dk > 2048 || dv > 2048) { orn_record_error("delta_step: bad head dims"); return ORNITH_ERR_FORMAT; }
    k_delta_step_raw<<<n_heads, 128, (size_t)(2 * dk + 2 * dv) * 4, as_stream(stream)>>>(S, dk, dv, q, k, v, alpha, beta, o);
    return orn_check_launch("k_delta_step_raw");
}

ornith_status ornith_cuda_delta_prefill(float *S, int dk, int dv, const float *Q, const float *K, const float *V,
                                        const float *alpha, const float *beta, int T, int chunk, float *O,
                                        void *stream) {
    ORN_TRY(orn_require_device());
    (void)chunk;                          // any tiling must give the result of T steps
    if (T <= 0) return ORNITH_OK;
    if (dk <= 0 || dv <= 0 || dk > 2048 || dv > 2048) { orn_record_error("delta_prefill: bad head dims"); return ORNITH_ERR_FORMAT; }
    k_delta_prefill_seq_raw<<<1, 128, (size_t)(2 * dk + 2 * dv) * 4, as_stream(stream)>>>(S, dk, dv, Q, K, V, alpha, beta, T, O);
    return orn_check_launch("k_delta_prefill_seq_raw");
}

ornith_status ornith_cuda_conv_image(float *image, int K, int C, const float *X, const float *w, const float *bias,
                                     int T, float *OUT, void *stream) {
    ORN_TRY(orn_require_device());
    if (K < 1 || K > 9 || C <= 0) { orn_record_error("conv: kernel size %d unsupported", K); return ORNITH_ERR_UNSUPPORTED; }
    if (T <= 0) return ORNITH_OK;
    k_conv_image<<<(C + 127) / 128, 128, 0, as_stream(stream)>>>(image, K, C, X, w, bias, T, OUT);
    return orn_check_launch("k_conv_image");
}

}  // extern "C"
