// linear_decode_ring.cu — persistent form of the fused delta-net decode step (dk = dv = 128,
// conv_k = 4): the recurrent state is streamed through a ring of bulk copies.
//
// Same arithmetic, operation order and results as k_linear_decode_128 (linear_attn.cu; reference:
// src/ornith_rforward.c:457-503, :300-319, src/ornith_attn.c:203-212, :373-381).  What differs is
// how the 64 KiB state of a head reaches the registers.  Two CTAs per SM stay resident and walk
// the (sequence, value head) units in a fixed stride; each keeps three 32 KiB stages (half a
// head) in shared memory, filled by cp.async.bulk with completion on an mbarrier, and requests
// half-head m+3 as soon as half-head m has been lifted into registers.  The copy engine thus has
// work queued for the whole life of the CTA, instead of each short-lived CTA starting with an
// empty pipe; the small per-unit operands (conv ring, activations, gates, z) of the next unit are
// requested one unit ahead.  Every mbarrier wait is bounded; a wait that gives up poisons the
// outputs of the CTA.
#include "bulk_copy.cuh"
#include "linear_attn.cuh"

namespace {

constexpr int STAGES = 3;
constexpr int STAGE_FLOATS = 64 * 128;                // half a head: 64 rows of the state, 32 KiB
constexpr uint32_t STAGE_BYTES = STAGE_FLOATS * 4;

// Everything a unit needs apart from its state.  Activations stay in their storage type until
// they are used: a conversion at the load would make the thread wait for the data there, and
// these loads are issued a whole unit ahead precisely so that nobody waits for them.
template <typename ACT>
struct UnitOperands {
    float h0[4], h1[4], bias0, bias1, acoef, dtb, nw[2][2];
    ACT x0, x1, ain, bin, zin[2][2];
    float4 w0, w1;
    int t;
};
__device__ __forceinline__ float act_f(float v) { return v; }
__device__ __forceinline__ float act_f(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename ACT>
__device__ __forceinline__ void load_operands(UnitOperands<ACT> &o, const LinArgs &a, int b, int hv, int tid, int w, int sr,
                                              int cc) {
    const int kh = key_head_of(a, hv), qd = a.nk * 128, vd = a.nv * 128, Cc = 2 * qd + vd;
    const float *ring = a.conv + (size_t)b * a.conv_stride;
    const ACT *x = (const ACT *)a.qkv + (size_t)b * Cc;
    const bool qk_thread = tid < 128;
    const int c0 = qk_thread ? kh * 128 + tid : 2 * qd + hv * 128 + (tid - 128);
    const int c1 = qd + kh * 128 + (tid & 127);
#pragma unroll
    for (int sl = 0; sl < 4; sl++) { o.h0[sl] = ring[(size_t)sl * Cc + c0]; o.h1[sl] = 0.0f; }
    o.x0 = x[c0];
    o.w0 = *reinterpret_cast<const float4 *>(a.conv_w + (size_t)c0 * 4);
    o.bias0 = a.conv_b ? a.conv_b[c0] : 0.0f;
    o.x1 = x[c0]; o.bias1 = 0.0f; o.w1 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);      // x1 only matters on q/k threads
    if (qk_thread) {
#pragma unroll
        for (int sl = 0; sl < 4; sl++) o.h1[sl] = ring[(size_t)sl * Cc + c1];
        o.x1 = x[c1];
        o.w1 = *reinterpret_cast<const float4 *>(a.conv_w + (size_t)c1 * 4);
        o.bias1 = a.conv_b ? a.conv_b[c1] : 0.0f;
    }
    o.t = a.pos[b];
    o.ain = ((const ACT *)a.a)[(size_t)b * a.nv + hv];
    o.bin = ((const ACT *)a.b)[(size_t)b * a.nv + hv];
    o.acoef = a.a_coef[hv]; o.dtb = a.dt_bias[hv];
    const size_t out_base = (size_t)b * vd + (size_t)hv * 128;
#pragma unroll
    for (int h = 0; h < 2; h++)
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int r = 64 * h + 8 * w + 4 * i + sr;
            o.zin[h][i] = ((const ACT *)a.z)[out_base + (cc == 0 ? r : 0)];
            o.nw[h][i] = (cc == 0) ? a.norm_w[r] : 0.0f;
        }
}

template <typename ACT>
__global__ void __launch_bounds__(256, 2) k_linear_decode_ring(LinArgs a, int n_units) {
    extern __shared__ __align__(128) unsigned char smraw[];
    float *stage = reinterpret_cast<float *>(smraw);
    __shared__ __align__(16) float q_s[128], k_s[128], v_s[128];
    __shared__ double redd[32];
    __shared__ float gates[2];
    __shared__ unsigned long long full[STAGES];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, sr = lane >> 3, cc = lane & 7;
    const int qd = a.nk * 128, vd = a.nv * 128, Cc = 2 * qd + vd;
    const int n_mine = (n_units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int M = 2 * n_mine;                            // half-heads this CTA walks

    auto half_src = [&](int m) -> const float * {        // state rows 64 (m&1) .. of this CTA's unit m/2
        const int u = (int)blockIdx.x + (m >> 1) * (int)gridDim.x;
        return a.S + (size_t)(u / a.nv) * a.S_stride + (size_t)(u % a.nv) * 128 * 128 + (size_t)(m & 1) * STAGE_FLOATS;
    };
    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) bc_mbar_init(bc_smem_u32(&full[s]), 1);
        bc_mbar_init_fence();
    }
    __syncthreads();
    if (tid == 0) {
        for (int m = 0; m < STAGES && m < M; m++) {
            bc_mbar_expect_tx(bc_smem_u32(&full[m]), STAGE_BYTES);
            bc_copy(bc_smem_u32(stage + m * STAGE_FLOATS), half_src(m), STAGE_BYTES, bc_smem_u32(&full[m]));
        }
    }
    bool ok = true;
    UnitOperands<ACT> nxt;
    load_operands<ACT>(nxt, a, (int)blockIdx.x / a.nv, (int)blockIdx.x % a.nv, tid, w, sr, cc);

    for (int k = 0; k < n_mine; k++) {
        const int u = (int)blockIdx.x + k * (int)gridDim.x, b = u / a.nv, hv = u % a.nv;
        const int kh = key_head_of(a, hv);
        float *S = a.S + (size_t)b * a.S_stride + (size_t)hv * 128 * 128;
        float *ring = a.conv + (size_t)b * a.conv_stride;
        const UnitOperands<ACT> cur = nxt;
        if (k + 1 < n_mine) {
            const int un = u + (int)gridDim.x;
            load_operands<ACT>(nxt, a, un / a.nv, un % a.nv, tid, w, sr, cc);
        }
        const bool qk_thread = tid < 128;
        const int c0 = qk_thread ? kh * 128 + tid : 2 * qd + hv * 128 + (tid - 128);
        const int c1 = qd + kh * 128 + (tid & 127);
        const int t = cur.t;

        // ---- conv + SiLU, q/k L2-norm (reference: src/ornith_tensor.c:155-160), gates ------------
        const int sb = (t + 1) & 3;
        const bool own = owns_key_head(a, hv);
        const float x0 = act_f(cur.x0), x1 = act_f(cur.x1);
        const float y0 = conv4_silu(cur.h0, x0, cur.w0, cur.bias0, sb);
        float y1 = 0.0f;
        if (qk_thread) {
            y1 = conv4_silu(cur.h1, x1, cur.w1, cur.bias1, sb);
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
            gates[0] = expf(cur.acoef * softplus_f(act_f(cur.ain) + cur.dtb));
            gates[1] = sigmoid_f(act_f(cur.bin));
        }
        __syncthreads();

        // ---- S <- alpha S; u = beta (v - S k); S += u k^T; o = S q  (reference: src/ornith_attn.c:203-212)
        const float alpha = gates[0], beta = gates[1];
        float4 kr[4], qr[4];                              // this lane's 16 columns of k and q, for all its rows
#pragma unroll
        for (int j = 0; j < 4; j++) {
            kr[j] = *reinterpret_cast<const float4 *>(k_s + (cc + j * 8) * 4);
            qr[j] = *reinterpret_cast<const float4 *>(q_s + (cc + j * 8) * 4);
        }
        float orow[2][2];
        double ss = 0.0;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int m = 2 * k + h, slot = m % STAGES;
            ok = ok && bc_mbar_wait(bc_smem_u32(&full[slot]), (uint32_t)(m / STAGES) & 1u);
            float4 s[2][4];
#pragma unroll
            for (int i = 0; i < 2; i++)
#pragma unroll
                for (int j = 0; j < 4; j++)
                    s[i][j] = lds128(stage + slot * STAGE_FLOATS + (8 * w + 4 * i + sr) * 128 + (cc + j * 8) * 4);
            __syncthreads();                              // the half-head is in registers everywhere: refill the slot
            if (tid == 0 && m + STAGES < M) {
                bc_fence_proxy_async();
                bc_mbar_expect_tx(bc_smem_u32(&full[slot]), STAGE_BYTES);
                bc_copy(bc_smem_u32(stage + slot * STAGE_FLOATS), half_src(m + STAGES), STAGE_BYTES, bc_smem_u32(&full[slot]));
            }
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const int r = 64 * h + 8 * w + 4 * i + sr;
                float recall = 0.0f;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    s[i][j].x *= alpha; s[i][j].y *= alpha; s[i][j].z *= alpha; s[i][j].w *= alpha;
                    recall += s[i][j].x * kr[j].x + s[i][j].y * kr[j].y + s[i][j].z * kr[j].z + s[i][j].w * kr[j].w;
                }
                recall += __shfl_xor_sync(0xffffffffu, recall, 1);
                recall += __shfl_xor_sync(0xffffffffu, recall, 2);
                recall += __shfl_xor_sync(0xffffffffu, recall, 4);
                const float uu = beta * (v_s[r] - recall);
                float read = 0.0f;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    s[i][j].x += uu * kr[j].x; s[i][j].y += uu * kr[j].y; s[i][j].z += uu * kr[j].z; s[i][j].w += uu * kr[j].w;
                    read += s[i][j].x * qr[j].x + s[i][j].y * qr[j].y + s[i][j].z * qr[j].z + s[i][j].w * qr[j].w;
                    if (!ok) s[i][j] = make_float4(NAN, NAN, NAN, NAN);
                    __stcs(reinterpret_cast<float4 *>(S + (size_t)r * 128) + cc + j * 8, s[i][j]);
                }
                read += __shfl_xor_sync(0xffffffffu, read, 1);
                read += __shfl_xor_sync(0xffffffffu, read, 2);
                read += __shfl_xor_sync(0xffffffffu, read, 4);
                orow[h][i] = read * a.out_scale;          // scaled head output of row r (all 8 lanes agree)
                if (cc == 0) ss += (double)orow[h][i] * (double)orow[h][i];
            }
        }

        // ---- per-head RMSNorm and SiLU(z) gate (reference: src/ornith_rforward.c:305-314) ---------
        ss = warp_sum(ss);
        if (lane == 0) redd[16 + w] = ss;
        __syncthreads();
        if (cc == 0) {
            double tot = 0.0;
#pragma unroll
            for (int i = 0; i < 8; i++) tot += redd[16 + i];
            const float inv = ok ? (float)(1.0 / sqrt(tot / 128.0 + (double)a.eps)) : NAN;
            const size_t out_base = (size_t)b * vd + (size_t)hv * 128;
#pragma unroll
            for (int h = 0; h < 2; h++)
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const int r = 64 * h + 8 * w + 4 * i + sr;
                    float y = orow[h][i] * inv * cur.nw[h][i];
                    y *= silu_f(act_f(cur.zin[h][i]));
                    act_st((ACT *)a.out, out_base + r, y);
                }
        }
    }
}

template <typename ACT>
ornith_status launch_ring(const LinArgs &x, int n_units, cudaStream_t s) {
    static int n_sm = 0;
    if (!n_sm) {
        int dev = 0;
        ORN_TRY(orn_check(cudaGetDevice(&dev), "cudaGetDevice"));
        ORN_TRY(orn_check(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev), "SM count"));
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_linear_decode_ring<ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)(STAGES * STAGE_BYTES)), "decode ring smem opt-in"));
    }
    const int grid = n_units < 2 * n_sm ? n_units : 2 * n_sm;
    k_linear_decode_ring<ACT><<<grid, 256, STAGES * STAGE_BYTES, s>>>(x, n_units);
    return orn_check_launch("k_linear_decode_ring");
}

}  // namespace

ornith_status launch_linear_decode_ring(const LinArgs &x, int n_seq, int act_dtype, cudaStream_t s) {
    const int n_units = n_seq * x.nv;
    return act_dtype == ORNITH_ACT_BF16 ? launch_ring<__nv_bfloat16>(x, n_units, s) : launch_ring<float>(x, n_units, s);
}
