// gqa_prefill_tc.cu — causal GQA prefill (head_dim 256) on the 5th-generation tensor cores:
// TMA-staged operands, tcgen05.mma with the score and output accumulators in tensor memory.
//
// Replaces the core of full_attn_prefill() (reference: src/ornith_rforward.c:529-551, which
// runs ornith_gqa_step once per token).  Inputs are the f16 images the front end prepares:
// query rows (k_q_rows_to_f16, each row scaled by a power of two into [-1, 1]) and the decoded
// rows of the cache (k_kv_rows_to_f16), so quantised caches are attended over in their decoded
// form, the current token included, exactly as the reference does.
//
// One CTA = 128 query tokens of one head, 14 warps (22 with four softmax threads per row):
//   warps 8,13  producers one lane each issues TMA loads (128B-swizzled boxes of 64 dims): warp 8
//                         dims 128..255 of the query tile once, then the 64-key K tiles (3
//                         stages); warp 13 the V tiles (2 stages)
//   warps 9-11  scores    one lane each issues S_j = Q K_j^T (16 x tcgen05.mma M128 N64 K16) for
//                         the tiles j = 0, 1, 2 (mod 3) into its own score buffer
//   warp 12     values    one lane issues O += P_j V_j (4 x M128 N256 K16)
//                         Several issuing threads because one thread issues at most one MMA per
//                         64-96 cycles, several times what an N = 64 product occupies the pipe;
//                         three score buffers so that the chain issue -> softmax -> value product
//                         -> next issue of a buffer spans three tiles.
//   warps 0-7   softmax   two threads per query row (= TMEM lane), 32 of the 64 scores each:
//                         they first put dims 0..127 of the query tile into tensor memory
//                         (tcgen05.st), then per tile tcgen05.ld the scores, online softmax in
//                         the log2 domain against a reference maximum that is only moved (and O
//                         rescaled through tcgen05.ld/st) when a row maximum exceeds it by 2^8,
//                         and store the f16 probabilities over the scores they came from;
//                         finally the epilogue (1/l, sigmoid output gate, store).
// Tensor memory columns: 0-255 the output tile, 256-447 three score / probability buffers,
// 448-511 dims 0..127 of the query tile (two f16 per column).  The A operands that live there
// (half of Q, all of P) keep shared-memory bandwidth for K, V and the other half of Q.
// Every wait on an mbarrier is bounded; a wait that gives up poisons the CTA's outputs.
#include <cuda.h>

#include "full_attn.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int HD = 256, BM = 128, BN = 64;
constexpr int SM_K = 0, SM_V = 98304, SM_Q = 163840, SM_BYTES = 196608;   // 3 K + 2 V stages of 32 KiB, half the query tile; + 1 KiB slack
constexpr int TM_O = 0, TM_S = 256, TM_Q = 448, TM_COLS = 512;   // tensor-memory columns
constexpr float LOG2E = 1.4426950408889634f;
constexpr float GROW = 8.0f;               // move the reference maximum when exceeded by 2^8

struct TcArgs {
    const int64_t *seq_off;
    const int32_t *kv_len;
    const __half *Qh;                      // [n_seq*nh*T][256] query rows, each scaled by a power of two
    const float *rs;                       // [n_seq*nh*T] per-row factor: scale * 2^e * log2(e)
    const void *qproj;
    void *out;
    int nh, nkv, T, Lmax, Lp, gated;
    unsigned int *status;                  // status word of the device: a wait that gives up reports here
};

using namespace tc5;

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

// ---- f16 image of the query rows: one warp per (token, head); rows scaled by 2^-e --------
__global__ void __launch_bounds__(128) k_q_rows_to_f16(const float *q_prep, __half *Qh, float *rs, int n_seq, int T,
                                                       int nh, float scale) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const size_t row = (size_t)blockIdx.x * 4 + w;       // (b*T + t)*nh + h
    if (row >= (size_t)n_seq * T * nh) return;
    const int h = (int)(row % nh);
    const size_t tok = row / nh;
    const int b = (int)(tok / T), t = (int)(tok % T);
    const float *q = q_prep + row * HD + lane * 8;
    const float4 v0 = *reinterpret_cast<const float4 *>(q), v1 = *reinterpret_cast<const float4 *>(q + 4);
    float mx = fmaxf(fmaxf(fmaxf(fabsf(v0.x), fabsf(v0.y)), fmaxf(fabsf(v0.z), fabsf(v0.w))),
                     fmaxf(fmaxf(fabsf(v1.x), fabsf(v1.y)), fmaxf(fabsf(v1.z), fabsf(v1.w))));
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    int e = 0;
    if (mx > 0.0f && mx < INFINITY) (void)frexpf(mx, &e);
    const float down = exp2f((float)-e);
    const size_t orow = ((size_t)b * nh + h) * T + t;
    *reinterpret_cast<uint4 *>(Qh + orow * HD + lane * 8) =
        make_uint4(pack_h2(v0.x * down, v0.y * down), pack_h2(v0.z * down, v0.w * down),
                   pack_h2(v1.x * down, v1.y * down), pack_h2(v1.z * down, v1.w * down));
    if (lane == 0) rs[orow] = scale * exp2f((float)e) * LOG2E;
}

constexpr int NSK = 3, NSV = 2;            // K and V stages
constexpr int NB = 3;                      // score / probability buffers in tensor memory

struct TcBars {
    unsigned long long q_full, k_full[NSK], k_empty[NSK], v_full[NSV], v_empty[NSV], s_full[NB], pv_done[NB], p_full;
};

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// barrier among the NQ softmax warps that share 32 query rows
template <int NQ>
__device__ __forceinline__ void row_sync(int id) { asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(32 * NQ) : "memory"); }
__device__ __forceinline__ void ld_scores(uint32_t t, float (&s)[32]) { tmem_ld32_wait(t, s); }
__device__ __forceinline__ void ld_scores(uint32_t t, float (&s)[16]) { tmem_ld16_wait(t, s); }
__device__ __forceinline__ void st_cols(uint32_t t, const float (&s)[32]) { tmem_st32(t, s); }
__device__ __forceinline__ void st_cols(uint32_t t, const float (&s)[16]) { tmem_st16(t, s); }
__device__ __forceinline__ void st_cols(uint32_t t, const float (&s)[8]) { tmem_st8(t, s); }

// NQ = softmax threads per query row (2 or 4): warps 0 .. 4 NQ - 1 are the softmax warps, then the K producer, the three
// score issuers, the value issuer and the V producer.  With 4 the per-tile softmax (its loads, the exchange of the row
// maxima, 64 exponentials per row, the store) is spread over twice the warps; it measures no faster (see the launch).
template <typename ACT, int NQ>
__global__ void __launch_bounds__((4 * NQ + 6) * 32, 1) k_gqa_prefill_tc(const __grid_constant__ CUtensorMap mq,
                                                           const __grid_constant__ CUtensorMap mk,
                                                           const __grid_constant__ CUtensorMap mv, TcArgs a) {
    extern __shared__ unsigned char smraw[];
    __shared__ TcBars bars;
    constexpr int W_K = 4 * NQ, W_QK = W_K + 1, W_PV = W_K + 4, W_V = W_K + 5, COLS = BN / NQ, OCOLS = HD / NQ;
    __shared__ float xch[NB][NQ][BM];                          // [score buffer][column part][row]: partial row maxima
    __shared__ float lx[NQ][BM];                               // [column part][row]: partial row sums
    __shared__ uint32_t tmem_base_s;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.y, b = blockIdx.z, kvh = h / (a.nh / a.nkv);
    const int q0 = (int)(gridDim.x - 1 - blockIdx.x) * BM;     // long rows first
    const int cap = (int)(a.seq_off[b + 1] - a.seq_off[b]);
    const int len0 = a.kv_len[b];
    // tokens that were really appended: the engine stops appending when the cache is full
    const int t_end = min(a.T, max(0, min(cap, a.Lmax) - len0));
    if (q0 >= t_end) return;
    const int rows_here = min(BM, t_end - q0);
    const int kmax = len0 + q0 + rows_here - 1;                // last key any row of the CTA sees
    const int n_tiles = kmax / BN + 1;
    const uint32_t base = (su32(smraw) + 1023u) & ~1023u;      // 128B-swizzle atoms are 1 KiB aligned

    if (tid == 0) {
        mbar_init(su32(&bars.q_full), 128 * NQ + 1);           // every softmax thread's share stored to tensor memory + the TMA half
        for (int s = 0; s < NSK; s++) { mbar_init(su32(&bars.k_full[s]), 1); mbar_init(su32(&bars.k_empty[s]), 1); }
        for (int s = 0; s < NSV; s++) { mbar_init(su32(&bars.v_full[s]), 1); mbar_init(su32(&bars.v_empty[s]), 1); }
        for (int s = 0; s < NB; s++) { mbar_init(su32(&bars.s_full[s]), 1); mbar_init(su32(&bars.pv_done[s]), 1); }
        mbar_init(su32(&bars.p_full), 128 * NQ);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == W_PV) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(su32(&tmem_base_s)), "r"((uint32_t)TM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = tmem_base_s;
    bool ok = true;

    if (warp == W_K) {
        // ================= producer =================
        if (lane == 0) {
            // dims 128..255 of the query tile stay in shared memory (two 64-dim slabs)
            mbar_expect_tx(su32(&bars.q_full), 32768u);
            const int qrow = (b * a.nh + h) * a.T + q0;
            for (int s = 0; s < 2; s++) tma_load_2d(base + SM_Q + s * 16384, &mq, 128 + s * 64, qrow, su32(&bars.q_full));
            const int krow = (b * a.nkv + kvh) * a.Lp;
            for (int j = 0; j < n_tiles; j++) {
                const int sk = j % NSK;
                if (j >= NSK) ok = mbar_wait(su32(&bars.k_empty[sk]), (uint32_t)(j / NSK - 1) & 1u);
                if (!ok) break;
                mbar_expect_tx(su32(&bars.k_full[sk]), 32768u);
                for (int s = 0; s < 4; s++)
                    tma_load_2d(base + SM_K + sk * 32768 + s * 8192, &mk, s * 64, krow + j * BN, su32(&bars.k_full[sk]));
            }
        }
    } else if (warp == W_V) {
        // ================= producer of the V tiles =================
        // its own lane: a V stage is released late (after the value product of its tile), and
        // waiting for that must not hold back the K tiles, which the score MMAs need much earlier
        if (lane == 0) {
            const int krow = (b * a.nkv + kvh) * a.Lp;
            for (int j = 0; j < n_tiles; j++) {
                const int sv = j % NSV;
                if (j >= NSV) ok = mbar_wait(su32(&bars.v_empty[sv]), (uint32_t)(j / NSV - 1) & 1u);
                if (!ok) break;
                mbar_expect_tx(su32(&bars.v_full[sv]), 32768u);
                for (int s = 0; s < 4; s++)
                    tma_load_2d(base + SM_V + sv * 32768 + s * 8192, &mv, s * 64, krow + j * BN, su32(&bars.v_full[sv]));
            }
        }
    } else if (warp >= W_QK && warp < W_QK + 3) {
        // ================= score MMAs: warp 9 + e issues the tiles j = e (mod 3) =================
        // One thread cannot issue tcgen05.mma faster than one per ~64-96 cycles, two to three times
        // the 32 cycles an M128 N64 K16 product occupies the pipe; several issuing threads overlap.
        // With three score buffers the chain issue -> softmax -> value product -> next issue of a
        // buffer spans three tiles.  Dims 0..127 of Q are a tensor-memory operand, dims 128..255 a
        // shared-memory one (512 columns: output 256, scores 3 x 64, query 64).
        if (lane == 0) {
            const int e = warp - W_QK;
            const uint32_t idesc_qk = (1u << 4) | (8u << 17) | (8u << 24);                 // f16 x f16 -> f32, N 64, M 128
            ok = mbar_wait(su32(&bars.q_full), 0);
            const uint64_t qd = smem_desc(base + SM_Q, 16, 1024);
            for (int j = e; j < n_tiles && ok; j += NB) {
                const int st = j % NSK;
                ok = mbar_wait(su32(&bars.k_full[st]), (uint32_t)(j / NSK) & 1u);
                // this buffer still holds the probabilities of tile j-3 until their value product is done
                if (ok && j >= NB) ok = mbar_wait(su32(&bars.pv_done[e]), (uint32_t)(j / NB - 1) & 1u);
                if (!ok) break;
                fence_after();
                const uint64_t kd = smem_desc(base + SM_K + st * 32768, 16, 1024);
#pragma unroll
                for (int ks = 0; ks < 8; ks++)
                    mma_f16_ts(tmem + TM_S + e * BN, tmem + TM_Q + ks * 8, kd + (uint64_t)(((ks >> 2) * 8192 + (ks & 3) * 32) >> 4),
                               idesc_qk, ks > 0);
#pragma unroll
                for (int ks = 8; ks < 16; ks++)
                    mma_f16_ss(tmem + TM_S + e * BN, qd + (uint64_t)((((ks - 8) >> 2) * 16384 + (ks & 3) * 32) >> 4),
                               kd + (uint64_t)(((ks >> 2) * 8192 + (ks & 3) * 32) >> 4), idesc_qk, 1u);
                mma_commit(su32(&bars.k_empty[st]));
                mma_commit(su32(&bars.s_full[e]));
            }
        }
    } else if (warp == W_PV) {
        // ================= value MMAs =================
        if (lane == 0) {
            const uint32_t idesc_pv = (1u << 4) | (1u << 16) | (32u << 17) | (8u << 24);   // B MN-major, N 256, M 128
            for (int j = 0; j < n_tiles && ok; j++) {
                const int st = j % NSV, sb = j % NB;
                ok = mbar_wait(su32(&bars.p_full), (uint32_t)j & 1u) &&
                     mbar_wait(su32(&bars.v_full[st]), (uint32_t)(j / NSV) & 1u);
                if (!ok) break;
                fence_after();
                const uint64_t vd = smem_desc(base + SM_V + st * 32768, 8192, 1024);
#pragma unroll
                for (int ks = 0; ks < 4; ks++)
                    mma_f16_ts(tmem + TM_O, tmem + TM_S + sb * BN + ks * 8, vd + (uint64_t)((ks * 2048) >> 4), idesc_pv,
                               (j > 0 || ks > 0) ? 1u : 0u);
                mma_commit(su32(&bars.v_empty[st]));
                mma_commit(su32(&bars.pv_done[sb]));
            }
        }
    } else {
        // ======== softmax + epilogue: NQ threads per query row (= TMEM lane), 64 / NQ columns each ========
        const int wq = warp & 3, part = warp >> 2;             // TMEM lane quarter, column part
        const int row = wq * 32 + lane;
        const bool live = row < rows_here;
        const int qpos = live ? len0 + q0 + row : 0x7fffffff;  // rows past the end mask nothing and are not stored
        const size_t qrow = ((size_t)b * a.nh + h) * a.T + q0 + row;
        const float rscale = live ? a.rs[qrow] : 0.0f;
        const uint32_t lane_t = tmem + ((uint32_t)(wq * 32) << 16);
        {   // dims 0..127 of the query row -> tensor memory: 128 / NQ halves per thread, two per 32-bit column
            const uint4 *src = reinterpret_cast<const uint4 *>(a.Qh + qrow * HD + (128 / NQ) * part);
            float q[COLS];
#pragma unroll
            for (int i = 0; i < COLS / 4; i++) {
                const uint4 v = live ? src[i] : make_uint4(0u, 0u, 0u, 0u);
                q[4 * i] = __uint_as_float(v.x); q[4 * i + 1] = __uint_as_float(v.y);
                q[4 * i + 2] = __uint_as_float(v.z); q[4 * i + 3] = __uint_as_float(v.w);
            }
            st_cols(lane_t + TM_Q + COLS * part, q);
            tmem_wait_st();
            fence_before();
            mbar_arrive(su32(&bars.q_full));
        }
        float m_ref = -INFINITY, l = 0.0f;
        for (int j = 0; j < n_tiles; j++) {
            const int sb = j % NB, key0 = j * BN + COLS * part;
            ok = ok && mbar_wait(su32(&bars.s_full[sb]), (uint32_t)(j / NB) & 1u);
            fence_after();
            float s[COLS];
            ld_scores(lane_t + TM_S + sb * BN + COLS * part, s);
            if (key0 + COLS - 1 > qpos) {                      // the tile reaches past this row's diagonal
#pragma unroll
                for (int c = 0; c < COLS; c++)
                    if (key0 + c > qpos) s[c] = -INFINITY;
            }
            float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < COLS; c += 4) {
                m4[0] = fmaxf(m4[0], s[c]); m4[1] = fmaxf(m4[1], s[c + 1]);
                m4[2] = fmaxf(m4[2], s[c + 2]); m4[3] = fmaxf(m4[3], s[c + 3]);
            }
            float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
            xch[sb][part][row] = mx;
            row_sync<NQ>(1 + wq);                              // also: every part holds its scores in registers now
#pragma unroll
            for (int p = 1; p < NQ; p++) mx = fmaxf(mx, xch[sb][(part + p) % NQ][row]);
            mx = live ? mx * rscale : 0.0f;                    // rscale > 0 on live rows
            float corr = 1.0f;
            const bool grow = mx > m_ref + GROW || m_ref == -INFINITY;
            if (grow && mx > -INFINITY) {
                corr = ex2_approx(m_ref - mx);                 // 0 on the first tile
                m_ref = mx;
                l *= corr;
            }
            const float msafe = (m_ref == -INFINITY) ? 0.0f : m_ref;
            float pk[COLS / 2];
            float p4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int c = 0; c < COLS / 4; c++) {
                const float e0 = ex2_approx(fmaf(s[4 * c], rscale, -msafe)), e1 = ex2_approx(fmaf(s[4 * c + 1], rscale, -msafe));
                const float e2 = ex2_approx(fmaf(s[4 * c + 2], rscale, -msafe)), e3 = ex2_approx(fmaf(s[4 * c + 3], rscale, -msafe));
                p4[0] += e0; p4[1] += e1; p4[2] += e2; p4[3] += e3;
                pk[2 * c] = __uint_as_float(pack_h2(e0, e1));
                pk[2 * c + 1] = __uint_as_float(pack_h2(e2, e3));
            }
            l += (p4[0] + p4[1]) + (p4[2] + p4[3]);
            if (j > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
                // O may only be touched between two value products: the last one is done, the next waits for us
                ok = ok && mbar_wait(su32(&bars.pv_done[(j - 1) % NB]), (uint32_t)((j - 1) / NB) & 1u);
                fence_after();
#pragma unroll 1
                for (int c = 0; c < OCOLS; c += 32) {          // this thread's part of the output row
                    float o[32];
                    tmem_ld32_wait(lane_t + TM_O + OCOLS * part + c, o);
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] *= corr;
                    tmem_st32(lane_t + TM_O + OCOLS * part + c, o);
                }
            }
            // probabilities over the scores: key k of the tile in the low / high half of column k / 2
            st_cols(lane_t + TM_S + sb * BN + (COLS / 2) * part, pk);
            tmem_wait_st();
            fence_before();
            mbar_arrive(su32(&bars.p_full));
        }
        // row sum = the parts' sums (all were rescaled by the same factors)
        lx[part][row] = l;
        row_sync<NQ>(1 + wq);
#pragma unroll
        for (int p = 1; p < NQ; p++) l += lx[(part + p) % NQ][row];
        ok = ok && mbar_wait(su32(&bars.pv_done[(n_tiles - 1) % NB]), (uint32_t)((n_tiles - 1) / NB) & 1u);
        fence_after();
        const float inv = ok ? 1.0f / l : NAN;
        const size_t tok = (size_t)b * a.T + q0 + row;
        const ACT *gate = (a.gated && live) ? (const ACT *)a.qproj + tok * a.nh * HD * 2 + (size_t)h * HD * 2 + HD : nullptr;
        ACT *out = (ACT *)a.out + (tok * a.nh + h) * HD;
#pragma unroll 1
        for (int c = OCOLS * part; c < OCOLS * part + OCOLS; c += 32) {
            float o[32];
            tmem_ld32_wait(lane_t + TM_O + c, o);
            if (live) {
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    float y = o[i] * inv;
                    if (gate) y *= sigmoid_f(act_ld(gate, c + i));
                    act_st(out, c + i, y);
                }
            }
        }
    }
    if (!ok) report_timeout(a.status, ORN_WAIT_GQA_PREFILL);
    fence_before();
    __syncthreads();
    if (warp == W_PV) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TM_COLS) : "memory");
    }
}

// [rows][256] f16, boxes of 64 dims x box_rows rows, 128-byte swizzle
ornith_status f16_rows_map(CUtensorMap *m, const void *basep, uint64_t rows, uint32_t box_rows) {
    OrnTensorMapEncodeFn enc = orn_tensor_map_encoder();
    if (!enc) { orn_record_error("prefill: cuTensorMapEncodeTiled is not available"); return (ornith_status)ORNITH_ERR_BACKEND; }
    cuuint64_t dims[2] = {(cuuint64_t)HD, rows};
    cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t es[2] = {1, 1};
    const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(basep), dims, strides, box, es,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { orn_record_error("prefill: cuTensorMapEncodeTiled failed (%d)", (int)r); return (ornith_status)ORNITH_ERR_BACKEND; }
    return ORNITH_OK;
}

}  // namespace

size_t gqa_prefill_tc_scratch(int n_seq, int nh, int T) {
    return align_up((size_t)n_seq * nh * T * HD * sizeof(__half), 256) + align_up((size_t)n_seq * nh * T * sizeof(float), 256);
}

ornith_status launch_gqa_prefill_tc(const KvView &kv, const int32_t *kv_len, const float *q_prep, const __half *Kh,
                                    const __half *Vh, void *q_scratch, const void *qproj, void *out, int nh, int T,
                                    int Lmax, int Lp, int gated, float scale, int n_seq, bool bf16_act, cudaStream_t st) {
    __half *Qh = (__half *)q_scratch;
    float *rs = (float *)((char *)q_scratch + align_up((size_t)n_seq * nh * T * HD * sizeof(__half), 256));
    const size_t qrows = (size_t)n_seq * nh * T;
    if (q_prep) {                                          // otherwise the front end has written the image itself
        k_q_rows_to_f16<<<(unsigned)((qrows + 3) / 4), 128, 0, st>>>(q_prep, Qh, rs, n_seq, T, nh, scale);
        ORN_TRY(orn_check_launch("k_q_rows_to_f16"));
    }
    CUtensorMap mq, mk, mv;
    ORN_TRY(f16_rows_map(&mq, Qh, qrows, BM));
    ORN_TRY(f16_rows_map(&mk, Kh, (uint64_t)n_seq * kv.nkv * Lp, BN));
    ORN_TRY(f16_rows_map(&mv, Vh, (uint64_t)n_seq * kv.nkv * Lp, BN));
    TcArgs a;
    a.seq_off = kv.seq_off; a.kv_len = kv_len; a.Qh = Qh; a.rs = rs; a.qproj = qproj; a.out = out;
    a.nh = nh; a.nkv = kv.nkv; a.T = T; a.Lmax = Lmax; a.Lp = Lp; a.gated = gated;
    a.status = orn_status_word();
    static bool configured_dev[ORN_MAX_DEVICES] = {};
    bool &configured = configured_dev[orn_device_index()];
    if (!configured) {
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_gqa_prefill_tc<float, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               SM_BYTES + 1024), "tcgen05 prefill smem opt-in"));
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_gqa_prefill_tc<__nv_bfloat16, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               SM_BYTES + 1024), "tcgen05 prefill smem opt-in"));
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_gqa_prefill_tc<float, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               SM_BYTES + 1024), "tcgen05 prefill smem opt-in"));
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_gqa_prefill_tc<__nv_bfloat16, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               SM_BYTES + 1024), "tcgen05 prefill smem opt-in"));
        configured = true;
    }
    dim3 grid((T + BM - 1) / BM, nh, n_seq);
    // softmax threads per query row: 2 (default) or 4.  Measured at 32768 tokens x 32 heads: 19.1 ms with 2, 19.8 ms
    // with 4 (back to back under the power cap): the softmax is not what bounds the kernel.  Every CTA pulls a 64 KB
    // K + V tile pair from L2 per 128 query rows: 137 GB per layer, 7.2 TB/s over the 148 SMs, and that traffic is the bound.
    const char *e = getenv("ORNITH_CUDA_PREFILL_SOFTMAX");
    const int nq = (e && e[0] == '4') ? 4 : 2;
    if (nq == 4) {
        if (bf16_act) k_gqa_prefill_tc<__nv_bfloat16, 4><<<grid, (4 * 4 + 6) * 32, SM_BYTES + 1024, st>>>(mq, mk, mv, a);
        else          k_gqa_prefill_tc<float, 4><<<grid, (4 * 4 + 6) * 32, SM_BYTES + 1024, st>>>(mq, mk, mv, a);
    } else {
        if (bf16_act) k_gqa_prefill_tc<__nv_bfloat16, 2><<<grid, (4 * 2 + 6) * 32, SM_BYTES + 1024, st>>>(mq, mk, mv, a);
        else          k_gqa_prefill_tc<float, 2><<<grid, (4 * 2 + 6) * 32, SM_BYTES + 1024, st>>>(mq, mk, mv, a);
    }
    return orn_check_launch("k_gqa_prefill_tc");
}
