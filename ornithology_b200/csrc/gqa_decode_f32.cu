// gqa_decode_f32.cu — split-K GQA decode over f32 KV rows on the tensor cores (tf32),
// head_dim 256, groups of up to 16 query heads per KV head (two CTAs of 8 heads beyond 8).
//
// Replaces the attend half of ornith_gqa_step for the f32 cache (reference:
// src/ornith_attn.c:111-148).  An f32 row is 1 KiB; at 8 query heads per KV head the
// step needs 4 FMA per byte read, more than the CUDA cores can give at HBM speed, so
// both products run on mma.sync m16n8k8 tf32 with fp32 accumulation — straight from
// the f32 bytes, no conversion pass:
//   scores   S[head][token] = Q K^T   heads on M (rows 8..15 unused), 8 tokens on N,
//                                     32 k-steps of 8 dims; the K tile is the B operand
//   output   O^T[dim][head] += V^T P^T  16 m-tiles of 16 dims, heads on N, the tile's 8
//                                     tokens are the one k-step; the V tile is the A operand
// One CTA per (KV head, split, sequence), four warps, each walking every fourth 8-token
// tile of the split with its own K and V staging slot: one cp.async.bulk per row (1 KiB),
// completion on a per-warp mbarrier (bounded waits); K of the next tile is requested as
// soon as the score product is done with the slot, V right after the value product.
// Online softmax in the log2 domain; the four warps merge in shared memory and the CTA
// writes one partial (m, l, o) per head, the format k_gqa_combine reads.
//
// Precision: q, K, V and the probabilities enter the MMAs rounded to tf32 (11-bit
// significand, like the f16 operands of the Q8_0 kernels); sums are fp32.
#include "bulk_copy.cuh"
#include "full_attn.cuh"

namespace {

constexpr int HD = 256, TILE = 8, NWARP = 4;
constexpr int LDQ = 260, LDKT = 260, LDVT = 264;      // row strides in floats: 4 / 4 / 8 mod 32 -> conflict-free fragments
constexpr int QS_BYTES = 8 * LDQ * 4;                 // 8320
constexpr int KT_BYTES = TILE * LDKT * 4;             // 8320
constexpr int VT_BYTES = TILE * LDVT * 4;             // 8448
constexpr int WARP_BYTES = KT_BYTES + VT_BYTES;       // 16768
constexpr int SMEM_BYTES = QS_BYTES + NWARP * WARP_BYTES;   // 75392: three CTAs per SM
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;

__device__ __forceinline__ float tf32r(float x) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return __uint_as_float(u);
}
// the tensor core drops the 13 low mantissa bits: adding half a tf32 ulp first makes that a rounding
__device__ __forceinline__ float tf32q(float x) { return __uint_as_float(__float_as_uint(x) + 0x1000u); }
__device__ __forceinline__ void mma_tf32(float (&d)[4], float a0, float a1, float a2, float a3, float b0, float b1) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(__float_as_uint(a0)), "r"(__float_as_uint(a1)), "r"(__float_as_uint(a2)), "r"(__float_as_uint(a3)),
          "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)));
}

// rows tok0 .. of one KV head into a staging slot; rows past t1 are not copied (the slot keeps
// earlier, finite contents and those tokens are masked in the softmax)
__device__ __forceinline__ void issue_rows8(float *slot, int ld, uint32_t bar, const float *src_base, size_t row_stride,
                                            int tok0, int t1, int lane) {
    const int valid = min(TILE, t1 - tok0);
    if (lane == 0) bc_mbar_expect_tx(bar, (uint32_t)valid * 1024u);
    __syncwarp();
    if (lane < valid) bc_copy(bc_smem_u32(slot + lane * ld), src_base + (size_t)(tok0 + lane) * row_stride, 1024u, bar);
}

__global__ void __launch_bounds__(128, 3) k_gqa_decode_f32_tc(DecodeArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float m_s[NWARP][8], l_s[NWARP][8];
    __shared__ __align__(8) unsigned long long bars[NWARP][2];
    __shared__ int pipe_failed;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, j = lane & 3;
    float *Q_s = reinterpret_cast<float *>(smem);                        // [8 heads][LDQ] tf32
    float *Kt = reinterpret_cast<float *>(smem + QS_BYTES + warp * WARP_BYTES), *Vt = Kt + TILE * LDKT;
    if (tid == 0) pipe_failed = 0;

    // a group of more than 8 query heads is walked by two CTAs of 8 heads each; they sit side by side on
    // the fastest grid axis, so the second one finds the rows the first one fetched in L2
    const int nkv = a.kv.nkv, Gall = a.nh / nkv, sub = (Gall + 7) / 8;
    const int kvh = (int)blockIdx.x / sub, hs = (int)blockIdx.x % sub, split = blockIdx.y, b = blockIdx.z;
    const int G = min(8, Gall - 8 * hs), head0 = kvh * Gall + 8 * hs;
    const int64_t base = a.kv.seq_off[b];
    const int cap = (int)(a.kv.seq_off[b + 1] - base);
    const int len0 = a.kv_len[b];
    if (len0 >= cap) return;
    const int L = len0 + 1;
    const int t0 = split * a.tokens_per_split, t1 = min(L, t0 + a.tokens_per_split);
    float *part0 = a.part + (((size_t)b * a.nh + (size_t)head0) * a.nsplit + split) * (HD + 2);
    const size_t part_stride = (size_t)a.nsplit * (HD + 2);
    if (t0 >= L) {
        if (tid < G) { part0[tid * part_stride] = -INFINITY; part0[tid * part_stride + 1] = 0.0f; }
        return;
    }
    // ---- query group -> shared memory, tf32; rows of heads the group does not have are zero
    for (int e = tid; e < 8 * HD; e += 128) {
        const int h = e >> 8, d = e & 255;
        Q_s[h * LDQ + d] = (h < G) ? tf32r(a.q_prep[((size_t)b * a.nh + (size_t)head0 + h) * HD + d]) : 0.0f;
    }
    // staging slots: zero once (skipped tail rows must stay finite), one mbarrier per slot
    for (int i = lane; i < WARP_BYTES / 16; i += 32) reinterpret_cast<uint4 *>(Kt)[i] = make_uint4(0u, 0u, 0u, 0u);
    if (lane == 0) {
        bc_mbar_init(bc_smem_u32(&bars[warp][0]), 1);
        bc_mbar_init(bc_smem_u32(&bars[warp][1]), 1);
        bc_mbar_init_fence();
    }
    bc_fence_proxy_async();                                              // generic-proxy zeros before async-proxy copies
    __syncthreads();
    const uint32_t barK = bc_smem_u32(&bars[warp][0]), barV = bc_smem_u32(&bars[warp][1]);
    const float rs = a.scale * LOG2E;
    const int ntiles = (t1 - t0 + TILE - 1) / TILE;
    const size_t row_stride = (size_t)nkv * HD;                          // floats between the rows of consecutive tokens
    const float *Kbase = reinterpret_cast<const float *>(a.kv.K) + ((size_t)base * nkv + kvh) * HD;
    const float *Vbase = reinterpret_cast<const float *>(a.kv.V) + ((size_t)base * nkv + kvh) * HD;

    float o[16][4];                        // O^T: o[mt][0..1] = dim 16mt+g, heads 2j, 2j+1; o[mt][2..3] = dim 16mt+g+8
#pragma unroll
    for (int i = 0; i < 16; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m_run = -INFINITY, l_run = 0.0f;                               // of head g (the four lanes of a row agree)
    bool pipe_ok = true;

    int it = warp;
    if (it < ntiles) {
        issue_rows8(Kt, LDKT, barK, Kbase, row_stride, t0 + it * TILE, t1, lane);
        issue_rows8(Vt, LDVT, barV, Vbase, row_stride, t0 + it * TILE, t1, lane);
    }
    for (uint32_t n = 0; it < ntiles; it += NWARP, n++) {
        const int tok0 = t0 + it * TILE;
        const bool more = it + NWARP < ntiles;
        if (!bc_mbar_wait(barK, n & 1)) { (void)bc_mbar_wait(barV, n & 1); pipe_ok = false; break; }

        // ---- S = Q K^T: 32 k-steps of 8 dims in two accumulator chains ----------------------
        float s0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, s1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const float *qrow = Q_s + g * LDQ + j, *krow = Kt + g * LDKT + j;
#pragma unroll
        for (int ks = 0; ks < 32; ks += 2) {
            mma_tf32(s0, qrow[8 * ks], 0.0f, qrow[8 * ks + 4], 0.0f, tf32q(krow[8 * ks]), tf32q(krow[8 * ks + 4]));
            mma_tf32(s1, qrow[8 * ks + 8], 0.0f, qrow[8 * ks + 12], 0.0f, tf32q(krow[8 * ks + 8]), tf32q(krow[8 * ks + 12]));
        }
        __syncwarp();                                                    // every lane is done with the K slot
        if (more) issue_rows8(Kt, LDKT, barK, Kbase, row_stride, tok0 + NWARP * TILE, t1, lane);

        // ---- online softmax of head g over tokens 2j, 2j+1 (and the other lanes of the row) --
        float x0 = (tok0 + 2 * j < t1) ? (s0[0] + s1[0]) * rs : -INFINITY;
        float x1 = (tok0 + 2 * j + 1 < t1) ? (s0[1] + s1[1]) * rs : -INFINITY;
        float mx = fmaxf(x0, x1);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);                            // finite: token tok0 is valid
        const float corr = exp2f(m_run - m_new);
        m_run = m_new;
        x0 = exp2f(x0 - m_new); x1 = exp2f(x1 - m_new);
        float ps = x0 + x1;
        ps += __shfl_xor_sync(0xffffffffu, ps, 1);
        ps += __shfl_xor_sync(0xffffffffu, ps, 2);
        l_run = l_run * corr + ps;
        // the output columns of this lane are heads 2j and 2j+1
        const float cA = __shfl_sync(0xffffffffu, corr, (2 * j) * 4), cB = __shfl_sync(0xffffffffu, corr, (2 * j + 1) * 4);
        if (__any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll
            for (int i = 0; i < 16; i++) { o[i][0] *= cA; o[i][1] *= cB; o[i][2] *= cA; o[i][3] *= cB; }
        }
        // P^T as B operand: b0 = P[head g][token j], b1 = P[head g][token j + 4]
        const int src0 = g * 4 + (j >> 1), src1 = src0 + 2;
        const float v00 = __shfl_sync(0xffffffffu, x0, src0), v01 = __shfl_sync(0xffffffffu, x1, src0);
        const float v10 = __shfl_sync(0xffffffffu, x0, src1), v11 = __shfl_sync(0xffffffffu, x1, src1);
        const float pb0 = tf32q((j & 1) ? v01 : v00), pb1 = tf32q((j & 1) ? v11 : v10);

        // ---- O^T += V^T P^T: 16 m-tiles of 16 dims, one k-step of 8 tokens -------------------
        if (!bc_mbar_wait(barV, n & 1)) { if (more) (void)bc_mbar_wait(barK, (n + 1) & 1); pipe_ok = false; break; }
        const float *vlo = Vt + j * LDVT + g, *vhi = Vt + (j + 4) * LDVT + g;
#pragma unroll
        for (int mt = 0; mt < 16; mt++)
            mma_tf32(o[mt], tf32q(vlo[16 * mt]), tf32q(vlo[16 * mt + 8]), tf32q(vhi[16 * mt]), tf32q(vhi[16 * mt + 8]), pb0, pb1);
        __syncwarp();                                                    // every lane is done with the V slot
        if (more) issue_rows8(Vt, LDVT, barV, Vbase, row_stride, tok0 + NWARP * TILE, t1, lane);
    }
    if (!pipe_ok && lane == 0) pipe_failed = 1;
    __syncwarp();

    // ---- merge the four warps, one partial per (head, split) -----------------------------------
    float *Ow = Kt;                                                      // [8 heads][256] f32 over this warp's slots
#pragma unroll
    for (int mt = 0; mt < 16; mt++) {
        Ow[(2 * j) * HD + 16 * mt + g] = o[mt][0];
        Ow[(2 * j + 1) * HD + 16 * mt + g] = o[mt][1];
        Ow[(2 * j) * HD + 16 * mt + g + 8] = o[mt][2];
        Ow[(2 * j + 1) * HD + 16 * mt + g + 8] = o[mt][3];
    }
    if (j == 0) { m_s[warp][g] = m_run; l_s[warp][g] = l_run; }
    __syncthreads();
    for (int h = 0; h < G; h++) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NWARP; w++) if (l_s[w][h] > 0.0f) M = fmaxf(M, m_s[w][h]);
        float ww[NWARP], Lt = 0.0f;
#pragma unroll
        for (int w = 0; w < NWARP; w++) {
            ww[w] = (l_s[w][h] > 0.0f) ? exp2f(m_s[w][h] - M) : 0.0f;
            Lt += l_s[w][h] * ww[w];
        }
        float *part = part0 + h * part_stride;
        // a staging copy that never completed poisons the partial (the result becomes NaN, not silently wrong)
        const float poison = pipe_failed ? NAN : 0.0f;
        if (tid == 0) { part[0] = M * LN2; part[1] = pipe_failed ? 1.0f : Lt; }
        for (int d = tid; d < HD; d += 128) {
            float acc = 0.0f;
#pragma unroll
            for (int w = 0; w < NWARP; w++)
                acc += ww[w] * reinterpret_cast<const float *>(smem + QS_BYTES + w * WARP_BYTES)[h * HD + d];
            part[2 + d] = acc + poison;
        }
    }
}

}  // namespace

bool gqa_decode_f32_tc_supported(const KvView &kv, int nh) {
    return kv.mode == ORNITH_KV_F32 && kv.hd == HD && nh % kv.nkv == 0 && nh / kv.nkv <= 16 &&
           ((uintptr_t)kv.K % 16) == 0 && ((uintptr_t)kv.V % 16) == 0;
}

ornith_status launch_gqa_decode_f32_tc(const DecodeArgs &a, int n_seq, cudaStream_t st) {
    static bool configured_dev[ORN_MAX_DEVICES] = {};
    bool &configured = configured_dev[orn_device_index()];
    if (!configured) {
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_gqa_decode_f32_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES),
                          "f32 gqa decode smem opt-in"));
        configured = true;
    }
    dim3 grid(a.kv.nkv * ((a.nh / a.kv.nkv + 7) / 8), a.nsplit, n_seq);
    k_gqa_decode_f32_tc<<<grid, 128, SMEM_BYTES, st>>>(a);
    return orn_check_launch("k_gqa_decode_f32_tc");
}
