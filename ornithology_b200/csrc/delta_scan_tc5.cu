// delta_scan_tc5.cu — gated delta-net prefill scan for dk = dv = 128 on the 5th-generation
// tensor cores: operands staged by TMA, tcgen05.mma (tf32) with the recurrent state and every
// intermediate of the chunk in tensor memory.
//
// Reference behaviour being replaced: the chunked scan of ornith_delta_prefill
// (src/ornith_attn.c:215-349) inside linear_attn_prefill (src/ornith_rforward.c:563-618), with
// linear_finish (src/ornith_rforward.c:300-314) as the epilogue.
//
// Per chunk of 64 tokens with incoming state S [dv][dk], raw (conv + SiLU) rows k_i, q_i with
// inverse norms rk_i, rq_i, G_i the running sum of the log-decay inside the chunk, p_i = exp(G_i),
// Gamma_ij = exp(G_i - G_j), w_j = Gamma_63,j:
//   M = diag(beta) strictLower(Gamma o Khat Khat^T),  A = (I + M)^-1,  P = lower(Gamma o Qhat Khat^T)
//   T = diag(beta) V - diag(beta p rk) (K S^T)
//   U = A T
//   O = diag(p rq) (Q S^T) + P U
//   S <- p_63 S + sum_j (w_j rk_j u_j) k_j^T
// (Khat, Qhat the normalised rows; the norms are folded into the per-token factors so that the
// tensor cores read the K / Q tiles straight from the conv output.)  A, P and the per-token
// factors do not depend on the state: k_delta_prep64 produces them for all chunks at once.
//
// k_delta_scan_tc5, one CTA per (value head, sequence), keeps everything transposed, dv on the
// 128 tensor-memory lanes:
//   KS^T | QS^T = S [K ; Q]^T     M128 N128 K128   A operand = the state itself (tensor memory)
//   U^T  = T^T A^T                M128 N64  K64    A operand = T^T (tensor memory)
//   (PU)^T = U^T P^T              M128 N64  K64    A operand = U^T
//   S   += (w rk U)^T K           M128 N128 K64    accumulator = the state; B = the K tile, MN-major
// so the fp32 state never leaves tensor memory during a prompt: it is the accumulator of the
// update and, read as tf32 (low mantissa bits ignored), the A operand of the next chunk.
//   warp 16    one lane issues the TMA loads: the K | Q tile (64 KiB, two buffers), a second copy of the K rows
//              for the state update (an MN-major tf32 operand must lie in 32-byte swizzle atoms, a K-major one in
//              16-byte atoms, so one image cannot serve both), A and P (lower triangles only), the V rows, factors
//   warp 17    one lane issues the tcgen05.mma of the dependency chain (KS | QS, U, state update)
//   warp 18    one lane issues (P U)^T, which nothing on the chain waits for
//   warps 0-7  chain epilogues, two threads per lane (32 tokens each): T from KS and V, the decay sweep of S
//              (while U^T is computed), U -> tf32 U and w rk U
//   warps 8-15 output epilogue, off the dependency chain: O, per-token RMSNorm over the head (transpose-reduce
//              by shuffles), SiLU(z) gate, store; z is requested one chunk ahead
// All warps keep the 96 registers of the launch (no setmaxnreg: the issuing warps run three different roles, and
// that instruction must be executed identically by all four warps of a warpgroup).
// Every wait is bounded in time; a wait that gives up is reported through the device status word and poisons
// the outputs.
#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>

#include <mutex>

#include "linear_attn.cuh"
#include "tcgen05.cuh"

namespace {
using namespace tc5;

constexpr int C = 64;                                   // tokens per chunk
constexpr float LOG2E_F = 1.4426950408889634f;
constexpr int AUX_FLOATS = 5 * C;                       // beta | beta p rk | w rk | p rq | p_63 (first word)
constexpr uint32_t AUX_BYTES = AUX_FLOATS * 4;
// A and P are lower triangular.  Stored per block as four dense pieces of 32 columns: A columns 0..31 (64 rows),
// A columns 32..63 of rows 32..63 (32 rows), then the same for P: 192 rows of 32 floats.
constexpr int AP_ROWS = 192, AP_A1 = 64, AP_P0 = 96, AP_P1 = 160;
constexpr int AP_FLOATS = AP_ROWS * 32;
constexpr uint32_t AP_BYTES = AP_FLOATS * 4;

// Round to tf32 (nearest, ties away from zero; finite inputs) with integer arithmetic: cvt.rna.tf32.f32 runs at
// the special-function rate, a sixteenth of this.  tf32r gives a clean tf32 value (low 13 mantissa bits zero) for
// operands that are stored; tf32q only adds the half ulp, for operands that go straight to the tensor core, which
// ignores the low bits.
__device__ __forceinline__ float tf32r(float x) { return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u); }
__device__ __forceinline__ float tf32q(float x) { return __uint_as_float(__float_as_uint(x) + 0x1000u); }

// =============================================================================
// state-independent part: one CTA per (chunk, key head, sequence), 256 threads
// =============================================================================
constexpr int LDK = 132;                                // K / Q rows: stride = 4 mod 32 keeps MMA fragments conflict-free
constexpr int LDG = 65;
constexpr int LDB = 36;                                 // 32x32 blocks, rows 16-byte aligned

struct PairSmem {                                       // one value head in flight per pair of warps
    float M11[32 * LDB], M21[32 * LDB], M22[32 * LDB];  // blocks of M = beta_i Gamma_il khat_i.khat_l (l < i)
    float A22[32 * LDB];
    float g[C], be[C];
};
struct PrepSmem {
    union {
        struct { float Ks[C * LDK], Qs[C * LDK]; } t;   // dead once the Gram matrices exist
        PairSmem pair[4];
    } u;
    float GK[C * LDG], GQ[C * LDG];                     // khat_i.khat_l, qhat_i.khat_l for l <= i
    float rk[C], rq[C];
};

__device__ __forceinline__ void mma_tf32_sync(float (&d)[4], const float (&a)[4], float b0, float b1) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(__float_as_uint(a[0])), "r"(__float_as_uint(a[1])), "r"(__float_as_uint(a[2])),
          "r"(__float_as_uint(a[3])), "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)));
}
__device__ __forceinline__ void pair_sync(int id) { asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory"); }

// (I + L)^-1 of a 32x32 strictly lower block by forward substitution; lane = column.  Four partial sums per
// row: the rows form one dependent chain, and a single accumulator would make it 496 multiply-adds long.
__device__ __forceinline__ void inv_unit_lower(const float *Mb, int lane, float (&x)[32]) {
#pragma unroll
    for (int i = 0; i < 32; i++) {
        float a0 = (i == lane) ? 1.0f : 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll
        for (int l4 = 0; l4 < (i + 3) / 4; l4++) {
            const float4 m = *reinterpret_cast<const float4 *>(Mb + i * LDB + 4 * l4);
            if (4 * l4 + 0 < i) a0 -= m.x * x[4 * l4 + 0];
            if (4 * l4 + 1 < i) a1 -= m.y * x[4 * l4 + 1];
            if (4 * l4 + 2 < i) a2 -= m.z * x[4 * l4 + 2];
            if (4 * l4 + 3 < i) a3 -= m.w * x[4 * l4 + 3];
        }
        x[i] = (a0 + a1) + (a2 + a3);
    }
}
// y[i] = sum_l B[row0 + i][l] x[l] for 16 rows of a 32x32 block in shared memory, x in registers
__device__ __forceinline__ void block_matvec16(const float *B, int row0, const float (&x)[32], float (&y)[16]) {
#pragma unroll
    for (int i = 0; i < 16; i++) {
        float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
        for (int l4 = 0; l4 < 8; l4++) {
            const float4 m = *reinterpret_cast<const float4 *>(B + (row0 + i) * LDB + 4 * l4);
            a0 = fmaf(m.x, x[4 * l4], a0); a1 = fmaf(m.y, x[4 * l4 + 1], a1);
            a0 = fmaf(m.z, x[4 * l4 + 2], a0); a1 = fmaf(m.w, x[4 * l4 + 3], a1);
        }
        y[i] = a0 + a1;
    }
}

template <typename ACT>
__global__ void __launch_bounds__(256, 2) k_delta_prep64(LinArgs a, const float *Y, const float *rqg, const float *rkg,
                                                      const float *la, const float *be, float *AP, float *aux,
                                                      int n_chunks, int chunk0) {
    extern __shared__ __align__(16) unsigned char smraw[];
    PrepSmem &sm = *reinterpret_cast<PrepSmem *>(smraw);
    const int chunk = chunk0 + blockIdx.x, kh = blockIdx.y, b = blockIdx.z, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int g = lane >> 2, j = lane & 3;
    const int qd = a.nk * 128, Cc = 2 * qd + a.nv * 128;
    const int t0 = chunk * C, n = min(C, a.T - t0);
    const size_t tok0 = (size_t)b * a.T + t0;

    for (int e = tid; e < C * 32; e += 256) {             // raw rows (tf32 values); rows past the end are zero
        const int i = e >> 5, c = (e & 31) * 4;
        float4 q = make_float4(0.f, 0.f, 0.f, 0.f), k = q;
        if (i < n) {
            const float *y = Y + (tok0 + i) * Cc + kh * 128 + c;
            q = *reinterpret_cast<const float4 *>(y);
            k = *reinterpret_cast<const float4 *>(y + qd);
        }
        *reinterpret_cast<float4 *>(&sm.u.t.Qs[i * LDK + c]) = q;
        *reinterpret_cast<float4 *>(&sm.u.t.Ks[i * LDK + c]) = k;
    }
    if (tid < C) {
        sm.rk[tid] = tid < n ? rkg[(tok0 + tid) * a.nk + kh] : 0.0f;
        sm.rq[tid] = tid < n ? rqg[(tok0 + tid) * a.nk + kh] : 0.0f;
    }
    __syncthreads();
    {   // Gram tiles on or below the diagonal: warps 0-3 K K^T, warps 4-7 Q K^T; 16 rows each
        const int which = w >> 2, mt = w & 3, ntn = 2 * mt + 2;
        float acc[8][4];
#pragma unroll
        for (int t = 0; t < 8; t++)
#pragma unroll
            for (int x = 0; x < 4; x++) acc[t][x] = 0.0f;
        const float *Am = (which ? sm.u.t.Qs : sm.u.t.Ks) + 16 * mt * LDK;
#pragma unroll 2
        for (int k0 = 0; k0 < 128; k0 += 8) {
            float af[4];
            af[0] = Am[g * LDK + k0 + j];
            af[1] = Am[(g + 8) * LDK + k0 + j];
            af[2] = Am[g * LDK + k0 + j + 4];
            af[3] = Am[(g + 8) * LDK + k0 + j + 4];
#pragma unroll
            for (int t = 0; t < 8; t++) {
                if (t < ntn) {
                    const float *kr = sm.u.t.Ks + (8 * t + g) * LDK + k0 + j;
                    mma_tf32_sync(acc[t], af, kr[0], kr[4]);
                }
            }
        }
        float *G = which ? sm.GQ : sm.GK;
        const float *rrow = which ? sm.rq : sm.rk;
#pragma unroll
        for (int t = 0; t < 8; t++)
            if (t < ntn) {
#pragma unroll
                for (int x = 0; x < 4; x++) {
                    const int i = 16 * mt + g + 8 * (x >> 1), l = 8 * t + 2 * j + (x & 1);
                    G[i * LDG + l] = acc[t][x] * rrow[i] * sm.rk[l];
                }
            }
    }
    __syncthreads();                                      // the tiles are dead: the pair buffers alias them
    const int nvk = a.nv / a.nk, pr = w >> 1, wl = w & 1, pt = tid & 63;
    PairSmem &ps = sm.u.pair[pr];
    for (int m = pr; m < nvk; m += 4) {                   // one pair of warps per value head of this key head
        const int hv = a.head_map == ORNITH_HEADMAP_GROUPED ? kh * nvk + m : kh + m * a.nk;
        const size_t blk = ((size_t)b * a.nv + hv) * n_chunks + chunk;
        float *Ag = AP + blk * AP_FLOATS, *ax = aux + blk * AUX_FLOATS;
        float gg = 0.0f, bb = 0.0f;                       // thread pt = token pt: log-decay and write gate
        if (pt < n) {
            if (la) { gg = la[(tok0 + pt) * a.nv + hv]; bb = be[(tok0 + pt) * a.nv + hv]; }
            else {                                        // reference: decay_alpha, src/ornith_rforward.c:282-284
                gg = a.a_coef[hv] * softplus_f(act_ld((const ACT *)a.a, (tok0 + pt) * a.nv + hv) + a.dt_bias[hv]);
                bb = sigmoid_f(act_ld((const ACT *)a.b, (tok0 + pt) * a.nv + hv));
            }
        }
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, gg, o);
            if (lane >= o) gg += up;
        }
        if (wl == 0) ps.g[pt] = gg;
        ps.be[pt] = bb;
        pair_sync(1 + pr);
        if (wl == 1) { gg += ps.g[31]; ps.g[pt] = gg; }
        pair_sync(1 + pr);
        const float gend = ps.g[C - 1], pp = expf(gg);
        ax[pt] = bb;
        ax[C + pt] = bb * pp * sm.rk[pt];
        ax[2 * C + pt] = expf(gend - gg) * sm.rk[pt];
        ax[3 * C + pt] = pp * sm.rq[pt];
        ax[4 * C + pt] = expf(gend);
        // thread pt = column l of M and P; rows 0..31 concern the first warp of the pair only (columns 32.. are zero there)
        if (wl == 0) {
#pragma unroll 8
            for (int i = 0; i < 32; i++) {
                const float gam = (pt <= i) ? ex2_fast((ps.g[i] - gg) * LOG2E_F) : 0.0f;
                ps.M11[i * LDB + pt] = (pt < i) ? ps.be[i] * gam * sm.GK[i * LDG + pt] : 0.0f;
                Ag[(AP_P0 + i) * 32 + pt] = (pt <= i) ? tf32r(gam * sm.GQ[i * LDG + pt]) : 0.0f;
            }
#pragma unroll 8
            for (int i = 32; i < C; i++) {                // pt < 32 <= i: below the diagonal throughout
                const float gam = ex2_fast((ps.g[i] - gg) * LOG2E_F);
                ps.M21[(i - 32) * LDB + pt] = ps.be[i] * gam * sm.GK[i * LDG + pt];
                Ag[(AP_P0 + i) * 32 + pt] = tf32r(gam * sm.GQ[i * LDG + pt]);
            }
        } else {
#pragma unroll 8
            for (int i = 32; i < C; i++) {
                const float gam = (pt <= i) ? ex2_fast((ps.g[i] - gg) * LOG2E_F) : 0.0f;
                ps.M22[(i - 32) * LDB + pt - 32] = (pt < i) ? ps.be[i] * gam * sm.GK[i * LDG + pt] : 0.0f;
                Ag[(AP_P1 + i - 32) * 32 + pt - 32] = (pt <= i) ? tf32r(gam * sm.GQ[i * LDG + pt]) : 0.0f;
            }
        }
        pair_sync(1 + pr);
        // A = (I + M)^-1 = [[A11, 0], [-A22 M21 A11, A22]]; lane = column.  The two diagonal blocks are inverted by one
        // warp each; the two products of the off-diagonal block are split by rows between the warps.
        float x[32];
        if (wl == 0) {
            inv_unit_lower(ps.M11, lane, x);
#pragma unroll
            for (int i = 0; i < 32; i++) { Ag[i * 32 + lane] = tf32r(x[i]); ps.M11[i * LDB + lane] = x[i]; }   // A11 over M11
        } else {
            inv_unit_lower(ps.M22, lane, x);
#pragma unroll
            for (int i = 0; i < 32; i++) { Ag[(AP_A1 + i) * 32 + lane] = tf32r(x[i]); ps.A22[i * LDB + lane] = x[i]; }
        }
        pair_sync(1 + pr);
        {
            float y[16];
#pragma unroll
            for (int l = 0; l < 32; l++) x[l] = ps.M11[l * LDB + lane];          // column `lane` of A11
            block_matvec16(ps.M21, 16 * wl, x, y);                               // rows 16 wl .. of M21 A11
            pair_sync(1 + pr);                                                   // M22 has been read for the last time
#pragma unroll
            for (int i = 0; i < 16; i++) ps.M22[(16 * wl + i) * LDB + lane] = y[i];   // B = M21 A11 over M22
            pair_sync(1 + pr);
#pragma unroll
            for (int l = 0; l < 32; l++) x[l] = ps.M22[l * LDB + lane];          // column `lane` of B
            block_matvec16(ps.A22, 16 * wl, x, y);
#pragma unroll
            for (int i = 0; i < 16; i++) Ag[(32 + 16 * wl + i) * 32 + lane] = tf32r(-y[i]);
        }
        pair_sync(1 + pr);                                // the pair buffers are reused by the next head
    }
}

// =============================================================================
// sequential part: one CTA per (value head, sequence), 18 warps
// =============================================================================
constexpr int W_TMA = 24, W_MMA = 25, W_PU = 26, NTHREADS = 27 * 32;
constexpr int TM_S = 0, TM_KQ = 128, TM_TU = 384, TM_U = 448, TM_COLS = 512;   // tensor-memory columns
// Shared memory.  The K | Q tile is needed first in a chunk and is double-buffered; the operands of the
// later products (second K copy for the state update, A, P) have one buffer each, refilled as soon as
// the product that reads them is complete, which is most of a chunk period before their next use.
constexpr int SM_KQ = 0;                 // 2 x [4 slabs of 32 dims x (64 K rows, then 64 Q rows) x 128 bytes]
constexpr int SM_KM = 131072;            // the K tile again, laid out for the state update (see below)
// A and P are lower triangular: of their second slab (columns 32..63) only rows 32..63 exist, and the
// products that read it are issued for those 32 rows only
constexpr int SM_A = 163840;             // slab 0: 64 rows x 32 columns (8 KiB); slab 1: rows 32..63 (4 KiB)
constexpr int SM_P = 176128;
constexpr int SM_V = 188416;             // [64 tokens][128] f32 rows of V, not swizzled
constexpr int SM_AUX = 221184;           // 2 x per-token factors for the chain epilogues
constexpr int SM_AUX2 = SM_AUX + 2 * (int)AUX_BYTES;   // one more copy for the output epilogue (freed later)
constexpr int SCAN_SMEM = SM_AUX2 + (int)AUX_BYTES + 1024;   // + alignment slack
constexpr uint32_t TX_KQ = 65536 + AUX_BYTES, TX_KM = 32768, TX_A = 12288, TX_P = 12288 + AUX_BYTES, TX_V = 32768;

struct ScanBars {
    unsigned long long full_kq[2], empty_kq[2], kq_done[2], pu_done[2], o_read[2], red[2][4];
    unsigned long long full_km, empty_km, full_a, empty_a, full_p, empty_p, full_v, empty_v, t_ready, u_done, u_ready, s_final;
};

struct ScanArgs {
    const float *Y, *aux;
    float *S;
    long long S_stride;
    const void *z;
    void *out;
    const float *norm_w;
    int nk, nv, head_map, T, n_chunks;
    int c_begin, c_count;                // the chunks one launch of the sequential form scans (a slab of the prompt)
    float out_scale, eps;
    // Segment-parallel form (n_seg > 1; for few heads): the prompt is cut into n_seg runs of seg_chunks chunks that
    // are scanned at the same time by different CTAs (grid.z = 2 n_seg - 1).  The state enters the recurrence
    // linearly, S_t = S_{t-1} M_t + beta_t v_t k_t^T with M_t = alpha_t (I - beta_t k_t k_t^T) acting on the key
    // index, so a run needs the incoming state only through two things that do not depend on it: the scan of
    // the run from a ZERO state (outputs o0_t, final state S0) and the scan of the run from the IDENTITY with
    // V = 0 (outputs qt_t = Phi_t q_t, final state Phi = prod M_t).  Then o_t = o0_t + S_in qt_t and
    // S_out = S_in Phi + S0; k_delta_seg_carry walks the runs, k_delta_seg_finish adds the correction and
    // applies the output norm and gate.  Run 0 starts from the real state and is final as it is.
    int n_seg, seg_chunks;
    float *seg_state;                    // [n_seq * nv][3 n_seg][128][128]: slot 3j: S0 (j = 0: end state of run 0), 3j+1: Phi, 3j+2: S_in
    float *seg_raw;                      // [2][n_seq * nv][T][128] f32: o0, then qt
    unsigned int *status;
    long long *trace;                    // bring-up aid: clock64 stamps of CTA (0, 0), [role][chunk][8]
    float *dbg;                          // bring-up aid: first chunk's KS, U, QS, PU and the state after it (nullptr in production)
};
constexpr int DBG_FLOATS = 4 * 128 * 64 + 128 * 128;

// MN-major tf32 operand: rows of 128 bytes along N, groups of 4 k, 32-byte swizzle atoms
// (the only shared-memory layout the tensor core accepts for a transposed 32-bit operand)
__device__ __forceinline__ uint64_t smem_desc_mn32(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((lbo >> 4) & 0x3FFF) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3FFF) << 32) | ((uint64_t)1 << 46) | ((uint64_t)1 << 61);
}

__device__ __forceinline__ void ld_row32(const float *p, float (&r)[32]) {
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float4 v = *reinterpret_cast<const float4 *>(p + 4 * i);
        r[4 * i] = v.x; r[4 * i + 1] = v.y; r[4 * i + 2] = v.z; r[4 * i + 3] = v.w;
    }
}

// activation loads whose conversion happens at the point of use (a converted copy made at load time would
// double the registers a batch of loads in flight occupies)
__device__ __forceinline__ uint32_t ld_raw(const float *p, size_t i) { return __float_as_uint(p[i]); }
__device__ __forceinline__ uint32_t ld_raw(const __nv_bfloat16 *p, size_t i) { return reinterpret_cast<const unsigned short *>(p)[i]; }
__device__ __forceinline__ float cvt_raw(const float *, uint32_t r) { return __uint_as_float(r); }
__device__ __forceinline__ float cvt_raw(const __nv_bfloat16 *, uint32_t r) { return __uint_as_float(r << 16); }

// D[dv][i] = sum_j X[dv][j] L[i][j] with L lower triangular (X in tensor memory at column x, L in shared memory
// at l): j < 32 feeds all 64 rows i of L, j >= 32 only rows 32..63
__device__ __forceinline__ void issue_tri(uint32_t d, uint32_t x, uint32_t l) {
    constexpr uint32_t ID_64 = idesc(2, 64, false), ID_32 = idesc(2, 32, false);
#pragma unroll
    for (int ks = 0; ks < 4; ks++) mma_tf32_ts(d, x + 8 * ks, smem_desc(l + ks * 32, 16, 1024), ID_64, ks > 0);
#pragma unroll
    for (int ks = 0; ks < 4; ks++) mma_tf32_ts(d + 32, x + 32 + 8 * ks, smem_desc(l + 8192 + ks * 32, 16, 1024), ID_32, 1u);
}

template <typename ACT, bool SEG>
__global__ void __launch_bounds__(NTHREADS, 1) k_delta_scan_tc5(const __grid_constant__ CUtensorMap map_y,
                                                               const __grid_constant__ CUtensorMap map_ym,
                                                               const __grid_constant__ CUtensorMap map_ap,
                                                               const __grid_constant__ CUtensorMap map_ap32,
                                                               const __grid_constant__ CUtensorMap map_v, ScanArgs a) {
    extern __shared__ unsigned char smraw[];
    __shared__ ScanBars bars;
    __shared__ float red[2][4][4][16];                    // [chunk parity][group of 16 tokens][lane quarter][token]
    __shared__ uint32_t tmem_slot;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int hv = blockIdx.x, b = blockIdx.y;
    // what this CTA scans: kind 0 = from the caller's state, final outputs; 1 = from zero, raw outputs;
    // 2 = from the identity with V = 0, raw outputs
    int kind = 0, seg = 0;
    if (SEG && blockIdx.z > 0) { seg = 1 + ((int)blockIdx.z - 1) / 2; kind = 1 + ((int)blockIdx.z - 1) % 2; }
    const int c0 = SEG ? seg * a.seg_chunks : a.c_begin;                       // first chunk
    const int N = SEG ? min(a.seg_chunks, a.n_chunks - c0) : a.c_count;        // chunks of this CTA
    const int kh = a.head_map == ORNITH_HEADMAP_GROUPED ? hv / (a.nv / a.nk) : hv % a.nk;
    const int qd = a.nk * 128, vd = a.nv * 128;
    const uint32_t base = (su32(smraw) + 1023u) & ~1023u; // swizzle atoms are 1 KiB aligned
    unsigned char *gbase = smraw + (base - su32(smraw));

    if (tid == 0) {
        for (int s = 0; s < 2; s++) {
            mbar_init(su32(&bars.full_kq[s]), 1); mbar_init(su32(&bars.empty_kq[s]), 9);
            mbar_init(su32(&bars.kq_done[s]), 1); mbar_init(su32(&bars.pu_done[s]), 1);
            mbar_init(su32(&bars.o_read[s]), 512);
            for (int g = 0; g < 4; g++) mbar_init(su32(&bars.red[s][g]), 128);
        }
        mbar_init(su32(&bars.full_km), 1); mbar_init(su32(&bars.empty_km), 1);
        mbar_init(su32(&bars.full_a), 1); mbar_init(su32(&bars.empty_a), 1);
        mbar_init(su32(&bars.full_p), 1); mbar_init(su32(&bars.empty_p), 17);
        mbar_init(su32(&bars.full_v), 1); mbar_init(su32(&bars.empty_v), 8);
        mbar_init(su32(&bars.t_ready), 256); mbar_init(su32(&bars.u_done), 1);
        mbar_init(su32(&bars.u_ready), 256); mbar_init(su32(&bars.s_final), 1);
        mbar_init_fence();
    }
    if (warp == W_MMA) tmem_alloc(&tmem_slot, TM_COLS);
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = tmem_slot;
    float *Sg = a.S + (size_t)b * a.S_stride + (size_t)hv * 128 * 128;     // incoming state (kind 0)
    float *Sout = Sg;                                                       // where the final state goes
    float *raw = nullptr;                                                   // raw output rows [T][128] (kinds 1, 2)
    if (SEG) {
        Sout = a.seg_state + (((size_t)b * a.nv + hv) * 3 * a.n_seg + 3 * seg + (kind == 2 ? 1 : 0)) * (128 * 128);
        if (kind) raw = a.seg_raw + ((size_t)(kind - 1) * gridDim.y * a.nv + (size_t)b * a.nv + hv) * (size_t)a.T * 128;
    }
    // lane quarter and token (column) half of an epilogue thread
    const int qtr = warp & 3, half = (warp >> 2) & 1, row = 32 * qtr + lane;
    const uint32_t lane_t = tmem + ((uint32_t)(32 * qtr) << 16);
#ifdef ORNITH_SCAN_TRACE
    float *dbg = a.dbg ? a.dbg + (size_t)(b * a.nv + hv) * DBG_FLOATS : nullptr;
#else
    constexpr float *dbg = nullptr;
#endif
    long long *trace = (a.trace && hv == 0 && b == 0) ? a.trace : nullptr;
#ifdef ORNITH_SCAN_TRACE
#define TR(role, n, pt) do { if (trace && (n) < 64) trace[((role) * 64 + (n)) * 8 + (pt)] = clock64(); } while (0)
#else
#define TR(role, n, pt) do { (void)trace; } while (0)
#endif

    if (warp < 8) {                                       // the state goes to tensor memory: S[r][c] in lane r, column c
#pragma unroll 1
        for (int cc = 0; cc < 2; cc++) {
            float s[32];
            if (kind == 0) ld_row32(Sg + (size_t)row * 128 + 64 * half + 32 * cc, s);
            else {
#pragma unroll
                for (int i = 0; i < 32; i++) s[i] = (SEG && kind == 2 && 64 * half + 32 * cc + i == row) ? 1.0f : 0.0f;
            }
            tmem_st32(lane_t + TM_S + 64 * half + 32 * cc, s);
        }
        tmem_wait_st();
    }
    fence_before();
    __syncthreads();
    bool ok = true;

    if (warp == W_TMA) {
        // ================= producer =================
        if (lane == 0) {
            const int yrow0 = b * a.T + c0 * C;                       // first row of this CTA's first chunk
            const size_t blk0 = ((size_t)b * a.nv + hv) * a.n_chunks + c0;
            auto load_kq = [&](int n) {
                const int s = n & 1;
                if (n >= 2 && !mbar_wait(su32(&bars.empty_kq[s]), (uint32_t)((n >> 1) - 1) & 1u)) return false;
                const uint32_t dst = base + SM_KQ + s * 65536, bar = su32(&bars.full_kq[s]);
                mbar_expect_tx(bar, TX_KQ);
                for (int sl = 0; sl < 4; sl++) {
                    tma_load_2d(dst + sl * 16384, &map_y, qd + kh * 128 + 32 * sl, yrow0 + n * C, bar);        // K rows
                    tma_load_2d(dst + sl * 16384 + 8192, &map_y, kh * 128 + 32 * sl, yrow0 + n * C, bar);      // Q rows
                }
                bulk_load(base + SM_AUX + s * AUX_BYTES, a.aux + (blk0 + n) * AUX_FLOATS, AUX_BYTES, bar);
                return true;
            };
            auto load_a = [&](int n) {
                if (n >= 1 && !mbar_wait(su32(&bars.empty_a), (uint32_t)(n - 1) & 1u)) return false;
                mbar_expect_tx(su32(&bars.full_a), TX_A);
                tma_load_2d(base + SM_A, &map_ap, 0, (int)((blk0 + n) * AP_ROWS), su32(&bars.full_a));
                tma_load_2d(base + SM_A + 8192, &map_ap32, 0, (int)((blk0 + n) * AP_ROWS) + AP_A1, su32(&bars.full_a));
                return true;
            };
            auto load_v = [&](int n) {
                if (n >= 1 && !mbar_wait(su32(&bars.empty_v), (uint32_t)(n - 1) & 1u)) return false;
                mbar_expect_tx(su32(&bars.full_v), TX_V);
                tma_load_2d(base + SM_V, &map_v, 2 * qd + hv * 128, yrow0 + n * C, su32(&bars.full_v));
                return true;
            };
            auto load_km = [&](int n) {
                if (n >= 1 && !mbar_wait(su32(&bars.empty_km), (uint32_t)(n - 1) & 1u)) return false;
                mbar_expect_tx(su32(&bars.full_km), TX_KM);
                for (int sl = 0; sl < 4; sl++)              // [64 tokens][128 dims]: 4 slabs of 32 dims, 32-byte swizzle atoms
                    tma_load_2d(base + SM_KM + sl * 8192, &map_ym, qd + kh * 128 + 32 * sl, yrow0 + n * C, su32(&bars.full_km));
                return true;
            };
            auto load_p = [&](int n) {
                if (n >= 1 && !mbar_wait(su32(&bars.empty_p), (uint32_t)(n - 1) & 1u)) return false;
                mbar_expect_tx(su32(&bars.full_p), TX_P);
                tma_load_2d(base + SM_P, &map_ap, 0, (int)((blk0 + n) * AP_ROWS) + AP_P0, su32(&bars.full_p));
                tma_load_2d(base + SM_P + 8192, &map_ap32, 0, (int)((blk0 + n) * AP_ROWS) + AP_P1, su32(&bars.full_p));
                bulk_load(base + SM_AUX2, a.aux + (blk0 + n) * AUX_FLOATS, AUX_BYTES, su32(&bars.full_p));
                return true;
            };
            // issue order = the order in which the buffers come free in the steady state
            ok = load_kq(0) && load_v(0) && load_a(0) && load_km(0);
            if (ok && N > 1) ok = load_kq(1);
            for (int m = 0; m < N && ok; m++) {
                TR(3, m, 0);
                if (m + 1 < N) ok = load_v(m + 1);
                if (ok) ok = load_p(m);
                TR(3, m, 1);
                if (ok && m + 1 < N) ok = load_a(m + 1);
                TR(3, m, 2);
                if (ok && m + 2 < N) ok = load_kq(m + 2);
                TR(3, m, 3);
                if (ok && m + 1 < N) ok = load_km(m + 1);
                TR(3, m, 4);
            }
        }
    } else if (warp == W_MMA) {
        // ================= every tcgen05.mma =================
        if (lane == 0) {
            constexpr uint32_t ID_KQ = idesc(2, 128, false), ID_SU = idesc(2, 128, true);
            fence_after();
            for (int n = 0; n < N; n++) {
                const int s = n & 1;
                const uint32_t kqs = base + SM_KQ + s * 65536, kq = tmem + TM_KQ + 128 * s;
                ok = mbar_wait(su32(&bars.full_kq[s]), (uint32_t)(n >> 1) & 1u);
                // this KS | QS buffer holds the output tiles of chunk n-2 until the output epilogue has read them
                if (ok && n >= 2) ok = mbar_wait(su32(&bars.o_read[s]), (uint32_t)((n >> 1) - 1) & 1u);
                if (!ok) break;
                TR(0, n, 0);
                fence_after();
#pragma unroll
                for (int ks = 0; ks < 16; ks++)           // KS^T | QS^T = S [K ; Q]^T
                    mma_tf32_ts(kq, tmem + TM_S + 8 * ks, smem_desc(kqs + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024), ID_KQ, ks > 0);
                mma_commit(su32(&bars.kq_done[s]));
                mma_commit(su32(&bars.empty_kq[s]));
                TR(0, n, 1);
                // U^T of this chunk overwrites the U^T that (P U)^T of the previous chunk reads (issued by warp 18)
                if (n >= 1) ok = mbar_wait(su32(&bars.pu_done[s ^ 1]), (uint32_t)((n - 1) >> 1) & 1u);
                if (!ok) break;
                TR(0, n, 3);
                ok = mbar_wait(su32(&bars.full_a), (uint32_t)n & 1u) && mbar_wait(su32(&bars.t_ready), (uint32_t)n & 1u);
                if (!ok) break;
                TR(0, n, 4);
                fence_after();
                issue_tri(tmem + TM_U, tmem + TM_TU, base + SM_A);   // U^T = T^T A^T
                mma_commit(su32(&bars.u_done));
                mma_commit(su32(&bars.empty_a));
                TR(0, n, 5);
                ok = mbar_wait(su32(&bars.full_km), (uint32_t)n & 1u) && mbar_wait(su32(&bars.u_ready), (uint32_t)n & 1u);
                if (!ok) break;
                TR(0, n, 6);
                fence_after();
#pragma unroll
                for (int ks = 0; ks < 8; ks++)            // S += (w rk U)^T K, the K tile read MN-major
                    mma_tf32_ts(tmem + TM_S, tmem + TM_TU + 8 * ks, smem_desc_mn32(base + SM_KM + ks * 1024, 8192, 512), ID_SU, 1u);
                mma_commit(su32(&bars.empty_km));
                TR(0, n, 7);
            }
            mma_commit(su32(&bars.s_final));
        }
    } else if (warp < 8) {
        // ================= chain epilogues: T, decay sweep, U =================
        const float *Vs = reinterpret_cast<const float *>(gbase + SM_V) + 32 * half * 128 + row;   // Vs[i * 128] = V[token 32 half + i][row]
        for (int n = 0; n < N && ok; n++) {
            const int s = n & 1;
            const float *aux = reinterpret_cast<const float *>(gbase + SM_AUX + s * AUX_BYTES);
            ok = mbar_wait(su32(&bars.full_kq[s]), (uint32_t)(n >> 1) & 1u) && mbar_wait(su32(&bars.full_v), (uint32_t)n & 1u) &&
                 mbar_wait(su32(&bars.kq_done[s]), (uint32_t)(n >> 1) & 1u);
            if (!ok) break;
            if (tid == 0) TR(1, n, 0);
            fence_after();
            float x[32];
            if (dbg && n == 1) {                                         // the state after the first update (before this chunk's decay)
#pragma unroll 1
                for (int cc = 0; cc < 2; cc++) {
                    tmem_ld32_wait(lane_t + TM_S + 64 * half + 32 * cc, x);
#pragma unroll
                    for (int i = 0; i < 32; i++) dbg[4 * 128 * 64 + row * 128 + 64 * half + 32 * cc + i] = x[i];
                }
            }
            tmem_ld32_wait(lane_t + TM_KQ + 128 * s + 32 * half, x);          // KS^T
            if (tid == 0) TR(4, n, 0);
            if (dbg && n == 0) {
#pragma unroll
                for (int i = 0; i < 32; i++) dbg[row * 64 + 32 * half + i] = x[i];
            }
#pragma unroll
            for (int hh = 0; hh < 4; hh++) {                             // T = beta v - (beta p rk) KS, 8 tokens at a time
                float v[8];
#pragma unroll
                for (int i = 0; i < 8; i++) v[i] = (SEG && kind == 2) ? 0.0f : Vs[(8 * hh + i) * 128];
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const float4 be4 = *reinterpret_cast<const float4 *>(aux + 32 * half + 8 * hh + 4 * i);
                    const float4 bp4 = *reinterpret_cast<const float4 *>(aux + C + 32 * half + 8 * hh + 4 * i);
                    const int k = 8 * hh + 4 * i;
                    x[k] = tf32q(fmaf(-bp4.x, x[k], be4.x * v[4 * i]));
                    x[k + 1] = tf32q(fmaf(-bp4.y, x[k + 1], be4.y * v[4 * i + 1]));
                    x[k + 2] = tf32q(fmaf(-bp4.z, x[k + 2], be4.z * v[4 * i + 2]));
                    x[k + 3] = tf32q(fmaf(-bp4.w, x[k + 3], be4.w * v[4 * i + 3]));
                }
            }
            if (tid == 0) TR(4, n, 1);
            tmem_st32(lane_t + TM_TU + 32 * half, x);                    // T^T
            tmem_wait_st();
            if (tid == 0) TR(4, n, 2);
            fence_before();
            mbar_arrive(su32(&bars.t_ready));
            if (tid == 0) TR(1, n, 1);
            __syncwarp();
            if (lane == 0) mbar_arrive(su32(&bars.empty_v));             // this warp has read its V rows
            if (tid == 0) TR(1, n, 2);
            {   // S *= p_63 while the tensor core computes U^T (nothing reads S until the update)
                const float pend = aux[4 * C];
#pragma unroll 1
                for (int cc = 0; cc < 2; cc++) {
                    tmem_ld32_wait(lane_t + TM_S + 64 * half + 32 * cc, x);
#pragma unroll
                    for (int i = 0; i < 32; i++) x[i] *= pend;
                    tmem_st32(lane_t + TM_S + 64 * half + 32 * cc, x);
                }
            }
            if (tid == 0) TR(1, n, 3);
            ok = mbar_wait(su32(&bars.u_done), (uint32_t)n & 1u);
            if (!ok) break;
            if (tid == 0) TR(1, n, 4);
            fence_after();
            tmem_ld32_wait(lane_t + TM_U + 32 * half, x);                     // U^T
            if (tid == 0) TR(4, n, 3);
            if (dbg && n == 0) {
#pragma unroll
                for (int i = 0; i < 32; i++) dbg[128 * 64 + row * 64 + 32 * half + i] = x[i];
            }
#pragma unroll
            for (int hh = 0; hh < 4; hh++) {                             // (w rk U)^T over T^T, 8 tokens at a time
                float f[8];
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const float4 w4 = *reinterpret_cast<const float4 *>(aux + 2 * C + 32 * half + 8 * hh + 4 * i);   // w rk
                    f[4 * i] = tf32q(w4.x * x[8 * hh + 4 * i]); f[4 * i + 1] = tf32q(w4.y * x[8 * hh + 4 * i + 1]);
                    f[4 * i + 2] = tf32q(w4.z * x[8 * hh + 4 * i + 2]); f[4 * i + 3] = tf32q(w4.w * x[8 * hh + 4 * i + 3]);
                }
                tmem_st8(lane_t + TM_TU + 32 * half + 8 * hh, f);
            }
#pragma unroll
            for (int i = 0; i < 32; i++) x[i] = tf32q(x[i]);
            if (tid == 0) TR(4, n, 4);
            tmem_st32(lane_t + TM_U + 32 * half, x);                     // tf32 U^T over the accumulator
            tmem_wait_st();
            if (tid == 0) TR(4, n, 5);
            fence_before();
            mbar_arrive(su32(&bars.u_ready));
            if (tid == 0) TR(1, n, 5);
            __syncwarp();
            if (lane == 0) mbar_arrive(su32(&bars.empty_kq[s]));         // this warp has read its factors
        }
        ok = ok && mbar_wait(su32(&bars.s_final), 0u);
        fence_after();
#pragma unroll 1
        for (int cc = 0; cc < 2; cc++) {                                 // the state goes home
            float x[32];
            tmem_ld32_wait(lane_t + TM_S + 64 * half + 32 * cc, x);
            float4 *dst = reinterpret_cast<float4 *>(Sout + (size_t)row * 128 + 64 * half + 32 * cc);
#pragma unroll
            for (int i = 0; i < 8; i++)
                dst[i] = ok ? make_float4(x[4 * i], x[4 * i + 1], x[4 * i + 2], x[4 * i + 3]) : make_float4(NAN, NAN, NAN, NAN);
        }
    } else if (warp < 24) {
        // ================= output epilogue =================
        // 16 warps: lane quarter qtr, group grp of 16 tokens
        const int grp = (warp - 8) >> 2;
        const float nwr = a.norm_w[row];
        const size_t zoff = (size_t)b * a.T * vd + (size_t)hv * 128 + row;
        const ACT *zp = (const ACT *)a.z;
        ACT *op = (ACT *)a.out;
        const float *aux = reinterpret_cast<const float *>(gbase + SM_AUX2) + 3 * C + 16 * grp;       // p rq of this group's tokens
        const uint32_t t_qs = lane_t + TM_KQ + 64 + 16 * grp, t_pu = lane_t + TM_KQ + 16 * grp;
        // z of this thread's 16 outputs of a chunk is requested one chunk ahead and stays in these registers until it
        // is used: the loads (DRAM latency, 2 bytes per lane) would otherwise be exposed in every chunk.  The output
        // tiles are read from tensor memory twice (for the sum of squares, then for the store) instead of being kept.
        uint32_t zr[16];
#pragma unroll
        for (int i = 0; i < 16; i++)
            zr[i] = (!(SEG && kind) && c0 * C + 16 * grp + i < a.T) ? ld_raw(zp, zoff + (size_t)(c0 * C + 16 * grp + i) * vd) : 0u;
        int n = 0;
        if (SEG && kind) {
            // raw outputs p rq QS + P U of a run scanned from zero / from the identity: no norm, no gate
            for (; n < N; n++) {
                const int s = n & 1, tok = (c0 + n) * C + 16 * grp;
                ok = mbar_wait(su32(&bars.full_p), (uint32_t)n & 1u) && mbar_wait(su32(&bars.pu_done[s]), (uint32_t)(n >> 1) & 1u);
                if (!ok) break;
                fence_after();
                float q[16], x[16];
                tmem_ld16x2_wait(t_qs + 128 * s, q, t_pu + 128 * s, x);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float4 p4 = *reinterpret_cast<const float4 *>(aux + 4 * i);
                    x[4 * i] = fmaf(p4.x, q[4 * i], x[4 * i]); x[4 * i + 1] = fmaf(p4.y, q[4 * i + 1], x[4 * i + 1]);
                    x[4 * i + 2] = fmaf(p4.z, q[4 * i + 2], x[4 * i + 2]); x[4 * i + 3] = fmaf(p4.w, q[4 * i + 3], x[4 * i + 3]);
                }
                fence_before();
                mbar_arrive(su32(&bars.o_read[s]));
                __syncwarp();
                if (lane == 0) mbar_arrive(su32(&bars.empty_p));
#pragma unroll
                for (int i = 0; i < 16; i++)
                    if (tok + i < a.T) raw[(size_t)(tok + i) * 128 + row] = x[i];
            }
            n = N;                                                       // nothing to poison: the finishing kernel reads the status
        }
        for (; n < N; n++) {
            const int s = n & 1, tok = (c0 + n) * C + 16 * grp;
            if (tid == 256) TR(2, n, 0);
            // the gate factors of this chunk, while the tensor core still works on it: norm weight x SiLU(z), in place
#pragma unroll
            for (int h8 = 0; h8 < 2; h8++) {
#pragma unroll
                for (int i = 0; i < 8; i++) zr[8 * h8 + i] = __float_as_uint(nwr * silu_fast(cvt_raw(zp, zr[8 * h8 + i])));
                asm volatile("" ::: "memory");                           // keeps the two batches apart (registers)
            }
            ok = mbar_wait(su32(&bars.full_p), (uint32_t)n & 1u) && mbar_wait(su32(&bars.pu_done[s]), (uint32_t)(n >> 1) & 1u);
            if (!ok) break;
            if (tid == 256) TR(2, n, 1);
            fence_after();
            {
                float x[16];
#pragma unroll
                for (int h8 = 0; h8 < 2; h8++) {                         // 8 tokens at a time: O = p rq QS + P U, squared
                    float q[8], y[8];
                    tmem_ld8x2_wait(t_qs + 128 * s + 8 * h8, q, t_pu + 128 * s + 8 * h8, y);   // QS^T, (P U)^T
                    if (dbg && n == 0) {
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            dbg[2 * 128 * 64 + row * 64 + 16 * grp + 8 * h8 + i] = q[i];
                            dbg[3 * 128 * 64 + row * 64 + 16 * grp + 8 * h8 + i] = y[i];
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 2; i++) {
                        const float4 p4 = *reinterpret_cast<const float4 *>(aux + 8 * h8 + 4 * i);
                        y[4 * i] = fmaf(p4.x, q[4 * i], y[4 * i]); y[4 * i + 1] = fmaf(p4.y, q[4 * i + 1], y[4 * i + 1]);
                        y[4 * i + 2] = fmaf(p4.z, q[4 * i + 2], y[4 * i + 2]); y[4 * i + 3] = fmaf(p4.w, q[4 * i + 3], y[4 * i + 3]);
                    }
#pragma unroll
                    for (int i = 0; i < 8; i++) x[8 * h8 + i] = y[i] * y[i];
                }
                // sum of squares over the 32 rows of this warp: token t of the 16 ends up in lanes t and t + 16
#pragma unroll
                for (int i = 0; i < 16; i++) x[i] += __shfl_xor_sync(0xffffffffu, x[i], 16);
#pragma unroll
                for (int off = 8; off >= 1; off >>= 1) {
                    const bool up = (lane & off) != 0;
#pragma unroll
                    for (int k = 0; k < off; k++) {
                        const float send = up ? x[k] : x[k + off], keep = up ? x[k + off] : x[k];
                        x[k] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                    }
                }
                if (lane < 16) red[s][grp][qtr][lane] = x[0];
            }
            if (tid == 256) TR(2, n, 2);
            mbar_arrive(su32(&bars.red[s][grp]));
            if (tid == 256) TR(2, n, 3);
            ok = mbar_wait(su32(&bars.red[s][grp]), (uint32_t)(n >> 1) & 1u);
            if (!ok) break;
            if (tid == 256) TR(2, n, 4);
            const int tl = lane & 15;
            const float ss = a.out_scale * a.out_scale *
                             ((red[s][grp][0][tl] + red[s][grp][1][tl]) + (red[s][grp][2][tl] + red[s][grp][3][tl]));
            const float inv = rsqrtf(ss * (1.0f / 128.0f) + a.eps) * a.out_scale;   // of token tl
#pragma unroll
            for (int ps = 0; ps < 2; ps++) {                             // 8 tokens at a time
                float q[8], x[8];
                tmem_ld8x2_wait(t_qs + 128 * s + 8 * ps, q, t_pu + 128 * s + 8 * ps, x);
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const float4 p4 = *reinterpret_cast<const float4 *>(aux + 8 * ps + 4 * i);
                    x[4 * i] = fmaf(p4.x, q[4 * i], x[4 * i]); x[4 * i + 1] = fmaf(p4.y, q[4 * i + 1], x[4 * i + 1]);
                    x[4 * i + 2] = fmaf(p4.z, q[4 * i + 2], x[4 * i + 2]); x[4 * i + 3] = fmaf(p4.w, q[4 * i + 3], x[4 * i + 3]);
                }
                if (ps == 1) {                                           // both tiles and the factors have been read for the last time
                    fence_before();
                    mbar_arrive(su32(&bars.o_read[s]));
                    __syncwarp();
                    if (lane == 0) mbar_arrive(su32(&bars.empty_p));
                }
                // Whole groups of 8 tokens take the path without per-token bounds checks: a conditional store per token
                // would end a basic block per token and keep the independent chains (shuffle, exp, reciprocal) from
                // overlapping.
                const size_t o0 = zoff + (size_t)(tok + 8 * ps) * vd;
#pragma unroll
                for (int i = 0; i < 8; i++) x[i] *= __shfl_sync(0xffffffffu, inv, 8 * ps + i) * __uint_as_float(zr[8 * ps + i]);
                if (tok + 8 * ps + 8 <= a.T) {
#pragma unroll
                    for (int i = 0; i < 8; i++) act_st(op, o0 + (size_t)i * vd, x[i]);
                } else {
#pragma unroll
                    for (int i = 0; i < 8; i++)
                        if (tok + 8 * ps + i < a.T) act_st(op, o0 + (size_t)i * vd, x[i]);
                }
                if (tok + C + 8 * ps + 8 <= a.T) {                       // the same tokens of the next chunk
#pragma unroll
                    for (int i = 0; i < 8; i++) zr[8 * ps + i] = ld_raw(zp, o0 + (size_t)(C + i) * vd);
                } else {
#pragma unroll
                    for (int i = 0; i < 8; i++)
                        zr[8 * ps + i] = (tok + C + 8 * ps + i < a.T) ? ld_raw(zp, o0 + (size_t)(C + i) * vd) : 0u;
                }
            }
            if (tid == 256) TR(2, n, 5);
        }
        for (; n < N; n++) {                                             // a wait gave up: poison what was not written
            const int tok = n * C + 16 * grp;
            for (int i = 0; i < 16; i++)
                if (tok + i < a.T) act_st(op, zoff + (size_t)(tok + i) * vd, NAN);
        }
    }
    else {
        // ================= (P U)^T, issued apart from the chain =================
        // Its operand U^T is ready at the same moment as the state update's; a thread of its own keeps these
        // eight instructions out of the issue stream the next chunk waits for.
        if (warp == W_PU && lane == 0) {
            fence_after();
            for (int n = 0; n < N; n++) {
                ok = mbar_wait(su32(&bars.full_p), (uint32_t)n & 1u) && mbar_wait(su32(&bars.u_ready), (uint32_t)n & 1u);
                if (!ok) break;
                fence_after();
                issue_tri(tmem + TM_KQ + 128 * (n & 1), tmem + TM_U, base + SM_P);   // over the KS columns of the chunk
                mma_commit(su32(&bars.pu_done[n & 1]));
                mma_commit(su32(&bars.empty_p));
            }
        }
    }
    if (!ok) report_timeout(a.status, ORN_WAIT_DELTA_SCAN);
    fence_before();
    __syncthreads();
    if (warp == W_MMA) tmem_dealloc(tmem, TM_COLS);
}

// =============================================================================
// segment-parallel form: carrying the state over the runs, and the finishing pass
// =============================================================================
// S_in of run j+1 = S_in of run j x Phi_j + S0_j, rows of the state independent of one another: one CTA per
// (sequence, head, group of 8 rows), 128 threads = the 128 columns.  Leaves S_in of every run j >= 1 in its slot
// of seg_state and the final state in the caller's S.
__global__ void __launch_bounds__(128) k_delta_seg_carry(ScanArgs a) {
    __shared__ float srow[8][128];
    __shared__ __align__(16) float phi[32][128];                                  // 32 rows of Phi at a time
    const int hv = blockIdx.x, b = blockIdx.y, r0 = 8 * blockIdx.z, c = threadIdx.x;
    float *slots = a.seg_state + ((size_t)b * a.nv + hv) * 3 * a.n_seg * (128 * 128);
    float s[8];
#pragma unroll
    for (int r = 0; r < 8; r++) s[r] = slots[(size_t)(r0 + r) * 128 + c];          // end state of run 0
    for (int j = 1; j < a.n_seg; j++) {
        const float *S0 = slots + (size_t)(3 * j) * (128 * 128), *Phi = S0 + 128 * 128;
        float *Sin = slots + (size_t)(3 * j + 2) * (128 * 128);
        float acc[8];
#pragma unroll
        for (int r = 0; r < 8; r++) { Sin[(size_t)(r0 + r) * 128 + c] = s[r]; srow[r][c] = s[r]; acc[r] = S0[(size_t)(r0 + r) * 128 + c]; }
        for (int l0 = 0; l0 < 128; l0 += 32) {
            __syncthreads();                                                      // srow written / phi free again
            float4 v[8];
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = reinterpret_cast<const float4 *>(Phi + (size_t)l0 * 128)[i * 128 + c];
#pragma unroll
            for (int i = 0; i < 8; i++) reinterpret_cast<float4 *>(&phi[0][0])[i * 128 + c] = v[i];
            __syncthreads();
#pragma unroll 8
            for (int l = 0; l < 32; l++) {
                const float p = phi[l][c];
#pragma unroll
                for (int r = 0; r < 8; r++) acc[r] = fmaf(srow[r][l0 + l], p, acc[r]);
            }
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < 8; r++) s[r] = acc[r];
    }
    float *Sg = a.S + (size_t)b * a.S_stride + (size_t)hv * 128 * 128;
#pragma unroll
    for (int r = 0; r < 8; r++) Sg[(size_t)(r0 + r) * 128 + c] = s[r];
}

// o_t = o0_t + S_in qt_t for the tokens of the runs j >= 1, then the output scale, the per-head RMSNorm and the
// SiLU(z) gate (reference: linear_finish, src/ornith_rforward.c:300-314).  One CTA per (256 tokens, head, sequence)
// walks four tiles of 64 tokens with S_in of its run in shared memory: a 64 x 128 x 128 product on tf32 mma.sync
// (A = the qt rows, B = S_in, both rounded to tf32), four warps of 16 tokens; the normalised tile then goes through
// shared memory so that z is read and the output written in whole rows.
constexpr int FIN_LD = 132, FIN_TOK = 256;
struct FinSmem { float Sin[128 * FIN_LD]; float Qt[64 * FIN_LD]; };
template <typename ACT>
__global__ void __launch_bounds__(128, 2) k_delta_seg_finish(ScanArgs a) {
    extern __shared__ __align__(16) unsigned char smraw[];
    FinSmem &sm = *reinterpret_cast<FinSmem *>(smraw);
    const int hv = blockIdx.y, b = blockIdx.z, tid = threadIdx.x, lane = tid & 31, w = tid >> 5, g = lane >> 2, j4 = lane & 3;
    const int seg_tokens = a.seg_chunks * C;                                       // a multiple of FIN_TOK? no: of 64
    const int tiles_per_seg = (seg_tokens + FIN_TOK - 1) / FIN_TOK;
    const int seg = 1 + (int)blockIdx.x / tiles_per_seg;                           // run 0 is final already
    const int tbeg = seg * seg_tokens + ((int)blockIdx.x % tiles_per_seg) * FIN_TOK;
    const int tend = min(min(tbeg + FIN_TOK, (seg + 1) * seg_tokens), a.T);
    if (tbeg >= tend) return;
    const size_t hb = (size_t)b * a.nv + hv, planes = (size_t)gridDim.z * a.nv;
    const float *Sin = a.seg_state + (hb * 3 * a.n_seg + 3 * seg + 2) * (128 * 128);
    const float *o0 = a.seg_raw + hb * (size_t)a.T * 128, *qt = a.seg_raw + (planes + hb) * (size_t)a.T * 128;
    const int vd = a.nv * 128;
    const ACT *zp = (const ACT *)a.z;
    ACT *op = (ACT *)a.out;
    for (int e = tid; e < 128 * 32; e += 128) {
        const int r = e >> 5, c4 = (e & 31) * 4;
        float4 v = *reinterpret_cast<const float4 *>(Sin + (size_t)r * 128 + c4);
        v.x = tf32r(v.x); v.y = tf32r(v.y); v.z = tf32r(v.z); v.w = tf32r(v.w);
        *reinterpret_cast<float4 *>(&sm.Sin[r * FIN_LD + c4]) = v;
    }
    const float4 nw4 = *reinterpret_cast<const float4 *>(a.norm_w + 4 * lane);     // channels 4 lane .. of the store pass
    for (int t0 = tbeg; t0 < tend; t0 += 64) {
        __syncthreads();                                                          // the tile buffer is free (and S_in is in place)
        for (int e = tid; e < 64 * 32; e += 128) {
            const int i = e >> 5, c4 = (e & 31) * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t0 + i < tend) v = *reinterpret_cast<const float4 *>(qt + (size_t)(t0 + i) * 128 + c4);
            v.x = tf32r(v.x); v.y = tf32r(v.y); v.z = tf32r(v.z); v.w = tf32r(v.w);
            *reinterpret_cast<float4 *>(&sm.Qt[i * FIN_LD + c4]) = v;
        }
        __syncthreads();
        // acc[nt][x]: token 16 w + g + 8 (x >> 1), value row 8 nt + 2 j4 + (x & 1)
        float acc[16][4];
#pragma unroll
        for (int nt = 0; nt < 16; nt++)
#pragma unroll
            for (int x = 0; x < 4; x++) acc[nt][x] = 0.0f;
        const float *A0 = sm.Qt + (16 * w) * FIN_LD;
#pragma unroll 2
        for (int k0 = 0; k0 < 128; k0 += 8) {
            float af[4];
            af[0] = A0[g * FIN_LD + k0 + j4];
            af[1] = A0[(g + 8) * FIN_LD + k0 + j4];
            af[2] = A0[g * FIN_LD + k0 + j4 + 4];
            af[3] = A0[(g + 8) * FIN_LD + k0 + j4 + 4];
#pragma unroll
            for (int nt = 0; nt < 16; nt++) {
                const float *br = sm.Sin + (8 * nt + g) * FIN_LD + k0 + j4;         // B[k][n] = S_in[n][k]
                mma_tf32_sync(acc[nt], af, br[0], br[4]);
            }
        }
        __syncthreads();                                                          // every warp is done reading the qt tile
        // the correction goes over the qt tile (own rows only), then whole rows: + o0, scale, norm, gate, store
#pragma unroll
        for (int nt = 0; nt < 16; nt++) {
            const int r = 8 * nt + 2 * j4;
            *reinterpret_cast<float2 *>(&sm.Qt[(16 * w + g) * FIN_LD + r]) = make_float2(acc[nt][0], acc[nt][1]);
            *reinterpret_cast<float2 *>(&sm.Qt[(16 * w + g + 8) * FIN_LD + r]) = make_float2(acc[nt][2], acc[nt][3]);
        }
        __syncwarp();
        // whole rows, 4 channels per lane; the loads of 8 tokens are issued together (memory latency, not arithmetic,
        // bounds this pass)
#pragma unroll
        for (int i0 = 0; i0 < 16; i0 += 8) {
            float4 b4[8], z4[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int t = min(t0 + 16 * w + i0 + i, tend - 1);               // rows past the end repeat the last row (never stored)
                b4[i] = *reinterpret_cast<const float4 *>(o0 + (size_t)t * 128 + 4 * lane);
                z4[i] = act_ld4(zp, ((size_t)b * a.T + t) * vd + (size_t)hv * 128 + 4 * lane);
            }
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int t = t0 + 16 * w + i0 + i;
                const float4 c4 = *reinterpret_cast<const float4 *>(&sm.Qt[(16 * w + i0 + i) * FIN_LD + 4 * lane]);
                float4 o = make_float4((c4.x + b4[i].x) * a.out_scale, (c4.y + b4[i].y) * a.out_scale,
                                       (c4.z + b4[i].z) * a.out_scale, (c4.w + b4[i].w) * a.out_scale);
                float ss = (o.x * o.x + o.y * o.y) + (o.z * o.z + o.w * o.w);
                ss = warp_sum(ss);
                const float inv = rsqrtf(ss * (1.0f / 128.0f) + a.eps);
                if (t < tend)
                    act_st4(op, ((size_t)b * a.T + t) * vd + (size_t)hv * 128 + 4 * lane,
                            make_float4(o.x * inv * nw4.x * silu_fast(z4[i].x), o.y * inv * nw4.y * silu_fast(z4[i].y),
                                        o.z * inv * nw4.z * silu_fast(z4[i].z), o.w * inv * nw4.w * silu_fast(z4[i].w)));
            }
        }
    }
}

// How many runs the prompt is cut into: only when the heads alone would leave most SMs idle (2 P - 1 CTAs per
// head), with at least 8 chunks per run.  ORNITH_CUDA_DELTA_SEGMENTS=<n> forces a count (1 = off).
int delta_seg_plan(int nv, int n_seq, int n_chunks, int *seg_chunks) {
    int p = 1;
    const char *e = getenv("ORNITH_CUDA_DELTA_SEGMENTS");
    if (e && e[0]) p = atoi(e);
    else {
        const int heads = nv * n_seq;
        if (heads <= 37) p = (148 / heads + 1) / 2;                  // 2 p - 1 <= 148 / heads
        if (p > 16) p = 16;
    }
    if (p > n_chunks / 8) p = n_chunks / 8;
    if (p < 1) p = 1;
    int sc = (n_chunks + p - 1) / p;
    p = (n_chunks + sc - 1) / sc;                                     // no empty run
    *seg_chunks = sc;
    return p;
}

// [rows][cols] f32, boxes of box_cols columns x box_rows rows; swz 0: no swizzle, 1: 128-byte swizzle, 2: the same with 32-byte atoms
ornith_status f32_rows_map(CUtensorMap *m, const void *basep, uint64_t cols, uint64_t rows, uint32_t box_rows, int swz, uint32_t box_cols = 32) {
    OrnTensorMapEncodeFn enc = orn_tensor_map_encoder();
    if (!enc) { orn_record_error("delta scan: cuTensorMapEncodeTiled is not available"); return (ornith_status)ORNITH_ERR_BACKEND; }
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 4};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t es[2] = {1, 1};
    const CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(basep), dims, strides, box, es,
                           CU_TENSOR_MAP_INTERLEAVE_NONE,
                           swz == 2 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : (swz == 1 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE),
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { orn_record_error("delta scan: cuTensorMapEncodeTiled failed (%d)", (int)r); return (ornith_status)ORNITH_ERR_BACKEND; }
    return ORNITH_OK;
}

}  // namespace

static size_t ap_part(int nv, int n_seq, int n_chunks) { return align_up((size_t)n_seq * nv * n_chunks * AP_BYTES, 256); }
static size_t aux_part(int nv, int n_seq, int n_chunks) { return align_up((size_t)n_seq * nv * n_chunks * AUX_BYTES, 256); }

static size_t seg_state_part(int nv, int n_seq, int n_seg) { return n_seg > 1 ? align_up((size_t)n_seq * nv * 3 * n_seg * 128 * 128 * 4, 256) : 0; }
static size_t seg_raw_part(int nv, int n_seq, int T, int n_seg) { return n_seg > 1 ? align_up((size_t)2 * n_seq * nv * T * 128 * 4, 256) : 0; }

size_t linear_prefill_tc5_work_bytes(int nk, int nv, int n_seq, int T) {
    const int n_chunks = (T + C - 1) / C;
    (void)nk;
    int sc;
    const int n_seg = delta_seg_plan(nv, n_seq, n_chunks, &sc);
    return ap_part(nv, n_seq, n_chunks) + aux_part(nv, n_seq, n_chunks) + seg_state_part(nv, n_seq, n_seg) + seg_raw_part(nv, n_seq, T, n_seg);
}
size_t linear_prefill_tc5_dump_floats() { return DBG_FLOATS; }

namespace {

// The second stream and the events of the slab pipeline, one set per device.  The lock covers one call's
// launches: a wait takes the event's state at the moment it is enqueued, so the next call may re-record.
constexpr int MAX_SLABS = 16;
struct SlabPipe {
    std::mutex lock;
    cudaStream_t scan_stream = nullptr;
    cudaEvent_t front_done[MAX_SLABS] = {}, scans_done = nullptr;
};
SlabPipe g_slab_pipe[ORN_MAX_DEVICES];

ornith_status slab_pipe_ready(SlabPipe &p) {
    if (p.scan_stream) return ORNITH_OK;
    int least = 0, greatest = 0;
    ORN_TRY(orn_check(cudaDeviceGetStreamPriorityRange(&least, &greatest), "stream priority range"));
    cudaStream_t st = nullptr;
    ORN_TRY(orn_check(cudaStreamCreateWithPriority(&st, cudaStreamNonBlocking, greatest), "delta scan stream"));
    for (int i = 0; i < MAX_SLABS; i++) ORN_TRY(orn_check(cudaEventCreateWithFlags(&p.front_done[i], cudaEventDisableTiming), "slab event"));
    ORN_TRY(orn_check(cudaEventCreateWithFlags(&p.scans_done, cudaEventDisableTiming), "slab event"));
    p.scan_stream = st;
    return ORNITH_OK;
}

// slabs of the prompt: 48 chunks or more each, at most 8; 1 = no pipeline (ORNITH_CUDA_DELTA_SLABS overrides)
int slab_plan(int heads, int n_chunks, int n_seg) {
    if (n_seg > 1 || heads > 148) return 1;
    int n = n_chunks / 48;                                            // a slab costs about 25 us of start-up and hand-over
    if (n > 8) n = 8;
    const char *e = getenv("ORNITH_CUDA_DELTA_SLABS");
    if (e && e[0]) n = atoi(e);
    if (n > MAX_SLABS) n = MAX_SLABS;
    if (n > n_chunks) n = n_chunks;
    return n < 1 ? 1 : n;
}

}  // namespace

// frees the current device's scan stream and events (the next long prefill makes new ones); the device is idle
ornith_status release_delta_slab_pipe() {
    SlabPipe &p = g_slab_pipe[orn_device_index()];
    std::lock_guard<std::mutex> hold(p.lock);
    if (!p.scan_stream) return ORNITH_OK;
    for (int i = 0; i < MAX_SLABS; i++) { if (p.front_done[i]) (void)cudaEventDestroy(p.front_done[i]); p.front_done[i] = nullptr; }
    if (p.scans_done) (void)cudaEventDestroy(p.scans_done);
    p.scans_done = nullptr;
    const cudaError_t e = cudaStreamDestroy(p.scan_stream);
    p.scan_stream = nullptr;
    return orn_check(e, "delta scan stream destroy");
}

ornith_status launch_linear_prefill_tc5(const LinArgs &x, int n_seq, int act_dtype, const float *Y, const float *rq,
                                        const float *rk, const float *la, const float *be, const TC5Front *front,
                                        float *work, float *dbg, cudaStream_t s) {
    extern long long *g_delta_scan_trace;
    const int n_chunks = (x.T + C - 1) / C;
    const size_t n_blocks = (size_t)n_seq * x.nv * n_chunks;
    const int Cc = 2 * x.nk * 128 + x.nv * 128;
    if ((size_t)n_seq * x.T >= (1u << 31) || n_blocks * AP_ROWS >= (1u << 31)) {
        orn_record_error("delta scan: %d sequences x %d tokens exceed the tensor-map coordinates", n_seq, x.T);
        return ORNITH_ERR_UNSUPPORTED;
    }
    float *AP = work, *aux = (float *)((char *)work + ap_part(x.nv, n_seq, n_chunks));
    static bool configured_dev[ORN_MAX_DEVICES] = {};
    bool &configured = configured_dev[orn_device_index()];
    if (!configured) {
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_delta_prep64<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(PrepSmem)),
                          "delta prep smem opt-in"));
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_delta_prep64<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(PrepSmem)),
                          "delta prep smem opt-in"));
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_delta_scan_tc5<float, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SCAN_SMEM),
                          "delta scan smem opt-in"));
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_delta_scan_tc5<__nv_bfloat16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SCAN_SMEM),
                          "delta scan smem opt-in"));
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_delta_scan_tc5<float, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SCAN_SMEM),
                          "delta scan smem opt-in"));
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_delta_scan_tc5<__nv_bfloat16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SCAN_SMEM),
                          "delta scan smem opt-in"));
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_delta_seg_finish<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(FinSmem)),
                          "delta finish smem opt-in"));
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_delta_seg_finish<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(FinSmem)),
                          "delta finish smem opt-in"));
        configured = true;
    }
    const bool bf = act_dtype == ORNITH_ACT_BF16;
    CUtensorMap my, mym, map_ap, map_ap32, map_v;
    ORN_TRY(f32_rows_map(&my, Y, (uint64_t)Cc, (uint64_t)n_seq * x.T, C, 1));
    ORN_TRY(f32_rows_map(&mym, Y, (uint64_t)Cc, (uint64_t)n_seq * x.T, C, 2));
    ORN_TRY(f32_rows_map(&map_v, Y, (uint64_t)Cc, (uint64_t)n_seq * x.T, C, 0, 128));
    ORN_TRY(f32_rows_map(&map_ap, AP, 32, n_blocks * AP_ROWS, C, 1));
    ORN_TRY(f32_rows_map(&map_ap32, AP, 32, n_blocks * AP_ROWS, 32, 1));
    ScanArgs a;
    a.Y = Y; a.aux = aux; a.S = x.S; a.S_stride = x.S_stride; a.z = x.z; a.out = x.out; a.norm_w = x.norm_w;
    a.nk = x.nk; a.nv = x.nv; a.head_map = x.head_map; a.T = x.T; a.n_chunks = n_chunks;
    a.c_begin = 0; a.c_count = n_chunks;
    a.out_scale = x.out_scale; a.eps = x.eps; a.status = orn_status_word(); a.dbg = dbg; a.trace = g_delta_scan_trace;
    a.n_seg = delta_seg_plan(x.nv, n_seq, n_chunks, &a.seg_chunks);
    a.seg_state = (float *)((char *)aux + aux_part(x.nv, n_seq, n_chunks));
    a.seg_raw = (float *)((char *)a.seg_state + seg_state_part(x.nv, n_seq, a.n_seg));

    auto prep = [&](int c_begin, int c_count, cudaStream_t ps) {
        const dim3 pgrid((unsigned)c_count, (unsigned)x.nk, (unsigned)n_seq);
        if (bf) k_delta_prep64<__nv_bfloat16><<<pgrid, 256, sizeof(PrepSmem), ps>>>(x, Y, rq, rk, la, be, AP, aux, n_chunks, c_begin);
        else    k_delta_prep64<float><<<pgrid, 256, sizeof(PrepSmem), ps>>>(x, Y, rq, rk, la, be, AP, aux, n_chunks, c_begin);
        return orn_check_launch("k_delta_prep64");
    };
    auto scan = [&](const ScanArgs &sa, cudaStream_t ss) {
        dim3 grid((unsigned)x.nv, (unsigned)n_seq);
        if (bf) k_delta_scan_tc5<__nv_bfloat16, false><<<grid, NTHREADS, SCAN_SMEM, ss>>>(my, mym, map_ap, map_ap32, map_v, sa);
        else    k_delta_scan_tc5<float, false><<<grid, NTHREADS, SCAN_SMEM, ss>>>(my, mym, map_ap, map_ap32, map_v, sa);
        return orn_check_launch("k_delta_scan_tc5");
    };

    // two runs per head (30-37 heads) lose to the slab pipeline on a long prompt: 2.41 against 2.07 ms for 32 heads x
    // 32768 tokens (the finishing pass costs more than the halved chain saves); three runs or more win (16 heads: 1.72
    // against 1.99 ms)
    const char *seg_env = getenv("ORNITH_CUDA_DELTA_SEGMENTS");
    if (front && a.n_seg == 2 && !(seg_env && seg_env[0]) && slab_plan(x.nv * n_seq, n_chunks, 1) >= 2) a.n_seg = 1;
    const int n_slabs = front ? slab_plan(x.nv * n_seq, n_chunks, a.n_seg) : 1;
    if (n_slabs > 1) {
        // front of slab k + 1 on the caller's stream beside the scan of slab k on the scan stream
        SlabPipe &pipe = g_slab_pipe[orn_device_index()];
        std::lock_guard<std::mutex> hold(pipe.lock);
        ORN_TRY(slab_pipe_ready(pipe));
        const int per = (n_chunks + n_slabs - 1) / n_slabs;
        auto slab = [&](int k, int cb, int cn) -> ornith_status {
            ORN_TRY(front->conv(cb * C, min(x.T, (cb + cn) * C), s));
            ORN_TRY(prep(cb, cn, s));
            ORN_TRY(orn_check(cudaEventRecord(pipe.front_done[k], s), "slab event record"));
            ORN_TRY(orn_check(cudaStreamWaitEvent(pipe.scan_stream, pipe.front_done[k], 0), "slab event wait"));
            ScanArgs sa = a;
            sa.c_begin = cb; sa.c_count = cn;
            return scan(sa, pipe.scan_stream);
        };
        ornith_status st = ORNITH_OK;
        int k = 0;
        for (int cb = 0; cb < n_chunks && st == ORNITH_OK; cb += per, k++) st = slab(k, cb, min(per, n_chunks - cb));
        if (st == ORNITH_OK) st = front->ring_refresh(s);     // after the conv that reads the old history
        // the caller's stream always rejoins the scan stream, also when a launch failed on the way
        ornith_status join = orn_check(cudaEventRecord(pipe.scans_done, pipe.scan_stream), "slab event record");
        if (join == ORNITH_OK) join = orn_check(cudaStreamWaitEvent(s, pipe.scans_done, 0), "slab event wait");
        return st != ORNITH_OK ? st : join;
    }
    if (front) {
        ORN_TRY(front->conv(0, x.T, s));
        ORN_TRY(front->ring_refresh(s));
    }
    ORN_TRY(prep(0, n_chunks, s));
    if (a.n_seg <= 1) return scan(a, s);
    // few heads: the runs of the prompt side by side, then the carry over the runs and the finishing pass
    dim3 grid((unsigned)x.nv, (unsigned)n_seq, (unsigned)(2 * a.n_seg - 1));
    if (bf) k_delta_scan_tc5<__nv_bfloat16, true><<<grid, NTHREADS, SCAN_SMEM, s>>>(my, mym, map_ap, map_ap32, map_v, a);
    else    k_delta_scan_tc5<float, true><<<grid, NTHREADS, SCAN_SMEM, s>>>(my, mym, map_ap, map_ap32, map_v, a);
    ORN_TRY(orn_check_launch("k_delta_scan_tc5 (runs)"));
    k_delta_seg_carry<<<dim3((unsigned)x.nv, (unsigned)n_seq, 16), 128, 0, s>>>(a);
    ORN_TRY(orn_check_launch("k_delta_seg_carry"));
    const int fin_tiles = (a.n_seg - 1) * ((a.seg_chunks * C + FIN_TOK - 1) / FIN_TOK);
    dim3 fgrid((unsigned)fin_tiles, (unsigned)x.nv, (unsigned)n_seq);
    if (bf) k_delta_seg_finish<__nv_bfloat16><<<fgrid, 128, sizeof(FinSmem), s>>>(a);
    else    k_delta_seg_finish<float><<<fgrid, 128, sizeof(FinSmem), s>>>(a);
    return orn_check_launch("k_delta_seg_finish");
}
