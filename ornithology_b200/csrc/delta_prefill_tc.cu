// delta_prefill_tc.cu — gated delta-net prefill scan for dk = dv = 128 with the
// chunk contractions on the tensor cores (tf32 operands, fp32 accumulation).
//
// Reference behaviour being replaced: the chunked scan of ornith_delta_prefill
// (src/ornith_attn.c:215-349) inside linear_attn_prefill (src/ornith_rforward.c:563-618).
//
// Per chunk of 32 tokens with incoming state S, G_i the running sum of the
// log-decay inside the chunk, p_i = exp(G_i), Gamma_ij = exp(G_i - G_j):
//   M = diag(beta) strictLower(Gamma o K K^T),  A = (I + M)^-1,  P = lower(Gamma o Q K^T)
//   T = diag(beta) (V - diag(p) K S^T)
//   U = A T
//   O = diag(p) Q S^T + P U
//   S <- p_31 S + sum_j Gamma_31,j u_j k_j^T
// A and P do not depend on the state, so they are produced for every chunk at
// once by k_delta_chunk_prep (Gram matrices on the tensor cores, the triangular
// inverse by fp32 substitution).  What remains sequential, k_delta_chunk_scan,
// is five small contractions per chunk.  Columns r of the state are independent
// of one another, so one (value head, sequence) is spread over a thread-block
// cluster of 128/NR CTAs owning NR columns each; the only thing they exchange
// is the per-token sum of squares for the output RMSNorm, through distributed
// shared memory.  The fp32 master copy of the state stays in registers (it is
// the accumulator of the state update); a tf32 image of it in shared memory is
// the B operand of the next chunk's K S^T / Q S^T.
#include <cuda_runtime.h>
#include <math.h>

#include "bulk_copy.cuh"
#include "linear_attn.cuh"

namespace {

constexpr int TC = 32;                   // tokens per chunk
constexpr int LDK = 132;                 // K / Q rows: stride = 4 mod 32 keeps A fragments conflict-free
constexpr int LDP = 36;                  // A / P rows
constexpr int LDG = 33;
constexpr int BLK_P = TC * LDP, BLK_AUX = 2 * TC * LDP;
constexpr int BLK_FLOATS = BLK_AUX + 4 * TC;              // A, P, then p | beta | w_end | beta*p
constexpr uint32_t BLK_BYTES = BLK_FLOATS * 4;
constexpr int TILE_FLOATS = TC * LDK;                     // one chunk of normalised k (or q) rows, padded as in shared memory
constexpr uint32_t TILE_BYTES = TILE_FLOATS * 4;

__device__ __forceinline__ float tf32r(float x) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return __uint_as_float(u);
}

// D(16x8) += A(16x8) B(8x8).  Fragment owners, g = lane / 4, j = lane % 4:
//   a0 (g, j) a1 (g+8, j) a2 (g, j+4) a3 (g+8, j+4);  b0 (k=j, n=g) b1 (k=j+4, n=g);
//   d0 (g, 2j) d1 (g, 2j+1) d2 (g+8, 2j) d3 (g+8, 2j+1).
__device__ __forceinline__ void mma_tf32(float (&d)[4], const float (&a)[4], float b0, float b1) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(__float_as_uint(a[0])), "r"(__float_as_uint(a[1])), "r"(__float_as_uint(a[2])),
          "r"(__float_as_uint(a[3])), "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)));
}

// A fragment of a row-major [m][k] tile whose (0, 0) element is at base
__device__ __forceinline__ void frag_a(float (&a)[4], const float *base, int ld, int g, int j) {
    a[0] = base[g * ld + j];
    a[1] = base[(g + 8) * ld + j];
    a[2] = base[g * ld + j + 4];
    a[3] = base[(g + 8) * ld + j + 4];
}

// =============================================================================
// state-independent part: one CTA per (chunk, key head, sequence)
// =============================================================================
// Writes the chunk's normalised, tf32-rounded q / k rows as two packed tiles [32][132] (the
// layout the scan keeps in shared memory, so that one bulk copy fetches a tile), then for
// every value head that reads this key head one block of BLK_FLOATS floats:
// A [32][36], P [32][36] (both tf32), p, beta, w_end, beta*p [32 each].
struct PrepSmem {
    float Ks[TC * LDK];
    float Qs[TC * LDK];
    float GK[TC * LDG];                  // raw k_i.k_j
    float GQ[TC * LDG];                  // raw q_i.k_j
    float Mw[4][TC * LDG];               // per warp: beta_i Gamma_ij k_i.k_j, j < i
    float Gw[4][TC], Bw[4][TC];
};

__global__ void __launch_bounds__(128) k_delta_chunk_prep(LinArgs a, const float *Y, const float *rq, const float *rk,
                                                          const float *la, const float *be, float *blocks,
                                                          float *Kp, float *Qp, int n_chunks) {
    extern __shared__ __align__(16) unsigned char smraw[];
    PrepSmem &sm = *reinterpret_cast<PrepSmem *>(smraw);
    const int chunk = blockIdx.x, kh = blockIdx.y, b = blockIdx.z, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int g = lane >> 2, j = lane & 3;
    const int qd = a.nk * 128, Cc = 2 * qd + a.nv * 128;
    const int t0 = chunk * TC, n = min(TC, a.T - t0);
    const size_t tok0 = (size_t)b * a.T + t0;

    for (int e = tid; e < TC * 32; e += 128) {            // rows past the end are zero
        const int i = e >> 5, c = (e & 31) * 4;
        float4 q = make_float4(0.f, 0.f, 0.f, 0.f), k = q;
        if (i < n) {
            const float *y = Y + (tok0 + i) * Cc + kh * 128 + c;
            const float sq = rq[(tok0 + i) * a.nk + kh], sk = rk[(tok0 + i) * a.nk + kh];
            q = *reinterpret_cast<const float4 *>(y);
            k = *reinterpret_cast<const float4 *>(y + qd);
            q.x = tf32r(q.x * sq); q.y = tf32r(q.y * sq); q.z = tf32r(q.z * sq); q.w = tf32r(q.w * sq);
            k.x = tf32r(k.x * sk); k.y = tf32r(k.y * sk); k.z = tf32r(k.z * sk); k.w = tf32r(k.w * sk);
        }
        *reinterpret_cast<float4 *>(&sm.Qs[i * LDK + c]) = q;
        *reinterpret_cast<float4 *>(&sm.Ks[i * LDK + c]) = k;
    }
    if (tid < TC) {                                       // the four pad columns travel with the tile
        *reinterpret_cast<float4 *>(&sm.Qs[tid * LDK + 128]) = make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4 *>(&sm.Ks[tid * LDK + 128]) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __syncthreads();
    {
        const size_t tile = (((size_t)b * a.nk + kh) * n_chunks + chunk) * TILE_FLOATS;
        for (int e = tid; e < TILE_FLOATS / 4; e += 128) {
            reinterpret_cast<float4 *>(Kp + tile)[e] = reinterpret_cast<const float4 *>(sm.Ks)[e];
            reinterpret_cast<float4 *>(Qp + tile)[e] = reinterpret_cast<const float4 *>(sm.Qs)[e];
        }
    }
    {   // Gram tiles on or below the diagonal: warps 0-1 K K^T, warps 2-3 Q K^T; mt = w & 1
        const int which = w >> 1, mt = w & 1, ntn = 2 * mt + 2;
        float acc[4][4];
#pragma unroll
        for (int t = 0; t < 4; t++)
#pragma unroll
            for (int x = 0; x < 4; x++) acc[t][x] = 0.0f;
        const float *A = (which ? sm.Qs : sm.Ks) + 16 * mt * LDK;
#pragma unroll 4
        for (int k0 = 0; k0 < 128; k0 += 8) {
            float af[4];
            frag_a(af, A + k0, LDK, g, j);
#pragma unroll
            for (int t = 0; t < 4; t++) {
                if (t < ntn) {
                    const float *kr = sm.Ks + (8 * t + g) * LDK + k0 + j;
                    mma_tf32(acc[t], af, kr[0], kr[4]);
                }
            }
        }
        float *G = which ? sm.GQ : sm.GK;
#pragma unroll
        for (int t = 0; t < 4; t++)
#pragma unroll
            for (int x = 0; x < 4; x++)
                G[(16 * mt + g + 8 * (x >> 1)) * LDG + 8 * t + 2 * j + (x & 1)] = acc[t][x];
    }
    __syncthreads();
    const int nvk = a.nv / a.nk;
    for (int m = w; m < nvk; m += 4) {                    // one warp per value head of this key head
        const int hv = a.head_map == ORNITH_HEADMAP_GROUPED ? kh * nvk + m : kh + m * a.nk;
        float gg = 0.0f, bb = 0.0f;
        if (lane < n) { gg = la[(tok0 + lane) * a.nv + hv]; bb = be[(tok0 + lane) * a.nv + hv]; }
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float up = __shfl_up_sync(0xffffffffu, gg, o);
            if (lane >= o) gg += up;
        }
        const float gl = __shfl_sync(0xffffffffu, gg, 31);
        float *blk = blocks + (((size_t)b * a.nv + hv) * n_chunks + chunk) * BLK_FLOATS;
        const float pp = expf(gg);
        blk[BLK_AUX + lane] = pp;
        blk[BLK_AUX + TC + lane] = bb;
        blk[BLK_AUX + 2 * TC + lane] = expf(gl - gg);
        blk[BLK_AUX + 3 * TC + lane] = bb * pp;
        __syncwarp();
        sm.Gw[w][lane] = gg; sm.Bw[w][lane] = bb;
        __syncwarp();
        float *Mw = sm.Mw[w];
#pragma unroll 4
        for (int i = 0; i < TC; i++) {                    // lane = column l of row i
            const float gam = (lane <= i) ? expf(sm.Gw[w][i] - gg) : 0.0f;
            Mw[i * LDG + lane] = (lane < i) ? sm.Bw[w][i] * gam * sm.GK[i * LDG + lane] : 0.0f;
            blk[BLK_P + i * LDP + lane] = (lane <= i) ? tf32r(gam * sm.GQ[i * LDG + lane]) : 0.0f;
        }
        __syncwarp();
        float x[TC];                                      // lane = column of the inverse
#pragma unroll
        for (int i = 0; i < TC; i++) {
            float acc = (i == lane) ? 1.0f : 0.0f;
#pragma unroll
            for (int l = 0; l < i; l++) acc -= Mw[i * LDG + l] * x[l];
            x[i] = acc;
        }
#pragma unroll
        for (int i = 0; i < TC; i++) blk[i * LDP + lane] = tf32r(x[i]);
        __syncwarp();
    }
}

// =============================================================================
// sequential part: a cluster of 128/NR CTAs per (value head, sequence)
// =============================================================================
// Every MMA operand that is re-read lives in shared memory with its contraction
// index contiguous and a row stride of 4 mod 32 words, so that one ldmatrix.x4
// (8x8 tiles of b16 pairs = 8 rows x 4 tf32 words) fetches a whole A fragment,
// or the B fragments of two k-steps, without bank conflicts.
template <int NR>
struct ScanSmem {
    static constexpr int LDN = NR + 8;
    struct Stage {
        float Ks[TC * LDK];
        float Qs[TC * LDK];
        float Vs[TC * LDN];
        float blk[BLK_FLOATS];           // A, P, p, beta, w_end, beta*p
    } stage[2];
    float Sn[NR * LDK];                  // Sn[r][c] = tf32(S[col0 + r][c])
    float Tt[NR * LDP];                  // Tt[r][token]
    float Ut[NR * LDP];                  // Ut[r][token]
    float Uw[NR * LDP];                  // Uw[r][token] = w_end[token] * U
    float red[2][TC][16];                // [chunk parity][token][4 * cluster rank + warp pair]
    unsigned long long bar[2];           // stage filled
    unsigned long long rbar[2];          // red[parity] complete (all CTAs of the cluster have stored their sums)
    int failed;
};

__device__ __forceinline__ void ldsm4(float (&r)[4], uint32_t addr) {
    uint32_t x0, x1, x2, x3;
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3) : "r"(addr));
    r[0] = __uint_as_float(x0); r[1] = __uint_as_float(x1); r[2] = __uint_as_float(x2); r[3] = __uint_as_float(x3);
}
// Round to tf32 for an MMA operand in one integer add (finite inputs): the tensor core
// ignores the 13 low mantissa bits, so adding half a tf32 ulp to the magnitude first
// turns its truncation into round-to-nearest (ties away from zero).
__device__ __forceinline__ float tf32q(float x) { return __uint_as_float(__float_as_uint(x) + 0x1000u); }
// store into another CTA of the cluster; the 4 bytes are credited to that CTA's mbarrier,
// and are visible to whoever sees the phase complete
__device__ __forceinline__ void st_async_f32(uint32_t addr, float v, uint32_t bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];\n"
                 ::"r"(addr), "r"(__float_as_uint(v)), "r"(bar) : "memory");
}
// Two adjacent activations, loaded raw: converting at the load would make the thread wait for
// the data there and then; the values are only needed at the end of the chunk.
struct Raw2 { uint32_t lo, hi; };
__device__ __forceinline__ Raw2 ld2_raw(const float *p, size_t i) {
    const uint2 u = *reinterpret_cast<const uint2 *>(p + i);
    return Raw2{u.x, u.y};
}
__device__ __forceinline__ Raw2 ld2_raw(const __nv_bfloat16 *p, size_t i) {
    return Raw2{*reinterpret_cast<const uint32_t *>(p + i), 0u};
}
__device__ __forceinline__ float2 cvt2(const float *, Raw2 r) { return make_float2(__uint_as_float(r.lo), __uint_as_float(r.hi)); }
__device__ __forceinline__ float2 cvt2(const __nv_bfloat16 *, Raw2 r) {
    return make_float2(__uint_as_float(r.lo << 16), __uint_as_float(r.lo & 0xffff0000u));
}
__device__ __forceinline__ void st2(float *p, size_t i, float x, float y) {
    *reinterpret_cast<float2 *>(p + i) = make_float2(x, y);
}
__device__ __forceinline__ void st2(__nv_bfloat16 *p, size_t i, float x, float y) {
    *reinterpret_cast<__nv_bfloat162 *>(p + i) = __floats2bfloat162_rn(x, y);
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
// the mbarrier counts this thread's earlier cp.async copies as one arrival when they land
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory");
}

// Request one chunk.  The copy engine takes tens of cycles per bulk request whatever its size
// (97 row-sized requests per chunk cost 2.6k of a 6.9k-cycle chunk), so a chunk is three bulk
// copies — the packed k tile, the packed q tile, the A / P / gate block — issued by thread 0,
// and its V columns arrive through per-thread 16-byte cp.async copies (one or two per thread)
// that arrive on the same mbarrier: 1 + 256 arrivals per phase.  V rows past the end of the
// sequence are not copied; they keep finite leftovers, which beta = 0 cancels.  No proxy fence:
// the stage was only read since its last fill, and those reads are ordered before this call by
// the CTA barrier at the top of the chunk loop.
template <int NR>
__device__ __forceinline__ void issue_chunk(typename ScanSmem<NR>::Stage &st, uint32_t bar, const float *Y,
                                            size_t tok0, int nvalid, int Cc, int voff, const float *ktile,
                                            const float *qtile, const float *blk, int tid) {
    constexpr int LDN = ScanSmem<NR>::LDN, CPR = NR / 4;  // 16-byte pieces per V row
    if (tid == 0) {
        bc_mbar_expect_tx(bar, 2u * TILE_BYTES + BLK_BYTES);
        bc_copy(bc_smem_u32(st.Ks), ktile, TILE_BYTES, bar);
        bc_copy(bc_smem_u32(st.Qs), qtile, TILE_BYTES, bar);
        bc_copy(bc_smem_u32(st.blk), blk, BLK_BYTES, bar);
    }
#pragma unroll
    for (int e = tid; e < TC * CPR; e += 256) {
        const int row = e / CPR, c = e % CPR;
        if (row < nvalid) cp_async16(bc_smem_u32(&st.Vs[row * LDN + 4 * c]), Y + (tok0 + row) * Cc + voff + 4 * c);
    }
    cp_async_arrive(bar);
}

template <int NR, typename ACT>
__global__ void __launch_bounds__(256, 1) k_delta_chunk_scan(LinArgs a, const float *Y, const float *blocks,
                                                             const float *Kp, const float *Qp, int n_chunks) {
    using SM = ScanSmem<NR>;
    constexpr int LDN = SM::LDN, CS = 128 / NR, NT = NR / 8, NTW = NR / 32;
    extern __shared__ __align__(16) unsigned char smraw[];
    SM &sm = *reinterpret_cast<SM *>(smraw);
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, g = lane >> 2, j = lane & 3;
    const int rank = (int)bc_cluster_rank(), hv = blockIdx.x / CS, b = blockIdx.y;
    const int kh = key_head_of(a, hv), qd = a.nk * 128, vd = a.nv * 128, Cc = 2 * qd + vd;
    const int col0 = rank * NR;
    const int voff = 2 * qd + hv * 128 + col0;
    const float *kt0 = Kp + ((size_t)b * a.nk + kh) * n_chunks * TILE_FLOATS, *qt0 = Qp + ((size_t)b * a.nk + kh) * n_chunks * TILE_FLOATS;
    float *S = a.S + (size_t)b * a.S_stride + (size_t)hv * 128 * 128 + (size_t)col0 * 128;
    const float *blk0 = blocks + ((size_t)b * a.nv + hv) * n_chunks * BLK_FLOATS;
    const int mt = w & 1, wp = w >> 1, ntb = wp * NTW;   // [token][r] tiles: rows 16 mt.., n-tiles ntb..
    const int m0 = 16 * w;                                // rows c of S^T in the state update
    // ldmatrix lane offsets in words: A fragment of a [m][k] tile (rows +0/+8, k +0/+4),
    // B fragments of two k-steps of an [n][k] tile (k +0/+4/+8/+12)
    const int arow = (lane & 7) + 8 * ((lane >> 3) & 1), acol = 4 * (lane >> 4);
    const int brow = lane & 7, bcol = 4 * (lane >> 3);
    const uint32_t sn_b = bc_smem_u32(sm.Sn) + 4u * (uint32_t)((8 * ntb + brow) * LDK + bcol);
    const uint32_t tt_b = bc_smem_u32(sm.Tt) + 4u * (uint32_t)((8 * ntb + brow) * LDP + bcol);
    const uint32_t ut_b = bc_smem_u32(sm.Ut) + 4u * (uint32_t)((8 * ntb + brow) * LDP + bcol);
    const uint32_t uw_all = bc_smem_u32(sm.Uw) + 4u * (uint32_t)(brow * LDP + bcol);

    if (tid == 0) {
        bc_mbar_init(bc_smem_u32(&sm.bar[0]), 257);      // thread 0's expect_tx + one cp.async arrival per thread
        bc_mbar_init(bc_smem_u32(&sm.bar[1]), 257);
        bc_mbar_init(bc_smem_u32(&sm.rbar[0]), 1);
        bc_mbar_init(bc_smem_u32(&sm.rbar[1]), 1);
        bc_mbar_init_fence();
        sm.failed = 0;
    }
    // V rows of a stage that a short last chunk does not fill must hold finite values
    for (int e = tid; e < TC * LDN; e += 256) { sm.stage[0].Vs[e] = 0.0f; sm.stage[1].Vs[e] = 0.0f; }
    // state: st[nt][x] = S[8 nt + 2j + (x & 1)][m0 + g + 8 (x >> 1)] (rows local to this CTA)
    float st[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int x = 0; x < 4; x++) st[nt][x] = S[(8 * nt + 2 * j + (x & 1)) * 128 + m0 + g + 8 * (x >> 1)];
    for (int e = tid; e < NR * 128; e += 256) sm.Sn[(e >> 7) * LDK + (e & 127)] = tf32r(S[e]);
    float nw[NTW][2];
#pragma unroll
    for (int t = 0; t < NTW; t++) {
        nw[t][0] = a.norm_w[col0 + 8 * (ntb + t) + 2 * j];
        nw[t][1] = a.norm_w[col0 + 8 * (ntb + t) + 2 * j + 1];
    }
    bc_fence_proxy_async();                               // the zeros above, before any bulk copy into the stages
    __syncthreads();
    bc_cluster_arrive();                                  // every CTA of the cluster is resident
    bc_cluster_wait();
    issue_chunk<NR>(sm.stage[0], bc_smem_u32(&sm.bar[0]), Y, (size_t)b * a.T, min(TC, a.T), Cc, voff, kt0, qt0, blk0, tid);
    bool ok = true;
    // where this thread's sums of squares go: slot [token][4 rank + wp] in every CTA of the cluster
    uint32_t red_peer[CS], rbar_peer[CS];
#pragma unroll
    for (int rr = 0; rr < CS; rr++) {
        red_peer[rr] = bc_map_rank(&sm.red[0][16 * mt + g][4 * rank + wp], (uint32_t)rr);
        rbar_peer[rr] = bc_map_rank(&sm.rbar[0], (uint32_t)rr);
    }

    for (int n = 0; n < n_chunks; n++) {
        const int buf = n & 1, t0 = n * TC, nvalid = min(TC, a.T - t0);
        const size_t tok0 = (size_t)b * a.T + t0;
        typename SM::Stage &sg = sm.stage[buf];
        __syncthreads();                                  // chunk n-1 is finished with the other stage, Tt, Ut, Sn
        if (n + 1 < n_chunks)
            issue_chunk<NR>(sm.stage[buf ^ 1], bc_smem_u32(&sm.bar[buf ^ 1]), Y, tok0 + TC, min(TC, a.T - t0 - TC), Cc, voff,
                            kt0 + (size_t)(n + 1) * TILE_FLOATS, qt0 + (size_t)(n + 1) * TILE_FLOATS,
                            blk0 + (size_t)(n + 1) * BLK_FLOATS, tid);
        if (tid == 32) bc_mbar_expect_tx(bc_smem_u32(&sm.rbar[buf]), (uint32_t)(TC * 4 * CS * 4));
        // z of this thread's outputs, requested now and used at the end of the chunk
        Raw2 zv[2][NTW];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int i = 16 * mt + g + 8 * h;
#pragma unroll
            for (int t = 0; t < NTW; t++) {
                zv[h][t] = Raw2{0u, 0u};
                if (i < nvalid)
                    zv[h][t] = ld2_raw((const ACT *)a.z, (tok0 + i) * vd + (size_t)hv * 128 + col0 + 8 * (ntb + t) + 2 * j);
            }
        }
        ok = ok && bc_mbar_wait(bc_smem_u32(&sm.bar[buf]), (uint32_t)(n >> 1) & 1u);   // one timeout at most
        const float *aux = sg.blk + BLK_AUX;
        const uint32_t ks_a = bc_smem_u32(sg.Ks) + 4u * (uint32_t)((16 * mt + arow) * LDK + acol);
        const uint32_t qs_a = bc_smem_u32(sg.Qs) + 4u * (uint32_t)((16 * mt + arow) * LDK + acol);
        const uint32_t as_a = bc_smem_u32(sg.blk) + 4u * (uint32_t)((16 * mt + arow) * LDP + acol);
        const uint32_t ps_a = as_a + 4u * BLK_P;

        // ---- K S^T and Q S^T; two accumulators per product shorten the dependent chain
        float sk[2][NTW][4], sq[2][NTW][4];
#pragma unroll
        for (int e = 0; e < 2; e++)
#pragma unroll
            for (int t = 0; t < NTW; t++)
#pragma unroll
                for (int x = 0; x < 4; x++) { sk[e][t][x] = 0.0f; sq[e][t][x] = 0.0f; }
#pragma unroll
        for (int kb = 0; kb < 8; kb++) {                  // 16 contraction indices per step
            float ak[2][4], aq[2][4];
            ldsm4(ak[0], ks_a + 64u * kb); ldsm4(ak[1], ks_a + 64u * kb + 32u);
            ldsm4(aq[0], qs_a + 64u * kb); ldsm4(aq[1], qs_a + 64u * kb + 32u);
#pragma unroll
            for (int t = 0; t < NTW; t++) {
                float bs[4];
                ldsm4(bs, sn_b + 4u * (uint32_t)(8 * t * LDK) + 64u * kb);
                mma_tf32(sk[0][t], ak[0], bs[0], bs[1]);
                mma_tf32(sq[0][t], aq[0], bs[0], bs[1]);
                mma_tf32(sk[1][t], ak[1], bs[2], bs[3]);
                mma_tf32(sq[1][t], aq[1], bs[2], bs[3]);
            }
        }
        // ---- T = beta V - (beta p) K S^T, stored transposed
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int i = 16 * mt + g + 8 * h;
            const float bi = aux[TC + i], bp = aux[3 * TC + i];
#pragma unroll
            for (int t = 0; t < NTW; t++) {
                const int r = 8 * (ntb + t) + 2 * j;
                const float2 v = *reinterpret_cast<const float2 *>(&sg.Vs[i * LDN + r]);
                sm.Tt[r * LDP + i] = tf32q(bi * v.x - bp * (sk[0][t][2 * h] + sk[1][t][2 * h]));
                sm.Tt[(r + 1) * LDP + i] = tf32q(bi * v.y - bp * (sk[0][t][2 * h + 1] + sk[1][t][2 * h + 1]));
            }
        }
        __syncthreads();
        // ---- U = A T (A is unit lower triangular), stored transposed
        {
            float u[NTW][4];
#pragma unroll
            for (int t = 0; t < NTW; t++)
#pragma unroll
                for (int x = 0; x < 4; x++) u[t][x] = 0.0f;
#pragma unroll
            for (int kb = 0; kb < 2; kb++) {
                if (mt == 0 && kb == 1) continue;
                float af[2][4];
                ldsm4(af[0], as_a + 64u * kb); ldsm4(af[1], as_a + 64u * kb + 32u);
#pragma unroll
                for (int t = 0; t < NTW; t++) {
                    float bt[4];
                    ldsm4(bt, tt_b + 4u * (uint32_t)(8 * t * LDP) + 64u * kb);
                    mma_tf32(u[t], af[0], bt[0], bt[1]);
                    mma_tf32(u[t], af[1], bt[2], bt[3]);
                }
            }
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int i = 16 * mt + g + 8 * h;
                const float we = aux[2 * TC + i];
#pragma unroll
                for (int t = 0; t < NTW; t++) {
                    const int r = 8 * (ntb + t) + 2 * j;
                    sm.Ut[r * LDP + i] = tf32q(u[t][2 * h]);
                    sm.Ut[(r + 1) * LDP + i] = tf32q(u[t][2 * h + 1]);
                    sm.Uw[r * LDP + i] = tf32q(we * u[t][2 * h]);
                    sm.Uw[(r + 1) * LDP + i] = tf32q(we * u[t][2 * h + 1]);
                }
            }
        }
        __syncthreads();
        // ---- O = p Q S^T + P U, scaled; this CTA's part of each token's sum of squares
        float o[NTW][4];
        {
            const float p0 = aux[16 * mt + g], p1 = aux[16 * mt + g + 8];
#pragma unroll
            for (int t = 0; t < NTW; t++) {
                o[t][0] = p0 * (sq[0][t][0] + sq[1][t][0]); o[t][1] = p0 * (sq[0][t][1] + sq[1][t][1]);
                o[t][2] = p1 * (sq[0][t][2] + sq[1][t][2]); o[t][3] = p1 * (sq[0][t][3] + sq[1][t][3]);
            }
#pragma unroll
            for (int kb = 0; kb < 2; kb++) {
                if (mt == 0 && kb == 1) continue;
                float af[2][4];
                ldsm4(af[0], ps_a + 64u * kb); ldsm4(af[1], ps_a + 64u * kb + 32u);
#pragma unroll
                for (int t = 0; t < NTW; t++) {
                    float bu[4];
                    ldsm4(bu, ut_b + 4u * (uint32_t)(8 * t * LDP) + 64u * kb);
                    mma_tf32(o[t], af[0], bu[0], bu[1]);
                    mma_tf32(o[t], af[1], bu[2], bu[3]);
                }
            }
#pragma unroll
            for (int h = 0; h < 2; h++) {
                float ss = 0.0f;
#pragma unroll
                for (int t = 0; t < NTW; t++)
#pragma unroll
                    for (int x = 0; x < 2; x++) {
                        const float v = o[t][2 * h + x] * a.out_scale;
                        o[t][2 * h + x] = v;
                        ss += v * v;
                    }
                ss += __shfl_xor_sync(0xffffffffu, ss, 1);
                ss += __shfl_xor_sync(0xffffffffu, ss, 2);
                if (j == 0) {
#pragma unroll
                    for (int rr = 0; rr < CS; rr++)
                        st_async_f32(red_peer[rr] + 4u * (uint32_t)(buf * TC * 16 + 8 * h * 16), ss,
                                     rbar_peer[rr] + 8u * (uint32_t)buf);
                }
            }
        }
        // ---- S^T <- p_end S^T + (diag(w_end) K)^T U, rows m0 .. m0+15
        {
            const float pend = aux[TC - 1];
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int x = 0; x < 4; x++) st[nt][x] *= pend;
#pragma unroll
            for (int kb = 0; kb < 2; kb++) {
                float af[2][4];
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int k0 = 16 * kb + 8 * e;
                    af[e][0] = sg.Ks[(k0 + j) * LDK + m0 + g];
                    af[e][1] = sg.Ks[(k0 + j) * LDK + m0 + g + 8];
                    af[e][2] = sg.Ks[(k0 + j + 4) * LDK + m0 + g];
                    af[e][3] = sg.Ks[(k0 + j + 4) * LDK + m0 + g + 8];
                }
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    float bu[4];
                    ldsm4(bu, uw_all + 4u * (uint32_t)(8 * nt * LDP) + 64u * kb);
                    mma_tf32(st[nt], af[0], bu[0], bu[1]);
                    mma_tf32(st[nt], af[1], bu[2], bu[3]);
                }
            }
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int x = 0; x < 4; x++)
                    sm.Sn[(8 * nt + 2 * j + (x & 1)) * LDK + m0 + g + 8 * (x >> 1)] = tf32q(st[nt][x]);
        }
        // everything of the epilogue that does not need the row sums: o * norm weight * SiLU(z)
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
            for (int t = 0; t < NTW; t++) {
                const float2 zz = cvt2((const ACT *)nullptr, zv[h][t]);
                o[t][2 * h] *= nw[t][0] * silu_fast(zz.x);
                o[t][2 * h + 1] *= nw[t][1] * silu_fast(zz.y);
            }
        ok = ok && bc_mbar_wait(bc_smem_u32(&sm.rbar[buf]), (uint32_t)(n >> 1) & 1u);
        // ---- RMSNorm over the head row, SiLU(z) gate, store
        const bool bad = !ok || *(volatile int *)&sm.failed;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int i = 16 * mt + g + 8 * h;
            if (i >= nvalid) continue;
            float ss = 0.0f;
#pragma unroll
            for (int q = 0; q < CS; q++) {
                const float4 r4 = *reinterpret_cast<const float4 *>(&sm.red[buf][i][4 * q]);
                ss += (r4.x + r4.y) + (r4.z + r4.w);
            }
            const float inv = bad ? NAN : rsqrtf(ss * (1.0f / 128.0f) + a.eps);
            const size_t off = (tok0 + i) * vd + (size_t)hv * 128 + col0;
#pragma unroll
            for (int t = 0; t < NTW; t++)
                st2((ACT *)a.out, off + 8 * (ntb + t) + 2 * j, o[t][2 * h] * inv, o[t][2 * h + 1] * inv);
        }
        if (!ok) sm.failed = 1;
    }
    __syncthreads();
    bc_cluster_arrive();                                  // no CTA leaves while a peer may still store into it
    bc_cluster_wait();
    const bool bad = !ok || sm.failed;
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int x = 0; x < 4; x++)
            S[(8 * nt + 2 * j + (x & 1)) * 128 + m0 + g + 8 * (x >> 1)] = bad ? NAN : st[nt][x];
}

template <int NR, typename ACT>
ornith_status launch_scan(const LinArgs &x, int n_seq, const float *Y, const float *blocks, const float *Kp,
                          const float *Qp, int n_chunks, cudaStream_t s) {
    static bool configured_dev[ORN_MAX_DEVICES] = {};
    bool &configured = configured_dev[orn_device_index()];
    if (!configured) {
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_delta_chunk_scan<NR, ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)sizeof(ScanSmem<NR>)),
                          "delta chunk scan smem opt-in"));
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(x.nv * (128 / NR)), (unsigned)n_seq);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = sizeof(ScanSmem<NR>);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 128 / NR;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    ORN_TRY(orn_check(cudaLaunchKernelEx(&cfg, k_delta_chunk_scan<NR, ACT>, x, Y, blocks, Kp, Qp, n_chunks),
                      "k_delta_chunk_scan launch"));
    return orn_check_launch("k_delta_chunk_scan");
}

}  // namespace

static size_t blocks_part(int nv, int n_seq, int n_chunks) { return align_up((size_t)n_seq * nv * n_chunks * BLK_BYTES, 256); }
static size_t tiles_part(int nk, int n_seq, int n_chunks) { return align_up((size_t)n_seq * nk * n_chunks * TILE_BYTES, 256); }

size_t linear_prefill_tc_blocks_bytes(int nk, int nv, int n_seq, int T) {
    const int n_chunks = (T + TC - 1) / TC;
    return blocks_part(nv, n_seq, n_chunks) + 2 * tiles_part(nk, n_seq, n_chunks);
}

ornith_status launch_linear_prefill_tc(const LinArgs &x, int n_seq, int act_dtype, float *Y, const float *rq,
                                       const float *rk, const float *la, const float *be, float *blocks,
                                       cudaStream_t s) {
    const int n_chunks = (x.T + TC - 1) / TC;
    static bool configured_dev[ORN_MAX_DEVICES] = {};
    bool &configured = configured_dev[orn_device_index()];
    if (!configured) {
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_delta_chunk_prep, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)sizeof(PrepSmem)),
                          "delta chunk prep smem opt-in"));
        configured = true;
    }
    float *Kp = (float *)((char *)blocks + blocks_part(x.nv, n_seq, n_chunks));
    float *Qp = (float *)((char *)Kp + tiles_part(x.nk, n_seq, n_chunks));
    k_delta_chunk_prep<<<dim3((unsigned)n_chunks, (unsigned)x.nk, (unsigned)n_seq), 128, sizeof(PrepSmem), s>>>(
        x, Y, rq, rk, la, be, blocks, Kp, Qp, n_chunks);
    ORN_TRY(orn_check_launch("k_delta_chunk_prep"));
    const bool bf = act_dtype == ORNITH_ACT_BF16;
    // 32-column CTAs (clusters of 4) while they all fit on the SMs at once, else 64-column (clusters of 2)
    if ((long long)x.nv * n_seq * 4 <= 148)
        return bf ? launch_scan<32, __nv_bfloat16>(x, n_seq, Y, blocks, Kp, Qp, n_chunks, s)
                  : launch_scan<32, float>(x, n_seq, Y, blocks, Kp, Qp, n_chunks, s);
    return bf ? launch_scan<64, __nv_bfloat16>(x, n_seq, Y, blocks, Kp, Qp, n_chunks, s)
              : launch_scan<64, float>(x, n_seq, Y, blocks, Kp, Qp, n_chunks, s);
}
