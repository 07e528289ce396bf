// gqa_decode_q8.cu — split-K GQA decode over Q8_0 KV rows on the tensor cores.
//
// Replaces the attend half of ornith_gqa_step (reference: src/ornith_attn.c:111-148)
// for head_dim 256 and up to 16 query heads per KV head.  One CTA = one
// (context split, KV head, sequence); the K and V rows of the split are read from
// HBM exactly once and serve every query head of the group.
//
// Data path per warp (each warp owns every 4th 16-token tile of the split):
//   cp.async 16-byte copies stage the raw Q8_0 rows (272 B each) in a 2-stage ring;
//   the 34-byte blocks are decoded to f16 (code * scale, one rounding) into a
//   16 x 256 tile; ldmatrix feeds mma.sync m16n8k16 (f16 in, f32 accumulate):
//   S = Q K^T with the 16 query-head rows as M, then O += P V with the same tile
//   buffer reused for V.  Online softmax in the log2 domain; the four warps'
//   (m, l, O) are merged in shared memory and one partial per CTA goes to the
//   scratch the combine kernel reads.
//
// Precision: q is pre-scaled per head by a power of two into [-1, 1] and rounded
// to f16 (11-bit significand, the same as tf32); decoded K/V elements carry one
// f16 rounding; probabilities are scaled by 2^8 before the f16 rounding so small
// weights stay in the normal range.  Accumulation is f32.
#include <stdlib.h>

#include "full_attn.cuh"

namespace {

constexpr int HD = 256;
constexpr int ROWB = 272;                 // bytes of one Q8_0 row of 256 values
constexpr int TILE = 16;                  // tokens per MMA tile
constexpr int LDH = 264;                  // f16 tile row stride (halves): 528 B, conflict-free ldmatrix
constexpr int NWARP = 4;
constexpr int RAW_TILE = TILE * ROWB;     // 4352
constexpr int QS_BYTES = 16 * LDH * 2;    // 8448
constexpr int WARP_RAW = 2 * 2 * RAW_TILE;            // 2 stages x (K, V)
constexpr int WARP_BYTES = WARP_RAW + TILE * LDH * 2; // + f16 tile = 25856
constexpr int SMEM_BYTES = QS_BYTES + NWARP * WARP_BYTES;
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

// Decode one staged tile (16 rows x 8 blocks of {f16 scale, 32 int8}) to f16.
// A lane handles 4 (row, block) units; its block index is lane >> 2, so the
// 2-byte misalignment of the codes (even blocks) is a per-lane constant shift,
// and the 8 lanes of one 128-bit store phase hit 8 distinct 16-byte bank groups
// (rows 0-3 x two neighbouring blocks).
__device__ __forceinline__ void decode_tile(const unsigned char *raw, __half *th, int lane) {
    const int blk = lane >> 2;
    const bool even = (blk & 1) == 0;
    const int start = 34 * blk - (even ? 0 : 2);          // 4-byte aligned
    const uint32_t sh = even ? 16u : 32u;
    const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int row = (lane & 3) + 4 * i;
        const uint32_t *w = reinterpret_cast<const uint32_t *>(raw + row * ROWB + start);
        uint32_t wd[9];
#pragma unroll
        for (int k = 0; k < 9; k++) wd[k] = w[k];
        const unsigned short sb = even ? (unsigned short)(wd[0] & 0xffffu) : (unsigned short)(wd[0] >> 16);
        const __half d = __ushort_as_half(sb);
        const __half2 d2 = __halves2half2(d, d);
        uint32_t outw[16];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const uint32_t cw = __funnelshift_rc(wd[k], wd[k + 1], sh) ^ 0x80808080u;
            uint32_t h01 = __byte_perm(cw, 0x64646464u, 0x4140);     // 1024 + (code + 128)
            uint32_t h23 = __byte_perm(cw, 0x64646464u, 0x4342);
            __half2 a = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&h01), bias), d2);
            __half2 b = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&h23), bias), d2);
            outw[2 * k] = *reinterpret_cast<uint32_t *>(&a);
            outw[2 * k + 1] = *reinterpret_cast<uint32_t *>(&b);
        }
        uint4 *dst = reinterpret_cast<uint4 *>(th + row * LDH + blk * 32);
#pragma unroll
        for (int k = 0; k < 4; k++) dst[k] = make_uint4(outw[4 * k], outw[4 * k + 1], outw[4 * k + 2], outw[4 * k + 3]);
    }
}

__global__ void __launch_bounds__(128, 2) k_gqa_decode_q8_mma(DecodeArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float rowscale_s[16];
    __shared__ float m_s[NWARP][16], l_s[NWARP][16];
    __half *Q_s = reinterpret_cast<__half *>(smem);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    unsigned char *wbase = smem + QS_BYTES + warp * WARP_BYTES;
    __half *th = reinterpret_cast<__half *>(wbase + WARP_RAW);

    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, nkv = a.kv.nkv;
    const int G = a.nh / nkv;
    const int64_t base = a.kv.seq_off[b];
    const int cap = (int)(a.kv.seq_off[b + 1] - base);
    const int len0 = a.kv_len[b];
    if (len0 >= cap) return;
    const int L = len0 + 1;
    const int t0 = split * a.tokens_per_split, t1 = min(L, t0 + a.tokens_per_split);
    float *part0 = a.part + (((size_t)b * a.nh + (size_t)kvh * G) * a.nsplit + split) * (HD + 2);
    const size_t part_stride = (size_t)a.nsplit * (HD + 2);             // next head of the group
    if (t0 >= L) {
        if (tid < G) { part0[tid * part_stride] = -INFINITY; part0[tid * part_stride + 1] = 0.0f; }
        return;
    }

    // ---- query rows -> f16, each scaled by a power of two into [-1, 1] ----------------
    for (int r = warp * 4; r < warp * 4 + 4; r++) {
        float v[8];
        float mx = 0.0f;
        if (r < G) {
            const float *q = a.q_prep + ((size_t)b * a.nh + (size_t)kvh * G + r) * HD + lane * 8;
#pragma unroll
            for (int i = 0; i < 8; i++) { v[i] = q[i]; mx = fmaxf(mx, fabsf(v[i])); }
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = 0.0f;
        }
        mx = warp_max(mx);
        int e = 0;
        if (mx > 0.0f && mx < INFINITY) (void)frexpf(mx, &e);            // mx = f * 2^e, f in [0.5, 1)
        const float down = exp2f((float)-e);
        uint4 packed = make_uint4(pack_h2(v[0] * down, v[1] * down), pack_h2(v[2] * down, v[3] * down),
                                  pack_h2(v[4] * down, v[5] * down), pack_h2(v[6] * down, v[7] * down));
        *reinterpret_cast<uint4 *>(Q_s + r * LDH + lane * 8) = packed;
        if (lane == 0) rowscale_s[r] = (r < G) ? a.scale * exp2f((float)e) * LOG2E : 0.0f;
    }
    __syncthreads();

    const int ntiles = (t1 - t0 + TILE - 1) / TILE;
    const size_t row_stride = (size_t)nkv * ROWB;
    const unsigned char *Kbase = a.kv.K + ((size_t)base * nkv + kvh) * ROWB;
    const unsigned char *Vbase = a.kv.V + ((size_t)base * nkv + kvh) * ROWB;

    auto issue = [&](int tile, int stage) {
        const int tok0 = t0 + tile * TILE;
        unsigned char *dK = wbase + (stage * 2 + 0) * RAW_TILE, *dV = wbase + (stage * 2 + 1) * RAW_TILE;
        for (int c = lane; c < TILE * 17; c += 32) {
            const int row = c / 17, ch = c - row * 17, tok = tok0 + row;
            const bool ok = tok < t1;
            const size_t off = ok ? (size_t)tok * row_stride + ch * 16 : 0;
            cp_async16(smem_u32(dK + row * ROWB + ch * 16), Kbase + off, ok ? 16 : 0);
            cp_async16(smem_u32(dV + row * ROWB + ch * 16), Vbase + off, ok ? 16 : 0);
        }
    };

    float o[32][4];
#pragma unroll
    for (int i = 0; i < 32; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m2[2] = {-INFINITY, -INFINITY}, lsum[2] = {0.0f, 0.0f};
    const float rs0 = rowscale_s[lane >> 2], rs1 = rowscale_s[(lane >> 2) + 8];
    const int j2 = (lane & 3) * 2;

    // ldmatrix lane addresses (bytes, relative to the tile / Q base)
    const uint32_t q_addr = smem_u32(Q_s) + ((lane & 15) * LDH + (lane >> 4) * 8) * 2;
    const uint32_t k_addr = smem_u32(th) + (((lane & 7) + (lane >> 4) * 8) * LDH + ((lane >> 3) & 1) * 8) * 2;
    const uint32_t v_addr = smem_u32(th) + (((lane & 7) + ((lane >> 3) & 1) * 8) * LDH + (lane >> 4) * 8) * 2;

    int it = warp;
    if (it < ntiles) issue(it, 0);
    cp_async_commit();
    for (int n = 0; it < ntiles; it += NWARP, n++) {
        if (it + NWARP < ntiles) issue(it + NWARP, (n + 1) & 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncwarp();
        const unsigned char *rawK = wbase + ((n & 1) * 2 + 0) * RAW_TILE, *rawV = rawK + RAW_TILE;
        const int tok0 = t0 + it * TILE;

        // ---- S = Q K^T -----------------------------------------------------------------
        decode_tile(rawK, th, lane);
        __syncwarp();
        float s0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, s1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        {   // four independent accumulator chains (even / odd k-steps), summed at the end
            float e0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, e1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int ks = 0; ks < 16; ks += 2) {
                uint32_t A[4], B[4], A2[4], B2[4];
                ldsm_x4(A, q_addr + ks * 32);
                ldsm_x4(B, k_addr + ks * 32);
                ldsm_x4(A2, q_addr + ks * 32 + 32);
                ldsm_x4(B2, k_addr + ks * 32 + 32);
                mma16816(s0, A, B[0], B[1]);
                mma16816(s1, A, B[2], B[3]);
                mma16816(e0, A2, B2[0], B2[1]);
                mma16816(e1, A2, B2[2], B2[3]);
            }
#pragma unroll
            for (int c = 0; c < 4; c++) { s0[c] += e0[c]; s1[c] += e1[c]; }
        }
        // ---- online softmax, log2 domain; rows r = lane/4 and r + 8 ----------------------
        const bool ok0 = tok0 + j2 < t1, ok1 = tok0 + j2 + 1 < t1, ok2 = tok0 + 8 + j2 < t1, ok3 = tok0 + 9 + j2 < t1;
        float x[2][4];
        x[0][0] = ok0 ? s0[0] * rs0 : -INFINITY; x[0][1] = ok1 ? s0[1] * rs0 : -INFINITY;
        x[0][2] = ok2 ? s1[0] * rs0 : -INFINITY; x[0][3] = ok3 ? s1[1] * rs0 : -INFINITY;
        x[1][0] = ok0 ? s0[2] * rs1 : -INFINITY; x[1][1] = ok1 ? s0[3] * rs1 : -INFINITY;
        x[1][2] = ok2 ? s1[2] * rs1 : -INFINITY; x[1][3] = ok3 ? s1[3] * rs1 : -INFINITY;
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            float mx = fmaxf(fmaxf(x[h][0], x[h][1]), fmaxf(x[h][2], x[h][3]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float mn = fmaxf(m2[h], mx);                // finite: token tok0 is always valid
            corr[h] = exp2f(m2[h] - mn);
            m2[h] = mn;
            float ps = 0.0f;
#pragma unroll
            for (int c = 0; c < 4; c++) { x[h][c] = exp2f(x[h][c] - mn); ps += x[h][c]; }
            lsum[h] = lsum[h] * corr[h] + ps;                 // per-thread partial; quad-reduced at the end
        }
        if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
            for (int i = 0; i < 32; i++) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
        }
        uint32_t P[4];
        P[0] = pack_h2(x[0][0] * 256.0f, x[0][1] * 256.0f);
        P[1] = pack_h2(x[1][0] * 256.0f, x[1][1] * 256.0f);
        P[2] = pack_h2(x[0][2] * 256.0f, x[0][3] * 256.0f);
        P[3] = pack_h2(x[1][2] * 256.0f, x[1][3] * 256.0f);

        // ---- O += P V (the f16 tile buffer is reused for V) ------------------------------
        __syncwarp();
        decode_tile(rawV, th, lane);
        __syncwarp();
#pragma unroll
        for (int np = 0; np < 16; np++) {
            uint32_t B[4];
            ldsm_x4_trans(B, v_addr + np * 32);
            mma16816(o[2 * np], P, B[0], B[1]);
            mma16816(o[2 * np + 1], P, B[2], B[3]);
        }
        __syncwarp();                                         // stage and tile free for the next round
    }
    cp_async_wait<0>();
    __syncwarp();

    // ---- merge the four warps, write one partial per (head, split) ---------------------------
#pragma unroll
    for (int h = 0; h < 2; h++) {
        lsum[h] += __shfl_xor_sync(0xffffffffu, lsum[h], 1);
        lsum[h] += __shfl_xor_sync(0xffffffffu, lsum[h], 2);
    }
    float *Ow = reinterpret_cast<float *>(wbase);             // [16][256] f32 over this warp's own buffers
    const int r0 = lane >> 2;
#pragma unroll
    for (int i = 0; i < 32; i++) {
        *reinterpret_cast<float2 *>(Ow + r0 * HD + i * 8 + j2) = make_float2(o[i][0], o[i][1]);
        *reinterpret_cast<float2 *>(Ow + (r0 + 8) * HD + i * 8 + j2) = make_float2(o[i][2], o[i][3]);
    }
    if ((lane & 3) == 0) {
        m_s[warp][r0] = m2[0]; m_s[warp][r0 + 8] = m2[1];
        l_s[warp][r0] = lsum[0]; l_s[warp][r0 + 8] = lsum[1];
    }
    __syncthreads();
    for (int r = 0; r < G; r++) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NWARP; w++) if (l_s[w][r] > 0.0f) M = fmaxf(M, m_s[w][r]);
        float ww[NWARP], Lt = 0.0f;
#pragma unroll
        for (int w = 0; w < NWARP; w++) {
            ww[w] = (l_s[w][r] > 0.0f) ? exp2f(m_s[w][r] - M) : 0.0f;
            Lt += l_s[w][r] * ww[w];
        }
        float *part = part0 + r * part_stride;
        if (tid == 0) { part[0] = M * LN2; part[1] = Lt; }
        for (int d = tid; d < HD; d += 128) {
            float acc = 0.0f;
#pragma unroll
            for (int w = 0; w < NWARP; w++)
                acc += ww[w] * reinterpret_cast<const float *>(smem + QS_BYTES + w * WARP_BYTES)[r * HD + d];
            part[2 + d] = acc * (1.0f / 256.0f);
        }
    }
}

// =============================================================================
// Variant for groups of up to 8 query heads: tokens on the MMA M axis
// =============================================================================
//
// S^T[token, head] = K Q^T and O^T[dim, head] += V^T P^T, so the 8 heads fill the
// N = 8 axis exactly (no padded rows), the output accumulator is 64 registers and
// the whole query group lives in registers as B fragments.  K never touches a
// second buffer: each lane converts the 8 consecutive codes it needs per 32-value
// block straight into A fragments (the contraction index is permuted the same
// way on the query side, which leaves the dot product unchanged).  V is decoded
// into the warp's f16 tile and read back transposed with ldmatrix.  One raw stage
// per warp (17 KB of shared memory in all) lets three CTAs share an SM; the next
// tile's K rows are requested right after the score loop and its V rows right
// after the V decode.
constexpr int W3_RAW = 2 * RAW_TILE;                    // K rows, V rows
constexpr int W3_BYTES = W3_RAW + TILE * LDH * 2;       // + f16 tile = 17152
constexpr int SMEM3_BYTES = NWARP * W3_BYTES;

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}

// 4 int8 codes (one word) -> two f16x2 words scaled by d2
__device__ __forceinline__ void cvt4(uint32_t w, __half2 d2, uint32_t &x01, uint32_t &x23) {
    const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);
    const uint32_t cw = w ^ 0x80808080u;
    uint32_t h01 = __byte_perm(cw, 0x64646464u, 0x4140), h23 = __byte_perm(cw, 0x64646464u, 0x4342);
    __half2 a = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&h01), bias), d2);
    __half2 b = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&h23), bias), d2);
    x01 = *reinterpret_cast<uint32_t *>(&a);
    x23 = *reinterpret_cast<uint32_t *>(&b);
}

// the 8 codes at in-block offset 8j of block B of one staged row, and the block scale
template <int B>
__device__ __forceinline__ void load_block8(const unsigned char *row, int j, uint32_t &lo, uint32_t &hi, __half2 &d2) {
    const __half d = __ushort_as_half(*reinterpret_cast<const unsigned short *>(row + 34 * B));
    d2 = __halves2half2(d, d);
    if (B % 2 == 0) {            // codes start 2 bytes past a word boundary
        const uint32_t *w = reinterpret_cast<const uint32_t *>(row + 34 * B + 8 * j);
        const uint32_t w0 = w[0], w1 = w[1], w2 = w[2];
        lo = __funnelshift_r(w0, w1, 16);
        hi = __funnelshift_r(w1, w2, 16);
    } else {
        const uint32_t *w = reinterpret_cast<const uint32_t *>(row + 34 * B + 2 + 8 * j);
        lo = w[0];
        hi = w[1];
    }
}

template <int B>
__device__ __forceinline__ void qk_block(const unsigned char *r0p, const unsigned char *r1p, int j,
                                         const uint32_t (&qf)[8][4], float (&s)[4], float (&e)[4]) {
    uint32_t lo0, hi0, lo1, hi1;
    __half2 d0, d1;
    load_block8<B>(r0p, j, lo0, hi0, d0);
    load_block8<B>(r1p, j, lo1, hi1, d1);
    uint32_t A0[4], A1[4];
    cvt4(lo0, d0, A0[0], A0[2]);     // row r:   k = 2j,2j+1 | 2j+8,2j+9 of the first k-step
    cvt4(lo1, d1, A0[1], A0[3]);     // row r+8
    cvt4(hi0, d0, A1[0], A1[2]);     // second k-step of the block
    cvt4(hi1, d1, A1[1], A1[3]);
    mma16816(s, A0, qf[B][0], qf[B][1]);
    mma16816(e, A1, qf[B][2], qf[B][3]);
}

__device__ __forceinline__ void issue_rows(unsigned char *dst, const unsigned char *src_base, size_t row_stride,
                                           int tok0, int t1, int lane) {
    // lane pair (2r, 2r+1) copies row r: 9 + 8 chunks of 16 bytes
    const int row = lane >> 1, first = (lane & 1) * 9, cnt = 9 - (lane & 1);
    const int tok = tok0 + row;
    const bool ok = tok < t1;
    const unsigned char *src = src_base + (ok ? (size_t)tok * row_stride : 0) + first * 16;
    uint32_t d = smem_u32(dst + row * ROWB + first * 16);
    for (int c = 0; c < cnt; c++) cp_async16(d + c * 16, src + (ok ? c * 16 : 0), ok ? 16 : 0);
}

__global__ void __launch_bounds__(128, 3) k_gqa_decode_q8_tok(DecodeArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float m_s[NWARP][8], l_s[NWARP][8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    unsigned char *wbase = smem + warp * W3_BYTES;
    unsigned char *rawK = wbase, *rawV = wbase + RAW_TILE;
    __half *th = reinterpret_cast<__half *>(wbase + W3_RAW);

    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, nkv = a.kv.nkv;
    const int G = a.nh / nkv;
    const int64_t base = a.kv.seq_off[b];
    const int cap = (int)(a.kv.seq_off[b + 1] - base);
    const int len0 = a.kv_len[b];
    if (len0 >= cap) return;
    const int L = len0 + 1;
    const int t0 = split * a.tokens_per_split, t1 = min(L, t0 + a.tokens_per_split);
    float *part0 = a.part + (((size_t)b * a.nh + (size_t)kvh * G) * a.nsplit + split) * (HD + 2);
    const size_t part_stride = (size_t)a.nsplit * (HD + 2);
    if (t0 >= L) {
        if (tid < G) { part0[tid * part_stride] = -INFINITY; part0[tid * part_stride + 1] = 0.0f; }
        return;
    }
    const int r = lane >> 2, j = lane & 3;

    // ---- query group -> B fragments in registers: lane (head r, quarter j) keeps q[r][32b + 8j .. +7]
    uint32_t qf[8][4];
    float rs_mine;
    {
        float v[8][8];
        float mx = 0.0f;
        const float *q = a.q_prep + ((size_t)b * a.nh + (size_t)kvh * G + r) * HD + 8 * j;
#pragma unroll
        for (int bb = 0; bb < 8; bb++)
#pragma unroll
            for (int i = 0; i < 8; i++) {
                v[bb][i] = (r < G) ? q[32 * bb + i] : 0.0f;
                mx = fmaxf(mx, fabsf(v[bb][i]));
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        int e = 0;
        if (mx > 0.0f && mx < INFINITY) (void)frexpf(mx, &e);
        const float down = exp2f((float)-e);
#pragma unroll
        for (int bb = 0; bb < 8; bb++)
#pragma unroll
            for (int i = 0; i < 4; i++) qf[bb][i] = pack_h2(v[bb][2 * i] * down, v[bb][2 * i + 1] * down);
        rs_mine = (r < G) ? a.scale * exp2f((float)e) * LOG2E : 0.0f;
    }
    // score scale of the two heads this lane sees as accumulator columns (2j, 2j+1)
    const float rsA = __shfl_sync(0xffffffffu, rs_mine, (2 * j) * 4);
    const float rsB = __shfl_sync(0xffffffffu, rs_mine, (2 * j + 1) * 4);

    const int ntiles = (t1 - t0 + TILE - 1) / TILE;
    const size_t row_stride = (size_t)nkv * ROWB;
    const unsigned char *Kbase = a.kv.K + ((size_t)base * nkv + kvh) * ROWB;
    const unsigned char *Vbase = a.kv.V + ((size_t)base * nkv + kvh) * ROWB;

    float o[16][4];
#pragma unroll
    for (int i = 0; i < 16; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float mA = -INFINITY, mB = -INFINITY, lA = 0.0f, lB = 0.0f;
    const unsigned char *r0p = rawK + r * ROWB, *r1p = r0p + 8 * ROWB;
    const uint32_t v_addr = smem_u32(th) + (((lane & 7) + (lane >> 4) * 8) * LDH) * 2 + ((lane >> 3) & 1) * 16;

    int it = warp;
    if (it < ntiles) issue_rows(rawK, Kbase, row_stride, t0 + it * TILE, t1, lane);
    cp_async_commit();
    if (it < ntiles) issue_rows(rawV, Vbase, row_stride, t0 + it * TILE, t1, lane);
    cp_async_commit();
    for (; it < ntiles; it += NWARP) {
        const int tok0 = t0 + it * TILE;
        const bool more = it + NWARP < ntiles;
        cp_async_wait<1>();                                   // this tile's K rows have landed
        __syncwarp();
        // ---- S^T = K Q^T, two accumulator chains ---------------------------------------
        float s[4] = {0.0f, 0.0f, 0.0f, 0.0f}, e2[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        qk_block<0>(r0p, r1p, j, qf, s, e2); qk_block<1>(r0p, r1p, j, qf, s, e2);
        qk_block<2>(r0p, r1p, j, qf, s, e2); qk_block<3>(r0p, r1p, j, qf, s, e2);
        qk_block<4>(r0p, r1p, j, qf, s, e2); qk_block<5>(r0p, r1p, j, qf, s, e2);
        qk_block<6>(r0p, r1p, j, qf, s, e2); qk_block<7>(r0p, r1p, j, qf, s, e2);
        __syncwarp();                                         // every lane is done with the K rows
        if (more) issue_rows(rawK, Kbase, row_stride, tok0 + NWARP * TILE, t1, lane);
        cp_async_commit();

        // ---- online softmax over tokens (rows r, r+8); columns = heads 2j, 2j+1 -----------
        const bool ok0 = tok0 + r < t1, ok1 = tok0 + r + 8 < t1;
        float x00 = ok0 ? (s[0] + e2[0]) * rsA : -INFINITY, x01 = ok0 ? (s[1] + e2[1]) * rsB : -INFINITY;
        float x10 = ok1 ? (s[2] + e2[2]) * rsA : -INFINITY, x11 = ok1 ? (s[3] + e2[3]) * rsB : -INFINITY;
        float cA = fmaxf(x00, x10), cB = fmaxf(x01, x11);
#pragma unroll
        for (int sft = 4; sft <= 16; sft <<= 1) {
            cA = fmaxf(cA, __shfl_xor_sync(0xffffffffu, cA, sft));
            cB = fmaxf(cB, __shfl_xor_sync(0xffffffffu, cB, sft));
        }
        const float nA = fmaxf(mA, cA), nB = fmaxf(mB, cB);   // finite: token tok0 is valid
        const float corrA = exp2f(mA - nA), corrB = exp2f(mB - nB);
        mA = nA; mB = nB;
        x00 = exp2f(x00 - nA); x10 = exp2f(x10 - nA); x01 = exp2f(x01 - nB); x11 = exp2f(x11 - nB);
        lA = lA * corrA + x00 + x10;                          // per-lane partial over its two rows
        lB = lB * corrB + x01 + x11;
        if (__any_sync(0xffffffffu, corrA != 1.0f || corrB != 1.0f)) {
#pragma unroll
            for (int i = 0; i < 16; i++) { o[i][0] *= corrA; o[i][1] *= corrB; o[i][2] *= corrA; o[i][3] *= corrB; }
        }
        // P^T as the B operand: transpose the two 8x8 (token x head) blocks across the warp
        const uint32_t pb0 = movmatrix_trans(pack_h2(x00 * 256.0f, x01 * 256.0f));
        const uint32_t pb1 = movmatrix_trans(pack_h2(x10 * 256.0f, x11 * 256.0f));

        // ---- O^T += V^T P^T -----------------------------------------------------------------
        cp_async_wait<1>();                                   // this tile's V rows have landed
        __syncwarp();
        decode_tile(rawV, th, lane);
        __syncwarp();
        if (more) issue_rows(rawV, Vbase, row_stride, tok0 + NWARP * TILE, t1, lane);
        cp_async_commit();
#pragma unroll
        for (int mt = 0; mt < 16; mt++) {
            uint32_t A[4];
            ldsm_x4_trans(A, v_addr + mt * 32);
            mma16816(o[mt], A, pb0, pb1);
        }
        __syncwarp();                                         // f16 tile free for the next round
    }
    cp_async_wait<0>();
    __syncwarp();

    // ---- merge the four warps, one partial per (head, split) -------------------------------
#pragma unroll
    for (int sft = 4; sft <= 16; sft <<= 1) {
        lA += __shfl_xor_sync(0xffffffffu, lA, sft);
        lB += __shfl_xor_sync(0xffffffffu, lB, sft);
    }
    float *Ow = reinterpret_cast<float *>(wbase);             // [8 heads][256] f32 over this warp's buffers
#pragma unroll
    for (int mt = 0; mt < 16; mt++) {
        Ow[(2 * j) * HD + mt * 16 + r] = o[mt][0];
        Ow[(2 * j + 1) * HD + mt * 16 + r] = o[mt][1];
        Ow[(2 * j) * HD + mt * 16 + r + 8] = o[mt][2];
        Ow[(2 * j + 1) * HD + mt * 16 + r + 8] = o[mt][3];
    }
    if (r == 0) {
        m_s[warp][2 * j] = mA; m_s[warp][2 * j + 1] = mB;
        l_s[warp][2 * j] = lA; l_s[warp][2 * j + 1] = lB;
    }
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
        if (tid == 0) { part[0] = M * LN2; part[1] = Lt; }
        for (int d = tid; d < HD; d += 128) {
            float acc = 0.0f;
#pragma unroll
            for (int w = 0; w < NWARP; w++)
                acc += ww[w] * reinterpret_cast<const float *>(smem + w * W3_BYTES)[h * HD + d];
            part[2 + d] = acc * (1.0f / 256.0f);
        }
    }
}

}  // namespace

bool gqa_decode_q8_mma_supported(const KvView &kv, int nh) {
    return kv.mode == ORNITH_KV_Q8_0 && kv.hd == HD && nh % kv.nkv == 0 && nh / kv.nkv <= 16 &&
           ((uintptr_t)kv.K % 16) == 0 && ((uintptr_t)kv.V % 16) == 0;
}

// ORNITH_CUDA_DECODE_VARIANT: unset = the raw-fragment kernel (groups of 9-16 heads as two CTAs of 8 heads per KV
// head: 0.51 of HBM bandwidth at 32 query / 2 KV heads against 0.40 for the f16-tile kernel); tile = the variant
// that decodes V into an f16 tile; mma = the f16-tile kernel for groups of 9-16 heads
static int decode_variant() {
    static int variant = -1;
    if (variant < 0) { const char *e = getenv("ORNITH_CUDA_DECODE_VARIANT"); variant = !e ? 0 : (e[0] == 't' ? 1 : (e[0] == 'm' ? 3 : 0)); }
    return variant;
}

// ORNITH_CUDA_DECODE_SCHED=grid keeps the grid of fixed splits for the raw-fragment kernel (A/B comparison)
bool gqa_decode_q8_raw_balanced(const KvView &kv, int nh) {
    static int grid_sched = -1;
    if (grid_sched < 0) { const char *e = getenv("ORNITH_CUDA_DECODE_SCHED"); grid_sched = (e && e[0] == 'g') ? 1 : 0; }
    if (grid_sched || !gqa_decode_q8_mma_supported(kv, nh)) return false;
    return decode_variant() == 0 || (decode_variant() == 3 && nh / kv.nkv <= 8);
}

ornith_status launch_gqa_decode_q8_mma(const DecodeArgs &a, int n_seq, cudaStream_t st, bool *merged) {
    *merged = false;
    static bool configured_dev[ORN_MAX_DEVICES] = {};
    bool &configured = configured_dev[orn_device_index()];
    if (!configured) {
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_gqa_decode_q8_mma, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               SMEM_BYTES), "gqa decode smem opt-in"));
        configured = true;
    }
    static bool configured3_dev[ORN_MAX_DEVICES] = {};
    bool &configured3 = configured3_dev[orn_device_index()];
    if (!configured3) {
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_gqa_decode_q8_tok, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               SMEM3_BYTES), "gqa decode smem opt-in"));
        configured3 = true;
    }
    dim3 grid(a.nsplit, a.kv.nkv, n_seq);
    const int variant = decode_variant();
    const int use_tile = variant == 1;
    if (a.nh / a.kv.nkv <= 8 || variant != 3) {          // (variant mma: groups of 9-16 heads on k_gqa_decode_q8_mma below)
        if (!use_tile) return launch_gqa_decode_q8_raw(a, n_seq, st, merged);
        k_gqa_decode_q8_tok<<<grid, 128, SMEM3_BYTES, st>>>(a);
        return orn_check_launch("k_gqa_decode_q8_tok");
    }
    k_gqa_decode_q8_mma<<<grid, 128, SMEM_BYTES, st>>>(a);
    return orn_check_launch("k_gqa_decode_q8_mma");
}
