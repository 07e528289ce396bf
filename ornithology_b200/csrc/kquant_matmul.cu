// kquant_matmul.cu — quantised weights x Q8_K activations on the integer tensor cores, bit for bit the engine's
// integer path.
//
// Replaces qdot_vec_dot as matmul_batch_q drives it (reference: src/ornith_rforward.c:138-192) for the three
// weight types that have an integer dot (qdot_can, src/ornith_qdot.c:167-177): Q4_K (vec_dot_q4_K :75-105),
// Q6_K (vec_dot_q6_K :109-141) and Q8_0 (vec_dot_q8_0 :144-163).
//
// The engine's arithmetic is integer up to one f32 product per super-block of 256 inputs (Q8_0: per block of 32):
// codes times activation codes summed over a sub-block, times a small integer sub-block scale, summed over the
// super-block, then (activation scale x weight scale) x (float)sum added to an f32 total, super-blocks in order.
// mma.sync with int8 operands and int32 sums is exact, so the kernel reproduces the engine's result bit for bit:
// a sub-block is one MMA (k = 32 for Q4_K / Q8_0, k = 16 for Q6_K, whose scales cover 16 inputs), its int32 tile
// is weighted by the sub-block scale with integer multiply-adds, and the f32 part is evaluated with the engine's
// association and without contraction.
//
//   weights      stay in HBM as the GGUF bytes.  A CTA owns 64 rows; per super-block one tensor copy brings the 64
//                row pieces (144 / 272 bytes; Q6_K: a 240-byte window around the 210 bytes, which start on a
//                2-byte boundary) into one stage of shared memory, up to eight stages on mbarriers.
//   unpacking    lane (g, j) of a warp builds the A operand of rows g and g + 8 for inputs 4 j .. 4 j + 3 of a
//                k-step straight from the packed bytes: nibble masks for Q4_K (codes 0..15, unsigned operand),
//                nibble + 2-bit planes and a per-byte -32 for Q6_K, a byte permute for Q8_0's 2-byte offset.
//                One unpacked operand feeds the MMAs of all token tiles of the pass.
//   activations  the Q8_K image of k_q8k_quantize: codes in B-operand order, so a lane's operand is one word.
//   Q4_K minimums  sum_j min_j x (sum of the activation codes of sub-block j) is itself a small matrix product: the
//                8 minimums of a row as an unsigned A operand, the sums split into low (unsigned) and high (signed)
//                bytes as two B operands: two more MMAs per tile instead of 32 multiply-adds per thread.
//
// Prompts are walked in passes of 128 tokens (grid.y; the weights are then re-read from L2).  Shapes the tensor copy
// cannot address (rows that do not start on 16-byte boundaries: Q6_K with n_in not a multiple of 2048) take a plain
// kernel with the same arithmetic.
#include <cuda.h>
#include <cuda_fp16.h>
#include <math.h>

#include "qproj.cuh"
#include "tcgen05.cuh"          // the tensor-map encoder entry point, bounded mbarrier waits

namespace {

constexpr int QK = 256;

enum { T_Q4K = 0, T_Q6K = 1, T_Q80 = 2 };
template <int TYPE> struct Fmt;
template <> struct Fmt<T_Q4K> { static constexpr int BLOCK = 144, BOX = 144; };
template <> struct Fmt<T_Q6K> { static constexpr int BLOCK = 210, BOX = 240; };   // 240: rows 60 words apart, no bank conflicts
template <> struct Fmt<T_Q80> { static constexpr int BLOCK = 272, BOX = 272; };

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tensor_copy_rows(uint32_t dst, const CUtensorMap *map, int word0, int row0, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(word0), "r"(row0) : "memory");
}

// d = a . b for one k-step, int32 sums from zero.  k = 32: a = {row g k 0..15 part, row g+8, row g k 16..31 part, row g+8}
#define ORN_MMA_K32(NAME, TA, TB)                                                                                   \
    __device__ __forceinline__ void NAME(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {           \
        asm("mma.sync.aligned.m16n8k32.row.col.s32." TA "." TB ".s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, " \
                     "{%10,%10,%10,%10};\n"                                                                          \
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])                                               \
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(0));                       \
    }
#define ORN_MMA_K16(NAME, TA, TB)                                                                                   \
    __device__ __forceinline__ void NAME(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {                      \
        asm("mma.sync.aligned.m16n8k16.row.col.s32." TA "." TB ".s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, "       \
                     "{%7,%7,%7,%7};\n"                                                                              \
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])                                               \
                     : "r"(a0), "r"(a1), "r"(b0), "r"(0));                                                          \
    }
ORN_MMA_K32(mma_k32_u8s8, "u8", "s8")
ORN_MMA_K32(mma_k32_s8s8, "s8", "s8")
ORN_MMA_K16(mma_k16_s8s8, "s8", "s8")
ORN_MMA_K16(mma_k16_u8u8, "u8", "u8")
ORN_MMA_K16(mma_k16_u8s8, "u8", "s8")

typedef const unsigned char *smem_ptr;
__device__ __forceinline__ uint32_t lds32(smem_ptr p) { return *reinterpret_cast<const uint32_t *>(p); }
// four bytes from a 2-byte-aligned shared address
__device__ __forceinline__ uint32_t lds32_any(smem_ptr p) {
    const uint32_t off = (uint32_t)(uintptr_t)p & 3u;
    smem_ptr base = p - off;
    return __funnelshift_r(lds32(base), lds32(base + 4), off * 8);
}
__device__ __forceinline__ float f16_bits_to_f32(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }
__device__ __forceinline__ int sbyte(uint32_t w, int k) { return (int)(w << (24 - 8 * k)) >> 24; }   // signed byte k of w

// The weight matrices of one launch: projections that read the same activations (attn_qkv, attn_gate, ssm_alpha and
// ssm_beta of a delta-net layer; attn_q / k / v of a full-attention layer) go as one grid, CTAs cta0[p] .. cta0[p+1]-1
// belonging to matrix p.
constexpr int MAX_GROUP = 8;
struct KqGroup {
    CUtensorMap map[MAX_GROUP];                   // [n_out rows][row bytes / 4 words] of each matrix
    void *y[MAX_GROUP];                           // [T][n_out]
    int n_out[MAX_GROUP];
    int cta0[MAX_GROUP + 1];
    int n;
};

struct KqArgs {
    const unsigned char *img;                     // [token tiles][nseg] Q8_K images
    void *y;                                      // [T][n_out]
    int T, n_out, nseg, out_dtype;
    int nstage, stage_bytes;                      // shared-memory stages of the tensor-core kernel
    unsigned int *status;
};


// ---- one super-block of one weight type: rows g and g + 8 of the warp's 16 against MT token tiles ---------------
// wrow0: shared address of row g's bytes of this super-block (row g + 8 is 8 * BOX further); xs: shared address of
// the group's first image; term: the super-block's f32 contribution [tile][(row g | g+8) x (token 2j | 2j+1)], which
// the engine adds to its running total (super-blocks in order).

template <int MT>
__device__ __forceinline__ void superblock_q4k(smem_ptr wrow0, smem_ptr xs, int lane, float (&term)[MT][4]) {
    constexpr int BOX = Fmt<T_Q4K>::BOX;
    const int j = lane & 3;
    smem_ptr wrow1 = wrow0 + 8 * BOX;
    // the packed 6-bit scales and minimums of the 8 sub-blocks, as bytes: sc_lo = scales 0..3, sc_hi = 4..7
    uint32_t sc_lo[2], sc_hi[2], mn_sel[2];
    float dw[2], dmw[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        smem_ptr base = r ? wrow1 : wrow0;
        const uint32_t hd = lds32(base), w0 = lds32(base + 4), w1 = lds32(base + 8), w2 = lds32(base + 12);
        dw[r] = f16_bits_to_f32(hd & 0xFFFFu);
        dmw[r] = f16_bits_to_f32(hd >> 16);
        sc_lo[r] = w0 & 0x3F3F3F3Fu;
        sc_hi[r] = (w2 & 0x0F0F0F0Fu) | ((w0 >> 2) & 0x30303030u);
        const uint32_t mn_lo = w1 & 0x3F3F3F3Fu, mn_hi = ((w2 >> 4) & 0x0F0F0F0Fu) | ((w1 >> 2) & 0x30303030u);
        mn_sel[r] = j == 0 ? mn_lo : (j == 1 ? mn_hi : 0u);          // A operand of the minimums product: k = sub-block
    }
    int isum[MT][4];
#pragma unroll
    for (int t = 0; t < MT; t++) isum[t][0] = isum[t][1] = isum[t][2] = isum[t][3] = 0;
#pragma unroll
    for (int p = 0; p < 4; p++) {                                     // sub-blocks 2p (low nibbles) and 2p + 1 (high)
        const uint32_t q00 = lds32(wrow0 + 16 + 32 * p + 4 * j), q01 = lds32(wrow0 + 16 + 32 * p + 16 + 4 * j);
        const uint32_t q10 = lds32(wrow1 + 16 + 32 * p + 4 * j), q11 = lds32(wrow1 + 16 + 32 * p + 16 + 4 * j);
#pragma unroll
        for (int hi = 0; hi < 2; hi++) {
            const int jb = 2 * p + hi;
            uint32_t A[4];
            A[0] = (q00 >> (4 * hi)) & 0x0F0F0F0Fu; A[1] = (q10 >> (4 * hi)) & 0x0F0F0F0Fu;
            A[2] = (q01 >> (4 * hi)) & 0x0F0F0F0Fu; A[3] = (q11 >> (4 * hi)) & 0x0F0F0F0Fu;
            const int s0 = (int)(((jb < 4 ? sc_lo[0] : sc_hi[0]) >> (8 * (jb & 3))) & 0xFFu);
            const int s1 = (int)(((jb < 4 ? sc_lo[1] : sc_hi[1]) >> (8 * (jb & 3))) & 0xFFu);
#pragma unroll
            for (int t = 0; t < MT; t++) {
                smem_ptr xb = xs + t * ORN_Q8K_IMG_BYTES + (2 * jb) * 128 + lane * 4;
                int D[4];
                mma_k32_u8s8(D, A, lds32(xb), lds32(xb + 128));
                isum[t][0] += D[0] * s0; isum[t][1] += D[1] * s0;
                isum[t][2] += D[2] * s1; isum[t][3] += D[3] * s1;
            }
        }
    }
#pragma unroll
    for (int t = 0; t < MT; t++) {
        smem_ptr xi = xs + t * ORN_Q8K_IMG_BYTES;
        int lo[4], hi[4];
        mma_k16_u8u8(lo, mn_sel[0], mn_sel[1], lds32(xi + ORN_Q8K_IMG_LO + lane * 4));
        mma_k16_u8s8(hi, mn_sel[0], mn_sel[1], lds32(xi + ORN_Q8K_IMG_HI + lane * 4));
        const float2 yd = *reinterpret_cast<const float2 *>(xi + ORN_Q8K_IMG_D + 8 * j);
#pragma unroll
        for (int x = 0; x < 4; x++) {
            const float ydx = (x & 1) ? yd.y : yd.x;
            const float d = __fmul_rn(ydx, dw[x >> 1]), dm = __fmul_rn(-ydx, dmw[x >> 1]);
            const int mins = lo[x] + hi[x] * 256;
            term[t][x] = __fadd_rn(__fmul_rn(d, (float)isum[t][x]), __fmul_rn(dm, (float)mins));
        }
    }
}

template <int MT>
__device__ __forceinline__ void superblock_q6k(smem_ptr wrow0, smem_ptr xs, int lane, float (&term)[MT][4]) {
    constexpr int BOX = Fmt<T_Q6K>::BOX;
    const int j = lane & 3;
    smem_ptr wrow1 = wrow0 + 8 * BOX;
    uint32_t scw[2][4];                                               // 16 signed sub-block scales per row
    float dw[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        smem_ptr base = r ? wrow1 : wrow0;
#pragma unroll
        for (int k = 0; k < 4; k++) scw[r][k] = lds32_any(base + 192 + 4 * k);
        dw[r] = f16_bits_to_f32(lds32_any(base + 208 - 2) >> 16);
    }
    int isum[MT][4];
#pragma unroll
    for (int t = 0; t < MT; t++) isum[t][0] = isum[t][1] = isum[t][2] = isum[t][3] = 0;
#pragma unroll
    for (int h = 0; h < 2; h++) {                                     // halves of 128 weights
#pragma unroll
        for (int u = 0; u < 2; u++) {                                 // l = 16 u + 4 j ..
            uint32_t ql[2][2], qh[2];                                 // [row][c % 2]
#pragma unroll
            for (int r = 0; r < 2; r++) {
                smem_ptr base = r ? wrow1 : wrow0;
                ql[r][0] = lds32_any(base + 64 * h + 16 * u + 4 * j);
                ql[r][1] = lds32_any(base + 64 * h + 32 + 16 * u + 4 * j);
                qh[r] = lds32_any(base + 128 + 32 * h + 16 * u + 4 * j);
            }
#pragma unroll
            for (int c = 0; c < 4; c++) {                             // quarter c of the half: weights 32 c + l
                const int s = 8 * h + 2 * c + u;                      // k-step = index of the 16-weight scale
                uint32_t a[2];
#pragma unroll
                for (int r = 0; r < 2; r++) {
                    const uint32_t v = ((ql[r][c & 1] >> (4 * (c >> 1))) & 0x0F0F0F0Fu) | (((qh[r] >> (2 * c)) & 0x03030303u) << 4);
                    a[r] = ((v | 0x80808080u) - 0x20202020u) ^ 0x80808080u;        // code - 32 in every byte
                }
                const int s0 = sbyte(scw[0][s >> 2], s & 3), s1 = sbyte(scw[1][s >> 2], s & 3);
#pragma unroll
                for (int t = 0; t < MT; t++) {
                    int D[4];
                    mma_k16_s8s8(D, a[0], a[1], lds32(xs + t * ORN_Q8K_IMG_BYTES + s * 128 + lane * 4));
                    isum[t][0] += D[0] * s0; isum[t][1] += D[1] * s0;
                    isum[t][2] += D[2] * s1; isum[t][3] += D[3] * s1;
                }
            }
        }
    }
#pragma unroll
    for (int t = 0; t < MT; t++) {
        const float2 yd = *reinterpret_cast<const float2 *>(xs + t * ORN_Q8K_IMG_BYTES + ORN_Q8K_IMG_D + 8 * j);
#pragma unroll
        for (int x = 0; x < 4; x++)
            term[t][x] = __fmul_rn(__fmul_rn((x & 1) ? yd.y : yd.x, dw[x >> 1]), (float)isum[t][x]);
    }
}

template <int MT>
__device__ __forceinline__ void superblock_q80(smem_ptr wrow0, smem_ptr xs, int lane, float (&term)[MT][4]) {
    constexpr int BOX = Fmt<T_Q80>::BOX;
    const int j = lane & 3;
    smem_ptr wrow1 = wrow0 + 8 * BOX;
    float blk[MT][4];
#pragma unroll
    for (int t = 0; t < MT; t++) blk[t][0] = blk[t][1] = blk[t][2] = blk[t][3] = 0.0f;
#pragma unroll
    for (int sb = 0; sb < 8; sb++) {                                  // block sb: f16 scale at 34 sb, 32 codes after it
        uint32_t A[4];
        float wd[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            smem_ptr base = (r ? wrow1 : wrow0) + 34 * sb;
            if ((sb & 1) == 0) {                                      // 34 sb is a multiple of 4: the codes start mid-word
                const uint32_t w0 = lds32(base + 4 * j), w1 = lds32(base + 4 * j + 4);
                const uint32_t w4 = lds32(base + 16 + 4 * j), w5 = lds32(base + 16 + 4 * j + 4);
                A[r] = __byte_perm(w0, w1, 0x5432);
                A[2 + r] = __byte_perm(w4, w5, 0x5432);
                wd[r] = f16_bits_to_f32(lds32(base) & 0xFFFFu);
            } else {                                                  // 34 sb + 2 is a multiple of 4
                A[r] = lds32(base + 2 + 4 * j);
                A[2 + r] = lds32(base + 2 + 16 + 4 * j);
                wd[r] = f16_bits_to_f32(lds32(base - 2) >> 16);
            }
        }
#pragma unroll
        for (int t = 0; t < MT; t++) {
            smem_ptr xb = xs + t * ORN_Q8K_IMG_BYTES + (2 * sb) * 128 + lane * 4;
            int D[4];
            mma_k32_s8s8(D, A, lds32(xb), lds32(xb + 128));
#pragma unroll
            for (int x = 0; x < 4; x++) blk[t][x] = __fadd_rn(blk[t][x], __fmul_rn(wd[x >> 1], (float)D[x]));
        }
    }
#pragma unroll
    for (int t = 0; t < MT; t++) {
        const float2 yd = *reinterpret_cast<const float2 *>(xs + t * ORN_Q8K_IMG_BYTES + ORN_Q8K_IMG_D + 8 * j);
#pragma unroll
        for (int x = 0; x < 4; x++) term[t][x] = __fmul_rn((x & 1) ? yd.y : yd.x, blk[t][x]);
    }
}

// grid: (ceil(n_out / (16 WR)), passes) CTAs of 16 warps.  A CTA owns 16 WR weight rows and one pass of
// 8 MT TS tokens; its warps split the work three ways, WR x KS x TS = 16:
//   WR ways over the rows (16 rows each: one MMA m-tile).  Few rows per CTA = more CTAs for a weight matrix with
//      few rows, which is what a memory-bound product of a few tokens needs;
//   KS ways over the super-blocks (ks takes super-blocks ks, ks + KS, ..): for few tokens one warp per scheduler
//      would run the dependent unpack -> MMA -> scale chain of a super-block alone; KS of them run side by side.
//      A super-block's f32 term goes through shared memory to the warps with ks = 0, which add the KS terms of a
//      round in super-block order, so the total has the engine's association whatever KS is;
//   TS ways over the token tiles (MT tiles each).
// Tiles past the pass's last one are multiplied too (against whatever the stage holds) and never stored: a test per
// tile would put every MMA into a basic block of its own and expose the latency of its operand load.
// Stages: a.nstage (up to 16) of a.stage_bytes on mbarriers; after the barrier that ends a round every stage of the
// round is free and thread 0 refills as far ahead as the stages allow.  The kernel is launched as a programmatic
// dependent of the quantiser: it starts the weight copies of its first stages at once and waits for the quantiser
// (griddepcontrol.wait) only before the first copy of an activation image.
constexpr int NWARP = 16, MAX_STAGES = 16;
template <int TYPE, int WR, int KS, int MT>
__global__ void __launch_bounds__(NWARP * 32, 1) k_matmul_kq(KqArgs a, const __grid_constant__ KqGroup grp) {
    constexpr int BLOCK = Fmt<TYPE>::BLOCK, BOX = Fmt<TYPE>::BOX, CTA_ROWS = 16 * WR, WBYTES = CTA_ROWS * BOX, TS = NWARP / (WR * KS);
    static_assert(WR * KS * TS == NWARP, "the warps split rows x super-blocks x token tiles");
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[MAX_STAGES];
    __shared__ int failed;
    unsigned char *smem = smem_raw + ((128 - (smem_u32(smem_raw) & 127)) & 127);
    const int tid = threadIdx.x, lane = tid & 31, w16 = tid >> 5, g = lane >> 2, j = lane & 3;
    const int wr = w16 % WR, ks = (w16 / WR) % KS, ts = w16 / (WR * KS), t_lo = ts * MT;
    int pj = 0;                                                       // the matrix this CTA belongs to
    while (pj + 1 < grp.n && (int)blockIdx.x >= grp.cta0[pj + 1]) pj++;
    const int n_out = grp.n_out[pj];
    const int cta_row0 = ((int)blockIdx.x - grp.cta0[pj]) * CTA_ROWS, row0 = cta_row0 + wr * 16;
    const int tok0 = (int)blockIdx.y * (8 * MT * TS);
    const int nt_all = min(MT * TS, (a.T - tok0 + 7) / 8);            // token tiles of this pass
    const int nstage = a.nstage, stage_bytes = a.stage_bytes;
    float *terms = reinterpret_cast<float *>(smem + (size_t)nstage * stage_bytes);   // [2][KS][TS * WR warps][32 lanes][MT * 4], KS > 1 only
    const int slot = (ts * WR + wr) * 32 + lane;                      // this thread's place among the threads with its ks
    if (tid == 0) {
        failed = 0;
        for (int i = 0; i < nstage; i++) tc5::mbar_init(smem_u32(&bars[i]), 1);
        tc5::mbar_init_fence();
    }
    __syncthreads();
    // rows past n_out and bytes past a row's end are outside the map: zeros
    auto issue_w = [&](int seg) {
        const uint32_t bar = smem_u32(&bars[seg % nstage]), base = smem_u32(smem + (size_t)(seg % nstage) * stage_bytes);
        tc5::mbar_expect_tx(bar, (uint32_t)(WBYTES + nt_all * ORN_Q8K_IMG_BYTES));
        tensor_copy_rows(base, &grp.map[pj], ((seg * BLOCK) & ~15) / 4, cta_row0, bar);
    };
    auto issue_x = [&](int seg) {
        const uint32_t bar = smem_u32(&bars[seg % nstage]), base = smem_u32(smem + (size_t)(seg % nstage) * stage_bytes);
        for (int t = 0; t < nt_all; t++)
            bulk_copy(base + WBYTES + t * ORN_Q8K_IMG_BYTES,
                      a.img + ((size_t)((tok0 >> 3) + t) * a.nseg + seg) * ORN_Q8K_IMG_BYTES, ORN_Q8K_IMG_BYTES, bar);
    };
    int issued = 0;
    if (tid == 0) {
        const int first = min(nstage, a.nseg);
        for (int i = 0; i < first; i++) issue_w(i);
        asm volatile("griddepcontrol.wait;\n" ::: "memory");         // the images come from the kernel in front
        for (int i = 0; i < first; i++) issue_x(i);
        issued = first;
    }
    float tot[MT][4];
#pragma unroll
    for (int t = 0; t < MT; t++) tot[t][0] = tot[t][1] = tot[t][2] = tot[t][3] = 0.0f;
    const bool active = row0 < n_out && t_lo < nt_all;
    bool ok = true;
    const int rounds = (a.nseg + KS - 1) / KS;
    for (int r = 0; r < rounds; r++) {
        const int seg = r * KS + ks;
        float term[MT][4];
#pragma unroll
        for (int t = 0; t < MT; t++) term[t][0] = term[t][1] = term[t][2] = term[t][3] = 0.0f;
        if (seg < a.nseg) {
            if (ok && !tc5::mbar_wait(smem_u32(&bars[seg % nstage]), (uint32_t)(seg / nstage) & 1u)) { ok = false; failed = 1; }
            if (ok && active) {
                smem_ptr stage = smem + (size_t)(seg % nstage) * stage_bytes;
                smem_ptr wrow0 = stage + (wr * 16 + g) * BOX + ((seg * BLOCK) & 15);
                smem_ptr xs = stage + WBYTES + t_lo * ORN_Q8K_IMG_BYTES;
                if (TYPE == T_Q4K) superblock_q4k<MT>(wrow0, xs, lane, term);
                else if (TYPE == T_Q6K) superblock_q6k<MT>(wrow0, xs, lane, term);
                else superblock_q80<MT>(wrow0, xs, lane, term);
            }
        }
        if (KS == 1) {
#pragma unroll
            for (int t = 0; t < MT; t++)
#pragma unroll
                for (int x = 0; x < 4; x++) tot[t][x] = __fadd_rn(tot[t][x], term[t][x]);
        } else {
            float4 *dst = reinterpret_cast<float4 *>(terms + ((size_t)((r & 1) * KS + ks) * (TS * WR * 32) + slot) * (MT * 4));
#pragma unroll
            for (int t = 0; t < MT; t++) dst[t] = make_float4(term[t][0], term[t][1], term[t][2], term[t][3]);
        }
        __syncthreads();                          // every warp is done with the stages of round r
        if (KS > 1 && ks == 0) {                  // the round's terms in super-block order
            for (int k = 0; k < KS && r * KS + k < a.nseg; k++) {
                const float4 *src = reinterpret_cast<const float4 *>(terms + ((size_t)((r & 1) * KS + k) * (TS * WR * 32) + slot) * (MT * 4));
#pragma unroll
                for (int t = 0; t < MT; t++) {
                    const float4 v = src[t];
                    tot[t][0] = __fadd_rn(tot[t][0], v.x); tot[t][1] = __fadd_rn(tot[t][1], v.y);
                    tot[t][2] = __fadd_rn(tot[t][2], v.z); tot[t][3] = __fadd_rn(tot[t][3], v.w);
                }
            }
        }
        if (tid == 0 && !failed) {
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            for (; issued < a.nseg && issued < (r + 1) * KS + nstage; issued++) { issue_w(issued); issue_x(issued); }
        }
        if (failed) ok = false;
    }
    if (!ok && tid == 0 && a.status) atomicOr(a.status, ORN_WAIT_DECODE);
    if (ks != 0) return;
#pragma unroll
    for (int t = 0; t < MT; t++)
#pragma unroll
        for (int x = 0; x < 4; x++) {
            const int row = row0 + g + 8 * (x >> 1), tok = tok0 + 8 * (t_lo + t) + 2 * j + (x & 1);
            if (row < n_out && t_lo + t < nt_all && tok < a.T) {
                const float val = ok ? tot[t][x] : NAN;
                if (a.out_dtype == ORNITH_ACT_BF16) act_st((__nv_bfloat16 *)grp.y[pj], (size_t)tok * n_out + row, val);
                else act_st((float *)grp.y[pj], (size_t)tok * n_out + row, val);
            }
        }
}

// ---- the plain form: one thread per (row, token), bytes from global memory; any alignment ----------------------
__device__ __forceinline__ int img_code(const unsigned char *im, int g, int e) { return (int)(signed char)im[(e >> 4) * 128 + g * 16 + (e & 15)]; }
__device__ __forceinline__ float ld_f16(const unsigned char *p) { return f16_bits_to_f32((uint32_t)p[0] | ((uint32_t)p[1] << 8)); }

template <int TYPE>
__global__ void __launch_bounds__(128) k_matmul_kq_plain(const unsigned char *W, KqArgs a) {
    constexpr int BLOCK = Fmt<TYPE>::BLOCK;
    const int row = blockIdx.y * 128 + threadIdx.x, tok = blockIdx.x;       // tokens on x: no 65535 limit
    if (row >= a.n_out) return;
    const unsigned char *wr = W + (size_t)row * a.nseg * BLOCK;
    const int g = tok & 7;
    float total = 0.0f;
    for (int i = 0; i < a.nseg; i++) {
        const unsigned char *blk = wr + (size_t)i * BLOCK;
        const unsigned char *im = a.img + ((size_t)(tok >> 3) * a.nseg + i) * ORN_Q8K_IMG_BYTES;
        const float yd = reinterpret_cast<const float *>(im + ORN_Q8K_IMG_D)[g];
        if (TYPE == T_Q4K) {
            const unsigned char *q = blk + 4, *codes = blk + 16;
            int dots = 0, mins = 0;
            for (int jb = 0; jb < 8; jb++) {
                int sc, mn;
                if (jb < 4) { sc = q[jb] & 63; mn = q[jb + 4] & 63; }
                else { sc = (q[jb + 4] & 0x0F) | ((q[jb - 4] >> 6) << 4); mn = (q[jb + 4] >> 4) | ((q[jb] >> 6) << 4); }
                mins += mn * ((int)im[ORN_Q8K_IMG_LO + g * 16 + jb] + 256 * (int)(signed char)im[ORN_Q8K_IMG_HI + g * 16 + jb]);
                int part = 0;
                for (int l = 0; l < 32; l++)
                    part += (int)((codes[32 * (jb >> 1) + l] >> (4 * (jb & 1))) & 0x0F) * img_code(im, g, 32 * jb + l);
                dots += part * sc;
            }
            const float d = __fmul_rn(yd, ld_f16(blk)), dm = __fmul_rn(-yd, ld_f16(blk + 2));
            total = __fadd_rn(total, __fadd_rn(__fmul_rn(d, (float)dots), __fmul_rn(dm, (float)mins)));
        } else if (TYPE == T_Q6K) {
            int dots = 0;
            for (int e = 0; e < 256; e++) {
                const int h = e >> 7, c = (e & 127) >> 5, l = e & 31;
                const int lo = (blk[64 * h + 32 * (c & 1) + l] >> (4 * (c >> 1))) & 0x0F, hi = (blk[128 + 32 * h + l] >> (2 * c)) & 3;
                dots += img_code(im, g, e) * ((lo | (hi << 4)) - 32) * (int)(signed char)blk[192 + (e >> 4)];
            }
            total = __fadd_rn(total, __fmul_rn(__fmul_rn(yd, ld_f16(blk + 208)), (float)dots));
        } else {
            float bs = 0.0f;
            for (int sb = 0; sb < 8; sb++) {
                int part = 0;
                for (int l = 0; l < 32; l++) part += (int)(signed char)blk[34 * sb + 2 + l] * img_code(im, g, 32 * sb + l);
                bs = __fadd_rn(bs, __fmul_rn(ld_f16(blk + 34 * sb), (float)part));
            }
            total = __fadd_rn(total, __fmul_rn(yd, bs));
        }
    }
    if (a.out_dtype == ORNITH_ACT_BF16) act_st((__nv_bfloat16 *)a.y, (size_t)tok * a.n_out + row, total);
    else act_st((float *)a.y, (size_t)tok * a.n_out + row, total);
}

// the weight matrix as [n_out rows][row_bytes / 4 words]; one box = box_rows rows x BOX bytes
template <int TYPE>
bool weight_map(CUtensorMap *m, const void *W, int n_in, int n_out, int box_rows) {
    OrnTensorMapEncodeFn enc = orn_tensor_map_encoder();
    const cuuint64_t row_bytes = (cuuint64_t)n_in / QK * Fmt<TYPE>::BLOCK;
    if (!enc || ((uintptr_t)W & 15) != 0 || (row_bytes & 15) != 0) return false;
    cuuint64_t dims[2] = {row_bytes / 4, (cuuint64_t)n_out};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {Fmt<TYPE>::BOX / 4, (cuuint32_t)box_rows};
    cuuint32_t es[2] = {1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(W), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

constexpr int SMEM_BUDGET = 200 * 1024;           // dynamic shared memory of one CTA (one CTA per SM: 512 threads)

// what the host knows of a group: the matrices (all of one weight type, one n_in), their outputs
struct HostGroup {
    const void *W[MAX_GROUP];
    void *y[MAX_GROUP];
    int n_out[MAX_GROUP];
    int n;
    int rows_total() const { int r = 0; for (int i = 0; i < n; i++) r += n_out[i]; return r; }
};

template <int TYPE, int WR, int KS, int MT>
ornith_status launch_tc(const HostGroup &h, int n_in, int T, KqArgs a, cudaStream_t stream) {
    constexpr int TS = NWARP / (WR * KS), PASS_TOK = 8 * MT * TS, CTA_ROWS = 16 * WR;
    KqGroup g;
    g.n = h.n;
    g.cta0[0] = 0;
    for (int i = 0; i < h.n; i++) {
        if (!weight_map<TYPE>(&g.map[i], h.W[i], n_in, h.n_out[i], CTA_ROWS)) {
            orn_record_error("matmul_q: the weight tensor map could not be made");
            return (ornith_status)ORNITH_ERR_BACKEND;
        }
        g.y[i] = h.y[i]; g.n_out[i] = h.n_out[i];
        g.cta0[i + 1] = g.cta0[i] + (h.n_out[i] + CTA_ROWS - 1) / CTA_ROWS;
    }
    // tiles of the fullest pass, rounded up to whole groups: a group multiplies all MT of its tiles, so the stage
    // must have room for them (the ones past the pass's last tile hold stale bytes and are never stored)
    const int nt_max = (((T < PASS_TOK ? T : PASS_TOK) + 7) / 8 + MT - 1) / MT * MT;
    a.stage_bytes = (int)align_up((size_t)CTA_ROWS * Fmt<TYPE>::BOX + (size_t)nt_max * ORN_Q8K_IMG_BYTES, 128);
    const int terms = KS > 1 ? 2 * NWARP * 32 * MT * 4 * (int)sizeof(float) : 0;
    int nstage = (SMEM_BUDGET - 128 - terms) / a.stage_bytes;
    if (nstage > MAX_STAGES) nstage = MAX_STAGES;
    if (nstage > a.nseg) nstage = a.nseg;
    if (nstage < KS && nstage < a.nseg) {         // a round reads KS stages at once
        orn_record_error("matmul_q: %d stages of %d bytes do not hold a round of %d super-blocks", nstage, a.stage_bytes, KS);
        return (ornith_status)ORNITH_ERR_BACKEND;
    }
    a.nstage = nstage;
    const int smem = nstage * a.stage_bytes + terms + 128;
    static bool opted[ORN_MAX_DEVICES] = {};
    bool &have = opted[orn_device_index()];
    if (!have) {
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_matmul_kq<TYPE, WR, KS, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BUDGET), "projection smem opt-in"));
        have = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)g.cta0[h.n], (unsigned)((T + PASS_TOK - 1) / PASS_TOK));
    cfg.blockDim = dim3(NWARP * 32);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // may start while the quantiser in front of it still runs
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    return orn_check(cudaLaunchKernelEx(&cfg, k_matmul_kq<TYPE, WR, KS, MT>, a, g), "k_matmul_kq");
}

// the split of the 16 warps: rows per CTA so that a few-token product has about one CTA per SM or more; the
// rest over the super-blocks (few tokens) or the token tiles
template <int TYPE, int WR>
ornith_status launch_wr(const HostGroup &h, int n_in, int T, KqArgs a, cudaStream_t stream) {
    if (T <= 16) return launch_tc<TYPE, WR, 16 / WR, 2>(h, n_in, T, a, stream);
    if (T <= 32) return launch_tc<TYPE, WR, 8 / WR, 2>(h, n_in, T, a, stream);
    // 33-64 tokens, k-quants: four tiles per warp where the stages still hold a round, so that an unpacked weight
    // operand (the expensive part for the packed 4- and 6-bit codes) feeds four MMAs instead of two: 2048 -> 8192 in
    // Q6_K 22.9 -> 19.8 us.  Q8_0 unpacks cheaply and pays per MMA for its exact f32 epilogue: 15.4 -> 16.4 us, not used.
    if (TYPE != T_Q80 && WR >= 2) return launch_tc<TYPE, WR, 8 / WR, 4>(h, n_in, T, a, stream);
    return launch_tc<TYPE, WR, 4 / WR, 2>(h, n_in, T, a, stream);
}

template <int TYPE>
ornith_status launch_kq(const HostGroup &h, int n_in, int T, KqArgs a, bool plain, cudaStream_t stream) {
    const size_t row_bytes = (size_t)n_in / QK * Fmt<TYPE>::BLOCK;
    bool tc = !plain && (row_bytes & 15) == 0 && orn_tensor_map_encoder();
    for (int i = 0; i < h.n; i++) tc = tc && ((uintptr_t)h.W[i] & 15) == 0;
    if (!tc) {                                    // the plain kernel, matrix by matrix
        for (int i = 0; i < h.n; i++) {
            a.y = h.y[i]; a.n_out = h.n_out[i];
            k_matmul_kq_plain<TYPE><<<dim3((unsigned)T, (unsigned)((h.n_out[i] + 127) / 128)), 128, 0, stream>>>((const unsigned char *)h.W[i], a);
            ORN_TRY(orn_check_launch("k_matmul_kq_plain"));
        }
        return ORNITH_OK;
    }
    const int n_out = h.rows_total();
    if (T > 64) {                                 // prompts: passes of 128 tokens; of 64 with fewer rows per CTA for a small matrix
        const long p128 = (T + 127) / 128, p64 = (T + 63) / 64;
        if ((n_out + 63) / 64 * p128 >= 100) return launch_tc<TYPE, 4, 1, 4>(h, n_in, T, a, stream);
        if ((n_out + 63) / 64 * p64 >= 100) return launch_tc<TYPE, 4, 1, 2>(h, n_in, T, a, stream);
        if ((n_out + 31) / 32 * p64 >= 100) return launch_tc<TYPE, 2, 2, 2>(h, n_in, T, a, stream);
        return launch_tc<TYPE, 1, 4, 2>(h, n_in, T, a, stream);
    }
    if (n_out >= 64 * 100) return launch_wr<TYPE, 4>(h, n_in, T, a, stream);
    if (n_out >= 32 * 100) return launch_wr<TYPE, 2>(h, n_in, T, a, stream);
    return launch_wr<TYPE, 1>(h, n_in, T, a, stream);
}

ornith_status run_group(int wtype, const HostGroup &h, int n_in, const void *image, int T, int out_dtype, cudaStream_t s) {
    KqArgs a;
    a.img = (const unsigned char *)image;
    a.y = nullptr; a.T = T; a.n_out = 0; a.nseg = n_in / QK; a.out_dtype = out_dtype; a.nstage = 0; a.stage_bytes = 0; a.status = orn_status_word();
    const char *e = getenv("ORNITH_CUDA_PROJ_PLAIN");                 // =1: the plain kernel for every shape
    const bool plain = e && e[0] == '1';
    if (wtype == ORNITH_GGML_Q4_K) return launch_kq<T_Q4K>(h, n_in, T, a, plain, s);
    if (wtype == ORNITH_GGML_Q6_K) return launch_kq<T_Q6K>(h, n_in, T, a, plain, s);
    return launch_kq<T_Q80>(h, n_in, T, a, plain, s);
}

}  // namespace

extern "C" {

size_t ornith_cuda_matmul_q_scratch(int wtype, int T, int n_in) {
    if (T <= 0 || n_in <= 0 || n_in % QK) return 0;
    if (wtype != ORNITH_GGML_Q4_K && wtype != ORNITH_GGML_Q6_K && wtype != ORNITH_GGML_Q8_0) return 0;
    return orn_q8k_image_bytes(T, n_in);       // the same for the three types: the image of the activations
}

static bool kq_type_ok(int wtype) { return wtype == ORNITH_GGML_Q4_K || wtype == ORNITH_GGML_Q6_K || wtype == ORNITH_GGML_Q8_0; }

ornith_status ornith_cuda_q8k_image(const void *x, int act_dtype, int T, int n_in, void *image, size_t image_bytes, void *stream) {
    ORN_TRY(orn_require_device());
    if (n_in <= 0 || n_in % QK) { orn_record_error("q8k_image: the row length must be a multiple of 256 (got %d)", n_in); return ORNITH_ERR_FORMAT; }
    if (T <= 0) return ORNITH_OK;
    if (!image || image_bytes < orn_q8k_image_bytes(T, n_in) || ((uintptr_t)image & 255) != 0) {
        orn_record_error("q8k_image: image buffer too small or not 256-byte aligned");
        return ORNITH_ERR_FORMAT;
    }
    return orn_q8k_quantize_image(x, act_dtype, T, n_in, image, (cudaStream_t)stream);
}

ornith_status ornith_cuda_matmul_q_group(const ornith_cuda_qproj *projs, int n, int n_in, const void *image, int T,
                                         int out_dtype, void *stream) {
    ORN_TRY(orn_require_device());
    if (n <= 0 || T <= 0) return ORNITH_OK;
    if (!projs) { orn_record_error("matmul_q: no projections given"); return ORNITH_ERR_FORMAT; }
    if (n_in <= 0 || n_in % QK) { orn_record_error("matmul_q: the row length must be a multiple of 256 (got %d)", n_in); return ORNITH_ERR_FORMAT; }
    if (!image || ((uintptr_t)image & 255) != 0) { orn_record_error("matmul_q: the activation image must be 256-byte aligned"); return ORNITH_ERR_FORMAT; }
    for (int i = 0; i < n; i++)
        if (!kq_type_ok(projs[i].wtype)) {
            orn_record_error("matmul_q: no integer path for weight type %d (Q8_0 = 8, Q4_K = 12, Q6_K = 14)", projs[i].wtype);
            return ORNITH_ERR_UNSUPPORTED;
        }
    // one launch per run of matrices of the same weight type (at most MAX_GROUP of them)
    for (int i = 0; i < n;) {
        HostGroup h;
        h.n = 0;
        const int wtype = projs[i].wtype;
        for (; i < n && projs[i].wtype == wtype && h.n < MAX_GROUP; i++) {
            if (projs[i].n_out <= 0) continue;
            h.W[h.n] = projs[i].W; h.y[h.n] = projs[i].y; h.n_out[h.n] = projs[i].n_out; h.n++;
        }
        if (h.n) ORN_TRY(run_group(wtype, h, n_in, image, T, out_dtype, (cudaStream_t)stream));
    }
    return ORNITH_OK;
}

ornith_status ornith_cuda_matmul_q_image(int wtype, const void *W, int n_in, int n_out, const void *image, int T, void *y,
                                         int out_dtype, void *stream) {
    ornith_cuda_qproj p;
    p.wtype = wtype; p.W = W; p.n_out = n_out; p.y = y;
    return ornith_cuda_matmul_q_group(&p, 1, n_in, image, T, out_dtype, stream);
}

ornith_status ornith_cuda_matmul_q(int wtype, const void *W, int n_in, int n_out, const void *x, int act_dtype, int T,
                                   void *y, int out_dtype, void *scratch, size_t scratch_bytes, void *stream) {
    if (!kq_type_ok(wtype)) {
        orn_record_error("matmul_q: no integer path for weight type %d (Q8_0 = 8, Q4_K = 12, Q6_K = 14)", wtype);
        return ORNITH_ERR_UNSUPPORTED;
    }
    if (T <= 0 || n_out <= 0) return ORNITH_OK;
    ORN_TRY(ornith_cuda_q8k_image(x, act_dtype, T, n_in, scratch, scratch_bytes, stream));
    return ornith_cuda_matmul_q_image(wtype, W, n_in, n_out, scratch, T, y, out_dtype, stream);
}

}  // extern "C"
