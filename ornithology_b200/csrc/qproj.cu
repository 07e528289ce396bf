// qproj.cu — the quantised projections around the attention core: Q8_0 weights x Q8_K activations.
//
// Replaces matmul_batch_q over Q8_0 weights (reference: src/ornith_rforward.c:138-192) and its two helpers,
// qdot_quantize_row_q8_K (src/ornith_qdot.c:38-70) and vec_dot_q8_0 (:144-163), for the decode-sized batches
// that bracket every attention kernel (attn_qkv, ssm_alpha/beta, attn_gate, ssm_out, attn_q/k/v/output).
//
// The engine quantises every activation row to Q8_K once (blocks of 256: scale -127/max, codes rounded to
// nearest even) and then takes, per weight row, an integer dot per Q8_0 block, scaled by the block's f16 scale,
// summed over the super-block, scaled by the activation's scale.  Here:
//
//   k_q8k_quantize   one warp per (token, super-block).  The codes and scales are the engine's bit for bit
//                    (same divide, multiply, round-to-nearest-even, first-maximum rule); they are written twice:
//                    as the engine's 292-byte blocks when asked (for parity and for hosts that want them), and
//                    as the image the product reads — the codes as exact f16 integers in MMA B-fragment order,
//                    plus the plane of scales.
//   k_matmul_q8_0    a weight row of 256 inputs is 8 Q8_0 blocks = 272 bytes = 17 chunks of 16 bytes, the same
//                    stream the Q8_0 KV rows have, so the product is built like the score product of the decode
//                    kernel: a warp stages 16 weight rows x 272 bytes by one tensor copy, ldmatrix hands each lane
//                    four codes per chunk, one byte permute + HSUB2 + HMUL2 turn them into f16 weights (code x
//                    block scale), and mma.sync m16n8k16 multiplies them with the activation fragments of up to
//                    8 token tiles (the conversion is shared by all of them).  The sum over a super-block is
//                    kept apart and scaled by the activation's d in f32, as the engine does.
//
// Precision: the integer codes of both operands are exact; a weight (code x f16 scale) is rounded once to f16
// (2^-12 relative), sums are f32.  Against the engine's integer path: <= 2e-4 of the output's maximum (the bar of
// this path is 2e-3).  Prompt-sized batches are a plain GEMM after dequantisation and are not built here: batches
// above 64 tokens are walked 64 at a time, re-reading the weights.
#include <cuda.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "qproj.cuh"
#include "tcgen05.cuh"          // the tensor-map encoder entry point

namespace {

constexpr int QK = 256;                       // inputs per super-block
constexpr int SEGB = 272;                     // bytes of one weight row over a super-block: 8 x (f16 scale + 32 codes)
constexpr int NCHUNK = 17;                    // 16-byte chunks per 272 bytes
constexpr int ROWS = 16;                      // weight rows per warp
constexpr int FRAG_WORDS2 = NCHUNK * 32;       // uint2 entries of the activation fragments of one (token tile of 8, super-block)
constexpr int FRAG_BYTES = FRAG_WORDS2 * 8 + 32; // the fragments (4352 bytes) followed by the 8 tokens' block scales (f32)
constexpr int MAXNT = 8;                      // token tiles per pass (64 tokens)
constexpr int WARPS = 4;                      // warps that share the CTA's 64 weight rows (16 each)

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t h2_mul_sub(uint32_t biased, uint32_t scale) {   // (x - 1152) * scale
    const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);
    __half2 v = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&biased), bias), *reinterpret_cast<__half2 *>(&scale));
    return *reinterpret_cast<uint32_t *>(&v);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
// bounded wait (poll limit and 2 s of wall time)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) { return tc5::mbar_wait(bar, parity); }
__device__ __forceinline__ void tensor_copy_rows(uint32_t dst, const CUtensorMap *map, int word0, int row0, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(word0), "r"(row0) : "memory");
}

// stream element e of a 272-byte segment: block e / 17; index 0 of a block is its scale, index i > 0 the code pair
// of inputs 2(i-1), 2(i-1)+1 of that block
__host__ __device__ constexpr int elem_block(int e) { return e / 17; }

// The f16 weights of chunk C for rows r and r + 8 (A operand of one k-step): raw0 / raw1 = the lane's ldmatrix
// registers (elements 8C+2j, 8C+2j+1), dk0 / dk1 = the rows' block scales as f16 pairs.
template <int C>
__device__ __forceinline__ void weights_chunk(uint32_t raw0, uint32_t raw1, const uint32_t (&dk0)[8], const uint32_t (&dk1)[8],
                                              int j, uint32_t (&A)[4]) {
    constexpr int BLO = elem_block(8 * C), BHI = elem_block(8 * C + 7) > 7 ? 7 : elem_block(8 * C + 7);
    const bool hi0 = (BHI != BLO) && (8 * C + 2 * j >= 17 * BHI);
    const bool hi1 = (BHI != BLO) && (8 * C + 2 * j + 1 >= 17 * BHI);
    const uint32_t s00 = hi0 ? dk0[BHI] : dk0[BLO], s01 = hi1 ? dk0[BHI] : dk0[BLO];
    const uint32_t s10 = hi0 ? dk1[BHI] : dk1[BLO], s11 = hi1 ? dk1[BHI] : dk1[BLO];
    const uint32_t x0 = raw0 ^ 0x80808080u, x1 = raw1 ^ 0x80808080u;
    A[0] = h2_mul_sub(__byte_perm(x0, 0x64646464u, 0x4140), s00);
    A[1] = h2_mul_sub(__byte_perm(x1, 0x64646464u, 0x4140), s10);
    A[2] = h2_mul_sub(__byte_perm(x0, 0x64646464u, 0x4342), s01);
    A[3] = h2_mul_sub(__byte_perm(x1, 0x64646464u, 0x4342), s11);
}

// ---- activations -> Q8_K ------------------------------------------------------------------------------
// grid (n_in / 256, T_pad), one warp each.  Tokens >= T are padding of the last tile of 8: zero fragments.
// blocks: [T][n_in/256] engine blocks of 292 bytes, or NULL.  frags: [T_pad/8][n_in/256] images of FRAG_BYTES:
// [17][32] uint2 fragments, then the 8 tokens' scales.
//
// img (or NULL): the image the integer products read (kquant_matmul.cu), [T_pad/8][n_in/256] images of
// ORN_Q8K_IMG_BYTES: the codes as int8 MMA B operands (16 k-steps of 16 inputs x [8 tokens][16 bytes]), the 8
// tokens' scales, and the sums of the codes over each run of 32 inputs split into an unsigned low byte and a signed
// high byte (two B operands of [8 tokens][16 bytes], bytes 8..15 zero).
template <typename ACT>
__global__ void __launch_bounds__(32) k_q8k_quantize(const ACT *x, int T, int n_in, unsigned char *blocks, uint2 *frags,
                                                     unsigned char *img) {
    const int seg = blockIdx.x, tok = blockIdx.y, lane = threadIdx.x, nseg = n_in / QK;
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");     // a product launched as a dependent may start its weight copies
    float v[8];
    float amax = 0.0f, mx = 0.0f;
    int arg = 0;
    if (tok < T) {
        const ACT *src = x + (size_t)tok * n_in + (size_t)seg * QK + 8 * lane;
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = act_ld(src, i);
        // the element of largest magnitude, the first one on ties (the engine scans in order with a strict >)
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (fabsf(v[i]) > amax) { amax = fabsf(v[i]); mx = v[i]; arg = 8 * lane + i; }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            const float a2 = __shfl_xor_sync(0xffffffffu, amax, o), m2 = __shfl_xor_sync(0xffffffffu, mx, o);
            const int g2 = __shfl_xor_sync(0xffffffffu, arg, o);
            if (a2 > amax || (a2 == amax && g2 < arg)) { amax = a2; mx = m2; arg = g2; }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = 0.0f;
    }
    int q[8];
    float d = 0.0f;
    if (amax != 0.0f) {
        const float iscale = __fdiv_rn(-127.0f, mx);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            int c = __float2int_rn(__fmul_rn(iscale, v[i]));
            q[i] = c > 127 ? 127 : (c < -128 ? -128 : c);
        }
        d = __fdiv_rn(1.0f, iscale);
    } else {
#pragma unroll
        for (int i = 0; i < 8; i++) q[i] = 0;
    }
    if (blocks && tok < T) {                      // the engine's block: f32 d, 256 codes, 16 sums of 16 codes
        unsigned char *blk = blocks + ((size_t)tok * nseg + seg) * 292;
        int sum = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) sum += q[i];
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        if (lane == 0) *reinterpret_cast<float *>(blk) = d;
        uint32_t w0 = 0, w1 = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) { w0 |= (uint32_t)(q[i] & 255) << (8 * i); w1 |= (uint32_t)(q[4 + i] & 255) << (8 * i); }
        *reinterpret_cast<uint32_t *>(blk + 4 + 8 * lane) = w0;                  // (blocks are 4-byte aligned only)
        *reinterpret_cast<uint32_t *>(blk + 8 + 8 * lane) = w1;
        if ((lane & 1) == 0) *reinterpret_cast<short *>(blk + 260 + lane) = (short)sum;
    }
    if (img) {
        unsigned char *im = img + ((size_t)(tok >> 3) * nseg + seg) * ORN_Q8K_IMG_BYTES;
        const int g = tok & 7;
        uint2 w;
        w.x = w.y = 0u;
#pragma unroll
        for (int i = 0; i < 4; i++) { w.x |= (uint32_t)(q[i] & 255) << (8 * i); w.y |= (uint32_t)(q[4 + i] & 255) << (8 * i); }
        *reinterpret_cast<uint2 *>(im + (lane >> 1) * 128 + g * 16 + 8 * (lane & 1)) = w;      // inputs 8 lane .. 8 lane + 7
        if (lane == 0) reinterpret_cast<float *>(im + ORN_Q8K_IMG_D)[g] = d;
        int s32 = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) s32 += q[i];
        s32 += __shfl_xor_sync(0xffffffffu, s32, 1);
        s32 += __shfl_xor_sync(0xffffffffu, s32, 2);                                           // inputs 32 (lane / 4) ..
        if ((lane & 3) == 0) {
            im[ORN_Q8K_IMG_LO + g * 16 + (lane >> 2)] = (unsigned char)(s32 & 255);
            im[ORN_Q8K_IMG_HI + g * 16 + (lane >> 2)] = (unsigned char)((s32 >> 8) & 255);
        } else if ((lane & 3) == 1) {
            im[ORN_Q8K_IMG_LO + g * 16 + 8 + (lane >> 2)] = 0;
            im[ORN_Q8K_IMG_HI + g * 16 + 8 + (lane >> 2)] = 0;
        }
    }
    if (!frags) return;
    // the product's image: pair p = inputs (2p, 2p+1) is stream element e = 17 (p / 16) + 1 + p % 16, which lies
    // in chunk e / 8 at position e % 8 = 2 j + h of lane (token % 8, j)
    unsigned char *fimg = reinterpret_cast<unsigned char *>(frags) + ((size_t)(tok >> 3) * nseg + seg) * FRAG_BYTES;
    uint32_t *fr = reinterpret_cast<uint32_t *>(fimg);
    if (lane == 0) reinterpret_cast<float *>(fimg + FRAG_WORDS2 * 8)[tok & 7] = d;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int p = 4 * lane + i, e = 17 * (p >> 4) + 1 + (p & 15);
        const __half2 h = __floats2half2_rn((float)q[2 * i], (float)q[2 * i + 1]);
        fr[((e >> 3) * 32 + (tok & 7) * 4 + ((e & 7) >> 1)) * 2 + (e & 1)] = *reinterpret_cast<const uint32_t *>(&h);
    }
    if (lane < 8) {                               // the slots that face a block scale in the weight stream: zero
        const int e = 17 * lane;
        fr[((e >> 3) * 32 + (tok & 7) * 4 + ((e & 7) >> 1)) * 2 + (e & 1)] = 0u;
    }
}

struct ProjArgs {
    const unsigned char *frags;                   // [token tiles][nseg] images of FRAG_BYTES
    void *y;                                      // [T][n_out]
    int T, n_out, nseg, ntiles, out_dtype;
    unsigned int *status;
};

// grid: ceil(n_out / 64) CTAs.  Warp w of group g owns weight rows 16 w .. 16 w + 15 of the CTA's 64 and the
// token tiles of group g (NG groups split the pass's tiles: more warps per SM to hide the latencies of a k-step).
// Per super-block one stage of shared memory holds the 64 weight rows (one tensor copy) and the activation images
// of the pass's token tiles (one bulk copy each); NSTAGE stages on NSTAGE mbarriers.
constexpr int CTA_ROWS = WARPS * ROWS;
constexpr int STAGE_W = CTA_ROWS * SEGB;          // 17408
constexpr int STAGE_X = MAXNT * FRAG_BYTES;       // 35072
constexpr int STAGE = STAGE_W + STAGE_X;
constexpr int NSTAGE = 3;
constexpr int PROJ_SMEM = NSTAGE * STAGE + 128;

__device__ __forceinline__ void bulk_copy(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

template <int NG>
__global__ void __launch_bounds__(NG * WARPS * 32) k_matmul_q8_0(ProjArgs a, const __grid_constant__ CUtensorMap map_w, int tok0) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[NSTAGE];
    __shared__ int failed;
    unsigned char *smem = smem_raw + ((128 - (smem_u32(smem_raw) & 127)) & 127);
    const int tid = threadIdx.x, lane = tid & 31, warp = (tid >> 5) & (WARPS - 1), grp = tid >> 7, r = lane >> 2, j = lane & 3;
    const int cta_row0 = (int)blockIdx.x * CTA_ROWS, row0 = cta_row0 + warp * ROWS;
    constexpr int MT = MAXNT / NG;                // token tiles of a group: tiles MT grp .. MT grp + MT - 1 of the pass
    const int nt_all = a.ntiles, t_lo = grp * MT;
    if (tid == 0) {
        failed = 0;
        for (int i = 0; i < NSTAGE; i++) mbar_init(smem_u32(&bars[i]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    auto issue = [&](int seg) {                   // rows past n_out are outside the map: the copy fills them with zeros
        const uint32_t bar = smem_u32(&bars[seg % NSTAGE]), base = smem_u32(smem + (seg % NSTAGE) * STAGE);
        mbar_expect_tx(bar, (uint32_t)(STAGE_W + nt_all * FRAG_BYTES));
        tensor_copy_rows(base, &map_w, seg * (SEGB / 4), cta_row0, bar);
        for (int t = 0; t < nt_all; t++)
            bulk_copy(base + STAGE_W + t * FRAG_BYTES, a.frags + ((size_t)((tok0 >> 3) + t) * a.nseg + seg) * FRAG_BYTES, FRAG_BYTES, bar);
    };
    if (tid == 0)
        for (int i = 0; i < NSTAGE - 1 && i < a.nseg; i++) issue(i);
    // Tiles past the pass's last one are multiplied too (against whatever the stage holds there) and never stored:
    // a test per tile would put every MMA into a basic block of its own and expose the latency of its fragment load.
    float tot[MT][4];
#pragma unroll
    for (int t = 0; t < MT; t++) tot[t][0] = tot[t][1] = tot[t][2] = tot[t][3] = 0.0f;
    const uint32_t lane_off = ((lane & 7) + ((lane >> 3) & 1) * 8) * SEGB + (lane >> 4) * 16;
    const bool active = row0 < a.n_out && t_lo < nt_all;
    bool ok = true;
    for (int seg = 0; seg < a.nseg; seg++) {
        const unsigned char *stage = smem + (seg % NSTAGE) * STAGE;
        if (ok && !mbar_wait(smem_u32(&bars[seg % NSTAGE]), (uint32_t)(seg / NSTAGE) & 1u)) { ok = false; failed = 1; }
        if (ok && active) {
            const unsigned char *wrows = stage + warp * (ROWS * SEGB);
            uint32_t dk0[8], dk1[8];
#pragma unroll
            for (int bb = 0; bb < 8; bb++) {
                const unsigned short u0 = *reinterpret_cast<const unsigned short *>(wrows + r * SEGB + 34 * bb);
                const unsigned short u1 = *reinterpret_cast<const unsigned short *>(wrows + (r + 8) * SEGB + 34 * bb);
                dk0[bb] = (uint32_t)u0 | ((uint32_t)u0 << 16);
                dk1[bb] = (uint32_t)u1 | ((uint32_t)u1 << 16);
            }
            float acc[MT][4];
#pragma unroll
            for (int t = 0; t < MT; t++) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f;
            const unsigned char *xst = stage + STAGE_W + t_lo * FRAG_BYTES;                   // this group's tile t at + t * FRAG_BYTES
            const uint32_t w_addr = smem_u32(wrows) + lane_off;
            uint32_t R[4], A[4];
#define PROJ_STEP(C, R0, R1)                                                   \
            weights_chunk<(C)>(R0, R1, dk0, dk1, j, A);                        \
            _Pragma("unroll")                                                  \
            for (int t = 0; t < MT; t++) {                                     \
                const uint2 b = reinterpret_cast<const uint2 *>(xst + t * FRAG_BYTES)[(C) * 32 + lane];   \
                mma16816(acc[t], A, b.x, b.y);                                 \
            }
#define PROJ_PAIR(C)                                                           \
            ldsm_x4(R, w_addr + (C) * 16);                                     \
            PROJ_STEP((C), R[0], R[1])                                         \
            PROJ_STEP((C) + 1, R[2], R[3])
            PROJ_PAIR(0) PROJ_PAIR(2) PROJ_PAIR(4) PROJ_PAIR(6) PROJ_PAIR(8) PROJ_PAIR(10) PROJ_PAIR(12) PROJ_PAIR(14)
            ldsm_x2(R, w_addr + 16 * 16);
            PROJ_STEP(16, R[0], R[1])
#undef PROJ_PAIR
#undef PROJ_STEP
            // the super-block's sum times the activation's scale (tokens 2j, 2j+1 of each tile)
#pragma unroll
            for (int t = 0; t < MT; t++) {
                const float2 d2 = reinterpret_cast<const float2 *>(xst + t * FRAG_BYTES + FRAG_WORDS2 * 8)[j];
                tot[t][0] = fmaf(d2.x, acc[t][0], tot[t][0]); tot[t][1] = fmaf(d2.y, acc[t][1], tot[t][1]);
                tot[t][2] = fmaf(d2.x, acc[t][2], tot[t][2]); tot[t][3] = fmaf(d2.y, acc[t][3], tot[t][3]);
            }
        }
        __syncthreads();                          // every warp is done with stage seg (and so with stage seg - 1, refilled now)
        if (tid == 0 && !failed && seg + NSTAGE - 1 < a.nseg) {
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            issue(seg + NSTAGE - 1);
        }
        if (failed) ok = false;
    }
    if (!ok && tid == 0 && a.status) atomicOr(a.status, ORN_WAIT_DECODE);
    // y[token][row]: rows r, r + 8 of the warp's 16; tokens 2j, 2j+1 of each tile
#pragma unroll
    for (int t = 0; t < MT; t++)
#pragma unroll
        for (int x = 0; x < 4; x++) {
            const int row = row0 + r + 8 * (x >> 1), tok = tok0 + 8 * (t_lo + t) + 2 * j + (x & 1);
            if (row < a.n_out && t_lo + t < nt_all && tok < a.T) {
                const float val = ok ? tot[t][x] : NAN;
                if (a.out_dtype == ORNITH_ACT_BF16) act_st((__nv_bfloat16 *)a.y, (size_t)tok * a.n_out + row, val);
                else act_st((float *)a.y, (size_t)tok * a.n_out + row, val);
            }
        }
}

// the weight matrix as [n_out rows][row_bytes / 4 words]; one box = 64 rows x 68 words (one super-block)
bool weight_map(CUtensorMap *m, const void *W, int n_in, int n_out) {
    OrnTensorMapEncodeFn enc = orn_tensor_map_encoder();
    if (!enc || ((uintptr_t)W & 15) != 0) return false;
    const cuuint64_t row_bytes = (cuuint64_t)n_in / 32 * 34;
    cuuint64_t dims[2] = {row_bytes / 4, (cuuint64_t)n_out};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {SEGB / 4, WARPS * ROWS};
    cuuint32_t es[2] = {1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(W), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

size_t frag_bytes(int T, int n_in) { return align_up((size_t)((T + 7) / 8) * (n_in / QK) * FRAG_BYTES, 256); }

}  // namespace

// x [T][n_in] -> the integer image of its Q8_K form (see k_q8k_quantize); img: orn_q8k_image_bytes(T, n_in) bytes
size_t orn_q8k_image_bytes(int T, int n_in) { return align_up((size_t)((T + 7) / 8) * (n_in / QK) * ORN_Q8K_IMG_BYTES, 256); }
ornith_status orn_q8k_quantize_image(const void *x, int act_dtype, int T, int n_in, void *img, cudaStream_t stream) {
    dim3 grid(n_in / QK, (T + 7) / 8 * 8);
    if (act_dtype == ORNITH_ACT_BF16)
        k_q8k_quantize<__nv_bfloat16><<<grid, 32, 0, stream>>>((const __nv_bfloat16 *)x, T, n_in, nullptr, nullptr, (unsigned char *)img);
    else
        k_q8k_quantize<float><<<grid, 32, 0, stream>>>((const float *)x, T, n_in, nullptr, nullptr, (unsigned char *)img);
    return orn_check_launch("k_q8k_quantize");
}

extern "C" {

size_t ornith_cuda_qproj_scratch(int T, int n_in) {
    if (T <= 0 || n_in <= 0 || n_in % QK) return 0;
    return frag_bytes(T, n_in);
}

// x [T][n_in] (act_dtype) -> Q8_K.  blocks: device [T][n_in/256][292] in the engine's layout, or NULL.
// scratch: ornith_cuda_qproj_scratch(T, n_in) bytes, 256-byte aligned: the image ornith_cuda_matmul_q8_0_q8k reads.
ornith_status ornith_cuda_q8k_quantize(const void *x, int act_dtype, int T, int n_in, void *blocks, void *scratch,
                                       size_t scratch_bytes, void *stream) {
    ORN_TRY(orn_require_device());
    if (T <= 0) return ORNITH_OK;
    if (n_in <= 0 || n_in % QK) { orn_record_error("q8k_quantize: the row length must be a multiple of 256 (got %d)", n_in); return ORNITH_ERR_FORMAT; }
    if (!scratch || scratch_bytes < ornith_cuda_qproj_scratch(T, n_in)) { orn_record_error("q8k_quantize: scratch too small"); return ORNITH_ERR_FORMAT; }
    uint2 *frags = (uint2 *)scratch;
    dim3 grid(n_in / QK, (T + 7) / 8 * 8);
    if (act_dtype == ORNITH_ACT_BF16)
        k_q8k_quantize<__nv_bfloat16><<<grid, 32, 0, (cudaStream_t)stream>>>((const __nv_bfloat16 *)x, T, n_in, (unsigned char *)blocks, frags, nullptr);
    else
        k_q8k_quantize<float><<<grid, 32, 0, (cudaStream_t)stream>>>((const float *)x, T, n_in, (unsigned char *)blocks, frags, nullptr);
    return orn_check_launch("k_q8k_quantize");
}

// y [T][n_out] = x [T][n_in] through W: device Q8_0 rows [n_out][n_in/32][34] (16-byte aligned, the GGUF tensor
// bytes as they are).  Quantises x into `scratch` first, then the product.  out_dtype: ORNITH_ACT_F32 / _BF16.
ornith_status ornith_cuda_matmul_q8_0(const void *W, int n_in, int n_out, const void *x, int act_dtype, int T, void *y,
                                      int out_dtype, void *scratch, size_t scratch_bytes, void *stream) {
    ORN_TRY(orn_require_device());
    if (T <= 0 || n_out <= 0) return ORNITH_OK;
    ORN_TRY(ornith_cuda_q8k_quantize(x, act_dtype, T, n_in, nullptr, scratch, scratch_bytes, stream));
    CUtensorMap map;
    if (!weight_map(&map, W, n_in, n_out)) { orn_record_error("matmul_q8_0: the weight rows must be 16-byte aligned"); return ORNITH_ERR_FORMAT; }
    ProjArgs a;
    a.frags = (const unsigned char *)scratch;
    a.y = y; a.T = T; a.n_out = n_out; a.nseg = n_in / QK; a.out_dtype = out_dtype; a.status = orn_status_word();
    const int grid = (n_out + WARPS * ROWS - 1) / (WARPS * ROWS);
    static bool configured_dev[ORN_MAX_DEVICES] = {};
    bool &configured = configured_dev[orn_device_index()];
    if (!configured) {
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_matmul_q8_0<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, PROJ_SMEM), "projection smem opt-in"));
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_matmul_q8_0<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, PROJ_SMEM), "projection smem opt-in"));
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_matmul_q8_0<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, PROJ_SMEM), "projection smem opt-in"));
        configured = true;
    }
    static int groups = -1;                       // ORNITH_CUDA_PROJ_GROUPS=1|2|4 caps the warp groups per CTA (default 4)
    if (groups < 0) { const char *e = getenv("ORNITH_CUDA_PROJ_GROUPS"); groups = e ? atoi(e) : 4; }
    for (int tok0 = 0; tok0 < T; tok0 += 8 * MAXNT) {                 // 64 tokens per pass over the weights
        a.ntiles = ((T - tok0 < 8 * MAXNT ? T - tok0 : 8 * MAXNT) + 7) / 8;
        // a group handles MAXNT / NG consecutive tiles of the pass; groups without a tile idle (every group multiplies
        // all of its MAXNT / NG tiles, so few groups would mean many wasted products for a small batch)
        // (measured at 2048 -> 8192: 64 tokens 17.7 us with 2 groups, 20.5 with 4; 1-16 tokens 10.8-11.8 us with 4, 12.6-13.5 with 2)
        const int want = a.ntiles > 4 ? 2 : 4, ng = groups >= want ? want : (groups >= 2 ? 2 : 1);
        if (ng == 4)      k_matmul_q8_0<4><<<grid, 4 * WARPS * 32, PROJ_SMEM, (cudaStream_t)stream>>>(a, map, tok0);
        else if (ng == 2) k_matmul_q8_0<2><<<grid, 2 * WARPS * 32, PROJ_SMEM, (cudaStream_t)stream>>>(a, map, tok0);
        else              k_matmul_q8_0<1><<<grid, WARPS * 32, PROJ_SMEM, (cudaStream_t)stream>>>(a, map, tok0);
        ORN_TRY(orn_check_launch("k_matmul_q8_0"));
    }
    return ORNITH_OK;
}

}  // extern "C"
