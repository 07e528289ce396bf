// gqa_decode_i8_raw.cu — split-K GQA decode over int8-per-head rows (the engine's own quantised
// cache: 256 codes per row and one f32 scale per row in a side array), groups of up to 16 query
// heads (two CTAs of 8 heads beyond 8), head_dim 256.  The structure is that of the Q8_0 kernel (gqa_decode_q8_raw.cu).
//
// Replaces the attend half of ornith_gqa_step for kv->quantized caches (reference:
// src/ornith_attn.c:111-148, codec src/ornith_attn.c:24-47).
//
// A row is 16 aligned 16-byte chunks of 16 codes, and ldmatrix moves them as they are:
//   K (A operand, tokens on M): plain ldmatrix hands lane (token r, quarter j) the codes of
//     dims 16c+4j .. 16c+4j+3 of chunk c — the two f16 pairs one k-step needs; the query B
//     fragments are built in the same order once per CTA.  One chunk = one k-step.
//   V (A operand of O^T = V^T P^T): ldmatrix.trans hands lane (element r, token pair j) the
//     codes of dims 16c+2r, 16c+2r+1 for two tokens; the int8 -> f16 byte permute pairs the two
//     tokens of the even dim (row r of the m-tile) and of the odd dim (row r + 8).
// The row scales never touch the elements: the K scale multiplies the score of its token after
// the MMAs, the V scale is folded into the probability of its token before the MMAs.  Rows are
// staged with one 256-byte cp.async.bulk each into slots with a 272-byte row pitch (256 would
// put the eight rows of an ldmatrix phase on the same banks).
//
// Precision: q scaled per head by a power of two and rounded to f16; the codes are exact in
// f16; probabilities times their V scale carry one f16 rounding; f32 accumulation.
#include "full_attn.cuh"

namespace {

constexpr int HD = 256;
constexpr int ROWB = 272;                          // row pitch of a staging slot
constexpr int ROWC = 256;                          // bytes of a cached row
constexpr int TILE = 16;
constexpr int NWARP = 4;
constexpr int NCHUNK = 16;                         // 16-byte chunks per row
constexpr int RAW_TILE = TILE * ROWB;              // 4352
constexpr int QS_BYTES = NCHUNK * 32 * 8;          // query B fragments, [k-step][lane] x 2 words = 4352
constexpr int WARP_BYTES = 2 * RAW_TILE;           // one slot of K rows + one of V rows = 8704
constexpr int SMEM_BYTES = QS_BYTES + NWARP * WARP_BYTES;     // 39168: four CTAs per SM
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
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
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ uint32_t h2_sub(uint32_t biased) {   // x - 1152: the code as f16, exactly
    const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);
    __half2 v = __hsub2(*reinterpret_cast<__half2 *>(&biased), bias);
    return *reinterpret_cast<uint32_t *>(&v);
}

// ---- one k-step of S^T = K Q^T from chunk C of the staged K rows -------------------------
// raw0 / raw1: the lane's ldmatrix registers for token rows r and r + 8 (codes of dims
// 16C+4j .. 16C+4j+3).
template <int C>
__device__ __forceinline__ void qk_chunk(uint32_t raw0, uint32_t raw1, const uint2 *q_frag, float (&acc)[4]) {
    const uint32_t x0 = raw0 ^ 0x80808080u, x1 = raw1 ^ 0x80808080u;
    uint32_t A[4];
    A[0] = h2_sub(__byte_perm(x0, 0x64646464u, 0x4140));    // row r,   dims 16C+4j, +1   -> k = 2j, 2j+1
    A[1] = h2_sub(__byte_perm(x1, 0x64646464u, 0x4140));    // row r+8
    A[2] = h2_sub(__byte_perm(x0, 0x64646464u, 0x4342));    // row r,   dims 16C+4j+2, +3 -> k = 2j+8, 2j+9
    A[3] = h2_sub(__byte_perm(x1, 0x64646464u, 0x4342));
    const uint2 qv = q_frag[C * 32];                         // this lane's B fragment of k-step C
    mma16816(acc, A, qv.x, qv.y);
}

// ---- one m-tile of O^T += V^T P^T from chunk C of the staged V rows ------------------------
// raw0 / raw1: transposed-ldmatrix registers: codes of dims 16C+2r, 16C+2r+1 for tokens
// (2j, 2j+1) and (2j+8, 2j+9).
__device__ __forceinline__ void pv_chunk(uint32_t raw0, uint32_t raw1, uint32_t pb0, uint32_t pb1, float (&acc)[4]) {
    const uint32_t x0 = raw0 ^ 0x80808080u, x1 = raw1 ^ 0x80808080u;
    uint32_t A[4];
    A[0] = h2_sub(__byte_perm(x0, 0x64646464u, 0x4240));     // even dim, tokens 2j, 2j+1
    A[1] = h2_sub(__byte_perm(x0, 0x64646464u, 0x4341));     // odd dim (rows 8..15 of the m-tile)
    A[2] = h2_sub(__byte_perm(x1, 0x64646464u, 0x4240));     // even dim, tokens 2j+8, 2j+9
    A[3] = h2_sub(__byte_perm(x1, 0x64646464u, 0x4341));
    mma16816(acc, A, pb0, pb1);
}

// ---- bulk-copy staging: one 256-byte cp.async.bulk per row, completion on an mbarrier ------
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    // the suspend-time hint lets the hardware park the thread (no issue slots burnt on polling)
    // until the phase completes or ~10 us pass
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(10000u) : "memory");
    return ok != 0;
}
// bounded wait: gives up (returns false) after ~1 s instead of waiting for ever
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (int i = 0; i < (1 << 18); i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_copy_row(uint32_t dst, const void *src, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(src), "r"(ROWC), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// Stage the 16 rows of one tile of K (or V): lanes 0-15 copy one row each.  Rows past the
// end of the split are not copied: the slot keeps earlier (finite) contents and the token
// is masked in the softmax.
__device__ __forceinline__ void issue_rows16(unsigned char *slot, uint32_t bar, const unsigned char *src_base,
                                             size_t row_stride, int tok0, int t1, int lane) {
    const int valid = min(TILE, t1 - tok0);
    if (lane == 0) mbar_expect_tx(bar, (uint32_t)(valid * ROWC));
    __syncwarp();
    if (lane < valid) bulk_copy_row(smem_u32(slot + lane * ROWB), src_base + (size_t)(tok0 + lane) * row_stride, bar);
}

template <int C>
__device__ __forceinline__ void store_chunk(float *Ow, const float (&acc)[4], int r, int j) {
    const int dim = 16 * C + 2 * r;                // row r of the m-tile is the even dim, row r + 8 the odd one
    Ow[(2 * j) * HD + dim] = acc[0];
    Ow[(2 * j + 1) * HD + dim] = acc[1];
    Ow[(2 * j) * HD + dim + 1] = acc[2];
    Ow[(2 * j + 1) * HD + dim + 1] = acc[3];
}

__global__ void __launch_bounds__(128, 4) k_gqa_decode_i8_raw(DecodeArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float m_s[NWARP][8], l_s[NWARP][8];
    __shared__ __align__(8) unsigned long long bars[NWARP][2];
    __shared__ int pipe_failed;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    unsigned char *wbase = smem + QS_BYTES + warp * WARP_BYTES;
    uint2 *Q_s = reinterpret_cast<uint2 *>(smem);               // [k-step][lane]
    if (tid == 0) pipe_failed = 0;

    // KV head on the fastest grid axis: the CTAs that read the two interleaved halves of the
    // same token rows are launched side by side and share DRAM pages while they are open
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
    const int r = lane >> 2, j = lane & 3;

    // ---- query group -> B fragments in the order the K fragments have: lane (head r, quarter j),
    //      k-step c holds q at dims 16c+4j .. 16c+4j+3
    float rs_mine;
    {
        const float *q = a.q_prep + ((size_t)b * a.nh + (size_t)head0 + (r < G ? r : 0)) * HD;
        float mx = 0.0f;
        {   // 16 independent 128-bit loads: the prologue is per CTA, keep it off the latency path
            const float4 *q4 = reinterpret_cast<const float4 *>(q + j * 64);
            float4 t[16];
#pragma unroll
            for (int i = 0; i < 16; i++) t[i] = q4[i];
#pragma unroll
            for (int i = 0; i < 16; i++)
                mx = fmaxf(mx, fmaxf(fmaxf(fabsf(t[i].x), fabsf(t[i].y)), fmaxf(fabsf(t[i].z), fabsf(t[i].w))));
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        int e = 0;
        if (mx > 0.0f && mx < INFINITY) (void)frexpf(mx, &e);
        const float down = (r < G) ? exp2f((float)-e) : 0.0f;
        for (int c = warp; c < NCHUNK; c += NWARP) {      // the four warps share the work; identical per warp otherwise
            const float4 v = *reinterpret_cast<const float4 *>(q + 16 * c + 4 * j);
            Q_s[c * 32 + lane] = make_uint2(pack_h2(v.x * down, v.y * down), pack_h2(v.z * down, v.w * down));
        }
        rs_mine = (r < G) ? a.scale * exp2f((float)e) * LOG2E : 0.0f;
    }
    const float rsA = __shfl_sync(0xffffffffu, rs_mine, (2 * j) * 4);
    const float rsB = __shfl_sync(0xffffffffu, rs_mine, (2 * j + 1) * 4);

    const int ntiles = (t1 - t0 + TILE - 1) / TILE;
    const size_t row_stride = (size_t)nkv * ROWC;
    const unsigned char *Kbase = a.kv.K + ((size_t)base * nkv + kvh) * ROWC;
    const unsigned char *Vbase = a.kv.V + ((size_t)base * nkv + kvh) * ROWC;
    const float *Ksc = a.kv.Ks + (size_t)base * nkv + kvh, *Vsc = a.kv.Vs + (size_t)base * nkv + kvh;   // [token * nkv]

    float o[NCHUNK][4];
#pragma unroll
    for (int i = 0; i < NCHUNK; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float mA = -INFINITY, mB = -INFINITY, lA = 0.0f, lB = 0.0f;
    // ldmatrix row address of this lane inside a staged tile: matrices 0,1 = chunk c (tokens 0-7, 8-15),
    // matrices 2,3 = chunk c + 1
    const uint32_t lane_off = ((lane & 7) + ((lane >> 3) & 1) * 8) * ROWB + (lane >> 4) * 16;

    // ---- per-warp staging slots (K rows, V rows): zero them once (skipped tail rows must stay
    //      finite), one mbarrier each.  K of the next tile is requested as soon as the score
    //      loop is done with the slot, V right after the value loop.
    unsigned char *rawK = wbase, *rawV = wbase + RAW_TILE;
    {
        uint4 *z = reinterpret_cast<uint4 *>(wbase);
        for (int i = lane; i < WARP_BYTES / 16; i += 32) z[i] = make_uint4(0u, 0u, 0u, 0u);
        if (lane == 0) {
            mbar_init(smem_u32(&bars[warp][0]), 1);
            mbar_init(smem_u32(&bars[warp][1]), 1);
            asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        }
        fence_proxy_async();                                      // generic-proxy zeros before async-proxy copies
    }
    __syncthreads();                                              // also publishes Q_s
    const uint32_t barK = smem_u32(&bars[warp][0]), barV = smem_u32(&bars[warp][1]);
    const uint2 *q_frag = Q_s + lane;
    bool pipe_ok = true;

    int it = warp;
    if (it < ntiles) {
        issue_rows16(rawK, barK, Kbase, row_stride, t0 + it * TILE, t1, lane);
        issue_rows16(rawV, barV, Vbase, row_stride, t0 + it * TILE, t1, lane);
    }
    for (uint32_t n = 0; it < ntiles; it += NWARP, n++) {
        const int tok0 = t0 + it * TILE;
        const bool more = it + NWARP < ntiles;
        if (!mbar_wait(barK, n & 1)) {
            (void)mbar_wait(barV, n & 1);                         // bounded chance for the other copy to drain
            pipe_ok = false;
            break;
        }

        // row scales of this lane's tokens (rows r, r + 8 of the tile); tokens past the split read token t1 - 1
        const int tk0 = min(tok0 + r, t1 - 1), tk1 = min(tok0 + r + 8, t1 - 1);
        const float ks0 = Ksc[(size_t)tk0 * nkv], ks1 = Ksc[(size_t)tk1 * nkv];
        const float vs0 = Vsc[(size_t)tk0 * nkv], vs1 = Vsc[(size_t)tk1 * nkv];

        // ---- S^T = K Q^T: 16 k-steps in two accumulator chains -----------------------------
        float s[4] = {0.0f, 0.0f, 0.0f, 0.0f}, s2[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const uint32_t k_addr = smem_u32(rawK) + lane_off;
        {
            uint32_t R[4];
#define QK_PAIR(C)                                                \
            ldsm_x4(R, k_addr + (C) * 16);                        \
            qk_chunk<(C)>(R[0], R[1], q_frag, s);                 \
            qk_chunk<(C) + 1>(R[2], R[3], q_frag, s2);
            QK_PAIR(0) QK_PAIR(2) QK_PAIR(4) QK_PAIR(6) QK_PAIR(8) QK_PAIR(10) QK_PAIR(12) QK_PAIR(14)
#undef QK_PAIR
        }
        __syncwarp();                                             // every lane is done with the K slot
        if (more) {
            fence_proxy_async();
            issue_rows16(rawK, barK, Kbase, row_stride, tok0 + NWARP * TILE, t1, lane);
        }

        // ---- online softmax over tokens (rows r, r+8); columns = heads 2j, 2j+1 -------------
        const bool ok0 = tok0 + r < t1, ok1 = tok0 + r + 8 < t1;
        float x00 = ok0 ? (s[0] + s2[0]) * (rsA * ks0) : -INFINITY, x01 = ok0 ? (s[1] + s2[1]) * (rsB * ks0) : -INFINITY;
        float x10 = ok1 ? (s[2] + s2[2]) * (rsA * ks1) : -INFINITY, x11 = ok1 ? (s[3] + s2[3]) * (rsB * ks1) : -INFINITY;
        float cA = fmaxf(x00, x10), cB = fmaxf(x01, x11);
#pragma unroll
        for (int sft = 4; sft <= 16; sft <<= 1) {
            cA = fmaxf(cA, __shfl_xor_sync(0xffffffffu, cA, sft));
            cB = fmaxf(cB, __shfl_xor_sync(0xffffffffu, cB, sft));
        }
        const float nA = fmaxf(mA, cA), nB = fmaxf(mB, cB);       // finite: token tok0 is valid
        const float corrA = exp2f(mA - nA), corrB = exp2f(mB - nB);
        mA = nA; mB = nB;
        x00 = exp2f(x00 - nA); x10 = exp2f(x10 - nA); x01 = exp2f(x01 - nB); x11 = exp2f(x11 - nB);
        lA = lA * corrA + x00 + x10;
        lB = lB * corrB + x01 + x11;
        if (__any_sync(0xffffffffu, corrA != 1.0f || corrB != 1.0f)) {
#pragma unroll
            for (int i = 0; i < NCHUNK; i++) { o[i][0] *= corrA; o[i][1] *= corrB; o[i][2] *= corrA; o[i][3] *= corrB; }
        }
        // the V scale of a token rides on its probability
        const float w0 = 256.0f * vs0, w1 = 256.0f * vs1;
        const uint32_t pb0 = movmatrix_trans(pack_h2(x00 * w0, x01 * w0));
        const uint32_t pb1 = movmatrix_trans(pack_h2(x10 * w1, x11 * w1));

        // ---- O^T += V^T P^T: one m-tile per chunk ---------------------------------------------
        if (!mbar_wait(barV, n & 1)) {
            if (more) (void)mbar_wait(barK, (n + 1) & 1);
            pipe_ok = false;
            break;
        }
        const uint32_t v_addr = smem_u32(rawV) + lane_off;
        {
            uint32_t R[4];
#define PV_PAIR(C)                                                \
            ldsm_x4_trans(R, v_addr + (C) * 16);                  \
            pv_chunk(R[0], R[1], pb0, pb1, o[(C)]);               \
            pv_chunk(R[2], R[3], pb0, pb1, o[(C) + 1]);
            PV_PAIR(0) PV_PAIR(2) PV_PAIR(4) PV_PAIR(6) PV_PAIR(8) PV_PAIR(10) PV_PAIR(12) PV_PAIR(14)
#undef PV_PAIR
        }
        __syncwarp();                                             // every lane is done with the V slot
        if (more) {
            fence_proxy_async();
            issue_rows16(rawV, barV, Vbase, row_stride, tok0 + NWARP * TILE, t1, lane);
        }
    }
    if (!pipe_ok && lane == 0) pipe_failed = 1;
    __syncwarp();

    // ---- merge the four warps, one partial per (head, split) -----------------------------------
#pragma unroll
    for (int sft = 4; sft <= 16; sft <<= 1) {
        lA += __shfl_xor_sync(0xffffffffu, lA, sft);
        lB += __shfl_xor_sync(0xffffffffu, lB, sft);
    }
    float *Ow = reinterpret_cast<float *>(wbase);                 // [8 heads][256] f32 over this warp's slots
    store_chunk<0>(Ow, o[0], r, j);   store_chunk<1>(Ow, o[1], r, j);   store_chunk<2>(Ow, o[2], r, j);
    store_chunk<3>(Ow, o[3], r, j);   store_chunk<4>(Ow, o[4], r, j);   store_chunk<5>(Ow, o[5], r, j);
    store_chunk<6>(Ow, o[6], r, j);   store_chunk<7>(Ow, o[7], r, j);   store_chunk<8>(Ow, o[8], r, j);
    store_chunk<9>(Ow, o[9], r, j);   store_chunk<10>(Ow, o[10], r, j); store_chunk<11>(Ow, o[11], r, j);
    store_chunk<12>(Ow, o[12], r, j); store_chunk<13>(Ow, o[13], r, j); store_chunk<14>(Ow, o[14], r, j);
    store_chunk<15>(Ow, o[15], r, j);
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
        // a staging copy that never completed poisons the partial (the result becomes NaN, not silently wrong)
        const float poison = pipe_failed ? NAN : 0.0f;
        if (tid == 0) { part[0] = M * LN2; part[1] = pipe_failed ? 1.0f : Lt; }
        for (int d = tid; d < HD; d += 128) {
            float acc = 0.0f;
#pragma unroll
            for (int w = 0; w < NWARP; w++)
                acc += ww[w] * reinterpret_cast<const float *>(smem + QS_BYTES + w * WARP_BYTES)[h * HD + d];
            part[2 + d] = acc * (1.0f / 256.0f) + poison;
        }
    }
}

}  // namespace

bool gqa_decode_i8_raw_supported(const KvView &kv, int nh) {
    return kv.mode == ORNITH_KV_INT8_HEAD && kv.hd == HD && nh % kv.nkv == 0 && nh / kv.nkv <= 16 &&
           ((uintptr_t)kv.K % 16) == 0 && ((uintptr_t)kv.V % 16) == 0;
}

ornith_status launch_gqa_decode_i8_raw(const DecodeArgs &a, int n_seq, cudaStream_t st) {
    static bool configured_dev[ORN_MAX_DEVICES] = {};
    bool &configured = configured_dev[orn_device_index()];
    if (!configured) {
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_gqa_decode_i8_raw, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               SMEM_BYTES), "int8 gqa decode smem opt-in"));
        configured = true;
    }
    dim3 grid(a.kv.nkv * ((a.nh / a.kv.nkv + 7) / 8), a.nsplit, n_seq);
    k_gqa_decode_i8_raw<<<grid, 128, SMEM_BYTES, st>>>(a);
    return orn_check_launch("k_gqa_decode_i8_raw");
}
