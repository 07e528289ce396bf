// gqa_decode_q8_raw.cu — split-K GQA decode over Q8_0 rows, fragments taken straight
// from the staged raw bytes (groups of up to 8 query heads, head_dim 256).
//
// Replaces the attend half of ornith_gqa_step (reference: src/ornith_attn.c:111-148).
//
// A Q8_0 row of 256 values is 8 blocks of {f16 scale, 32 int8} = 272 bytes.  Read
// as a stream of 136 16-bit elements it is  [scale, 16 code pairs] x 8, and the
// 17 aligned 16-byte chunks of the row are exactly what ldmatrix moves:
//
//   K (A operand, tokens on M): plain ldmatrix hands lane (token r, quarter j) the
//     elements 8c+2j and 8c+2j+1 of chunk c — four codes, i.e. the two f16 pairs
//     one k-step needs.  The contraction index is whatever order the stream has;
//     the query B fragments are built in the same order once per CTA, with zeros
//     where the stream holds a scale.  One chunk = one k-step, 17 per tile.
//   V (A operand of O^T = V^T P^T): ldmatrix.trans hands lane (element r, token
//     pair j) one stream element for two tokens: codes (d, d+1) x (t, t+1).  The
//     int8 -> f16 byte permute picks (t, t+1) of dim d and of dim d+1, which are
//     the rows of two 8-row halves of one m-tile.  One chunk = one m-tile; the
//     lane whose element is the block's scale holds both tokens' scales as an
//     f16 pair and broadcasts it with one shuffle.
//
// Nothing is decoded into a second shared-memory buffer: per 16-token tile the
// shared-memory pipe moves the staged bytes once in and once out (ldmatrix), plus 16
// two-byte scale loads for K.
//
// Staging: the rows of one KV head are 272 bytes long and nkv * 272 bytes apart.  A full
// 16-token tile is fetched by ONE tensor copy (cp.async.bulk.tensor, 3-d view
// [token][kv head][68 words], box 16 x 1 x 68) that lands the rows back to back; a
// per-row bulk copy costs a dozen issue slots per row (the copy instruction takes uniform
// registers, so per-lane addresses are walked one lane at a time), which was a third of all
// instructions of this kernel.  Only the ragged last tile of a split still uses row copies.
//
// Precision: as the other tensor-core decode kernel — q scaled per head by a
// power of two and rounded to f16, decoded K/V elements carry one f16 rounding,
// probabilities scaled by 2^8 before the f16 rounding, f32 accumulation.
#include <cuda.h>
#include "full_attn.cuh"

namespace {

constexpr int HD = 256;
constexpr int ROWB = 272;
constexpr int TILE = 16;
constexpr int NWARP = 4;
constexpr int NCHUNK = 17;                         // 16-byte chunks per row
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
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
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
__device__ __forceinline__ uint32_t h2_mul_sub(uint32_t biased, uint32_t scale) {   // (x - 1152) * scale
    const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);
    __half2 v = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&biased), bias), *reinterpret_cast<__half2 *>(&scale));
    return *reinterpret_cast<uint32_t *>(&v);
}

// stream element e of a row: block e / 17; index 0 of a block is its scale, index i > 0
// is the code pair of dims 2(i-1), 2(i-1)+1.
__host__ __device__ constexpr int elem_block(int e) { return e / 17; }

// ---- one k-step of S^T = K Q^T from chunk C of the staged K rows -------------------------
// raw0 / raw1: the lane's ldmatrix registers for token rows r and r + 8 (elements
// 8C+2j and 8C+2j+1); dk0 / dk1: that row's block scales as f16 pairs.
template <int C>
__device__ __forceinline__ void qk_chunk(uint32_t raw0, uint32_t raw1, const uint32_t (&dk0)[8], const uint32_t (&dk1)[8],
                                         int j, const uint2 *q_frag, float (&acc)[4]) {
    constexpr int BLO = elem_block(8 * C), BHI = elem_block(8 * C + 7) > 7 ? 7 : elem_block(8 * C + 7);
    // block of element 8C+2j+h: BHI once the element index reaches 17*BHI
    const bool hi0 = (BHI != BLO) && (8 * C + 2 * j >= 17 * BHI);
    const bool hi1 = (BHI != BLO) && (8 * C + 2 * j + 1 >= 17 * BHI);
    const uint32_t s00 = hi0 ? dk0[BHI] : dk0[BLO], s01 = hi1 ? dk0[BHI] : dk0[BLO];
    const uint32_t s10 = hi0 ? dk1[BHI] : dk1[BLO], s11 = hi1 ? dk1[BHI] : dk1[BLO];
    const uint32_t x0 = raw0 ^ 0x80808080u, x1 = raw1 ^ 0x80808080u;
    uint32_t A[4];
    A[0] = h2_mul_sub(__byte_perm(x0, 0x64646464u, 0x4140), s00);    // row r,   element 8C+2j   -> k = 2j, 2j+1
    A[1] = h2_mul_sub(__byte_perm(x1, 0x64646464u, 0x4140), s10);    // row r+8
    A[2] = h2_mul_sub(__byte_perm(x0, 0x64646464u, 0x4342), s01);    // row r,   element 8C+2j+1 -> k = 2j+8, 2j+9
    A[3] = h2_mul_sub(__byte_perm(x1, 0x64646464u, 0x4342), s11);
    const uint2 qv = q_frag[C * 32];                                 // this lane's B fragment of k-step C
    mma16816(acc, A, qv.x, qv.y);
}

__device__ __forceinline__ unsigned short lds_u16(uint32_t addr) {
    unsigned short u;
    asm volatile("ld.shared.u16 %0, [%1];\n" : "=h"(u) : "r"(addr));
    return u;
}

// ---- one m-tile of O^T += V^T P^T from chunk C of the staged V rows ------------------------
// raw0 / raw1: transposed-ldmatrix registers: element 8C+r for tokens (2j, 2j+1) and
// (2j+8, 2j+9).  sc*: the f16 scale pairs of the two candidate blocks for those tokens.
template <int C>
__device__ __forceinline__ void pv_chunk(uint32_t raw0, uint32_t raw1, uint32_t sc_lo0, uint32_t sc_lo1,
                                         uint32_t sc_hi0, uint32_t sc_hi1, int r, uint32_t pb0, uint32_t pb1,
                                         float (&acc)[4]) {
    constexpr int BLO = elem_block(8 * C), BHI = elem_block(8 * C + 7) > 7 ? 7 : elem_block(8 * C + 7);
    const bool hi = (BHI != BLO) && (8 * C + r >= 17 * BHI);
    const uint32_t s0 = hi ? sc_hi0 : sc_lo0, s1 = hi ? sc_hi1 : sc_lo1;
    const uint32_t x0 = raw0 ^ 0x80808080u, x1 = raw1 ^ 0x80808080u;
    uint32_t A[4];
    A[0] = h2_mul_sub(__byte_perm(x0, 0x64646464u, 0x4240), s0);     // even dim, tokens 2j, 2j+1
    A[1] = h2_mul_sub(__byte_perm(x0, 0x64646464u, 0x4341), s0);     // odd dim (rows 8..15 of the m-tile)
    A[2] = h2_mul_sub(__byte_perm(x1, 0x64646464u, 0x4240), s1);     // even dim, tokens 2j+8, 2j+9
    A[3] = h2_mul_sub(__byte_perm(x1, 0x64646464u, 0x4341), s1);
    mma16816(acc, A, pb0, pb1);
}

// ---- bulk-copy staging: one 272-byte cp.async.bulk per row, completion on an mbarrier ------
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
                 ::"r"(dst), "l"(src), "r"(ROWB), "r"(bar) : "memory");
}
__device__ __forceinline__ void tensor_copy_tile(uint32_t dst, const CUtensorMap *map, int head, int token, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(0), "r"(head), "r"(token) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// Stage the 16 rows of one tile of K (or V).  A full tile is one tensor copy (map != nullptr;
// tok_abs = the tile's first token counted from the start of the pool); otherwise lanes 0-15
// copy one row each, and rows past the end of the piece are not copied: the slot keeps
// earlier (finite) contents and the token is masked in the softmax.  The row addresses of
// that rare path are worked out here, from the pool, rather than carried through the tile loop.
__device__ __forceinline__ void issue_rows16(uint32_t slot, uint32_t bar, const unsigned char *pool, int nkv,
                                             int valid, int lane, const CUtensorMap *map, int head, int tok_abs) {
    if (map != nullptr && valid >= TILE) {
        if (lane == 0) {
            mbar_expect_tx(bar, (uint32_t)RAW_TILE);
            tensor_copy_tile(slot, map, head, tok_abs, bar);
        }
        return;
    }
    valid = min(valid, TILE);
    if (lane == 0) mbar_expect_tx(bar, (uint32_t)(valid * ROWB));
    __syncwarp();
    if (lane < valid) bulk_copy_row(slot + lane * ROWB, pool + ((size_t)(tok_abs + lane) * nkv + head) * ROWB, bar);
}

template <int C>
__device__ __forceinline__ void store_chunk(float *Ow, const float (&acc)[4], int r, int j) {
    const int e = 8 * C + r;
    if (e % 17 == 0 || e >= 136) return;          // this lane's rows of the m-tile were a scale, not values
    const int dim = 32 * (e / 17) + 2 * (e % 17 - 1);
    Ow[(2 * j) * HD + dim] = acc[0];
    Ow[(2 * j + 1) * HD + dim] = acc[1];
    Ow[(2 * j) * HD + dim + 1] = acc[2];
    Ow[(2 * j + 1) * HD + dim + 1] = acc[3];
}

// Tiles (16 tokens) a decode step reads for sequence b: its context plus the token being appended; nothing for a
// sequence whose cache is full (the step leaves it alone).
__device__ __forceinline__ int seq_tiles(const DecodeArgs &a, int b) {
    const int len0 = a.kv_len[b];
    const int cap = (int)(a.kv.seq_off[b + 1] - a.kv.seq_off[b]);
    return len0 >= cap ? 0 : (len0 + TILE) / TILE;
}

// Inclusive prefix sum of v over the 128 threads of the CTA; *total = the sum.  wt: 4 ints of shared memory.
__device__ __forceinline__ int block_scan128(int v, int *wt, int *total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    if (lane == 31) wt[warp] = incl;
    __syncthreads();
    int add = 0, tot = 0;
#pragma unroll
    for (int w = 0; w < NWARP; w++) { const int x = wt[w]; if (w < warp) add += x; tot += x; }
    __syncthreads();
    *total = tot;
    return incl + add;
}

// BALANCED = false: one CTA per (head group, split of tokens_per_split tokens, sequence); grid (groups, nsplit, n_seq).
// BALANCED = true:  grid (groups, ranges).  The 16-token tiles of all sequences, laid end to end, are cut into
//   gridDim.y ranges of equal length (found on the device from kv_len: the host never learns the contexts), and a
//   CTA walks the pieces of the sequences that fall into its range, one partial per piece.  Every CTA is resident
//   at once and all of them stream the same number of rows, so no SM runs dry before the others; a sequence
//   shorter than a range costs one partial, a longer one as many as the ranges it touches.  The CTAs of the head
//   groups that share the same rows (blockIdx.x) walk the same range side by side.
template <bool BALANCED>
__global__ void __launch_bounds__(128, 4) k_gqa_decode_q8_raw(DecodeArgs a, const __grid_constant__ CUtensorMap map_k,
                                                              const __grid_constant__ CUtensorMap map_v, int tensor_copies) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ float m_s[NWARP][8], l_s[NWARP][8];
    __shared__ __align__(8) unsigned long long bars[NWARP][2];
    __shared__ int pipe_failed, last_one, scan_s[NWARP], found_s[2];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // the next layer's front-end kernel may become resident now; it waits for this grid before it does anything
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    unsigned char *wbase = smem + QS_BYTES + warp * WARP_BYTES;
    uint2 *Q_s = reinterpret_cast<uint2 *>(smem);               // [k-step][lane]
    if (tid == 0) pipe_failed = 0;
    if (lane == 0) {
        mbar_init(smem_u32(&bars[warp][0]), 1);
        mbar_init(smem_u32(&bars[warp][1]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }

    // a group of more than 8 query heads is walked by two CTAs of 8 heads each; they and the CTAs of the other KV
    // heads sit side by side on the fastest grid axis: the rows of the KV heads interleave in memory, so these CTAs
    // share DRAM pages while they are open, and the second CTA of a group finds the rows of the first one in L2
    const int nkv = a.kv.nkv, Gall = a.nh / nkv, sub = (Gall + 7) / 8;
    const int kvh = (int)blockIdx.x / sub, hs = (int)blockIdx.x % sub;
    const int G = min(8, Gall - 8 * hs), head0 = kvh * Gall + 8 * hs;
    const int r = lane >> 2, j = lane & 3;
    const CUtensorMap *mk = tensor_copies ? &map_k : nullptr, *mv = tensor_copies ? &map_v : nullptr;
    const uint32_t barK = smem_u32(&bars[warp][0]), barV = smem_u32(&bars[warp][1]);
    const uint32_t rawK = smem_u32(wbase), rawV = rawK + RAW_TILE;      // staging slots, as shared-memory addresses
    // ldmatrix row address of this lane inside a staged tile: matrices 0,1 = chunk c (tokens 0-7, 8-15),
    // matrices 2,3 = chunk c + 1
    const uint32_t lane_off = ((lane & 7) + ((lane >> 3) & 1) * 8) * ROWB + (lane >> 4) * 16;

    // ---- the range of this CTA (kv_len and seq_off are not written by the kernel in front, so this runs before
    //      the wait on it) ------------------------------------------------------------------------------------
    // the walk's state lives in shared memory (the tile loop needs every register): sequence b, index of its first
    // tile, next tile to read, end of the range, range length
    __shared__ int walk_s[9];                                    // [5..8]: sequence, slot, first slot and partial count of the current piece
    if (BALANCED) {
        // Ranges are cut in units of cost: a tile costs 1, and every sequence is charged a.piece_cost extra units in
        // front of its first tile for the fixed work of a piece (query fragments, restart of the copy pipeline,
        // partial write), so a CTA that walks pieces of several sequences gets fewer tiles.
        const int pad = a.piece_cost;
        int pos, range_end, W, total = 0, mine_n = 0, mine_incl = 0;
        for (int b0 = 0; b0 < a.n_seq; b0 += 128) {
            const int n = b0 + tid < a.n_seq ? seq_tiles(a, b0 + tid) : 0;
            int t;
            const int incl = block_scan128(n ? n + pad : 0, scan_s, &t);
            if (b0 == 0) { mine_n = n; mine_incl = incl; }           // kept for the search below when the batch is one pass
            total += t;
        }
        // range length: an equal share, but no shorter than 16 tiles nor than 1/32 of the longest context the call
        // allows (the last CTA of a sequence merges its partials alone; past ~32 of them that outweighs the gain)
        const int floor_w = max(16, ((a.max_len + TILE - 1) / TILE + 31) / 32);
        W = max((total + (int)gridDim.y - 1) / (int)gridDim.y, floor_w);
        pos = (int)blockIdx.y * W;
        range_end = min(total, pos + W);
        if (pos >= total) { asm volatile("griddepcontrol.wait;\n" ::: "memory"); return; }
        // the sequence whose units hold `pos`
        if (a.n_seq <= 128) {
            const int cost = mine_n ? mine_n + pad : 0;
            if (mine_incl - cost <= pos && pos < mine_incl) { found_s[0] = tid; found_s[1] = mine_incl - cost; }
        } else {
            int running = 0;
            for (int b0 = 0; b0 < a.n_seq; b0 += 128) {
                const int n = b0 + tid < a.n_seq ? seq_tiles(a, b0 + tid) : 0, cost = n ? n + pad : 0;
                int t;
                const int incl = running + block_scan128(cost, scan_s, &t);
                if (incl - cost <= pos && pos < incl) { found_s[0] = b0 + tid; found_s[1] = incl - cost; }
                running += t;
                if (running > pos) break;
            }
        }
        __syncthreads();
        if (tid == 0) { walk_s[0] = found_s[0]; walk_s[1] = found_s[1]; walk_s[2] = pos; walk_s[3] = range_end; walk_s[4] = W; }
        __syncthreads();
    }

    uint32_t phase = 0;                                           // tiles this warp has consumed: parity of its two barriers
    bool pipe_ok = true, waited = false;
    for (bool first_piece = true;; first_piece = false) {
        // ---- next piece: tiles [tile_lo, tile_hi) of sequence b --------------------------------------------------
        int tile_lo, tile_hi, slot, slot0, nlive, len0, b;
        if (BALANCED) {
            if (!first_piece) __syncthreads();                    // everybody has read the state of the previous piece
            b = walk_s[0];
            int seq_first = walk_s[1], pos = walk_s[2];
            const int range_end = walk_s[3], W = walk_s[4];
            if (pos >= range_end) break;
            const int pad = a.piece_cost;
            int nb = seq_tiles(a, b);
            // units of sequence b: [seq_first, seq_first + pad + nb); pos < total, so b stays inside the batch
            while (nb == 0 || seq_first + pad + nb <= pos) { seq_first += nb ? nb + pad : 0; b++; nb = seq_tiles(a, b); }
            const int real0 = seq_first + pad;                    // unit of the sequence's first tile
            tile_lo = max(pos - real0, 0);
            tile_hi = min(nb, range_end - real0);
            if (tile_hi <= tile_lo) break;                        // the range ends inside the charge in front of sequence b
            len0 = a.kv_len[b];
            const int c_first = real0 / W;
            slot0 = c_first + b;                                  // (range, sequence) pairs in walking order: range + sequence is unique
            slot = (int)blockIdx.y + b;
            nlive = (real0 + nb - 1) / W - c_first + 1;           // ranges that hold a piece of this sequence
            __syncthreads();                                      // everybody has read the old state
            if (tid == 0) {
                walk_s[0] = b; walk_s[1] = seq_first; walk_s[2] = seq_first + a.piece_cost + tile_hi;
                walk_s[5] = b; walk_s[6] = slot; walk_s[7] = slot0; walk_s[8] = nlive;
            }
        } else {
            if (!first_piece) break;
            b = blockIdx.z;
            len0 = a.kv_len[b];
            // A CTA that leaves early still has to wait for the grid in front (programmatic dependent launch):
            // a grid whose CTAs all returned without waiting would retire, and let the next kernel in the
            // stream start, before the append kernel has finished.
            if (len0 >= (int)(a.kv.seq_off[b + 1] - a.kv.seq_off[b])) { asm volatile("griddepcontrol.wait;\n" ::: "memory"); return; }
            const int tps_tiles = a.tokens_per_split / TILE, nb = (len0 + TILE) / TILE;
            slot = blockIdx.y; slot0 = 0;
            tile_lo = slot * tps_tiles;
            tile_hi = min(nb, tile_lo + tps_tiles);
            nlive = min(a.nsplit, (len0 + a.tokens_per_split) / a.tokens_per_split);     // splits with t0 < L
        }
        const int64_t base = a.kv.seq_off[b];
        const int L = len0 + 1;
        const int t0 = tile_lo * TILE, t1 = min(L, tile_hi * TILE);
        if (!BALANCED && t0 >= L) {
            asm volatile("griddepcontrol.wait;\n" ::: "memory");
            float *pd = a.part + (((size_t)b * a.nh + (size_t)head0) * a.nsplit + slot) * (HD + 2);
            const size_t part_stride = (size_t)a.nsplit * (HD + 2);
            if (tid < G) { pd[tid * part_stride] = -INFINITY; pd[tid * part_stride + 1] = 0.0f; }
            return;
        }
        // this warp's tiles: the piece's tiles warp, warp + 4, ...  rem = tokens from the start of the warp's current
        // tile to the end of the piece (<= 0: no tile left); tok_abs = that tile's first token, counted from the
        // start of the pool
        int rem = t1 - t0 - warp * TILE, tok_abs = (int)base + t0 + warp * TILE;

        // ---- per-warp staging slots (K rows, V rows): zero them (skipped tail rows must stay finite; the slots
        //      also held the warp's output tile of the piece before).  K of the next tile is requested as soon as
        //      the score loop is done with the slot, V right after the value loop.  The first tile is requested
        //      before anything else so that its latency hides behind the query prologue; under programmatic
        //      dependent launch that happens while the append kernel of this call may still be running, so only
        //      for tiles that end before the row it appends (token len0).
        if (!BALANCED && !first_piece) __syncthreads();           // (BALANCED: the barriers of the walk above already separate the pieces)
        {
            uint4 *z = reinterpret_cast<uint4 *>(wbase);
            for (int i = lane; i < WARP_BYTES / 16; i += 32) z[i] = make_uint4(0u, 0u, 0u, 0u);
            fence_proxy_async();                                  // generic-proxy zeros before async-proxy copies
            __syncwarp();
        }
        const bool first_issued = pipe_ok && rem > 0 && (waited || t0 + (warp + 1) * TILE <= len0);
        if (first_issued) {
            issue_rows16(rawK, barK, a.kv.K, nkv, rem, lane, mk, kvh, tok_abs);
            issue_rows16(rawV, barV, a.kv.V, nkv, rem, lane, mv, kvh, tok_abs);
        }
        // everything below reads what the append kernel of this call wrote (query rows, the new K/V row, zeroed counters)
        if (!waited) { asm volatile("griddepcontrol.wait;\n" ::: "memory"); waited = true; }

        // ---- query group -> B fragments in stream order: lane (head r, quarter j), k-step c
        //      holds q at the dims of elements 8c+2j and 8c+2j+1 (zeros where the stream has a scale)
        float rs_mine;
        {
            const float *q = a.q_prep + ((size_t)b * a.nh + (size_t)head0 + (r < G ? r : 0)) * HD;
            float mx = 0.0f;
            {   // 16 independent 128-bit loads: the prologue is per piece, keep it off the latency path
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
                uint32_t pk[2];
    #pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int el = 8 * c + 2 * j + h;
                    const int bl = el / 17, idx = el - 17 * bl;
                    // scale slots read dims 0,1 (any valid address) and are zeroed by the multiplier
                    const int d = (idx != 0) ? 32 * bl + 2 * (idx - 1) : 0;
                    const float2 v = *reinterpret_cast<const float2 *>(q + d);
                    const float mul = (idx != 0) ? down : 0.0f;
                    pk[h] = pack_h2(v.x * mul, v.y * mul);
                }
                Q_s[c * 32 + lane] = make_uint2(pk[0], pk[1]);
            }
            rs_mine = (r < G) ? a.scale * exp2f((float)e) * LOG2E : 0.0f;
        }
        const float rsA = __shfl_sync(0xffffffffu, rs_mine, (2 * j) * 4);
        const float rsB = __shfl_sync(0xffffffffu, rs_mine, (2 * j + 1) * 4);

        float o[NCHUNK][4];
#pragma unroll
        for (int i = 0; i < NCHUNK; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
        float mA = -INFINITY, mB = -INFINITY, lA = 0.0f, lB = 0.0f;

        __syncthreads();                                          // publishes Q_s
        const uint2 *q_frag = Q_s + lane;
        if (pipe_ok && rem > 0 && !first_issued) {
            issue_rows16(rawK, barK, a.kv.K, nkv, rem, lane, mk, kvh, tok_abs);
            issue_rows16(rawV, barV, a.kv.V, nkv, rem, lane, mv, kvh, tok_abs);
        }
        for (; pipe_ok && rem > 0; rem -= NWARP * TILE, tok_abs += NWARP * TILE, phase++) {
            const bool more = rem > NWARP * TILE;
            if (!mbar_wait(barK, phase & 1)) {
                (void)mbar_wait(barV, phase & 1);                 // bounded chance for the other copy to drain
                pipe_ok = false;
                break;
            }

            // ---- S^T = K Q^T: 17 k-steps in two accumulator chains -----------------------------
            uint32_t dk0[8], dk1[8];
    #pragma unroll
            for (int bb = 0; bb < 8; bb++) {
                const unsigned short u0 = lds_u16(rawK + r * ROWB + 34 * bb);
                const unsigned short u1 = lds_u16(rawK + (r + 8) * ROWB + 34 * bb);
                dk0[bb] = (uint32_t)u0 | ((uint32_t)u0 << 16);
                dk1[bb] = (uint32_t)u1 | ((uint32_t)u1 << 16);
            }
            float s[4] = {0.0f, 0.0f, 0.0f, 0.0f}, s2[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            const uint32_t k_addr = rawK + lane_off;
            {
                uint32_t R[4];
    #define QK_PAIR(C)                                                \
                ldsm_x4(R, k_addr + (C) * 16);                        \
                qk_chunk<(C)>(R[0], R[1], dk0, dk1, j, q_frag, s);    \
                qk_chunk<(C) + 1>(R[2], R[3], dk0, dk1, j, q_frag, s2);
                QK_PAIR(0) QK_PAIR(2) QK_PAIR(4) QK_PAIR(6) QK_PAIR(8) QK_PAIR(10) QK_PAIR(12) QK_PAIR(14)
    #undef QK_PAIR
                ldsm_x2(R, k_addr + 16 * 16);                         // lanes 0-15 address chunk 16
                qk_chunk<16>(R[0], R[1], dk0, dk1, j, q_frag, s);
            }
            __syncwarp();                                             // every lane is done with the K slot
            if (more) {
                fence_proxy_async();
                issue_rows16(rawK, barK, a.kv.K, nkv, rem - NWARP * TILE, lane, mk, kvh, tok_abs + NWARP * TILE);
            }

            // ---- online softmax over tokens (rows r, r+8); columns = heads 2j, 2j+1 -------------
            const bool ok0 = r < rem, ok1 = r + 8 < rem;
            float x00 = ok0 ? (s[0] + s2[0]) * rsA : -INFINITY, x01 = ok0 ? (s[1] + s2[1]) * rsB : -INFINITY;
            float x10 = ok1 ? (s[2] + s2[2]) * rsA : -INFINITY, x11 = ok1 ? (s[3] + s2[3]) * rsB : -INFINITY;
            float cA = fmaxf(x00, x10), cB = fmaxf(x01, x11);
#pragma unroll
            for (int sft = 4; sft <= 16; sft <<= 1) {
                cA = fmaxf(cA, __shfl_xor_sync(0xffffffffu, cA, sft));
                cB = fmaxf(cB, __shfl_xor_sync(0xffffffffu, cB, sft));
            }
            // The reference maximum only moves when the tile maximum exceeds it by more than 2^6: the
            // probabilities then stay below 2^6 (times 2^8 still inside f16) and the 68 multiplies that
            // rescale the output tile are skipped on almost every tile.  (m, l, o) stay consistent, so
            // the merge of the partials is unchanged.
            const float nA = (cA > mA + 6.0f) ? cA : mA, nB = (cB > mB + 6.0f) ? cB : mB;   // finite: the tile's first token is valid
            const float corrA = exp2f(mA - nA), corrB = exp2f(mB - nB);
            mA = nA; mB = nB;
            x00 = exp2f(x00 - nA); x10 = exp2f(x10 - nA); x01 = exp2f(x01 - nB); x11 = exp2f(x11 - nB);
            lA = lA * corrA + x00 + x10;
            lB = lB * corrB + x01 + x11;
            if (__any_sync(0xffffffffu, corrA != 1.0f || corrB != 1.0f)) {
#pragma unroll
                for (int i = 0; i < NCHUNK; i++) { o[i][0] *= corrA; o[i][1] *= corrB; o[i][2] *= corrA; o[i][3] *= corrB; }
            }
            const uint32_t pb0 = movmatrix_trans(pack_h2(x00 * 256.0f, x01 * 256.0f));
            const uint32_t pb1 = movmatrix_trans(pack_h2(x10 * 256.0f, x11 * 256.0f));

            // ---- O^T += V^T P^T: one m-tile per chunk; block scales arrive with chunk 2b ---------
            if (!mbar_wait(barV, phase & 1)) {
                if (more) (void)mbar_wait(barK, (phase + 1) & 1);
                pipe_ok = false;
                break;
            }
            const uint32_t v_addr = rawV + lane_off;
            {
                uint32_t R[4];
                uint32_t lo0 = 0, lo1 = 0, hi0 = 0, hi1 = 0;          // scale pairs of the current two blocks
#define PV_PAIR(C)                                                                         \
                ldsm_x4_trans(R, v_addr + (C) * 16);                                           \
                lo0 = hi0; lo1 = hi1;                                                          \
                hi0 = __shfl_sync(0xffffffffu, R[0], ((C) / 2) * 4 + j);   /* scale of block C/2 */ \
                hi1 = __shfl_sync(0xffffffffu, R[1], ((C) / 2) * 4 + j);                        \
                if ((C) == 0) { lo0 = hi0; lo1 = hi1; }                                         \
                pv_chunk<(C)>(R[0], R[1], lo0, lo1, hi0, hi1, r, pb0, pb1, o[(C)]);             \
                pv_chunk<(C) + 1>(R[2], R[3], hi0, hi1, hi0, hi1, r, pb0, pb1, o[(C) + 1]);
                PV_PAIR(0) PV_PAIR(2) PV_PAIR(4) PV_PAIR(6) PV_PAIR(8) PV_PAIR(10) PV_PAIR(12) PV_PAIR(14)
#undef PV_PAIR
                ldsm_x2_trans(R, v_addr + 16 * 16);
                pv_chunk<16>(R[0], R[1], hi0, hi1, hi0, hi1, r, pb0, pb1, o[16]);
            }
            __syncwarp();                                             // every lane is done with the V slot
            if (more) {
                fence_proxy_async();
                issue_rows16(rawV, barV, a.kv.V, nkv, rem - NWARP * TILE, lane, mv, kvh, tok_abs + NWARP * TILE);
            }
        }
        // a copy that never completed: this warp stops streaming for good (its barriers are in an unknown phase),
        // the CTA poisons what it writes from here on, and the host learns of it at its next synchronisation
        if (!pipe_ok && lane == 0 && !pipe_failed) { pipe_failed = 1; if (a.status) atomicOr(a.status, ORN_WAIT_DECODE); }
        __syncwarp();

        // ---- merge the four warps, one partial per (head, piece) ------------------------------------
#pragma unroll
        for (int sft = 4; sft <= 16; sft <<= 1) {
            lA += __shfl_xor_sync(0xffffffffu, lA, sft);
            lB += __shfl_xor_sync(0xffffffffu, lB, sft);
        }
        if (BALANCED) {                                               // (published by the barrier behind the query fragments)
            const volatile int *w = walk_s;
            b = w[5]; slot = w[6]; slot0 = w[7]; nlive = w[8];
        }
        // partials: BALANCED [head][slot], else [sequence][head][split]; a.nsplit = partial slots per head
        const size_t part_stride = (size_t)a.nsplit * (HD + 2);     // next head
        float *part_g = a.part + (BALANCED ? (size_t)head0 * a.nsplit : ((size_t)b * a.nh + (size_t)head0) * a.nsplit) * (HD + 2);
        float *part0 = part_g + (size_t)slot * (HD + 2);
        float *Ow = reinterpret_cast<float *>(smem + QS_BYTES + warp * WARP_BYTES);   // [8 heads][256] f32 over this warp's slots
        store_chunk<0>(Ow, o[0], r, j);   store_chunk<1>(Ow, o[1], r, j);   store_chunk<2>(Ow, o[2], r, j);
        store_chunk<3>(Ow, o[3], r, j);   store_chunk<4>(Ow, o[4], r, j);   store_chunk<5>(Ow, o[5], r, j);
        store_chunk<6>(Ow, o[6], r, j);   store_chunk<7>(Ow, o[7], r, j);   store_chunk<8>(Ow, o[8], r, j);
        store_chunk<9>(Ow, o[9], r, j);   store_chunk<10>(Ow, o[10], r, j); store_chunk<11>(Ow, o[11], r, j);
        store_chunk<12>(Ow, o[12], r, j); store_chunk<13>(Ow, o[13], r, j); store_chunk<14>(Ow, o[14], r, j);
        store_chunk<15>(Ow, o[15], r, j); store_chunk<16>(Ow, o[16], r, j);
        if (r == 0) {
            m_s[warp][2 * j] = mA; m_s[warp][2 * j + 1] = mB;
            l_s[warp][2 * j] = lA; l_s[warp][2 * j + 1] = lB;
        }
        __syncthreads();
#pragma unroll                                                    // unrolled: the heads' loads and stores overlap
        for (int h = 0; h < 8; h++) {
            if (h >= G) break;
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
        if (a.group_ctr == nullptr) continue;                         // (only without BALANCED: the combine kernel merges)

        // ---- fused merge: the last CTA of this (sequence, head group) to get here combines the group's partials
        //      (reference: src/ornith_attn.c:131-148 normalisation, src/ornith_rforward.c:450 gate).  Nobody waits:
        //      every CTA publishes its partials, counts itself, and only the one that counts last goes on.
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            int *ctr = a.group_ctr + (size_t)b * gridDim.x + blockIdx.x;
            last_one = (atomicAdd(ctr, 1) == nlive - 1);
        }
        __syncthreads();
        if (!last_one) continue;
        __threadfence();
        // 16 threads per head, all heads at once: thread (h, q) owns the float2 columns q + 16 k of head h.
        // Partials of other SMs are read past L1.  Four partials' rows are in flight per thread at a time.
        const int h = tid >> 4, q = tid & 15;
        if (h < G) {
            const unsigned hm = 0xffffu << (lane & 16);           // this half-warp (the other half may belong to no head)
            const float *ph = part_g + (size_t)slot0 * (HD + 2) + h * part_stride;   // first partial of head h
            float M = -INFINITY;
            for (int s = q; s < nlive; s += 16) {
                const float2 ml = __ldcg(reinterpret_cast<const float2 *>(ph + (size_t)s * (HD + 2)));
                if (ml.y > 0.0f) M = fmaxf(M, ml.x);
            }
#pragma unroll
            for (int sft = 8; sft >= 1; sft >>= 1) M = fmaxf(M, __shfl_xor_sync(hm, M, sft, 16));
            float lsum = 0.0f;
            float2 acc[8];
#pragma unroll
            for (int k = 0; k < 8; k++) acc[k] = make_float2(0.0f, 0.0f);
            for (int s0 = 0; s0 < nlive; s0 += 16) {
                const int s = s0 + q;
                const float2 ml = s < nlive ? __ldcg(reinterpret_cast<const float2 *>(ph + (size_t)s * (HD + 2))) : make_float2(0.0f, 0.0f);
                const float w = (ml.y > 0.0f) ? expf(ml.x - M) : 0.0f;
                lsum += ml.y * w;
                const int n = min(16, nlive - s0);
                for (int i0 = 0; i0 < n; i0 += 4) {
                    float2 v[4][8];
                    float wi[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        wi[u] = __shfl_sync(hm, w, (i0 + u) & 15, 16);
                        if (i0 + u >= n) wi[u] = 0.0f;
                        const float2 *o2 = reinterpret_cast<const float2 *>(ph + (size_t)(s0 + min(i0 + u, n - 1)) * (HD + 2) + 2);
#pragma unroll
                        for (int k = 0; k < 8; k++) v[u][k] = __ldcg(o2 + q + 16 * k);       // dims 2 (q + 16 k), +1
                    }
#pragma unroll
                    for (int u = 0; u < 4; u++)
                        if (wi[u] != 0.0f) {
#pragma unroll
                            for (int k = 0; k < 8; k++) { acc[k].x += v[u][k].x * wi[u]; acc[k].y += v[u][k].y * wi[u]; }
                        }
                }
            }
#pragma unroll
            for (int sft = 8; sft >= 1; sft >>= 1) lsum += __shfl_xor_sync(hm, lsum, sft, 16);
            const float inv = 1.0f / lsum;
            const size_t head = (size_t)b * a.nh + (size_t)head0 + h;
#pragma unroll
            for (int k = 0; k < 8; k++)
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int d = 2 * (q + 16 * k) + e;
                    float o = (e ? acc[k].y : acc[k].x) * inv;
                    if (a.act_dtype == ORNITH_ACT_BF16) {
                        if (a.gated) o *= sigmoid_f(act_ld((const __nv_bfloat16 *)a.qproj, head * HD * 2 + HD + d));
                        act_st((__nv_bfloat16 *)a.out, head * HD + d, o);
                    } else {
                        if (a.gated) o *= sigmoid_f(act_ld((const float *)a.qproj, head * HD * 2 + HD + d));
                        act_st((float *)a.out, head * HD + d, o);
                    }
                }
        }
    }
}

typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                             const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn tensor_map_encoder() {
    static EncodeFn fn = nullptr;
    if (!fn) {
        cudaDriverEntryPointQueryResult q;
        void *p = nullptr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeFn)p;
    }
    return fn;
}

// View of a pool of Q8_0 rows as [token][kv head][68 32-bit words]; one box = the 16 rows of one
// head for 16 consecutive tokens.  Only full tiles of valid tokens are ever requested, so the
// token extent is left open-ended rather than tied to the size of the pool.
bool q8_rows_map(CUtensorMap *m, const void *pool, int nkv) {
    EncodeFn enc = tensor_map_encoder();
    if (!enc || ((uintptr_t)pool & 15) != 0) return false;
    cuuint64_t dims[3] = {(cuuint64_t)(ROWB / 4), (cuuint64_t)nkv, (cuuint64_t)1 << 31};
    cuuint64_t strides[2] = {(cuuint64_t)ROWB, (cuuint64_t)nkv * ROWB};
    cuuint32_t box[3] = {(cuuint32_t)(ROWB / 4), 1, (cuuint32_t)TILE};
    cuuint32_t es[3] = {1, 1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void *>(pool), dims, strides, box, es,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// ranges of the balanced schedule: one per resident CTA of a head-group column (4 CTAs on each of 148 SMs), fewer when
// the batch is too small for ranges of at least floor_w tiles (same rule as in the kernel)
static int balanced_ranges(int nkv, int nh, int n_seq, int max_len) {
    const int X = nkv * ((nh / nkv + 7) / 8);
    const long long tiles = (max_len + TILE - 1) / TILE, floor_w = (tiles + 31) / 32 > 16 ? (tiles + 31) / 32 : 16;
    const long long by_work = ((long long)n_seq * tiles + floor_w - 1) / floor_w, cap = 592 / X > 0 ? 592 / X : 1;
    return (int)(by_work < cap ? (by_work > 0 ? by_work : 1) : cap);
}
int gqa_decode_q8_raw_slots(int nkv, int nh, int n_seq, int max_len) {
    return balanced_ranges(nkv, nh, n_seq, max_len) + n_seq;
}

ornith_status launch_gqa_decode_q8_raw(const DecodeArgs &a_in, int n_seq, cudaStream_t st, bool *merged) {
    DecodeArgs a = a_in;
    *merged = a.group_ctr != nullptr;
    const bool balanced = gqa_decode_q8_raw_balanced(a.kv, a.nh);
    if (balanced && !a.group_ctr) {
        orn_record_error("k_gqa_decode_q8_raw: the balanced schedule merges its partials itself and needs the arrival counters");
        return ORNITH_ERR_FORMAT;
    }
    static bool configured_dev[ORN_MAX_DEVICES] = {};
    bool &configured = configured_dev[orn_device_index()];
    if (!configured) {
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_gqa_decode_q8_raw<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               SMEM_BYTES), "gqa decode smem opt-in"));
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_gqa_decode_q8_raw<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               SMEM_BYTES), "gqa decode smem opt-in"));
        configured = true;
    }
    // without the tensor maps (driver entry point missing, pool not 16-byte aligned) every tile falls back to row copies
    CUtensorMap mk, mv;
    memset(&mk, 0, sizeof mk);
    memset(&mv, 0, sizeof mv);
    const char *env = getenv("ORNITH_CUDA_DECODE_ROW_COPIES");
    const int tensor_copies = !(env && env[0] == '1') && q8_rows_map(&mk, a.kv.K, a.kv.nkv) && q8_rows_map(&mv, a.kv.V, a.kv.nkv);
    const int X = a.kv.nkv * ((a.nh / a.kv.nkv + 7) / 8);
    a.n_seq = n_seq;
    a.status = orn_status_word();
    static int piece_cost = -1;                                   // ORNITH_CUDA_DECODE_PIECE_COST=<tiles>: see the kernel
    if (piece_cost < 0) { const char *e = getenv("ORNITH_CUDA_DECODE_PIECE_COST"); piece_cost = e ? atoi(e) : 4; if (piece_cost < 0 || piece_cost > 15) piece_cost = 4; }
    a.piece_cost = piece_cost;
    dim3 grid(X, a.nsplit, n_seq);
    if (balanced) grid = dim3(X, balanced_ranges(a.kv.nkv, a.nh, n_seq, a.max_len), 1);
    // may start while the append kernel in front of it still runs: it waits (griddepcontrol.wait) before it reads that kernel's output
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(128); cfg.dynamicSmemBytes = SMEM_BYTES; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    if (balanced) return orn_check(cudaLaunchKernelEx(&cfg, k_gqa_decode_q8_raw<true>, a, mk, mv, tensor_copies), "k_gqa_decode_q8_raw");
    return orn_check(cudaLaunchKernelEx(&cfg, k_gqa_decode_q8_raw<false>, a, mk, mv, tensor_copies), "k_gqa_decode_q8_raw");
}
