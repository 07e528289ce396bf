// gqa_prefill_mma.cu — causal GQA prefill on the tensor cores (head_dim 256).
//
// Replaces the core of full_attn_prefill() (reference: src/ornith_rforward.c:529-551, which
// runs ornith_gqa_step once per token) for T new tokens per sequence that attend over
// everything already cached plus themselves.  As in the reference, quantised caches are
// attended over in their DECODED form, current token included: the rows are first appended
// to the cache (k_full_prep), then every cached row the prefill can see is decoded once into
// an f16 image (k_kv_rows_to_f16), and the attention kernel reads only that image.
//
// k_gqa_prefill_mma: one CTA = 64 query tokens of one head, 4 warps x 16 rows.  Flash-
// attention schedule: K and V tiles of 64 keys are staged with cp.async (one slot each; the
// next K tile is requested as soon as the score MMAs are done with the slot, the next V tile
// after the value MMAs), S = Q K^T and O += P V run on mma.sync m16n8k16 (f16 in, f32
// accumulate) with ldmatrix-fed fragments, the softmax stays in registers (log2 domain,
// rescale only when a row maximum moves).  The 8 heads of a KV group read the same f16 tiles
// through L2.
//
// Precision: q rows are scaled by a power of two into [-1, 1] and rounded to f16; K, V and
// the probabilities (scaled by 2^8) are f16 — an 11-bit significand, like tf32; sums are f32.
#include "full_attn.cuh"

namespace {

constexpr int HD = 256;
constexpr int BM = 64, BN = 64;            // query rows per CTA, keys per tile
constexpr int LDT = 264;                   // smem row stride in halves (528 B): conflict-free ldmatrix
constexpr int TILE_BYTES = BN * LDT * 2;   // 33792
constexpr int SMEM_BYTES = 3 * TILE_BYTES; // Q tile + K slot + V slot = 101376 -> two CTAs per SM
constexpr float LOG2E = 1.4426950408889634f;

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

struct PrefillMmaArgs {
    KvView kv;
    const int32_t *kv_len;
    const float *q_prep;            // [n_seq*T][nh][256] f32, normalised + rotated
    __half *Kh, *Vh;                // [n_seq][nkv][Lp][256] decoded rows, zero past the rows the prefill sees
    const void *qproj;
    void *out;
    int nh, T, Lmax, gated;
    int Lp;                         // row pitch of the images: Lmax rounded up to a multiple of 64
    float scale;
};

// ---- decoded f16 image of every cached row the prefill can see: one warp per row -----------
template <int MODE>
__global__ void __launch_bounds__(128) k_kv_rows_to_f16(PrefillMmaArgs a) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int pos = blockIdx.x * 4 + w, kvh = blockIdx.y, b = blockIdx.z, nkv = a.kv.nkv;
    const int64_t base = a.kv.seq_off[b];
    const int cap = (int)(a.kv.seq_off[b + 1] - base);
    const int seen = min(min(a.kv_len[b] + a.T, cap), a.Lmax);
    if (pos >= a.Lp) return;
    const size_t o = (((size_t)b * nkv + kvh) * a.Lp + pos) * HD + lane * 8;
    if (pos >= seen) {                                    // whole 64-key tiles are read: keep the tail finite
        *reinterpret_cast<uint4 *>(a.Kh + o) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4 *>(a.Vh + o) = make_uint4(0u, 0u, 0u, 0u);
        return;
    }
    const size_t r = (size_t)(base + pos) * nkv + kvh;
    const size_t rb = kv_row_bytes(MODE, HD);
    const uint8_t *krow = a.kv.K + r * rb, *vrow = a.kv.V + r * rb;
    float ks = 1.0f, vs = 1.0f;
    if (MODE == ORNITH_KV_INT8_HEAD) { ks = a.kv.Ks[r]; vs = a.kv.Vs[r]; }
    uint32_t ko[4], vo[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int d = lane * 8 + 2 * i;
        ko[i] = pack_h2(kv_elem<MODE>(krow, d) * ks, kv_elem<MODE>(krow, d + 1) * ks);
        vo[i] = pack_h2(kv_elem<MODE>(vrow, d) * vs, kv_elem<MODE>(vrow, d + 1) * vs);
    }
    *reinterpret_cast<uint4 *>(a.Kh + o) = make_uint4(ko[0], ko[1], ko[2], ko[3]);
    *reinterpret_cast<uint4 *>(a.Vh + o) = make_uint4(vo[0], vo[1], vo[2], vo[3]);
}

// copy 64 rows x 256 halves (row pitch 512 B in global) into a padded smem tile; rows at or
// past `rows_valid` are zero-filled
__device__ __forceinline__ void stage_tile(__half *dst, const __half *src, int rows_valid, int tid) {
    for (int c = tid; c < BN * 32; c += 128) {            // 32 chunks of 16 bytes per row
        const int row = c >> 5, ch = c & 31;
        const bool ok = row < rows_valid;
        cp_async16(smem_u32(dst + row * LDT + ch * 8), src + (ok ? (size_t)row * HD + ch * 8 : 0), ok ? 16 : 0);
    }
}

template <typename ACT>
__global__ void __launch_bounds__(128, 2) k_gqa_prefill_mma(PrefillMmaArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    __half *Q_s = reinterpret_cast<__half *>(smem);
    __half *K_s = reinterpret_cast<__half *>(smem + TILE_BYTES);
    __half *V_s = reinterpret_cast<__half *>(smem + 2 * TILE_BYTES);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, r = lane >> 2, j = lane & 3;
    const int h = blockIdx.y, b = blockIdx.z, nkv = a.kv.nkv, kvh = h / (a.nh / nkv);
    const int q0 = blockIdx.x * BM;                       // first new token of this CTA
    const int cap = (int)(a.kv.seq_off[b + 1] - a.kv.seq_off[b]);
    const int len0 = a.kv_len[b];
    // tokens that were really appended: the engine stops appending when the cache is full
    const int t_end = min(a.T, max(0, min(cap, a.Lmax) - len0));
    if (q0 >= t_end) return;
    const int rows_here = min(BM, t_end - q0);
    const int kmax = len0 + q0 + rows_here - 1;           // last key any row of the CTA sees

    // ---- stage the query tile: f32 -> f16, each row scaled by a power of two --------------
    float rowscale[2];
    {
        // warp w converts rows 16w .. 16w+15; 8 lanes per row pass (4 passes x 4 rows)
        for (int rr = 0; rr < 16; rr += 4) {
            const int row = warp * 16 + rr + (lane >> 3), c8 = lane & 7;
            const bool ok = row < rows_here;
            const float *q = a.q_prep + (((size_t)b * a.T + q0 + (ok ? row : 0)) * a.nh + h) * HD;
            float4 v[8];
            float mx = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                v[i] = ok ? *reinterpret_cast<const float4 *>(q + (c8 + 8 * i) * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
                mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v[i].x), fabsf(v[i].y)), fmaxf(fabsf(v[i].z), fabsf(v[i].w))));
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            int e = 0;
            if (mx > 0.0f && mx < INFINITY) (void)frexpf(mx, &e);
            const float down = exp2f((float)-e);
#pragma unroll
            for (int i = 0; i < 8; i++)
                *reinterpret_cast<uint2 *>(Q_s + row * LDT + (c8 + 8 * i) * 4) =
                    make_uint2(pack_h2(v[i].x * down, v[i].y * down), pack_h2(v[i].z * down, v[i].w * down));
            if (c8 == 0) reinterpret_cast<float *>(K_s)[row] = a.scale * exp2f((float)e) * LOG2E;   // parked in the K slot
        }
        __syncthreads();
        rowscale[0] = reinterpret_cast<const float *>(K_s)[warp * 16 + r];
        rowscale[1] = reinterpret_cast<const float *>(K_s)[warp * 16 + r + 8];
        __syncthreads();
    }

    const __half *Kg = a.Kh + (((size_t)b * nkv + kvh) * a.Lp) * HD;
    const __half *Vg = a.Vh + (((size_t)b * nkv + kvh) * a.Lp) * HD;
    stage_tile(K_s, Kg, min(BN, kmax + 1), tid);
    cp_async_commit();
    stage_tile(V_s, Vg, min(BN, kmax + 1), tid);
    cp_async_commit();

    float o[32][4];
#pragma unroll
    for (int i = 0; i < 32; i++) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    float m2[2] = {-INFINITY, -INFINITY}, lsum[2] = {0.0f, 0.0f};
    const int qpos0 = len0 + q0 + warp * 16 + r, qpos1 = qpos0 + 8;   // absolute positions of this lane's rows

    const uint32_t q_addr = smem_u32(Q_s) + ((warp * 16 + (lane & 15)) * LDT + (lane >> 4) * 8) * 2;
    const uint32_t k_addr = smem_u32(K_s) + (((lane & 7) + (lane >> 4) * 8) * LDT + ((lane >> 3) & 1) * 8) * 2;
    const uint32_t v_addr = smem_u32(V_s) + (((lane & 7) + ((lane >> 3) & 1) * 8) * LDT + (lane >> 4) * 8) * 2;

    for (int kb = 0; kb <= kmax; kb += BN) {
        const bool more = kb + BN <= kmax;
        cp_async_wait<1>();                                   // this tile's K has landed
        __syncthreads();
        // ---- S = Q K^T : 16 rows x 64 keys per warp -----------------------------------------
        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; n++) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f; }
#pragma unroll
        for (int ks = 0; ks < 16; ks++) {
            uint32_t A[4];
            ldsm_x4(A, q_addr + ks * 32);
#pragma unroll
            for (int np = 0; np < 4; np++) {                  // two key n-tiles per ldmatrix
                uint32_t B[4];
                ldsm_x4(B, k_addr + (np * 16 * LDT) * 2 + ks * 32);
                mma16816(s[2 * np], A, B[0], B[1]);
                mma16816(s[2 * np + 1], A, B[2], B[3]);
            }
        }
        __syncthreads();                                      // every warp is done with the K slot
        if (more) stage_tile(K_s, Kg + (size_t)(kb + BN) * HD, min(BN, kmax + 1 - (kb + BN)), tid);
        cp_async_commit();

        // ---- online softmax (log2 domain); causal mask on the absolute key position ----------
        float corr[2];
#pragma unroll
        for (int hh = 0; hh < 2; hh++) {
            const int qp = hh ? qpos1 : qpos0;
            float mx = -INFINITY;
#pragma unroll
            for (int n = 0; n < 8; n++)
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const int key = kb + n * 8 + 2 * j + c;
                    float x = s[n][2 * hh + c] * rowscale[hh];
                    x = (key <= qp) ? x : -INFINITY;
                    s[n][2 * hh + c] = x;
                    mx = fmaxf(mx, x);
                }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float mn = fmaxf(m2[hh], mx);
            // rows past the end of the prompt see no key at all in early tiles: keep them inert
            const float msafe = (mn == -INFINITY) ? 0.0f : mn;
            corr[hh] = exp2f(m2[hh] - msafe);
            m2[hh] = mn;
            float ps = 0.0f;
#pragma unroll
            for (int n = 0; n < 8; n++)
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    const float p = exp2f(s[n][2 * hh + c] - msafe);
                    s[n][2 * hh + c] = p;
                    ps += p;
                }
            lsum[hh] = lsum[hh] * corr[hh] + ps;
        }
        if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
            for (int i = 0; i < 32; i++) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
        }

        // ---- O += P V : 4 k-steps of 16 keys x 32 dim n-tiles -----------------------------------
        cp_async_wait<1>();                                   // this tile's V has landed
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
            uint32_t P[4];
            P[0] = pack_h2(s[2 * ks][0] * 256.0f, s[2 * ks][1] * 256.0f);
            P[1] = pack_h2(s[2 * ks][2] * 256.0f, s[2 * ks][3] * 256.0f);
            P[2] = pack_h2(s[2 * ks + 1][0] * 256.0f, s[2 * ks + 1][1] * 256.0f);
            P[3] = pack_h2(s[2 * ks + 1][2] * 256.0f, s[2 * ks + 1][3] * 256.0f);
#pragma unroll
            for (int np = 0; np < 16; np++) {
                uint32_t B[4];
                ldsm_x4_trans(B, v_addr + (ks * 16 * LDT) * 2 + np * 32);
                mma16816(o[2 * np], P, B[0], B[1]);
                mma16816(o[2 * np + 1], P, B[2], B[3]);
            }
        }
        __syncthreads();                                      // every warp is done with the V slot
        if (more) stage_tile(V_s, Vg + (size_t)(kb + BN) * HD, min(BN, kmax + 1 - (kb + BN)), tid);
        cp_async_commit();
    }
    cp_async_wait<0>();

    // ---- normalise, sigmoid output gate (reference: src/ornith_rforward.c:551), store --------
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
        lsum[hh] += __shfl_xor_sync(0xffffffffu, lsum[hh], 1);
        lsum[hh] += __shfl_xor_sync(0xffffffffu, lsum[hh], 2);
    }
#pragma unroll
    for (int hh = 0; hh < 2; hh++) {
        const int row = warp * 16 + r + 8 * hh;
        if (row >= rows_here) continue;
        const float inv = 1.0f / (lsum[hh] * 256.0f);
        const size_t tok = (size_t)b * a.T + q0 + row;
        const ACT *gate = a.gated ? (const ACT *)a.qproj + tok * a.nh * HD * 2 + (size_t)h * HD * 2 + HD : nullptr;
        ACT *out = (ACT *)a.out + (tok * a.nh + h) * HD;
#pragma unroll
        for (int n = 0; n < 32; n++) {
            const int d = n * 8 + 2 * j;
            float y0 = o[n][2 * hh] * inv, y1 = o[n][2 * hh + 1] * inv;
            if (gate) { y0 *= sigmoid_f(act_ld(gate, d)); y1 *= sigmoid_f(act_ld(gate, d + 1)); }
            act_st(out, d, y0);
            act_st(out, d + 1, y1);
        }
    }
}

}  // namespace

bool gqa_prefill_mma_supported(const KvView &kv) { return kv.hd == HD; }

static int image_pitch(int Lmax) { return (Lmax + 63) / 64 * 64; }
static size_t image_bytes(int n_seq, int nkv, int Lmax) {   // one of the two images; 1 KiB keeps TMA bases aligned
    return align_up((size_t)n_seq * nkv * image_pitch(Lmax) * HD * sizeof(__half), 1024);
}

size_t gqa_prefill_mma_scratch(int n_seq, int nkv, int nh, int T, int Lmax) {
    return 2 * image_bytes(n_seq, nkv, Lmax) + gqa_prefill_tc_scratch(n_seq, nh, T);
}

// ORNITH_CUDA_PREFILL_VARIANT=mma keeps the mma.sync kernel; the default is the tcgen05 kernel
static bool prefer_mma_sync() {
    const char *v = getenv("ORNITH_CUDA_PREFILL_VARIANT");
    return v && v[0] == 'm';
}

// whether the tcgen05 kernel is the one launch_gqa_prefill_mma will use (then the front end writes the f16 query
// image itself and no f32 query image is needed)
bool gqa_prefill_tc_selected() { return !prefer_mma_sync(); }

bool gqa_prefill_q_image(void *kvh_scratch, int n_seq, int nkv, int nh, int T, int Lmax, __half **Qh, float **rs) {
    if (prefer_mma_sync() || ((uintptr_t)kvh_scratch % 16) != 0) return false;
    char *q = (char *)kvh_scratch + 2 * image_bytes(n_seq, nkv, Lmax);
    *Qh = (__half *)q;
    *rs = (float *)(q + align_up((size_t)n_seq * nh * T * HD * sizeof(__half), 256));
    return true;
}

ornith_status launch_gqa_prefill_mma(const KvView &kv, const int32_t *kv_len, const float *q_prep, void *kvh_scratch,
                                     const void *qproj, void *out, int nh, int T, int Lmax, int gated, float scale,
                                     int n_seq, bool bf16_act, cudaStream_t st) {
    PrefillMmaArgs a;
    a.kv = kv; a.kv_len = kv_len; a.q_prep = q_prep; a.qproj = qproj; a.out = out;
    a.nh = nh; a.T = T; a.Lmax = Lmax; a.gated = gated; a.scale = scale;
    a.Lp = image_pitch(Lmax);
    const size_t half_bytes = image_bytes(n_seq, kv.nkv, Lmax);
    a.Kh = (__half *)kvh_scratch;
    a.Vh = (__half *)((char *)kvh_scratch + half_bytes);
    dim3 cgrid((a.Lp + 3) / 4, kv.nkv, n_seq);
    switch (kv.mode) {
    case ORNITH_KV_F32:       k_kv_rows_to_f16<ORNITH_KV_F32><<<cgrid, 128, 0, st>>>(a); break;
    case ORNITH_KV_INT8_HEAD: k_kv_rows_to_f16<ORNITH_KV_INT8_HEAD><<<cgrid, 128, 0, st>>>(a); break;
    default:                  k_kv_rows_to_f16<ORNITH_KV_Q8_0><<<cgrid, 128, 0, st>>>(a); break;
    }
    ORN_TRY(orn_check_launch("k_kv_rows_to_f16"));
    if (!prefer_mma_sync() && ((uintptr_t)kvh_scratch % 16) == 0)
        return launch_gqa_prefill_tc(kv, kv_len, q_prep, a.Kh, a.Vh, (char *)kvh_scratch + 2 * half_bytes, qproj, out, nh,
                                     T, Lmax, a.Lp, gated, scale, n_seq, bf16_act, st);
    static bool configured_dev[ORN_MAX_DEVICES] = {};
    bool &configured = configured_dev[orn_device_index()];
    if (!configured) {
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_gqa_prefill_mma<float>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               SMEM_BYTES), "prefill smem opt-in"));
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_gqa_prefill_mma<__nv_bfloat16>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES), "prefill smem opt-in"));
        configured = true;
    }
    dim3 grid((T + BM - 1) / BM, nh, n_seq);
    if (bf16_act) k_gqa_prefill_mma<__nv_bfloat16><<<grid, 128, SMEM_BYTES, st>>>(a);
    else          k_gqa_prefill_mma<float><<<grid, 128, SMEM_BYTES, st>>>(a);
    return orn_check_launch("k_gqa_prefill_mma");
}
