// linear_decode_ring.cu — persistent form of the fused delta-net decode step (dk = dv = 128,
// conv_k = 4): a small front-end kernel, then the recurrent state streamed through a ring of
// bulk copies.
//
// Same arithmetic, operation order and results as k_linear_decode_128 (linear_attn.cu; reference:
// src/ornith_rforward.c:457-503, :300-319, src/ornith_attn.c:203-212, :373-381).  What differs is
// how the work is cut.
//
// k_linear_decode_front does everything that does not touch the state, once per (sequence, head):
// conv + SiLU of the q, k and v channels, the new conv history slot, the L2 norms of q and k, the
// decay and write gates.  It leaves, per sequence, one 1 KiB block per key head (q then k,
// normalised) and one 528-byte block per value head (v, then the two gates).  In the one-CTA-per-
// head kernel these steps sit, with their double-precision reductions and two CTA barriers, in
// front of every head's state traffic, and each key head is recomputed by all its value heads.
//
// k_linear_decode_ring then only moves state.  Two CTAs per SM stay resident and walk the
// (sequence, value head) units in a fixed stride; each keeps three 32 KiB stages (half a head) in
// shared memory, filled by cp.async.bulk with completion on an mbarrier, and requests half-head
// m+3 as soon as half-head m has been lifted into registers.  The unit's two front-end blocks
// arrive with its first half on the same mbarrier.  The copy engine thus has work queued for the
// whole life of the CTA.  The RMSNorm + SiLU(z) epilogue of a unit is finished after the first
// barrier of the next unit, so a unit costs two CTA barriers.  Every mbarrier wait is bounded; a
// wait that gives up poisons the outputs of the CTA.
#include <map>
#include <mutex>
#include <utility>
#include "bulk_copy.cuh"
#include "linear_attn.cuh"

namespace {

constexpr int STAGES = 3;
constexpr int STAGE_FLOATS = 64 * 128;                // half a head: 64 rows of the state, 32 KiB
constexpr uint32_t STAGE_BYTES = STAGE_FLOATS * 4;
constexpr int QK_FLOATS = 256;                        // front-end block of a key head: q[128], k[128]
constexpr int VB_FLOATS = 132;                        // of a value head: v[128], alpha, beta, 0, 0
constexpr uint32_t QK_BYTES = QK_FLOATS * 4, VB_BYTES = VB_FLOATS * 4;
constexpr int OPND_FLOATS = QK_FLOATS + VB_FLOATS;
constexpr int RING_SMEM = STAGES * (STAGE_FLOATS + OPND_FLOATS) * 4;

__device__ __forceinline__ float act_f(float v) { return v; }
__device__ __forceinline__ float act_f(__nv_bfloat16 v) { return __bfloat162float(v); }

__host__ __device__ inline size_t front_stride(int nk, int nv) { return (size_t)nk * QK_FLOATS + (size_t)nv * VB_FLOATS; }

// grid (nk + ceil(nv / 2), n_seq), 128 threads: blocks 0..nk-1 take a key head, the rest two value heads each
template <typename ACT>
__global__ void __launch_bounds__(128) k_linear_decode_front(LinArgs a, float *front) {
    __shared__ double redd[8];
    // This grid is launched as a programmatic dependent of the kernel in front of it (the layer before): its CTAs are
    // resident when that kernel ends, and await its end before anything else.  Only then may the state kernel of this
    // call start its prologue (it reads the recurrent state early, which the same layer's previous step may still be
    // writing until this wait returns); it waits for this grid before it reads the blocks.
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, b = blockIdx.y, j = blockIdx.x;
    const int qd = a.nk * 128, vd = a.nv * 128, Cc = 2 * qd + vd;
    float *ring = a.conv + (size_t)b * a.conv_stride;
    const ACT *x = (const ACT *)a.qkv + (size_t)b * Cc;
    float *fb = front + (size_t)b * front_stride(a.nk, a.nv);
    const int t = a.pos[b], sb = (t + 1) & 3;

    auto channel = [&](int c) -> float {               // conv + SiLU of channel c; stores the new history slot
        float h[4];
#pragma unroll
        for (int sl = 0; sl < 4; sl++) h[sl] = ring[(size_t)sl * Cc + c];
        const float xin = act_f(x[c]);
        const float4 wt = *reinterpret_cast<const float4 *>(a.conv_w + (size_t)c * 4);
        const float y = conv4_silu(h, xin, wt, a.conv_b ? a.conv_b[c] : 0.0f, sb);
        ring[(size_t)(t & 3) * Cc + c] = xin;
        return y;
    };

    if (j < a.nk) {                                    // q/k L2-norm (reference: src/ornith_tensor.c:155-160)
        const float y0 = channel(j * 128 + tid), y1 = channel(qd + j * 128 + tid);
        double sq = (double)y0 * (double)y0, sk = (double)y1 * (double)y1;
        sq = warp_sum(sq); sk = warp_sum(sk);
        if (lane == 0) { redd[w] = sq; redd[4 + w] = sk; }
        __syncthreads();
        const double ssq = redd[0] + redd[1] + redd[2] + redd[3], ssk = redd[4] + redd[5] + redd[6] + redd[7];
        fb[(size_t)j * QK_FLOATS + tid] = y0 * (float)(1.0 / sqrt(ssq + (double)1e-6f));
        fb[(size_t)j * QK_FLOATS + 128 + tid] = y1 * (float)(1.0 / sqrt(ssk + (double)1e-6f));
    } else {                                           // two value heads per block, one channel of each per thread
        const int hv0 = 2 * (j - a.nk);
        float y[2];
#pragma unroll
        for (int e = 0; e < 2; e++) y[e] = hv0 + e < a.nv ? channel(2 * qd + (hv0 + e) * 128 + tid) : 0.0f;
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const int hv = hv0 + e;
            if (hv >= a.nv) break;
            float *vb = fb + (size_t)a.nk * QK_FLOATS + (size_t)hv * VB_FLOATS;
            vb[tid] = y[e];
            if (tid == 32 * e) {   // decay and write gates (reference: src/ornith_rforward.c:282-284, :493-496)
                const float ain = act_f(((const ACT *)a.a)[(size_t)b * a.nv + hv]);
                const float bin = act_f(((const ACT *)a.b)[(size_t)b * a.nv + hv]);
                vb[128] = expf(a.a_coef[hv] * softplus_f(ain + a.dt_bias[hv]));
                vb[129] = sigmoid_f(bin);
                vb[130] = 0.0f; vb[131] = 0.0f;
            }
        }
    }
}

template <typename ACT>
__global__ void __launch_bounds__(256, 2) k_linear_decode_ring(LinArgs a, const float *front, int n_units) {
    // the next call's front-end kernel may become resident now; it waits for this grid before it does anything
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    extern __shared__ __align__(128) unsigned char smraw[];
    float *stage = reinterpret_cast<float *>(smraw);
    float *opnd = stage + STAGES * STAGE_FLOATS;       // per stage: the front-end blocks of the unit whose first half it holds
    __shared__ double redd[2][8];
    __shared__ unsigned long long full[STAGES];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5, sr = lane >> 3, cc = lane & 7;
    const int vd = a.nv * 128;
    const int n_mine = (n_units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int M = 2 * n_mine;                          // half-heads this CTA walks
    const size_t fstride = front_stride(a.nk, a.nv);

    // one thread: request half-head m (parts & 1) and, with a first half, its unit's front-end blocks (parts & 2)
    auto issue = [&](int m, int parts) {
        const int slot = m % STAGES, u = (int)blockIdx.x + (m >> 1) * (int)gridDim.x, b = u / a.nv, hv = u % a.nv;
        const uint32_t bar = bc_smem_u32(&full[slot]);
        if (parts & 1) {
            const float *src = a.S + (size_t)b * a.S_stride + (size_t)hv * 128 * 128 + (size_t)(m & 1) * STAGE_FLOATS;
            bc_mbar_expect_tx(bar, (m & 1) ? STAGE_BYTES : STAGE_BYTES + QK_BYTES + VB_BYTES);
            bc_copy(bc_smem_u32(stage + slot * STAGE_FLOATS), src, STAGE_BYTES, bar);
        }
        if ((parts & 2) && !(m & 1)) {
            const float *fb = front + (size_t)b * fstride;
            bc_copy(bc_smem_u32(opnd + slot * OPND_FLOATS), fb + (size_t)key_head_of(a, hv) * QK_FLOATS, QK_BYTES, bar);
            bc_copy(bc_smem_u32(opnd + slot * OPND_FLOATS + QK_FLOATS), fb + (size_t)a.nk * QK_FLOATS + (size_t)hv * VB_FLOATS,
                    VB_BYTES, bar);
        }
    };
    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) bc_mbar_init(bc_smem_u32(&full[s]), 1);
        bc_mbar_init_fence();
    }
    __syncthreads();
    // The state does not depend on the front-end kernel of this call: its first copies start while
    // that kernel is still running (programmatic dependent launch); the blocks follow once it is done.
    if (tid == 0)
        for (int m = 0; m < STAGES && m < M; m++) issue(m, 1);
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    if (tid == 0)
        for (int m = 0; m < STAGES && m < M; m++) issue(m, 2);

    float nw[2][2];                                    // RMSNorm weights of this thread's rows (lanes with cc == 0 store)
    ACT zn[2][2];                                      // z of the next unit, requested a unit ahead
    auto load_z = [&](int u) {
        const size_t base = (size_t)(u / a.nv) * vd + (size_t)(u % a.nv) * 128;
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
            for (int i = 0; i < 2; i++) zn[h][i] = ((const ACT *)a.z)[base + (cc == 0 ? 64 * h + 8 * w + 4 * i + sr : 0)];
    };
#pragma unroll
    for (int h = 0; h < 2; h++)
#pragma unroll
        for (int i = 0; i < 2; i++) nw[h][i] = (cc == 0) ? a.norm_w[64 * h + 8 * w + 4 * i + sr] : 0.0f;
    load_z((int)blockIdx.x);

    bool ok = true;
    float po[2][2] = {};                               // the previous unit, waiting for its epilogue
    ACT pz[2][2] = {};
    size_t pbase = 0;

    // per-head RMSNorm and SiLU(z) gate of the previous unit (reference: src/ornith_rforward.c:305-314);
    // its partial sums in redd[p] are complete once a CTA barrier has passed
    auto finish = [&](int p) {
        if (cc == 0) {
            double tot = 0.0;
#pragma unroll
            for (int i = 0; i < 8; i++) tot += redd[p][i];
            const float inv = ok ? (float)(1.0 / sqrt(tot / 128.0 + (double)a.eps)) : NAN;
#pragma unroll
            for (int h = 0; h < 2; h++)
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    float y = po[h][i] * inv * nw[h][i];
                    y *= silu_f(act_f(pz[h][i]));
                    act_st((ACT *)a.out, pbase + 64 * h + 8 * w + 4 * i + sr, y);
                }
        }
    };

    for (int k = 0; k < n_mine; k++) {
        const int u = (int)blockIdx.x + k * (int)gridDim.x, b = u / a.nv, hv = u % a.nv;
        float *S = a.S + (size_t)b * a.S_stride + (size_t)hv * 128 * 128;
        ACT zc[2][2];
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
            for (int i = 0; i < 2; i++) zc[h][i] = zn[h][i];
        if (k + 1 < n_mine) load_z(u + (int)gridDim.x);

        // ---- S <- alpha S; u = beta (v - S k); S += u k^T; o = S q  (reference: src/ornith_attn.c:203-212)
        float4 kr[4], qr[4];                               // this lane's 16 columns of k and q, for all its rows
        float vv[2][2], alpha = 0.0f, beta = 0.0f;
        float orow[2][2];
        double ss = 0.0;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int m = 2 * k + h, slot = m % STAGES;
            ok = ok && bc_mbar_wait(bc_smem_u32(&full[slot]), (uint32_t)(m / STAGES) & 1u);
            if (h == 0) {
                const float *op = opnd + slot * OPND_FLOATS;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    qr[j] = *reinterpret_cast<const float4 *>(op + (cc + j * 8) * 4);
                    kr[j] = *reinterpret_cast<const float4 *>(op + 128 + (cc + j * 8) * 4);
                }
#pragma unroll
                for (int hh = 0; hh < 2; hh++)
#pragma unroll
                    for (int i = 0; i < 2; i++) vv[hh][i] = op[QK_FLOATS + 64 * hh + 8 * w + 4 * i + sr];
                alpha = op[QK_FLOATS + 128]; beta = op[QK_FLOATS + 129];
            }
            float4 s[2][4];
#pragma unroll
            for (int i = 0; i < 2; i++)
#pragma unroll
                for (int j = 0; j < 4; j++)
                    s[i][j] = lds128(stage + slot * STAGE_FLOATS + (8 * w + 4 * i + sr) * 128 + (cc + j * 8) * 4);
            __syncthreads();                              // the half-head is in registers everywhere: refill the slot
            if (tid == 0 && m + STAGES < M) {
                bc_fence_proxy_async();
                issue(m + STAGES, 3);
            }
            if (h == 0 && k > 0) finish((k - 1) & 1);
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const int r = 64 * h + 8 * w + 4 * i + sr;
                float recall = 0.0f;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    s[i][j].x *= alpha; s[i][j].y *= alpha; s[i][j].z *= alpha; s[i][j].w *= alpha;
                    recall += s[i][j].x * kr[j].x + s[i][j].y * kr[j].y + s[i][j].z * kr[j].z + s[i][j].w * kr[j].w;
                }
                recall += __shfl_xor_sync(0xffffffffu, recall, 1);
                recall += __shfl_xor_sync(0xffffffffu, recall, 2);
                recall += __shfl_xor_sync(0xffffffffu, recall, 4);
                const float uu = beta * (vv[h][i] - recall);
                float read = 0.0f;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    s[i][j].x += uu * kr[j].x; s[i][j].y += uu * kr[j].y; s[i][j].z += uu * kr[j].z; s[i][j].w += uu * kr[j].w;
                    read += s[i][j].x * qr[j].x + s[i][j].y * qr[j].y + s[i][j].z * qr[j].z + s[i][j].w * qr[j].w;
                    if (!ok) s[i][j] = make_float4(NAN, NAN, NAN, NAN);
                    __stcs(reinterpret_cast<float4 *>(S + (size_t)r * 128) + cc + j * 8, s[i][j]);
                }
                read += __shfl_xor_sync(0xffffffffu, read, 1);
                read += __shfl_xor_sync(0xffffffffu, read, 2);
                read += __shfl_xor_sync(0xffffffffu, read, 4);
                orow[h][i] = read * a.out_scale;          // scaled head output of row r (all 8 lanes agree)
                if (cc == 0) ss += (double)orow[h][i] * (double)orow[h][i];
            }
        }
        ss = warp_sum(ss);
        if (lane == 0) redd[k & 1][w] = ss;
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
            for (int i = 0; i < 2; i++) { po[h][i] = orow[h][i]; pz[h][i] = zc[h][i]; }
        pbase = (size_t)b * vd + (size_t)hv * 128;
    }
    __syncthreads();
    if (n_mine > 0) finish((n_mine - 1) & 1);
}

// The front-end blocks of a call live in a buffer kept per (device, stream): calls on one stream
// run in order and may share it, calls on different streams must not.  It only ever grows, so a
// host that has made one call at its largest batch allocates nothing on the token path afterwards
// (growing frees the old buffer with cudaFree, which waits for the work that still reads it).
struct FrontBuf { float *p = nullptr; size_t bytes = 0; };
std::mutex g_front_mu;
std::map<std::pair<int, cudaStream_t>, FrontBuf> g_front_bufs;

ornith_status front_blocks(cudaStream_t s, size_t bytes, float **out) {
    int dev = 0;
    ORN_TRY(orn_check(cudaGetDevice(&dev), "cudaGetDevice"));
    std::lock_guard<std::mutex> lock(g_front_mu);
    FrontBuf &fb = g_front_bufs[{dev, s}];
    if (fb.bytes < bytes) {
        if (fb.p) ORN_TRY(orn_check(cudaFree(fb.p), "decode front-end blocks (free)"));
        fb.p = nullptr; fb.bytes = 0;
        ORN_TRY(orn_device_alloc((void **)&fb.p, bytes, "decode front-end blocks"));
        fb.bytes = bytes;
    }
    *out = fb.p;
    return ORNITH_OK;
}

template <typename ACT>
ornith_status launch_ring(const LinArgs &x, int n_seq, cudaStream_t s) {
    static int n_sm_dev[ORN_MAX_DEVICES] = {};             // SM count and smem opt-in are per device
    int &n_sm = n_sm_dev[orn_device_index()];
    if (!n_sm) {
        int dev = 0, n = 0;
        ORN_TRY(orn_check(cudaGetDevice(&dev), "cudaGetDevice"));
        ORN_TRY(orn_check(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev), "SM count"));
        ORN_TRY(orn_check(cudaFuncSetAttribute(k_linear_decode_ring<ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, RING_SMEM),
                          "decode ring smem opt-in"));
        n_sm = n;
    }
    float *front = nullptr;
    ORN_TRY(front_blocks(s, (size_t)n_seq * front_stride(x.nk, x.nv) * sizeof(float), &front));
    const int n_units = n_seq * x.nv;
    ornith_status st = orn_check(orn_launch_dependent(k_linear_decode_front<ACT>, dim3(x.nk + (x.nv + 1) / 2, n_seq), dim3(128), 0, s, x, front),
                                 "k_linear_decode_front");
    if (st == ORNITH_OK) {
        const int grid = n_units < 2 * n_sm ? n_units : 2 * n_sm;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = RING_SMEM; cfg.stream = s;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        st = orn_check(cudaLaunchKernelEx(&cfg, k_linear_decode_ring<ACT>, x, (const float *)front, n_units), "k_linear_decode_ring");
    }
    return st;
}

}  // namespace

// Frees the front-end buffer kept for `s` on the current device (all streams of the device when
// all is set), after the work queued on it has finished.
ornith_status release_linear_decode_buffers(cudaStream_t s, bool all) {
    int dev = 0;
    ORN_TRY(orn_check(cudaGetDevice(&dev), "cudaGetDevice"));
    std::lock_guard<std::mutex> lock(g_front_mu);
    ornith_status rc = ORNITH_OK;
    for (auto it = g_front_bufs.begin(); it != g_front_bufs.end();) {
        if (it->first.first == dev && (all || it->first.second == s)) {
            if (it->second.p && cudaFree(it->second.p) != cudaSuccess) { (void)cudaGetLastError(); rc = (ornith_status)ORNITH_ERR_BACKEND; }
            it = g_front_bufs.erase(it);
        } else {
            ++it;
        }
    }
    return rc;
}

ornith_status launch_linear_decode_ring(const LinArgs &x, int n_seq, int act_dtype, cudaStream_t s) {
    return act_dtype == ORNITH_ACT_BF16 ? launch_ring<__nv_bfloat16>(x, n_seq, s) : launch_ring<float>(x, n_seq, s);
}
