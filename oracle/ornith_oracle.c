/* ornith_oracle.c — CPU restatement of the ornithology attention hot path.
 *
 * TEST INFRASTRUCTURE ONLY: the checker for the CUDA kernels, never part of the
 * product path. Each routine keeps the reference's arithmetic order so that,
 * built with the same flags, it reproduces the reference bit for bit; the
 * reference location is cited at every routine.
 */
#include "ornith_oracle.h"
#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ====================================================================== */
/* RNG — splitmix64 (src/ornith_tensor.c:44-62)                           */
/* ====================================================================== */

void orc_rng_seed(orc_rng *r, uint64_t seed) { r->s = seed; }

static uint64_t rng_u64(orc_rng *r) {
    r->s += 0x9E3779B97F4A7C15ULL;
    uint64_t z = r->s;
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ULL;
    z ^= z >> 27; z *= 0x94D049BB133111EBULL;
    z ^= z >> 31;
    return z;
}

float orc_rng_uniform(orc_rng *r, float lo, float hi) {
    uint32_t top24 = (uint32_t)(rng_u64(r) >> 40);
    float unit = (float)top24 / (float)(1u << 24);
    return lo + (hi - lo) * unit;
}

void orc_rng_fill(orc_rng *r, float *dst, int64_t n, float lo, float hi) {
    for (int64_t i = 0; i < n; i++) dst[i] = orc_rng_uniform(r, lo, hi);
}

/* ====================================================================== */
/* elementwise helpers (src/ornith_tensor.c:100-178)                      */
/* ====================================================================== */

float orc_dot(const float *a, const float *b, int n) {
    float s = 0.0f;
    for (int i = 0; i < n; i++) s += a[i] * b[i];
    return s;
}

static double sumsq_f64(const float *x, int n) {
    double s = 0.0;
    for (int i = 0; i < n; i++) s += (double)x[i] * x[i];
    return s;
}

void orc_rmsnorm(const float *x, const float *w, float *out, int n, float eps) {
    float inv = (float)(1.0 / sqrt(sumsq_f64(x, n) / (double)n + (double)eps));
    for (int i = 0; i < n; i++) out[i] = x[i] * inv * (w ? w[i] : 1.0f);
}

void orc_l2norm_eps(const float *x, float *out, int n, float eps) {
    float inv = (float)(1.0 / sqrt(sumsq_f64(x, n) + (double)eps));
    for (int i = 0; i < n; i++) out[i] = x[i] * inv;
}

void orc_softmax(float *x, int n) {
    float top = x[0];
    for (int i = 1; i < n; i++) if (x[i] > top) top = x[i];
    double z = 0.0;
    for (int i = 0; i < n; i++) { x[i] = expf(x[i] - top); z += x[i]; }
    float inv = (float)(1.0 / z);
    for (int i = 0; i < n; i++) x[i] *= inv;
}

float orc_sigmoid(float x)  { return 1.0f / (1.0f + expf(-x)); }
float orc_silu(float x)     { return x * orc_sigmoid(x); }
float orc_softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

void orc_rope_partial(float *v, int head_dim, int rotary_dim, int pos, float theta) {
    if (rotary_dim <= 0 || rotary_dim > head_dim) rotary_dim = head_dim;
    int half = rotary_dim / 2;
    for (int i = 0; i < half; i++) {
        float freq = powf(theta, -2.0f * (float)i / (float)rotary_dim);
        float ang = (float)pos * freq;
        float c = cosf(ang), s = sinf(ang);
        float lo = v[i], hi = v[i + half];
        v[i]        = lo * c - hi * s;
        v[i + half] = lo * s + hi * c;
    }
}

/* ====================================================================== */
/* f16 conversion + Q8_0 (src/ornith_quant.c:14-65, :155-184)             */
/* ====================================================================== */

/* round-to-nearest-even f32 -> f16, subnormals kept, overflow to inf,
 * NaN -> quiet NaN with the sign kept. */
uint16_t orc_f32_to_f16(float f) {
    uint32_t bits; memcpy(&bits, &f, 4);
    uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
    uint32_t bexp = (bits >> 23) & 0xffu;
    uint32_t frac = bits & 0x7fffffu;
    if (bexp == 0xffu) return (uint16_t)(sign | 0x7c00u | (frac ? 0x0200u : 0u));
    int e = (int)bexp - 112;                 /* re-biased half exponent */
    if (e >= 31) return (uint16_t)(sign | 0x7c00u);
    if (e <= 0) {
        if (e < -10) return sign;            /* below half of the least subnormal */
        uint32_t sig = frac | 0x800000u;
        unsigned sh = (unsigned)(14 - e);    /* 14..24 */
        uint32_t keep = sig >> sh;
        uint32_t lost = sig & ((1u << sh) - 1u);
        uint32_t mid  = 1u << (sh - 1);
        if (lost > mid || (lost == mid && (keep & 1u))) keep++;
        return (uint16_t)(sign | keep);
    }
    uint32_t h = ((uint32_t)e << 10) | (frac >> 13);
    uint32_t lost = frac & 0x1fffu;
    if (lost > 0x1000u || (lost == 0x1000u && (h & 1u))) h++;   /* may carry into exp */
    return (uint16_t)(sign | h);
}

float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu, bits;
    if (e == 0x1fu)      bits = sign | 0x7f800000u | (m << 13);
    else if (e)          bits = sign | ((e + 112u) << 23) | (m << 13);
    else if (!m)         bits = sign;
    else {
        int be = 113;
        while (!(m & 0x400u)) { m <<= 1; be--; }
        bits = sign | ((uint32_t)be << 23) | ((m & 0x3ffu) << 13);
    }
    float out; memcpy(&out, &bits, 4);
    return out;
}

/* block of 32: d = amax/127, id = d ? 1/d : 0, code = lroundf(x*id) clamped,
 * scale stored as little-endian f16 (src/ornith_quant.c:155-175). */
int orc_q8_0_encode(const float *src, uint8_t *dst, size_t n) {
    if (n % 32) return -1;
    for (size_t b = 0; b < n / 32; b++) {
        const float *x = src + 32 * b;
        uint8_t *blk = dst + 34 * b;
        float amax = 0.0f;
        for (int j = 0; j < 32; j++) { float a = fabsf(x[j]); if (a > amax) amax = a; }
        float d = amax / 127.0f;
        float id = d ? 1.0f / d : 0.0f;
        uint16_t hd = orc_f32_to_f16(d);
        blk[0] = (uint8_t)(hd & 0xff); blk[1] = (uint8_t)(hd >> 8);
        for (int j = 0; j < 32; j++) {
            float scaled = x[j] * id;
            int32_t q = (int32_t)lroundf(scaled);
            if (q > 127) q = 127;
            if (q < -127) q = -127;
            blk[2 + j] = (uint8_t)(int8_t)q;
        }
    }
    return 0;
}

int orc_q8_0_decode(const uint8_t *src, float *dst, size_t n) {   /* :177-184 */
    if (n % 32) return -1;
    for (size_t b = 0; b < n / 32; b++) {
        const uint8_t *blk = src + 34 * b;
        float d = orc_f16_to_f32((uint16_t)(blk[0] | ((uint16_t)blk[1] << 8)));
        for (int j = 0; j < 32; j++) dst[32 * b + j] = (float)(int8_t)blk[2 + j] * d;
    }
    return 0;
}

/* src/ornith_attn.c:65-77 — note lrintf (ties to even) and inv = 127/amax. */
float orc_kv_int8_encode(const float *x, int n, int8_t *q) {
    float amax = 0.0f;
    for (int i = 0; i < n; i++) { float a = fabsf(x[i]); if (a > amax) amax = a; }
    if (amax == 0.0f) { memset(q, 0, (size_t)n); return 0.0f; }
    float scale = amax / 127.0f, inv = 127.0f / amax;
    for (int i = 0; i < n; i++) {
        int c = (int)lrintf(x[i] * inv);
        if (c > 127) c = 127;
        if (c < -127) c = -127;
        q[i] = (int8_t)c;
    }
    return scale;
}

/* ====================================================================== */
/* KV cache + GQA (src/ornith_attn.c:12-176)                              */
/* ====================================================================== */

size_t orc_kv_bytes_per_token(int nkv, int hd, int mode) {
    size_t n = (size_t)nkv * hd;
    if (mode == ORC_KV_INT8_HEAD) return 2 * (n + (size_t)nkv * sizeof(float));   /* :12-18 */
    if (mode == ORC_KV_Q8_0)      return 2 * (n / 32) * 34;
    return 2 * n * sizeof(float);
}

int orc_kv_init(orc_kv *c, int capacity, int nkv, int hd, int mode) {
    memset(c, 0, sizeof(*c));
    c->mode = mode; c->capacity = capacity; c->n_kv_heads = nkv; c->head_dim = hd;
    size_t rows = (size_t)capacity * nkv, elems = rows * hd;
    if (mode == ORC_KV_INT8_HEAD) {
        c->Kq = calloc(elems, 1); c->Vq = calloc(elems, 1);
        c->Ks = calloc(rows, sizeof(float)); c->Vs = calloc(rows, sizeof(float));
        if (!c->Kq || !c->Vq || !c->Ks || !c->Vs) { orc_kv_free(c); return -1; }
        return 0;
    }
    c->K = calloc(elems, sizeof(float)); c->V = calloc(elems, sizeof(float));
    if (!c->K || !c->V) { orc_kv_free(c); return -1; }
    if (mode == ORC_KV_Q8_0) {
        if (hd % 32) { orc_kv_free(c); return -1; }
        c->Kb = calloc(rows * (hd / 32), 34); c->Vb = calloc(rows * (hd / 32), 34);
        if (!c->Kb || !c->Vb) { orc_kv_free(c); return -1; }
    }
    return 0;
}

void orc_kv_free(orc_kv *c) {
    if (!c) return;
    free(c->K); free(c->V); free(c->Kq); free(c->Vq);
    free(c->Ks); free(c->Vs); free(c->Kb); free(c->Vb);
    memset(c, 0, sizeof(*c));
}

/* scale * sum(q_i * (float)code_i), skipped for a zero scale (:80-85) */
static float dot_int8(const float *q, const int8_t *code, float scale, int n) {
    if (scale == 0.0f) return 0.0f;
    float s = 0.0f;
    for (int i = 0; i < n; i++) s += q[i] * (float)code[i];
    return s * scale;
}

void orc_gqa_step(orc_kv *c, const float *q, const float *k_new, const float *v_new,
                  int n_heads, float *out, float scale) {
    int hd = c->head_dim, nkv = c->n_kv_heads;
    if (scale <= 0.0f) scale = 1.0f / sqrtf((float)hd);
    if (c->len >= c->capacity) return;                     /* full cache: no-op (:92) */
    int pos = c->len;
    size_t row0 = (size_t)pos * nkv;
    if (c->mode == ORC_KV_INT8_HEAD) {
        for (int h = 0; h < nkv; h++) {
            c->Ks[row0 + h] = orc_kv_int8_encode(k_new + (size_t)h * hd, hd, c->Kq + (row0 + h) * hd);
            c->Vs[row0 + h] = orc_kv_int8_encode(v_new + (size_t)h * hd, hd, c->Vq + (row0 + h) * hd);
        }
    } else if (c->mode == ORC_KV_Q8_0) {
        size_t rb = (size_t)(hd / 32) * 34;
        for (int h = 0; h < nkv; h++) {
            orc_q8_0_encode(k_new + (size_t)h * hd, c->Kb + (row0 + h) * rb, hd);
            orc_q8_0_encode(v_new + (size_t)h * hd, c->Vb + (row0 + h) * rb, hd);
            orc_q8_0_decode(c->Kb + (row0 + h) * rb, c->K + (row0 + h) * hd, hd);
            orc_q8_0_decode(c->Vb + (row0 + h) * rb, c->V + (row0 + h) * hd, hd);
        }
    } else {
        memcpy(c->K + row0 * hd, k_new, (size_t)nkv * hd * sizeof(float));
        memcpy(c->V + row0 * hd, v_new, (size_t)nkv * hd * sizeof(float));
    }
    c->len++;

    int T = c->len, per_kv = n_heads / nkv;
    float *w = malloc((size_t)T * sizeof(float));
    for (int h = 0; h < n_heads; h++) {
        int kvh = h / per_kv;
        const float *qh = q + (size_t)h * hd;
        float *oh = out + (size_t)h * hd;
        if (c->mode == ORC_KV_INT8_HEAD) {
            for (int t = 0; t < T; t++) {
                size_t r = (size_t)t * nkv + kvh;
                w[t] = dot_int8(qh, c->Kq + r * hd, c->Ks[r], hd) * scale;
            }
        } else {
            for (int t = 0; t < T; t++)
                w[t] = orc_dot(qh, c->K + ((size_t)t * nkv + kvh) * hd, hd) * scale;
        }
        orc_softmax(w, T);
        memset(oh, 0, (size_t)hd * sizeof(float));
        if (c->mode == ORC_KV_INT8_HEAD) {
            for (int t = 0; t < T; t++) {
                size_t r = (size_t)t * nkv + kvh;
                float pw = w[t] * c->Vs[r];
                if (pw == 0.0f) continue;
                const int8_t *vt = c->Vq + r * hd;
                for (int i = 0; i < hd; i++) oh[i] += pw * (float)vt[i];
            }
        } else {
            for (int t = 0; t < T; t++) {
                const float *vt = c->V + ((size_t)t * nkv + kvh) * hd;
                for (int i = 0; i < hd; i++) oh[i] += w[t] * vt[i];
            }
        }
    }
    free(w);
}

void orc_gqa_reference(const float *Q, const float *K, const float *V, int T,
                       int n_heads, int nkv, int hd, float *O, float scale) {
    if (scale <= 0.0f) scale = 1.0f / sqrtf((float)hd);
    int per_kv = n_heads / nkv;
    float *w = malloc((size_t)T * sizeof(float));
    for (int i = 0; i < T; i++)
        for (int h = 0; h < n_heads; h++) {
            int kvh = h / per_kv;
            const float *qh = Q + ((size_t)i * n_heads + h) * hd;
            float *oh = O + ((size_t)i * n_heads + h) * hd;
            for (int j = 0; j <= i; j++)
                w[j] = orc_dot(qh, K + ((size_t)j * nkv + kvh) * hd, hd) * scale;
            orc_softmax(w, i + 1);
            memset(oh, 0, (size_t)hd * sizeof(float));
            for (int j = 0; j <= i; j++) {
                const float *vj = V + ((size_t)j * nkv + kvh) * hd;
                for (int d = 0; d < hd; d++) oh[d] += w[j] * vj[d];
            }
        }
    free(w);
}

/* ====================================================================== */
/* gated delta rule (src/ornith_attn.c:196-349). S is [dv][dk] row-major. */
/* ====================================================================== */

void orc_delta_step(float *S, int dk, int dv, const float *q, const float *k,
                    const float *v, float alpha, float beta, float *o) {
    for (int i = 0; i < dk * dv; i++) S[i] *= alpha;
    for (int r = 0; r < dv; r++) {
        float *row = S + (size_t)r * dk;
        float recall = orc_dot(row, k, dk);
        float u = beta * (v[r] - recall);
        for (int c = 0; c < dk; c++) row[c] += u * k[c];
        o[r] = orc_dot(row, q, dk);
    }
}

/* One chunk of C tokens against the incoming state (src/ornith_attn.c:244-335).
 * Decay ratios p_i/p_j are built as running sub-products of alpha, never as a
 * quotient of cumulative products. */
static void delta_one_chunk(float *S, int dk, int dv, const float *Q, const float *K,
                            const float *V, const float *alpha, const float *beta,
                            int C, float *O) {
    float *p   = malloc((size_t)C * sizeof(float));
    float *SK  = malloc((size_t)C * dv * sizeof(float));
    float *SQ  = malloc((size_t)C * dv * sizeof(float));
    float *U   = malloc((size_t)C * dv * sizeof(float));
    float *Gkk = malloc((size_t)C * C * sizeof(float));
    float *Gkq = malloc((size_t)C * C * sizeof(float));

    for (int i = 0; i < C; i++) p[i] = i ? p[i - 1] * alpha[i] : alpha[0];

    for (int i = 0; i < C; i++) {
        const float *ki = K + (size_t)i * dk, *qi = Q + (size_t)i * dk;
        for (int r = 0; r < dv; r++) {
            const float *row = S + (size_t)r * dk;
            SK[(size_t)i * dv + r] = orc_dot(row, ki, dk);
            SQ[(size_t)i * dv + r] = orc_dot(row, qi, dk);
        }
        for (int j = 0; j < C; j++) {
            const float *kj = K + (size_t)j * dk;
            Gkk[(size_t)i * C + j] = orc_dot(kj, ki, dk);
            Gkq[(size_t)i * C + j] = orc_dot(kj, qi, dk);
        }
    }

    /* forward substitution for the write values u_i */
    for (int i = 0; i < C; i++) {
        float b = beta[i], pi = p[i];
        float *ui = U + (size_t)i * dv;
        const float *vi = V + (size_t)i * dv;
        for (int r = 0; r < dv; r++) ui[r] = b * vi[r] - b * pi * SK[(size_t)i * dv + r];
        float ratio = 1.0f;
        for (int j = i - 1; j >= 0; j--) {
            ratio *= alpha[j + 1];
            float m = b * ratio * Gkk[(size_t)i * C + j];
            if (m != 0.0f) {
                const float *uj = U + (size_t)j * dv;
                for (int r = 0; r < dv; r++) ui[r] -= m * uj[r];
            }
        }
    }

    /* reads: carried state, then the diagonal term, then earlier writes newest first */
    for (int i = 0; i < C; i++) {
        float pi = p[i];
        float *oi = O + (size_t)i * dv;
        for (int r = 0; r < dv; r++) oi[r] = pi * SQ[(size_t)i * dv + r];
        float wd = Gkq[(size_t)i * C + i];
        const float *ui = U + (size_t)i * dv;
        for (int r = 0; r < dv; r++) oi[r] += wd * ui[r];
        float ratio = 1.0f;
        for (int j = i - 1; j >= 0; j--) {
            ratio *= alpha[j + 1];
            float w = ratio * Gkq[(size_t)i * C + j];
            const float *uj = U + (size_t)j * dv;
            for (int r = 0; r < dv; r++) oi[r] += w * uj[r];
        }
    }

    /* carry the state across the chunk */
    float pend = p[C - 1];
    for (int i = 0; i < dk * dv; i++) S[i] *= pend;
    float ratio = 1.0f;
    for (int j = C - 1; j >= 0; j--) {
        const float *uj = U + (size_t)j * dv, *kj = K + (size_t)j * dk;
        for (int r = 0; r < dv; r++) {
            float ur = ratio * uj[r];
            if (ur == 0.0f) continue;
            float *row = S + (size_t)r * dk;
            for (int c = 0; c < dk; c++) row[c] += ur * kj[c];
        }
        ratio *= alpha[j];
    }
    free(p); free(SK); free(SQ); free(U); free(Gkk); free(Gkq);
}

void orc_delta_prefill(float *S, int dk, int dv, const float *Q, const float *K,
                       const float *V, const float *alpha, const float *beta,
                       int T, int chunk, float *O) {
    if (chunk < 1) chunk = 1;
    if (chunk > T) chunk = T;
    for (int t0 = 0; t0 < T; t0 += chunk) {
        int C = t0 + chunk <= T ? chunk : T - t0;
        delta_one_chunk(S, dk, dv, Q + (size_t)t0 * dk, K + (size_t)t0 * dk,
                        V + (size_t)t0 * dv, alpha + t0, beta + t0, C, O + (size_t)t0 * dv);
    }
}

/* ====================================================================== */
/* causal depthwise conv (src/ornith_attn.c:369-397)                      */
/* ====================================================================== */

void orc_conv_step(float *buf, int K, int C, const float *x, const float *w,
                   const float *bias, float *out) {
    for (int c = 0; c < C; c++) {
        float acc = bias ? bias[c] : 0.0f;
        const float *wc = w + (size_t)c * K;
        for (int j = 0; j < K - 1; j++) acc += wc[j] * buf[(size_t)j * C + c];
        acc += wc[K - 1] * x[c];
        out[c] = acc;
    }
    if (K >= 2) {
        memmove(buf, buf + C, (size_t)(K - 2) * C * sizeof(float));
        memcpy(buf + (size_t)(K - 2) * C, x, (size_t)C * sizeof(float));
    }
}

void orc_conv_prefill(float *buf, int K, int C, const float *X, const float *w,
                      const float *bias, int T, float *OUT) {
    for (int t = 0; t < T; t++)
        orc_conv_step(buf, K, C, X + (size_t)t * C, w, bias, OUT + (size_t)t * C);
}

/* ====================================================================== */
/* layer wiring without the projections                                    */
/* ====================================================================== */

static int key_head_of(const orc_linear_params *p, int hv) {
    return p->head_map == ORC_HEADMAP_GROUPED ? hv / (p->nv / p->nk) : hv % p->nk;
}

/* exp(a_coef * softplus(a_in + dt_bias)) (src/ornith_rforward.c:282-284) */
static float decay_of(float a_in, float a_coef, float dt_bias) {
    return expf(a_coef * orc_softplus(a_in + dt_bias));
}

/* scale, per-head RMSNorm, SiLU(z) gate (src/ornith_rforward.c:305-314);
 * o_all is overwritten by the scale like the reference does. */
static void gated_norm_out(const orc_linear_params *p, float *o_all, const float *z, float *out) {
    int vd = p->nv * p->dv;
    if (p->out_scale != 1.0f) for (int i = 0; i < vd; i++) o_all[i] *= p->out_scale;
    for (int hv = 0; hv < p->nv; hv++)
        orc_rmsnorm(o_all + (size_t)hv * p->dv, p->norm_w, out + (size_t)hv * p->dv, p->dv, p->eps);
    for (int i = 0; i < vd; i++) out[i] *= orc_silu(z[i]);
}

void orc_linear_attn_step(const orc_linear_params *p, float *S, float *conv_buf,
                          const float *qkv, const float *a, const float *b,
                          const float *z, float *out) {
    int nk = p->nk, nv = p->nv, dk = p->dk, dv = p->dv;
    int qd = nk * dk, vd = nv * dv, Cc = 2 * qd + vd;
    float *conv = malloc((size_t)Cc * sizeof(float));
    float *qn = malloc((size_t)qd * sizeof(float));
    float *kn = malloc((size_t)qd * sizeof(float));
    float *o_all = malloc((size_t)vd * sizeof(float));
    orc_conv_step(conv_buf, p->conv_k, Cc, qkv, p->conv_w, p->conv_b, conv);
    for (int i = 0; i < Cc; i++) conv[i] = orc_silu(conv[i]);
    const float *q = conv, *k = conv + qd, *v = conv + 2 * qd;
    for (int h = 0; h < nk; h++) {
        orc_l2norm_eps(q + (size_t)h * dk, qn + (size_t)h * dk, dk, 1e-6f);
        orc_l2norm_eps(k + (size_t)h * dk, kn + (size_t)h * dk, dk, 1e-6f);
    }
    for (int hv = 0; hv < nv; hv++) {
        int kh = key_head_of(p, hv);
        float alpha = decay_of(a[hv], p->a_coef[hv], p->dt_bias[hv]);
        orc_delta_step(S + (size_t)hv * dv * dk, dk, dv, qn + (size_t)kh * dk, kn + (size_t)kh * dk,
                       v + (size_t)hv * dv, alpha, orc_sigmoid(b[hv]), o_all + (size_t)hv * dv);
    }
    gated_norm_out(p, o_all, z, out);
    free(conv); free(qn); free(kn); free(o_all);
}

void orc_linear_attn_prefill(const orc_linear_params *p, float *S, float *conv_buf,
                             const float *QKV, const float *A, const float *B,
                             const float *Z, int T, int chunk, float *OUT) {
    int nk = p->nk, nv = p->nv, dk = p->dk, dv = p->dv;
    int qd = nk * dk, vd = nv * dv, Cc = 2 * qd + vd;
    float *CONV = malloc((size_t)T * Cc * sizeof(float));
    orc_conv_prefill(conv_buf, p->conv_k, Cc, QKV, p->conv_w, p->conv_b, T, CONV);
    for (size_t i = 0; i < (size_t)T * Cc; i++) CONV[i] = orc_silu(CONV[i]);
    float *Qh = malloc((size_t)T * dk * sizeof(float));
    float *Kh = malloc((size_t)T * dk * sizeof(float));
    float *Vh = malloc((size_t)T * dv * sizeof(float));
    float *Oh = malloc((size_t)T * dv * sizeof(float));
    float *al = malloc((size_t)T * sizeof(float));
    float *be = malloc((size_t)T * sizeof(float));
    float *O_all = malloc((size_t)T * vd * sizeof(float));
    for (int hv = 0; hv < nv; hv++) {
        int kh = key_head_of(p, hv);
        for (int t = 0; t < T; t++) {
            const float *row = CONV + (size_t)t * Cc;
            orc_l2norm_eps(row + kh * dk, Qh + (size_t)t * dk, dk, 1e-6f);
            orc_l2norm_eps(row + qd + kh * dk, Kh + (size_t)t * dk, dk, 1e-6f);
            memcpy(Vh + (size_t)t * dv, row + 2 * qd + hv * dv, (size_t)dv * sizeof(float));
            al[t] = decay_of(A[(size_t)t * nv + hv], p->a_coef[hv], p->dt_bias[hv]);
            be[t] = orc_sigmoid(B[(size_t)t * nv + hv]);
        }
        orc_delta_prefill(S + (size_t)hv * dv * dk, dk, dv, Qh, Kh, Vh, al, be, T, chunk, Oh);
        for (int t = 0; t < T; t++)
            memcpy(O_all + (size_t)t * vd + hv * dv, Oh + (size_t)t * dv, (size_t)dv * sizeof(float));
    }
    for (int t = 0; t < T; t++)
        gated_norm_out(p, O_all + (size_t)t * vd, Z + (size_t)t * vd, OUT + (size_t)t * vd);
    free(CONV); free(Qh); free(Kh); free(Vh); free(Oh); free(al); free(be); free(O_all);
}

void orc_full_attn_step(const orc_full_params *p, orc_kv *c, int pos,
                        const float *qproj, const float *k, const float *v, float *out) {
    int nh = p->nh, nkv = p->nkv, hd = p->hd;
    float *q  = malloc((size_t)nh * hd * sizeof(float));
    float *g  = malloc((size_t)nh * hd * sizeof(float));
    float *kk = malloc((size_t)nkv * hd * sizeof(float));
    for (int h = 0; h < nh; h++) {                       /* head h packs [q | gate] */
        memcpy(q + (size_t)h * hd, qproj + (size_t)h * 2 * hd, (size_t)hd * sizeof(float));
        memcpy(g + (size_t)h * hd, qproj + (size_t)h * 2 * hd + hd, (size_t)hd * sizeof(float));
    }
    memcpy(kk, k, (size_t)nkv * hd * sizeof(float));
    for (int h = 0; h < nh; h++) {
        orc_rmsnorm(q + (size_t)h * hd, p->q_norm_w, q + (size_t)h * hd, hd, p->eps);
        orc_rope_partial(q + (size_t)h * hd, hd, p->rope_dim, pos, p->theta);
    }
    for (int h = 0; h < nkv; h++) {
        orc_rmsnorm(kk + (size_t)h * hd, p->k_norm_w, kk + (size_t)h * hd, hd, p->eps);
        orc_rope_partial(kk + (size_t)h * hd, hd, p->rope_dim, pos, p->theta);
    }
    orc_gqa_step(c, q, kk, v, nh, out, 0.0f);
    for (int i = 0; i < nh * hd; i++) out[i] *= orc_sigmoid(g[i]);
    free(q); free(g); free(kk);
}

void orc_full_attn_prefill(const orc_full_params *p, orc_kv *c, int base, int T,
                           const float *QP, const float *K, const float *V, float *OUT) {
    size_t qp = (size_t)p->nh * 2 * p->hd, kvd = (size_t)p->nkv * p->hd, qd = (size_t)p->nh * p->hd;
    for (int t = 0; t < T; t++)
        orc_full_attn_step(p, c, base + t, QP + t * qp, K + t * kvd, V + t * kvd, OUT + t * qd);
}

/* ======================================================================== */
/* quantised projections                                                     */
/* ======================================================================== */

/* src/ornith_qdot.c:38-70: the element of largest magnitude (first one on ties) fixes the scale
 * -127/max, values are rounded to nearest even, d = 1/iscale; an all-zero block stays zero. */
void orc_q8k_quantize(const float *x, orc_q8k_block *y, int64_t k) {
    const int64_t nb = k / 256;
    for (int64_t b = 0; b < nb; b++, x += 256) {
        float amax = 0.0f, max = 0.0f;
        for (int j = 0; j < 256; j++) {
            const float ax = fabsf(x[j]);
            if (ax > amax) { amax = ax; max = x[j]; }
        }
        if (amax == 0.0f) {
            y[b].d = 0.0f;
            memset(y[b].qs, 0, sizeof y[b].qs);
            memset(y[b].bsums, 0, sizeof y[b].bsums);
            continue;
        }
        const float iscale = -127.0f / max;
        for (int j = 0; j < 256; j++) {
            int v = (int)lrintf(iscale * x[j]);
            v = v > 127 ? 127 : (v < -128 ? -128 : v);
            y[b].qs[j] = (int8_t)v;
        }
        for (int g = 0; g < 16; g++) {
            int sum = 0;
            for (int i = 0; i < 16; i++) sum += y[b].qs[16 * g + i];
            y[b].bsums[g] = (int16_t)sum;
        }
        y[b].d = 1.0f / iscale;
    }
}

/* src/ornith_qdot.c:144-163: per super-block of 256 the eight Q8_0 blocks give wd * (float)isum, summed in
 * order; the super-block sum is scaled by the activation's d and added to the running total, in order. */
float orc_vec_dot_q8_0(int n, const uint8_t *wrow, const orc_q8k_block *y) {
    const int nb = n / 256;
    float sumf = 0.0f;
    for (int i = 0; i < nb; i++) {
        const uint8_t *w = wrow + (size_t)i * 8 * 34;
        float blk_sum = 0.0f;
        for (int sb = 0; sb < 8; sb++) {
            const uint8_t *wb = w + (size_t)sb * 34;
            const float wd = orc_f16_to_f32((uint16_t)(wb[0] | ((uint16_t)wb[1] << 8)));
            const int8_t *wq = (const int8_t *)(wb + 2), *yq = y[i].qs + 32 * sb;
            int isum = 0;
            for (int l = 0; l < 32; l++) isum += (int)wq[l] * (int)yq[l];
            blk_sum += wd * (float)isum;
        }
        sumf += y[i].d * blk_sum;
    }
    return sumf;
}

int orc_matmul_q8_0(const uint8_t *W, int n_in, int n_out, const float *X, int T, float *Y) {
    if (n_in % 256 != 0) return -1;
    const size_t nblk = (size_t)n_in / 256, rb = (size_t)n_in / 32 * 34;
    orc_q8k_block *xq = malloc((size_t)T * nblk * sizeof *xq);
    if (!xq) return -1;
    for (int t = 0; t < T; t++) orc_q8k_quantize(X + (size_t)t * n_in, xq + (size_t)t * nblk, n_in);
    for (int o = 0; o < n_out; o++)
        for (int t = 0; t < T; t++)
            Y[(size_t)t * n_out + o] = orc_vec_dot_q8_0(n_in, W + (size_t)o * rb, xq + (size_t)t * nblk);
    free(xq);
    return 0;
}

/* ---- k-quant weights x Q8_K activations (src/ornith_qdot.c:63-141) ----------------------------------------
 * Both formats hold 256 weights per super-block.  The dot over a super-block is an integer: codes times
 * activation codes, weighted by small integer sub-block scales; one f32 product per super-block applies the
 * weight's f16 scale and the activation's f32 scale.  The running total is f32, super-blocks in order. */

/* Q4_K block, 144 bytes: f16 d, f16 dmin, 12 bytes of packed 6-bit (scale, min) pairs for 8 sub-blocks of 32,
 * 128 bytes of 4-bit codes (sub-blocks 2p and 2p+1 share bytes 32p..32p+31: low and high nibbles).
 * Sub-block j < 4 has its scale in the low 6 bits of byte j and its min in the low 6 bits of byte j + 4; for
 * j >= 4 the low 4 bits come from the two nibbles of byte j + 4 and the top 2 bits from the top bits of bytes
 * j - 4 (scale) and j (min) (src/ornith_qdot.c:65-71). */
static void orc_q4k_scale_min(const uint8_t *sc12, int j, int *scale, int *min) {
    if (j < 4) {
        *scale = sc12[j] & 0x3F;
        *min = sc12[j + 4] & 0x3F;
    } else {
        *scale = (sc12[j + 4] & 0x0F) | ((sc12[j - 4] >> 6) << 4);
        *min = (sc12[j + 4] >> 4) | ((sc12[j] >> 6) << 4);
    }
}

/* src/ornith_qdot.c:75-105: value of weight e = d * scale_j * code_e - dmin * min_j, so the dot splits into
 * d * sum_j scale_j (codes . activation codes) and -dmin * sum_j min_j (sum of the sub-block's activation codes,
 * taken from the block's 16-sums). */
float orc_vec_dot_q4_K(int n, const uint8_t *wrow, const orc_q8k_block *y) {
    float total = 0.0f;
    for (int i = 0; i < n / 256; i++) {
        const uint8_t *blk = wrow + (size_t)i * 144, *sc12 = blk + 4, *codes = blk + 16;
        const float d = y[i].d * orc_f16_to_f32((uint16_t)(blk[0] | ((uint16_t)blk[1] << 8)));
        const float dmin = -y[i].d * orc_f16_to_f32((uint16_t)(blk[2] | ((uint16_t)blk[3] << 8)));
        int dots = 0, mins = 0;
        for (int j = 0; j < 8; j++) {
            int scale, min;
            orc_q4k_scale_min(sc12, j, &scale, &min);
            mins += min * ((int)y[i].bsums[2 * j] + (int)y[i].bsums[2 * j + 1]);
            const uint8_t *src = codes + 32 * (j / 2);
            int part = 0;
            for (int l = 0; l < 32; l++) {
                const int code = (j & 1) ? (src[l] >> 4) : (src[l] & 0x0F);
                part += code * (int)y[i].qs[32 * j + l];
            }
            dots += part * scale;
        }
        total += d * (float)dots + dmin * (float)mins;
    }
    return total;
}

/* Q6_K block, 210 bytes: 128 bytes of low nibbles, 64 bytes of 2-bit high parts, 16 signed 8-bit scales (one per
 * 16 weights), f16 d.  Weight e (0..255): half h = e / 128, quarter c = (e % 128) / 32, l = e % 32; low nibble =
 * nibble (c / 2) of ql[64 h + 32 (c % 2) + l], high bits = bits 2c, 2c+1 of qh[32 h + l]; code - 32 is the value;
 * its scale is sc[e / 16] (src/ornith_qdot.c:109-141). */
float orc_vec_dot_q6_K(int n, const uint8_t *wrow, const orc_q8k_block *y) {
    float total = 0.0f;
    for (int i = 0; i < n / 256; i++) {
        const uint8_t *blk = wrow + (size_t)i * 210, *ql = blk, *qh = blk + 128;
        const int8_t *sc = (const int8_t *)(blk + 192);
        const float d = y[i].d * orc_f16_to_f32((uint16_t)(blk[208] | ((uint16_t)blk[209] << 8)));
        int dots = 0;
        for (int e = 0; e < 256; e++) {
            const int h = e / 128, c = (e % 128) / 32, l = e % 32;
            const int lo = (ql[64 * h + 32 * (c % 2) + l] >> (4 * (c / 2))) & 0x0F;
            const int hi = (qh[32 * h + l] >> (2 * c)) & 3;
            dots += (int)y[i].qs[e] * ((lo | (hi << 4)) - 32) * (int)sc[e / 16];
        }
        total += d * (float)dots;
    }
    return total;
}

size_t orc_qrow_bytes(int wtype, int n_in) {
    switch (wtype) {
    case ORC_GGML_Q8_0: return (size_t)n_in / 32 * 34;
    case ORC_GGML_Q4_K: return (size_t)n_in / 256 * 144;
    case ORC_GGML_Q6_K: return (size_t)n_in / 256 * 210;
    default: return 0;
    }
}

/* matmul_batch_q (src/ornith_rforward.c:138-192) for any of the three integer paths (qdot_can, src/ornith_qdot.c:167-177) */
int orc_matmul_q(int wtype, const uint8_t *W, int n_in, int n_out, const float *X, int T, float *Y) {
    const size_t rb = orc_qrow_bytes(wtype, n_in);
    if (n_in % 256 != 0 || rb == 0) return -1;
    const size_t nblk = (size_t)n_in / 256;
    orc_q8k_block *xq = malloc((size_t)T * nblk * sizeof *xq);
    if (!xq) return -1;
    for (int t = 0; t < T; t++) orc_q8k_quantize(X + (size_t)t * n_in, xq + (size_t)t * nblk, n_in);
    for (int o = 0; o < n_out; o++)
        for (int t = 0; t < T; t++) {
            const uint8_t *w = W + (size_t)o * rb;
            const orc_q8k_block *a = xq + (size_t)t * nblk;
            Y[(size_t)t * n_out + o] = wtype == ORC_GGML_Q4_K ? orc_vec_dot_q4_K(n_in, w, a)
                                     : wtype == ORC_GGML_Q6_K ? orc_vec_dot_q6_K(n_in, w, a)
                                                              : orc_vec_dot_q8_0(n_in, w, a);
        }
    free(xq);
    return 0;
}
