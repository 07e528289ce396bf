/* ornith_attn_compat.c — tier 1 of the CUDA backend: the engine's attention
 * header (reference: src/ornith_attn.h:71-147), same names, structs, argument
 * meaning and error behaviour, executed by the CUDA kernels.
 *
 * The structs stay what they are in the engine: caller-allocated, with HOST
 * buffers the caller may read, write, memcpy into or fread over
 * (reference call sites: src/ornith_forward.c:458-462, src/ornith_rforward.c:494,
 * :1039-1063, :1129-1152).  Every compute call therefore stages its operands to
 * the device, runs the kernels and copies the results back into the same host
 * images.  KV caches keep a device mirror between calls and re-upload only when
 * the host side moved `len` behind the library's back.  Correct and
 * deliberately simple; the fast path is tier 2 (ornith_cuda.h).
 *
 * There is no CPU implementation here.  Without a usable GPU the init functions
 * still build the host images (so struct handling keeps working) and the
 * compute functions record an error and leave their outputs untouched — they
 * return void in the engine and cannot report failure any other way.
 */
#include <pthread.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "ornith_cuda.h"

/* ---- error text (reference: src/ornith_util.c:7-30) ------------------------- */
static char g_err[512];

const char *ornith_strerror(ornith_status s) {
    switch ((int)s) {
    case ORNITH_OK:              return "ok";
    case ORNITH_ERR_IO:          return "I/O error";
    case ORNITH_ERR_FORMAT:      return "format error";
    case ORNITH_ERR_UNSUPPORTED: return "unsupported";
    case ORNITH_ERR_OOM:         return "out of memory";
    case ORNITH_ERR_NOTFOUND:    return "not found";
    case ORNITH_ERR_BACKEND:     return "CUDA backend error";
    }
    return "unknown error";
}
const char *ornith_last_error(void) { return g_err[0] ? g_err : "(no detail)"; }
void ornith_set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

/* one lock for the whole tier: the engine calls it from arbitrary threads under
 * its own generation mutex (reference: src/ornith_server.c:791) */
static pthread_mutex_t g_lock = PTHREAD_MUTEX_INITIALIZER;

/* ---- grow-only device workspace, carved per call ------------------------------ */
static char  *g_ws;
static size_t g_ws_bytes;

static int ws_reserve(size_t bytes) {
    if (bytes <= g_ws_bytes) return 1;
    if (g_ws) ornith_cuda_free(g_ws);
    g_ws = NULL; g_ws_bytes = 0;
    size_t want = bytes + bytes / 2 + 4096;
    void *p = NULL;
    if (ornith_cuda_malloc(&p, want) != ORNITH_OK) return 0;
    g_ws = p; g_ws_bytes = want;
    return 1;
}
static size_t up256(size_t x) { return (x + 255) / 256 * 256; }

/* ---- KV cache mirrors ---------------------------------------------------------- */
typedef struct {
    const ornith_kv_cache *key;          /* host struct this mirrors, NULL = free slot */
    void  *K, *V;                        /* device pools, engine layout */
    float *Ks, *Vs;
    int64_t *seq_off;                    /* device [2] = {0, capacity} */
    int32_t *len;                        /* device [1] */
    int synced_len, capacity, nkv, hd, quantized;
    const void *hostK;                   /* host image identity at the last sync */
} kv_mirror;

#define MAX_MIRRORS 1024
static kv_mirror g_mir[MAX_MIRRORS];

static void mirror_release(kv_mirror *m) {
    ornith_cuda_free(m->K); ornith_cuda_free(m->V); ornith_cuda_free(m->Ks); ornith_cuda_free(m->Vs);
    ornith_cuda_free(m->seq_off); ornith_cuda_free(m->len);
    memset(m, 0, sizeof(*m));
}

static kv_mirror *mirror_find(const ornith_kv_cache *c) {
    for (int i = 0; i < MAX_MIRRORS; i++) if (g_mir[i].key == c) return &g_mir[i];
    return NULL;
}

static kv_mirror *mirror_get(const ornith_kv_cache *c) {
    kv_mirror *m = mirror_find(c);
    const void *hk = c->quantized ? (const void *)c->Kq : (const void *)c->K;
    if (m && (m->capacity != c->capacity || m->nkv != c->n_kv_heads || m->hd != c->head_dim ||
              m->quantized != c->quantized || m->hostK != hk)) {
        mirror_release(m);               /* the struct was re-initialised in place */
        m = NULL;
    }
    if (m) return m;
    for (int i = 0; i < MAX_MIRRORS && !m; i++) if (!g_mir[i].key) m = &g_mir[i];
    if (!m) { ornith_set_error("too many live KV caches for the CUDA drop-in (%d)", MAX_MIRRORS); return NULL; }
    size_t rows = (size_t)c->capacity * c->n_kv_heads, elems = rows * c->head_dim;
    size_t eb = c->quantized ? 1 : sizeof(float);
    int ok = ornith_cuda_malloc(&m->K, elems * eb) == ORNITH_OK &&
             ornith_cuda_malloc(&m->V, elems * eb) == ORNITH_OK &&
             ornith_cuda_malloc((void **)&m->seq_off, 2 * sizeof(int64_t)) == ORNITH_OK &&
             ornith_cuda_malloc((void **)&m->len, sizeof(int32_t)) == ORNITH_OK;
    if (ok && c->quantized)
        ok = ornith_cuda_malloc((void **)&m->Ks, rows * sizeof(float)) == ORNITH_OK &&
             ornith_cuda_malloc((void **)&m->Vs, rows * sizeof(float)) == ORNITH_OK;
    int64_t off[2] = {0, c->capacity};
    if (ok) ok = ornith_cuda_h2d(m->seq_off, off, sizeof(off)) == ORNITH_OK;
    if (!ok) { mirror_release(m); return NULL; }
    m->key = c; m->capacity = c->capacity; m->nkv = c->n_kv_heads; m->hd = c->head_dim;
    m->quantized = c->quantized; m->hostK = hk; m->synced_len = 0;
    return m;
}

/* copy host rows [from, to) up, or device rows down */
static int mirror_copy(kv_mirror *m, ornith_kv_cache *c, int from, int to, int up) {
    if (to <= from) return 1;
    size_t row = (size_t)c->n_kv_heads * c->head_dim;
    size_t eb = c->quantized ? 1 : sizeof(float);
    size_t o = (size_t)from * row * eb, n = (size_t)(to - from) * row * eb;
    char *hK = c->quantized ? (char *)c->Kq : (char *)c->K, *hV = c->quantized ? (char *)c->Vq : (char *)c->V;
    int ok;
    if (up) ok = ornith_cuda_h2d((char *)m->K + o, hK + o, n) == ORNITH_OK &&
                 ornith_cuda_h2d((char *)m->V + o, hV + o, n) == ORNITH_OK;
    else    ok = ornith_cuda_d2h(hK + o, (char *)m->K + o, n) == ORNITH_OK &&
                 ornith_cuda_d2h(hV + o, (char *)m->V + o, n) == ORNITH_OK;
    if (ok && c->quantized) {
        size_t so = (size_t)from * c->n_kv_heads, sn = (size_t)(to - from) * c->n_kv_heads * sizeof(float);
        if (up) ok = ornith_cuda_h2d(m->Ks + so, c->Ks + so, sn) == ORNITH_OK &&
                     ornith_cuda_h2d(m->Vs + so, c->Vs + so, sn) == ORNITH_OK;
        else    ok = ornith_cuda_d2h(c->Ks + so, m->Ks + so, sn) == ORNITH_OK &&
                     ornith_cuda_d2h(c->Vs + so, m->Vs + so, sn) == ORNITH_OK;
    }
    return ok;
}

/* ---- KV cache API (reference: src/ornith_attn.c:12-60) -------------------------- */

size_t ornith_kv_bytes_per_token(int n_kv_heads, int head_dim, int quantized) {
    size_t n = (size_t)n_kv_heads * head_dim;
    return quantized ? 2 * (n + (size_t)n_kv_heads * sizeof(float)) : 2 * n * sizeof(float);
}

ornith_status ornith_kv_init_ex(ornith_kv_cache *c, int capacity, int n_kv_heads, int head_dim, int quantized) {
    pthread_mutex_lock(&g_lock);
    kv_mirror *stale = mirror_find(c);
    if (stale) mirror_release(stale);
    pthread_mutex_unlock(&g_lock);
    memset(c, 0, sizeof(*c));
    c->capacity = capacity; c->n_kv_heads = n_kv_heads; c->head_dim = head_dim;
    c->quantized = quantized ? 1 : 0;
    size_t rows = (size_t)capacity * n_kv_heads, elems = rows * head_dim;
    if (c->quantized) {
        c->Kq = calloc(elems, 1); c->Vq = calloc(elems, 1);
        c->Ks = calloc(rows, sizeof(float)); c->Vs = calloc(rows, sizeof(float));
        if (!c->Kq || !c->Vq || !c->Ks || !c->Vs) {
            free(c->Kq); free(c->Vq); free(c->Ks); free(c->Vs);
            memset(c, 0, sizeof(*c));
            ornith_set_error("kv cache (q8) oom (capacity %d)", capacity);
            return ORNITH_ERR_OOM;
        }
        return ORNITH_OK;
    }
    c->K = calloc(elems, sizeof(float)); c->V = calloc(elems, sizeof(float));
    if (!c->K || !c->V) {
        free(c->K); free(c->V);
        memset(c, 0, sizeof(*c));
        ornith_set_error("kv cache oom (capacity %d)", capacity);
        return ORNITH_ERR_OOM;
    }
    return ORNITH_OK;
}

ornith_status ornith_kv_init(ornith_kv_cache *c, int capacity, int n_kv_heads, int head_dim) {
    return ornith_kv_init_ex(c, capacity, n_kv_heads, head_dim, 0);
}

void ornith_kv_free(ornith_kv_cache *c) {
    if (!c) return;
    pthread_mutex_lock(&g_lock);
    kv_mirror *m = mirror_find(c);
    if (m) mirror_release(m);
    pthread_mutex_unlock(&g_lock);
    free(c->K); free(c->V); free(c->Kq); free(c->Vq); free(c->Ks); free(c->Vs);
    memset(c, 0, sizeof(*c));
}

void ornith_kv_reset(ornith_kv_cache *c) { c->len = 0; }

/* reference: src/ornith_attn.c:87-149 */
void ornith_gqa_step(ornith_kv_cache *c, const float *q, const float *k_new, const float *v_new,
                     int n_heads, float *out, float scale) {
    if (c->len >= c->capacity) return;                   /* caller guarantees capacity */
    pthread_mutex_lock(&g_lock);
    kv_mirror *m = mirror_get(c);
    if (!m) goto done;
    if (m->synced_len != c->len) {                       /* host image changed under us */
        if (!mirror_copy(m, c, 0, c->len, 1)) goto done;
        m->synced_len = c->len;
    }
    {
        const int hd = c->head_dim, nkv = c->n_kv_heads;
        const size_t qn = (size_t)n_heads * hd * sizeof(float), kn = (size_t)nkv * hd * sizeof(float);
        ornith_cuda_full_layer L;
        memset(&L, 0, sizeof(L));
        L.n_heads = n_heads; L.n_kv_heads = nkv; L.head_dim = hd; L.scale = scale; L.eps = 1e-6f;
        ornith_cuda_kv kv;
        memset(&kv, 0, sizeof(kv));
        kv.mode = c->quantized ? ORNITH_KV_INT8_HEAD : ORNITH_KV_F32;
        kv.n_kv_heads = nkv; kv.head_dim = hd; kv.n_seq = 1;
        kv.K = m->K; kv.V = m->V; kv.Ks = m->Ks; kv.Vs = m->Vs; kv.seq_off = m->seq_off;
        const size_t sb = ornith_cuda_full_attn_step_scratch(&L, 1, c->len + 1);
        const size_t need = up256(qn) * 2 + up256(kn) * 2 + up256(sb);
        if (!ws_reserve(need)) goto done;
        char *dq = g_ws, *dk = dq + up256(qn), *dv = dk + up256(kn), *dout = dv + up256(kn), *ds = dout + up256(qn);
        int32_t len = c->len;
        if (ornith_cuda_h2d(dq, q, qn) != ORNITH_OK || ornith_cuda_h2d(dk, k_new, kn) != ORNITH_OK ||
            ornith_cuda_h2d(dv, v_new, kn) != ORNITH_OK || ornith_cuda_h2d(m->len, &len, sizeof(len)) != ORNITH_OK)
            goto done;
        if (ornith_cuda_full_attn_step(&L, &kv, m->len, NULL, dq, dk, dv, dout, ORNITH_ACT_F32, c->len + 1,
                                       ds, sb, NULL) != ORNITH_OK)
            goto done;
        if (ornith_cuda_d2h(out, dout, qn) != ORNITH_OK) goto done;
        if (!mirror_copy(m, c, c->len, c->len + 1, 0)) goto done;   /* keep the host image current */
        c->len++;
        m->synced_len = c->len;
    }
done:
    pthread_mutex_unlock(&g_lock);
}

/* reference: src/ornith_attn.c:151-176 */
void ornith_gqa_reference(const float *Q, const float *K, const float *V, int T, int n_heads,
                          int n_kv_heads, int head_dim, float *O, float scale) {
    if (T <= 0) return;
    pthread_mutex_lock(&g_lock);
    const size_t qn = (size_t)T * n_heads * head_dim * sizeof(float);
    const size_t kn = (size_t)T * n_kv_heads * head_dim * sizeof(float);
    ornith_cuda_full_layer L;
    memset(&L, 0, sizeof(L));
    L.n_heads = n_heads; L.n_kv_heads = n_kv_heads; L.head_dim = head_dim; L.scale = scale; L.eps = 1e-6f;
    const size_t sb = ornith_cuda_full_attn_prefill_scratch(&L, 1, T, T);
    const size_t need = up256(qn) * 2 + up256(kn) * 4 + up256(sb) + 512;
    if (!ws_reserve(need)) goto done;
    {
        char *dq = g_ws, *dk = dq + up256(qn), *dv = dk + up256(kn), *dout = dv + up256(kn);
        char *cK = dout + up256(qn), *cV = cK + up256(kn), *ds = cV + up256(kn), *meta = ds + up256(sb);
        int64_t off[2] = {0, T};
        int32_t zero = 0;
        ornith_cuda_kv kv;
        memset(&kv, 0, sizeof(kv));
        kv.mode = ORNITH_KV_F32; kv.n_kv_heads = n_kv_heads; kv.head_dim = head_dim; kv.n_seq = 1;
        kv.K = cK; kv.V = cV; kv.seq_off = (const int64_t *)meta;
        int32_t *dlen = (int32_t *)(meta + 256);
        if (ornith_cuda_h2d(dq, Q, qn) != ORNITH_OK || ornith_cuda_h2d(dk, K, kn) != ORNITH_OK ||
            ornith_cuda_h2d(dv, V, kn) != ORNITH_OK || ornith_cuda_h2d(meta, off, sizeof(off)) != ORNITH_OK ||
            ornith_cuda_h2d(dlen, &zero, sizeof(zero)) != ORNITH_OK)
            goto done;
        if (ornith_cuda_full_attn_prefill(&L, &kv, dlen, NULL, dq, dk, dv, dout, ORNITH_ACT_F32, T, T, ds, sb, NULL)
            != ORNITH_OK)
            goto done;
        if (ornith_cuda_d2h(O, dout, qn) != ORNITH_OK) ornith_set_error("gqa_reference: copy of the output back to the host failed");
    }
done:
    pthread_mutex_unlock(&g_lock);
}

/* ---- delta-net state (reference: src/ornith_attn.c:182-349) ---------------------- */

ornith_status ornith_delta_init(ornith_delta_state *s, int dk, int dv) {
    s->dk = dk; s->dv = dv;
    s->S = calloc((size_t)dk * dv, sizeof(float));
    if (!s->S) { ornith_set_error("delta state oom"); return ORNITH_ERR_OOM; }
    return ORNITH_OK;
}
void ornith_delta_free(ornith_delta_state *s) { if (!s) return; free(s->S); s->S = NULL; }
void ornith_delta_reset(ornith_delta_state *s) { memset(s->S, 0, (size_t)s->dk * s->dv * sizeof(float)); }

void ornith_delta_step(ornith_delta_state *s, const float *q, const float *k, const float *v,
                       float alpha, float beta, float *o) {
    pthread_mutex_lock(&g_lock);
    const int dk = s->dk, dv = s->dv;
    const size_t sn = (size_t)dk * dv * sizeof(float), kn = (size_t)dk * sizeof(float), vn = (size_t)dv * sizeof(float);
    if (!ws_reserve(up256(sn) + 2 * up256(kn) + 2 * up256(vn) + 512)) goto done;
    {
        char *dS = g_ws, *dq = dS + up256(sn), *dkk = dq + up256(kn), *dvv = dkk + up256(kn);
        char *dout = dvv + up256(vn), *dg = dout + up256(vn);
        float gates[2] = {alpha, beta};
        if (ornith_cuda_h2d(dS, s->S, sn) != ORNITH_OK || ornith_cuda_h2d(dq, q, kn) != ORNITH_OK ||
            ornith_cuda_h2d(dkk, k, kn) != ORNITH_OK || ornith_cuda_h2d(dvv, v, vn) != ORNITH_OK ||
            ornith_cuda_h2d(dg, gates, sizeof(gates)) != ORNITH_OK)
            goto done;
        if (ornith_cuda_delta_step((float *)dS, 1, dk, dv, (float *)dq, (float *)dkk, (float *)dvv,
                                   (float *)dg, (float *)dg + 1, (float *)dout, NULL) != ORNITH_OK)
            goto done;
        if (ornith_cuda_d2h(o, dout, vn) != ORNITH_OK) goto done;
        if (ornith_cuda_d2h(s->S, dS, sn) != ORNITH_OK) ornith_set_error("delta: copy of the state back to the host failed");
    }
done:
    pthread_mutex_unlock(&g_lock);
}

void ornith_delta_prefill(ornith_delta_state *s, const float *Q, const float *K, const float *V,
                          const float *alpha, const float *beta, int T, int chunk, float *O) {
    if (T <= 0) return;
    pthread_mutex_lock(&g_lock);
    const int dk = s->dk, dv = s->dv;
    const size_t sn = (size_t)dk * dv * sizeof(float), kn = (size_t)T * dk * sizeof(float);
    const size_t vn = (size_t)T * dv * sizeof(float), gn = (size_t)T * sizeof(float);
    if (!ws_reserve(up256(sn) + 2 * up256(kn) + 2 * up256(vn) + 2 * up256(gn))) goto done;
    {
        char *dS = g_ws, *dq = dS + up256(sn), *dkk = dq + up256(kn), *dvv = dkk + up256(kn);
        char *dout = dvv + up256(vn), *da = dout + up256(vn), *db = da + up256(gn);
        if (ornith_cuda_h2d(dS, s->S, sn) != ORNITH_OK || ornith_cuda_h2d(dq, Q, kn) != ORNITH_OK ||
            ornith_cuda_h2d(dkk, K, kn) != ORNITH_OK || ornith_cuda_h2d(dvv, V, vn) != ORNITH_OK ||
            ornith_cuda_h2d(da, alpha, gn) != ORNITH_OK || ornith_cuda_h2d(db, beta, gn) != ORNITH_OK)
            goto done;
        if (ornith_cuda_delta_prefill((float *)dS, dk, dv, (float *)dq, (float *)dkk, (float *)dvv, (float *)da,
                                      (float *)db, T, chunk, (float *)dout, NULL) != ORNITH_OK)
            goto done;
        if (ornith_cuda_d2h(O, dout, vn) != ORNITH_OK) goto done;
        if (ornith_cuda_d2h(s->S, dS, sn) != ORNITH_OK) ornith_set_error("delta: copy of the state back to the host failed");
    }
done:
    pthread_mutex_unlock(&g_lock);
}

/* ---- causal conv (reference: src/ornith_attn.c:355-397) -------------------------- */

ornith_status ornith_conv_init(ornith_conv_state *cs, int K, int C) {
    cs->K = K; cs->C = C;
    cs->buf = calloc((size_t)(K > 0 ? K - 1 : 0) * C + 1, sizeof(float));
    if (!cs->buf) { ornith_set_error("conv state oom"); return ORNITH_ERR_OOM; }
    return ORNITH_OK;
}
void ornith_conv_free(ornith_conv_state *cs) { if (!cs) return; free(cs->buf); cs->buf = NULL; }
void ornith_conv_reset(ornith_conv_state *cs) {
    memset(cs->buf, 0, (size_t)(cs->K > 0 ? cs->K - 1 : 0) * cs->C * sizeof(float));
}

void ornith_conv_prefill(ornith_conv_state *cs, const float *X, const float *weight, const float *bias,
                         int T, float *OUT) {
    if (T <= 0) return;
    pthread_mutex_lock(&g_lock);
    const int K = cs->K, C = cs->C;
    const size_t in = (size_t)(K > 0 ? K - 1 : 0) * C * sizeof(float), xn = (size_t)T * C * sizeof(float);
    const size_t wn = (size_t)C * K * sizeof(float), bn = (size_t)C * sizeof(float);
    if (!ws_reserve(up256(in) + 2 * up256(xn) + up256(wn) + up256(bn))) goto done;
    {
        char *di = g_ws, *dx = di + up256(in), *dout = dx + up256(xn), *dw = dout + up256(xn), *db = dw + up256(wn);
        if (ornith_cuda_h2d(di, cs->buf, in) != ORNITH_OK || ornith_cuda_h2d(dx, X, xn) != ORNITH_OK ||
            ornith_cuda_h2d(dw, weight, wn) != ORNITH_OK || (bias && ornith_cuda_h2d(db, bias, bn) != ORNITH_OK))
            goto done;
        if (ornith_cuda_conv_image((float *)di, K, C, (float *)dx, (float *)dw, bias ? (float *)db : NULL, T,
                                   (float *)dout, NULL) != ORNITH_OK)
            goto done;
        if (ornith_cuda_d2h(OUT, dout, xn) != ORNITH_OK) goto done;
        if (ornith_cuda_d2h(cs->buf, di, in) != ORNITH_OK) ornith_set_error("conv: copy of the history back to the host failed");
    }
done:
    pthread_mutex_unlock(&g_lock);
}

void ornith_conv_step(ornith_conv_state *cs, const float *x_in, const float *weight, const float *bias,
                      float *out) {
    ornith_conv_prefill(cs, x_in, weight, bias, 1, out);
}
