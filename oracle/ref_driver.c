/* ref_driver.c — drives the REFERENCE's own attention functions through one
 * decode token of a layer, for the CPU-baseline leg of the benchmark and for
 * cross-checking the restatement.
 *
 * TEST INFRASTRUCTURE ONLY.  This file contains no attention arithmetic of its
 * own: every operation is a call into the reference objects it is linked with
 * (ornith_attn.c, ornith_tensor.c, ornith_quant.c — compiled from the reference
 * checkout by oracle/Makefile into _ref/libornith_ref.so).  The call sequence
 * follows the reference's layer wiring with the projections left out:
 *   linear layer  src/ornith_rforward.c:466-500 and :305-314
 *   full layer    src/ornith_rforward.c:432-450
 * The reference has no Q8_0 KV cache; the Q8_0 run is the composition
 * oq_quantize -> oq_dequantize on the appended rows + the f32 cache.
 */
#include <stdlib.h>
#include <string.h>
#include <math.h>

#include "ornith_attn.h"
#include "ornith_tensor.h"
#include "ornith_quant.h"

typedef struct {
    int nk, nv, dk, dv, conv_k;
    float eps;
    const float *conv_w, *a_coef, *dt_bias, *norm_w;
} refdrv_linear;

/* one token of a gated delta-net layer, real-weights conventions
 * (kh = hv % nk, no conv bias, 1/sqrt(dk) output scale) */
void refdrv_linear_step(const refdrv_linear *p, float *S, float *conv_buf, const float *qkv,
                        const float *a, const float *b, const float *z, float *out) {
    int nk = p->nk, nv = p->nv, dk = p->dk, dv = p->dv, qd = nk * dk, vd = nv * dv, Cc = 2 * qd + vd;
    float *conv = malloc((size_t)Cc * sizeof(float));
    float *qn = malloc((size_t)qd * sizeof(float)), *kn = malloc((size_t)qd * sizeof(float));
    float *o_all = malloc((size_t)vd * sizeof(float)), *gate = malloc((size_t)vd * sizeof(float));
    ornith_conv_state cs = { conv_buf, p->conv_k, Cc };
    ornith_conv_step(&cs, qkv, p->conv_w, NULL, conv);
    ot_silu_(conv, Cc);
    for (int h = 0; h < nk; h++) {
        ot_l2norm_eps(conv + (size_t)h * dk, qn + (size_t)h * dk, dk, 1e-6f);
        ot_l2norm_eps(conv + qd + (size_t)h * dk, kn + (size_t)h * dk, dk, 1e-6f);
    }
    for (int hv = 0; hv < nv; hv++) {
        int kh = hv % nk;
        float alpha = expf(p->a_coef[hv] * ot_softplus(a[hv] + p->dt_bias[hv]));
        ornith_delta_state st = { S + (size_t)hv * dv * dk, dk, dv };
        ornith_delta_step(&st, qn + (size_t)kh * dk, kn + (size_t)kh * dk, conv + 2 * qd + (size_t)hv * dv,
                          alpha, ot_sigmoid(b[hv]), o_all + (size_t)hv * dv);
    }
    ot_scale_(o_all, 1.0f / sqrtf((float)dk), vd);
    memcpy(gate, z, (size_t)vd * sizeof(float));
    ot_silu_(gate, vd);
    for (int hv = 0; hv < nv; hv++)
        ot_rmsnorm(o_all + (size_t)hv * dv, p->norm_w, out + (size_t)hv * dv, dv, p->eps);
    ot_mul_(out, gate, vd);
    free(conv); free(qn); free(kn); free(o_all); free(gate);
}

typedef struct {
    int nh, nkv, hd, rope_dim;
    float theta, eps;
    const float *q_norm_w, *k_norm_w;
    int q8_0;                /* 1: appended K/V rows pass through the Q8_0 codec first */
} refdrv_full;

/* one token of a full-attention layer over the reference's f32 cache */
void refdrv_full_step(const refdrv_full *p, ornith_kv_cache *c, int pos, const float *qproj,
                      const float *k, const float *v, float *out) {
    int nh = p->nh, nkv = p->nkv, hd = p->hd, qd = nh * hd, kvd = nkv * hd;
    float *q = malloc((size_t)qd * sizeof(float)), *g = malloc((size_t)qd * sizeof(float));
    float *kk = malloc((size_t)kvd * sizeof(float)), *vv = malloc((size_t)kvd * sizeof(float));
    for (int h = 0; h < nh; h++) {
        memcpy(q + (size_t)h * hd, qproj + (size_t)h * 2 * hd, (size_t)hd * sizeof(float));
        memcpy(g + (size_t)h * hd, qproj + (size_t)h * 2 * hd + hd, (size_t)hd * sizeof(float));
    }
    memcpy(kk, k, (size_t)kvd * sizeof(float));
    memcpy(vv, v, (size_t)kvd * sizeof(float));
    for (int h = 0; h < nh; h++) {
        ot_rmsnorm(q + (size_t)h * hd, p->q_norm_w, q + (size_t)h * hd, hd, p->eps);
        ot_rope_partial(q + (size_t)h * hd, hd, p->rope_dim, pos, p->theta);
    }
    for (int h = 0; h < nkv; h++) {
        ot_rmsnorm(kk + (size_t)h * hd, p->k_norm_w, kk + (size_t)h * hd, hd, p->eps);
        ot_rope_partial(kk + (size_t)h * hd, hd, p->rope_dim, pos, p->theta);
    }
    if (p->q8_0) {
        size_t nb = oq_row_bytes(OGGML_Q8_0, (size_t)kvd);
        unsigned char *tmp = malloc(nb);
        oq_quantize(OGGML_Q8_0, kk, tmp, (size_t)kvd); oq_dequantize(OGGML_Q8_0, tmp, kk, (size_t)kvd);
        oq_quantize(OGGML_Q8_0, vv, tmp, (size_t)kvd); oq_dequantize(OGGML_Q8_0, tmp, vv, (size_t)kvd);
        free(tmp);
    }
    ornith_gqa_step(c, q, kk, vv, nh, out, 0.0f);
    for (int i = 0; i < qd; i++) out[i] *= ot_sigmoid(g[i]);
    free(q); free(g); free(kk); free(vv);
}

/* ---- quantised projections: the reference's own quantiser and integer dot (src/ornith_qdot.c), driven the way
 *      matmul_batch_q drives them (src/ornith_rforward.c:165-175, :108-115) ---- */
#include "ornith_qdot.h"
#include "ornith_quant.h"

void refdrv_q8k_quantize(const float *x, void *y, long long k) { qdot_quantize_row_q8_K(x, (oq8k_block *)y, k); }

/* any weight type the reference has an integer dot for; rows quantised by the reference's own encoder */
int refdrv_matmul_q(unsigned wtype, const unsigned char *W, int n_in, int n_out, const float *X, int T, float *Y) {
    if (!qdot_can(wtype, n_in)) return -1;
    const size_t nblk = (size_t)n_in / OQDOT_QK_K, rb = oq_row_bytes(wtype, (size_t)n_in);
    oq8k_block *xq = malloc((size_t)T * nblk * sizeof *xq);
    if (!xq) return -1;
    for (int t = 0; t < T; t++) qdot_quantize_row_q8_K(X + (size_t)t * n_in, xq + (size_t)t * nblk, n_in);
    for (int o = 0; o < n_out; o++)
        for (int t = 0; t < T; t++)
            qdot_vec_dot(wtype, n_in, &Y[(size_t)t * n_out + o], W + (size_t)o * rb, xq + (size_t)t * nblk);
    free(xq);
    return 0;
}
/* f32 rows -> quantised rows of `wtype` with the reference's encoder (src/ornith_quant.c oq_quantize) */
long long refdrv_quantize_rows(unsigned wtype, const float *src, void *dst, long long n_elems) {
    if (oq_quantize(wtype, src, dst, (size_t)n_elems) != 0) return -1;
    return (long long)oq_row_bytes(wtype, (size_t)n_elems);
}

int refdrv_matmul_q8_0(const unsigned char *W, int n_in, int n_out, const float *X, int T, float *Y) {
    if (!qdot_can(OGGML_Q8_0, n_in)) return -1;
    const size_t nblk = (size_t)n_in / OQDOT_QK_K, rb = oq_row_bytes(OGGML_Q8_0, (size_t)n_in);
    oq8k_block *xq = malloc((size_t)T * nblk * sizeof *xq);
    if (!xq) return -1;
    for (int t = 0; t < T; t++) qdot_quantize_row_q8_K(X + (size_t)t * n_in, xq + (size_t)t * nblk, n_in);
    for (int o = 0; o < n_out; o++)
        for (int t = 0; t < T; t++)
            qdot_vec_dot(OGGML_Q8_0, n_in, &Y[(size_t)t * n_out + o], W + (size_t)o * rb, xq + (size_t)t * nblk);
    free(xq);
    return 0;
}
