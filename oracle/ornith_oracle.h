/* ornith_oracle.h — CPU restatement of the ornithology attention hot path.
 *
 * TEST INFRASTRUCTURE ONLY. This library is the checker the CUDA path is
 * compared against (tests/, the smoke check and the cpu_baseline leg of the
 * benchmark). Nothing in the product library links, loads or calls it.
 *
 * Every function restates, in the same arithmetic order (strict sequential f32,
 * f64 only where the reference uses it), one function of the reference engine;
 * the citation next to each declaration is the reference file:line it follows.
 * The restatement is pinned bit-for-bit against the reference's own objects
 * (oracle/_ref, built from the reference sources by oracle/Makefile) and
 * against the known-answer values in the reference's tests
 * (tests/test_tensor.c, tests/test_attn.c, tests/test_quant.c).
 *
 * Build with the reference's flags (-O3 -std=c11: ISO mode keeps FP
 * contraction off, so a*b+c is never fused).
 */
#ifndef ORNITH_ORACLE_H
#define ORNITH_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- seeded RNG: splitmix64, 24-bit uniform (src/ornith_tensor.c:44-62) -- */
typedef struct { uint64_t s; } orc_rng;
void  orc_rng_seed(orc_rng *r, uint64_t seed);
float orc_rng_uniform(orc_rng *r, float lo, float hi);
void  orc_rng_fill(orc_rng *r, float *dst, int64_t n, float lo, float hi);

/* ---- elementwise helpers (src/ornith_tensor.c:100-178) ------------------- */
float orc_dot(const float *a, const float *b, int n);                 /* :143-147 */
void  orc_rmsnorm(const float *x, const float *w, float *out, int n, float eps); /* :100-106 */
void  orc_softmax(float *x, int n);                                   /* :108-115 */
float orc_sigmoid(float x);                                           /* :117 */
float orc_silu(float x);                                              /* :118 */
float orc_softplus(float x);                                          /* :119 */
void  orc_l2norm_eps(const float *x, float *out, int n, float eps);   /* :155-160 */
void  orc_rope_partial(float *v, int head_dim, int rotary_dim, int pos, float theta); /* :167-178 */

/* ---- f16 + Q8_0 codec (src/ornith_quant.c:14-65, :155-184) --------------- */
uint16_t orc_f32_to_f16(float f);
float    orc_f16_to_f32(uint16_t h);
/* n must be a multiple of 32; 34 bytes per block. Returns 0, or -1 on bad n. */
int orc_q8_0_encode(const float *src, uint8_t *dst, size_t n);
int orc_q8_0_decode(const uint8_t *src, float *dst, size_t n);
/* per-vector int8 + f32 scale used by the reference's own quantised KV cache
 * (src/ornith_attn.c:65-77); returns the scale. */
float orc_kv_int8_encode(const float *x, int n, int8_t *q);

/* ---- KV cache + GQA (src/ornith_attn.c:12-176) --------------------------- */
enum { ORC_KV_F32 = 0, ORC_KV_INT8_HEAD = 1, ORC_KV_Q8_0 = 2 };

typedef struct {
    int mode, capacity, len, n_kv_heads, head_dim;
    float   *K, *V;      /* F32: stored rows. Q8_0: decoded rows (what attention reads) */
    int8_t  *Kq, *Vq;    /* INT8_HEAD codes [cap][nkv][hd]                              */
    float   *Ks, *Vs;    /* INT8_HEAD scales [cap][nkv]                                 */
    uint8_t *Kb, *Vb;    /* Q8_0 bytes [cap][nkv][hd/32][34]                            */
} orc_kv;

int    orc_kv_init(orc_kv *c, int capacity, int n_kv_heads, int head_dim, int mode);
void   orc_kv_free(orc_kv *c);
size_t orc_kv_bytes_per_token(int n_kv_heads, int head_dim, int mode);
/* append one token then attend over the whole cache (src/ornith_attn.c:87-149).
 * Q8_0 mode is the composition quantize -> dequantize -> f32 attention. */
void orc_gqa_step(orc_kv *c, const float *q, const float *k_new, const float *v_new,
                  int n_heads, float *out, float scale);
void orc_gqa_reference(const float *Q, const float *K, const float *V, int T,
                       int n_heads, int n_kv_heads, int head_dim, float *O, float scale); /* :151-176 */

/* ---- gated delta rule (src/ornith_attn.c:196-349) ------------------------ */
void orc_delta_step(float *S, int dk, int dv, const float *q, const float *k,
                    const float *v, float alpha, float beta, float *o);         /* :198-213 */
void orc_delta_prefill(float *S, int dk, int dv, const float *Q, const float *K,
                       const float *V, const float *alpha, const float *beta,
                       int T, int chunk, float *O);                             /* :244-349 */

/* ---- causal depthwise conv (src/ornith_attn.c:369-397) ------------------- */
/* buf is the reference history image: [(K-1)][C], oldest row first. */
void orc_conv_step(float *buf, int K, int C, const float *x, const float *w,
                   const float *bias, float *out);
void orc_conv_prefill(float *buf, int K, int C, const float *X, const float *w,
                      const float *bias, int T, float *OUT);

/* ---- layer wiring without the projections -------------------------------- */
enum { ORC_HEADMAP_TILED = 0, ORC_HEADMAP_GROUPED = 1 };

typedef struct {
    int nk, nv, dk, dv, conv_k;     /* key heads, value heads, head dims, conv taps  */
    int head_map;                   /* TILED: kh = hv % nk (src/ornith_rforward.c:491);
                                       GROUPED: kh = hv / (nv/nk) (src/ornith_forward.c:387) */
    float out_scale;                /* 1/sqrt(dk) in the real-weights engine
                                       (src/ornith_rforward.c:305), 1 in the synthetic one  */
    float eps;                      /* rms_norm_eps                                  */
    const float *conv_w;            /* [Cc][conv_k]                                  */
    const float *conv_b;            /* [Cc] or NULL                                  */
    const float *a_coef;            /* [nv] negative decay coefficient               */
    const float *dt_bias;           /* [nv]                                          */
    const float *norm_w;            /* [dv] shared by all heads                      */
} orc_linear_params;

/* One token through a gated delta-net layer between the projections:
 * conv step + SiLU, q/k L2-norm, decay/write gates, recurrent update per value
 * head, output scale, per-head RMSNorm, SiLU(z) gate.
 * Follows src/ornith_rforward.c:466-500 and :305-314.
 * S [nv][dv][dk], conv_buf [(K-1)][Cc], qkv [Cc], a,b [nv], z,out [nv*dv]. */
void orc_linear_attn_step(const orc_linear_params *p, float *S, float *conv_buf,
                          const float *qkv, const float *a, const float *b,
                          const float *z, float *out);
/* T tokens via the chunked scan (src/ornith_rforward.c:571-616, :305-314).
 * QKV [T][Cc], A,B [T][nv], Z,OUT [T][nv*dv]. */
void orc_linear_attn_prefill(const orc_linear_params *p, float *S, float *conv_buf,
                             const float *QKV, const float *A, const float *B,
                             const float *Z, int T, int chunk, float *OUT);

typedef struct {
    int nh, nkv, hd, rope_dim;
    float theta, eps;
    const float *q_norm_w;          /* [hd] */
    const float *k_norm_w;          /* [hd] */
} orc_full_params;

/* One token through a full-attention layer between the projections: q|gate
 * split, q/k RMSNorm, partial RoPE, append + attend, sigmoid output gate
 * (src/ornith_rforward.c:432-450). qproj [nh][2*hd], k,v [nkv*hd], out [nh*hd]. */
void orc_full_attn_step(const orc_full_params *p, orc_kv *c, int pos,
                        const float *qproj, const float *k, const float *v, float *out);
/* T tokens (src/ornith_rforward.c:529-551): the same step once per token. */
void orc_full_attn_prefill(const orc_full_params *p, orc_kv *c, int base, int T,
                           const float *QP, const float *K, const float *V, float *OUT);

/* ---- quantised projections (src/ornith_qdot.c, src/ornith_rforward.c:138-196) ---- */
/* Q8_K activation super-block, 292 bytes (src/ornith_qdot.h:30-34) */
typedef struct {
    float   d;
    int8_t  qs[256];
    int16_t bsums[16];
} orc_q8k_block;
/* k f32 values (multiple of 256) -> k/256 blocks (src/ornith_qdot.c:38-70) */
void orc_q8k_quantize(const float *x, orc_q8k_block *y, int64_t k);
/* one Q8_0 weight row (n/32 blocks of 34 bytes) . one Q8_K activation row (src/ornith_qdot.c:144-163) */
float orc_vec_dot_q8_0(int n, const uint8_t *wrow, const orc_q8k_block *y);
/* Y[t][o] = W[o] . X[t] for T activation rows: every row quantised to Q8_K once, then the integer dot per
 * (row of W, token) (matmul_batch_q, src/ornith_rforward.c:138-192).  W: [out] rows of n_in/32 Q8_0 blocks. */
int orc_matmul_q8_0(const uint8_t *W, int n_in, int n_out, const float *X, int T, float *Y);
/* the other two integer paths: Q4_K rows (144-byte super-blocks, src/ornith_qdot.c:75-105) and Q6_K rows
 * (210-byte super-blocks, :109-141); weight type ids as in the GGUF file (src/ornith_gguf.h:24-30) */
enum { ORC_GGML_Q8_0 = 8, ORC_GGML_Q4_K = 12, ORC_GGML_Q6_K = 14 };
float orc_vec_dot_q4_K(int n, const uint8_t *wrow, const orc_q8k_block *y);
float orc_vec_dot_q6_K(int n, const uint8_t *wrow, const orc_q8k_block *y);
size_t orc_qrow_bytes(int wtype, int n_in);
int orc_matmul_q(int wtype, const uint8_t *W, int n_in, int n_out, const float *X, int T, float *Y);

#ifdef __cplusplus
}
#endif
#endif
