/* ornith_cuda.h — C ABI of the B200 attention backend for ornithology.
 *
 * One shared library (libornith_cuda.so) exports two tiers:
 *
 *  Tier 1 — the drop-in.  The seventeen functions of the engine's attention
 *  header (reference: src/ornith_attn.h:71-147) plus the backend probe
 *  (reference: src/ornith_cuda.cu:12), with the same names, structs, argument
 *  meaning and error behaviour.  Host pointers in and out; every call runs the
 *  CUDA kernels below and keeps the caller-visible struct fields valid host
 *  images, so code that pokes `K`, `len`, `S` or `buf` directly keeps working.
 *  Link this library instead of the engine's ornith_attn.o.
 *
 *  Tier 2 — the device-resident API (ornith_cuda_*).  Layer-level entry points
 *  that take DEVICE pointers and batch descriptors, keep the KV cache, the
 *  recurrent state and the conv history in HBM, and never touch the host on the
 *  data path.  This is what the engine's layer wiring calls under
 *  ORNITH_BACKEND_CUDA (reference call sites: src/ornith_rforward.c:419-618,
 *  src/ornith_forward.c:338-531).
 *
 * There is no CPU fallback: every compute entry point fails with
 * ORNITH_ERR_BACKEND (tier 2) or leaves its outputs untouched and records an
 * error (tier 1, whose compute functions return void like the reference's) when
 * no CUDA device is usable.
 *
 * All pointers are plain C pointers; `stream` is a cudaStream_t passed as void*
 * (NULL = the default stream).  Unless stated otherwise tier-2 calls are
 * asynchronous on `stream`.
 */
#ifndef ORNITH_CUDA_H
#define ORNITH_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes (reference: src/ornith.h:34-41) ------------------------- */
#ifndef ORNITH_H
typedef enum {
    ORNITH_OK = 0,
    ORNITH_ERR_IO,
    ORNITH_ERR_FORMAT,
    ORNITH_ERR_UNSUPPORTED,
    ORNITH_ERR_OOM,
    ORNITH_ERR_NOTFOUND
} ornith_status;
const char *ornith_last_error(void);              /* reference: src/ornith_util.c:21-23 */
void        ornith_set_error(const char *fmt, ...);   /* reference: src/ornith_util.c:25-30 */
#endif
/* one code beyond the reference's enum: a CUDA runtime / launch failure */
#define ORNITH_ERR_BACKEND 6

/* 1 when a CUDA device of compute capability 10.x is usable, else 0.
 * Replaces the stub at src/ornith_cuda.cu:12-15 (which always returns 0). */
int ornith_backend_cuda_available(void);

/* ======================================================================== */
/* Tier 1 — drop-in for src/ornith_attn.h                                    */
/* ======================================================================== */
#ifndef ORNITH_ATTN_H

/* reference: src/ornith_attn.h:57-69 (field order and types are ABI)
 * The device copy of a cache is refreshed when `len` or the address of the host
 * buffers differs from what the last call left.  A host that rewrites cached rows in
 * place WITHOUT changing `len` must call ornith_kv_reset (and set `len` again) or
 * ornith_kv_init_ex before the next ornith_gqa_step; the engine's own session load
 * re-initialises the cache first (src/ornith_rforward.c:1129), so it needs nothing. */
typedef struct {
    float  *K, *V;
    int8_t *Kq, *Vq;
    float  *Ks, *Vs;
    int     quantized;
    int     capacity;
    int     len;
    int     n_kv_heads;
    int     head_dim;
} ornith_kv_cache;

/* reference: src/ornith_attn.h:104-107 */
typedef struct { float *S; int dk, dv; } ornith_delta_state;

/* reference: src/ornith_attn.h:129-132 */
typedef struct { float *buf; int K, C; } ornith_conv_state;

/* reference: src/ornith_attn.h:72-82, src/ornith_attn.c:12-60 */
ornith_status ornith_kv_init(ornith_kv_cache *c, int capacity, int n_kv_heads, int head_dim);
ornith_status ornith_kv_init_ex(ornith_kv_cache *c, int capacity, int n_kv_heads, int head_dim,
                                int quantized);
size_t        ornith_kv_bytes_per_token(int n_kv_heads, int head_dim, int quantized);
void          ornith_kv_free(ornith_kv_cache *c);
void          ornith_kv_reset(ornith_kv_cache *c);

/* reference: src/ornith_attn.h:89-91, src/ornith_attn.c:87-149.
 * Appends k_new/v_new at position c->len, then attends over the whole cache.
 * A full cache is a silent no-op, as in the reference. */
void ornith_gqa_step(ornith_kv_cache *c, const float *q, const float *k_new, const float *v_new,
                     int n_heads, float *out, float scale);
/* reference: src/ornith_attn.h:97-99, src/ornith_attn.c:151-176 */
void ornith_gqa_reference(const float *Q, const float *K, const float *V, int T, int n_heads,
                          int n_kv_heads, int head_dim, float *O, float scale);

/* reference: src/ornith_attn.h:109-123, src/ornith_attn.c:182-349 */
ornith_status ornith_delta_init(ornith_delta_state *s, int dk, int dv);
void          ornith_delta_free(ornith_delta_state *s);
void          ornith_delta_reset(ornith_delta_state *s);
void ornith_delta_step(ornith_delta_state *s, const float *q, const float *k, const float *v,
                       float alpha, float beta, float *o);
void ornith_delta_prefill(ornith_delta_state *s, const float *Q, const float *K, const float *V,
                          const float *alpha, const float *beta, int T, int chunk, float *O);

/* reference: src/ornith_attn.h:134-147, src/ornith_attn.c:355-397 */
ornith_status ornith_conv_init(ornith_conv_state *cs, int K, int C);
void          ornith_conv_free(ornith_conv_state *cs);
void          ornith_conv_reset(ornith_conv_state *cs);
void ornith_conv_step(ornith_conv_state *cs, const float *x_in, const float *weight,
                      const float *bias, float *out);
void ornith_conv_prefill(ornith_conv_state *cs, const float *X, const float *weight,
                         const float *bias, int T, float *OUT);
#endif /* ORNITH_ATTN_H */

/* ======================================================================== */
/* Tier 2 — device-resident API                                              */
/* ======================================================================== */

/* activation I/O format of the layer entry points (state and accumulation are
 * always f32) */
enum { ORNITH_ACT_F32 = 0, ORNITH_ACT_BF16 = 1 };

/* KV row formats.
 *  F32        rows of head_dim f32 (reference: src/ornith_attn.h:59)
 *  INT8_HEAD  int8 codes + one f32 scale per (position, head), the engine's own
 *             quantised cache (reference: src/ornith_attn.h:46-52, src/ornith_attn.c:65-77)
 *  Q8_0       ggml Q8_0 blocks, 34 bytes per 32 values, byte-identical to the
 *             engine's codec (reference: src/ornith_quant.c:155-175) */
enum { ORNITH_KV_F32 = 0, ORNITH_KV_INT8_HEAD = 1, ORNITH_KV_Q8_0 = 2 };

/* key-head -> value-head pairing of the delta-net layers
 *  TILED   kh = hv % nk        (reference: src/ornith_rforward.c:491)
 *  GROUPED kh = hv / (nv/nk)   (reference: src/ornith_forward.c:387) */
enum { ORNITH_HEADMAP_TILED = 0, ORNITH_HEADMAP_GROUPED = 1 };

/* ---- runtime helpers (synchronous; for hosts that do not link cudart) ------ */
const char   *ornith_cuda_last_error(void);
ornith_status ornith_cuda_set_device(int device);
ornith_status ornith_cuda_malloc(void **dev_ptr, size_t bytes);      /* zero-filled */
ornith_status ornith_cuda_free(void *dev_ptr);
ornith_status ornith_cuda_memset(void *dev_ptr, int value, size_t bytes);
ornith_status ornith_cuda_h2d(void *dev_dst, const void *host_src, size_t bytes);
ornith_status ornith_cuda_d2h(void *host_dst, const void *dev_src, size_t bytes);
/* Waits for `stream`; returns ORNITH_ERR_BACKEND (with a message) when a kernel of this library
 * gave up a bounded wait since the last check — its outputs are then NaN-poisoned, not valid. */
ornith_status ornith_cuda_sync(void *stream);
/* The same check without waiting: reads and clears the current device's status word. */
ornith_status ornith_cuda_poll_status(void);
/* Every wait inside the kernels (on an mbarrier, for a copy or a tensor-core result) is bounded.
 * This runs a one-thread kernel that waits `polls` polls on a barrier nobody arrives on, and checks
 * that the wait comes back and is reported: the expected return value is ORNITH_ERR_BACKEND with
 * the status word set; ORNITH_ERR_FORMAT means the give-up path did not work.  Nothing faults. */
ornith_status ornith_cuda_selftest_wait_timeout(int polls);
/* Allocation hook (host-side failure injection; reference: the OOM checks of the init functions,
 * src/ornith_attn.c:32-46): when set, every device allocation the library makes — ornith_cuda_malloc,
 * the tier-1 mirrors, the delta-net decode work buffer — first calls hook(bytes, user); a non-zero
 * return makes that allocation fail with ORNITH_ERR_OOM without touching the device.  NULL clears it. */
typedef int (*ornith_cuda_alloc_hook)(size_t bytes, void *user);
void ornith_cuda_set_alloc_hook(ornith_cuda_alloc_hook hook, void *user);
/* Frees the work buffer the delta-net decode step keeps for `stream` on the current device (for every
 * stream of the device when all_streams != 0, and then also the second stream and the events the
 * delta-net prefill keeps per device), after waiting for the work queued there.  Call it
 * before destroying a stream that ran ornith_cuda_linear_attn_step. */
ornith_status ornith_cuda_stream_release(void *stream, int all_streams);
/* inverse RoPE frequencies theta^(-2i/rotary_dim), i < rotary_dim/2, computed on
 * the host with the engine's own expression (reference: src/ornith_tensor.c:171);
 * upload them once and pass the device copy as `rope_inv_freq`. */
void ornith_cuda_rope_inv_freq(float theta, int rotary_dim, float *host_out);

/* ---- codec entry points (reference: src/ornith_quant.c:155-184, src/ornith_attn.c:65-77) */
/* n f32 values (multiple of 32) -> n/32 blocks of 34 bytes, and back. */
ornith_status ornith_cuda_q8_0_encode(const float *dev_src, void *dev_dst, size_t n, void *stream);
ornith_status ornith_cuda_q8_0_decode(const void *dev_src, float *dev_dst, size_t n, void *stream);

/* ---- full (GQA) attention layers ------------------------------------------ */

/* One layer's KV cache for a batch of sequences.  Sequence b owns positions
 * [seq_off[b], seq_off[b+1]) of the pools; its capacity is the difference.
 *   F32        K,V: float   [positions][n_kv_heads][head_dim]
 *   INT8_HEAD  K,V: int8    [positions][n_kv_heads][head_dim]; Ks,Vs: float [positions][n_kv_heads]
 *   Q8_0       K,V: uint8   [positions][n_kv_heads][head_dim/32][34]
 * Within a sequence these are exactly the engine's cache images
 * (reference: src/ornith_attn.h:57-69), so a session dump is a plain copy. */
typedef struct {
    int32_t mode, n_kv_heads, head_dim, n_seq;
    void   *K, *V;                 /* device */
    float  *Ks, *Vs;               /* device, INT8_HEAD only */
    const int64_t *seq_off;        /* device [n_seq + 1] */
} ornith_cuda_kv;

/* reference: src/ornith_rforward.c:419-455 (weights and shape of one full layer) */
typedef struct {
    int32_t n_heads, n_kv_heads, head_dim, rope_dim;
    int32_t gated;                 /* 1: q projection packs [q | gate] per head (:432-435) */
    float   eps, scale;            /* scale <= 0: 1/sqrt(head_dim) (src/ornith_attn.c:91) */
    const float *q_norm_w;         /* device [head_dim], NULL: q,k arrive normalised + rotated */
    const float *k_norm_w;         /* device [head_dim] */
    const float *rope_inv_freq;    /* device [rope_dim/2], NULL with rope_dim == 0 */
} ornith_cuda_full_layer;

/* scratch bytes ornith_cuda_full_attn_step asks for with n_seq sequences whose
 * longest context (after the append) is max_len: room for the split length that fills
 * the GPU at this batch (short splits for few sequences), for any cache mode and head
 * size (the query does not see the cache, so it also covers the CUDA-core kernel's
 * 512-token splits).  The step adapts to what it is given: with less it uses longer
 * splits; when one of the tensor-core kernels serves the cache (head_dim 256, groups
 * of up to 16 heads) the least it accepts is the need of the coarse split length
 * (2048 tokens above a 16k context, 1024 above 8k, 512 above 1k, else 256), otherwise
 * that of 512-token splits; below that it fails with ORNITH_ERR_FORMAT. */
size_t ornith_cuda_full_attn_step_scratch(const ornith_cuda_full_layer *layer, int n_seq, int max_len);

/* One decode step of a full-attention layer for n_seq sequences, between the
 * projections: split q|gate, q/k RMSNorm, partial RoPE, append to the cache at
 * kv_len[b], attend over [0, kv_len[b]], sigmoid output gate.
 * Replaces the body of full_attn() (reference: src/ornith_rforward.c:432-450).
 *   qproj [n_seq][n_heads*(gated?2:1)*head_dim], k,v [n_seq][n_kv_heads*head_dim],
 *   out [n_seq][n_heads*head_dim]                       (act_dtype)
 *   kv_len  device int32 [n_seq]: positions already in the cache (not modified)
 *   rope_pos device int32 [n_seq] or NULL (= kv_len)
 *   max_len: host upper bound on kv_len[b] + 1
 * A sequence whose cache is full is skipped, as the reference does. */
ornith_status ornith_cuda_full_attn_step(const ornith_cuda_full_layer *layer, const ornith_cuda_kv *kv,
                                         const int32_t *kv_len, const int32_t *rope_pos,
                                         const void *qproj, const void *k, const void *v, void *out,
                                         int act_dtype, int max_len,
                                         void *scratch, size_t scratch_bytes, void *stream);

size_t ornith_cuda_full_attn_prefill_scratch(const ornith_cuda_full_layer *layer, int n_seq, int T, int max_len);

/* Causal prefill of T tokens per sequence, appended at kv_len[b].. and attending
 * over everything already cached plus the new tokens; quantised modes attend
 * over the decoded rows, current token included, like T decode steps do.
 * Replaces the body of full_attn_prefill() (reference: src/ornith_rforward.c:529-551).
 *   qproj [n_seq][T][...], k,v [n_seq][T][...], out [n_seq][T][n_heads*head_dim]
 *   max_len: host upper bound on kv_len[b] + T (sizes the decoded-row image in the scratch)
 * head_dim 256 runs on the tcgen05 tensor cores (f16 operands, f32 accumulation);
 * ORNITH_CUDA_PREFILL_VARIANT=mma in the environment selects the mma.sync kernel instead. */
ornith_status ornith_cuda_full_attn_prefill(const ornith_cuda_full_layer *layer, const ornith_cuda_kv *kv,
                                            const int32_t *kv_len, const int32_t *rope_pos,
                                            const void *qproj, const void *k, const void *v, void *out,
                                            int act_dtype, int T, int max_len,
                                            void *scratch, size_t scratch_bytes, void *stream);

/* The append half alone: k RMSNorm + RoPE, then f32 copy / Q8_0 / int8 encode of k
 * and v into positions kv_len[b] .. kv_len[b]+T-1 (reference: the append part of
 * ornith_gqa_step, src/ornith_attn.c:94-110, after src/ornith_rforward.c:443-447).
 *   k,v [n_seq][T][n_kv_heads*head_dim] */
ornith_status ornith_cuda_kv_append(const ornith_cuda_full_layer *layer, const ornith_cuda_kv *kv,
                                    const int32_t *kv_len, const int32_t *rope_pos,
                                    const void *k, const void *v, int act_dtype, int T, void *stream);

/* The same decode step for hosts that are not allowed to allocate device memory.
 * (No counterpart in the reference: its attention code is CPU-only and mallocs its
 * score buffer per call, src/ornith_attn.c:114.)
 *
 * Who needs it: an engine that split its device memory among its subsystems once at
 * start-up and has no allocator left to ask on the token path; a serving loop that
 * cannot afford cudaMalloc's device-wide synchronisation (or its failure) between
 * two tokens; an embedding host that gives this library no allocator at all.  The
 * caller still passes every input and the output; only the scratch (prepared query
 * rows + split-K partials) comes from a fixed array inside the library image, which
 * every GPU that loads the library keeps resident until the process exits.
 *
 *  - Limit: the scratch of the step at its coarsest split length must not exceed
 *    ORNITH_CUDA_STATIC_SCRATCH_BYTES (8 MiB; e.g. 8 sequences x 16 heads x 256 at an
 *    8k context); within the array the step uses the shortest splits that fit.
 *    Larger requests return ORNITH_ERR_UNSUPPORTED with a message.
 *  - The first call on each device looks up the array's device address (with that
 *    device current); make that call before starting any stream capture.
 *  - Calls never call cudaMalloc/cudaFree or any allocating library routine.
 *  - All calls share the array and it keeps the previous call's contents; a step
 *    rewrites every word before reading it, so nothing needs clearing, but two calls
 *    whose kernels overlap on the GPU race — keep them on one stream. */
#define ORNITH_CUDA_STATIC_SCRATCH_BYTES (8u << 20)
ornith_status ornith_cuda_full_attn_step_static(const ornith_cuda_full_layer *layer, const ornith_cuda_kv *kv,
                                                const int32_t *kv_len, const int32_t *rope_pos,
                                                const void *qproj, const void *k, const void *v, void *out,
                                                int act_dtype, int max_len, void *stream);

/* kv_len[b] += delta for every sequence (call once per token after all layers). */
ornith_status ornith_cuda_advance(int32_t *counters, int n, int delta, void *stream);

/* ---- gated delta-net (linear attention) layers ------------------------------ */

/* reference: src/ornith_rforward.c:457-503, :300-314 (weights and shape of one layer) */
typedef struct {
    int32_t nk, nv, dk, dv, conv_k, head_map;
    float   out_scale;             /* 1/sqrt(dk) in the real-weights engine (:305) */
    float   eps;
    const float *conv_w;           /* device [Cc][conv_k], Cc = 2*nk*dk + nv*dv */
    const float *conv_b;           /* device [Cc] or NULL */
    const float *a_coef;           /* device [nv]: decay = exp(a_coef*softplus(a+dt_bias)) (:282-284) */
    const float *dt_bias;          /* device [nv] */
    const float *norm_w;           /* device [dv] */
} ornith_cuda_linear_layer;

/* One layer's recurrent state for a batch of sequences.
 *   S     f32 [nv][dv][dk] per sequence (reference image: src/ornith_rforward.c:261)
 *   conv  f32 [conv_k][Cc] per sequence: a ring, token t lives in slot t % conv_k.
 *         Use ornith_cuda_conv_import/export for the engine's oldest-first
 *         [(conv_k-1)][Cc] image (reference: src/ornith_attn.h:129-132). */
typedef struct {
    float  *S;
    float  *conv;
    int64_t S_seq_stride;          /* elements between consecutive sequences */
    int64_t conv_seq_stride;
} ornith_cuda_linear_state;

/* One decode step of a delta-net layer for n_seq sequences, between the
 * projections: conv + SiLU, q/k L2-norm, decay and write gates, recurrent
 * update, output scale, per-head RMSNorm, SiLU(z) gate.
 * Replaces the bodies of linear_attn() and linear_finish() minus their matvecs
 * (reference: src/ornith_rforward.c:466-500, :305-314).
 *   qkv [n_seq][Cc], a,b [n_seq][nv], z,out [n_seq][nv*dv]   (act_dtype)
 *   pos device int32 [n_seq]: index of the token being processed (conv ring phase) */
ornith_status ornith_cuda_linear_attn_step(const ornith_cuda_linear_layer *layer,
                                           const ornith_cuda_linear_state *st, const int32_t *pos,
                                           const void *qkv, const void *a, const void *b,
                                           const void *z, void *out, int act_dtype, int n_seq,
                                           void *stream);

size_t ornith_cuda_linear_attn_prefill_scratch(const ornith_cuda_linear_layer *layer, int n_seq, int T);

/* T tokens per sequence through the chunked scan; state and conv history end
 * exactly where T decode steps would leave them.
 * Replaces linear_attn_prefill() minus its matvecs (reference: src/ornith_rforward.c:571-616).
 *   qkv [n_seq][T][Cc], a,b [n_seq][T][nv], z,out [n_seq][T][nv*dv]
 *   scratch: 256-byte aligned.  With dk = dv = 128 the scan runs in 64-token chunks on the
 *   tcgen05 tensor cores (tf32 products, f32 accumulation; the state of a head stays in tensor
 *   memory for the whole prompt) whatever `chunk` says.  When the batch has too few
 *   (sequence, value head) units to fill the GPU the prompt is cut into runs of chunks that are
 *   scanned side by side and stitched by their transition matrices; ORNITH_CUDA_DELTA_SEGMENTS=n
 *   forces n runs (1 = off).  Long prompts with one wave of heads or less are cut into slabs:
 *   conv and chunk preparation of the next slab run on `stream` while the current slab is
 *   scanned on an internal second stream of the device; `stream` waits for the last scan before
 *   the call returns, so the caller sees ordinary stream order (and may capture the call into a
 *   graph).  Results do not depend on the slab count (ORNITH_CUDA_DELTA_SLABS=n, 1 = off).
 *   ORNITH_CUDA_DELTA_SCAN=mma selects the older mma.sync scan
 *   (32-token chunks); ORNITH_CUDA_PREFILL_FP32=1 keeps every product in fp32 on the CUDA cores
 *   (chunk >= 32 / < 32 selects 32 / 16 tokens). */
ornith_status ornith_cuda_linear_attn_prefill(const ornith_cuda_linear_layer *layer,
                                              const ornith_cuda_linear_state *st, const int32_t *pos,
                                              const void *qkv, const void *a, const void *b,
                                              const void *z, void *out, int act_dtype,
                                              int n_seq, int T, int chunk,
                                              void *scratch, size_t scratch_bytes, void *stream);

/* conv ring <-> the engine's history image [(conv_k-1)][Cc], oldest first
 * (reference: src/ornith_attn.c:369, session dump src/ornith_rforward.c:1056-1063).
 * `pos` is the index of the next token of that sequence. */
ornith_status ornith_cuda_conv_export(const float *dev_ring, int conv_k, int Cc, int pos,
                                      float *dev_image, void *stream);
ornith_status ornith_cuda_conv_import(float *dev_ring, int conv_k, int Cc, int pos,
                                      const float *dev_image, void *stream);

/* ---- multi-GPU plan (one process per GPU, or one process driving several devices) ---------------------- */

/* What rank `rank` of `world` owns under head sharding (reference: heads never interact — loop bodies
 * src/ornith_rforward.c:488-498, :594-611; KV head of a query head src/ornith_attn.c:113-116):
 * nv/world value heads of every delta-net layer with the key heads they pair with (tiled map kh = hv % nk),
 * nh/world query heads of every full layer with the KV heads they read (replicated once world > n_kv_heads).
 * A shard is just a smaller layer: slice the weights and the projection outputs to these heads and call the
 * layer entry points above with the shard's head counts.  Pure host arithmetic. */
typedef struct {
    int32_t rank, world;
    int32_t v_head0, n_v_heads;     /* value heads [v_head0, v_head0 + n_v_heads) */
    int32_t k_head0, n_k_heads;     /* key heads */
    int32_t q_head0, n_q_heads;     /* query heads */
    int32_t kv_head0, n_kv_heads;   /* KV heads */
} ornith_cuda_shard;
ornith_status ornith_cuda_head_shard(int nk, int nv, int nh, int nkv, int rank, int world, ornith_cuda_shard *out);

/* After an all-gather of per-rank head outputs (NCCL or any other transport; it delivers rank blocks one after
 * the other, gathered [world][rows][width]), lay them out as the full-width rows the output projection consumes,
 * full [rows][world * width] (reference call sites of that projection: src/ornith_rforward.c:452, :316).
 * elem_bytes: 2 (bf16) or 4 (f32); width * elem_bytes must be a multiple of 16. */
ornith_status ornith_cuda_gather_layout(const void *gathered, void *full, int world, size_t rows, int width,
                                        int elem_bytes, void *stream);

/* ---- session records of device-resident state ------------------------------
 * The engine's session file is a header, one record per layer, the token history and the
 * last logits (writer: src/ornith_rforward.c:1020-1076, reader: :1078-1171).  These entry
 * points produce and consume the per-layer records in HOST memory, from and into the device
 * pools; the engine keeps writing its header, history and logits itself, and its layer loop
 * becomes one fwrite / fread of a record per layer.  They are synchronous.
 *
 *   full-attention layer: int32 q, len, n_kv_heads, head_dim, then (:1042-1052)
 *     q = 0  K, V f32 [len][n_kv_heads][head_dim]
 *     q = 1  Kq, Vq int8 [len][n_kv_heads][head_dim], Ks, Vs f32 [len][n_kv_heads]
 *     q = 2  K, V ggml Q8_0 rows [len][n_kv_heads][head_dim/32][34] — an extension for
 *            ORNITH_KV_Q8_0 pools; the engine has no such mode and rejects the record by q
 *   delta-net layer: S f32 [nv][dv][dk], int32 conv_k, Cc, history f32 [(conv_k-1)][Cc],
 *     oldest token first (:1054-1063)
 * Records with q = 0 / 1 and the delta-net records are byte for byte the engine's, so a
 * snapshot taken on the device loads into the CPU engine and the other way round. */
size_t ornith_cuda_kv_record_bytes(const ornith_cuda_kv *kv, int len);
/* the first `len` positions of sequence `seq` */
ornith_status ornith_cuda_kv_export(const ornith_cuda_kv *kv, int seq, int len, void *host_dst,
                                    size_t dst_bytes, void *stream);
/* checks q, n_kv_heads, head_dim and the capacity; *len_out (may be NULL) = positions loaded;
 * dev_kv_len (may be NULL): the batch's device length array, entry `seq` is set too */
ornith_status ornith_cuda_kv_import(const ornith_cuda_kv *kv, int seq, const void *host_src,
                                    size_t src_bytes, int32_t *len_out, int32_t *dev_kv_len,
                                    void *stream);
size_t ornith_cuda_linear_record_bytes(const ornith_cuda_linear_layer *layer);
/* pos = tokens the sequence has seen so far (it fixes where the conv ring starts) */
ornith_status ornith_cuda_linear_export(const ornith_cuda_linear_layer *layer,
                                        const ornith_cuda_linear_state *st, int seq, int pos,
                                        void *host_dst, size_t dst_bytes, void *stream);
ornith_status ornith_cuda_linear_import(const ornith_cuda_linear_layer *layer,
                                        const ornith_cuda_linear_state *st, int seq, int pos,
                                        const void *host_src, size_t src_bytes, void *stream);

/* ---- quantised projections around the attention core ---------------------------
 * Q8_0 weights x Q8_K activations, the engine's integer path for attn_qkv, ssm_alpha/beta,
 * attn_gate, ssm_out, attn_q/k/v/output (matmul_batch_q, reference: src/ornith_rforward.c:138-192;
 * qdot_quantize_row_q8_K src/ornith_qdot.c:38-70; vec_dot_q8_0 :144-163).  This first pair is the
 * f16-product form for Q8_0 (decode-sized batches: more than 64 tokens are walked 64 at a time,
 * re-reading the weights); the bit-exact integer path for Q8_0, Q4_K and Q6_K follows below. */
size_t ornith_cuda_qproj_scratch(int T, int n_in);       /* n_in: a multiple of 256 */
/* x [T][n_in] -> Q8_K.  The codes and scales are the engine's bit for bit.  blocks: device
 * [T][n_in/256][292 bytes] in the engine's block layout (f32 d, 256 int8, 16 int16 sums), or NULL;
 * scratch: ornith_cuda_qproj_scratch bytes, 256-byte aligned (the form the product reads). */
ornith_status ornith_cuda_q8k_quantize(const void *x, int act_dtype, int T, int n_in, void *blocks,
                                       void *scratch, size_t scratch_bytes, void *stream);
/* y [T][n_out] = x [T][n_in] through W = device Q8_0 rows [n_out][n_in/32][34] (the GGUF tensor bytes,
 * 16-byte aligned).  Quantises x into scratch, then the product on the tensor cores: integer codes of
 * both operands exact, a weight (code x f16 block scale) rounded once to f16, f32 sums, the activation's
 * scale applied per block of 256 in f32.  out_dtype: ORNITH_ACT_F32 or ORNITH_ACT_BF16. */
ornith_status ornith_cuda_matmul_q8_0(const void *W, int n_in, int n_out, const void *x, int act_dtype,
                                      int T, void *y, int out_dtype, void *scratch, size_t scratch_bytes,
                                      void *stream);

/* The engine's integer path for any weight type that has one (qdot_can, reference: src/ornith_qdot.c:167-177):
 * Q8_0 (vec_dot_q8_0 :144-163), Q4_K (vec_dot_q4_K :75-105), Q6_K (vec_dot_q6_K :109-141), against Q8_K
 * activations, bit for bit: int8 tensor-core products with int32 sums, integer sub-block scales, and the
 * engine's f32 association per super-block.  W: the GGUF tensor bytes on the device, [n_out] rows of
 * n_in/256 super-blocks (144 / 210 / 272 bytes); wtype: the GGUF type id.  Rows that start on 16-byte
 * boundaries (always for Q4_K and Q8_0; Q6_K when n_in is a multiple of 2048) and a 16-byte-aligned W take the
 * tensor-core kernel, any other shape a plain kernel with the same result.  scratch: 256-byte aligned,
 * ornith_cuda_matmul_q_scratch bytes.  Any T: a prompt is walked in passes of 128 tokens inside one launch. */
enum { ORNITH_GGML_Q8_0 = 8, ORNITH_GGML_Q4_K = 12, ORNITH_GGML_Q6_K = 14 };   /* src/ornith_gguf.h:24-30 */
size_t ornith_cuda_matmul_q_scratch(int wtype, int T, int n_in);
ornith_status ornith_cuda_matmul_q(int wtype, const void *W, int n_in, int n_out, const void *x,
                                   int act_dtype, int T, void *y, int out_dtype, void *scratch,
                                   size_t scratch_bytes, void *stream);
/* The two halves of ornith_cuda_matmul_q, for projections that share an input (attn_qkv, attn_gate,
 * ssm_alpha and ssm_beta all read the layer's normalised hidden state; the engine quantises it once,
 * reference: src/ornith_rforward.c:165-170): quantise x [T][n_in] into an image of
 * ornith_cuda_matmul_q_scratch bytes once, then any number of products against it.  The product starts
 * its weight copies before the kernel launched in front of it on the stream has finished (it waits
 * for that kernel only before it reads the image), so that kernel must not be one that writes W. */
ornith_status ornith_cuda_q8k_image(const void *x, int act_dtype, int T, int n_in, void *image,
                                    size_t image_bytes, void *stream);
ornith_status ornith_cuda_matmul_q_image(int wtype, const void *W, int n_in, int n_out,
                                         const void *image, int T, void *y, int out_dtype, void *stream);
/* Several projections of the same input in one launch (one per run of matrices of the same weight type):
 * for a decode-sized batch the launches cost as much as the weight traffic, and a small matrix (ssm_alpha,
 * ssm_beta: 32 rows) cannot fill the GPU alone.  y [T][n_out] per projection; results as the single call's. */
typedef struct {
    int         wtype;      /* ORNITH_GGML_Q8_0 / _Q4_K / _Q6_K */
    const void *W;          /* device, [n_out] rows of n_in/256 super-blocks */
    int         n_out;
    void       *y;          /* device, [T][n_out] */
} ornith_cuda_qproj;
ornith_status ornith_cuda_matmul_q_group(const ornith_cuda_qproj *projs, int n, int n_in,
                                         const void *image, int T, int out_dtype, void *stream);

/* ---- host-fed layer calls over device-resident state -------------------------
 * For an engine whose projections still run on the host: one object holds the state of all
 * layers of one sequence on the device (what rstate holds on the host, reference:
 * src/ornith_rforward.c:212-264), and the four wiring functions (full_attn :419-455,
 * linear_attn :457-503, full_attn_prefill :513-556, linear_attn_prefill :563-618) hand over
 * their projection outputs (host f32) and get the attention output back (host f32).  T == 1
 * runs the decode kernels, T > 1 the prefill kernels.  Synchronous.  Conventions of the
 * real-weights engine (tiled head map, no conv bias, 1/sqrt(dk) output scale, gated q).
 * kv_mode: ORNITH_KV_F32 / ORNITH_KV_INT8_HEAD (the engine's ORNITH_KV_Q8=1) / ORNITH_KV_Q8_0. */
typedef struct ornith_cuda_engine ornith_cuda_engine;
ornith_cuda_engine *ornith_cuda_engine_new(int num_layers, int capacity, int kv_mode, int n_heads,
                                           int n_kv_heads, int head_dim, int rope_dim, float rope_theta,
                                           float rms_eps, int nk, int nv, int dk, int dv, int conv_k);
void ornith_cuda_engine_free(ornith_cuda_engine *e);
/* weights the attention math needs, host pointers; uploaded on the first call for a layer
 * (which also creates that layer's zeroed state), ignored afterwards */
ornith_status ornith_cuda_engine_full_layer(ornith_cuda_engine *e, int layer, const float *q_norm_w,
                                            const float *k_norm_w);
ornith_status ornith_cuda_engine_linear_layer(ornith_cuda_engine *e, int layer, const float *conv_w,
                                              const float *a_coef, const float *dt_bias,
                                              const float *norm_w);
/* qproj [T][n_heads][2*head_dim], k, v [T][n_kv_heads*head_dim], out [T][n_heads*head_dim];
 * pos = rows already in the cache = position of the first token */
ornith_status ornith_cuda_engine_full_attn(ornith_cuda_engine *e, int layer, int pos, int T,
                                           const float *qproj, const float *k, const float *v, float *out);
/* qkv [T][Cc] (before the conv), a, b [T][nv], z [T][nv*dv] (gate projection, before SiLU),
 * out [T][nv*dv] (scaled, normalised, gated: what ssm_out multiplies) */
ornith_status ornith_cuda_engine_linear_attn(ornith_cuda_engine *e, int layer, int pos, int T,
                                             const float *qkv, const float *a, const float *b,
                                             const float *z, float *out);
/* the layer's session record after `pos` tokens (layouts: the session-record entry points above);
 * import needs the layer's weights call first and, for a full layer, a record of `pos` positions */
size_t ornith_cuda_engine_record_bytes(const ornith_cuda_engine *e, int layer, int pos);
ornith_status ornith_cuda_engine_export(const ornith_cuda_engine *e, int layer, int pos, void *host_dst,
                                        size_t dst_bytes);
ornith_status ornith_cuda_engine_import(ornith_cuda_engine *e, int layer, int pos, const void *host_src,
                                        size_t src_bytes);

/* ---- per-head primitives on device pointers (what tier 1 is built from) ---- */

/* reference: src/ornith_attn.c:198-213; n_heads independent states S [h][dv][dk],
 * q,k [h][dk], v,o [h][dv], alpha,beta [h] (device) */
ornith_status ornith_cuda_delta_step(float *S, int n_heads, int dk, int dv, const float *q,
                                     const float *k, const float *v, const float *alpha,
                                     const float *beta, float *o, void *stream);
/* reference: src/ornith_attn.c:337-349; one head, T tokens, any dk,dv; the chunk
 * size only selects the tiling, the result is that of T steps */
ornith_status ornith_cuda_delta_prefill(float *S, int dk, int dv, const float *Q, const float *K,
                                        const float *V, const float *alpha, const float *beta,
                                        int T, int chunk, float *O, void *stream);
/* reference: src/ornith_attn.c:370-397; image = [(K-1)][C] oldest first, X,OUT [T][C] */
ornith_status ornith_cuda_conv_image(float *image, int K, int C, const float *X, const float *w,
                                     const float *bias, int T, float *OUT, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* ORNITH_CUDA_H */
