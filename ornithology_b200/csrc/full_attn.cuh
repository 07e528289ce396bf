// full_attn.cuh — argument block shared by the split-K decode kernels.
#pragma once
#include "common.cuh"
#include "kv_rows.cuh"

struct DecodeArgs {
    KvView kv;
    const int32_t *kv_len;
    const float *q_prep;                 // [n_seq][nh][hd] f32, normalised + rotated
    float *part;                         // [n_seq][nh][nsplit][hd + 2]: m, l, o[hd]
    int nh, nsplit, tokens_per_split;
    float scale;
    // Fused merge (kernels that support it; group_ctr == nullptr leaves the merge to k_gqa_combine): the last CTA
    // of a (sequence, head group) to finish merges the group's partials, applies the output gate and stores.
    int *group_ctr;                      // [n_seq][grid.x] arrival counters, zero when the kernel starts
    const void *qproj;                   // gate = second half of each head's projection row (gated != 0)
    void *out;
    int gated, act_dtype;
    int n_seq, max_len;                  // batch size and the call's bound on any context after the append
    int piece_cost;                      // balanced schedule: tiles charged per sequence for the fixed work of a piece
    unsigned int *status;                // device status word (a bounded wait that gave up sets ORN_WAIT_DECODE), or NULL
};

// Tensor-core split-K decode over Q8_0 rows, head_dim 256, up to 16 query heads
// per KV head.  Writes the same partials as the generic kernel.
bool gqa_decode_q8_mma_supported(const KvView &kv, int nh);
// *merged is set when the launched kernel did the merge itself (a.group_ctr given and supported).
ornith_status launch_gqa_decode_q8_mma(const DecodeArgs &a, int n_seq, cudaStream_t st, bool *merged);

// Variant for groups of up to 8 query heads that builds its MMA fragments straight
// from the staged raw rows (gqa_decode_q8_raw.cu).
ornith_status launch_gqa_decode_q8_raw(const DecodeArgs &a, int n_seq, cudaStream_t st, bool *merged);
// Whether a step over this cache is served by that kernel with its balanced schedule (token ranges of equal
// length found on the device instead of a grid of fixed splits), and then how many partial slots per head its
// scratch needs: a.nsplit = gqa_decode_q8_raw_slots(...) and a.part laid out [head][slot][hd + 2].
bool gqa_decode_q8_raw_balanced(const KvView &kv, int nh);
int gqa_decode_q8_raw_slots(int nkv, int nh, int n_seq, int max_len);

// The same for int8-per-head rows (gqa_decode_i8_raw.cu), up to 8 query heads per KV head.
bool gqa_decode_i8_raw_supported(const KvView &kv, int nh);
ornith_status launch_gqa_decode_i8_raw(const DecodeArgs &a, int n_seq, cudaStream_t st);

// Tensor-core (tf32) split-K decode over f32 rows, head_dim 256, up to 8 query heads per KV head
// (gqa_decode_f32.cu).  Same partials.
bool gqa_decode_f32_tc_supported(const KvView &kv, int nh);
ornith_status launch_gqa_decode_f32_tc(const DecodeArgs &a, int n_seq, cudaStream_t st);

// Tensor-core causal prefill for head_dim 256 (gqa_prefill_mma.cu): decodes the visible cache
// rows into an f16 image in `kvh_scratch` (gqa_prefill_mma_scratch bytes), then attends with
// the tcgen05 kernel (gqa_prefill_tc.cu) or, on request, the mma.sync one.
bool gqa_prefill_mma_supported(const KvView &kv);
size_t gqa_prefill_mma_scratch(int n_seq, int nkv, int nh, int T, int Lmax);
ornith_status launch_gqa_prefill_mma(const KvView &kv, const int32_t *kv_len, const float *q_prep, void *kvh_scratch,
                                     const void *qproj, void *out, int nh, int T, int Lmax, int gated, float scale,
                                     int n_seq, bool bf16_act, cudaStream_t st);

// tcgen05 / TMEM / TMA causal prefill (gqa_prefill_tc.cu).  Kh / Vh: decoded f16 rows
// [n_seq][nkv][Lp][256], zero past the rows the prefill sees, Lp a multiple of 64;
// q_scratch: gqa_prefill_tc_scratch bytes for the f16 query image and its row factors.
size_t gqa_prefill_tc_scratch(int n_seq, int nh, int T);
// Where the f16 query image and its per-row factors live inside `kvh_scratch`, if the tcgen05 kernel is
// going to run: the front end may then write them itself and pass q_prep = nullptr to the launchers below.
bool gqa_prefill_tc_selected();
bool gqa_prefill_q_image(void *kvh_scratch, int n_seq, int nkv, int nh, int T, int Lmax, __half **Qh, float **rs);
ornith_status launch_gqa_prefill_tc(const KvView &kv, const int32_t *kv_len, const float *q_prep, const __half *Kh,
                                    const __half *Vh, void *q_scratch, const void *qproj, void *out, int nh, int T,
                                    int Lmax, int Lp, int gated, float scale, int n_seq, bool bf16_act, cudaStream_t st);
