// session_image.cu — per-layer session records of device-resident state.
//
// The engine's session file is a header, one record per layer, the token history and the last
// logits (reference: src/ornith_rforward.c:1020-1076 writes it, :1078-1171 reads it).  The per-layer
// records are what lives on the device here, so these entry points produce and consume exactly
// those records in host memory; the engine keeps writing its header, history and logits itself.
//
//   full-attention layer:  int32 q, len, n_kv_heads, head_dim, then
//        q = 0   K, V as f32   [len][n_kv_heads][head_dim]
//        q = 1   Kq, Vq as int8 [len][n_kv_heads][head_dim], then Ks, Vs as f32 [len][n_kv_heads]
//        q = 2   K, V as ggml Q8_0 rows [len][n_kv_heads][head_dim/32][34]   (an extension: the engine has no
//                such cache mode; a reader that does not know it rejects the record by its q)
//   delta-net layer:       S as f32 [nv][dv][dk], int32 conv_k, Cc, then the conv history as f32
//                          [(conv_k-1)][Cc], oldest token first.
//
// Records with q = 0 or 1 and the delta-net records are byte for byte what rmodel_session_save writes,
// so a snapshot taken on the device loads into the CPU engine and the other way round.
//
// These calls are synchronous (they are not on the token path): they return after the copies.
#include <cstring>
#include <vector>

#include "common.cuh"

namespace {

struct KvGeom {
    size_t row_bytes;            // one (position, kv head) row of K or V
    int64_t first;               // first position of the sequence in the pools
    int64_t capacity;
};

ornith_status kv_geom(const ornith_cuda_kv *kv, int seq, KvGeom *g) {
    if (!kv || seq < 0 || seq >= kv->n_seq || kv->n_kv_heads <= 0 || kv->head_dim <= 0) {
        orn_record_error("kv record: bad cache descriptor or sequence index");
        return ORNITH_ERR_FORMAT;
    }
    if (kv->mode == ORNITH_KV_Q8_0 && kv->head_dim % 32 != 0) {
        orn_record_error("kv record: Q8_0 rows need head_dim to be a multiple of 32");
        return ORNITH_ERR_FORMAT;
    }
    g->row_bytes = kv->mode == ORNITH_KV_F32 ? (size_t)kv->head_dim * 4
                   : kv->mode == ORNITH_KV_Q8_0 ? (size_t)(kv->head_dim / 32) * 34 : (size_t)kv->head_dim;
    int64_t off[2];
    ORN_TRY(orn_check(cudaMemcpy(off, kv->seq_off + seq, sizeof off, cudaMemcpyDeviceToHost), "kv record: read seq_off"));
    g->first = off[0];
    g->capacity = off[1] - off[0];
    return ORNITH_OK;
}

int record_q(int mode) { return mode == ORNITH_KV_F32 ? 0 : mode == ORNITH_KV_INT8_HEAD ? 1 : 2; }

}  // namespace

extern "C" {

size_t ornith_cuda_kv_record_bytes(const ornith_cuda_kv *kv, int len) {
    if (!kv || len < 0) return 0;
    const size_t rows = (size_t)len * kv->n_kv_heads;
    const size_t row = kv->mode == ORNITH_KV_F32 ? (size_t)kv->head_dim * 4
                       : kv->mode == ORNITH_KV_Q8_0 ? (size_t)(kv->head_dim / 32) * 34 : (size_t)kv->head_dim;
    return 16 + 2 * rows * row + (kv->mode == ORNITH_KV_INT8_HEAD ? 2 * rows * sizeof(float) : 0);
}

ornith_status ornith_cuda_kv_export(const ornith_cuda_kv *kv, int seq, int len, void *host_dst, size_t dst_bytes,
                                    void *stream) {
    ORN_TRY(orn_require_device());
    KvGeom g;
    ORN_TRY(kv_geom(kv, seq, &g));
    if (len < 0 || len > g.capacity) { orn_record_error("kv_export: %d positions, the sequence holds at most %lld", len, (long long)g.capacity); return ORNITH_ERR_FORMAT; }
    const size_t need = ornith_cuda_kv_record_bytes(kv, len);
    if (!host_dst || dst_bytes < need) { orn_record_error("kv_export: the record needs %zu bytes, %zu given", need, dst_bytes); return ORNITH_ERR_FORMAT; }
    ORN_TRY(orn_check(cudaStreamSynchronize((cudaStream_t)stream), "kv_export: sync"));   // the steps that filled the cache
    unsigned char *dst = (unsigned char *)host_dst;
    const int32_t head[4] = {record_q(kv->mode), len, kv->n_kv_heads, kv->head_dim};
    memcpy(dst, head, 16);
    dst += 16;
    const size_t rows = (size_t)len * kv->n_kv_heads, bytes = rows * g.row_bytes;
    const size_t pool_off = (size_t)g.first * kv->n_kv_heads * g.row_bytes, scale_off = (size_t)g.first * kv->n_kv_heads;
    ORN_TRY(orn_check(cudaMemcpy(dst, (const unsigned char *)kv->K + pool_off, bytes, cudaMemcpyDeviceToHost), "kv_export: K"));
    ORN_TRY(orn_check(cudaMemcpy(dst + bytes, (const unsigned char *)kv->V + pool_off, bytes, cudaMemcpyDeviceToHost), "kv_export: V"));
    if (kv->mode == ORNITH_KV_INT8_HEAD) {
        dst += 2 * bytes;
        ORN_TRY(orn_check(cudaMemcpy(dst, kv->Ks + scale_off, rows * sizeof(float), cudaMemcpyDeviceToHost), "kv_export: Ks"));
        ORN_TRY(orn_check(cudaMemcpy(dst + rows * sizeof(float), kv->Vs + scale_off, rows * sizeof(float), cudaMemcpyDeviceToHost), "kv_export: Vs"));
    }
    return ORNITH_OK;
}

ornith_status ornith_cuda_kv_import(const ornith_cuda_kv *kv, int seq, const void *host_src, size_t src_bytes,
                                    int32_t *len_out, int32_t *dev_kv_len, void *stream) {
    ORN_TRY(orn_require_device());
    KvGeom g;
    ORN_TRY(kv_geom(kv, seq, &g));
    if (!host_src || src_bytes < 16) { orn_record_error("kv_import: truncated record"); return ORNITH_ERR_FORMAT; }
    int32_t head[4];
    memcpy(head, host_src, 16);
    const int len = head[1];
    if (head[0] != record_q(kv->mode) || head[2] != kv->n_kv_heads || head[3] != kv->head_dim) {
        orn_record_error("kv_import: the record (q %d, %d kv heads x %d) does not match the cache (q %d, %d x %d)", head[0], head[2],
                         head[3], record_q(kv->mode), kv->n_kv_heads, kv->head_dim);
        return ORNITH_ERR_FORMAT;
    }
    if (len < 0 || len > g.capacity) { orn_record_error("kv_import: %d positions do not fit a capacity of %lld", len, (long long)g.capacity); return ORNITH_ERR_FORMAT; }
    if (src_bytes < ornith_cuda_kv_record_bytes(kv, len)) { orn_record_error("kv_import: truncated record"); return ORNITH_ERR_FORMAT; }
    ORN_TRY(orn_check(cudaStreamSynchronize((cudaStream_t)stream), "kv_import: sync"));
    const unsigned char *src = (const unsigned char *)host_src + 16;
    const size_t rows = (size_t)len * kv->n_kv_heads, bytes = rows * g.row_bytes;
    const size_t pool_off = (size_t)g.first * kv->n_kv_heads * g.row_bytes, scale_off = (size_t)g.first * kv->n_kv_heads;
    ORN_TRY(orn_check(cudaMemcpy((unsigned char *)kv->K + pool_off, src, bytes, cudaMemcpyHostToDevice), "kv_import: K"));
    ORN_TRY(orn_check(cudaMemcpy((unsigned char *)kv->V + pool_off, src + bytes, bytes, cudaMemcpyHostToDevice), "kv_import: V"));
    if (kv->mode == ORNITH_KV_INT8_HEAD) {
        src += 2 * bytes;
        ORN_TRY(orn_check(cudaMemcpy(kv->Ks + scale_off, src, rows * sizeof(float), cudaMemcpyHostToDevice), "kv_import: Ks"));
        ORN_TRY(orn_check(cudaMemcpy(kv->Vs + scale_off, src + rows * sizeof(float), rows * sizeof(float), cudaMemcpyHostToDevice), "kv_import: Vs"));
    }
    if (dev_kv_len) {
        const int32_t l = len;
        ORN_TRY(orn_check(cudaMemcpy(dev_kv_len + seq, &l, sizeof l, cudaMemcpyHostToDevice), "kv_import: kv_len"));
    }
    if (len_out) *len_out = len;
    return ORNITH_OK;
}

size_t ornith_cuda_linear_record_bytes(const ornith_cuda_linear_layer *l) {
    if (!l) return 0;
    const size_t Cc = (size_t)2 * l->nk * l->dk + (size_t)l->nv * l->dv;
    return ((size_t)l->nv * l->dv * l->dk + (size_t)(l->conv_k > 0 ? l->conv_k - 1 : 0) * Cc) * sizeof(float) + 8;
}

// pos = number of tokens the sequence has seen (the index of its next token): it fixes where the ring starts.
ornith_status ornith_cuda_linear_export(const ornith_cuda_linear_layer *l, const ornith_cuda_linear_state *st, int seq,
                                        int pos, void *host_dst, size_t dst_bytes, void *stream) {
    ORN_TRY(orn_require_device());
    if (!l || !st || seq < 0 || pos < 0 || l->conv_k < 1) { orn_record_error("linear_export: bad arguments"); return ORNITH_ERR_FORMAT; }
    const size_t need = ornith_cuda_linear_record_bytes(l);
    if (!host_dst || dst_bytes < need) { orn_record_error("linear_export: the record needs %zu bytes, %zu given", need, dst_bytes); return ORNITH_ERR_FORMAT; }
    const size_t ns = (size_t)l->nv * l->dv * l->dk;
    const int Cc = 2 * l->nk * l->dk + l->nv * l->dv;
    const size_t ni = (size_t)(l->conv_k - 1) * Cc;
    unsigned char *dst = (unsigned char *)host_dst;
    ORN_TRY(orn_check(cudaStreamSynchronize((cudaStream_t)stream), "linear_export: sync"));
    ORN_TRY(orn_check(cudaMemcpy(dst, st->S + (size_t)seq * st->S_seq_stride, ns * sizeof(float), cudaMemcpyDeviceToHost), "linear_export: S"));
    dst += ns * sizeof(float);
    const int32_t kc[2] = {l->conv_k, Cc};
    memcpy(dst, kc, 8);
    dst += 8;
    if (ni) {
        void *image = nullptr;
        ORN_TRY(orn_device_alloc(&image, ni * sizeof(float), "conv history image"));
        ornith_status s = ornith_cuda_conv_export(st->conv + (size_t)seq * st->conv_seq_stride, l->conv_k, Cc, pos, (float *)image, stream);
        if (s == ORNITH_OK) s = orn_check(cudaStreamSynchronize((cudaStream_t)stream), "linear_export: sync");
        if (s == ORNITH_OK) s = orn_check(cudaMemcpy(dst, image, ni * sizeof(float), cudaMemcpyDeviceToHost), "linear_export: conv");
        cudaFree(image);
        ORN_TRY(s);
    }
    return ORNITH_OK;
}

ornith_status ornith_cuda_linear_import(const ornith_cuda_linear_layer *l, const ornith_cuda_linear_state *st, int seq,
                                        int pos, const void *host_src, size_t src_bytes, void *stream) {
    ORN_TRY(orn_require_device());
    if (!l || !st || seq < 0 || pos < 0 || l->conv_k < 1) { orn_record_error("linear_import: bad arguments"); return ORNITH_ERR_FORMAT; }
    if (!host_src || src_bytes < ornith_cuda_linear_record_bytes(l)) { orn_record_error("linear_import: truncated record"); return ORNITH_ERR_FORMAT; }
    const size_t ns = (size_t)l->nv * l->dv * l->dk;
    const int Cc = 2 * l->nk * l->dk + l->nv * l->dv;
    const size_t ni = (size_t)(l->conv_k - 1) * Cc;
    const unsigned char *src = (const unsigned char *)host_src;
    int32_t kc[2];
    memcpy(kc, src + ns * sizeof(float), 8);
    if (kc[0] != l->conv_k || kc[1] != Cc) {
        orn_record_error("linear_import: the record's conv history is %d x %d, the layer's %d x %d", kc[0], kc[1], l->conv_k, Cc);
        return ORNITH_ERR_FORMAT;
    }
    ORN_TRY(orn_check(cudaStreamSynchronize((cudaStream_t)stream), "linear_import: sync"));
    ORN_TRY(orn_check(cudaMemcpy(st->S + (size_t)seq * st->S_seq_stride, src, ns * sizeof(float), cudaMemcpyHostToDevice), "linear_import: S"));
    if (ni) {
        void *image = nullptr;
        ORN_TRY(orn_device_alloc(&image, ni * sizeof(float), "conv history image"));
        ornith_status s = orn_check(cudaMemcpy(image, src + ns * sizeof(float) + 8, ni * sizeof(float), cudaMemcpyHostToDevice), "linear_import: conv");
        if (s == ORNITH_OK) s = ornith_cuda_conv_import(st->conv + (size_t)seq * st->conv_seq_stride, l->conv_k, Cc, pos, (const float *)image, stream);
        if (s == ORNITH_OK) s = orn_check(cudaStreamSynchronize((cudaStream_t)stream), "linear_import: sync");
        cudaFree(image);
        ORN_TRY(s);
    }
    return ORNITH_OK;
}

}  // extern "C"
