// engine_session.cu — host-fed layer calls over device-resident state.
//
// The engine's four wiring functions (reference: src/ornith_rforward.c:419-455 full_attn, :457-503 linear_attn,
// :513-556 full_attn_prefill, :563-618 linear_attn_prefill) run their projections on the host and keep one
// sequence's state per session (rstate, :212-218).  This tier is what they call when the state lives on the
// device: the engine hands over the projection outputs of one layer (host pointers), gets the attention output
// back (host pointer), and never sees the KV cache, the recurrent state or the conv history, which stay in HBM
// between calls.  One object holds all layers of one sequence, like rstate.  Weights that the attention math
// itself needs (norm weights, conv taps, gate parameters) are passed with every call and uploaded the first
// time a layer is seen.
//
// The calls are synchronous: activations go up, kernels run, the result comes down.  An engine whose
// projections run on the GPU as well calls the device-pointer entry points directly instead.
#include <vector>

#include "common.cuh"

struct ornith_cuda_engine {
    int num_layers, capacity, kv_mode;
    int nh, nkv, hd, rope_dim;
    float rope_theta, eps;
    int nk, nv, dk, dv, conv_k;
    struct Layer {
        int kind = 0;                        // 0: not seen yet, 1: full attention, 2: delta-net
        ornith_cuda_full_layer full{};
        ornith_cuda_kv kv{};
        ornith_cuda_linear_layer lin{};
        ornith_cuda_linear_state st{};
        std::vector<void *> owned;           // device allocations of this layer
    };
    std::vector<Layer> layers;
    int32_t *d_pos = nullptr;                // one device int: position / cache length of the call
    int64_t *d_seq_off = nullptr;            // {0, capacity}
    void *scratch = nullptr, *act = nullptr;
    size_t scratch_bytes = 0, act_bytes = 0;
};

namespace {

ornith_status dev_alloc(ornith_cuda_engine::Layer &l, void **p, size_t bytes, bool zero) {
    ORN_TRY(ornith_cuda_malloc(p, bytes ? bytes : 16));
    l.owned.push_back(*p);
    if (zero) ORN_TRY(orn_check(cudaMemset(*p, 0, bytes ? bytes : 16), "engine: clear state"));
    return ORNITH_OK;
}
ornith_status upload(ornith_cuda_engine::Layer &l, const float **dst, const float *host, size_t n) {
    if (!host) { *dst = nullptr; return ORNITH_OK; }
    void *p = nullptr;
    ORN_TRY(dev_alloc(l, &p, n * sizeof(float), false));
    ORN_TRY(ornith_cuda_h2d(p, host, n * sizeof(float)));
    *dst = (const float *)p;
    return ORNITH_OK;
}
ornith_status grow(void **buf, size_t *have, size_t need) {
    if (need <= *have) return ORNITH_OK;
    if (*buf) ornith_cuda_free(*buf);
    *buf = nullptr; *have = 0;
    ORN_TRY(ornith_cuda_malloc(buf, need));
    *have = need;
    return ORNITH_OK;
}
ornith_status layer_at(ornith_cuda_engine *e, int L, int kind, ornith_cuda_engine::Layer **out) {
    if (!e || L < 0 || L >= e->num_layers) { orn_record_error("engine: layer %d out of range", L); return ORNITH_ERR_FORMAT; }
    ornith_cuda_engine::Layer &l = e->layers[L];
    if (l.kind != kind) {
        orn_record_error(l.kind ? "engine: layer %d was set up as the other kind of layer" : "engine: layer %d has no weights yet", L);
        return ORNITH_ERR_FORMAT;
    }
    *out = &l;
    return ORNITH_OK;
}
ornith_status set_pos(ornith_cuda_engine *e, int pos) {
    const int32_t p = pos;
    return ornith_cuda_h2d(e->d_pos, &p, sizeof p);
}

}  // namespace

extern "C" {

ornith_cuda_engine *ornith_cuda_engine_new(int num_layers, int capacity, int kv_mode, int n_heads, int n_kv_heads,
                                           int head_dim, int rope_dim, float rope_theta, float rms_eps, int nk, int nv,
                                           int dk, int dv, int conv_k) {
    if (orn_require_device() != ORNITH_OK) return nullptr;
    if (num_layers <= 0 || capacity <= 0) { orn_record_error("engine_new: bad geometry"); return nullptr; }
    ornith_cuda_engine *e = new ornith_cuda_engine();
    e->num_layers = num_layers; e->capacity = capacity; e->kv_mode = kv_mode;
    e->nh = n_heads; e->nkv = n_kv_heads; e->hd = head_dim; e->rope_dim = rope_dim; e->rope_theta = rope_theta; e->eps = rms_eps;
    e->nk = nk; e->nv = nv; e->dk = dk; e->dv = dv; e->conv_k = conv_k;
    e->layers.resize(num_layers);
    const int64_t off[2] = {0, capacity};
    if (ornith_cuda_malloc((void **)&e->d_pos, 16) != ORNITH_OK || ornith_cuda_malloc((void **)&e->d_seq_off, sizeof off) != ORNITH_OK ||
        ornith_cuda_h2d(e->d_seq_off, off, sizeof off) != ORNITH_OK) {
        ornith_cuda_engine_free(e);
        return nullptr;
    }
    return e;
}

void ornith_cuda_engine_free(ornith_cuda_engine *e) {
    if (!e) return;
    for (auto &l : e->layers)
        for (void *p : l.owned) ornith_cuda_free(p);
    if (e->d_pos) ornith_cuda_free(e->d_pos);
    if (e->d_seq_off) ornith_cuda_free(e->d_seq_off);
    if (e->scratch) ornith_cuda_free(e->scratch);
    if (e->act) ornith_cuda_free(e->act);
    delete e;
}

// First call for layer L: cache pools and the device copies of the two norm weights.  Later calls: nothing.
ornith_status ornith_cuda_engine_full_layer(ornith_cuda_engine *e, int L, const float *q_norm_w, const float *k_norm_w) {
    if (!e || L < 0 || L >= e->num_layers) { orn_record_error("engine: layer %d out of range", L); return ORNITH_ERR_FORMAT; }
    ornith_cuda_engine::Layer &l = e->layers[L];
    if (l.kind == 1) return ORNITH_OK;
    if (l.kind) { orn_record_error("engine: layer %d is a delta-net layer", L); return ORNITH_ERR_FORMAT; }
    l.full.n_heads = e->nh; l.full.n_kv_heads = e->nkv; l.full.head_dim = e->hd; l.full.rope_dim = e->rope_dim;
    l.full.gated = 1; l.full.eps = e->eps; l.full.scale = 0.0f;
    ORN_TRY(upload(l, &l.full.q_norm_w, q_norm_w, e->hd));
    ORN_TRY(upload(l, &l.full.k_norm_w, k_norm_w, e->hd));
    if (e->rope_dim > 0) {
        std::vector<float> f(e->rope_dim / 2);
        ornith_cuda_rope_inv_freq(e->rope_theta, e->rope_dim, f.data());
        ORN_TRY(upload(l, &l.full.rope_inv_freq, f.data(), f.size()));
    }
    const size_t rows = (size_t)e->capacity * e->nkv;
    const size_t row = e->kv_mode == ORNITH_KV_F32 ? (size_t)e->hd * 4 : e->kv_mode == ORNITH_KV_Q8_0 ? (size_t)(e->hd / 32) * 34 : (size_t)e->hd;
    l.kv.mode = e->kv_mode; l.kv.n_kv_heads = e->nkv; l.kv.head_dim = e->hd; l.kv.n_seq = 1; l.kv.seq_off = e->d_seq_off;
    ORN_TRY(dev_alloc(l, &l.kv.K, rows * row, true));
    ORN_TRY(dev_alloc(l, &l.kv.V, rows * row, true));
    if (e->kv_mode == ORNITH_KV_INT8_HEAD) {
        ORN_TRY(dev_alloc(l, (void **)&l.kv.Ks, rows * sizeof(float), true));
        ORN_TRY(dev_alloc(l, (void **)&l.kv.Vs, rows * sizeof(float), true));
    }
    l.kind = 1;
    return ORNITH_OK;
}

// First call for layer L: zeroed state and conv history, device copies of the taps and gate parameters
// (conventions of the real-weights engine: tiled head map, no conv bias, 1/sqrt(dk) output scale).
ornith_status ornith_cuda_engine_linear_layer(ornith_cuda_engine *e, int L, const float *conv_w, const float *a_coef,
                                              const float *dt_bias, const float *norm_w) {
    if (!e || L < 0 || L >= e->num_layers) { orn_record_error("engine: layer %d out of range", L); return ORNITH_ERR_FORMAT; }
    ornith_cuda_engine::Layer &l = e->layers[L];
    if (l.kind == 2) return ORNITH_OK;
    if (l.kind) { orn_record_error("engine: layer %d is a full-attention layer", L); return ORNITH_ERR_FORMAT; }
    const size_t Cc = (size_t)2 * e->nk * e->dk + (size_t)e->nv * e->dv;
    l.lin.nk = e->nk; l.lin.nv = e->nv; l.lin.dk = e->dk; l.lin.dv = e->dv; l.lin.conv_k = e->conv_k;
    l.lin.head_map = ORNITH_HEADMAP_TILED; l.lin.out_scale = 1.0f / sqrtf((float)e->dk); l.lin.eps = e->eps;
    ORN_TRY(upload(l, &l.lin.conv_w, conv_w, Cc * e->conv_k));
    l.lin.conv_b = nullptr;
    ORN_TRY(upload(l, &l.lin.a_coef, a_coef, e->nv));
    ORN_TRY(upload(l, &l.lin.dt_bias, dt_bias, e->nv));
    ORN_TRY(upload(l, &l.lin.norm_w, norm_w, e->dv));
    l.st.S_seq_stride = (int64_t)e->nv * e->dv * e->dk;
    l.st.conv_seq_stride = (int64_t)e->conv_k * Cc;
    ORN_TRY(dev_alloc(l, (void **)&l.st.S, (size_t)l.st.S_seq_stride * sizeof(float), true));
    ORN_TRY(dev_alloc(l, (void **)&l.st.conv, (size_t)l.st.conv_seq_stride * sizeof(float), true));
    l.kind = 2;
    return ORNITH_OK;
}

// T tokens of a full-attention layer at positions pos .. pos+T-1 (the cache holds `pos` rows).
//   qproj [T][n_heads][2*head_dim] ([q | gate] per head), k, v [T][n_kv_heads][head_dim], out [T][n_heads*head_dim], host f32.
ornith_status ornith_cuda_engine_full_attn(ornith_cuda_engine *e, int L, int pos, int T, const float *qproj, const float *k,
                                           const float *v, float *out) {
    ornith_cuda_engine::Layer *l;
    ORN_TRY(layer_at(e, L, 1, &l));
    if (T <= 0) return ORNITH_OK;
    if (pos < 0 || pos + T > e->capacity) { orn_record_error("engine: positions %d..%d do not fit a capacity of %d", pos, pos + T, e->capacity); return ORNITH_ERR_FORMAT; }
    const size_t qn = (size_t)T * e->nh * 2 * e->hd, kn = (size_t)T * e->nkv * e->hd, on = (size_t)T * e->nh * e->hd;
    ORN_TRY(grow(&e->act, &e->act_bytes, (qn + 2 * kn + on) * sizeof(float)));
    float *dq = (float *)e->act, *dk = dq + qn, *dv = dk + kn, *dout = dv + kn;
    ORN_TRY(ornith_cuda_h2d(dq, qproj, qn * sizeof(float)));
    ORN_TRY(ornith_cuda_h2d(dk, k, kn * sizeof(float)));
    ORN_TRY(ornith_cuda_h2d(dv, v, kn * sizeof(float)));
    ORN_TRY(set_pos(e, pos));
    if (T == 1) {
        ORN_TRY(grow(&e->scratch, &e->scratch_bytes, ornith_cuda_full_attn_step_scratch(&l->full, 1, pos + 1)));
        ORN_TRY(ornith_cuda_full_attn_step(&l->full, &l->kv, e->d_pos, nullptr, dq, dk, dv, dout, ORNITH_ACT_F32, pos + 1, e->scratch,
                                           e->scratch_bytes, nullptr));
    } else {
        ORN_TRY(grow(&e->scratch, &e->scratch_bytes, ornith_cuda_full_attn_prefill_scratch(&l->full, 1, T, pos + T)));
        ORN_TRY(ornith_cuda_full_attn_prefill(&l->full, &l->kv, e->d_pos, nullptr, dq, dk, dv, dout, ORNITH_ACT_F32, T, pos + T,
                                              e->scratch, e->scratch_bytes, nullptr));
    }
    return ornith_cuda_d2h(out, dout, on * sizeof(float));
}

// T tokens of a delta-net layer.  qkv [T][Cc] (the fused projection, before the conv), a, b [T][nv] (gate
// projections), z [T][nv*dv] (the output gate projection, before SiLU), out [T][nv*dv], host f32.
ornith_status ornith_cuda_engine_linear_attn(ornith_cuda_engine *e, int L, int pos, int T, const float *qkv, const float *a,
                                             const float *b, const float *z, float *out) {
    ornith_cuda_engine::Layer *l;
    ORN_TRY(layer_at(e, L, 2, &l));
    if (T <= 0) return ORNITH_OK;
    const size_t Cc = (size_t)2 * e->nk * e->dk + (size_t)e->nv * e->dv, vd = (size_t)e->nv * e->dv;
    const size_t cn = (size_t)T * Cc, gn = (size_t)T * e->nv, on = (size_t)T * vd;
    ORN_TRY(grow(&e->act, &e->act_bytes, (cn + 2 * gn + 2 * on) * sizeof(float)));
    float *dc = (float *)e->act, *da = dc + cn, *db = da + gn, *dz = db + gn, *dout = dz + on;
    ORN_TRY(ornith_cuda_h2d(dc, qkv, cn * sizeof(float)));
    ORN_TRY(ornith_cuda_h2d(da, a, gn * sizeof(float)));
    ORN_TRY(ornith_cuda_h2d(db, b, gn * sizeof(float)));
    ORN_TRY(ornith_cuda_h2d(dz, z, on * sizeof(float)));
    ORN_TRY(set_pos(e, pos));
    if (T == 1) {
        ORN_TRY(ornith_cuda_linear_attn_step(&l->lin, &l->st, e->d_pos, dc, da, db, dz, dout, ORNITH_ACT_F32, 1, nullptr));
    } else {
        ORN_TRY(grow(&e->scratch, &e->scratch_bytes, ornith_cuda_linear_attn_prefill_scratch(&l->lin, 1, T)));
        ORN_TRY(ornith_cuda_linear_attn_prefill(&l->lin, &l->st, e->d_pos, dc, da, db, dz, dout, ORNITH_ACT_F32, 1, T, 64, e->scratch,
                                                e->scratch_bytes, nullptr));
    }
    return ornith_cuda_d2h(out, dout, on * sizeof(float));
}

// Session records of layer L after `pos` tokens (see the session-record entry points for the layouts).
size_t ornith_cuda_engine_record_bytes(const ornith_cuda_engine *e, int L, int pos) {
    if (!e || L < 0 || L >= e->num_layers) return 0;
    const ornith_cuda_engine::Layer &l = e->layers[L];
    return l.kind == 1 ? ornith_cuda_kv_record_bytes(&l.kv, pos) : l.kind == 2 ? ornith_cuda_linear_record_bytes(&l.lin) : 0;
}
ornith_status ornith_cuda_engine_export(const ornith_cuda_engine *e, int L, int pos, void *host_dst, size_t dst_bytes) {
    if (!e || L < 0 || L >= e->num_layers || !e->layers[L].kind) { orn_record_error("engine_export: layer %d has no state", L); return ORNITH_ERR_FORMAT; }
    const ornith_cuda_engine::Layer &l = e->layers[L];
    return l.kind == 1 ? ornith_cuda_kv_export(&l.kv, 0, pos, host_dst, dst_bytes, nullptr)
                       : ornith_cuda_linear_export(&l.lin, &l.st, 0, pos, host_dst, dst_bytes, nullptr);
}
ornith_status ornith_cuda_engine_import(ornith_cuda_engine *e, int L, int pos, const void *host_src, size_t src_bytes) {
    if (!e || L < 0 || L >= e->num_layers || !e->layers[L].kind) { orn_record_error("engine_import: set the layer's weights first (layer %d)", L); return ORNITH_ERR_FORMAT; }
    ornith_cuda_engine::Layer &l = e->layers[L];
    if (l.kind == 1) {
        int32_t len = 0;
        ORN_TRY(ornith_cuda_kv_import(&l.kv, 0, host_src, src_bytes, &len, nullptr, nullptr));
        if (len != pos) { orn_record_error("engine_import: the record of layer %d holds %d positions, the session is at %d", L, len, pos); return ORNITH_ERR_FORMAT; }
        return ORNITH_OK;
    }
    return ornith_cuda_linear_import(&l.lin, &l.st, 0, pos, host_src, src_bytes, nullptr);
}

}  // extern "C"
