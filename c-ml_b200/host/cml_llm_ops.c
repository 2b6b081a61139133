/*
 * The KV-cache / GQA / RoPE subset of C-ML's include/nn/llm_ops.h:13-89 as stand-alone entry
 * points: host tensors in, host tensors out, arithmetic on the device (src/nn/llm_ops.c:79-444,
 * 702-805 are the CPU loops they replace). The cache object itself stays what C-ML defines -- two
 * dense fp32 host tensors that callers read directly -- so append / reset / get are the same
 * copies C-ML does; cml_llama_forward does not go through it (its cache lives on the device).
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "cml_internal.h"

#define FAIL(call, who) CML_DEV_FAIL(call, who)

/* ---- src/nn/llm_ops.c:79-192 ---------------------------------------------------------------- */
CMLKVCache* cml_kv_cache_create(int max_seq_len, int num_kv_heads, int head_dim) {
    if (max_seq_len <= 0 || num_kv_heads <= 0 || head_dim <= 0) {
        LOG_ERROR("cml_kv_cache_create: invalid parameters (max_seq=%d, kv_heads=%d, head_dim=%d)", max_seq_len, num_kv_heads, head_dim);
        return NULL;
    }
    CMLKVCache* cache = (CMLKVCache*)calloc(1, sizeof *cache);
    if (!cache) { LOG_ERROR("cml_kv_cache_create: allocation failed"); return NULL; }
    cache->max_seq_len = max_seq_len;
    cache->num_kv_heads = num_kv_heads;
    cache->head_dim = head_dim;
    const int shape[3] = {max_seq_len, num_kv_heads, head_dim};
    cache->key_cache = cml_tensor_alloc(DTYPE_FLOAT32, shape, 3, true);
    cache->value_cache = cml_tensor_alloc(DTYPE_FLOAT32, shape, 3, true);
    if (!cache->key_cache || !cache->value_cache) {
        LOG_ERROR("cml_kv_cache_create: failed to allocate cache tensors");
        tensor_free(cache->key_cache);
        tensor_free(cache->value_cache);
        free(cache);
        return NULL;
    }
    return cache;
}

void cml_kv_cache_free(CMLKVCache* cache) {
    if (!cache) return;
    tensor_free(cache->key_cache);
    tensor_free(cache->value_cache);
    free(cache);
}

int cml_kv_cache_append(CMLKVCache* cache, Tensor* new_key, Tensor* new_value) {
    if (!cache || !new_key || !new_value) { LOG_ERROR("cml_kv_cache_append: NULL argument"); return -1; }
    if (!cache->key_cache || !cache->value_cache || !cache->key_cache->data || !cache->value_cache->data || !new_key->data ||
        !new_value->data || new_key->ndim < 1) {
        LOG_ERROR("cml_kv_cache_append: failed to get data pointers");
        return -1;
    }
    const int append_len = new_key->shape[0];
    if (cache->current_len + append_len > cache->max_seq_len) {
        LOG_ERROR("cml_kv_cache_append: cache overflow (%d + %d > %d)", cache->current_len, append_len, cache->max_seq_len);
        return -1;
    }
    const size_t row = (size_t)cache->num_kv_heads * cache->head_dim;
    const size_t off = (size_t)cache->current_len * row, bytes = (size_t)append_len * row * sizeof(float);
    memcpy((float*)cache->key_cache->data + off, new_key->data, bytes);
    memcpy((float*)cache->value_cache->data + off, new_value->data, bytes);
    cache->current_len += append_len;
    return cache->current_len;
}

void cml_kv_cache_reset(CMLKVCache* cache) {
    if (cache) cache->current_len = 0;
}

static Tensor* cache_prefix(CMLKVCache* cache, Tensor* src) {
    if (!cache || cache->current_len == 0 || !src || !src->data) return NULL;
    int shape[3] = {cache->current_len, cache->num_kv_heads, cache->head_dim};
    TensorConfig cfg = {.dtype = DTYPE_FLOAT32, .device = DEVICE_CPU, .has_dtype = true, .has_device = true};
    return tensor_from_data(src->data, shape, 3, &cfg);
}
Tensor* cml_kv_cache_get_keys(CMLKVCache* cache) { return cache_prefix(cache, cache ? cache->key_cache : NULL); }
Tensor* cml_kv_cache_get_values(CMLKVCache* cache) { return cache_prefix(cache, cache ? cache->value_cache : NULL); }

/* ---- src/nn/llm_ops.c:194-372 --------------------------------------------------------------- */
static Tensor* gqa_device(const float* q, const float* k, const float* v, int batch, int seq_q, int kv_len, const CMLGQAConfig* config,
                          Tensor* mask, DType out_dtype, DeviceType out_device, const char* who) {
    const int H = config->num_heads, KH = config->num_kv_heads, D = config->head_dim;
    float scale = config->scale;
    if (scale <= 0.0f) scale = 1.0f / sqrtf((float)D);
    const size_t qn = (size_t)batch * seq_q * H * D, kn = (size_t)batch * kv_len * KH * D;
    size_t mn = 0;
    if (mask) mn = mask->ndim == 2 ? (size_t)seq_q * kv_len : (size_t)batch * seq_q * kv_len;
    if (mask && (!mask->data || mask->numel < mn)) { LOG_ERROR("%s: mask smaller than [seq_q, kv_len]", who); return NULL; }
    int oshape[3] = {batch, seq_q, H * D};
    Tensor* out = cml_tensor_alloc(DTYPE_FLOAT32, oshape, 3, false);
    void *d_q = NULL, *d_k = NULL, *d_v = NULL, *d_m = NULL, *d_o = NULL;
    int ok = out != NULL;
    ok = ok && !FAIL(cmlb200_malloc(&d_q, qn * 4), who) && !FAIL(cmlb200_malloc(&d_k, kn * 4), who) &&
         !FAIL(cmlb200_malloc(&d_v, kn * 4), who) && !FAIL(cmlb200_malloc(&d_o, qn * 4), who);
    ok = ok && !FAIL(cmlb200_memcpy_h2d(d_q, q, qn * 4, NULL), who) && !FAIL(cmlb200_memcpy_h2d(d_k, k, kn * 4, NULL), who) &&
         !FAIL(cmlb200_memcpy_h2d(d_v, v, kn * 4, NULL), who);
    if (ok && mask) ok = !FAIL(cmlb200_malloc(&d_m, mn * 4), who) && !FAIL(cmlb200_memcpy_h2d(d_m, mask->data, mn * 4, NULL), who);
    ok = ok && !FAIL(cmlb200_gqa_f32((const float*)d_q, (const float*)d_k, (const float*)d_v, (const float*)d_m, mask && mask->ndim != 2,
                                     batch, seq_q, kv_len, H, KH, D, scale, config->causal ? 1 : 0, config->window_size, (float*)d_o, NULL),
                     who);
    ok = ok && !FAIL(cmlb200_memcpy_d2h(out->data, d_o, qn * 4, NULL), who) && !FAIL(cmlb200_stream_sync(NULL), who);
    cmlb200_free(d_q); cmlb200_free(d_k); cmlb200_free(d_v); cmlb200_free(d_m); cmlb200_free(d_o);
    if (!ok) { tensor_free(out); LOG_ERROR("%s: failed to create output tensor", who); return NULL; }
    out->dtype = out_dtype;
    out->device = out_device;
    return out;
}

static int gqa_check(const Tensor* Q, const Tensor* K, const Tensor* V, const CMLGQAConfig* config, const char* who) {
    if (Q->ndim != 3 || K->ndim != 3 || V->ndim != 3) { LOG_ERROR("%s: expected 3D tensors [batch, seq, dim]", who); return -1; }
    if (config->num_heads <= 0 || config->num_kv_heads <= 0 || config->head_dim <= 0) {
        LOG_ERROR("%s: invalid config (num_heads=%d, kv_heads=%d, head_dim=%d)", who, config->num_heads, config->num_kv_heads, config->head_dim);
        return -1;
    }
    if (config->num_heads % config->num_kv_heads != 0) {
        LOG_ERROR("%s: num_heads (%d) must be divisible by num_kv_heads (%d)", who, config->num_heads, config->num_kv_heads);
        return -1;
    }
    if (!Q->data || !K->data || !V->data) { LOG_ERROR("%s: failed to get data pointers", who); return -1; }
    return 0;
}

Tensor* cml_gqa_forward(Tensor* Q, Tensor* K, Tensor* V, const CMLGQAConfig* config, Tensor* mask) {
    if (!Q || !K || !V || !config) { LOG_ERROR("cml_gqa_forward: NULL argument"); return NULL; }
    if (gqa_check(Q, K, V, config, "cml_gqa_forward")) return NULL;
    return gqa_device((const float*)Q->data, (const float*)K->data, (const float*)V->data, Q->shape[0], Q->shape[1], K->shape[1], config, mask,
                      Q->dtype, Q->device, "cml_gqa_forward");
}

/* src/nn/llm_ops.c:374-444: append the new K, V rows (batch 1) to the host cache, then attend the
 * whole cached prefix; the causal mask of the config is the call-relative one of cml_gqa_forward. */
Tensor* cml_gqa_forward_cached(Tensor* Q, Tensor* K, Tensor* V, CMLKVCache* kv_cache, const CMLGQAConfig* config) {
    if (!Q || !K || !V || !kv_cache || !config) { LOG_ERROR("cml_gqa_forward_cached: NULL argument"); return NULL; }
    if (gqa_check(Q, K, V, config, "cml_gqa_forward_cached")) return NULL;
    int kv_shape[3] = {K->shape[1], config->num_kv_heads, config->head_dim};
    TensorConfig cfg = {.dtype = DTYPE_FLOAT32, .device = DEVICE_CPU, .has_dtype = true, .has_device = true};
    Tensor* k_append = tensor_from_data(K->data, kv_shape, 3, &cfg);
    Tensor* v_append = tensor_from_data(V->data, kv_shape, 3, &cfg);
    int new_len = -1;
    if (k_append && v_append) new_len = cml_kv_cache_append(kv_cache, k_append, v_append);
    tensor_free(k_append);
    tensor_free(v_append);
    if (new_len < 0) return NULL;
    return gqa_device((const float*)Q->data, (const float*)kv_cache->key_cache->data, (const float*)kv_cache->value_cache->data, 1, Q->shape[1],
                      kv_cache->current_len, config, NULL, Q->dtype, Q->device, "cml_gqa_forward_cached");
}

/* ---- src/nn/llm_ops.c:702-805 --------------------------------------------------------------- */
Tensor* cml_rope_forward(Tensor* x, int start_pos, const CMLRoPEConfig* config) {
    if (!x || !config) { LOG_ERROR("cml_rope_forward: NULL argument"); return NULL; }
    if (x->ndim < 2) { LOG_ERROR("cml_rope_forward: input must have at least 2 dims"); return NULL; }
    if (!x->data) { LOG_ERROR("cml_rope_forward: failed to get data pointer"); return NULL; }
    const int last_dim = x->shape[x->ndim - 1];
    /* which vectors rotate and at which position: [batch, seq, heads, head_dim] -> position = index
     * along dim 1; [batch, seq, dim] likewise; anything else is read as [seq, dim] over the first
     * shape[0] vectors, as C-ML does */
    size_t nvec;
    int seq_len, inner;
    if (x->ndim == 4) { nvec = (size_t)x->shape[0] * x->shape[1] * x->shape[2]; seq_len = x->shape[1]; inner = x->shape[2]; }
    else if (x->ndim == 3) { nvec = (size_t)x->shape[0] * x->shape[1]; seq_len = x->shape[1]; inner = 1; }
    else { nvec = (size_t)x->shape[0]; seq_len = x->shape[0]; inner = 1; }
    if (nvec == 0 || last_dim <= 0 || config->dim <= 0) return x;
    const size_t bytes = nvec * (size_t)last_dim * sizeof(float);
    void* d_x = NULL;
    int ok = !FAIL(cmlb200_malloc(&d_x, bytes), "cml_rope_forward") && !FAIL(cmlb200_memcpy_h2d(d_x, x->data, bytes, NULL), "cml_rope_forward") &&
             !FAIL(cmlb200_rope_f32((float*)d_x, nvec, last_dim, config->dim, config->base, start_pos, seq_len, inner, NULL), "cml_rope_forward") &&
             !FAIL(cmlb200_memcpy_d2h(x->data, d_x, bytes, NULL), "cml_rope_forward") && !FAIL(cmlb200_stream_sync(NULL), "cml_rope_forward");
    cmlb200_free(d_x);
    return ok ? x : NULL;     /* modified in place, same tensor returned for chaining */
}
