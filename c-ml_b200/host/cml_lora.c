/*
 * LoRA over an fp32 base weight (C-ML: src/nn/lora.c, include/nn/lora.h):
 *   y = x W^T + (alpha / rank) (x A^T) B^T,  W [out, in] not owned, A [rank, in], B [out, rank].
 * Same structs, ownership and error returns as C-ML; the arithmetic runs on the device: the base
 * product through cmlb200_linear_f32, the rank-r term through cmlb200_lora_accum (the kernels the
 * quantized QLoRA layer uses), the merge W += scaling B A through cmlb200_lora_merge. The tensors
 * are host tensors the caller may edit between calls, so every call uploads what it reads.
 * The initial A follows C-ML's recipe call for call (two rand() per element, Box-Muller, scale
 * sqrt(2 / (rank + in))), so a program that seeds rand() gets the adapter C-ML would have made.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "cml_internal.h"

#define WHO_FAIL(call, who) CML_DEV_FAIL(call, who)

CMLLoRALinear* cml_lora_linear_create(Tensor* base_weight, int rank, float alpha) {
    if (!base_weight) { LOG_ERROR("base_weight is NULL"); return NULL; }
    if (base_weight->ndim != 2) { LOG_ERROR("base_weight must be 2D [out_features, in_features], got ndim=%d", base_weight->ndim); return NULL; }
    if (rank <= 0) { LOG_ERROR("rank must be positive, got %d", rank); return NULL; }
    CMLLoRALinear* lora = (CMLLoRALinear*)calloc(1, sizeof *lora);
    if (!lora) { LOG_ERROR("Failed to allocate CMLLoRALinear"); return NULL; }
    lora->out_features = base_weight->shape[0];
    lora->in_features = base_weight->shape[1];
    lora->rank = rank;
    lora->alpha = alpha;
    lora->scaling = alpha / (float)rank;
    lora->base_weight = base_weight;
    int sa[2] = {rank, lora->in_features}, sb[2] = {lora->out_features, rank};
    lora->lora_A = cml_tensor_alloc(DTYPE_FLOAT32, sa, 2, false);
    lora->lora_B = cml_tensor_alloc(DTYPE_FLOAT32, sb, 2, true);
    if (!lora->lora_A || !lora->lora_B) {
        LOG_ERROR("Failed to allocate the LoRA matrices");
        tensor_free(lora->lora_A);
        tensor_free(lora->lora_B);
        free(lora);
        return NULL;
    }
    const float xavier = sqrtf(2.0f / (float)(rank + lora->in_features));
    float* a = (float*)lora->lora_A->data;
    for (int i = 0; i < rank * lora->in_features; i++) {
        const float u1 = (float)rand() / (float)RAND_MAX;
        const float u2 = (float)rand() / (float)RAND_MAX;
        a[i] = sqrtf(-2.0f * logf(u1 + 1e-10f)) * cosf(2.0f * 3.14159265f * u2) * xavier;
    }
    return lora;
}

void cml_lora_linear_free(CMLLoRALinear* lora) {
    if (!lora) return;
    tensor_free(lora->lora_A);
    tensor_free(lora->lora_B);
    tensor_free(lora->frozen_base);
    free(lora);
}

Tensor* cml_lora_linear_forward(CMLLoRALinear* lora, Tensor* input) {
    static const char* who = "cml_lora_linear_forward";
    if (!lora || !input) { LOG_ERROR("NULL argument to cml_lora_linear_forward"); return NULL; }
    if (input->ndim != 2) { LOG_ERROR("Input must be 2D [batch, in_features], got ndim=%d", input->ndim); return NULL; }
    const int M = input->shape[0], K = input->shape[1], N = lora->out_features, r = lora->rank;
    if (K != lora->in_features) { LOG_ERROR("Input in_features mismatch: got %d, expected %d", K, lora->in_features); return NULL; }
    if (!input->data || !lora->base_weight || !lora->base_weight->data || !lora->lora_A || !lora->lora_B) {
        LOG_ERROR("Failed to get data pointers for forward pass");
        return NULL;
    }
    int oshape[2] = {M, N};
    Tensor* out = cml_tensor_alloc(DTYPE_FLOAT32, oshape, 2, false);
    void *d_x = NULL, *d_w = NULL, *d_y = NULL, *d_A = NULL, *d_B = NULL, *d_t = NULL;
    int ok = out != NULL && M > 0;
    ok = ok && !WHO_FAIL(cmlb200_malloc(&d_x, (size_t)M * K * 4), who) && !WHO_FAIL(cmlb200_malloc(&d_w, (size_t)N * K * 4), who) &&
         !WHO_FAIL(cmlb200_malloc(&d_y, (size_t)M * N * 4), who);
    ok = ok && !WHO_FAIL(cmlb200_memcpy_h2d(d_x, input->data, (size_t)M * K * 4, NULL), who) &&
         !WHO_FAIL(cmlb200_memcpy_h2d(d_w, lora->base_weight->data, (size_t)N * K * 4, NULL), who);
    ok = ok && !WHO_FAIL(cmlb200_linear_f32((const float*)d_x, (const float*)d_w, NULL, M, N, K, (float*)d_y, NULL), who);
    if (ok && !lora->merged) {                       /* merged: the pair is already inside W (src/nn/lora.c:172-175) */
        ok = !WHO_FAIL(cmlb200_malloc(&d_A, (size_t)r * K * 4), who) && !WHO_FAIL(cmlb200_malloc(&d_B, (size_t)N * r * 4), who) &&
             !WHO_FAIL(cmlb200_malloc(&d_t, (size_t)M * r * 4), who);
        ok = ok && !WHO_FAIL(cmlb200_memcpy_h2d(d_A, lora->lora_A->data, (size_t)r * K * 4, NULL), who) &&
             !WHO_FAIL(cmlb200_memcpy_h2d(d_B, lora->lora_B->data, (size_t)N * r * 4, NULL), who);
        ok = ok && !WHO_FAIL(cmlb200_lora_accum((const float*)d_x, (const float*)d_A, (const float*)d_B, M, K, N, r, lora->scaling, (float*)d_t,
                                                (float*)d_y, NULL), who);
    }
    ok = ok && !WHO_FAIL(cmlb200_memcpy_d2h(out->data, d_y, (size_t)M * N * 4, NULL), who) && !WHO_FAIL(cmlb200_stream_sync(NULL), who);
    cmlb200_free(d_x); cmlb200_free(d_w); cmlb200_free(d_y); cmlb200_free(d_A); cmlb200_free(d_B); cmlb200_free(d_t);
    if (!ok) { tensor_free(out); return NULL; }
    return out;
}

int cml_lora_linear_merge(CMLLoRALinear* lora) {
    static const char* who = "cml_lora_linear_merge";
    if (!lora) { LOG_ERROR("NULL LoRA layer"); return -1; }
    if (lora->merged) { LOG_ERROR("LoRA layer is already merged"); return -1; }
    Tensor* W = lora->base_weight;
    if (!W || !W->data || !lora->lora_A || !lora->lora_B) { LOG_ERROR("Failed to get data pointers for merge"); return -1; }
    const int N = lora->out_features, K = lora->in_features, r = lora->rank;
    int shape[2] = {N, K};
    Tensor* frozen = cml_tensor_alloc(DTYPE_FLOAT32, shape, 2, false);
    if (!frozen) { LOG_ERROR("Failed to clone base_weight for frozen copy"); return -1; }
    memcpy(frozen->data, W->data, (size_t)N * K * 4);
    void *d_w = NULL, *d_A = NULL, *d_B = NULL;
    int ok = !WHO_FAIL(cmlb200_malloc(&d_w, (size_t)N * K * 4), who) && !WHO_FAIL(cmlb200_malloc(&d_A, (size_t)r * K * 4), who) &&
             !WHO_FAIL(cmlb200_malloc(&d_B, (size_t)N * r * 4), who);
    ok = ok && !WHO_FAIL(cmlb200_memcpy_h2d(d_w, W->data, (size_t)N * K * 4, NULL), who) &&
         !WHO_FAIL(cmlb200_memcpy_h2d(d_A, lora->lora_A->data, (size_t)r * K * 4, NULL), who) &&
         !WHO_FAIL(cmlb200_memcpy_h2d(d_B, lora->lora_B->data, (size_t)N * r * 4, NULL), who);
    ok = ok && !WHO_FAIL(cmlb200_lora_merge((float*)d_w, (const float*)d_A, (const float*)d_B, N, K, r, lora->scaling, NULL), who);
    ok = ok && !WHO_FAIL(cmlb200_memcpy_d2h(W->data, d_w, (size_t)N * K * 4, NULL), who) && !WHO_FAIL(cmlb200_stream_sync(NULL), who);
    cmlb200_free(d_w); cmlb200_free(d_A); cmlb200_free(d_B);
    if (!ok) {                                       /* the weight is as it was: the copy back is the last step */
        tensor_free(frozen);
        return -1;
    }
    tensor_free(lora->frozen_base);
    lora->frozen_base = frozen;
    lora->merged = true;
    LOG_DEBUG("Merged LoRA into base weight (rank=%d, scaling=%.4f)", r, lora->scaling);
    return 0;
}

int cml_lora_linear_unmerge(CMLLoRALinear* lora) {
    if (!lora) { LOG_ERROR("NULL LoRA layer"); return -1; }
    if (!lora->merged) { LOG_ERROR("LoRA layer is not merged, cannot unmerge"); return -1; }
    if (!lora->frozen_base) { LOG_ERROR("No frozen base weight available for unmerge"); return -1; }
    if (!lora->base_weight || !lora->base_weight->data || !lora->frozen_base->data) { LOG_ERROR("Failed to get data pointers for unmerge"); return -1; }
    /* the weight returns to the saved copy bit for bit (src/nn/lora.c:306-312) */
    memcpy(lora->base_weight->data, lora->frozen_base->data, (size_t)lora->out_features * lora->in_features * 4);
    tensor_free(lora->frozen_base);
    lora->frozen_base = NULL;
    lora->merged = false;
    return 0;
}

CMLLoRAAdapter* cml_lora_adapter_create(const char* name, int rank, float alpha) {
    if (!name) { LOG_ERROR("Adapter name is NULL"); return NULL; }
    if (rank <= 0) { LOG_ERROR("rank must be positive, got %d", rank); return NULL; }
    CMLLoRAAdapter* ad = (CMLLoRAAdapter*)calloc(1, sizeof *ad);
    if (!ad) { LOG_ERROR("Failed to allocate CMLLoRAAdapter"); return NULL; }
    strncpy(ad->name, name, sizeof ad->name - 1);
    ad->name[sizeof ad->name - 1] = 0;
    ad->rank = rank;
    ad->alpha = alpha;
    ad->scaling = alpha / (float)rank;
    return ad;
}

void cml_lora_adapter_free(CMLLoRAAdapter* adapter) {
    if (!adapter) return;
    for (int i = 0; i < adapter->num_layers; i++) cml_lora_linear_free(adapter->layers[i]);
    free(adapter->layers);
    free(adapter);
}

int cml_lora_adapter_add_layer(CMLLoRAAdapter* adapter, CMLLoRALinear* layer) {
    if (!adapter || !layer) { LOG_ERROR("NULL argument to cml_lora_adapter_add_layer"); return -1; }
    CMLLoRALinear** grown = (CMLLoRALinear**)realloc(adapter->layers, (size_t)(adapter->num_layers + 1) * sizeof *grown);
    if (!grown) { LOG_ERROR("Failed to grow adapter layers array"); return -1; }
    adapter->layers = grown;
    adapter->layers[adapter->num_layers++] = layer;
    return 0;
}

int cml_lora_adapter_merge_all(CMLLoRAAdapter* adapter) {
    if (!adapter) { LOG_ERROR("NULL adapter"); return -1; }
    if (adapter->merged) { LOG_ERROR("Adapter '%s' is already merged", adapter->name); return -1; }
    for (int i = 0; i < adapter->num_layers; i++) {
        if (cml_lora_linear_merge(adapter->layers[i]) != 0) {
            LOG_ERROR("Failed to merge layer %d of adapter '%s'", i, adapter->name);
            for (int j = 0; j < i; j++) cml_lora_linear_unmerge(adapter->layers[j]);      /* leave no layer half way */
            return -1;
        }
    }
    adapter->merged = true;
    return 0;
}

int cml_lora_adapter_unmerge_all(CMLLoRAAdapter* adapter) {
    if (!adapter) { LOG_ERROR("NULL adapter"); return -1; }
    if (!adapter->merged) { LOG_ERROR("Adapter '%s' is not merged", adapter->name); return -1; }
    for (int i = 0; i < adapter->num_layers; i++) {
        if (cml_lora_linear_unmerge(adapter->layers[i]) != 0) {
            LOG_ERROR("Failed to unmerge layer %d of adapter '%s'", i, adapter->name);
            return -1;
        }
    }
    adapter->merged = false;
    return 0;
}
