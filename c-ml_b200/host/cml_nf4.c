/*
 * NF4 quantisation and the quantized Linear forward (C-ML: src/core/quantization.c:195-370,
 * src/nn/qlora.c). Same objects, ownership and error behaviour; the arithmetic runs on the GPU.
 * The forward never materialises the fp32 weight: it is the dequant-fused matmul.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "cml_internal.h"

const float CML_NF4_TABLE[16] = {-1.0f, -0.6962f, -0.5251f, -0.3949f, -0.2844f, -0.1848f, -0.0911f, 0.0f,
                                 0.0796f, 0.1609f, 0.2461f, 0.3379f, 0.4407f, 0.5626f, 0.7230f, 1.0f};

Tensor* cml_quantize_nf4(Tensor* tensor, int block_size, float** out_scales, int* out_num_scales) {
    if (!tensor) { LOG_ERROR("cml_quantize_nf4: NULL tensor"); return NULL; }
    if (block_size <= 0) { LOG_ERROR("cml_quantize_nf4: block_size must be positive, got %d", block_size); return NULL; }
    if (!out_scales || !out_num_scales) { LOG_ERROR("cml_quantize_nf4: NULL output pointers"); return NULL; }
    if (!tensor->data) { LOG_ERROR("cml_quantize_nf4: tensor has no data"); return NULL; }
    const size_t numel = tensor->numel;
    if (numel == 0) { LOG_ERROR("cml_quantize_nf4: tensor has 0 elements"); return NULL; }
    const size_t nbytes = (numel + 1) / 2;
    const int nblocks = (int)((numel + (size_t)block_size - 1) / (size_t)block_size);
    int pshape[1] = {(int)nbytes};
    Tensor* packed = cml_tensor_alloc(DTYPE_UINT8, pshape, 1, false);
    float* scales = (float*)malloc((size_t)nblocks * sizeof(float));
    void *d_x = NULL, *d_p = NULL, *d_s = NULL;
    int ok = packed && scales;
    ok = ok && !CML_DEV_FAIL(cmlb200_malloc(&d_x, numel * 4), "cml_quantize_nf4");
    ok = ok && !CML_DEV_FAIL(cmlb200_malloc(&d_p, nbytes), "cml_quantize_nf4");
    ok = ok && !CML_DEV_FAIL(cmlb200_malloc(&d_s, (size_t)nblocks * 4), "cml_quantize_nf4");
    ok = ok && !CML_DEV_FAIL(cmlb200_memcpy_h2d(d_x, tensor->data, numel * 4, NULL), "cml_quantize_nf4");
    ok = ok && !CML_DEV_FAIL(cmlb200_quantize_nf4((const float*)d_x, numel, block_size, (uint8_t*)d_p, (float*)d_s, NULL), "cml_quantize_nf4");
    ok = ok && !CML_DEV_FAIL(cmlb200_memcpy_d2h(packed->data, d_p, nbytes, NULL), "cml_quantize_nf4");
    ok = ok && !CML_DEV_FAIL(cmlb200_memcpy_d2h(scales, d_s, (size_t)nblocks * 4, NULL), "cml_quantize_nf4");
    ok = ok && !CML_DEV_FAIL(cmlb200_stream_sync(NULL), "cml_quantize_nf4");
    cmlb200_free(d_x); cmlb200_free(d_p); cmlb200_free(d_s);
    if (!ok) { tensor_free(packed); free(scales); return NULL; }
    *out_scales = scales;
    *out_num_scales = nblocks;
    return packed;
}

Tensor* cml_dequantize_nf4(Tensor* nf4_tensor, const float* scales, int num_scales, int block_size, size_t original_numel) {
    if (!nf4_tensor || !scales) { LOG_ERROR("cml_dequantize_nf4: NULL argument"); return NULL; }
    if (num_scales <= 0 || block_size <= 0 || original_numel == 0) { LOG_ERROR("cml_dequantize_nf4: invalid parameters"); return NULL; }
    if (!nf4_tensor->data) { LOG_ERROR("cml_dequantize_nf4: tensor has no data"); return NULL; }
    int oshape[1] = {(int)original_numel};
    Tensor* out = cml_tensor_alloc(DTYPE_FLOAT32, oshape, 1, false);
    const size_t nbytes = (original_numel + 1) / 2;
    void *d_p = NULL, *d_s = NULL, *d_o = NULL;
    int ok = out != NULL;
    ok = ok && !CML_DEV_FAIL(cmlb200_malloc(&d_p, nbytes), "cml_dequantize_nf4");
    ok = ok && !CML_DEV_FAIL(cmlb200_malloc(&d_s, (size_t)num_scales * 4), "cml_dequantize_nf4");
    ok = ok && !CML_DEV_FAIL(cmlb200_malloc(&d_o, original_numel * 4), "cml_dequantize_nf4");
    ok = ok && !CML_DEV_FAIL(cmlb200_memcpy_h2d(d_p, nf4_tensor->data, nbytes, NULL), "cml_dequantize_nf4");
    ok = ok && !CML_DEV_FAIL(cmlb200_memcpy_h2d(d_s, scales, (size_t)num_scales * 4, NULL), "cml_dequantize_nf4");
    ok = ok && !CML_DEV_FAIL(cmlb200_dequantize_nf4((const uint8_t*)d_p, (const float*)d_s, num_scales, block_size, original_numel, (float*)d_o, NULL), "cml_dequantize_nf4");
    ok = ok && !CML_DEV_FAIL(cmlb200_memcpy_d2h(out->data, d_o, original_numel * 4, NULL), "cml_dequantize_nf4");
    ok = ok && !CML_DEV_FAIL(cmlb200_stream_sync(NULL), "cml_dequantize_nf4");
    cmlb200_free(d_p); cmlb200_free(d_s); cmlb200_free(d_o);
    if (!ok) { tensor_free(out); return NULL; }
    return out;
}

CMLNF4Tensor* cml_nf4_tensor_create(Tensor* float_tensor, int block_size) {
    if (!float_tensor) { LOG_ERROR("cml_nf4_tensor_create: NULL tensor"); return NULL; }
    if (block_size <= 0) { LOG_ERROR("cml_nf4_tensor_create: block_size must be positive, got %d", block_size); return NULL; }
    if (!float_tensor->data) { LOG_ERROR("cml_nf4_tensor_create: tensor has no data"); return NULL; }
    CMLNF4Tensor* nf4 = (CMLNF4Tensor*)calloc(1, sizeof *nf4);
    if (!nf4) { LOG_ERROR("cml_nf4_tensor_create: allocation failed"); return NULL; }
    nf4->block_size = block_size;
    nf4->original_numel = float_tensor->numel;
    nf4->original_ndim = float_tensor->ndim;
    nf4->original_shape = (int*)malloc((size_t)float_tensor->ndim * sizeof(int));
    if (!nf4->original_shape) { free(nf4); return NULL; }
    memcpy(nf4->original_shape, float_tensor->shape, (size_t)float_tensor->ndim * sizeof(int));
    nf4->packed_data = cml_quantize_nf4(float_tensor, block_size, &nf4->scales, &nf4->num_scales);
    if (!nf4->packed_data) {
        LOG_ERROR("cml_nf4_tensor_create: NF4 quantization failed");
        free(nf4->original_shape);
        free(nf4);
        return NULL;
    }
    return nf4;
}

void cml_nf4_tensor_free(CMLNF4Tensor* nf4) {
    if (!nf4) return;
    tensor_free(nf4->packed_data);
    free(nf4->scales);
    free(nf4->original_shape);
    free(nf4);
}

Tensor* cml_nf4_tensor_dequantize(const CMLNF4Tensor* nf4) {
    if (!nf4) { LOG_ERROR("cml_nf4_tensor_dequantize: NULL NF4 tensor"); return NULL; }
    if (!nf4->packed_data || !nf4->scales) { LOG_ERROR("cml_nf4_tensor_dequantize: incomplete NF4 tensor"); return NULL; }
    Tensor* flat = cml_dequantize_nf4(nf4->packed_data, nf4->scales, nf4->num_scales, nf4->block_size, nf4->original_numel);
    if (!flat) return NULL;
    if (nf4->original_ndim != 1) {                    /* give the flat result its original shape */
        int* sh = (int*)realloc(flat->shape, (size_t)nf4->original_ndim * sizeof(int));
        size_t* st = (size_t*)realloc(flat->strides, (size_t)nf4->original_ndim * sizeof(size_t));
        if (!sh || !st) { if (sh) flat->shape = sh; if (st) flat->strides = st; tensor_free(flat); return NULL; }
        flat->shape = sh;
        flat->strides = st;
        flat->ndim = nf4->original_ndim;
        size_t s = 1;
        for (int i = flat->ndim - 1; i >= 0; i--) { sh[i] = nf4->original_shape[i]; st[i] = s; s *= (size_t)sh[i]; }
    }
    return flat;
}

/* ---- device-resident state of a CMLQLoRALinear, kept in a side table keyed by its address ---- */
typedef struct QloraDev {
    const CMLQLoRALinear* key;
    void *d_packed, *d_scales;
    struct QloraDev* next;
} QloraDev;
static QloraDev* g_qlora_dev = NULL;

static QloraDev* qdev_find(const CMLQLoRALinear* q) {
    for (QloraDev* d = g_qlora_dev; d; d = d->next) if (d->key == q) return d;
    return NULL;
}

void cml_qlora_linear_invalidate(CMLQLoRALinear* qlora) {
    QloraDev** pp = &g_qlora_dev;
    while (*pp) {
        if ((*pp)->key == qlora) {
            QloraDev* d = *pp;
            *pp = d->next;
            cmlb200_free(d->d_packed);
            cmlb200_free(d->d_scales);
            free(d);
            return;
        }
        pp = &(*pp)->next;
    }
}

CMLQLoRALinear* cml_qlora_linear_create(Tensor* base_weight, int rank, float alpha, int block_size) {
    if (!base_weight) { LOG_ERROR("cml_qlora_linear_create: base_weight is NULL"); return NULL; }
    if (base_weight->ndim != 2) { LOG_ERROR("cml_qlora_linear_create: base_weight must be 2D [out_features, in_features], got ndim=%d", base_weight->ndim); return NULL; }
    if (rank <= 0) { LOG_ERROR("cml_qlora_linear_create: rank must be positive, got %d", rank); return NULL; }
    if (block_size <= 0) { LOG_ERROR("cml_qlora_linear_create: block_size must be positive, got %d", block_size); return NULL; }
    CMLQLoRALinear* q = (CMLQLoRALinear*)calloc(1, sizeof *q);
    if (!q) { LOG_ERROR("cml_qlora_linear_create: allocation failed"); return NULL; }
    q->out_features = base_weight->shape[0];
    q->in_features = base_weight->shape[1];
    q->rank = rank;
    q->alpha = alpha;
    q->scaling = alpha / (float)rank;
    q->base_weight_nf4 = cml_nf4_tensor_create(base_weight, block_size);
    int sa[2] = {rank, q->in_features}, sb[2] = {q->out_features, rank};
    q->lora_A = q->base_weight_nf4 ? cml_tensor_alloc(DTYPE_FLOAT32, sa, 2, false) : NULL;
    q->lora_B = q->lora_A ? cml_tensor_alloc(DTYPE_FLOAT32, sb, 2, true) : NULL;
    if (!q->lora_B) {
        LOG_ERROR("cml_qlora_linear_create: failed to build the layer");
        cml_qlora_linear_free(q);
        return NULL;
    }
    /* lora_A: Xavier-scaled normal draws from rand() via Box-Muller (src/nn/qlora.c:192-206) */
    const float xs = sqrtf(2.0f / (float)(rank + q->in_features));
    float* a = (float*)q->lora_A->data;
    for (int i = 0; i < rank * q->in_features; i++) {
        const float u1 = (float)rand() / (float)RAND_MAX, u2 = (float)rand() / (float)RAND_MAX;
        a[i] = sqrtf(-2.0f * logf(u1 + 1e-10f)) * cosf(2.0f * 3.14159265f * u2) * xs;
    }
    return q;
}

void cml_qlora_linear_free(CMLQLoRALinear* qlora) {
    if (!qlora) return;
    cml_qlora_linear_invalidate(qlora);
    cml_nf4_tensor_free(qlora->base_weight_nf4);
    tensor_free(qlora->lora_A);
    tensor_free(qlora->lora_B);
    free(qlora);
}

Tensor* cml_qlora_linear_forward(CMLQLoRALinear* qlora, Tensor* input) {
    if (!qlora || !input) { LOG_ERROR("cml_qlora_linear_forward: NULL argument"); return NULL; }
    if (input->ndim != 2) { LOG_ERROR("cml_qlora_linear_forward: input must be 2D [batch, in_features], got ndim=%d", input->ndim); return NULL; }
    const int M = input->shape[0], K = input->shape[1], N = qlora->out_features, r = qlora->rank;
    if (K != qlora->in_features) { LOG_ERROR("cml_qlora_linear_forward: input in_features mismatch: got %d, expected %d", K, qlora->in_features); return NULL; }
    const CMLNF4Tensor* w = qlora->base_weight_nf4;
    if (!w || !w->packed_data || !w->scales || !qlora->lora_A || !qlora->lora_B || !input->data) {
        LOG_ERROR("cml_qlora_linear_forward: incomplete layer");
        return NULL;
    }
    /* shapes the vectorised kernels take; everything else (C-ML accepts any) goes element by element */
    const int fast = K % 32 == 0 && w->block_size % 32 == 0 && K % w->block_size == 0;
    QloraDev* dev = qdev_find(qlora);
    if (!dev) {
        dev = (QloraDev*)calloc(1, sizeof *dev);
        if (!dev) return NULL;
        dev->key = qlora;
        const size_t pb = (w->original_numel + 1) / 2, sb = (size_t)w->num_scales * 4;
        if (CML_DEV_FAIL(cmlb200_malloc(&dev->d_packed, pb), "cml_qlora_linear_forward") ||
            CML_DEV_FAIL(cmlb200_malloc(&dev->d_scales, sb), "cml_qlora_linear_forward") ||
            CML_DEV_FAIL(cmlb200_memcpy_h2d(dev->d_packed, w->packed_data->data, pb, NULL), "cml_qlora_linear_forward") ||
            CML_DEV_FAIL(cmlb200_memcpy_h2d(dev->d_scales, w->scales, sb, NULL), "cml_qlora_linear_forward")) {
            cmlb200_free(dev->d_packed); cmlb200_free(dev->d_scales); free(dev);
            return NULL;
        }
        dev->next = g_qlora_dev;
        g_qlora_dev = dev;
    }
    cmlb200_qmat W = {CMLB200_NF4, N, K, w->block_size, dev->d_packed, dev->d_scales, 0, NULL};
    int oshape[2] = {M, N};
    Tensor* out = cml_tensor_alloc(DTYPE_FLOAT32, oshape, 2, false);
    void *d_x = NULL, *d_y = NULL, *d_xb = NULL, *d_yb = NULL, *d_A = NULL, *d_B = NULL, *d_t = NULL;
    int ok = out != NULL;
    ok = ok && !CML_DEV_FAIL(cmlb200_malloc(&d_x, (size_t)M * K * 4), "cml_qlora_linear_forward");
    ok = ok && !CML_DEV_FAIL(cmlb200_malloc(&d_y, (size_t)M * N * 4), "cml_qlora_linear_forward");
    ok = ok && !CML_DEV_FAIL(cmlb200_memcpy_h2d(d_x, input->data, (size_t)M * K * 4, NULL), "cml_qlora_linear_forward");
    if (ok && !fast) {
        ok = !CML_DEV_FAIL(cmlb200_linear_nf4_general((const uint8_t*)dev->d_packed, (const float*)dev->d_scales, w->num_scales, w->block_size,
                                                      N, K, (const float*)d_x, M, (float*)d_y, NULL), "cml_qlora_linear_forward");
    } else if (ok && M <= 32) {
        ok = !CML_DEV_FAIL(cmlb200_gemv(&W, (const float*)d_x, (float*)d_y, M, NULL), "cml_qlora_linear_forward");
    } else if (ok) {                                   /* prefill-sized batch: bf16 tensor-core path */
        ok = ok && !CML_DEV_FAIL(cmlb200_malloc(&d_xb, (size_t)M * K * 2), "cml_qlora_linear_forward");
        ok = ok && !CML_DEV_FAIL(cmlb200_malloc(&d_yb, (size_t)M * N * 2), "cml_qlora_linear_forward");
        ok = ok && !CML_DEV_FAIL(cmlb200_f32_to_bf16((const float*)d_x, (uint16_t*)d_xb, (size_t)M * K, NULL), "cml_qlora_linear_forward");
        ok = ok && !CML_DEV_FAIL(cmlb200_gemm_bf16(&W, (const uint16_t*)d_xb, (uint16_t*)d_yb, M, NULL), "cml_qlora_linear_forward");
        ok = ok && !CML_DEV_FAIL(cmlb200_bf16_to_f32((const uint16_t*)d_yb, (float*)d_y, (size_t)M * N, NULL), "cml_qlora_linear_forward");
    }
    /* LoRA term: the adapters live in host tensors the caller may edit between calls, so they
     * are uploaded on every call (rank * (in + out) floats). */
    ok = ok && !CML_DEV_FAIL(cmlb200_malloc(&d_A, (size_t)r * K * 4), "cml_qlora_linear_forward");
    ok = ok && !CML_DEV_FAIL(cmlb200_malloc(&d_B, (size_t)N * r * 4), "cml_qlora_linear_forward");
    ok = ok && !CML_DEV_FAIL(cmlb200_malloc(&d_t, (size_t)M * r * 4), "cml_qlora_linear_forward");
    ok = ok && !CML_DEV_FAIL(cmlb200_memcpy_h2d(d_A, qlora->lora_A->data, (size_t)r * K * 4, NULL), "cml_qlora_linear_forward");
    ok = ok && !CML_DEV_FAIL(cmlb200_memcpy_h2d(d_B, qlora->lora_B->data, (size_t)N * r * 4, NULL), "cml_qlora_linear_forward");
    ok = ok && !CML_DEV_FAIL(cmlb200_lora_accum((const float*)d_x, (const float*)d_A, (const float*)d_B, M, K, N, r, qlora->scaling,
                                                (float*)d_t, (float*)d_y, NULL), "cml_qlora_linear_forward");
    ok = ok && !CML_DEV_FAIL(cmlb200_memcpy_d2h(out->data, d_y, (size_t)M * N * 4, NULL), "cml_qlora_linear_forward");
    ok = ok && !CML_DEV_FAIL(cmlb200_stream_sync(NULL), "cml_qlora_linear_forward");
    cmlb200_free(d_x); cmlb200_free(d_y); cmlb200_free(d_xb); cmlb200_free(d_yb);
    cmlb200_free(d_A); cmlb200_free(d_B); cmlb200_free(d_t);
    if (!ok) { tensor_free(out); return NULL; }
    return out;
}

size_t cml_qlora_memory_usage(const CMLQLoRALinear* qlora) {
    if (!qlora) return 0;
    size_t mem = 0;
    if (qlora->base_weight_nf4) {
        mem += (qlora->base_weight_nf4->original_numel + 1) / 2;
        mem += (size_t)qlora->base_weight_nf4->num_scales * sizeof(float);
    }
    mem += (size_t)qlora->rank * (size_t)qlora->in_features * sizeof(float);
    mem += (size_t)qlora->out_features * (size_t)qlora->rank * sizeof(float);
    return mem;
}

size_t cml_qlora_full_memory_usage(int in_features, int out_features) {
    return (size_t)in_features * (size_t)out_features * sizeof(float);
}
