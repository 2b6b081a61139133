/*
 * Logging and the minimal eager host Tensor the quantized-LLM path needs at its API boundary
 * (C-ML: src/core/logging.c:7-32, src/tensor/tensor.c). Tensors created here are always
 * realised and contiguous; the lazy-graph fields of the struct stay NULL.
 */
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "cml_internal.h"

LogLevel g_log_level = LOG_LEVEL_ERROR;

/* ---- library set-up (src/cml.c:376-440) and the tensor seed (include/tensor/tensor.h:143) ------ */
static int g_init_count = 0;
static uint64_t g_tensor_seed = 0;

int cml_init(void) {
    if (g_init_count++ == 0) cml_set_log_level(LOG_LEVEL_ERROR);
    return 0;
}

int cml_cleanup(void) {
    if (g_init_count > 0) g_init_count--;
    return 0;
}

void tensor_manual_seed(uint64_t seed) { g_tensor_seed = seed; }
uint64_t tensor_get_seed(void) { return g_tensor_seed; }

void cml_set_log_level(LogLevel level) { g_log_level = level; }

void cml_log_message(LogLevel level, const char* file, int line, const char* func, const char* format, ...) {
    if (level < g_log_level) return;
    static const char* names[] = {"DEBUG", "INFO", "WARNING", "ERROR"};
    time_t now = time(NULL);
    struct tm tmv;
    localtime_r(&now, &tmv);
    char ts[32];
    strftime(ts, sizeof ts, "%Y-%m-%d %H:%M:%S", &tmv);
    fprintf(stderr, "[%s] [%s] %s:%d %s(): ", ts, names[level], file, line, func);
    va_list ap;
    va_start(ap, format);
    vfprintf(stderr, format, ap);
    va_end(ap);
    fputc('\n', stderr);
}

size_t cml_dtype_size(DType dtype) {
    switch (dtype) {
        case DTYPE_FLOAT32: case DTYPE_INT32: case DTYPE_UINT32: return 4;
        case DTYPE_FLOAT64: case DTYPE_INT64: case DTYPE_UINT64: return 8;
        case DTYPE_FLOAT16: case DTYPE_BFLOAT16: case DTYPE_INT16: case DTYPE_UINT16: return 2;
        default: return 1;
    }
}

Tensor* cml_tensor_alloc(DType dtype, const int* shape, int ndim, bool zero) {
    if (!shape || ndim <= 0 || ndim > 8) {
        LOG_ERROR("tensor: invalid shape (ndim=%d)", ndim);
        return NULL;
    }
    size_t numel = 1;
    for (int i = 0; i < ndim; i++) {
        if (shape[i] < 0) { LOG_ERROR("tensor: negative dimension"); return NULL; }
        numel *= (size_t)shape[i];
    }
    Tensor* t = (Tensor*)calloc(1, sizeof(Tensor));
    if (!t) { LOG_ERROR("tensor: allocation failed"); return NULL; }
    t->shape = (int*)malloc((size_t)ndim * sizeof(int));
    t->strides = (size_t*)malloc((size_t)ndim * sizeof(size_t));
    const size_t bytes = numel * cml_dtype_size(dtype);
    t->data = zero ? calloc(bytes ? bytes : 1, 1) : malloc(bytes ? bytes : 1);
    if (!t->shape || !t->strides || !t->data) {
        LOG_ERROR("tensor: allocation of %zu bytes failed", bytes);
        free(t->shape); free(t->strides); free(t->data); free(t);
        return NULL;
    }
    size_t st = 1;
    for (int i = ndim - 1; i >= 0; i--) { t->shape[i] = shape[i]; t->strides[i] = st; st *= (size_t)shape[i]; }
    t->ndim = ndim;
    t->numel = numel;
    t->dtype = dtype;
    t->device = DEVICE_CPU;
    t->is_executed = true;
    t->owns_data = true;
    t->ref_count = 1;
    t->is_contiguous = true;
    return t;
}

static DType cfg_dtype(const TensorConfig* c) { return (c && c->has_dtype) ? c->dtype : DTYPE_FLOAT32; }

Tensor* tensor_empty(int* shape, int ndim, const TensorConfig* config) { return cml_tensor_alloc(cfg_dtype(config), shape, ndim, false); }
Tensor* tensor_zeros(int* shape, int ndim, const TensorConfig* config) { return cml_tensor_alloc(cfg_dtype(config), shape, ndim, true); }

Tensor* tensor_from_data(const void* data, int* shape, int ndim, const TensorConfig* config) {
    if (!data) { LOG_ERROR("tensor_from_data: NULL data"); return NULL; }
    Tensor* t = cml_tensor_alloc(cfg_dtype(config), shape, ndim, false);
    if (t) memcpy(t->data, data, t->numel * cml_dtype_size(t->dtype));
    return t;
}

void tensor_free(Tensor* t) {
    if (!t) return;
    if (--t->ref_count > 0) return;
    if (t->owns_data) free(t->data);
    free(t->shape);
    free(t->strides);
    free(t->user_data);
    free(t);
}

void* tensor_data_ptr(Tensor* t) { return t ? t->data : NULL; }
int tensor_ensure_executed(Tensor* t) { return (t && t->data) ? 0 : -1; }

/* IEEE binary16 <-> binary32 on the host, round to nearest even. */
uint16_t cml_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u, ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (ax > 0x7F800000u ? 0x200u : 0));
    if (ax >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);
    if (ax < 0x33000001u) return (uint16_t)sign;
    const int e = (int)(ax >> 23) - 127;
    const uint32_t m = (ax & 0x7FFFFFu) | 0x800000u;
    const int shift = (e < -14) ? (13 + (-14 - e)) : 13;
    uint32_t half = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1u))) half++;
    const uint32_t out = (e < -14) ? half : ((uint32_t)(e + 15) << 10) + (half - 0x400u);
    return (uint16_t)(sign | out);
}

float cml_f16_to_f32(uint16_t h) {
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16, e = (h >> 10) & 0x1Fu;
    uint32_t m = h & 0x3FFu, bits;
    if (e == 0) {
        if (!m) bits = sign;
        else {
            int lz = 0;
            while (!(m & 0x400u)) { m <<= 1; lz++; }
            bits = sign | ((uint32_t)(113 - lz) << 23) | ((m & 0x3FFu) << 13);
        }
    } else if (e == 31) bits = sign | 0x7F800000u | (m << 13);
    else bits = sign | ((e + 112u) << 23) | (m << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}
