/*
 * Per-tensor affine quantisation to int8 / uint8 (C-ML: src/core/quantization.c:8-192,
 * include/core/quantization.h:16-25): same signatures, parameters and results; the scan for the
 * value range, the quantisation and the dequantisation run on the device (csrc/quant_int8.cu). The
 * handful of scalar operations that turn a range into (scale, zero_point) stay on the host, written
 * as C-ML writes them. fp32 tensors only: the other dtypes C-ML reads through tensor_get_float are
 * refused with an error.
 */
#include <float.h>
#include <math.h>
#include <stdlib.h>

#include "cml_internal.h"

/* min and max of an fp32 host tensor, found on the device; 0 on success */
static int tensor_range(Tensor* t, float* lo, float* hi, const char* who) {
    void *d_x = NULL, *d_s = NULL, *d_o = NULL;
    float out[2] = {FLT_MAX, -FLT_MAX};
    int ok = !CML_DEV_FAIL(cmlb200_malloc(&d_x, t->numel * 4), who) && !CML_DEV_FAIL(cmlb200_malloc(&d_s, cmlb200_range_scratch_floats() * 4), who) &&
             !CML_DEV_FAIL(cmlb200_malloc(&d_o, 8), who);
    ok = ok && !CML_DEV_FAIL(cmlb200_memcpy_h2d(d_x, t->data, t->numel * 4, NULL), who) &&
         !CML_DEV_FAIL(cmlb200_range_f32((const float*)d_x, t->numel, (float*)d_s, (float*)d_o, NULL), who) &&
         !CML_DEV_FAIL(cmlb200_memcpy_d2h(out, d_o, 8, NULL), who) && !CML_DEV_FAIL(cmlb200_stream_sync(NULL), who);
    cmlb200_free(d_x); cmlb200_free(d_s); cmlb200_free(d_o);
    *lo = out[0];
    *hi = out[1];
    return ok ? 0 : -1;
}

static int usable(const Tensor* t, const char* who) {
    if (t->dtype != DTYPE_FLOAT32) { LOG_ERROR("%s: only fp32 tensors are supported (dtype %d)", who, (int)t->dtype); return 0; }
    return 1;
}

QuantParams cml_quantize_compute_params(Tensor* tensor, bool symmetric) {
    QuantParams params = {.scale = 1.0f, .zero_point = 0};
    if (!tensor || !tensor->data || tensor->numel == 0 || !usable(tensor, "cml_quantize_compute_params")) return params;
    float lo, hi;
    if (tensor_range(tensor, &lo, &hi, "cml_quantize_compute_params")) return params;
    if (symmetric) {
        params.scale = fmaxf(fabsf(lo), fabsf(hi)) / 127.0f;
        params.zero_point = 0;
    } else {
        params.scale = (hi - lo) / 255.0f;
        if (params.scale < 1e-10f) params.scale = 1e-10f;
        params.zero_point = (int32_t)roundf(-lo / params.scale) - 128;
    }
    if (params.scale < 1e-10f) params.scale = 1e-10f;
    return params;
}

static Tensor* quantize8(Tensor* tensor, const QuantParams* params, QuantParams* out_params, int is_unsigned, const char* who) {
    if (!tensor) { LOG_ERROR("%s: NULL tensor", who); return NULL; }
    if (!tensor->data) { LOG_ERROR("%s: tensor has no data", who); return NULL; }
    if (!usable(tensor, who) || tensor->numel == 0) return NULL;
    QuantParams qp;
    if (params) qp = *params;
    else if (!is_unsigned) qp = cml_quantize_compute_params(tensor, true);
    else {                                            /* src/core/quantization.c:126-139: the uint8 zero point has no -128 */
        float lo, hi;
        if (tensor_range(tensor, &lo, &hi, who)) return NULL;
        qp.scale = (hi - lo) / 255.0f;
        if (qp.scale < 1e-10f) qp.scale = 1e-10f;
        qp.zero_point = (int32_t)roundf(-lo / qp.scale);
    }
    if (out_params) *out_params = qp;
    Tensor* q = cml_tensor_alloc(is_unsigned ? DTYPE_UINT8 : DTYPE_INT8, tensor->shape, tensor->ndim, false);
    if (!q) return NULL;
    void *d_x = NULL, *d_q = NULL;
    int ok = !CML_DEV_FAIL(cmlb200_malloc(&d_x, tensor->numel * 4), who) && !CML_DEV_FAIL(cmlb200_malloc(&d_q, tensor->numel), who);
    ok = ok && !CML_DEV_FAIL(cmlb200_memcpy_h2d(d_x, tensor->data, tensor->numel * 4, NULL), who) &&
         !CML_DEV_FAIL(cmlb200_quantize_8bit((const float*)d_x, tensor->numel, qp.scale, qp.zero_point, is_unsigned, d_q, NULL), who) &&
         !CML_DEV_FAIL(cmlb200_memcpy_d2h(q->data, d_q, tensor->numel, NULL), who) && !CML_DEV_FAIL(cmlb200_stream_sync(NULL), who);
    cmlb200_free(d_x); cmlb200_free(d_q);
    if (!ok) { tensor_free(q); return NULL; }
    return q;
}

static Tensor* dequantize8(Tensor* tensor, const QuantParams* params, int is_unsigned, const char* who) {
    if (!tensor || !params) { LOG_ERROR("%s: NULL tensor or params", who); return NULL; }
    if (!tensor->data) { LOG_ERROR("%s: tensor has no data", who); return NULL; }
    if (tensor->dtype != (is_unsigned ? DTYPE_UINT8 : DTYPE_INT8) || tensor->numel == 0) { LOG_ERROR("%s: not a%s tensor", who, is_unsigned ? " uint8" : "n int8"); return NULL; }
    Tensor* out = cml_tensor_alloc(DTYPE_FLOAT32, tensor->shape, tensor->ndim, false);
    if (!out) return NULL;
    void *d_q = NULL, *d_o = NULL;
    int ok = !CML_DEV_FAIL(cmlb200_malloc(&d_q, tensor->numel), who) && !CML_DEV_FAIL(cmlb200_malloc(&d_o, tensor->numel * 4), who);
    ok = ok && !CML_DEV_FAIL(cmlb200_memcpy_h2d(d_q, tensor->data, tensor->numel, NULL), who) &&
         !CML_DEV_FAIL(cmlb200_dequantize_8bit(d_q, tensor->numel, params->scale, params->zero_point, is_unsigned, (float*)d_o, NULL), who) &&
         !CML_DEV_FAIL(cmlb200_memcpy_d2h(out->data, d_o, tensor->numel * 4, NULL), who) && !CML_DEV_FAIL(cmlb200_stream_sync(NULL), who);
    cmlb200_free(d_q); cmlb200_free(d_o);
    if (!ok) { tensor_free(out); return NULL; }
    return out;
}

Tensor* cml_quantize_int8(Tensor* tensor, const QuantParams* params, QuantParams* out_params) {
    return quantize8(tensor, params, out_params, 0, "cml_quantize_int8");
}
Tensor* cml_dequantize_int8(Tensor* tensor, const QuantParams* params) { return dequantize8(tensor, params, 0, "cml_dequantize_int8"); }
Tensor* cml_quantize_uint8(Tensor* tensor, const QuantParams* params, QuantParams* out_params) {
    return quantize8(tensor, params, out_params, 1, "cml_quantize_uint8");
}
Tensor* cml_dequantize_uint8(Tensor* tensor, const QuantParams* params) { return dequantize8(tensor, params, 1, "cml_dequantize_uint8"); }
