/*
 * GGUF v3 reader and the block-type helpers (C-ML: src/core/gguf.c:105-310,
 * src/core/gguf_quant.c:313-391). The file format handling is host work; dequantisation runs on
 * the device. Layout read: magic, version, n_tensors, n_kv, the key/values (skipped by type),
 * the tensor infos (name, ndim, dims, type, offset) and data at align32(end of infos) + offset.
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "cml_internal.h"

struct GGUFContext {
    FILE* file;
    int num_tensors;
    GGUFTensorInfo* tensors;
    uint64_t data_offset;
};

bool gguf_type_is_quantized(GGUFTensorType type) {
    switch ((int)type) {
        case GGUF_TENSOR_Q4_0: case GGUF_TENSOR_Q4_1: case GGUF_TENSOR_Q8_0:
        case GGUF_TENSOR_Q4_K: case GGUF_TENSOR_Q5_K: case GGUF_TENSOR_Q6_K: return true;
        default: return false;
    }
}

int gguf_quant_block_size(GGUFTensorType type) {
    switch ((int)type) {
        case GGUF_TENSOR_Q4_0: case GGUF_TENSOR_Q4_1: case GGUF_TENSOR_Q8_0: return 32;
        case GGUF_TENSOR_Q4_K: case GGUF_TENSOR_Q5_K: case GGUF_TENSOR_Q6_K: return 256;
        default: return 0;
    }
}

size_t gguf_quant_type_size(GGUFTensorType type) {
    switch ((int)type) {
        case GGUF_TENSOR_Q4_0: return 18;
        case GGUF_TENSOR_Q4_1: return 20;
        case GGUF_TENSOR_Q8_0: return 34;
        case GGUF_TENSOR_Q4_K: return 144;
        case GGUF_TENSOR_Q5_K: return 176;
        case GGUF_TENSOR_Q6_K: return 210;
        default: return 0;
    }
}

int gguf_dequantize(GGUFTensorType type, const void* src, float* dst, size_t numel) {
    if (!src || !dst || numel == 0) return -1;
    const int bs = gguf_quant_block_size(type);
    if (bs == 0 || numel % (size_t)bs != 0) return -1;
    const size_t in_bytes = numel / (size_t)bs * gguf_quant_type_size(type);
    void *d_in = NULL, *d_out = NULL;
    int rc = -1;
    if (CML_DEV_FAIL(cmlb200_malloc(&d_in, in_bytes), "gguf_dequantize")) goto done;
    if (CML_DEV_FAIL(cmlb200_malloc(&d_out, numel * 4), "gguf_dequantize")) goto done;
    if (CML_DEV_FAIL(cmlb200_memcpy_h2d(d_in, src, in_bytes, NULL), "gguf_dequantize")) goto done;
    if (CML_DEV_FAIL(cmlb200_gguf_dequantize((int)type, d_in, (float*)d_out, numel, NULL), "gguf_dequantize")) goto done;
    if (CML_DEV_FAIL(cmlb200_memcpy_d2h(dst, d_out, numel * 4, NULL), "gguf_dequantize")) goto done;
    if (CML_DEV_FAIL(cmlb200_stream_sync(NULL), "gguf_dequantize")) goto done;
    rc = 0;
done:
    cmlb200_free(d_in);
    cmlb200_free(d_out);
    return rc;
}

static char* read_string(FILE* f) {
    uint64_t len;
    if (fread(&len, 8, 1, f) != 1 || len > 65536) return NULL;       /* same bound as gguf.c:61 */
    char* s = (char*)malloc((size_t)len + 1);
    if (!s) return NULL;
    if (len && fread(s, 1, (size_t)len, f) != len) { free(s); return NULL; }
    s[len] = 0;
    return s;
}

static int skip_value(FILE* f, uint32_t type) {
    static const int sizes[] = {1, 1, 2, 2, 4, 4, 4, 1, -1, -2, 8, 8, 8};
    if (type > 12) return -1;
    const int sz = sizes[type];
    if (sz > 0) return fseek(f, sz, SEEK_CUR);
    if (sz == -1) { char* s = read_string(f); if (!s) return -1; free(s); return 0; }
    uint32_t et;
    uint64_t n;
    if (fread(&et, 4, 1, f) != 1 || fread(&n, 8, 1, f) != 1) return -1;
    for (uint64_t i = 0; i < n; i++) if (skip_value(f, et)) return -1;
    return 0;
}

static DType gguf_dtype(GGUFTensorType t) {
    switch ((int)t) {
        case GGUF_TENSOR_F16: return DTYPE_FLOAT16;
        case GGUF_TENSOR_I8: return DTYPE_INT8;
        case GGUF_TENSOR_I16: return DTYPE_INT16;
        case GGUF_TENSOR_I32: return DTYPE_INT32;
        default: return DTYPE_FLOAT32;
    }
}

GGUFContext* gguf_open_read(const char* filepath) {
    if (!filepath) { LOG_ERROR("gguf_open_read: NULL path"); return NULL; }
    FILE* f = fopen(filepath, "rb");
    if (!f) { LOG_ERROR("gguf_open_read: cannot open %s", filepath); return NULL; }
    uint32_t magic = 0, version = 0;
    uint64_t nt = 0, nkv = 0;
    if (fread(&magic, 4, 1, f) != 1 || magic != GGUF_MAGIC) { LOG_ERROR("gguf_open_read: invalid GGUF magic"); fclose(f); return NULL; }
    if (fread(&version, 4, 1, f) != 1 || fread(&nt, 8, 1, f) != 1 || fread(&nkv, 8, 1, f) != 1 || nt > (1u << 24)) {
        LOG_ERROR("gguf_open_read: truncated header");
        fclose(f);
        return NULL;
    }
    GGUFContext* ctx = (GGUFContext*)calloc(1, sizeof *ctx);
    if (!ctx) { fclose(f); return NULL; }
    ctx->file = f;
    for (uint64_t i = 0; i < nkv; i++) {
        char* key = read_string(f);
        uint32_t vt;
        if (!key || fread(&vt, 4, 1, f) != 1 || skip_value(f, vt)) {
            free(key);
            LOG_ERROR("gguf_open_read: malformed metadata entry %llu", (unsigned long long)i);
            gguf_close(ctx);
            return NULL;
        }
        free(key);
    }
    ctx->tensors = (GGUFTensorInfo*)calloc(nt ? (size_t)nt : 1, sizeof(GGUFTensorInfo));
    if (!ctx->tensors) { gguf_close(ctx); return NULL; }
    for (uint64_t i = 0; i < nt; i++) {
        GGUFTensorInfo* ti = &ctx->tensors[i];
        uint32_t nd = 0, ty = 0;
        ti->name = read_string(f);
        if (!ti->name || fread(&nd, 4, 1, f) != 1 || nd > 8) goto bad;
        ti->ndim = (int)nd;
        size_t numel = 1;
        for (uint32_t d = 0; d < nd; d++) {
            uint64_t dim;
            if (fread(&dim, 8, 1, f) != 1) goto bad;
            ti->shape[d] = (int64_t)dim;
            numel *= (size_t)dim;
        }
        if (fread(&ty, 4, 1, f) != 1 || fread(&ti->offset, 8, 1, f) != 1) goto bad;
        ti->type = (GGUFTensorType)ty;
        if (gguf_type_is_quantized(ti->type)) {
            const size_t bs = (size_t)gguf_quant_block_size(ti->type);
            ti->data_size = (numel + bs - 1) / bs * gguf_quant_type_size(ti->type);
        } else {
            ti->data_size = numel * cml_dtype_size(gguf_dtype(ti->type));
        }
        ctx->num_tensors = (int)i + 1;
        continue;
    bad:
        LOG_ERROR("gguf_open_read: truncated tensor info %llu", (unsigned long long)i);
        ctx->num_tensors = (int)i + (ti->name ? 1 : 0);
        gguf_close(ctx);
        return NULL;
    }
    const long pos = ftell(f);
    ctx->data_offset = (uint64_t)((pos + 31) & ~31L);
    return ctx;
}

void gguf_close(GGUFContext* ctx) {
    if (!ctx) return;
    if (ctx->tensors) {
        for (int i = 0; i < ctx->num_tensors; i++) free(ctx->tensors[i].name);
        free(ctx->tensors);
    }
    if (ctx->file) fclose(ctx->file);
    free(ctx);
}

int gguf_get_num_tensors(GGUFContext* ctx) { return ctx ? ctx->num_tensors : 0; }

const char* gguf_get_tensor_name(GGUFContext* ctx, int index) {
    if (!ctx || index < 0 || index >= ctx->num_tensors) return NULL;
    return ctx->tensors[index].name;
}

const GGUFTensorInfo* cml_gguf_find(GGUFContext* ctx, const char* name) {
    if (!ctx || !name) return NULL;
    for (int i = 0; i < ctx->num_tensors; i++)
        if (ctx->tensors[i].name && strcmp(ctx->tensors[i].name, name) == 0) return &ctx->tensors[i];
    return NULL;
}

void* cml_gguf_read_raw(GGUFContext* ctx, const GGUFTensorInfo* info) {
    if (!ctx || !info) return NULL;
    void* raw = malloc(info->data_size ? info->data_size : 1);
    if (!raw) { LOG_ERROR("gguf: allocation of %zu bytes failed", info->data_size); return NULL; }
    if (fseek(ctx->file, (long)(ctx->data_offset + info->offset), SEEK_SET) != 0 ||
        fread(raw, 1, info->data_size, ctx->file) != info->data_size) {
        LOG_ERROR("gguf: short read of tensor '%s'", info->name);
        free(raw);
        return NULL;
    }
    return raw;
}

Tensor* gguf_read_tensor(GGUFContext* ctx, const char* name) {
    const GGUFTensorInfo* info = cml_gguf_find(ctx, name);
    if (!info) return NULL;
    int shape[8];
    size_t numel = 1;
    for (int d = 0; d < info->ndim; d++) { shape[d] = (int)info->shape[d]; numel *= (size_t)info->shape[d]; }
    void* raw = cml_gguf_read_raw(ctx, info);
    if (!raw) return NULL;
    Tensor* t = NULL;
    if (gguf_type_is_quantized(info->type)) {
        t = cml_tensor_alloc(DTYPE_FLOAT32, shape, info->ndim, false);
        if (t && gguf_dequantize(info->type, raw, (float*)t->data, numel) != 0) { tensor_free(t); t = NULL; }
    } else {
        t = cml_tensor_alloc(gguf_dtype(info->type), shape, info->ndim, false);
        if (t) memcpy(t->data, raw, info->data_size);
    }
    free(raw);
    return t;
}
