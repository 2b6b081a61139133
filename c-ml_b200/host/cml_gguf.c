/*
 * GGUF v3 reader and the block-type helpers (C-ML: src/core/gguf.c:105-310,
 * src/core/gguf_quant.c:313-391). The file format handling is host work; dequantisation runs on
 * the device. Layout read: magic, version, n_tensors, n_kv, the key/values, the tensor infos
 * (name, ndim, dims, type, offset) and data at align32(end of infos) + offset. C-ML steps over the
 * key/values (src/core/gguf.c:75-103); here they are kept, so that a file's tokenizer and
 * hyper-parameters can be used (gguf_get_metadata_*, gguf_create_tokenizer,
 * cml_llama_config_from_gguf). A malformed entry fails the open exactly where C-ML's skip would.
 * The writer (src/core/gguf.c:47-56, 181-232, 312-340) collects tensors and emits the file on
 * gguf_close with C-ML's layout byte for byte: header with zero key/values, the infos, zero padding to
 * a multiple of 32, then the tensors' bytes back to back. Beyond C-ML it can also carry key/values
 * and block-quantized tensors, so a complete model file can be produced from C.
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>

#include "cml_internal.h"

/* One key/value. Scalars sit in `bits` as read; a string in `str`; an array of scalars packed in
 * `data`, an array of strings in `strs`; an array of arrays is stepped over (count kept, no data). */
typedef struct GGUFMeta {
    char* key;
    uint32_t type, elem_type;
    uint64_t count;
    uint64_t bits;
    char* str;
    void* data;
    char** strs;
} GGUFMeta;

/* write mode: a tensor waiting for gguf_close, and serialized key/values */
typedef struct GGUFPending {
    char* name;
    int ndim;
    uint64_t shape[8];
    uint32_t type;
    void* data;
    size_t bytes;
} GGUFPending;

struct GGUFContext {
    FILE* file;
    int num_tensors;
    GGUFTensorInfo* tensors;
    uint64_t data_offset;
    int num_meta;
    GGUFMeta* meta;
    /* write mode */
    char* write_path;
    GGUFPending* pending;
    int num_pending, cap_pending;
    unsigned char* kv_bytes;
    size_t kv_size, kv_cap;
    uint64_t num_kv;
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

/* Bytes between the read position and the end of the file. Counts read from the file are checked
 * against it before anything is allocated or looped over: `count` items of at least `each` bytes. */
static uint64_t bytes_left(FILE* f) {
    struct stat sb;
    const long pos = ftell(f);
    if (pos < 0 || fstat(fileno(f), &sb) != 0 || sb.st_size < pos) return 0;
    return (uint64_t)(sb.st_size - pos);
}
static int fits(FILE* f, uint64_t count, uint64_t each) { return count <= bytes_left(f) / each; }

static int skip_value(FILE* f, uint32_t type) {
    static const int sizes[] = {1, 1, 2, 2, 4, 4, 4, 1, -1, -2, 8, 8, 8};
    if (type > 12) return -1;
    const int sz = sizes[type];
    if (sz > 0) return fits(f, 1, (uint64_t)sz) ? fseek(f, sz, SEEK_CUR) : -1;
    if (sz == -1) { char* s = read_string(f); if (!s) return -1; free(s); return 0; }
    uint32_t et;
    uint64_t n;
    if (fread(&et, 4, 1, f) != 1 || fread(&n, 8, 1, f) != 1 || et > 12) return -1;
    if (sizes[et] > 0) return fits(f, n, (uint64_t)sizes[et]) ? fseek(f, (long)(n * (uint64_t)sizes[et]), SEEK_CUR) : -1;
    if (!fits(f, n, sizes[et] == -1 ? 8 : 12)) return -1;           /* a string is at least its length field, an array its header */
    for (uint64_t i = 0; i < n; i++) if (skip_value(f, et)) return -1;
    return 0;
}

static const int kMetaSize[] = {1, 1, 2, 2, 4, 4, 4, 1, -1, -2, 8, 8, 8};     /* bytes of a scalar of each GGUF value type */

static void meta_release(GGUFMeta* m) {
    free(m->key);
    free(m->str);
    free(m->data);
    if (m->strs) {
        for (uint64_t i = 0; i < m->count; i++) free(m->strs[i]);
        free(m->strs);
    }
    memset(m, 0, sizeof *m);
}

/* The value of type m->type at the file position; 0 when it was read (or stepped over) whole. */
static int read_meta_value(FILE* f, GGUFMeta* m) {
    if (m->type > 12) return -1;
    const int sz = kMetaSize[m->type];
    if (sz > 0) return fread(&m->bits, (size_t)sz, 1, f) == 1 ? 0 : -1;
    if (sz == -1) return (m->str = read_string(f)) ? 0 : -1;
    if (fread(&m->elem_type, 4, 1, f) != 1 || fread(&m->count, 8, 1, f) != 1 || m->elem_type > 12) return -1;
    const int esz = kMetaSize[m->elem_type];
    if (esz > 0) {
        if (!fits(f, m->count, (uint64_t)esz)) return -1;
        m->data = malloc(m->count ? (size_t)m->count * (size_t)esz : 1);
        return m->data && fread(m->data, (size_t)esz, (size_t)m->count, f) == m->count ? 0 : -1;
    }
    if (esz == -1) {
        if (!fits(f, m->count, 8)) return -1;
        m->strs = (char**)calloc(m->count ? (size_t)m->count : 1, sizeof(char*));
        if (!m->strs) return -1;
        for (uint64_t i = 0; i < m->count; i++)
            if (!(m->strs[i] = read_string(f))) { m->count = i; return -1; }
        return 0;
    }
    if (!fits(f, m->count, 12)) return -1;
    for (uint64_t i = 0; i < m->count; i++)
        if (skip_value(f, 9)) return -1;
    return 0;
}

static const GGUFMeta* meta_find(GGUFContext* ctx, const char* key) {
    if (!ctx || !key) return NULL;
    for (int i = 0; i < ctx->num_meta; i++)
        if (strcmp(ctx->meta[i].key, key) == 0) return &ctx->meta[i];
    return NULL;
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
    /* an entry is at least a key length, a type and one byte; a tensor info a name length, ndim, type and offset */
    if (!fits(f, nkv, 13) || !fits(f, nt, 24) || !(ctx->meta = (GGUFMeta*)calloc(nkv ? (size_t)nkv : 1, sizeof(GGUFMeta)))) {
        LOG_ERROR("gguf_open_read: the header counts (%llu key/values, %llu tensors) exceed the file", (unsigned long long)nkv, (unsigned long long)nt);
        gguf_close(ctx);
        return NULL;
    }
    for (uint64_t i = 0; i < nkv; i++) {
        GGUFMeta* m = &ctx->meta[i];
        ctx->num_meta = (int)i + 1;
        if (!(m->key = read_string(f)) || fread(&m->type, 4, 1, f) != 1 || read_meta_value(f, m)) {
            LOG_ERROR("gguf_open_read: malformed metadata entry %llu", (unsigned long long)i);
            gguf_close(ctx);
            return NULL;
        }
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
            if (dim > 0 && numel > ((size_t)1 << 48) / (size_t)(dim > ((uint64_t)1 << 48) ? ((uint64_t)1 << 48) : dim)) goto bad;   /* more elements than any file holds */
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

static void write_flush(GGUFContext* ctx);

void gguf_close(GGUFContext* ctx) {
    if (!ctx) return;
    if (ctx->write_path) {
        write_flush(ctx);
        for (int i = 0; i < ctx->num_pending; i++) { free(ctx->pending[i].name); free(ctx->pending[i].data); }
        free(ctx->pending);
        free(ctx->kv_bytes);
        free(ctx->write_path);
    }
    if (ctx->tensors) {
        for (int i = 0; i < ctx->num_tensors; i++) free(ctx->tensors[i].name);
        free(ctx->tensors);
    }
    if (ctx->meta) {
        for (int i = 0; i < ctx->num_meta; i++) meta_release(&ctx->meta[i]);
        free(ctx->meta);
    }
    if (ctx->file) fclose(ctx->file);
    free(ctx);
}

/* ---- key/value metadata ------------------------------------------------------------------------ */
int gguf_get_num_metadata(GGUFContext* ctx) { return ctx ? ctx->num_meta : 0; }

const char* gguf_get_metadata_key(GGUFContext* ctx, int index) {
    return ctx && index >= 0 && index < ctx->num_meta ? ctx->meta[index].key : NULL;
}

int gguf_get_metadata_type(GGUFContext* ctx, const char* key) {
    const GGUFMeta* m = meta_find(ctx, key);
    return m ? (int)m->type : -1;
}

static int scalar_as_int(uint32_t type, const void* p, int64_t* out) {
    switch (type) {
        case 0: case 7: *out = *(const uint8_t*)p; return 0;
        case 1: *out = *(const int8_t*)p; return 0;
        case 2: { uint16_t v; memcpy(&v, p, 2); *out = v; return 0; }
        case 3: { int16_t v; memcpy(&v, p, 2); *out = v; return 0; }
        case 4: { uint32_t v; memcpy(&v, p, 4); *out = v; return 0; }
        case 5: { int32_t v; memcpy(&v, p, 4); *out = v; return 0; }
        case 10: { uint64_t v; memcpy(&v, p, 8); *out = (int64_t)v; return 0; }
        case 11: memcpy(out, p, 8); return 0;
        default: return -1;
    }
}

int gguf_get_metadata_int(GGUFContext* ctx, const char* key, int64_t* out) {
    const GGUFMeta* m = meta_find(ctx, key);
    return m && out ? scalar_as_int(m->type, &m->bits, out) : -1;
}

int gguf_get_metadata_float(GGUFContext* ctx, const char* key, double* out) {
    const GGUFMeta* m = meta_find(ctx, key);
    if (!m || !out) return -1;
    if (m->type == 6) { float v; memcpy(&v, &m->bits, 4); *out = v; return 0; }
    if (m->type == 12) { memcpy(out, &m->bits, 8); return 0; }
    int64_t i;
    if (scalar_as_int(m->type, &m->bits, &i)) return -1;
    *out = (double)i;
    return 0;
}

const char* gguf_get_metadata_string(GGUFContext* ctx, const char* key) {
    const GGUFMeta* m = meta_find(ctx, key);
    return m && m->type == 8 ? m->str : NULL;
}

int64_t gguf_get_metadata_array_length(GGUFContext* ctx, const char* key, int* elem_type) {
    const GGUFMeta* m = meta_find(ctx, key);
    if (!m || m->type != 9) return -1;
    if (elem_type) *elem_type = (int)m->elem_type;
    return (int64_t)m->count;
}

const char* gguf_get_metadata_array_string(GGUFContext* ctx, const char* key, int64_t index) {
    const GGUFMeta* m = meta_find(ctx, key);
    return m && m->type == 9 && m->strs && index >= 0 && (uint64_t)index < m->count ? m->strs[index] : NULL;
}

const void* gguf_get_metadata_array_data(GGUFContext* ctx, const char* key) {
    const GGUFMeta* m = meta_find(ctx, key);
    return m && m->type == 9 ? m->data : NULL;
}

CMLTokenizer* gguf_create_tokenizer(GGUFContext* ctx) {
    const GGUFMeta* toks = meta_find(ctx, "tokenizer.ggml.tokens");
    if (!toks || toks->type != 9 || !toks->strs || toks->count == 0 || toks->count > 0x7fffffffu) return NULL;
    const GGUFMeta* mg = meta_find(ctx, "tokenizer.ggml.merges");
    const int nm = mg && mg->type == 9 && mg->strs && mg->count <= 0x7fffffffu ? (int)mg->count : 0;
    char** pairs = nm ? (char**)calloc((size_t)nm, sizeof(char*)) : NULL;
    for (int i = 0; pairs && i < nm; i++) {
        /* "left right" -> "leftright": the separator is the first space after the first byte (a
         * left part may itself be a space) */
        const char* s = mg->strs[i];
        const size_t n = strlen(s);
        const char* sp = n > 1 ? strchr(s + 1, ' ') : NULL;
        if (!(pairs[i] = (char*)malloc(n + 1))) continue;
        if (sp) { memcpy(pairs[i], s, (size_t)(sp - s)); strcpy(pairs[i] + (sp - s), sp + 1); }
        else strcpy(pairs[i], s);
    }
    CMLTokenizer* tok = cml_tokenizer_create(toks->strs, (int)toks->count, pairs, pairs ? nm : 0);
    for (int i = 0; pairs && i < nm; i++) free(pairs[i]);
    free(pairs);
    if (!tok) return NULL;
    int64_t id[4] = {-1, -1, -1, -1};
    static const char* const keys[4] = {"tokenizer.ggml.bos_token_id", "tokenizer.ggml.eos_token_id", "tokenizer.ggml.padding_token_id",
                                        "tokenizer.ggml.unknown_token_id"};
    for (int k = 0; k < 4; k++)
        if (gguf_get_metadata_int(ctx, keys[k], &id[k])) id[k] = -1;
    cml_tokenizer_set_special(tok, (int)id[0], (int)id[1], (int)id[2], (int)id[3]);
    return tok;
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
    struct stat sb;
    if (fstat(fileno(ctx->file), &sb) != 0 || (uint64_t)sb.st_size < ctx->data_offset || info->offset > (uint64_t)sb.st_size - ctx->data_offset ||
        info->data_size > (uint64_t)sb.st_size - ctx->data_offset - info->offset) {
        LOG_ERROR("gguf: tensor '%s' reaches past the end of the file", info->name);
        return NULL;
    }
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

/* ---- writer ------------------------------------------------------------------------------------ */
#define GGUF_MAX_WRITE_TENSORS 4096          /* src/core/gguf.c:10 */

GGUFContext* gguf_open_write(const char* filepath) {
    if (!filepath) return NULL;
    GGUFContext* ctx = (GGUFContext*)calloc(1, sizeof *ctx);
    if (!ctx) return NULL;
    ctx->write_path = strdup(filepath);
    if (!ctx->write_path) { free(ctx); return NULL; }
    return ctx;
}

static uint32_t gguf_type_of(DType dtype) {      /* src/core/gguf.c:47-56: anything else is labelled F32 */
    switch (dtype) {
        case DTYPE_FLOAT16: return GGUF_TENSOR_F16;
        case DTYPE_INT8: return GGUF_TENSOR_I8;
        case DTYPE_INT16: return GGUF_TENSOR_I16;
        case DTYPE_INT32: return GGUF_TENSOR_I32;
        default: return GGUF_TENSOR_F32;
    }
}

static int write_add(GGUFContext* ctx, const char* name, uint32_t type, const int64_t* shape, int ndim, const void* data, size_t bytes) {
    if (!ctx || !ctx->write_path || !name || !data || ndim < 0 || ndim > 8 || ctx->num_pending >= GGUF_MAX_WRITE_TENSORS) return -1;
    if (ctx->num_pending == ctx->cap_pending) {
        const int cap = ctx->cap_pending ? 2 * ctx->cap_pending : 16;
        GGUFPending* grown = (GGUFPending*)realloc(ctx->pending, (size_t)cap * sizeof *grown);
        if (!grown) return -1;
        ctx->pending = grown;
        ctx->cap_pending = cap;
    }
    GGUFPending* pt = &ctx->pending[ctx->num_pending];
    memset(pt, 0, sizeof *pt);
    pt->name = strdup(name);
    pt->data = malloc(bytes ? bytes : 1);
    if (!pt->name || !pt->data) { free(pt->name); free(pt->data); return -1; }
    memcpy(pt->data, data, bytes);
    pt->bytes = bytes;
    pt->type = type;
    pt->ndim = ndim;
    for (int d = 0; d < ndim; d++) pt->shape[d] = (uint64_t)shape[d];
    ctx->num_pending++;
    return 0;
}

int gguf_write_tensor(GGUFContext* ctx, const char* name, Tensor* tensor) {
    if (!ctx || !name || !tensor || !ctx->write_path || !tensor->data || tensor->ndim > 8) return -1;
    int64_t shape[8];
    for (int d = 0; d < tensor->ndim; d++) shape[d] = tensor->shape[d];
    return write_add(ctx, name, gguf_type_of(tensor->dtype), shape, tensor->ndim, tensor->data, tensor->numel * cml_dtype_size(tensor->dtype));
}

int gguf_write_blocks(GGUFContext* ctx, const char* name, GGUFTensorType type, const int64_t* shape, int ndim, const void* blocks) {
    if (!shape || ndim < 1 || ndim > 8 || !gguf_type_is_quantized(type)) return -1;
    uint64_t numel = 1;
    for (int d = 0; d < ndim; d++) {
        if (shape[d] <= 0) return -1;
        numel *= (uint64_t)shape[d];
    }
    const uint64_t bs = (uint64_t)gguf_quant_block_size(type);
    if (numel % bs) return -1;
    return write_add(ctx, name, (uint32_t)type, shape, ndim, blocks, (size_t)(numel / bs) * gguf_quant_type_size(type));
}

static int kv_append(GGUFContext* ctx, const void* src, size_t n) {
    if (ctx->kv_size + n > ctx->kv_cap) {
        size_t cap = ctx->kv_cap ? ctx->kv_cap : 256;
        while (cap < ctx->kv_size + n) cap *= 2;
        unsigned char* grown = (unsigned char*)realloc(ctx->kv_bytes, cap);
        if (!grown) return -1;
        ctx->kv_bytes = grown;
        ctx->kv_cap = cap;
    }
    memcpy(ctx->kv_bytes + ctx->kv_size, src, n);
    ctx->kv_size += n;
    return 0;
}
static int kv_append_string(GGUFContext* ctx, const char* s) {
    const uint64_t len = strlen(s);
    return len > 65536 || kv_append(ctx, &len, 8) || kv_append(ctx, s, (size_t)len) ? -1 : 0;   /* longer strings would not read back */
}

int gguf_write_metadata(GGUFContext* ctx, const char* key, int type, const void* value) {
    if (!ctx || !ctx->write_path || !key || !value || type < 0 || type > 12 || type == 9) return -1;
    const size_t mark = ctx->kv_size;
    const uint32_t t = (uint32_t)type;
    int rc = kv_append_string(ctx, key) || kv_append(ctx, &t, 4);
    if (!rc) rc = type == 8 ? kv_append_string(ctx, (const char*)value) : kv_append(ctx, value, (size_t)kMetaSize[type]);
    if (rc) { ctx->kv_size = mark; return -1; }
    ctx->num_kv++;
    return 0;
}

int gguf_write_metadata_array(GGUFContext* ctx, const char* key, int elem_type, const void* values, uint64_t count) {
    if (!ctx || !ctx->write_path || !key || (!values && count) || elem_type < 0 || elem_type > 12 || elem_type == 9) return -1;
    const size_t mark = ctx->kv_size;
    const uint32_t t = 9, et = (uint32_t)elem_type;
    int rc = kv_append_string(ctx, key) || kv_append(ctx, &t, 4) || kv_append(ctx, &et, 4) || kv_append(ctx, &count, 8);
    if (!rc && elem_type == 8) {
        const char* const* strs = (const char* const*)values;
        for (uint64_t i = 0; !rc && i < count; i++) rc = !strs[i] || kv_append_string(ctx, strs[i]);
    } else if (!rc) {
        rc = kv_append(ctx, values, (size_t)count * (size_t)kMetaSize[elem_type]);
    }
    if (rc) { ctx->kv_size = mark; return -1; }
    ctx->num_kv++;
    return 0;
}

/* Emits the file (nothing when no tensor was added, as src/core/gguf.c:184). */
static void write_flush(GGUFContext* ctx) {
    if (ctx->num_pending == 0) return;
    FILE* f = fopen(ctx->write_path, "wb");
    if (!f) { LOG_ERROR("gguf_close: cannot write %s", ctx->write_path); return; }
    const uint32_t magic = GGUF_MAGIC, version = 3;
    const uint64_t nt = (uint64_t)ctx->num_pending;
    fwrite(&magic, 4, 1, f);
    fwrite(&version, 4, 1, f);
    fwrite(&nt, 8, 1, f);
    fwrite(&ctx->num_kv, 8, 1, f);
    if (ctx->kv_size) fwrite(ctx->kv_bytes, 1, ctx->kv_size, f);
    uint64_t offset = 0;
    for (int i = 0; i < ctx->num_pending; i++) {
        const GGUFPending* pt = &ctx->pending[i];
        const uint64_t len = strlen(pt->name);
        const uint32_t nd = (uint32_t)pt->ndim;
        fwrite(&len, 8, 1, f);
        fwrite(pt->name, 1, (size_t)len, f);
        fwrite(&nd, 4, 1, f);
        for (int d = 0; d < pt->ndim; d++) fwrite(&pt->shape[d], 8, 1, f);
        fwrite(&pt->type, 4, 1, f);
        fwrite(&offset, 8, 1, f);
        offset += pt->bytes;                         /* back to back: C-ML's reader needs no per-tensor alignment */
    }
    static const unsigned char zeros[32] = {0};
    const long pos = ftell(f);
    fwrite(zeros, 1, (size_t)(((pos + 31) & ~31L) - pos), f);
    for (int i = 0; i < ctx->num_pending; i++) fwrite(ctx->pending[i].data, 1, ctx->pending[i].bytes, f);
    if (fclose(f) != 0) LOG_ERROR("gguf_close: short write to %s", ctx->write_path);
}
