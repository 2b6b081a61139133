/* C-ML's paged KV cache and paged grouped-query attention (include/nn/paged_attention.h:14-80,
 * src/nn/paged_attention.c) with the attention on the device.
 *
 * The bookkeeping (block pool with a stack free list, per-sequence block tables, statistics) is
 * host code with C-ML's struct layouts and return values, so callers that read free_count,
 * block_ids or a block's key_data keep working. Every block's key_data / value_data is a slice of
 * one host pool; the same pool exists once on the device ([blocks][16][kv_heads * head_dim] per K and
 * V, allocated at the first forward call), and a forward call first uploads the tokens appended
 * since the previous one (whole slot ranges per block), then launches cmlb200_paged_gqa_f32 with
 * the sequence's block table. Tokens must be written through cml_paged_cache_append. */
#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

#include "cml_internal.h"

#define FAIL(call, who) CML_DEV_FAIL(call, who)

/* Device side of a cache, found by the cache's address (the public struct has no room for it). */
typedef struct PagedDev {
    const CMLPagedKVCache* key;
    float *h_k, *h_v;                 /* host pools the blocks' key_data / value_data point into */
    void *d_k, *d_v;                  /* device pools, NULL until the first forward call */
    int* dev_tokens;                  /* per block: slots already uploaded since it was allocated */
    void *d_ids, *d_q, *d_o;          /* scratch, grown on demand */
    size_t ids_cap, q_cap, o_cap;
    struct PagedDev* next;
} PagedDev;

static PagedDev* g_paged = NULL;
static pthread_mutex_t g_paged_mu = PTHREAD_MUTEX_INITIALIZER;

static PagedDev* pd_find(const CMLPagedKVCache* c) {
    pthread_mutex_lock(&g_paged_mu);
    PagedDev* p = g_paged;
    while (p && p->key != c) p = p->next;
    pthread_mutex_unlock(&g_paged_mu);
    return p;
}

static size_t token_floats(const CMLPagedKVCache* c) { return (size_t)c->num_kv_heads * c->head_dim; }
static size_t block_floats(const CMLPagedKVCache* c) { return (size_t)c->block_size * token_floats(c); }

CMLPagedKVCache* cml_paged_kv_cache_create(int max_blocks, int max_sequences, int num_kv_heads, int head_dim) {
    if (max_blocks <= 0 || max_sequences <= 0 || num_kv_heads <= 0 || head_dim <= 0) {
        LOG_ERROR("cml_paged_kv_cache_create: invalid parameters (max_blocks=%d, max_sequences=%d, num_kv_heads=%d, head_dim=%d)",
                  max_blocks, max_sequences, num_kv_heads, head_dim);
        return NULL;
    }
    CMLPagedKVCache* c = (CMLPagedKVCache*)calloc(1, sizeof *c);
    PagedDev* p = (PagedDev*)calloc(1, sizeof *p);
    if (!c || !p) { LOG_ERROR("cml_paged_kv_cache_create: allocation failed"); free(c); free(p); return NULL; }
    c->max_blocks = c->num_blocks = max_blocks;
    c->max_sequences = max_sequences;
    c->num_kv_heads = num_kv_heads;
    c->head_dim = head_dim;
    c->block_size = CML_PAGE_BLOCK_SIZE;
    const size_t bf = block_floats(c);
    c->blocks = (CMLPageBlock*)calloc((size_t)max_blocks, sizeof(CMLPageBlock));
    c->free_list = (int*)malloc((size_t)max_blocks * sizeof(int));
    c->sequences = (CMLBlockTable*)calloc((size_t)max_sequences, sizeof(CMLBlockTable));
    p->h_k = (float*)calloc((size_t)max_blocks * bf, sizeof(float));
    p->h_v = (float*)calloc((size_t)max_blocks * bf, sizeof(float));
    p->dev_tokens = (int*)calloc((size_t)max_blocks, sizeof(int));
    if (!c->blocks || !c->free_list || !c->sequences || !p->h_k || !p->h_v || !p->dev_tokens) {
        LOG_ERROR("cml_paged_kv_cache_create: allocation failed");
        free(c->blocks); free(c->free_list); free(c->sequences); free(p->h_k); free(p->h_v); free(p->dev_tokens); free(c); free(p);
        return NULL;
    }
    for (int i = 0; i < max_blocks; i++) {
        c->blocks[i].key_data = p->h_k + (size_t)i * bf;
        c->blocks[i].value_data = p->h_v + (size_t)i * bf;
        c->blocks[i].block_id = i;
        c->free_list[i] = i;                               /* top of the stack = last element */
    }
    c->free_count = max_blocks;
    p->key = c;
    pthread_mutex_lock(&g_paged_mu);
    p->next = g_paged;
    g_paged = p;
    pthread_mutex_unlock(&g_paged_mu);
    return c;
}

void cml_paged_kv_cache_free(CMLPagedKVCache* cache) {
    if (!cache) return;
    pthread_mutex_lock(&g_paged_mu);
    PagedDev** pp = &g_paged;
    while (*pp && (*pp)->key != cache) pp = &(*pp)->next;
    PagedDev* p = *pp;
    if (p) *pp = p->next;
    pthread_mutex_unlock(&g_paged_mu);
    if (p) {
        cmlb200_free(p->d_k); cmlb200_free(p->d_v); cmlb200_free(p->d_ids); cmlb200_free(p->d_q); cmlb200_free(p->d_o);
        free(p->h_k); free(p->h_v); free(p->dev_tokens); free(p);
    }
    if (cache->sequences) {
        for (int i = 0; i < cache->max_sequences; i++) free(cache->sequences[i].block_ids);
        free(cache->sequences);
    }
    free(cache->blocks);
    free(cache->free_list);
    free(cache);
}

int cml_paged_cache_alloc_block(CMLPagedKVCache* cache) {
    if (!cache) { LOG_ERROR("cml_paged_cache_alloc_block: NULL cache"); return -1; }
    if (cache->free_count <= 0) { LOG_ERROR("cml_paged_cache_alloc_block: no free blocks"); return -1; }
    const int id = cache->free_list[--cache->free_count];
    CMLPageBlock* b = &cache->blocks[id];
    b->in_use = true;
    b->num_tokens = 0;
    memset(b->key_data, 0, block_floats(cache) * sizeof(float));
    memset(b->value_data, 0, block_floats(cache) * sizeof(float));
    PagedDev* p = pd_find(cache);
    if (p) p->dev_tokens[id] = 0;                          /* nothing of the new owner's tokens is on the device yet */
    cache->total_allocated++;
    return id;
}

void cml_paged_cache_free_block(CMLPagedKVCache* cache, int block_id) {
    if (!cache) { LOG_ERROR("cml_paged_cache_free_block: NULL cache"); return; }
    if (block_id < 0 || block_id >= cache->num_blocks) { LOG_ERROR("cml_paged_cache_free_block: invalid block_id %d", block_id); return; }
    if (!cache->blocks[block_id].in_use) { LOG_WARNING("cml_paged_cache_free_block: block %d already free", block_id); return; }
    cache->blocks[block_id].in_use = false;
    cache->blocks[block_id].num_tokens = 0;
    cache->free_list[cache->free_count++] = block_id;
    cache->total_freed++;
}

int cml_paged_cache_init_sequence(CMLPagedKVCache* cache) {
    if (!cache) { LOG_ERROR("cml_paged_cache_init_sequence: NULL cache"); return -1; }
    int id = -1;
    for (int i = 0; i < cache->max_sequences && id < 0; i++) if (!cache->sequences[i].block_ids) id = i;
    if (id < 0) { LOG_ERROR("cml_paged_cache_init_sequence: no free sequence slots (max=%d)", cache->max_sequences); return -1; }
    CMLBlockTable* bt = &cache->sequences[id];
    bt->block_ids = (int*)malloc(8 * sizeof(int));
    if (!bt->block_ids) { LOG_ERROR("cml_paged_cache_init_sequence: allocation failed"); return -1; }
    bt->num_blocks = 0;
    bt->capacity = 8;
    bt->seq_len = 0;
    cache->num_sequences++;
    return id;
}

void cml_paged_cache_free_sequence(CMLPagedKVCache* cache, int seq_id) {
    if (!cache) { LOG_ERROR("cml_paged_cache_free_sequence: NULL cache"); return; }
    if (seq_id < 0 || seq_id >= cache->max_sequences) { LOG_ERROR("cml_paged_cache_free_sequence: invalid seq_id %d", seq_id); return; }
    CMLBlockTable* bt = &cache->sequences[seq_id];
    if (!bt->block_ids) { LOG_WARNING("cml_paged_cache_free_sequence: sequence %d not initialised", seq_id); return; }
    for (int i = 0; i < bt->num_blocks; i++) cml_paged_cache_free_block(cache, bt->block_ids[i]);
    free(bt->block_ids);
    bt->block_ids = NULL;
    bt->num_blocks = bt->capacity = bt->seq_len = 0;
    cache->num_sequences--;
}

int cml_paged_cache_append(CMLPagedKVCache* cache, int seq_id, const float* key, const float* value) {
    if (!cache || !key || !value) { LOG_ERROR("cml_paged_cache_append: NULL argument"); return -1; }
    if (seq_id < 0 || seq_id >= cache->max_sequences) { LOG_ERROR("cml_paged_cache_append: invalid seq_id %d", seq_id); return -1; }
    CMLBlockTable* bt = &cache->sequences[seq_id];
    if (!bt->block_ids) { LOG_ERROR("cml_paged_cache_append: sequence %d not initialised", seq_id); return -1; }
    if (bt->num_blocks == 0 || cache->blocks[bt->block_ids[bt->num_blocks - 1]].num_tokens >= cache->block_size) {
        const int nb = cml_paged_cache_alloc_block(cache);
        if (nb < 0) { LOG_ERROR("cml_paged_cache_append: failed to allocate new block for seq %d", seq_id); return -1; }
        if (bt->num_blocks >= bt->capacity) {
            int* ids = (int*)realloc(bt->block_ids, (size_t)bt->capacity * 2 * sizeof(int));
            if (!ids) { LOG_ERROR("cml_paged_cache_append: block table realloc failed"); cml_paged_cache_free_block(cache, nb); return -1; }
            bt->block_ids = ids;
            bt->capacity *= 2;
        }
        bt->block_ids[bt->num_blocks++] = nb;
    }
    CMLPageBlock* b = &cache->blocks[bt->block_ids[bt->num_blocks - 1]];
    const size_t tf = token_floats(cache), off = (size_t)b->num_tokens * tf;
    memcpy(b->key_data + off, key, tf * sizeof(float));
    memcpy(b->value_data + off, value, tf * sizeof(float));
    b->num_tokens++;
    bt->seq_len++;
    return 0;
}

static int grow(void** d_ptr, size_t* cap, size_t bytes, const char* who) {
    if (bytes <= *cap) return 0;
    cmlb200_free(*d_ptr);
    *d_ptr = NULL;
    *cap = 0;
    if (FAIL(cmlb200_malloc(d_ptr, bytes), who)) return -1;
    *cap = bytes;
    return 0;
}

Tensor* cml_paged_gqa_forward(CMLPagedKVCache* cache, int seq_id, Tensor* Q, const CMLGQAConfig* config) {
    static const char* who = "cml_paged_gqa_forward";
    if (!cache || !Q || !config) { LOG_ERROR("%s: NULL argument", who); return NULL; }
    if (seq_id < 0 || seq_id >= cache->max_sequences) { LOG_ERROR("%s: invalid seq_id %d", who, seq_id); return NULL; }
    CMLBlockTable* bt = &cache->sequences[seq_id];
    if (!bt->block_ids) { LOG_ERROR("%s: sequence %d not initialised", who, seq_id); return NULL; }
    if (Q->ndim != 3) { LOG_ERROR("%s: Q must be 3D [batch, seq_len, num_heads*head_dim], got ndim=%d", who, Q->ndim); return NULL; }
    const int H = config->num_heads, KH = config->num_kv_heads, D = config->head_dim;
    if (H <= 0 || KH <= 0 || D <= 0) { LOG_ERROR("%s: invalid config (num_heads=%d, kv_heads=%d, head_dim=%d)", who, H, KH, D); return NULL; }
    if (H % KH != 0) { LOG_ERROR("%s: num_heads (%d) must be divisible by num_kv_heads (%d)", who, H, KH); return NULL; }
    if (KH != cache->num_kv_heads || D != cache->head_dim) {
        LOG_ERROR("%s: config mismatch with cache (config kv_heads=%d vs cache %d, config head_dim=%d vs cache %d)", who, KH, cache->num_kv_heads,
                  D, cache->head_dim);
        return NULL;
    }
    const int seq_q = Q->shape[1], kv_len = bt->seq_len;
    if (Q->shape[0] != 1) { LOG_ERROR("%s: paged attention only supports batch=1, got %d", who, Q->shape[0]); return NULL; }
    if (kv_len == 0) { LOG_ERROR("%s: sequence %d has no cached tokens", who, seq_id); return NULL; }
    if (!Q->data || seq_q <= 0 || Q->shape[2] != H * D) { LOG_ERROR("%s: failed to get Q data pointer", who); return NULL; }
    float scale = config->scale;
    if (scale <= 0.0f) scale = 1.0f / sqrtf((float)D);
    PagedDev* p = pd_find(cache);
    if (!p) { LOG_ERROR("%s: the cache was not created by cml_paged_kv_cache_create", who); return NULL; }

    const size_t tf = token_floats(cache), bf = block_floats(cache), pool_bytes = (size_t)cache->num_blocks * bf * sizeof(float);
    if (!p->d_k && (FAIL(cmlb200_malloc(&p->d_k, pool_bytes), who) || FAIL(cmlb200_malloc(&p->d_v, pool_bytes), who))) {
        cmlb200_free(p->d_k); p->d_k = NULL;
        return NULL;
    }
    /* upload what was appended to this sequence's blocks since their last upload */
    for (int i = 0; i < bt->num_blocks; i++) {
        const int id = bt->block_ids[i], have = p->dev_tokens[id], want = cache->blocks[id].num_tokens;
        if (want > have) {
            const size_t off = (size_t)id * bf + (size_t)have * tf, bytes = (size_t)(want - have) * tf * sizeof(float);
            if (FAIL(cmlb200_memcpy_h2d((float*)p->d_k + off, p->h_k + off, bytes, NULL), who) ||
                FAIL(cmlb200_memcpy_h2d((float*)p->d_v + off, p->h_v + off, bytes, NULL), who))
                return NULL;
            p->dev_tokens[id] = want;
        }
    }
    const size_t qn = (size_t)seq_q * H * D;
    if (grow(&p->d_ids, &p->ids_cap, (size_t)bt->num_blocks * sizeof(int), who) || grow(&p->d_q, &p->q_cap, qn * 4, who) ||
        grow(&p->d_o, &p->o_cap, qn * 4, who))
        return NULL;
    int oshape[3] = {1, seq_q, H * D};
    Tensor* out = cml_tensor_alloc(DTYPE_FLOAT32, oshape, 3, false);
    int ok = out != NULL;
    ok = ok && !FAIL(cmlb200_memcpy_h2d(p->d_ids, bt->block_ids, (size_t)bt->num_blocks * sizeof(int), NULL), who) &&
         !FAIL(cmlb200_memcpy_h2d(p->d_q, Q->data, qn * 4, NULL), who) &&
         !FAIL(cmlb200_paged_gqa_f32((const float*)p->d_q, (const float*)p->d_k, (const float*)p->d_v, (const int*)p->d_ids, cache->block_size,
                                     seq_q, kv_len, H, KH, D, scale, config->causal ? 1 : 0, (float*)p->d_o, NULL), who) &&
         !FAIL(cmlb200_memcpy_d2h(out->data, p->d_o, qn * 4, NULL), who) && !FAIL(cmlb200_stream_sync(NULL), who);
    if (!ok) { tensor_free(out); LOG_ERROR("%s: failed to create output tensor", who); return NULL; }
    out->dtype = Q->dtype;
    out->device = Q->device;
    return out;
}
