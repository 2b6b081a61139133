/*
 * LLaMA inference entry points on the GPU (C-ML: src/nn/llama.c). The public structs and
 * functions keep C-ML's shape; the device-side state (packed weights, KV cache, activation
 * buffers, stream, CUDA graph, NCCL communicator) hangs off the model in a side table keyed
 * by the model's address, so the public struct layout is untouched.
 *
 * Forward pass per layer (src/nn/llama.c:454-548): RMSNorm -> Q/K/V projections -> RoPE ->
 * append K,V to the cache -> grouped-query attention over the cache -> output projection +
 * residual -> RMSNorm -> SwiGLU FFN -> down projection + residual. Up to 32 rows run the fp32
 * decode kernels (dequant-GEMV); longer prompts run the bf16 tcgen05 dequant-GEMM.
 *
 * Tensor parallelism (src/distributed/tensor_parallel.c): Q/K/V/gate/up are split by output
 * rows (column-parallel, whole heads per rank), O/down by input columns (row-parallel); the
 * partial outputs of the row-parallel projections are summed with an NCCL all-reduce.
 */
#include <math.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "cml_internal.h"

#define DEV(call) do { if (CML_DEV_FAIL((call), __func__)) return -1; } while (0)
#define SKINNY_ROWS 32
#define ATT_DECODE_CHUNK 32
#define ATT_CHUNK 64

typedef struct DevLayer {
    cmlb200_qmat wqkv, wo, wg, wu, wd;     /* Q, K and V rows are stacked into one matrix at load */
    void *n1, *n2;                         /* fp16 norm weights */
    uint8_t* pend[3];                      /* host blocks of q, k, v waiting for each other */
    int pend_type;
} DevLayer;

typedef struct DevModel {
    const CMLLLaMAModel* key;
    struct DevModel* next;
    int flags, max_batch, max_rows;
    int tp, rank, device;
    void* comm;
    /* peer-memory all-reduce for decode-sized rows: every rank's workspace as mapped here
     * (ar_ws[rank] is this rank's own allocation), NULL when only NCCL is available */
    void* ar_ws[8];
    size_t ar_max_floats;
    int ar_ok;
    /* the same for prompt-sized messages (second workspace, slices summed by rank); arb_ok only when
     * its start-up check passed on every rank and it was faster there than ncclAllReduce */
    void* arb_ws[8];
    size_t arb_max_floats;
    int arb_ok;
    float arb_ms[2];                       /* start-up timing of one sum: peer memory, ncclAllReduce + add */
    size_t arb_probe_floats;
    float* lineup;                         /* 4 zero floats for tp_line_up */
    int generic_w;                         /* some projection is Q4_1 / Q4_K / Q5_K / Q6_K: fp32 row-block path for every call */
    int hd, heads_l, kvh_l, qw_l, kvw_l, inter_l;
    DevLayer* L;
    void *embed, *fnorm;
    cmlb200_qmat lm_head;
    void *kc, *vc;                         /* [layers][n_seq][max_seq][kvw_l] */
    size_t kv_layer_elems;
    void* stream;
    int qkv_w;                             /* qw_l + 2 * kvw_l */
    float *h, *nrm, *qkv, *att, *ffn, *g, *u, *tmp, *logits, *att_scratch, *rope_cs;
    /* vocabulary projection split by rows over the ranks (vocab % tp == 0): this rank's slice of
     * the logits, the slices of all ranks as gathered, and the (value, index) pairs of the greedy pick */
    int vocab_l;
    float *logits_l, *logits_g, *pairs;
    uint16_t *b_a, *b_b, *b_c, *b_d;       /* bf16 staging of the prefill path */
    int *d_tokens, *d_cur, *row_seq, *row_pos, *row_limit, *d_hist;
    int* h_cur;
    int att_splits_cap;
    void* graph;
    int graph_batch, graph_splits;
} DevModel;

/* Side table of device state, keyed by the public model's address. The list itself is guarded
 * (threads may create and free different models concurrently); one model is still driven by one
 * thread at a time, as in C-ML. */
static DevModel* g_models = NULL;
static pthread_mutex_t g_models_mu = PTHREAD_MUTEX_INITIALIZER;

static DevModel* dm_find(const CMLLLaMAModel* m) {
    pthread_mutex_lock(&g_models_mu);
    DevModel* d = g_models;
    while (d && d->key != m) d = d->next;
    pthread_mutex_unlock(&g_models_mu);
    return d;
}

/* ---- configuration presets (src/nn/llama.c:14-69) ------------------------------------------- */
static CMLLLaMAConfig make_cfg(int hidden, int inter, int layers, int heads, int kv, int max_seq) {
    CMLLLaMAConfig c = {.vocab_size = 32000, .hidden_size = hidden, .intermediate_size = inter, .num_layers = layers,
                        .num_heads = heads, .num_kv_heads = kv, .max_seq_len = max_seq, .rope_theta = 10000.0f,
                        .rms_norm_eps = 1e-5f, .tensor_parallel_size = 0, .tensor_parallel_rank = 0};
    return c;
}
CMLLLaMAConfig cml_llama_config_7b(void) { return make_cfg(4096, 11008, 32, 32, 32, 2048); }
CMLLLaMAConfig cml_llama_config_13b(void) { return make_cfg(5120, 13824, 40, 40, 40, 2048); }
CMLLLaMAConfig cml_llama_config_70b(void) { return make_cfg(8192, 28672, 80, 64, 8, 4096); }

CMLGenerationConfig cml_generation_default_config(void) {
    CMLGenerationConfig c = {.temperature = 0.8f, .top_p = 0.9f, .top_k = 40, .max_new_tokens = 256, .eos_token_id = 2, .do_sample = true};
    return c;
}

/* ---- create / free ---------------------------------------------------------------------------- */
CMLLLaMAModel* cml_llama_create(const CMLLLaMAConfig* config) {
    if (!config) { LOG_ERROR("cml_llama_create: NULL config"); return NULL; }
    if (config->num_layers <= 0 || config->num_heads <= 0 || config->num_kv_heads <= 0 || config->hidden_size <= 0 ||
        config->max_seq_len <= 0 || config->hidden_size % config->num_heads || config->num_heads % config->num_kv_heads) {
        LOG_ERROR("cml_llama_create: invalid configuration");
        return NULL;
    }
    CMLLLaMAModel* m = (CMLLLaMAModel*)calloc(1, sizeof *m);
    if (!m) { LOG_ERROR("cml_llama_create: allocation failed"); return NULL; }
    m->config = *config;
    m->num_layers = config->num_layers;
    m->layers = (CMLLLaMALayer**)calloc((size_t)config->num_layers, sizeof(CMLLLaMALayer*));
    if (!m->layers) { free(m); return NULL; }
    for (int i = 0; i < config->num_layers; i++) {
        m->layers[i] = (CMLLLaMALayer*)calloc(1, sizeof(CMLLLaMALayer));
        CMLKVCache* kv = m->layers[i] ? (CMLKVCache*)calloc(1, sizeof(CMLKVCache)) : NULL;
        if (!kv) { LOG_ERROR("cml_llama_create: layer %d creation failed", i); cml_llama_free(m); return NULL; }
        kv->max_seq_len = config->max_seq_len;
        kv->num_kv_heads = config->num_kv_heads;
        kv->head_dim = config->hidden_size / config->num_heads;
        m->layers[i]->kv_cache = kv;
    }
    LOG_INFO("LLaMA model created: %d layers, hidden=%d, heads=%d, kv_heads=%d", config->num_layers, config->hidden_size,
             config->num_heads, config->num_kv_heads);
    return m;
}

static void qmat_free(cmlb200_qmat* w) {
    cmlb200_free(w->qs);
    cmlb200_free(w->scales);
    cmlb200_free(w->tiles);
    memset(w, 0, sizeof *w);
}

static void dm_destroy(DevModel* d) {
    if (!d) return;
    if (d->graph) cmlb200_graph_destroy(d->graph);
    if (d->L) {
        for (int i = 0; i < d->key->num_layers; i++) {
            DevLayer* l = &d->L[i];
            qmat_free(&l->wqkv); qmat_free(&l->wo);
            qmat_free(&l->wg); qmat_free(&l->wu); qmat_free(&l->wd);
            cmlb200_free(l->n1); cmlb200_free(l->n2);
            for (int k = 0; k < 3; k++) free(l->pend[k]);
        }
        free(d->L);
    }
    qmat_free(&d->lm_head);
    void* bufs[] = {d->embed, d->fnorm, d->kc, d->vc, d->h, d->nrm, d->qkv, d->att, d->ffn, d->g, d->u, d->tmp,
                    d->logits, d->logits_l, d->logits_g, d->pairs, d->att_scratch, d->rope_cs, d->b_a, d->b_b, d->b_c, d->b_d, d->d_tokens, d->d_cur, d->row_seq,
                    d->row_pos, d->row_limit, d->d_hist};
    for (size_t i = 0; i < sizeof bufs / sizeof bufs[0]; i++) cmlb200_free(bufs[i]);
    free(d->h_cur);
    for (int r = 0; r < 8; r++) {
        if (d->arb_ws[r]) { if (r == d->rank) cmlb200_free(d->arb_ws[r]); else cmlb200_ipc_close(d->arb_ws[r]); }
        if (!d->ar_ws[r]) continue;
        if (r == d->rank) cmlb200_free(d->ar_ws[r]);
        else cmlb200_ipc_close(d->ar_ws[r]);
    }
    cmlb200_free(d->lineup);
    if (d->comm) cml_nccl_destroy(d->comm);
    if (d->stream) cmlb200_stream_destroy(d->stream);
    free(d);
}

/* cml_tokenizer.c unless the caller installed its own pair (cml_llama_set_tokenizer_functions) */
static CMLTokenizerEncodeFn g_tok_encode = NULL;
static CMLTokenizerDecodeFn g_tok_decode = NULL;

void cml_llama_free(CMLLLaMAModel* model) {
    if (!model) return;
    DevModel* gone = NULL;
    pthread_mutex_lock(&g_models_mu);
    for (DevModel** pp = &g_models; *pp; pp = &(*pp)->next)
        if ((*pp)->key == model) { gone = *pp; *pp = gone->next; break; }
    pthread_mutex_unlock(&g_models_mu);
    dm_destroy(gone);
    if (model->layers) {
        for (int i = 0; i < model->num_layers; i++) {
            CMLLLaMALayer* l = model->layers[i];
            if (!l) continue;
            Tensor* ts[] = {l->q_proj, l->k_proj, l->v_proj, l->o_proj, l->gate_proj, l->up_proj, l->down_proj,
                            l->input_layernorm, l->post_attn_layernorm};
            for (size_t k = 0; k < sizeof ts / sizeof ts[0]; k++) tensor_free(ts[k]);
            free(l->kv_cache);
            free(l);
        }
        free(model->layers);
    }
    if (model->lm_head && model->lm_head != model->embed_tokens) tensor_free(model->lm_head);
    tensor_free(model->embed_tokens);
    tensor_free(model->norm);
    /* the model owns its tokenizer (src/nn/llama.c:258-259), unless the caller's own functions drive it */
    if (model->tokenizer && !g_tok_encode && !g_tok_decode) cml_tokenizer_free(model->tokenizer);
    free(model);
}

/* ---- device state ------------------------------------------------------------------------------ */
static DevModel* dm_get(CMLLLaMAModel* m) {
    DevModel* d = dm_find(m);
    if (d) return d;
    d = (DevModel*)calloc(1, sizeof *d);
    if (!d) return NULL;
    d->key = m;
    d->max_batch = 1;
    d->tp = m->config.tensor_parallel_size > 1 ? m->config.tensor_parallel_size : 1;
    d->rank = d->tp > 1 ? m->config.tensor_parallel_rank : 0;
    d->device = -1;
    pthread_mutex_lock(&g_models_mu);
    d->next = g_models;
    g_models = d;
    pthread_mutex_unlock(&g_models_mu);
    return d;
}

int cml_llama_set_options(CMLLLaMAModel* model, int flags, int max_batch) {
    if (!model || max_batch < 1 || max_batch > SKINNY_ROWS) { LOG_ERROR("cml_llama_set_options: invalid arguments (max_batch must be 1..%d)", SKINNY_ROWS); return -1; }
    DevModel* d = dm_get(model);
    if (!d) return -1;
    if (d->h) { LOG_ERROR("cml_llama_set_options: must be called before weights are loaded"); return -1; }
    d->flags = flags;
    d->max_batch = max_batch;
    return 0;
}

int cml_llama_tp_unique_id(void* id128) { return cml_nccl_unique_id(id128); }

/* Every rank contributes one 64-byte record; all[r] receives rank r's. The collective is always
 * entered, so ranks that hit a local error before it still meet the others. */
static int tp_gather64(DevModel* d, const unsigned char mine[64], unsigned char all[8 * 64]) {
    void *d_mine = NULL, *d_all = NULL;
    int rc = -1;
    if (cmlb200_malloc(&d_mine, 64) || cmlb200_malloc(&d_all, 64 * (size_t)d->tp)) goto done;
    if (cmlb200_memcpy_h2d(d_mine, mine, 64, NULL) || cmlb200_device_sync()) goto done;
    if (cml_nccl_allgather_bytes(d->comm, d_mine, d_all, 64, NULL) || cmlb200_device_sync()) goto done;
    if (cmlb200_memcpy_d2h(all, d_all, 64 * (size_t)d->tp, NULL) || cmlb200_device_sync()) goto done;
    rc = 0;
done:
    cmlb200_free(d_mine);
    cmlb200_free(d_all);
    return rc;
}

/* 1 when `local_ok` holds on every rank. */
static int tp_all_agree(DevModel* d, int local_ok) {
    unsigned char mine[64] = {0}, all[8 * 64];
    mine[0] = local_ok ? 1 : 0;
    if (tp_gather64(d, mine, all)) return 0;
    for (int r = 0; r < d->tp; r++)
        if (!all[64 * r]) return 0;
    return 1;
}

/* Allocates this rank's workspace of `bytes` (zero-filled) and maps every other rank's into this
 * process through CUDA IPC handles. ws[rank] = own allocation. 0 only when it worked on all ranks. */
static int tp_map_workspaces(DevModel* d, size_t bytes, void** ws) {
    unsigned char mine[64] = {0}, all[8 * 64], zero[64] = {0};
    int ok = !cmlb200_malloc(&ws[d->rank], bytes) && !cmlb200_memset(ws[d->rank], 0, bytes, NULL) && !cmlb200_device_sync() &&
             !cmlb200_ipc_get_handle(ws[d->rank], mine);
    if (!ok) memset(mine, 0, 64);                    /* an all-zero handle tells the others */
    if (tp_gather64(d, mine, all)) ok = 0;
    for (int r = 0; ok && r < d->tp; r++)
        if (!memcmp(all + 64 * r, zero, 64)) ok = 0;
    for (int r = 0; ok && r < d->tp; r++)
        if (r != d->rank && cmlb200_ipc_open(all + 64 * r, &ws[r])) ok = 0;
    return tp_all_agree(d, ok) ? 0 : -1;
}

/* Peer-memory all-reduce for decode-sized rows. Ranks must be separate processes on GPUs with peer
 * access; anything else leaves ar_ok = 0 and the NCCL path in charge. */
static int tp_peer_setup(DevModel* d) {
    const int H = d->key->config.hidden_size;
    if (d->tp > 8) return -1;
    d->ar_max_floats = (size_t)SKINNY_ROWS * H;
    const int rc = tp_map_workspaces(d, cmlb200_tp_ar_workspace_bytes(d->ar_max_floats), d->ar_ws);
    d->ar_ok = rc == 0;
    return rc;
}

static double now_ms(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec * 1e3 + ts.tv_nsec * 1e-6;
}

/* The prompt-sized all-reduce over peer memory is used when (a) its workspaces map on every rank,
 * (b) one sum of a known pattern comes out exact on every rank and (c) it is faster than
 * ncclAllReduce + add on the same message by the slowest rank's clock. CML_B200_TP_BULK=1 skips
 * (c), =0 keeps NCCL. Every rank enters the same collectives and takes the same decision. */
static void tp_bulk_setup(DevModel* d) {
    const char* env = getenv("CML_B200_TP_BULK");
    const int H = d->key->config.hidden_size;
    if (d->tp > 8 || (env && env[0] == '0')) return;
    int rows = d->key->config.max_seq_len;
    if (rows < SKINNY_ROWS) rows = SKINNY_ROWS;
    if (rows > 2048) rows = 2048;
    d->arb_max_floats = ((size_t)rows * H + 3) & ~(size_t)3;
    if (tp_map_workspaces(d, cmlb200_tp_ar_bulk_workspace_bytes(d->arb_max_floats, d->tp), d->arb_ws)) return;
    const size_t n = d->arb_max_floats < ((size_t)4 << 20) ? d->arb_max_floats : ((size_t)4 << 20);
    float *hp = malloc(n * 4), *dh = NULL, *dp = NULL;
    float ms_bulk = 0.f, ms_nccl = 0.f, worst_bulk = 0.f, worst_nccl = 0.f;
    const float tri = (float)(d->tp * (d->tp + 1) / 2);
    unsigned char mine[64] = {0}, all[8 * 64];
    double t0 = 0.0;
    int st = 0;
    int good = hp && !cmlb200_malloc((void**)&dh, n * 4) && !cmlb200_malloc((void**)&dp, n * 4);
    if (!tp_all_agree(d, good)) goto done;
    /* (b) exactness: partial = (i mod 251) * (rank + 1) on zeros -> (i mod 251) * tp (tp + 1) / 2 */
    for (size_t i = 0; i < n; i++) hp[i] = (float)((i % 251) * (size_t)(d->rank + 1));
    good = !cmlb200_memcpy_h2d(dp, hp, n * 4, NULL) && !cmlb200_memset(dh, 0, n * 4, NULL) && !cmlb200_device_sync() &&
           !cmlb200_tp_allreduce_bulk_add(dh, dp, n, d->tp, d->rank, d->arb_ws, d->arb_max_floats, NULL) && !cmlb200_device_sync() &&
           !cmlb200_tp_ar_status(d->arb_ws[d->rank], &st) && st == 0 && !cmlb200_memcpy_d2h(hp, dh, n * 4, NULL) && !cmlb200_device_sync();
    for (size_t i = 0; good && i < n; i++) good = hp[i] == (float)(i % 251) * tri;
    if (!tp_all_agree(d, good)) {
        LOG_WARNING("cml_llama_tp_init: the peer-memory all-reduce for prompts failed its start-up check%s; NCCL serves prompts", good ? " on another rank" : "");
        goto done;
    }
    /* (c) the clock: 4 sums of n values each way */
    t0 = now_ms();
    for (int k = 0; k < 4; k++) cmlb200_tp_allreduce_bulk_add(dh, dp, n, d->tp, d->rank, d->arb_ws, d->arb_max_floats, NULL);
    cmlb200_device_sync();
    ms_bulk = (float)(now_ms() - t0);
    cml_nccl_allreduce_sum_f32(d->comm, dp, n, NULL);
    cmlb200_device_sync();
    t0 = now_ms();
    for (int k = 0; k < 4; k++) { cml_nccl_allreduce_sum_f32(d->comm, dp, n, NULL); cmlb200_add_f32(dh, dp, n, NULL); }
    cmlb200_device_sync();
    ms_nccl = (float)(now_ms() - t0);
    st = 0;
    good = !cmlb200_tp_ar_status(d->arb_ws[d->rank], &st) && st == 0;      /* no wait expired while timing */
    memcpy(mine, &ms_bulk, 4);
    memcpy(mine + 4, &ms_nccl, 4);
    mine[8] = good ? 1 : 0;
    if (tp_gather64(d, mine, all)) goto done;
    for (int r = 0; r < d->tp; r++) {                 /* the same records, hence the same decision, on every rank */
        float b, c;
        memcpy(&b, all + 64 * r, 4);
        memcpy(&c, all + 64 * r + 4, 4);
        if (b > worst_bulk) worst_bulk = b;
        if (c > worst_nccl) worst_nccl = c;
        if (!all[64 * r + 8]) good = 0;
    }
    if (!good) goto done;
    d->arb_ok = (env && env[0] == '1') || worst_bulk < worst_nccl;
    d->arb_ms[0] = worst_bulk / 4;
    d->arb_ms[1] = worst_nccl / 4;
    d->arb_probe_floats = n;
    LOG_INFO("cml_llama_tp_init: all-reduce of %zu floats over %d ranks: peer memory %.3f ms, NCCL + add %.3f ms -> %s for prompts",
             n, d->tp, worst_bulk / 4, worst_nccl / 4, d->arb_ok ? "peer memory" : "NCCL");
done:
    free(hp);
    cmlb200_free(dh);
    cmlb200_free(dp);
}

int cml_llama_tp_init(CMLLLaMAModel* model, const void* id128, int device) {
    if (!model || !id128) { LOG_ERROR("cml_llama_tp_init: NULL argument"); return -1; }
    DevModel* d = dm_get(model);
    if (!d) return -1;
    if (d->tp <= 1) { LOG_ERROR("cml_llama_tp_init: config.tensor_parallel_size is %d", model->config.tensor_parallel_size); return -1; }
    if (d->rank < 0 || d->rank >= d->tp) { LOG_ERROR("cml_llama_tp_init: rank %d outside 0..%d", d->rank, d->tp - 1); return -1; }
    DEV(cmlb200_set_device(device));
    d->device = device;
    if (cml_nccl_init(&d->comm, d->tp, d->rank, id128)) return -1;
    const char* only = getenv("CML_B200_TP_NCCL_ONLY");
    if (only && only[0] == '1') return 0;
    if (cmlb200_malloc((void**)&d->lineup, 16) || cmlb200_memset(d->lineup, 0, 16, NULL) || cmlb200_device_sync()) {
        LOG_ERROR("cml_llama_tp_init: %s", cmlb200_last_error());       /* the other ranks are about to enter collectives: fail loudly */
        return -1;
    }
    if (tp_peer_setup(d)) { LOG_WARNING("cml_llama_tp_init: no peer-memory all-reduce, using NCCL for every size"); return 0; }
    tp_bulk_setup(d);
    return 0;
}

int cml_llama_config_from_gguf(const char* filepath, CMLLLaMAConfig* config) {
    if (!filepath || !config) { LOG_ERROR("cml_llama_config_from_gguf: NULL argument"); return -1; }
    GGUFContext* g = gguf_open_read(filepath);
    if (!g) return -1;
    const char* arch = gguf_get_metadata_string(g, "general.architecture");
    if (!arch || strlen(arch) > 64) arch = "llama";
    char key[160];
    int64_t layers = 0, hidden = 0, heads = 0, v = 0;
    double f = 0.0;
#define ARCH_KEY(suffix) (snprintf(key, sizeof key, "%s.%s", arch, suffix), key)
    if (gguf_get_metadata_int(g, ARCH_KEY("block_count"), &layers) || gguf_get_metadata_int(g, ARCH_KEY("embedding_length"), &hidden) ||
        gguf_get_metadata_int(g, ARCH_KEY("attention.head_count"), &heads) || layers <= 0 || hidden <= 0 || heads <= 0 ||
        layers > 4096 || hidden > (1 << 20) || heads > hidden) {
        LOG_ERROR("cml_llama_config_from_gguf: %s lacks %s.block_count / embedding_length / attention.head_count", filepath, arch);
        gguf_close(g);
        return -1;
    }
    CMLLLaMAConfig c = cml_llama_config_7b();
    c.num_layers = (int)layers;
    c.hidden_size = (int)hidden;
    c.num_heads = (int)heads;
    c.num_kv_heads = (int)heads;
    if (!gguf_get_metadata_int(g, ARCH_KEY("attention.head_count_kv"), &v) && v > 0 && v <= heads) c.num_kv_heads = (int)v;
    if (!gguf_get_metadata_int(g, ARCH_KEY("feed_forward_length"), &v) && v > 0 && v < (1 << 24)) c.intermediate_size = (int)v;
    if (!gguf_get_metadata_int(g, ARCH_KEY("context_length"), &v) && v > 0 && v < (1 << 24)) c.max_seq_len = (int)v;
    if (!gguf_get_metadata_float(g, ARCH_KEY("rope.freq_base"), &f) && f > 0.0) c.rope_theta = (float)f;
    if (!gguf_get_metadata_float(g, ARCH_KEY("attention.layer_norm_rms_epsilon"), &f) && f > 0.0) c.rms_norm_eps = (float)f;
    const GGUFTensorInfo* emb = cml_gguf_find(g, "token_embd.weight");
    if (!emb) emb = cml_gguf_find(g, "model.embed_tokens.weight");
    if (!gguf_get_metadata_int(g, ARCH_KEY("vocab_size"), &v) && v > 0 && v < (1 << 24)) c.vocab_size = (int)v;
    else if ((v = gguf_get_metadata_array_length(g, "tokenizer.ggml.tokens", NULL)) > 0 && v < (1 << 24)) c.vocab_size = (int)v;
    else if (emb && emb->ndim == 2 && emb->shape[0] > 0 && emb->shape[0] < (1 << 24)) c.vocab_size = (int)emb->shape[0];
#undef ARCH_KEY
    gguf_close(g);
    *config = c;
    return 0;
}

int cml_llama_load_gguf_tokenizer(CMLLLaMAModel* model, const char* filepath) {
    if (!model || !filepath) { LOG_ERROR("cml_llama_load_gguf_tokenizer: NULL argument"); return -1; }
    GGUFContext* g = gguf_open_read(filepath);
    if (!g) return -1;
    CMLTokenizer* tok = gguf_create_tokenizer(g);
    gguf_close(g);
    if (!tok) { LOG_ERROR("cml_llama_load_gguf_tokenizer: %s has no tokenizer.ggml.tokens", filepath); return -1; }
    if (model->tokenizer && !g_tok_encode && !g_tok_decode) cml_tokenizer_free(model->tokenizer);
    model->tokenizer = tok;
    return 0;
}

int cml_llama_tp_prompt_allreduce(CMLLLaMAModel* model, size_t* probe_floats, float* peer_ms, float* nccl_ms) {
    DevModel* d = model ? dm_get(model) : NULL;
    if (!d) return -1;
    if (probe_floats) *probe_floats = d->arb_probe_floats;
    if (peer_ms) *peer_ms = d->arb_ms[0];
    if (nccl_ms) *nccl_ms = d->arb_ms[1];
    return d->arb_ok;
}

static int dm_alloc_buffers(DevModel* d) {
    const CMLLLaMAConfig* c = &d->key->config;
    const int H = c->hidden_size;
    d->hd = H / c->num_heads;
    if (c->num_heads % d->tp || c->num_kv_heads % d->tp || c->intermediate_size % d->tp || (c->intermediate_size / d->tp) % 32) {
        LOG_ERROR("tensor parallel size %d must divide heads (%d), kv heads (%d) and the FFN width (%d) into multiples of 32",
                  d->tp, c->num_heads, c->num_kv_heads, c->intermediate_size);
        return -1;
    }
    if (d->hd != 32 && d->hd != 64 && d->hd != 128) { LOG_ERROR("head_dim %d not supported (32, 64 or 128)", d->hd); return -1; }
    d->heads_l = c->num_heads / d->tp;
    d->kvh_l = c->num_kv_heads / d->tp;
    d->qw_l = d->heads_l * d->hd;
    d->kvw_l = d->kvh_l * d->hd;
    d->inter_l = c->intermediate_size / d->tp;
    d->qkv_w = d->qw_l + 2 * d->kvw_l;
    d->max_rows = c->max_seq_len > SKINNY_ROWS ? c->max_seq_len : SKINNY_ROWS;
    if (d->device >= 0) DEV(cmlb200_set_device(d->device));
    DEV(cmlb200_stream_create(&d->stream));
    const size_t R = (size_t)d->max_rows;
    const int kvf32 = (d->flags & CML_B200_KV_FP32) != 0;
    d->kv_layer_elems = (size_t)d->max_batch * c->max_seq_len * d->kvw_l;
    const size_t kv_bytes = d->kv_layer_elems * c->num_layers * (kvf32 ? 4 : 2);
    DEV(cmlb200_malloc(&d->kc, kv_bytes));
    DEV(cmlb200_malloc(&d->vc, kv_bytes));
    DEV(cmlb200_memset(d->kc, 0, kv_bytes, d->stream));
    DEV(cmlb200_memset(d->vc, 0, kv_bytes, d->stream));
    const size_t wide = (size_t)(d->inter_l > d->qkv_w ? d->inter_l : d->qkv_w);
    DEV(cmlb200_malloc((void**)&d->h, R * H * 4));
    DEV(cmlb200_malloc((void**)&d->nrm, R * H * 4));
    DEV(cmlb200_malloc((void**)&d->qkv, R * d->qkv_w * 4));
    DEV(cmlb200_malloc((void**)&d->att, R * d->qw_l * 4));
    DEV(cmlb200_malloc((void**)&d->ffn, (size_t)SKINNY_ROWS * d->inter_l * 4));
    DEV(cmlb200_malloc((void**)&d->g, (size_t)SKINNY_ROWS * d->inter_l * 4));
    DEV(cmlb200_malloc((void**)&d->u, (size_t)SKINNY_ROWS * d->inter_l * 4));
    DEV(cmlb200_malloc((void**)&d->tmp, R * H * 4));
    DEV(cmlb200_malloc((void**)&d->logits, R * c->vocab_size * 4));
    d->vocab_l = (d->tp > 1 && c->vocab_size % d->tp == 0) ? c->vocab_size / d->tp : c->vocab_size;
    if (d->vocab_l != c->vocab_size) {
        DEV(cmlb200_malloc((void**)&d->logits_l, R * d->vocab_l * 4));
        DEV(cmlb200_malloc((void**)&d->logits_g, R * c->vocab_size * 4));
        DEV(cmlb200_malloc((void**)&d->pairs, (size_t)(d->tp + 1) * SKINNY_ROWS * 8));
    }
    DEV(cmlb200_malloc((void**)&d->b_a, R * (wide > (size_t)H ? wide : (size_t)H) * 2));
    DEV(cmlb200_malloc((void**)&d->b_b, R * (wide > (size_t)c->vocab_size ? wide : (size_t)c->vocab_size) * 2));
    DEV(cmlb200_malloc((void**)&d->b_c, R * wide * 2));
    DEV(cmlb200_malloc((void**)&d->b_d, R * wide * 2));
    d->att_splits_cap = (c->max_seq_len + ATT_CHUNK - 1) / ATT_CHUNK;
    {   /* the larger of: split partials for a skinny call (+ the decode kernel's counters), one split for a prefill call */
        const size_t bytes = cmlb200_attention_decode_scratch_bytes(SKINNY_ROWS, d->heads_l, d->hd, 2 * d->att_splits_cap) +
                             cmlb200_attention_scratch_floats(d->max_rows, d->heads_l, d->hd, 1) * 4;
        DEV(cmlb200_malloc((void**)&d->att_scratch, bytes));
        DEV(cmlb200_memset(d->att_scratch, 0, bytes, NULL));
        DEV(cmlb200_malloc((void**)&d->rope_cs, (size_t)SKINNY_ROWS * d->hd * sizeof(float)));
    }
    DEV(cmlb200_malloc((void**)&d->d_tokens, R * 4));
    DEV(cmlb200_malloc((void**)&d->d_cur, (size_t)d->max_batch * 4));
    DEV(cmlb200_malloc((void**)&d->row_seq, R * 4));
    DEV(cmlb200_malloc((void**)&d->row_pos, R * 4));
    DEV(cmlb200_malloc((void**)&d->row_limit, R * 4));
    DEV(cmlb200_malloc((void**)&d->d_hist, (size_t)c->max_seq_len * d->max_batch * 4));
    DEV(cmlb200_memset(d->d_cur, 0, (size_t)d->max_batch * 4, d->stream));
    d->h_cur = (int*)calloc((size_t)d->max_batch, sizeof(int));
    return d->h_cur ? 0 : -1;
}

/* GGUF blocks of a [rows, cols] weight -> both device layouts. */
static int upload_qmat(DevModel* d, int type, const uint8_t* blocks, int rows, int cols, cmlb200_qmat* out) {
    memset(out, 0, sizeof *out);
    out->type = type;
    out->rows = rows;
    out->cols = cols;
    out->block = 32;
    if (type != GGUF_TENSOR_Q4_0 && type != GGUF_TENSOR_Q8_0) {
        /* Q4_1 / Q4_K / Q5_K / Q6_K: the block stream goes to the device as it is; the model then runs
         * every call on the fp32 row-block path (no fused or tensor-core kernels for these types) */
        const size_t bs = gguf_quant_block_size((GGUFTensorType)type), bytes = (size_t)rows * ((size_t)cols / bs) * gguf_quant_type_size((GGUFTensorType)type);
        out->block = (int)bs;
        if (CML_DEV_FAIL(cmlb200_malloc(&out->qs, bytes), "upload") || CML_DEV_FAIL(cmlb200_memcpy_h2d(out->qs, blocks, bytes, d->stream), "upload") ||
            CML_DEV_FAIL(cmlb200_stream_sync(d->stream), "upload"))
            return -1;
        d->generic_w = 1;
        return 0;
    }
    const size_t qb = cmlb200_qs_bytes(type, rows, cols, 32), sb = cmlb200_scale_bytes(type, rows, cols, 32);
    void *h_qs = malloc(qb), *h_sc = malloc(sb), *h_t = NULL;
    int rc = -1;
    if (!h_qs || !h_sc) goto done;
    if (CML_DEV_FAIL(cmlb200_repack_gguf(type, blocks, rows, cols, h_qs, h_sc), "upload")) goto done;
    out->flags = cmlb200_scales_have_subnormals(h_sc, sb / 2) ? CMLB200_QMAT_SUBNORMAL_SCALES : 0;
    if (CML_DEV_FAIL(cmlb200_malloc(&out->qs, qb), "upload") || CML_DEV_FAIL(cmlb200_malloc(&out->scales, sb), "upload")) goto done;
    if (CML_DEV_FAIL(cmlb200_memcpy_h2d(out->qs, h_qs, qb, d->stream), "upload") ||
        CML_DEV_FAIL(cmlb200_memcpy_h2d(out->scales, h_sc, sb, d->stream), "upload")) goto done;
    /* the tcgen05 decode path serves batches of 3..32 from a tile-major copy, unless the 8-row
     * mma.sync kernel takes this weight from the planes (Q4_0, cols % 256 == 0) */
    if (cols % 128 == 0 && d->max_batch > 2 && !cmlb200_gemv_batched_from_planes(out)) {
        const size_t tb = cmlb200_tiles_bytes(type, rows, cols);
        h_t = malloc(tb);
        if (!h_t) goto done;
        if (CML_DEV_FAIL(cmlb200_repack_tiles(type, blocks, rows, cols, h_t), "upload")) goto done;
        if (CML_DEV_FAIL(cmlb200_malloc(&out->tiles, tb), "upload")) goto done;
        if (CML_DEV_FAIL(cmlb200_memcpy_h2d(out->tiles, h_t, tb, d->stream), "upload")) goto done;
    }
    if (CML_DEV_FAIL(cmlb200_stream_sync(d->stream), "upload")) goto done;
    rc = 0;
done:
    free(h_qs); free(h_sc); free(h_t);
    return rc;
}

/* fp16 (or fp32) host vector -> fp16 device vector */
static int upload_f16(DevModel* d, const void* raw, GGUFTensorType type, size_t numel, void** out) {
    uint16_t* tmp = NULL;
    const void* src = raw;
    if (type == GGUF_TENSOR_F32) {
        tmp = (uint16_t*)malloc(numel * 2);
        if (!tmp) return -1;
        for (size_t i = 0; i < numel; i++) tmp[i] = cml_f32_to_f16(((const float*)raw)[i]);
        src = tmp;
    } else if (type != GGUF_TENSOR_F16) {
        LOG_ERROR("norm / embedding tensors must be F16 or F32 (got GGUF type %d)", (int)type);
        return -1;
    }
    int rc = -1;
    if (!CML_DEV_FAIL(cmlb200_malloc(out, numel * 2), "upload") && !CML_DEV_FAIL(cmlb200_memcpy_h2d(*out, src, numel * 2, d->stream), "upload") &&
        !CML_DEV_FAIL(cmlb200_stream_sync(d->stream), "upload")) rc = 0;
    free(tmp);
    return rc;
}

static Tensor* placeholder(int d0, int d1) {
    /* shape-only tensor: the weight lives on the device, there is no host copy */
    Tensor* t = (Tensor*)calloc(1, sizeof(Tensor));
    if (!t) return NULL;
    t->ndim = d1 > 0 ? 2 : 1;
    t->shape = (int*)malloc(2 * sizeof(int));
    t->strides = (size_t*)malloc(2 * sizeof(size_t));
    if (!t->shape || !t->strides) { free(t->shape); free(t->strides); free(t); return NULL; }
    t->shape[0] = d0; t->shape[1] = d1 > 0 ? d1 : 1;
    t->strides[0] = d1 > 0 ? (size_t)d1 : 1; t->strides[1] = 1;
    t->numel = (size_t)d0 * (size_t)(d1 > 0 ? d1 : 1);
    t->dtype = DTYPE_UINT8;
    t->device = DEVICE_CUDA;
    t->ref_count = 1;
    t->is_contiguous = true;
    return t;
}

enum { SLOT_NONE, SLOT_EMBED, SLOT_NORM, SLOT_HEAD, SLOT_Q, SLOT_K, SLOT_V, SLOT_O, SLOT_G, SLOT_U, SLOT_D, SLOT_N1, SLOT_N2 };

/* llama.cpp ("blk.N.attn_q.weight") and Hugging Face ("model.layers.N.self_attn.q_proj.weight")
 * tensor names, as src/nn/llama.c:272-368 recognises them. */
static int classify(const char* name, int* layer) {
    *layer = -1;
    if (!strcmp(name, "token_embd.weight") || !strcmp(name, "model.embed_tokens.weight")) return SLOT_EMBED;
    if (!strcmp(name, "output_norm.weight") || !strcmp(name, "model.norm.weight")) return SLOT_NORM;
    if (!strcmp(name, "output.weight") || !strcmp(name, "lm_head.weight")) return SLOT_HEAD;
    const char* rest = NULL;
    if (!strncmp(name, "blk.", 4)) rest = name + 4;
    else if (!strncmp(name, "model.layers.", 13)) rest = name + 13;
    if (!rest) return SLOT_NONE;
    char* end;
    const long l = strtol(rest, &end, 10);
    if (end == rest || *end != '.') return SLOT_NONE;
    *layer = (int)l;
    const char* s = end + 1;
    static const struct { const char* n; int slot; } map[] = {
        {"attn_q.weight", SLOT_Q}, {"self_attn.q_proj.weight", SLOT_Q}, {"attn_k.weight", SLOT_K}, {"self_attn.k_proj.weight", SLOT_K},
        {"attn_v.weight", SLOT_V}, {"self_attn.v_proj.weight", SLOT_V}, {"attn_output.weight", SLOT_O}, {"self_attn.o_proj.weight", SLOT_O},
        {"ffn_gate.weight", SLOT_G}, {"mlp.gate_proj.weight", SLOT_G}, {"ffn_up.weight", SLOT_U}, {"mlp.up_proj.weight", SLOT_U},
        {"ffn_down.weight", SLOT_D}, {"mlp.down_proj.weight", SLOT_D}, {"attn_norm.weight", SLOT_N1}, {"input_layernorm.weight", SLOT_N1},
        {"ffn_norm.weight", SLOT_N2}, {"post_attention_layernorm.weight", SLOT_N2}};
    for (size_t i = 0; i < sizeof map / sizeof map[0]; i++) if (!strcmp(s, map[i].n)) return map[i].slot;
    return SLOT_NONE;
}

/* cml_tp_shard_weight (src/distributed/tensor_parallel.c:25-101) on quantized blocks: dim 0 keeps
 * rows [rank*rows/tp, (rank+1)*rows/tp), dim 1 keeps columns [rank*cols/tp, (rank+1)*cols/tp) of
 * every row, which must fall on block boundaries. Same argument checks, -1 on failure. */
int cml_tp_shard_qblocks(int type, const void* blocks, int rows, int cols, int dim, int tp_size, int tp_rank, void* out) {
    const size_t bb = gguf_quant_type_size((GGUFTensorType)type);
    if (!blocks || !out) { LOG_ERROR("cml_tp_shard_qblocks: NULL argument"); return -1; }
    const int bs = (int)gguf_quant_block_size((GGUFTensorType)type);
    if (!bb || bs <= 1) { LOG_ERROR("cml_tp_shard_qblocks: type %d is not a block-quantized type", type); return -1; }
    if (dim != 0 && dim != 1) { LOG_ERROR("cml_tp_shard_qblocks: dim must be 0 or 1, got %d", dim); return -1; }
    if (tp_size <= 0 || tp_rank < 0 || tp_rank >= tp_size) { LOG_ERROR("cml_tp_shard_qblocks: invalid tp_size=%d or tp_rank=%d", tp_size, tp_rank); return -1; }
    if (rows <= 0 || cols <= 0 || cols % bs) { LOG_ERROR("cml_tp_shard_qblocks: bad shape %dx%d for %d-element blocks", rows, cols, bs); return -1; }
    const int nblk = cols / bs;
    const uint8_t* full = (const uint8_t*)blocks;
    uint8_t* dst = (uint8_t*)out;
    if (dim == 0) {
        if (rows % tp_size) { LOG_ERROR("cml_tp_shard_qblocks: rows (%d) not divisible by tp_size (%d)", rows, tp_size); return -1; }
        const size_t n = (size_t)(rows / tp_size) * nblk * bb;
        memcpy(dst, full + (size_t)tp_rank * n, n);
    } else {
        if (cols % tp_size || (cols / tp_size) % bs) { LOG_ERROR("cml_tp_shard_qblocks: cols (%d) must split into %d multiples of %d", cols, tp_size, bs); return -1; }
        const int lb = nblk / tp_size;
        for (int r = 0; r < rows; r++) memcpy(dst + (size_t)r * lb * bb, full + ((size_t)r * nblk + (size_t)tp_rank * lb) * bb, (size_t)lb * bb);
    }
    return 0;
}

static uint8_t* shard_blocks(const uint8_t* full, int type, int rows, int cols, int tp, int rank, int by_rows, int* orow, int* ocol) {
    *orow = by_rows ? rows / tp : rows;
    *ocol = by_rows ? cols : cols / tp;
    const size_t bs = gguf_quant_block_size((GGUFTensorType)type);
    if (bs <= 1 || *ocol % (int)bs) { LOG_ERROR("a shard of %d columns is not a whole number of %zu-element blocks", *ocol, bs); return NULL; }
    uint8_t* out = (uint8_t*)malloc((size_t)*orow * ((size_t)*ocol / bs) * gguf_quant_type_size((GGUFTensorType)type));
    if (out && cml_tp_shard_qblocks(type, full, rows, cols, by_rows ? 0 : 1, tp, rank, out)) { free(out); out = NULL; }
    return out;
}

int cml_llama_load_gguf(CMLLLaMAModel* model, const char* filepath) {
    if (!model || !filepath) { LOG_ERROR("cml_llama_load_gguf: NULL argument"); return -1; }
    DevModel* d = dm_get(model);
    if (!d) return -1;
    if (d->tp > 1 && !d->comm) { LOG_ERROR("cml_llama_load_gguf: tensor_parallel_size=%d but cml_llama_tp_init was not called", d->tp); return -1; }
    GGUFContext* ctx = gguf_open_read(filepath);
    if (!ctx) { LOG_ERROR("cml_llama_load_gguf: failed to open '%s'", filepath); return -1; }
    if (!d->h && dm_alloc_buffers(d)) { gguf_close(ctx); return -1; }
    if (!d->L) d->L = (DevLayer*)calloc((size_t)model->num_layers, sizeof(DevLayer));
    if (!d->L) { gguf_close(ctx); return -1; }
    const CMLLLaMAConfig* c = &model->config;
    const int H = c->hidden_size, hdm = d->hd, QW = c->num_heads * hdm, KVW = c->num_kv_heads * hdm, I = c->intermediate_size;
    int loaded = 0, skipped = 0, failed = 0;
    const int n = gguf_get_num_tensors(ctx);
    for (int i = 0; i < n; i++) {
        const char* name = gguf_get_tensor_name(ctx, i);
        int layer, slot = name ? classify(name, &layer) : SLOT_NONE;
        const GGUFTensorInfo* info = cml_gguf_find(ctx, name);
        if (slot == SLOT_NONE || !info || (layer >= model->num_layers)) {
            LOG_WARNING("cml_llama_load_gguf: unrecognized tensor name: %s", name ? name : "(null)");
            skipped++;
            continue;
        }
        void* raw = cml_gguf_read_raw(ctx, info);
        if (!raw) { failed++; continue; }
        int rc = -1;
        if (slot == SLOT_EMBED || slot == SLOT_NORM || slot == SLOT_N1 || slot == SLOT_N2) {
            size_t numel = 1;
            for (int k = 0; k < info->ndim; k++) numel *= (size_t)info->shape[k];
            const size_t want = slot == SLOT_EMBED ? (size_t)c->vocab_size * H : (size_t)H;
            void** dst = slot == SLOT_EMBED ? &d->embed : slot == SLOT_NORM ? &d->fnorm : slot == SLOT_N1 ? &d->L[layer].n1 : &d->L[layer].n2;
            Tensor** pub = slot == SLOT_EMBED ? &model->embed_tokens : slot == SLOT_NORM ? &model->norm
                           : slot == SLOT_N1 ? &model->layers[layer]->input_layernorm : &model->layers[layer]->post_attn_layernorm;
            if (numel != want) LOG_ERROR("cml_llama_load_gguf: tensor '%s' has %zu elements, expected %zu", name, numel, want);
            else {
                cmlb200_free(*dst); *dst = NULL;
                rc = upload_f16(d, raw, info->type, numel, dst);
                if (!rc) { tensor_free(*pub); *pub = slot == SLOT_EMBED ? placeholder(c->vocab_size, H) : placeholder(H, 0); }
            }
        } else {
            /* projections: GGUF dims are (in_features, out_features) */
            int out_f, in_f, by_rows = 1, qkv_slot = -1;
            cmlb200_qmat* dst = NULL;
            Tensor** pub;
            switch (slot) {
                case SLOT_Q: out_f = QW; in_f = H; qkv_slot = 0; pub = &model->layers[layer]->q_proj; break;
                case SLOT_K: out_f = KVW; in_f = H; qkv_slot = 1; pub = &model->layers[layer]->k_proj; break;
                case SLOT_V: out_f = KVW; in_f = H; qkv_slot = 2; pub = &model->layers[layer]->v_proj; break;
                case SLOT_O: out_f = H; in_f = QW; by_rows = 0; dst = &d->L[layer].wo; pub = &model->layers[layer]->o_proj; break;
                case SLOT_G: out_f = I; in_f = H; dst = &d->L[layer].wg; pub = &model->layers[layer]->gate_proj; break;
                case SLOT_U: out_f = I; in_f = H; dst = &d->L[layer].wu; pub = &model->layers[layer]->up_proj; break;
                case SLOT_D: out_f = H; in_f = I; by_rows = 0; dst = &d->L[layer].wd; pub = &model->layers[layer]->down_proj; break;
                default:                                        /* split by rows when the vocabulary divides, else replicated */
                    out_f = c->vocab_size; in_f = H; by_rows = d->vocab_l != c->vocab_size ? 1 : -1; dst = &d->lm_head; pub = &model->lm_head; break;
            }
            if (info->type != GGUF_TENSOR_Q4_0 && info->type != GGUF_TENSOR_Q8_0 && info->type != GGUF_TENSOR_Q4_1 &&
                info->type != GGUF_TENSOR_Q4_K && info->type != GGUF_TENSOR_Q5_K && info->type != GGUF_TENSOR_Q6_K)
                LOG_ERROR("cml_llama_load_gguf: tensor '%s' has GGUF type %d; projections must be Q4_0, Q8_0, Q4_1, Q4_K, Q5_K or Q6_K", name, (int)info->type);
            else if (in_f % (int)gguf_quant_block_size(info->type))
                LOG_ERROR("cml_llama_load_gguf: tensor '%s': in_features %d is not a whole number of %zu-element blocks", name, in_f, gguf_quant_block_size(info->type));
            else if (info->ndim != 2 || info->shape[0] != in_f || info->shape[1] != out_f)
                LOG_ERROR("cml_llama_load_gguf: tensor '%s' has dims (%lld, %lld), expected (in=%d, out=%d)", name,
                          (long long)info->shape[0], (long long)(info->ndim > 1 ? info->shape[1] : 0), in_f, out_f);
            else if (qkv_slot >= 0) {
                /* Q, K, V: keep this rank's rows on the host until all three are there, then
                 * upload them stacked as one [q | k | v] matrix (one GEMV instead of three). */
                DevLayer* L = &d->L[layer];
                int lr = out_f, lc = in_f;
                uint8_t* sh = shard_blocks((const uint8_t*)raw, (int)info->type, out_f, in_f, d->tp, d->rank, 1, &lr, &lc);
                const int have_other = L->pend[0] || L->pend[1] || L->pend[2];
                if (sh && have_other && L->pend_type != (int)info->type) {
                    LOG_ERROR("cml_llama_load_gguf: layer %d mixes block types across attn_q/k/v", layer);
                    free(sh);
                } else if (sh) {
                    free(L->pend[qkv_slot]);
                    L->pend[qkv_slot] = sh;
                    L->pend_type = (int)info->type;
                    rc = 0;
                    if (L->pend[0] && L->pend[1] && L->pend[2]) {
                        const size_t bb = gguf_quant_type_size(info->type), rowb = ((size_t)H / gguf_quant_block_size(info->type)) * bb;
                        const size_t qb = (size_t)d->qw_l * rowb, kb = (size_t)d->kvw_l * rowb;
                        uint8_t* all = (uint8_t*)malloc(qb + 2 * kb);
                        if (all) {
                            memcpy(all, L->pend[0], qb);
                            memcpy(all + qb, L->pend[1], kb);
                            memcpy(all + qb + kb, L->pend[2], kb);
                            qmat_free(&L->wqkv);
                            rc = upload_qmat(d, (int)info->type, all, d->qkv_w, H, &L->wqkv);
                            free(all);
                        } else rc = -1;
                        for (int k = 0; k < 3; k++) { free(L->pend[k]); L->pend[k] = NULL; }
                    }
                    if (!rc) { tensor_free(*pub); *pub = placeholder(in_f, out_f); }
                }
            } else {
                qmat_free(dst);
                if (d->tp > 1 && by_rows >= 0) {
                    int lr, lc;
                    uint8_t* sh = shard_blocks((const uint8_t*)raw, (int)info->type, out_f, in_f, d->tp, d->rank, by_rows, &lr, &lc);
                    rc = sh ? upload_qmat(d, (int)info->type, sh, lr, lc, dst) : -1;
                    free(sh);
                } else rc = upload_qmat(d, (int)info->type, (const uint8_t*)raw, out_f, in_f, dst);
                if (!rc) { tensor_free(*pub); *pub = placeholder(in_f, out_f); }
            }
        }
        free(raw);
        if (rc) failed++; else loaded++;
    }
    gguf_close(ctx);
    if (!model->lm_head && model->embed_tokens) LOG_WARNING("cml_llama_load_gguf: no output.weight tensor; tied embeddings are not supported on the quantized path");
    model->weights_loaded = failed == 0;
    LOG_INFO("GGUF loading complete: %d loaded, %d skipped, %d failed", loaded, skipped, failed);
    return failed ? -1 : 0;
}

/* ---- forward ------------------------------------------------------------------------------------ */
/* After the stream has drained: did a bounded device-side wait give up? (tcgen05 pipelines, the
 * stream-K fix-up, and the peer-memory all-reduce, whose launch then left the residual without the
 * projection.) Returns -1 and logs; a failed all-reduce also retires the peer path, because the
 * ranks' sequence counters may no longer agree, and NCCL serves every size from then on. */
static int dm_check_waits(DevModel* d, const char* who) {
    int st = 0;
    if (cmlb200_gemm_status(&st, 1) == CMLB200_OK && st == 0) cmlb200_gemv_tiles_status(&st, 1);
    if (st) { LOG_ERROR("%s: a bounded device-side wait expired (code %d)", who, st); return -1; }
    if (d->ar_ok && d->ar_ws[d->rank]) {
        if (cmlb200_tp_ar_status(d->ar_ws[d->rank], &st) != CMLB200_OK) { LOG_ERROR("%s: %s", who, cmlb200_last_error()); return -1; }
        if (st) {
            LOG_ERROR("%s: the all-reduce gave up waiting for rank %d; the result is incomplete (falling back to NCCL)", who, st - 1);
            cmlb200_tp_ar_status_reset(d->ar_ws[d->rank]);
            d->ar_ok = 0;
            if (d->graph) { cmlb200_graph_destroy(d->graph); d->graph = NULL; }
            return -1;
        }
    }
    if (d->arb_ok && d->arb_ws[d->rank]) {
        if (cmlb200_tp_ar_status(d->arb_ws[d->rank], &st) != CMLB200_OK) { LOG_ERROR("%s: %s", who, cmlb200_last_error()); return -1; }
        if (st) {
            LOG_ERROR("%s: the prompt-sized all-reduce gave up waiting for rank %d; the result is incomplete (falling back to NCCL)", who, st - 1);
            cmlb200_tp_ar_status_reset(d->arb_ws[d->rank]);
            d->arb_ok = 0;
            return -1;
        }
    }
    return 0;
}

static int model_ready(const CMLLLaMAModel* m, const DevModel* d) {
    if (!d || !d->embed || !d->fnorm || !d->lm_head.qs) return 0;
    for (int i = 0; i < m->num_layers; i++) {
        const DevLayer* l = &d->L[i];
        if (!l->wqkv.qs || !l->wo.qs || !l->wg.qs || !l->wu.qs || !l->wd.qs || !l->n1 || !l->n2) return 0;
    }
    return 1;
}

/* y = x . W^T (accumulate == 0) or y += x . W^T over `rows` rows on the fp32 decode kernels */
static int lin_f32(DevModel* d, const cmlb200_qmat* W, const float* x, float* y, int rows, int accumulate) {
    for (int r0 = 0; r0 < rows; r0 += SKINNY_ROWS) {
        const int m = rows - r0 < SKINNY_ROWS ? rows - r0 : SKINNY_ROWS;
        const float* xp = x + (size_t)r0 * W->cols;
        float* yp = y + (size_t)r0 * W->rows;
        if (accumulate) DEV(cmlb200_gemv_accum(W, xp, yp, m, d->stream));
        else DEV(cmlb200_gemv(W, xp, yp, m, d->stream));
    }
    return 0;
}

/* Row-parallel projection + residual: h += all_reduce(x . W_shard^T) */
static int proj_residual_f32(DevModel* d, const cmlb200_qmat* W, const float* x, int rows) {
    if (d->tp == 1) return lin_f32(d, W, x, d->h, rows, 1);
    if (d->ar_ok && rows <= 4 && W->rows == d->key->config.hidden_size && (size_t)rows * W->rows * 2 <= d->ar_max_floats &&
        cmlb200_gemv_tp_fused_ok(W, rows)) {       /* projection and all-reduce in one launch */
        DEV(cmlb200_gemv_tp_allreduce(W, x, d->h, rows, d->tp, d->rank, d->ar_ws, d->ar_max_floats, d->stream));
        return 0;
    }
    if (lin_f32(d, W, x, d->tmp, rows, 0)) return -1;
    if (d->ar_ok && (size_t)rows * W->rows <= d->ar_max_floats && ((size_t)rows * W->rows) % 4 == 0) {
        DEV(cmlb200_tp_allreduce_add(d->h, d->tmp, (size_t)rows * W->rows, d->tp, d->rank, d->ar_ws, d->ar_max_floats, d->stream));
        return 0;
    }
    if (cml_nccl_allreduce_sum_f32(d->comm, d->tmp, (size_t)rows * W->rows, d->stream)) return -1;
    DEV(cmlb200_add_f32(d->h, d->tmp, (size_t)rows * W->rows, d->stream));
    return 0;
}

static int proj_residual_bf16(DevModel* d, const cmlb200_qmat* W, const uint16_t* x, int rows) {
    const size_t n = (size_t)rows * W->rows;
    /* one GPU: the GEMM adds onto the fp32 residual in its epilogue; several: fp32 partial sums, all-reduce, add */
    if (d->tp == 1) { DEV(cmlb200_gemm_bf16_ex(W, x, rows, CMLB200_GEMM_ACC_F32, d->h, NULL, d->stream)); return 0; }
    DEV(cmlb200_gemm_bf16_ex(W, x, rows, CMLB200_GEMM_OUT_F32, d->tmp, NULL, d->stream));
    if (d->arb_ok && n % 4 == 0) {               /* slices summed by rank over peer memory, added onto h in the same launch */
        for (size_t o = 0; o < n; o += d->arb_max_floats) {
            const size_t len = n - o < d->arb_max_floats ? n - o : d->arb_max_floats;
            DEV(cmlb200_tp_allreduce_bulk_add(d->h + o, d->tmp + o, len, d->tp, d->rank, d->arb_ws, d->arb_max_floats, d->stream));
        }
        return 0;
    }
    if (cml_nccl_allreduce_sum_f32(d->comm, d->tmp, n, d->stream)) return -1;
    DEV(cmlb200_add_f32(d->h, d->tmp, n, d->stream));
    return 0;
}

/* Enqueues one forward call over `rows` rows whose tokens are in d->d_tokens.
 * mode 0: one sequence (`seq`), consecutive positions; mode 1: one token for each of `rows`
 * sequences. plan_limit bounds the cache positions the call may touch (sizes the attention
 * splits); logits for all rows land in d->logits. */
static int enqueue_forward_ex(DevModel* d, int rows, int mode, int seq, int plan_limit, int only_layer, int with_head) {
    const CMLLLaMAModel* m = d->key;
    const CMLLLaMAConfig* c = &m->config;
    const int H = c->hidden_size, quirks = (d->flags & CML_B200_REFERENCE_QUIRKS) != 0, kvf32 = (d->flags & CML_B200_KV_FP32) != 0;
    const int skinny = rows <= SKINNY_ROWS || (d->flags & CML_B200_ALL_LOGITS_FP32) || d->generic_w;
    const int tiny = rows <= 8 && !d->generic_w;   /* tensor-core decode GEMV with RMSNorm applied inside the projection launch */
    void* st = d->stream;
    DEV(cmlb200_prepare_rows(d->d_cur, rows, mode, quirks, seq, d->row_seq, d->row_pos, d->row_limit, st));
    if (only_layer < 0) DEV(cmlb200_embed_f16((const uint16_t*)d->embed, d->d_tokens, rows, H, c->vocab_size, d->h, st));
    const int max_limit_raw = quirks ? (mode == 0 ? rows - 1 : 0) : plan_limit;
    const int max_limit = max_limit_raw < c->max_seq_len ? max_limit_raw : c->max_seq_len - 1;
    int splits = 1;
    if (rows <= SKINNY_ROWS) {
        splits = (max_limit + ATT_CHUNK) / ATT_CHUNK;
        if (splits > d->att_splits_cap) splits = d->att_splits_cap;
        if (splits < 1) splits = 1;
    }
    /* With tensor parallelism head 0 lives on rank 0 only, so C-ML's "head 0 only" rotation
     * touches nothing on the other ranks. */
    const int rotate = quirks ? (d->rank == 0 ? 1 : 0) : -1;
    /* one new token per sequence, position-correct behaviour: RoPE, cache append, attention and merge in one launch,
     * one CTA of four warps per 32 keys */
    const int fused_att = !quirks && rows <= SKINNY_ROWS && (mode == 1 || rows == 1) && rows * d->heads_l <= 4096;
    if (fused_att) {
        /* one row: 32 keys per CTA (latency); more rows: at least 64, and as many as keep the launch
         * within about 1280 CTAs (measured at 8 rows x 32 heads x 576 keys: 29.9 us with 19 splits,
         * 22.4 us with 5) */
        int dchunk = rows == 1 ? ATT_DECODE_CHUNK : 2 * ATT_DECODE_CHUNK;
        while (rows > 1 && dchunk < 1024 && rows * d->heads_l * ((max_limit + dchunk) / dchunk) > 1280) dchunk += ATT_DECODE_CHUNK;
        splits = (max_limit + dchunk) / dchunk;
        if (splits > 2 * d->att_splits_cap) splits = 2 * d->att_splits_cap;
        if (splits > 256) splits = 256;
    }
    if (fused_att) DEV(cmlb200_rope_table(d->row_pos, rows, d->hd, c->rope_theta, d->rope_cs, st));
    const size_t esz = kvf32 ? 4 : 2;
    for (int li = 0; li < m->num_layers; li++) {
        if (only_layer >= 0 && li != only_layer) continue;
        const DevLayer* L = &d->L[li];
        void* kc = (char*)d->kc + (size_t)li * d->kv_layer_elems * esz;
        void* vc = (char*)d->vc + (size_t)li * d->kv_layer_elems * esz;
        /* ---- attention block: norm -> fused QKV projection -> RoPE + cache append -> attention */
        if (tiny) {
            DEV(cmlb200_gemv_rmsnorm(&L->wqkv, NULL, d->h, (const uint16_t*)L->n1, c->rms_norm_eps, d->qkv, rows, 0, st));
        } else if (skinny) {
            DEV(cmlb200_rmsnorm(d->h, (const uint16_t*)L->n1, rows, H, c->rms_norm_eps, d->nrm, NULL, st));
            if (lin_f32(d, &L->wqkv, d->nrm, d->qkv, rows, 0)) return -1;
        } else {
            DEV(cmlb200_rmsnorm(d->h, (const uint16_t*)L->n1, rows, H, c->rms_norm_eps, NULL, d->b_a, st));
            DEV(cmlb200_gemm_bf16_ex(&L->wqkv, d->b_a, rows, CMLB200_GEMM_OUT_F32, d->qkv, NULL, st));
        }
        /* prompt-sized call on the bf16 path with an fp16 cache: tiled tensor-core attention, bf16 output
         * straight into the attention-out GEMM's operand buffer */
        const int tiled_att = !skinny && !kvf32 && mode == 0 && (d->hd == 64 || d->hd == 128);
        if (tiled_att) {
            DEV(cmlb200_qkv_rope_append(d->qkv, d->qkv_w, d->row_seq, d->row_pos, rows, d->heads_l, d->kvh_l, d->hd, c->rope_theta,
                                        rotate, kc, vc, c->max_seq_len, kvf32, st));
            DEV(cmlb200_attention_prefill(d->qkv, d->qkv_w, kc, vc, seq, d->row_limit, rows, d->heads_l, d->kvh_l, d->hd, c->max_seq_len,
                                          NULL, d->b_a, st));
        } else if (fused_att) {
            DEV(cmlb200_attention_decode(d->qkv, d->qkv_w, kc, vc, d->row_seq, d->row_pos, d->row_limit, rows, d->heads_l, d->kvh_l,
                                         d->hd, c->max_seq_len, max_limit, kvf32, d->rope_cs, d->att, d->att_scratch, splits, st));
        } else {
            DEV(cmlb200_qkv_rope_append(d->qkv, d->qkv_w, d->row_seq, d->row_pos, rows, d->heads_l, d->kvh_l, d->hd, c->rope_theta,
                                        rotate, kc, vc, c->max_seq_len, kvf32, st));
            DEV(cmlb200_attention_ex(d->qkv, d->qkv_w, kc, vc, d->row_seq, d->row_limit, rows, d->heads_l, d->kvh_l, d->hd,
                                     c->max_seq_len, max_limit, kvf32, d->att, NULL, (float*)d->att_scratch + 4096, splits, st));
        }
        /* ---- output projection + residual, FFN + residual */
        if (tiny) {
            if (proj_residual_f32(d, &L->wo, d->att, rows)) return -1;
            DEV(cmlb200_gemv_rmsnorm(&L->wg, &L->wu, d->h, (const uint16_t*)L->n2, c->rms_norm_eps, d->ffn, rows, 2, st));
            if (proj_residual_f32(d, &L->wd, d->ffn, rows)) return -1;
        } else if (skinny) {
            if (proj_residual_f32(d, &L->wo, d->att, rows)) return -1;
            DEV(cmlb200_rmsnorm(d->h, (const uint16_t*)L->n2, rows, H, c->rms_norm_eps, d->nrm, NULL, st));
            for (int r0 = 0; r0 < rows; r0 += SKINNY_ROWS) {
                const int mr = rows - r0 < SKINNY_ROWS ? rows - r0 : SKINNY_ROWS;
                const float* xp = d->nrm + (size_t)r0 * H;
                DEV(cmlb200_gemv(&L->wg, xp, d->g, mr, st));
                DEV(cmlb200_gemv(&L->wu, xp, d->u, mr, st));
                DEV(cmlb200_swiglu_f32(d->g, d->u, d->ffn, (size_t)mr * d->inter_l, st));
                if (d->tp == 1) DEV(cmlb200_gemv_accum(&L->wd, d->ffn, d->h + (size_t)r0 * H, mr, st));
                else {
                    DEV(cmlb200_gemv(&L->wd, d->ffn, d->tmp, mr, st));
                    if (cml_nccl_allreduce_sum_f32(d->comm, d->tmp, (size_t)mr * H, st)) return -1;
                    DEV(cmlb200_add_f32(d->h + (size_t)r0 * H, d->tmp, (size_t)mr * H, st));
                }
            }
        } else {
            if (!tiled_att) DEV(cmlb200_f32_to_bf16(d->att, d->b_a, (size_t)rows * d->qw_l, st));
            if (proj_residual_bf16(d, &L->wo, d->b_a, rows)) return -1;
            DEV(cmlb200_rmsnorm(d->h, (const uint16_t*)L->n2, rows, H, c->rms_norm_eps, NULL, d->b_a, st));
            DEV(cmlb200_gemm_bf16(&L->wg, d->b_a, d->b_c, rows, st));
            DEV(cmlb200_gemm_bf16_ex(&L->wu, d->b_a, rows, CMLB200_GEMM_SWIGLU_BF16, d->b_c, d->b_c, st));   /* silu(gate) * up, in place */
            if (proj_residual_bf16(d, &L->wd, d->b_c, rows)) return -1;
        }
    }
    if (only_layer >= 0) return 0;              /* cml_llama_layer_forward: no head, positions stay where they are */
    if (!with_head) {                           /* cache fill only (cml_llama_prefill_sequence): nobody reads these logits */
        DEV(cmlb200_advance_rows(d->d_cur, rows, mode, seq, st));
        return 0;
    }
    const int split_head = d->vocab_l != c->vocab_size;
    float* lg = split_head ? d->logits_l : d->logits;          /* [rows, vocab_l] */
    if (tiny) {
        DEV(cmlb200_gemv_rmsnorm(&d->lm_head, NULL, d->h, (const uint16_t*)d->fnorm, c->rms_norm_eps, lg, rows, 0, st));
    } else if (skinny) {
        DEV(cmlb200_rmsnorm(d->h, (const uint16_t*)d->fnorm, rows, H, c->rms_norm_eps, d->nrm, NULL, st));
        if (lin_f32(d, &d->lm_head, d->nrm, lg, rows, 0)) return -1;
    } else {
        DEV(cmlb200_rmsnorm(d->h, (const uint16_t*)d->fnorm, rows, H, c->rms_norm_eps, NULL, d->b_a, st));
        DEV(cmlb200_gemm_bf16_ex(&d->lm_head, d->b_a, rows, CMLB200_GEMM_OUT_F32, lg, NULL, st));
    }
    if (split_head && with_head == 1) {                        /* full logits wanted: all-gather the slices, put them side by side */
        if (cml_nccl_allgather_bytes(d->comm, d->logits_l, d->logits_g, (size_t)rows * d->vocab_l * 4, st)) return -1;
        DEV(cmlb200_gather_columns(d->logits_g, d->tp, rows, d->vocab_l, d->logits, st));
    }
    DEV(cmlb200_advance_rows(d->d_cur, rows, mode, seq, st));
    return 0;
}

static int enqueue_forward(DevModel* d, int rows, int mode, int seq, int plan_limit) {
    return enqueue_forward_ex(d, rows, mode, seq, plan_limit, -1, 1);
}

/* The peer-memory all-reduces wait for a peer for a bounded time (seconds, then a status word and a
 * failed call). Ranks may reach a call further apart than that: one is still reading its weights,
 * or was descheduled. A 4-byte ncclAllReduce at the head of every call lines the ranks' streams
 * up first (NCCL waits without a limit); inside a call the ranks then stay within a kernel's
 * length of one another. */
static int tp_line_up(DevModel* d) {
    if (d->tp <= 1 || !d->comm || !d->lineup || !(d->ar_ok || d->arb_ok)) return 0;
    return cml_nccl_allreduce_sum_f32(d->comm, d->lineup, 4, d->stream);
}

/* One forward call. with_logits: the fp32 logits of every row come back as a host tensor (what
 * C-ML's forward returns); without, the head is skipped and a 1 x 1 placeholder is returned. */
static Tensor* run_forward(CMLLLaMAModel* model, const int* token_ids, int rows, int mode, int seq, int with_logits, const char* who) {
    DevModel* d = dm_find(model);
    if (!model_ready(model, d)) { LOG_ERROR("%s: weights are not loaded", who); return NULL; }
    const CMLLLaMAConfig* c = &model->config;
    int max_pos = 0;
    if (mode == 0) {
        if (seq >= d->max_batch) { LOG_ERROR("%s: sequence %d outside the configured batch of %d", who, seq, d->max_batch); return NULL; }
        max_pos = d->h_cur[seq] + rows;
    } else {
        if (rows > d->max_batch) { LOG_ERROR("%s: batch %d exceeds the configured maximum %d", who, rows, d->max_batch); return NULL; }
        for (int b = 0; b < rows; b++) if (d->h_cur[b] + 1 > max_pos) max_pos = d->h_cur[b] + 1;
    }
    if (max_pos > c->max_seq_len) {                     /* cache overflow, as src/nn/llm_ops.c:133-137 */
        LOG_ERROR("%s: cache overflow (%d > %d)", who, max_pos, c->max_seq_len);
        return NULL;
    }
    int shape[2] = {with_logits ? rows : 1, with_logits ? c->vocab_size : 1};
    Tensor* out = cml_tensor_alloc(DTYPE_FLOAT32, shape, 2, !with_logits);
    if (!out) return NULL;
    if (CML_DEV_FAIL(cmlb200_memcpy_h2d(d->d_tokens, token_ids, (size_t)rows * 4, d->stream), who) || tp_line_up(d) ||
        enqueue_forward_ex(d, rows, mode, seq, max_pos - 1, -1, with_logits) ||
        (with_logits && CML_DEV_FAIL(cmlb200_memcpy_d2h(out->data, d->logits, (size_t)rows * c->vocab_size * 4, d->stream), who)) ||
        CML_DEV_FAIL(cmlb200_stream_sync(d->stream), who)) {
        tensor_free(out);
        return NULL;
    }
    if (dm_check_waits(d, who)) { tensor_free(out); return NULL; }
    if (mode == 0) d->h_cur[seq] += rows;
    else for (int b = 0; b < rows; b++) d->h_cur[b] += 1;
    model->current_seq_len = d->h_cur[0];
    for (int i = 0; i < model->num_layers; i++) model->layers[i]->kv_cache->current_len = d->h_cur[0];
    return out;
}

Tensor* cml_llama_forward(CMLLLaMAModel* model, const int* token_ids, int seq_len) {
    if (!model || !token_ids || seq_len <= 0) { LOG_ERROR("cml_llama_forward: invalid arguments"); return NULL; }
    if (!model->embed_tokens) { LOG_ERROR("cml_llama_forward: embed_tokens not loaded"); return NULL; }
    return run_forward(model, token_ids, seq_len, 0, 0, 1, "cml_llama_forward");
}

Tensor* cml_llama_forward_batch(CMLLLaMAModel* model, const int* token_ids, int batch) {
    if (!model || !token_ids || batch <= 0) { LOG_ERROR("cml_llama_forward_batch: invalid arguments"); return NULL; }
    return run_forward(model, token_ids, batch, 1, 0, 1, "cml_llama_forward_batch");
}

int cml_llama_prefill_sequence(CMLLLaMAModel* model, int seq, const int* token_ids, int seq_len) {
    if (!model || !token_ids || seq_len <= 0 || seq < 0) { LOG_ERROR("cml_llama_prefill_sequence: invalid arguments"); return -1; }
    Tensor* t = run_forward(model, token_ids, seq_len, 0, seq, 0, "cml_llama_prefill_sequence");
    if (!t) return -1;
    tensor_free(t);
    return 0;
}

/* One decode step and its greedy pick, enqueued: the next token of every sequence into d->d_tokens.
 * With a split vocabulary projection no logits travel: every rank reduces its slice to one
 * (value, index) pair per row, the pairs are all-gathered (8 bytes per row and rank) and merged. */
static int enqueue_greedy_step(DevModel* d, int batch, int plan_limit) {
    const CMLLLaMAConfig* c = &d->key->config;
    void* st = d->stream;
    if (d->vocab_l == c->vocab_size) {
        if (enqueue_forward(d, batch, 1, 0, plan_limit)) return -1;
        DEV(cmlb200_argmax(d->logits, batch, c->vocab_size, d->d_tokens, st));
        return 0;
    }
    if (enqueue_forward_ex(d, batch, 1, 0, plan_limit, -1, 2)) return -1;
    DEV(cmlb200_argmax_slice(d->logits_l, batch, d->vocab_l, d->rank * d->vocab_l, d->pairs, st));
    if (cml_nccl_allgather_bytes(d->comm, d->pairs, d->pairs + 2 * SKINNY_ROWS, (size_t)batch * 8, st)) return -1;
    DEV(cmlb200_argmax_merge(d->pairs + 2 * SKINNY_ROWS, d->tp, batch, d->d_tokens, st));
    return 0;
}

int cml_llama_decode_greedy(CMLLLaMAModel* model, const int* first_tokens, int batch, int steps, int* out_tokens, float* elapsed_ms) {
    if (!model || !first_tokens || !out_tokens || batch <= 0 || steps <= 0) { LOG_ERROR("cml_llama_decode_greedy: invalid arguments"); return -1; }
    DevModel* d = dm_find(model);
    if (!model_ready(model, d)) { LOG_ERROR("cml_llama_decode_greedy: weights are not loaded"); return -1; }
    const CMLLLaMAConfig* c = &model->config;
    if (batch > d->max_batch) { LOG_ERROR("cml_llama_decode_greedy: batch %d exceeds the configured maximum %d", batch, d->max_batch); return -1; }
    int max_pos = 0;
    for (int b = 0; b < batch; b++) if (d->h_cur[b] + steps > max_pos) max_pos = d->h_cur[b] + steps;
    if (max_pos > c->max_seq_len) { LOG_ERROR("cml_llama_decode_greedy: cache overflow (%d > %d)", max_pos, c->max_seq_len); return -1; }
    void* st = d->stream;
    DEV(cmlb200_memcpy_h2d(d->d_tokens, first_tokens, (size_t)batch * 4, st));
    const int quirks = (d->flags & CML_B200_REFERENCE_QUIRKS) != 0;
    int splits = quirks ? 1 : (max_pos - 1 + ATT_CHUNK) / ATT_CHUNK;
    if (splits > d->att_splits_cap) splits = d->att_splits_cap;
    /* every step of the loop sees the same attention geometry: `splits` chunks of ATT_CHUNK keys */
    int plan_limit = splits * ATT_CHUNK - 1;
    if (plan_limit > c->max_seq_len - 1) plan_limit = c->max_seq_len - 1;
    void *e0 = NULL, *e1 = NULL;
    if (tp_line_up(d)) return -1;
    DEV(cmlb200_event_create(&e0));
    DEV(cmlb200_event_create(&e1));
    DEV(cmlb200_event_record(e0, st));
    int s0 = 0;
    if (!d->graph || d->graph_batch != batch || d->graph_splits != splits) {
        if (d->graph) { cmlb200_graph_destroy(d->graph); d->graph = NULL; }
        /* The first step runs eagerly: first-use initialisation inside the kernels' launchers
         * (function attributes, scratch allocation) must not happen during stream capture. */
        if (enqueue_greedy_step(d, batch, plan_limit)) return -1;
        DEV(cmlb200_memcpy_d2d(d->d_hist, d->d_tokens, (size_t)batch * 4, st));
        DEV(cmlb200_stream_sync(st));
        s0 = 1;
        if (steps > 1) {
            DEV(cmlb200_graph_begin(st));
            int rc = enqueue_greedy_step(d, batch, plan_limit);
            void* g = NULL;
            if (CML_DEV_FAIL(cmlb200_graph_end(st, &g), "cml_llama_decode_greedy") || rc) { if (g) cmlb200_graph_destroy(g); return -1; }
            d->graph = g;
            d->graph_batch = batch;
            d->graph_splits = splits;
        }
    }
    for (int s = s0; s < steps; s++) {
        DEV(cmlb200_graph_launch(d->graph, st));
        DEV(cmlb200_memcpy_d2d(d->d_hist + (size_t)s * batch, d->d_tokens, (size_t)batch * 4, st));
    }
    DEV(cmlb200_event_record(e1, st));
    float ms = 0.f;
    DEV(cmlb200_event_elapsed_ms(e0, e1, &ms));
    DEV(cmlb200_memcpy_d2h(out_tokens, d->d_hist, (size_t)steps * batch * 4, st));
    DEV(cmlb200_stream_sync(st));
    cmlb200_event_destroy(e0);
    cmlb200_event_destroy(e1);
    if (dm_check_waits(d, "cml_llama_decode_greedy")) return -1;
    if (elapsed_ms) *elapsed_ms = ms;
    for (int b = 0; b < batch; b++) d->h_cur[b] += steps;
    model->current_seq_len = d->h_cur[0];
    for (int i = 0; i < model->num_layers; i++) model->layers[i]->kv_cache->current_len = d->h_cur[0];
    return 0;
}

/* ---- sampling (src/nn/llama.c:614-737) ----------------------------------------------------------- */
typedef struct { float value; int index; } LogitEntry;
static int entry_cmp_desc(const void* a, const void* b) {
    const float va = ((const LogitEntry*)a)->value, vb = ((const LogitEntry*)b)->value;
    return va > vb ? -1 : (va < vb ? 1 : 0);
}

int cml_llama_sample_token(Tensor* logits, const CMLGenerationConfig* config) {
    if (!logits || !config || !logits->data) return -1;
    const float* data = (const float*)logits->data;
    int vocab;
    const float* row;
    if (logits->ndim == 2) { vocab = logits->shape[1]; row = data + (size_t)(logits->shape[0] - 1) * vocab; }
    else if (logits->ndim == 1) { vocab = logits->shape[0]; row = data; }
    else { LOG_ERROR("cml_llama_sample_token: unexpected logits ndim=%d", logits->ndim); return -1; }
    if (!config->do_sample || config->temperature <= 0.0f) {        /* greedy: first strict maximum */
        int best = 0;
        for (int i = 1; i < vocab; i++) if (row[i] > row[best]) best = i;
        return best;
    }
    LogitEntry* e = (LogitEntry*)malloc((size_t)vocab * sizeof *e);
    if (!e) return -1;
    const float inv_t = 1.0f / config->temperature;
    for (int i = 0; i < vocab; i++) { e[i].value = row[i] * inv_t; e[i].index = i; }
    qsort(e, (size_t)vocab, sizeof *e, entry_cmp_desc);
    int k = config->top_k;
    if (k <= 0 || k > vocab) k = vocab;
    const float mx = e[0].value;
    float sum = 0.f;
    for (int i = 0; i < k; i++) { e[i].value = expf(e[i].value - mx); sum += e[i].value; }
    for (int i = 0; i < k; i++) e[i].value /= sum;
    int cutoff = k;
    if (config->top_p > 0.0f && config->top_p < 1.0f) {
        float cum = 0.f;
        for (int i = 0; i < k; i++) { cum += e[i].value; if (cum >= config->top_p) { cutoff = i + 1; break; } }
    }
    if (cutoff < k) {
        float rs = 0.f;
        for (int i = 0; i < cutoff; i++) rs += e[i].value;
        if (rs > 0.f) for (int i = 0; i < cutoff; i++) e[i].value /= rs;
    }
    const float r = (float)rand() / (float)RAND_MAX;
    float acc = 0.f;
    int id = e[0].index;
    for (int i = 0; i < cutoff; i++) { acc += e[i].value; if (r <= acc) { id = e[i].index; break; } }
    free(e);
    return id;
}


void cml_llama_set_tokenizer_functions(CMLTokenizerEncodeFn encode, CMLTokenizerDecodeFn decode) {
    g_tok_encode = encode;
    g_tok_decode = decode;
}

CMLGenerationResult* cml_llama_generate(CMLLLaMAModel* model, const char* prompt, const CMLGenerationConfig* config) {
    if (!model || !prompt || !config) { LOG_ERROR("cml_llama_generate: NULL argument"); return NULL; }
    if (!model->weights_loaded) { LOG_ERROR("cml_llama_generate: weights not loaded"); return NULL; }
    const CMLTokenizerEncodeFn enc = g_tok_encode ? g_tok_encode : cml_tokenizer_encode;
    const CMLTokenizerDecodeFn dec = g_tok_decode ? g_tok_decode : cml_tokenizer_decode;
    int n_prompt = 0;
    int* ids = (model->tokenizer && enc) ? enc(model->tokenizer, prompt, &n_prompt) : NULL;
    if (!ids || n_prompt <= 0) {                     /* no tokenizer: the same failure as src/nn/llama.c:759-763 */
        LOG_ERROR("cml_llama_generate: tokenization failed or empty prompt");
        free(ids);
        return NULL;
    }
    const int budget = config->max_new_tokens > 0 ? config->max_new_tokens : 0;
    CMLGenerationResult* res = (CMLGenerationResult*)calloc(1, sizeof *res);
    if (res) res->token_ids = (int*)malloc((size_t)(n_prompt + budget) * sizeof(int));
    if (!res || !res->token_ids) { free(ids); free(res); return NULL; }
    memcpy(res->token_ids, ids, (size_t)n_prompt * sizeof(int));
    res->num_tokens = n_prompt;

    cml_llama_reset(model);
    struct timespec t0, t1;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    Tensor* logits = cml_llama_forward(model, ids, n_prompt);       /* prefill; the sampler reads the last row */
    free(ids);
    if (!logits) {
        LOG_ERROR("cml_llama_generate: prefill forward failed");
        cml_generation_result_free(res);
        return NULL;
    }
    for (int step = 0; step < budget; step++) {
        int next = cml_llama_sample_token(logits, config);
        tensor_free(logits);
        logits = NULL;
        if (next < 0) { LOG_ERROR("cml_llama_generate: sampling failed at step %d", step); break; }
        res->token_ids[res->num_tokens++] = next;
        if (next == config->eos_token_id) break;
        if (model->current_seq_len >= model->config.max_seq_len) { LOG_WARNING("cml_llama_generate: max sequence length reached"); break; }
        logits = cml_llama_forward(model, &next, 1);
        if (!logits) { LOG_ERROR("cml_llama_generate: decode forward failed at step %d", step); break; }
    }
    tensor_free(logits);
    clock_gettime(CLOCK_MONOTONIC, &t1);
    const double ms = (double)(t1.tv_sec - t0.tv_sec) * 1e3 + (double)(t1.tv_nsec - t0.tv_nsec) / 1e6;
    res->total_time_ms = (float)ms;
    const int generated = res->num_tokens - n_prompt;
    if (ms > 0.0) res->tokens_per_second = (float)(generated * 1e3 / ms);
    res->text = dec ? dec(model->tokenizer, res->token_ids, res->num_tokens) : NULL;
    LOG_INFO("Generation complete: %d tokens in %.1f ms (%.1f tok/s)", generated, res->total_time_ms, res->tokens_per_second);
    return res;
}

void cml_generation_result_free(CMLGenerationResult* result) {
    if (!result) return;
    free(result->token_ids);
    free(result->text);
    free(result);
}

/* One transformer block on host activations (src/nn/llama.c:454-548): hidden [seq, hidden_size]
 * fp32 in, a new tensor of the same shape out. The rows take positions start_pos .. start_pos+seq-1
 * of sequence 0: their keys and values are written into the layer's device cache at those positions
 * and they attend everything before them. The model's own position counter is left as it was. */
Tensor* cml_llama_layer_forward(CMLLLaMAModel* model, CMLLLaMALayer* layer, Tensor* hidden, int start_pos) {
    if (!model || !layer || !hidden) return NULL;
    const char* who = "cml_llama_layer_forward";
    DevModel* d = dm_find(model);
    if (!model_ready(model, d)) { LOG_ERROR("%s: weights are not loaded", who); return NULL; }
    const CMLLLaMAConfig* c = &model->config;
    int li = -1;
    for (int i = 0; i < model->num_layers; i++) if (model->layers[i] == layer) li = i;
    if (li < 0) { LOG_ERROR("%s: the layer does not belong to the model", who); return NULL; }
    if (hidden->ndim != 2 || hidden->shape[1] != c->hidden_size || !hidden->data) {
        LOG_ERROR("%s: hidden must be [seq, %d] fp32", who, c->hidden_size);
        return NULL;
    }
    const int rows = hidden->shape[0];
    if (rows <= 0 || rows > d->max_rows) { LOG_ERROR("%s: seq %d outside 1..%d", who, rows, d->max_rows); return NULL; }
    if (start_pos < 0 || start_pos + rows > c->max_seq_len) { LOG_ERROR("%s: cache overflow (%d + %d > %d)", who, start_pos, rows, c->max_seq_len); return NULL; }
    int shape[2] = {rows, c->hidden_size};
    Tensor* out = cml_tensor_alloc(DTYPE_FLOAT32, shape, 2, false);
    if (!out) return NULL;
    const size_t bytes = (size_t)rows * c->hidden_size * sizeof(float);
    const int saved = d->h_cur[0];
    int ok = !CML_DEV_FAIL(cmlb200_memcpy_h2d(d->h, hidden->data, bytes, d->stream), who) &&
             !CML_DEV_FAIL(cmlb200_memcpy_h2d(d->d_cur, &start_pos, sizeof(int), d->stream), who) &&
             !CML_DEV_FAIL(cmlb200_stream_sync(d->stream), who) &&          /* start_pos is a stack variable */
             !tp_line_up(d) && !enqueue_forward_ex(d, rows, 0, 0, start_pos + rows - 1, li, 0) &&
             !CML_DEV_FAIL(cmlb200_memcpy_d2h(out->data, d->h, bytes, d->stream), who);
    /* put the model's own position back whatever happened */
    if (CML_DEV_FAIL(cmlb200_memcpy_h2d(d->d_cur, &saved, sizeof(int), d->stream), who) || CML_DEV_FAIL(cmlb200_stream_sync(d->stream), who)) ok = 0;
    if (dm_check_waits(d, who)) ok = 0;
    if (!ok) { tensor_free(out); return NULL; }
    return out;
}

void cml_llama_reset(CMLLLaMAModel* model) {
    if (!model) return;
    DevModel* d = dm_find(model);
    if (d && d->d_cur) {
        cmlb200_memset(d->d_cur, 0, (size_t)d->max_batch * 4, d->stream);
        cmlb200_stream_sync(d->stream);
        memset(d->h_cur, 0, (size_t)d->max_batch * sizeof(int));
    }
    for (int i = 0; i < model->num_layers; i++)
        if (model->layers[i] && model->layers[i]->kv_cache) model->layers[i]->kv_cache->current_len = 0;
    model->current_seq_len = 0;
}

/* Rolls sequence `seq` back to new_len tokens: the cache entries below new_len stay valid, the
 * next call continues at position new_len (speculative decoding drops rejected drafts this way).
 * A model without device state (weights not loaded yet) only accepts new_len == 0. */
int cml_llama_truncate(CMLLLaMAModel* model, int seq, int new_len) {
    if (!model || seq < 0 || new_len < 0) { LOG_ERROR("cml_llama_truncate: invalid arguments"); return -1; }
    DevModel* d = dm_find(model);
    if (!d || !d->d_cur) {
        if (new_len == 0 && seq == 0) return 0;
        LOG_ERROR("cml_llama_truncate: the model holds no device state");
        return -1;
    }
    if (seq >= d->max_batch) { LOG_ERROR("cml_llama_truncate: sequence %d outside the configured batch of %d", seq, d->max_batch); return -1; }
    if (new_len > d->h_cur[seq]) { LOG_ERROR("cml_llama_truncate: new length %d exceeds the %d cached tokens", new_len, d->h_cur[seq]); return -1; }
    if (new_len == d->h_cur[seq]) return 0;
    if (CML_DEV_FAIL(cmlb200_memcpy_h2d(d->d_cur + seq, &new_len, sizeof(int), d->stream), "cml_llama_truncate") ||
        CML_DEV_FAIL(cmlb200_stream_sync(d->stream), "cml_llama_truncate"))
        return -1;
    d->h_cur[seq] = new_len;
    if (seq == 0) {
        model->current_seq_len = new_len;
        for (int i = 0; i < model->num_layers; i++)
            if (model->layers[i] && model->layers[i]->kv_cache) model->layers[i]->kv_cache->current_len = new_len;
    }
    return 0;
}

void cml_llama_print_config(const CMLLLaMAConfig* config) {
    if (!config) return;
    const int hd = config->hidden_size / config->num_heads;
    const long long layer = (long long)config->hidden_size * config->num_heads * hd + 2LL * config->hidden_size * config->num_kv_heads * hd +
                            3LL * config->hidden_size * config->intermediate_size;
    const long long total = config->num_layers * layer + 2LL * config->vocab_size * config->hidden_size;
    printf("LLaMA Configuration:\n  vocab_size:        %d\n  hidden_size:       %d\n  intermediate_size: %d\n  num_layers:        %d\n"
           "  num_heads:         %d\n  num_kv_heads:      %d\n  head_dim:          %d\n  max_seq_len:       %d\n  rope_theta:        %.1f\n"
           "  rms_norm_eps:      %.1e\n  est. parameters:   %.1fB\n",
           config->vocab_size, config->hidden_size, config->intermediate_size, config->num_layers, config->num_heads,
           config->num_kv_heads, hd, config->max_seq_len, config->rope_theta, config->rms_norm_eps, total / 1e9);
}
