/* Speculative decoding (include/nn/speculative.h:15-90, src/nn/speculative.c in the C-ML tree): a
 * draft model proposes K tokens one by one, the target model scores prefix + drafts in ONE call,
 * the longest run of drafts that equal the target's arg-max is kept and one more token (the
 * target's correction, or its bonus prediction after K hits) is appended. The decoder itself is
 * host control flow over two pairs of callbacks, as in C-ML; cml_speculative_llama_* below are
 * callbacks for device-resident CMLLLaMAModels that keep the KV cache between calls, so that a
 * draft step costs one decode row and the verification is a single (K+1)-row call of the skinny
 * GEMM path instead of a re-run of the whole sequence. */
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "cml_internal.h"

static double wall_ms(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return 1e3 * (double)ts.tv_sec + 1e-6 * (double)ts.tv_nsec;
}

/* first index of the strict maximum of row `row` (src/nn/speculative.c:16-36) */
static int row_argmax(const Tensor* logits, int row, int vocab) {
    const float* p = logits && logits->data ? (const float*)logits->data + (size_t)row * vocab : NULL;
    if (!p) return 0;
    int best = 0;
    for (int i = 1; i < vocab; i++) if (p[i] > p[best]) best = i;
    return best;
}

CMLSpeculativeConfig cml_speculative_default_config(void) {
    CMLSpeculativeConfig c = {.num_draft_tokens = 5, .temperature = 0.8f, .top_p = 0.9f, .top_k = 40, .do_sample = true};
    return c;
}

CMLSpeculativeDecoder* cml_speculative_create(const CMLSpeculativeConfig* config, int vocab_size) {
    if (!config) { LOG_ERROR("cml_speculative_create: config is NULL"); return NULL; }
    if (vocab_size <= 0) { LOG_ERROR("cml_speculative_create: vocab_size must be > 0"); return NULL; }
    if (config->num_draft_tokens <= 0 || config->num_draft_tokens > CML_SPEC_MAX_DRAFT_TOKENS) {
        LOG_ERROR("cml_speculative_create: num_draft_tokens must be in [1, %d]", CML_SPEC_MAX_DRAFT_TOKENS);
        return NULL;
    }
    CMLSpeculativeDecoder* d = (CMLSpeculativeDecoder*)calloc(1, sizeof *d);
    if (!d) { LOG_ERROR("cml_speculative_create: allocation failed"); return NULL; }
    d->config = *config;
    d->vocab_size = vocab_size;
    return d;
}

void cml_speculative_free(CMLSpeculativeDecoder* decoder) { free(decoder); }

void cml_speculative_set_draft_model(CMLSpeculativeDecoder* dec, void* ctx, CMLModelForwardFn forward_fn, CMLSampleTokenFn sample_fn) {
    if (!dec) return;
    dec->draft_model_ctx = ctx;
    dec->draft_forward = forward_fn;
    dec->draft_sample = sample_fn;
}

void cml_speculative_set_target_model(CMLSpeculativeDecoder* dec, void* ctx, CMLModelForwardFn forward_fn, CMLSampleTokenFn sample_fn) {
    if (!dec) return;
    dec->target_model_ctx = ctx;
    dec->target_forward = forward_fn;
    dec->target_sample = sample_fn;
}

CMLSpeculativeResult* cml_speculative_decode_step(CMLSpeculativeDecoder* dec, const int* prefix_tokens, int prefix_len) {
    if (!dec) { LOG_ERROR("cml_speculative_decode_step: decoder is NULL"); return NULL; }
    if (!dec->draft_forward || !dec->draft_sample || !dec->target_forward || !dec->target_sample) {
        LOG_ERROR("cml_speculative_decode_step: model callbacks not set");
        return NULL;
    }
    if (!prefix_tokens || prefix_len <= 0) { LOG_ERROR("cml_speculative_decode_step: invalid prefix"); return NULL; }
    int K = dec->config.num_draft_tokens;
    int* seq = (int*)malloc((size_t)(prefix_len + K) * sizeof(int));
    CMLSpeculativeResult* res = (CMLSpeculativeResult*)calloc(1, sizeof *res);
    if (res) res->accepted_tokens = (int*)malloc((size_t)(K + 1) * sizeof(int));
    if (!seq || !res || !res->accepted_tokens) {
        LOG_ERROR("cml_speculative_decode_step: allocation failed");
        free(seq);
        cml_speculative_result_free(res);
        return NULL;
    }
    memcpy(seq, prefix_tokens, (size_t)prefix_len * sizeof(int));

    /* draft: K tokens, each from the draft model's last row; a failed draft call ends the run early */
    const double t0 = wall_ms();
    for (int i = 0; i < K; i++) {
        Tensor* lg = dec->draft_forward(dec->draft_model_ctx, seq, prefix_len + i);
        if (!lg) { LOG_WARNING("draft forward returned NULL at step %d", i); K = i; break; }
        seq[prefix_len + i] = dec->draft_sample(dec->draft_model_ctx, lg, dec->config.temperature);
        tensor_free(lg);
    }
    const double t1 = wall_ms();
    /* verify: one target call over prefix + drafts; row prefix_len - 1 + i predicts draft i */
    Tensor* tl = dec->target_forward(dec->target_model_ctx, seq, prefix_len + K);
    const double t2 = wall_ms();
    if (!tl) {
        LOG_ERROR("target forward returned NULL");
        free(seq);
        cml_speculative_result_free(res);
        return NULL;
    }
    int hits = 0, extra = -1;
    while (hits < K) {
        const int want = row_argmax(tl, prefix_len - 1 + hits, dec->vocab_size);
        if (want != seq[prefix_len + hits]) { extra = want; break; }      /* the target's own token replaces the first miss */
        hits++;
    }
    if (hits == K) extra = row_argmax(tl, prefix_len + K - 1, dec->vocab_size);   /* all accepted: one bonus token */
    tensor_free(tl);
    memcpy(res->accepted_tokens, seq + prefix_len, (size_t)hits * sizeof(int));
    res->accepted_tokens[hits] = extra;
    res->num_accepted = hits + 1;
    res->num_drafted = K;
    res->num_verified = 1;
    res->acceptance_rate = K > 0 ? (float)hits / (float)K : 0.0f;
    res->draft_time_ms = t1 - t0;
    res->verify_time_ms = t2 - t1;
    res->total_time_ms = t2 - t0;
    dec->total_drafted += (size_t)K;
    dec->total_accepted += (size_t)hits;
    dec->total_steps++;
    free(seq);
    return res;
}

void cml_speculative_result_free(CMLSpeculativeResult* result) {
    if (!result) return;
    free(result->accepted_tokens);
    free(result);
}

float cml_speculative_acceptance_rate(const CMLSpeculativeDecoder* dec) {
    return dec && dec->total_drafted ? (float)dec->total_accepted / (float)dec->total_drafted : 0.0f;
}

/* ---- callbacks for device-resident LLaMA models -------------------------------------------------
 * The decoder hands every call the whole token sequence. The context remembers which tokens the
 * model's KV cache holds; a call rolls the cache back to the longest common prefix and forwards
 * only the rest, but never fewer than min_rows rows: 1 for a draft model (its sampler reads the last
 * row), CML_SPEC_MAX_DRAFT_TOKENS + 1 for a target model (the decoder reads the rows of the last K
 * drafts and the one before them). The returned tensor is [seq_len, vocab] as the callback type
 * demands; the rows of the reused prefix are zero. */
CMLSpeculativeLlama* cml_speculative_llama_create(CMLLLaMAModel* model, bool is_target) {
    if (!model) { LOG_ERROR("cml_speculative_llama_create: NULL model"); return NULL; }
    CMLSpeculativeLlama* s = (CMLSpeculativeLlama*)calloc(1, sizeof *s);
    if (!s) return NULL;
    s->model = model;
    s->min_rows = is_target ? CML_SPEC_MAX_DRAFT_TOKENS + 1 : 1;
    s->capacity = model->config.max_seq_len > 0 ? model->config.max_seq_len : 1;
    s->cached_tokens = (int*)malloc((size_t)s->capacity * sizeof(int));
    if (!s->cached_tokens) { free(s); return NULL; }
    cml_llama_reset(model);
    return s;
}

void cml_speculative_llama_free(CMLSpeculativeLlama* ctx) {
    if (!ctx) return;
    free(ctx->cached_tokens);
    free(ctx);
}

Tensor* cml_speculative_llama_forward(void* model_ctx, const int* token_ids, int seq_len) {
    CMLSpeculativeLlama* s = (CMLSpeculativeLlama*)model_ctx;
    if (!s || !s->model || !token_ids || seq_len <= 0) { LOG_ERROR("cml_speculative_llama_forward: invalid arguments"); return NULL; }
    if (seq_len > s->capacity) { LOG_ERROR("cml_speculative_llama_forward: %d tokens exceed max_seq_len %d", seq_len, s->capacity); return NULL; }
    int keep = 0, lim = seq_len - s->min_rows;
    if (lim > s->cached_len) lim = s->cached_len;
    while (keep < lim && s->cached_tokens[keep] == token_ids[keep]) keep++;
    if (cml_llama_truncate(s->model, 0, keep)) return NULL;
    s->cached_len = keep;
    const int vocab = s->model->config.vocab_size;
    Tensor* part = cml_llama_forward(s->model, token_ids + keep, seq_len - keep);
    if (!part) return NULL;
    int shape[2] = {seq_len, vocab};
    Tensor* full = cml_tensor_alloc(DTYPE_FLOAT32, shape, 2, true);
    if (full) memcpy((float*)full->data + (size_t)keep * vocab, part->data, (size_t)(seq_len - keep) * vocab * sizeof(float));
    tensor_free(part);
    if (!full) return NULL;
    memcpy(s->cached_tokens + keep, token_ids + keep, (size_t)(seq_len - keep) * sizeof(int));
    s->cached_len = seq_len;
    s->rows_computed += (size_t)(seq_len - keep);
    s->calls++;
    return full;
}

/* temperature <= 0: first strict maximum of the last row; otherwise a draw from softmax(logits / T)
 * through cml_llama_sample_token (no top-k / top-p cut). */
int cml_speculative_llama_sample(void* model_ctx, Tensor* logits, float temperature) {
    (void)model_ctx;
    if (!logits || !logits->data || logits->ndim != 2) return 0;
    if (temperature <= 0.0f) return row_argmax(logits, logits->shape[0] - 1, logits->shape[1]);
    CMLGenerationConfig g = cml_generation_default_config();
    g.temperature = temperature;
    g.top_p = 1.0f;
    g.top_k = 0;
    g.do_sample = true;
    return cml_llama_sample_token(logits, &g);
}
