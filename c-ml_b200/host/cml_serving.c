/* Continuous-batching scheduler (include/nn/serving.h, src/nn/serving.c in the C-ML tree): a
 * circular queue of submitted requests, an active batch of at most max_batch_size of them, status
 * and timing bookkeeping. As in C-ML this layer does not run the model: cml_serving_step admits
 * queued requests and moves them PREFILL -> DECODING, and whoever runs the model appends tokens
 * and calls cml_serving_finish_request.
 *
 * cml_serving_run_llama (no C-ML counterpart) is such a runner for a device-resident LLaMA: every
 * active request owns one of the model's batch slots, a newly admitted request is prefilled into
 * its slot (cml_llama_truncate + cml_llama_prefill_sequence), and all slots take one greedy decode
 * step per iteration through the batched forward, so requests of different lengths start and
 * finish independently while the weights are streamed once per step for all of them. */
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "cml_internal.h"

static double wall_ms(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return 1e3 * (double)ts.tv_sec + 1e-6 * (double)ts.tv_nsec;
}

static void request_free(CMLSequenceRequest* r) {
    if (!r) return;
    free(r->prompt_tokens);
    free(r->generated_tokens);
    free(r);
}

/* queued requests first (oldest first), then the active batch */
static CMLSequenceRequest* lookup(CMLServingContext* ctx, int request_id) {
    if (!ctx) return NULL;
    for (int i = 0; i < ctx->queue_count; i++) {
        CMLSequenceRequest* r = ctx->queue[(ctx->queue_head + i) % ctx->queue_capacity];
        if (r && r->request_id == request_id) return r;
    }
    for (int i = 0; i < ctx->batch_size; i++)
        if (ctx->active_batch[i] && ctx->active_batch[i]->request_id == request_id) return ctx->active_batch[i];
    return NULL;
}

CMLServingConfig cml_serving_default_config(void) {
    CMLServingConfig c = {.max_batch_size = 8, .max_queue_size = 256, .max_seq_len = 2048, .max_new_tokens_default = 256,
                          .temperature_default = 0.8f, .top_p_default = 0.9f};
    return c;
}

CMLServingContext* cml_serving_create(const CMLServingConfig* config) {
    if (!config) { LOG_ERROR("cml_serving_create: NULL config"); return NULL; }
    CMLServingContext* ctx = (CMLServingContext*)calloc(1, sizeof *ctx);
    if (!ctx) { LOG_ERROR("cml_serving_create: allocation failed"); return NULL; }
    ctx->config = *config;
    if (ctx->config.max_batch_size <= 0) ctx->config.max_batch_size = 8;
    if (ctx->config.max_batch_size > CML_SERVING_MAX_BATCH) ctx->config.max_batch_size = CML_SERVING_MAX_BATCH;
    if (ctx->config.max_queue_size <= 0) ctx->config.max_queue_size = 256;
    if (ctx->config.max_queue_size > CML_SERVING_MAX_QUEUE) ctx->config.max_queue_size = CML_SERVING_MAX_QUEUE;
    ctx->queue_capacity = ctx->config.max_queue_size;
    ctx->queue = (CMLSequenceRequest**)calloc((size_t)ctx->queue_capacity, sizeof *ctx->queue);
    ctx->active_batch = (CMLSequenceRequest**)calloc((size_t)ctx->config.max_batch_size, sizeof *ctx->active_batch);
    if (!ctx->queue || !ctx->active_batch) {
        LOG_ERROR("cml_serving_create: queue allocation failed");
        free(ctx->queue); free(ctx->active_batch); free(ctx);
        return NULL;
    }
    ctx->next_request_id = 1;
    LOG_INFO("Serving context created: max_batch=%d, max_queue=%d", ctx->config.max_batch_size, ctx->config.max_queue_size);
    return ctx;
}

void cml_serving_free(CMLServingContext* ctx) {
    if (!ctx) return;
    for (int i = 0; i < ctx->queue_count; i++) request_free(ctx->queue[(ctx->queue_head + i) % ctx->queue_capacity]);
    for (int i = 0; i < ctx->batch_size; i++) request_free(ctx->active_batch[i]);
    LOG_INFO("Serving context freed (total_requests=%zu, completed=%zu)", ctx->stats.total_requests, ctx->stats.completed_requests);
    free(ctx->queue);
    free(ctx->active_batch);
    free(ctx);
}

void cml_serving_set_kv_cache(CMLServingContext* ctx, CMLPagedKVCache* cache) {
    if (!ctx) return;
    ctx->kv_cache = cache;
    LOG_INFO("Paged KV cache set on serving context");
}

int cml_serving_submit(CMLServingContext* ctx, const int* prompt_tokens, int num_tokens, int max_new_tokens) {
    if (!ctx) { LOG_ERROR("cml_serving_submit: NULL context"); return -1; }
    if (!prompt_tokens || num_tokens <= 0) { LOG_ERROR("cml_serving_submit: invalid prompt (tokens=%p, n=%d)", (const void*)prompt_tokens, num_tokens); return -1; }
    if (ctx->queue_count >= ctx->queue_capacity) { LOG_WARNING("cml_serving_submit: queue full (%d/%d)", ctx->queue_count, ctx->queue_capacity); return -1; }
    CMLSequenceRequest* r = (CMLSequenceRequest*)calloc(1, sizeof *r);
    if (!r) { LOG_ERROR("cml_serving_submit: request allocation failed"); return -1; }
    r->max_new_tokens = max_new_tokens > 0 ? max_new_tokens : ctx->config.max_new_tokens_default;
    r->gen_capacity = r->max_new_tokens;
    r->prompt_tokens = (int*)malloc((size_t)num_tokens * sizeof(int));
    r->generated_tokens = (int*)calloc((size_t)(r->gen_capacity > 0 ? r->gen_capacity : 1), sizeof(int));
    if (!r->prompt_tokens || !r->generated_tokens) {
        LOG_ERROR("cml_serving_submit: token buffer allocation failed");
        request_free(r);
        return -1;
    }
    memcpy(r->prompt_tokens, prompt_tokens, (size_t)num_tokens * sizeof(int));
    r->num_prompt_tokens = num_tokens;
    r->request_id = ctx->next_request_id++;
    r->temperature = ctx->config.temperature_default;
    r->top_p = ctx->config.top_p_default;
    r->status = CML_SEQ_STATUS_QUEUED;
    r->paged_seq_id = -1;
    r->submit_time_ms = wall_ms();
    ctx->queue[ctx->queue_tail] = r;
    ctx->queue_tail = (ctx->queue_tail + 1) % ctx->queue_capacity;
    ctx->queue_count++;
    ctx->stats.total_requests++;
    return r->request_id;
}

int cml_serving_step(CMLServingContext* ctx) {
    if (!ctx) return 0;
    while (ctx->queue_count > 0 && ctx->batch_size < ctx->config.max_batch_size) {     /* oldest request first */
        CMLSequenceRequest* r = ctx->queue[ctx->queue_head];
        ctx->queue[ctx->queue_head] = NULL;
        ctx->queue_head = (ctx->queue_head + 1) % ctx->queue_capacity;
        ctx->queue_count--;
        r->status = CML_SEQ_STATUS_PREFILL;
        ctx->active_batch[ctx->batch_size++] = r;
        ctx->stats.active_sequences++;
    }
    /* the prefill compute is the runner's business: an admitted request counts as decoding */
    for (int i = 0; i < ctx->batch_size; i++) {
        CMLSequenceRequest* r = ctx->active_batch[i];
        if (r && r->status == CML_SEQ_STATUS_PREFILL) {
            r->status = CML_SEQ_STATUS_DECODING;
            r->first_token_time_ms = wall_ms();
        }
    }
    return ctx->batch_size;
}

CMLSequenceStatus cml_serving_get_status(CMLServingContext* ctx, int request_id) {
    const CMLSequenceRequest* r = lookup(ctx, request_id);
    return r ? r->status : CML_SEQ_STATUS_ERROR;
}

const int* cml_serving_get_tokens(CMLServingContext* ctx, int request_id, int* out_count) {
    if (out_count) *out_count = 0;
    const CMLSequenceRequest* r = lookup(ctx, request_id);
    if (!r) return NULL;
    if (out_count) *out_count = r->num_generated;
    return r->generated_tokens;
}

int cml_serving_finish_request(CMLServingContext* ctx, int request_id) {
    if (!ctx) return -1;
    int at = -1;
    for (int i = 0; i < ctx->batch_size && at < 0; i++)
        if (ctx->active_batch[i] && ctx->active_batch[i]->request_id == request_id) at = i;
    if (at < 0) { LOG_WARNING("cml_serving_finish_request: request %d not in active batch", request_id); return -1; }
    CMLSequenceRequest* r = ctx->active_batch[at];
    r->status = CML_SEQ_STATUS_FINISHED;
    r->finish_time_ms = wall_ms();
    CMLServingStats* s = &ctx->stats;
    s->completed_requests++;
    s->total_tokens_generated += (size_t)r->num_generated;
    if (s->active_sequences > 0) s->active_sequences--;
    s->total_time_ms += r->finish_time_ms - r->submit_time_ms;
    if (r->first_token_time_ms > 0.0) {                       /* running mean over the completed requests */
        const double n = (double)s->completed_requests;
        s->avg_time_to_first_token_ms = (s->avg_time_to_first_token_ms * (n - 1.0) + (r->first_token_time_ms - r->submit_time_ms)) / n;
    }
    if (s->total_time_ms > 0.0) s->avg_tokens_per_second = (double)s->total_tokens_generated / (s->total_time_ms / 1000.0);
    request_free(r);
    ctx->active_batch[at] = ctx->active_batch[ctx->batch_size - 1];     /* the last active request takes the hole */
    ctx->active_batch[--ctx->batch_size] = NULL;
    return 0;
}

CMLServingStats cml_serving_get_stats(const CMLServingContext* ctx) {
    CMLServingStats none;
    memset(&none, 0, sizeof none);
    return ctx ? ctx->stats : none;
}

/* ---- a runner over a device-resident LLaMA ---------------------------------------------------------
 * Runs until the queue and the batch are empty, or for max_steps batched decode steps (0: no
 * limit). A request's slot is kept in paged_seq_id. on_finish, when given, sees every request
 * (its generated_tokens are complete) just before cml_serving_finish_request frees it. eos_token
 * < 0: requests only end at max_new_tokens or when the model's max_seq_len is reached. Returns the
 * number of decode steps taken, -1 on error. The model must have been given
 * cml_llama_set_options(model, flags, max_batch >= the context's max_batch_size) before loading. */
int cml_serving_run_llama(CMLServingContext* ctx, CMLLLaMAModel* model, int eos_token, int max_steps,
                          void (*on_finish)(const CMLSequenceRequest* request, void* user), void* user) {
    if (!ctx || !model) { LOG_ERROR("cml_serving_run_llama: NULL argument"); return -1; }
    const int B = ctx->config.max_batch_size, vocab = model->config.vocab_size, max_len = model->config.max_seq_len;
    int* slot_req = (int*)malloc((size_t)B * sizeof(int));            /* request id per model slot, 0 = free */
    int* step_tok = (int*)calloc((size_t)B, sizeof(int));
    int steps = 0, rc = 0;
    if (!slot_req || !step_tok) { free(slot_req); free(step_tok); return -1; }
    memset(slot_req, 0, (size_t)B * sizeof(int));
    for (int i = 0; i < ctx->batch_size; i++)                          /* requests admitted by an earlier call keep their slots */
        if (ctx->active_batch[i] && ctx->active_batch[i]->paged_seq_id >= 0 && ctx->active_batch[i]->paged_seq_id < B)
            slot_req[ctx->active_batch[i]->paged_seq_id] = ctx->active_batch[i]->request_id;
    CMLGenerationConfig greedy = cml_generation_default_config();
    greedy.do_sample = false;
    while (rc == 0 && (ctx->queue_count > 0 || ctx->batch_size > 0) && (max_steps <= 0 || steps < max_steps)) {
        cml_serving_step(ctx);
        /* prefill whoever has no slot yet; its first token comes from the prompt's last row */
        for (int i = 0; i < ctx->batch_size && rc == 0; i++) {
            CMLSequenceRequest* r = ctx->active_batch[i];
            if (r->paged_seq_id >= 0) continue;
            int s = 0;
            while (s < B && slot_req[s]) s++;
            if (s == B) { LOG_ERROR("cml_serving_run_llama: no free model slot"); rc = -1; break; }
            if (r->num_prompt_tokens + 1 > max_len) { r->status = CML_SEQ_STATUS_ERROR; r->paged_seq_id = s; slot_req[s] = r->request_id; continue; }
            slot_req[s] = r->request_id;
            r->paged_seq_id = s;
            if (cml_llama_truncate(model, s, 0) ||
                (r->num_prompt_tokens > 1 && cml_llama_prefill_sequence(model, s, r->prompt_tokens, r->num_prompt_tokens - 1))) { rc = -1; break; }
            r->current_pos = r->num_prompt_tokens - 1;
        }
        if (rc) break;
        /* one batched step: slot s feeds its pending token (the prompt's last one right after the prefill) */
        int live = 0;
        for (int s = 0; s < B; s++) step_tok[s] = 0;
        for (int i = 0; i < ctx->batch_size; i++) {
            CMLSequenceRequest* r = ctx->active_batch[i];
            if (r->status != CML_SEQ_STATUS_DECODING) continue;
            step_tok[r->paged_seq_id] = r->num_generated ? r->generated_tokens[r->num_generated - 1] : r->prompt_tokens[r->num_prompt_tokens - 1];
            live++;
        }
        if (live) {
            for (int s = 0; s < B; s++)                                 /* idle slots take a dummy row at position 0 */
                if (!slot_req[s] && cml_llama_truncate(model, s, 0)) rc = -1;
            Tensor* lg = rc ? NULL : cml_llama_forward_batch(model, step_tok, B);
            if (!lg) { rc = -1; break; }
            steps++;
            for (int i = 0; i < ctx->batch_size; i++) {
                CMLSequenceRequest* r = ctx->active_batch[i];
                if (r->status != CML_SEQ_STATUS_DECODING) continue;
                int row_shape[2] = {1, vocab};
                TensorConfig tc = {.dtype = DTYPE_FLOAT32, .device = DEVICE_CPU, .has_dtype = true, .has_device = true};
                Tensor* row = tensor_from_data((float*)lg->data + (size_t)r->paged_seq_id * vocab, row_shape, 2, &tc);
                const int tok = row ? cml_llama_sample_token(row, &greedy) : -1;
                tensor_free(row);
                if (tok < 0) { rc = -1; break; }
                if (r->num_generated < r->gen_capacity) r->generated_tokens[r->num_generated++] = tok;
                r->current_pos++;
            }
            tensor_free(lg);
        }
        /* retire what is done (finish_request moves the last active request into the hole) */
        for (int i = 0; i < ctx->batch_size && rc == 0;) {
            CMLSequenceRequest* r = ctx->active_batch[i];
            const int last = r->num_generated ? r->generated_tokens[r->num_generated - 1] : -1;
            const int done = r->status == CML_SEQ_STATUS_ERROR || r->num_generated >= r->max_new_tokens ||
                             (eos_token >= 0 && last == eos_token) || r->current_pos + 1 >= max_len;
            if (!done) { i++; continue; }
            if (on_finish) on_finish(r, user);
            slot_req[r->paged_seq_id] = 0;
            cml_serving_finish_request(ctx, r->request_id);
        }
    }
    free(slot_req);
    free(step_tok);
    return rc ? -1 : steps;
}
