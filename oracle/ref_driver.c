/*
 * ref_driver.c -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * Flat-pointer wrappers around the *compiled C-ML reference* so the tests and
 * the benchmark's CPU-baseline leg can call C-ML's own functions via ctypes
 * without re-declaring its structs in Python. This file is compiled against
 * the reference's headers and linked with oracle/_ref/libcml_ref.so (see
 * oracle/Makefile); it contains no C-ML source.
 */
#include <fcntl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include "cml.h"
#include "core/gguf_quant.h"
#include "core/quantization.h"
#include "distributed/tensor_parallel.h"
#include "nn/llama.h"
#include "nn/llm_ops.h"
#include "nn/paged_attention.h"
#include "nn/qlora.h"
#include "nn/speculative.h"
#include "ops/uops.h"
#include "tensor/tensor.h"

static TensorConfig f32cfg(void) {
    TensorConfig c = {.dtype = DTYPE_FLOAT32, .device = DEVICE_CPU, .has_dtype = true, .has_device = true};
    return c;
}

static Tensor* t_from(const float* data, int ndim, const int* shape) {
    int sh[4];
    for (int i = 0; i < ndim; i++) sh[i] = shape[i];
    TensorConfig c = f32cfg();
    return tensor_from_data(data, sh, ndim, &c);
}

/* The reference prints "No BLAS library found" to stderr on every matmul when no BLAS
 * shared object is installed (src/backend/blas.c:250, retried from src/ops/ir/execution.c:220).
 * The wrappers that reach a matmul silence fd 2 for the duration of the call. */
static int g_saved_err = -1;
static void quiet_begin(void) {
    fflush(stderr);
    g_saved_err = dup(2);
    int nul = open("/dev/null", O_WRONLY);
    if (nul >= 0) { dup2(nul, 2); close(nul); }
}
static void quiet_end(void) {
    fflush(stderr);
    if (g_saved_err >= 0) { dup2(g_saved_err, 2); close(g_saved_err); g_saved_err = -1; }
}

int ref_init(void) { return cml_init(); }

/* gguf_dequantize (src/core/gguf_quant.c:351) */
int ref_gguf_dequantize(int type, const void* src, float* dst, size_t numel) {
    return gguf_dequantize((GGUFTensorType)type, src, dst, numel);
}
int ref_gguf_type_is_quantized(int type) { return gguf_type_is_quantized((GGUFTensorType)type) ? 1 : 0; }
int ref_gguf_quant_block_size(int type) { return gguf_quant_block_size((GGUFTensorType)type); }
size_t ref_gguf_quant_type_size(int type) { return gguf_quant_type_size((GGUFTensorType)type); }

const float* ref_nf4_table(void) { return CML_NF4_TABLE; }

/* cml_quantize_nf4 (src/core/quantization.c:213). Returns num_scales or -1. */
int ref_nf4_quantize(const float* x, size_t numel, int block, uint8_t* packed, float* scales) {
    int sh[1] = {(int)numel};
    Tensor* t = t_from(x, 1, sh);
    if (!t) return -1;
    float* sc = NULL;
    int ns = 0;
    Tensor* p = cml_quantize_nf4(t, block, &sc, &ns);
    tensor_free(t);
    if (!p) return -1;
    memcpy(packed, tensor_data_ptr(p), (numel + 1) / 2);
    memcpy(scales, sc, (size_t)ns * sizeof(float));
    free(sc);
    tensor_free(p);
    return ns;
}

/* cml_dequantize_nf4 (src/core/quantization.c:314) */
int ref_nf4_dequantize(const uint8_t* packed, const float* scales, int num_scales, int block,
                       size_t numel, float* out) {
    int sh[1] = {(int)((numel + 1) / 2)};
    TensorConfig c = {.dtype = DTYPE_UINT8, .device = DEVICE_CPU, .has_dtype = true, .has_device = true};
    Tensor* p = tensor_from_data(packed, sh, 1, &c);
    if (!p) return -1;
    Tensor* o = cml_dequantize_nf4(p, scales, num_scales, block, numel);
    tensor_free(p);
    if (!o) return -1;
    memcpy(out, tensor_data_ptr(o), numel * sizeof(float));
    tensor_free(o);
    return 0;
}

/* uop_linear(x[M,K], W[N,K], NULL) (src/ops/uops.c:663 -> src/ops/ir/execution.c:3090) */
int ref_linear(const float* x, const float* W, int M, int N, int K, float* y) {
    int xs[2] = {M, K}, ws[2] = {N, K};
    Tensor* tx = t_from(x, 2, xs);
    Tensor* tw = t_from(W, 2, ws);
    if (!tx || !tw) return -1;
    quiet_begin();
    Tensor* ty = uop_linear(tx, tw, NULL);
    float* d = ty ? (float*)tensor_data_ptr(ty) : NULL;
    quiet_end();
    if (!d) return -1;
    memcpy(y, d, (size_t)M * N * sizeof(float));
    tensor_free(ty);
    tensor_free(tx);
    tensor_free(tw);
    return 0;
}

/* The same call on a weight tensor that stays resident between calls, as the reference's
 * own forward pass has it (weights are Tensor objects created once at load). */
void* ref_weight_create(const float* W, int N, int K) {
    int ws[2] = {N, K};
    return t_from(W, 2, ws);
}
void ref_weight_free(void* w) { if (w) tensor_free((Tensor*)w); }
int ref_linear_resident(const float* x, void* w, int M, float* y) {
    Tensor* tw = (Tensor*)w;
    int xs[2] = {M, tw->shape[1]};
    Tensor* tx = t_from(x, 2, xs);
    if (!tx) return -1;
    quiet_begin();
    Tensor* ty = uop_linear(tx, tw, NULL);
    float* d = ty ? (float*)tensor_data_ptr(ty) : NULL;
    quiet_end();
    if (!d) return -1;
    memcpy(y, d, (size_t)M * tw->shape[0] * sizeof(float));
    tensor_free(ty);
    tensor_free(tx);
    return 0;
}

/* cml_qlora_linear_forward (src/nn/qlora.c:240) on a weight that this wrapper
 * quantizes through cml_qlora_linear_create (:134). If packed_in is non-NULL
 * its bytes and scales replace the freshly quantized ones, so callers can
 * feed arbitrary NF4 indices. lora_B may be NULL (stays zero). */
int ref_qlora_forward(const float* x, int M, int in_f, int out_f, const float* W_fp32,
                      const uint8_t* packed_in, const float* scales_in, int block, int rank,
                      float alpha, const float* lora_A, const float* lora_B, float* y) {
    int ws[2] = {out_f, in_f}, xs[2] = {M, in_f};
    float* zeros = NULL;
    if (!W_fp32) {
        zeros = (float*)calloc((size_t)out_f * in_f, sizeof(float));
        W_fp32 = zeros;
    }
    Tensor* tw = t_from(W_fp32, 2, ws);
    free(zeros);
    if (!tw) return -1;
    CMLQLoRALinear* q = cml_qlora_linear_create(tw, rank, alpha, block);
    tensor_free(tw);
    if (!q) return -1;
    if (packed_in && scales_in) {
        memcpy(tensor_data_ptr(q->base_weight_nf4->packed_data), packed_in, ((size_t)out_f * in_f + 1) / 2);
        memcpy(q->base_weight_nf4->scales, scales_in, (size_t)q->base_weight_nf4->num_scales * sizeof(float));
    }
    if (lora_A) memcpy(tensor_data_ptr(q->lora_A), lora_A, (size_t)rank * in_f * sizeof(float));
    if (lora_B) memcpy(tensor_data_ptr(q->lora_B), lora_B, (size_t)out_f * rank * sizeof(float));
    Tensor* tx = t_from(x, 2, xs);
    Tensor* ty = tx ? cml_qlora_linear_forward(q, tx) : NULL;
    int rc = -1;
    if (ty) {
        memcpy(y, tensor_data_ptr(ty), (size_t)M * out_f * sizeof(float));
        tensor_free(ty);
        rc = 0;
    }
    if (tx) tensor_free(tx);
    cml_qlora_linear_free(q);
    return rc;
}

/* A reference LLaMA built from flat fp32 arrays in the reference's own
 * orientation (projections [in,out]); the fill pattern follows what the
 * reference's tests do with the public struct fields. */
typedef struct {
    int vocab, hidden, inter, layers, heads, kv_heads, max_seq;
    float rope_theta, eps;
} RefLlamaCfg;

void* ref_llama_create(const RefLlamaCfg* c, const float* embed, const float* final_norm,
                       const float* lm_head, const float* const* wq, const float* const* wk,
                       const float* const* wv, const float* const* wo, const float* const* wg,
                       const float* const* wu, const float* const* wd, const float* const* n1,
                       const float* const* n2) {
    CMLLLaMAConfig cfg = {.vocab_size = c->vocab, .hidden_size = c->hidden, .intermediate_size = c->inter,
                          .num_layers = c->layers, .num_heads = c->heads, .num_kv_heads = c->kv_heads,
                          .max_seq_len = c->max_seq, .rope_theta = c->rope_theta, .rms_norm_eps = c->eps,
                          .tensor_parallel_size = 1, .tensor_parallel_rank = 0};
    CMLLLaMAModel* m = cml_llama_create(&cfg);
    if (!m) return NULL;
    int hd = c->hidden / c->heads, qw = c->heads * hd, kvw = c->kv_heads * hd;
    int es[2] = {c->vocab, c->hidden}, ns[1] = {c->hidden}, ls[2] = {c->hidden, c->vocab};
    int qs[2] = {c->hidden, qw}, ks[2] = {c->hidden, kvw}, os[2] = {qw, c->hidden};
    int gs[2] = {c->hidden, c->inter}, ds[2] = {c->inter, c->hidden};
    m->embed_tokens = t_from(embed, 2, es);
    m->norm = final_norm ? t_from(final_norm, 1, ns) : NULL;
    m->lm_head = t_from(lm_head, 2, ls);
    for (int l = 0; l < c->layers; l++) {
        CMLLLaMALayer* L = m->layers[l];
        L->q_proj = t_from(wq[l], 2, qs);
        L->k_proj = t_from(wk[l], 2, ks);
        L->v_proj = t_from(wv[l], 2, ks);
        L->o_proj = t_from(wo[l], 2, os);
        L->gate_proj = t_from(wg[l], 2, gs);
        L->up_proj = t_from(wu[l], 2, gs);
        L->down_proj = t_from(wd[l], 2, ds);
        L->input_layernorm = t_from(n1[l], 1, ns);
        L->post_attn_layernorm = t_from(n2[l], 1, ns);
    }
    m->weights_loaded = true;
    return m;
}

/* cml_llama_forward (src/nn/llama.c:550); logits [seq, vocab] copied out. */
int ref_llama_forward(void* model, const int* tokens, int seq, float* logits) {
    CMLLLaMAModel* m = (CMLLLaMAModel*)model;
    quiet_begin();
    Tensor* t = cml_llama_forward(m, tokens, seq);
    float* d = t ? (float*)tensor_data_ptr(t) : NULL;
    quiet_end();
    if (!d) return -1;
    memcpy(logits, d, (size_t)seq * m->config.vocab_size * sizeof(float));
    return 0; /* the logits tensor is left to the IR context, as the reference's own callers do mid-sequence */
}

void ref_llama_reset(void* model) { cml_llama_reset((CMLLLaMAModel*)model); }
int ref_llama_cur_len(void* model) { return ((CMLLLaMAModel*)model)->current_seq_len; }
void ref_llama_free(void* model) { cml_llama_free((CMLLLaMAModel*)model); }

int ref_sample_greedy(const float* logits, int rows, int vocab) {
    int sh[2] = {rows, vocab};
    Tensor* t = t_from(logits, 2, sh);
    CMLGenerationConfig g = cml_generation_default_config();
    g.do_sample = false;
    int id = cml_llama_sample_token(t, &g);
    tensor_free(t);
    return id;
}

/* cml_llama_sample_token (src/nn/llama.c:627-737) with every field of the generation config
 * given and the C library generator seeded first, so that the draw is reproducible. */
int ref_sample_token(const float* logits, int rows, int vocab, float temperature, float top_p, int top_k,
                     int do_sample, unsigned seed) {
    int sh[2] = {rows, vocab};
    Tensor* t = t_from(logits, 2, sh);
    if (!t) return -1;
    CMLGenerationConfig g = cml_generation_default_config();
    g.temperature = temperature;
    g.top_p = top_p;
    g.top_k = top_k;
    g.do_sample = do_sample != 0;
    srand(seed);
    int id = cml_llama_sample_token(t, &g);
    tensor_free(t);
    return id;
}

/* cml_rope_forward on a 2-D tensor (src/nn/llm_ops.c:702), in place. */
int ref_rope_2d(float* x, int seq, int width, int head_dim, int start_pos, float base) {
    int sh[2] = {seq, width};
    Tensor* t = t_from(x, 2, sh);
    CMLRoPEConfig rc = {.dim = head_dim, .max_seq_len = 1 << 20, .base = base};
    if (!t || !cml_rope_forward(t, start_pos, &rc)) return -1;
    memcpy(x, tensor_data_ptr(t), (size_t)seq * width * sizeof(float));
    tensor_free(t);
    return 0;
}

/* cml_gqa_forward (src/nn/llm_ops.c:194), batch 1, causal, no external mask. */
int ref_gqa(const float* q, const float* k, const float* v, int seq, int kv_len, int heads,
            int kv_heads, int hd, float* out) {
    int qs[3] = {1, seq, heads * hd}, ks[3] = {1, kv_len, kv_heads * hd};
    Tensor* tq = t_from(q, 3, qs);
    Tensor* tk = t_from(k, 3, ks);
    Tensor* tv = t_from(v, 3, ks);
    CMLGQAConfig g = {.num_heads = heads, .num_kv_heads = kv_heads, .head_dim = hd, .scale = 0.f,
                      .causal = true, .window_size = 0};
    Tensor* o = (tq && tk && tv) ? cml_gqa_forward(tq, tk, tv, &g, NULL) : NULL;
    int rc = -1;
    if (o) {
        memcpy(out, tensor_data_ptr(o), (size_t)seq * heads * hd * sizeof(float));
        tensor_free(o);
        rc = 0;
    }
    if (tq) tensor_free(tq);
    if (tk) tensor_free(tk);
    if (tv) tensor_free(tv);
    return rc;
}

/* The paged KV cache and cml_paged_gqa_forward (src/nn/paged_attention.c): a pool of max_blocks
 * blocks, one sequence, kv_len appended tokens (`spoil` tokens of another sequence appended and
 * freed first, so that the block table is not the identity), then one forward call. Returns the
 * number of blocks the sequence holds, or -1. */
int ref_paged_gqa(const float* q, const float* k, const float* v, int seq_q, int kv_len, int heads, int kv_heads,
                  int hd, float scale, int causal, int max_blocks, int spoil, float* out) {
    CMLPagedKVCache* c = cml_paged_kv_cache_create(max_blocks, 4, kv_heads, hd);
    if (!c) return -1;
    const size_t kvw = (size_t)kv_heads * hd;
    int rc = -1, other = -1;
    if (spoil > 0) {
        other = cml_paged_cache_init_sequence(c);
        for (int i = 0; i < spoil && other >= 0; i++) if (cml_paged_cache_append(c, other, k, v)) other = -2;
    }
    int s = cml_paged_cache_init_sequence(c);
    if (s >= 0 && other != -2) {
        int ok = 1;
        for (int t = 0; t < kv_len && ok; t++) {
            if (other >= 0 && t == kv_len / 2) { cml_paged_cache_free_sequence(c, other); other = -1; }   /* its blocks come back mid-way */
            ok = cml_paged_cache_append(c, s, k + (size_t)t * kvw, v + (size_t)t * kvw) == 0;
        }
        int qs[3] = {1, seq_q, heads * hd};
        Tensor* tq = ok ? t_from(q, 3, qs) : NULL;
        CMLGQAConfig g = {.num_heads = heads, .num_kv_heads = kv_heads, .head_dim = hd, .scale = scale,
                          .causal = causal != 0, .window_size = 0};
        Tensor* o = tq ? cml_paged_gqa_forward(c, s, tq, &g) : NULL;
        if (o) {
            memcpy(out, tensor_data_ptr(o), (size_t)seq_q * heads * hd * sizeof(float));
            tensor_free(o);
            rc = c->sequences[s].num_blocks;
        }
        if (tq) tensor_free(tq);
    }
    cml_paged_kv_cache_free(c);
    return rc;
}

/* cml_speculative_decode_step (src/nn/speculative.c:88-250) over two table-driven stand-in models:
 * after token t a model predicts next[t] (logit 1.0, and the same value again at index next[t] + 1
 * when t is odd, which pins the first-maximum rule). The draft model returns NULL for sequences of
 * draft_fail_len tokens or more (0: never). out_tokens takes K + 1 entries; meta = {num_accepted,
 * num_drafted, num_verified, total_drafted, total_accepted, total_steps}. */
typedef struct { const int* next; int vocab; int fail_len; } TableLM;
static Tensor* table_forward(void* ctx, const int* toks, int n) {
    const TableLM* m = (const TableLM*)ctx;
    if (m->fail_len > 0 && n >= m->fail_len) return NULL;
    float* lg = (float*)calloc((size_t)n * m->vocab, sizeof(float));
    if (!lg) return NULL;
    for (int r = 0; r < n; r++) {
        const int nx = m->next[toks[r]];
        lg[(size_t)r * m->vocab + nx] = 1.0f;
        if ((toks[r] & 1) && nx + 1 < m->vocab) lg[(size_t)r * m->vocab + nx + 1] = 1.0f;
    }
    int sh[2] = {n, m->vocab};
    Tensor* t = t_from(lg, 2, sh);
    free(lg);
    return t;
}
static int table_sample(void* ctx, Tensor* lg, float temperature) {
    (void)temperature;
    const TableLM* m = (const TableLM*)ctx;
    const float* p = (const float*)tensor_data_ptr(lg) + (size_t)(lg->shape[0] - 1) * m->vocab;
    int best = 0;
    for (int i = 1; i < m->vocab; i++) if (p[i] > p[best]) best = i;
    return best;
}
int ref_speculative_step(const int* draft_next, const int* target_next, int vocab, int draft_fail_len, const int* prefix,
                         int prefix_len, int K, int* out_tokens, int* meta, float* rates) {
    CMLSpeculativeConfig cfg = cml_speculative_default_config();
    cfg.num_draft_tokens = K;
    CMLSpeculativeDecoder* dec = cml_speculative_create(&cfg, vocab);
    if (!dec) return -1;
    TableLM dm = {draft_next, vocab, draft_fail_len}, tm = {target_next, vocab, 0};
    cml_speculative_set_draft_model(dec, &dm, table_forward, table_sample);
    cml_speculative_set_target_model(dec, &tm, table_forward, table_sample);
    CMLSpeculativeResult* r = cml_speculative_decode_step(dec, prefix, prefix_len);
    int rc = -1;
    if (r) {
        for (int i = 0; i < r->num_accepted; i++) out_tokens[i] = r->accepted_tokens[i];
        meta[0] = r->num_accepted; meta[1] = r->num_drafted; meta[2] = r->num_verified;
        meta[3] = (int)dec->total_drafted; meta[4] = (int)dec->total_accepted; meta[5] = (int)dec->total_steps;
        rates[0] = r->acceptance_rate;
        rates[1] = cml_speculative_acceptance_rate(dec);
        cml_speculative_result_free(r);
        rc = 0;
    }
    cml_speculative_free(dec);
    return rc;
}

/* cml_tp_shard_weight / column / row forward / all-reduce
 * (src/distributed/tensor_parallel.c). Runs all tp ranks in-process, as the
 * reference's own test does, and returns the reduced [M, N] result of a
 * column-parallel W1[N1,K] followed by row-parallel W2[N,N1]. */
int ref_tp_column_then_row(const float* x, int M, int K, const float* W1, int N1, const float* W2,
                           int N, int tp, float* y) {
    int xs[2] = {M, K}, w1s[2] = {N1, K}, w2s[2] = {N, N1};
    Tensor* tx = t_from(x, 2, xs);
    Tensor* t1 = t_from(W1, 2, w1s);
    Tensor* t2 = t_from(W2, 2, w2s);
    Tensor** parts = (Tensor**)calloc((size_t)tp, sizeof(Tensor*));
    int rc = -1;
    if (!tx || !t1 || !t2 || !parts) return -1;
    for (int r = 0; r < tp; r++) {
        CMLColumnParallelLinear* cp = cml_column_parallel_create(t1, NULL, tp, r);
        CMLRowParallelLinear* rp = cml_row_parallel_create(t2, NULL, tp, r);
        if (!cp || !rp) goto done;
        Tensor* mid = cml_column_parallel_forward(cp, tx);
        if (!mid) goto done;
        parts[r] = cml_row_parallel_forward(rp, mid);
        tensor_free(mid);
        cml_column_parallel_free(cp);
        cml_row_parallel_free(rp);
        if (!parts[r]) goto done;
    }
    Tensor* sum = cml_tp_all_reduce_sum(parts, tp);
    if (sum) {
        memcpy(y, tensor_data_ptr(sum), (size_t)M * N * sizeof(float));
        tensor_free(sum);
        rc = 0;
    }
done:
    for (int r = 0; r < tp; r++) if (parts[r]) tensor_free(parts[r]);
    free(parts);
    tensor_free(tx);
    tensor_free(t1);
    tensor_free(t2);
    return rc;
}

/* cml_tokenizer_create / encode / decode (src/nn/llm_ops.c:1140-1389). Strings travel as blobs of
 * NUL-terminated spellings back to back. Returns the token count (ids in out, at most cap), or the
 * decoded length (text in out_text). */
static char** blob_strings(const char* blob, int n) {
    char** v = (char**)calloc(n > 0 ? (size_t)n : 1, sizeof(char*));
    for (int i = 0; v && i < n; i++) { v[i] = (char*)blob; blob += strlen(blob) + 1; }
    return v;
}
int ref_tokenizer_encode(const char* vocab_blob, int n_vocab, const char* merges_blob, int n_merges, int unk,
                         const char* text, int* out, int cap) {
    char** vocab = blob_strings(vocab_blob, n_vocab);
    char** merges = n_merges > 0 ? blob_strings(merges_blob, n_merges) : NULL;
    CMLTokenizer* tok = cml_tokenizer_create(vocab, n_vocab, merges, n_merges);
    int n = -1;
    if (tok) {
        if (unk >= -1) cml_tokenizer_set_special(tok, -1, -1, -1, unk);
        int* ids = cml_tokenizer_encode(tok, text, &n);
        for (int i = 0; ids && i < n && i < cap; i++) out[i] = ids[i];
        free(ids);
        cml_tokenizer_free(tok);
    }
    free(vocab);
    free(merges);
    return n;
}
int ref_tokenizer_decode(const char* vocab_blob, int n_vocab, const int* ids, int n, char* out_text, int cap) {
    char** vocab = blob_strings(vocab_blob, n_vocab);
    CMLTokenizer* tok = cml_tokenizer_create(vocab, n_vocab, NULL, 0);
    int len = -1;
    if (tok) {
        char* s = cml_tokenizer_decode(tok, ids, n);
        if (s) {
            len = (int)strlen(s);
            if (len < cap) memcpy(out_text, s, (size_t)len + 1);
            free(s);
        }
        cml_tokenizer_free(tok);
    }
    free(vocab);
    return len;
}

/* cml_lora_linear_create / forward / merge / unmerge (src/nn/lora.c:10-320). srand(seed) before the
 * create; a_init receives the A the create drew. With a_in / b_in given the pair is replaced before
 * the forward passes. y: forward with the pair applied on the fly; w_merged: the base weight after
 * merge; y_merged: forward on the merged weight. Returns 0 when the unmerge restored W exactly. */
#include "nn/lora.h"
int ref_lora(const float* x, int M, int K, int N, const float* W, int rank, float alpha, unsigned seed, const float* a_in,
             const float* b_in, float* a_init, float* y, float* w_merged, float* y_merged) {
    int ws[2] = {N, K}, xs[2] = {M, K};
    Tensor* tw = t_from(W, 2, ws);
    Tensor* tx = t_from(x, 2, xs);
    if (!tw || !tx) return -1;
    srand(seed);
    CMLLoRALinear* l = cml_lora_linear_create(tw, rank, alpha);
    if (!l) return -1;
    memcpy(a_init, tensor_data_ptr(l->lora_A), (size_t)rank * K * sizeof(float));
    if (a_in) memcpy(tensor_data_ptr(l->lora_A), a_in, (size_t)rank * K * sizeof(float));
    if (b_in) memcpy(tensor_data_ptr(l->lora_B), b_in, (size_t)N * rank * sizeof(float));
    int rc = -1;
    Tensor* o1 = cml_lora_linear_forward(l, tx);
    if (o1 && cml_lora_linear_merge(l) == 0) {
        memcpy(y, tensor_data_ptr(o1), (size_t)M * N * sizeof(float));
        memcpy(w_merged, tensor_data_ptr(tw), (size_t)N * K * sizeof(float));
        Tensor* o2 = cml_lora_linear_forward(l, tx);
        if (o2 && cml_lora_linear_unmerge(l) == 0) {
            memcpy(y_merged, tensor_data_ptr(o2), (size_t)M * N * sizeof(float));
            rc = memcmp(tensor_data_ptr(tw), W, (size_t)N * K * sizeof(float)) == 0 ? 0 : 1;
        }
        if (o2) tensor_free(o2);
    }
    if (o1) tensor_free(o1);
    cml_lora_linear_free(l);
    tensor_free(tx);
    tensor_free(tw);
    return rc;
}

/* cml_quantize_compute_params / cml_quantize_int8 / uint8 / cml_dequantize_* (src/core/quantization.c:8-192).
 * params_out = {scale bits, zero_point}. use_params == 0 lets the quantiser derive them. */
#include "core/quantization.h"
int ref_quant_params(const float* x, int n, int symmetric, int32_t* params_out) {
    int s[1] = {n};
    Tensor* t = t_from(x, 1, s);
    if (!t) return -1;
    QuantParams p = cml_quantize_compute_params(t, symmetric != 0);
    memcpy(&params_out[0], &p.scale, 4);
    params_out[1] = p.zero_point;
    tensor_free(t);
    return 0;
}
int ref_quant8(const float* x, int n, int is_unsigned, int use_params, float scale, int zero_point, uint8_t* q_out, int32_t* params_out,
               float* deq_out) {
    int s[1] = {n};
    Tensor* t = t_from(x, 1, s);
    if (!t) return -1;
    QuantParams in = {scale, zero_point}, used = {0.f, 0};
    Tensor* q = is_unsigned ? cml_quantize_uint8(t, use_params ? &in : NULL, &used) : cml_quantize_int8(t, use_params ? &in : NULL, &used);
    int rc = -1;
    if (q) {
        memcpy(q_out, tensor_data_ptr(q), (size_t)n);
        memcpy(&params_out[0], &used.scale, 4);
        params_out[1] = used.zero_point;
        Tensor* d = is_unsigned ? cml_dequantize_uint8(q, &used) : cml_dequantize_int8(q, &used);
        if (d) { memcpy(deq_out, tensor_data_ptr(d), (size_t)n * sizeof(float)); tensor_free(d); rc = 0; }
        tensor_free(q);
    }
    tensor_free(t);
    return rc;
}

/* gguf_open_write / gguf_write_tensor / gguf_close (src/core/gguf.c:47-56, 181-232, 312-340): an fp32
 * [rows, cols] tensor "w.f32", an int32 vector "v.i32" and an fp16 vector "h.f16" into `path`. */
#include "core/gguf.h"
int ref_gguf_write(const char* path, const float* a, int rows, int cols, const int32_t* b, int nb, const uint16_t* c, int nc) {
    GGUFContext* ctx = gguf_open_write(path);
    if (!ctx) return -1;
    int sa[2] = {rows, cols}, sb[1] = {nb}, sc[1] = {nc};
    TensorConfig cb = {.dtype = DTYPE_INT32, .device = DEVICE_CPU, .has_dtype = true, .has_device = true};
    TensorConfig cc = {.dtype = DTYPE_FLOAT16, .device = DEVICE_CPU, .has_dtype = true, .has_device = true};
    Tensor* ta = t_from(a, 2, sa);
    Tensor* tb = tensor_from_data(b, sb, 1, &cb);
    Tensor* tc = tensor_from_data(c, sc, 1, &cc);
    int rc = -1;
    if (ta && tb && tc) rc = gguf_write_tensor(ctx, "w.f32", ta) | gguf_write_tensor(ctx, "v.i32", tb) | gguf_write_tensor(ctx, "h.f16", tc);
    gguf_close(ctx);
    if (ta) tensor_free(ta);
    if (tb) tensor_free(tb);
    if (tc) tensor_free(tc);
    return rc;
}
