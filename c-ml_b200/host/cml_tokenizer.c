/*
 * Byte-level BPE tokenizer behind cml_llama_generate (C-ML: src/nn/llm_ops.c:1140-1403,
 * include/nn/llm_ops.h:123-153). Same public struct and results as C-ML's:
 *   - the text starts as one token per byte;
 *   - merge rule m (in list order) joins every adjacent pair whose concatenation spells merges[m].pair,
 *     leftmost first, re-examining the joined token against its neighbours;
 *   - each final token is looked up by its spelling; of several vocabulary entries with the same
 *     spelling the last one wins; an unknown spelling maps to unk_token_id, or 0 when that is unset.
 * C-ML does this with heap strings and a rescan from the start after every merge, O(rules x n^2).
 * A token is always a contiguous span of the text, so here the tokens are span ends in one int
 * array and a rule is one left-to-right pass over a stack: push the next span, and while the two
 * spans on top spell the rule, fuse them. That performs the same merges in the same order (the
 * leftmost candidate is always the one on top of the stack) in O(rules x n).
 * Host code: nothing here touches the device.
 */
#include <stdlib.h>
#include <string.h>

#include "cml_internal.h"

/* token_to_id is an open-addressing table of vocabulary ids (-1 = empty), hash_size a power of two */
static uint32_t span_hash(const char* s, size_t len) {
    uint32_t h = 0x9E3779B9u;
    for (size_t i = 0; i < len; i++) h = (h ^ (unsigned char)s[i]) * 0x01000193u;
    return h ^ (h >> 15);
}

static int table_find(const CMLTokenizer* tok, const char* s, size_t len) {
    if (!tok->token_to_id) return -1;
    const uint32_t mask = (uint32_t)tok->hash_size - 1;
    for (uint32_t slot = span_hash(s, len) & mask, n = 0; n <= mask; slot = (slot + 1) & mask, n++) {
        const int id = tok->token_to_id[slot];
        if (id < 0) return -1;
        const char* v = tok->vocab[id];
        if (strncmp(v, s, len) == 0 && v[len] == 0) return id;
    }
    return -1;
}

static void table_put(CMLTokenizer* tok, int id) {
    const char* s = tok->vocab[id];
    const size_t len = strlen(s);
    const uint32_t mask = (uint32_t)tok->hash_size - 1;
    for (uint32_t slot = span_hash(s, len) & mask;; slot = (slot + 1) & mask) {
        const int have = tok->token_to_id[slot];
        if (have < 0 || strcmp(tok->vocab[have], s) == 0) { tok->token_to_id[slot] = id; return; }   /* later duplicates replace earlier ones */
    }
}

CMLTokenizer* cml_tokenizer_create(char** vocab, int vocab_size, char** merge_pairs, int num_merges) {
    if (!vocab || vocab_size <= 0) {
        LOG_ERROR("cml_tokenizer_create: invalid vocab (ptr=%p, size=%d)", (void*)vocab, vocab_size);
        return NULL;
    }
    CMLTokenizer* tok = (CMLTokenizer*)calloc(1, sizeof *tok);
    if (!tok) { LOG_ERROR("cml_tokenizer_create: allocation failed"); return NULL; }
    tok->vocab_size = vocab_size;
    tok->bos_token_id = tok->eos_token_id = tok->pad_token_id = tok->unk_token_id = -1;
    tok->num_merges = num_merges;
    tok->hash_size = 64;
    while (tok->hash_size < 2 * vocab_size) tok->hash_size *= 2;
    tok->vocab = (char**)calloc((size_t)vocab_size, sizeof(char*));
    tok->token_to_id = (int*)malloc((size_t)tok->hash_size * sizeof(int));
    if (!tok->vocab || !tok->token_to_id) goto oom;
    for (int i = 0; i < tok->hash_size; i++) tok->token_to_id[i] = -1;
    for (int i = 0; i < vocab_size; i++) {
        if (!vocab[i]) continue;
        if (!(tok->vocab[i] = strdup(vocab[i]))) goto oom;
        table_put(tok, i);
    }
    if (num_merges > 0 && merge_pairs) {
        tok->merges = (CMLBPEMerge*)calloc((size_t)num_merges, sizeof(CMLBPEMerge));
        if (!tok->merges) goto oom;
        for (int i = 0; i < num_merges; i++) {
            if (!merge_pairs[i]) continue;
            if (!(tok->merges[i].pair = strdup(merge_pairs[i]))) goto oom;
            tok->merges[i].new_token_id = table_find(tok, merge_pairs[i], strlen(merge_pairs[i]));   /* -1: not in the vocabulary */
        }
    }
    return tok;
oom:
    LOG_ERROR("cml_tokenizer_create: allocation failed");
    cml_tokenizer_free(tok);
    return NULL;
}

void cml_tokenizer_free(CMLTokenizer* tok) {
    if (!tok) return;
    if (tok->vocab) {
        for (int i = 0; i < tok->vocab_size; i++) free(tok->vocab[i]);
        free(tok->vocab);
    }
    if (tok->merges) {
        for (int i = 0; i < tok->num_merges; i++) free(tok->merges[i].pair);
        free(tok->merges);
    }
    free(tok->token_to_id);
    free(tok);
}

int* cml_tokenizer_encode(CMLTokenizer* tok, const char* text, int* num_tokens) {
    if (!tok || !text || !num_tokens) {
        LOG_ERROR("cml_tokenizer_encode: NULL argument");
        if (num_tokens) *num_tokens = 0;
        return NULL;
    }
    *num_tokens = 0;
    const size_t len = strlen(text);
    if (len == 0 || len > 0x7fffffffu) return NULL;
    /* end[i] = one past the last byte of token i; token i starts where token i - 1 ends */
    int* end = (int*)malloc(len * sizeof(int));
    if (!end) return NULL;
    int count = (int)len;
    for (int i = 0; i < count; i++) end[i] = i + 1;
    for (int m = 0; tok->merges && m < tok->num_merges && count > 1; m++) {
        const char* pair = tok->merges[m].pair;
        if (!pair) continue;
        const int plen = (int)strlen(pair);
        if (plen < 2) continue;                       /* two non-empty tokens spell at least two bytes */
        int top = 0;                                  /* tokens 0..top-1 are settled for this rule */
        for (int i = 0; i < count; i++) {
            end[top++] = end[i];
            while (top >= 2) {
                const int start = top >= 3 ? end[top - 3] : 0;
                if (end[top - 1] - start != plen || memcmp(text + start, pair, (size_t)plen) != 0) break;
                end[top - 2] = end[top - 1];
                top--;
            }
        }
        count = top;
    }
    int* ids = (int*)malloc((size_t)count * sizeof(int));
    if (!ids) { free(end); return NULL; }
    const int unknown = tok->unk_token_id >= 0 ? tok->unk_token_id : 0;
    for (int i = 0, start = 0; i < count; start = end[i++]) {
        const int id = table_find(tok, text + start, (size_t)(end[i] - start));
        ids[i] = id >= 0 ? id : unknown;
    }
    free(end);
    *num_tokens = count;
    return ids;
}

char* cml_tokenizer_decode(CMLTokenizer* tok, const int* tokens, int num_tokens) {
    if (!tok || !tokens || num_tokens <= 0) { LOG_ERROR("cml_tokenizer_decode: invalid arguments"); return NULL; }
    size_t total = 0;
    for (int i = 0; i < num_tokens; i++)
        if (tokens[i] >= 0 && tokens[i] < tok->vocab_size && tok->vocab[tokens[i]]) total += strlen(tok->vocab[tokens[i]]);
    char* out = (char*)malloc(total + 1);
    if (!out) { LOG_ERROR("cml_tokenizer_decode: allocation failed"); return NULL; }
    size_t pos = 0;
    for (int i = 0; i < num_tokens; i++) {                      /* ids outside the vocabulary contribute nothing */
        if (tokens[i] < 0 || tokens[i] >= tok->vocab_size || !tok->vocab[tokens[i]]) continue;
        const size_t n = strlen(tok->vocab[tokens[i]]);
        memcpy(out + pos, tok->vocab[tokens[i]], n);
        pos += n;
    }
    out[pos] = 0;
    return out;
}

void cml_tokenizer_set_special(CMLTokenizer* tok, int bos, int eos, int pad, int unk) {
    if (!tok) return;
    tok->bos_token_id = bos;
    tok->eos_token_id = eos;
    tok->pad_token_id = pad;
    tok->unk_token_id = unk;
}

int cml_tokenizer_vocab_size(const CMLTokenizer* tok) { return tok ? tok->vocab_size : 0; }
