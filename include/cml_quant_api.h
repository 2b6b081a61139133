/*
 * cml_quant_api.h -- the C11 host API of the quantized-LLM path, with the names, argument
 * meaning, ownership and error behaviour of C-ML's public headers, so that callers of that
 * path (examples/llama_inference.c, src/nn/openai_api.c, the speculative-decoding forward
 * callback) can link against this library instead. Behind it everything runs on the GPU
 * through the cmlb200 C-ABI (cmlb200.h); there is no CPU fallback.
 *
 * Struct layouts are part of C-ML's ABI because its callers and tests read and write the
 * fields directly; they are reproduced field for field. Each declaration cites the C-ML
 * header (relative to the C-ML source tree) it stands in for.
 *
 * Errors: pointer-returning functions return NULL, int-returning ones -1 (0 = success), and
 * every failure logs through cml_log_message at LOG_LEVEL_ERROR, as in C-ML.
 */
#ifndef CML_QUANT_API_H
#define CML_QUANT_API_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- include/core/logging.h:6-27 ------------------------------------------------------- */
typedef enum { LOG_LEVEL_DEBUG = 0, LOG_LEVEL_INFO = 1, LOG_LEVEL_WARNING = 2, LOG_LEVEL_ERROR = 3 } LogLevel;
extern LogLevel g_log_level;
void cml_set_log_level(LogLevel level);
void cml_log_message(LogLevel level, const char* file, int line, const char* func, const char* format, ...);
#define LOG_DEBUG(...) cml_log_message(LOG_LEVEL_DEBUG, __FILE__, __LINE__, __func__, __VA_ARGS__)
#define LOG_INFO(...) cml_log_message(LOG_LEVEL_INFO, __FILE__, __LINE__, __func__, __VA_ARGS__)
#define LOG_WARNING(...) cml_log_message(LOG_LEVEL_WARNING, __FILE__, __LINE__, __func__, __VA_ARGS__)
#define LOG_ERROR(...) cml_log_message(LOG_LEVEL_ERROR, __FILE__, __LINE__, __func__, __VA_ARGS__)

/* ---- include/cml.h:423-424 (src/cml.c:376-440): reference-counted library set-up. Nothing on this
 * path needs global state beyond the log level (set to LOG_LEVEL_ERROR by the first cml_init, as
 * C-ML does); both return 0. cml_cleanup without a matching cml_init is a no-op. */
int cml_init(void);
int cml_cleanup(void);
/* include/tensor/tensor.h:143: seed of the tensor random generator. No operator of this path
 * draws from it (sampling uses rand(), src/nn/llama.c:716); the value is kept and returned by
 * tensor_get_seed so that callers' set-up code links and behaves the same. */
void tensor_manual_seed(uint64_t seed);
uint64_t tensor_get_seed(void);

/* ---- include/backend/device.h:13-21, include/tensor/tensor.h:16-34,40-75,88-93 ----------- */
typedef enum { DEVICE_CPU, DEVICE_CUDA, DEVICE_METAL, DEVICE_ROCM, DEVICE_OPENCL, DEVICE_SIM_GPU, DEVICE_AUTO } DeviceType;

typedef enum {
    DTYPE_FLOAT32, DTYPE_FLOAT64, DTYPE_INT32, DTYPE_INT64, DTYPE_BOOL, DTYPE_FLOAT16, DTYPE_BFLOAT16,
    DTYPE_INT8, DTYPE_UINT8, DTYPE_INT16, DTYPE_UINT16, DTYPE_UINT32, DTYPE_UINT64,
    DTYPE_FLOAT8_E4M3, DTYPE_FLOAT8_E5M2, DTYPE_FLOAT8_E4M3_FNUZ, DTYPE_FLOAT8_E5M2_FNUZ
} DType;

struct IRNode;
struct CMLGraph;
struct CMLBackendBuffer;

/* Host tensors handed across this API are always realised (is_executed, data != NULL,
 * contiguous); the lazy-graph fields exist for layout compatibility and stay NULL. */
typedef struct Tensor {
    int* shape;
    int ndim;
    size_t numel;
    DType dtype;
    DeviceType device;
    struct IRNode* ir_node;
    struct CMLGraph* ir_context;
    struct IRNode* saved_ir_node;
    struct CMLGraph* saved_ir_context;
    bool is_executed;
    void* data;
    bool owns_data;
    bool from_buffer_cache;
    bool requires_grad;
    struct Tensor* grad;
    int ref_count;
    struct Tensor* base;
    size_t* strides;
    size_t storage_offset;
    bool is_contiguous;
    struct CMLBackendBuffer* buffer_handle;
    void* user_data;
} Tensor;

typedef struct TensorConfig {
    DType dtype;
    DeviceType device;
    bool has_dtype;
    bool has_device;
} TensorConfig;

size_t cml_dtype_size(DType dtype);
Tensor* tensor_empty(int* shape, int ndim, const TensorConfig* config);
Tensor* tensor_zeros(int* shape, int ndim, const TensorConfig* config);
Tensor* tensor_from_data(const void* data, int* shape, int ndim, const TensorConfig* config);
void tensor_free(Tensor* t);
void* tensor_data_ptr(Tensor* t);
int tensor_ensure_executed(Tensor* t);

/* ---- include/core/gguf.h:11-50, include/core/gguf_quant.h:14-62 --------------------------- */
#define GGUF_MAGIC 0x46475547
typedef enum {
    GGUF_TENSOR_F32 = 0, GGUF_TENSOR_F16 = 1, GGUF_TENSOR_Q4_0 = 2, GGUF_TENSOR_Q4_1 = 3, GGUF_TENSOR_Q8_0 = 7,
    GGUF_TENSOR_Q4_K = 12, GGUF_TENSOR_Q5_K = 13, GGUF_TENSOR_Q6_K = 14, GGUF_TENSOR_I8 = 16, GGUF_TENSOR_I16 = 17,
    GGUF_TENSOR_I32 = 18
} GGUFTensorType;

/* block layouts of the GGUF types (d, dmin, m: fp16 bits) */
#define QK4_0 32
typedef struct { uint16_t d; uint8_t qs[QK4_0 / 2]; } BlockQ4_0;                                   /* 18 B: d * (nibble - 8) */
#define QK4_1 32
typedef struct { uint16_t d; uint16_t m; uint8_t qs[QK4_1 / 2]; } BlockQ4_1;                       /* 20 B: d * nibble + m */
#define QK8_0 32
typedef struct { uint16_t d; int8_t qs[QK8_0]; } BlockQ8_0;                                        /* 34 B: d * q */
#define QK_K 256
typedef struct { uint16_t d; uint16_t dmin; uint8_t scales[12]; uint8_t qs[QK_K / 2]; } BlockQ4_K;                      /* 144 B */
typedef struct { uint16_t d; uint16_t dmin; uint8_t scales[12]; uint8_t qh[QK_K / 8]; uint8_t qs[QK_K / 2]; } BlockQ5_K; /* 176 B */
typedef struct { uint8_t ql[QK_K / 2]; uint8_t qh[QK_K / 4]; int8_t scales[QK_K / 16]; uint16_t d; } BlockQ6_K;         /* 210 B */

bool gguf_type_is_quantized(GGUFTensorType type);
int gguf_quant_block_size(GGUFTensorType type);
size_t gguf_quant_type_size(GGUFTensorType type);
/* Host pointers in, host fp32 out, computed on the device; -1 on NULL, numel == 0, a type
 * that is not block-quantized (Q4_0, Q4_1, Q8_0, Q4_K, Q5_K, Q6_K are) or numel % block != 0. */
int gguf_dequantize(GGUFTensorType type, const void* src, float* dst, size_t numel);

typedef struct GGUFContext GGUFContext;
GGUFContext* gguf_open_read(const char* filepath);
void gguf_close(GGUFContext* ctx);
int gguf_get_num_tensors(GGUFContext* ctx);
const char* gguf_get_tensor_name(GGUFContext* ctx, int index);
/* As in C-ML: quantized tensors come back dequantized to fp32, others in their own dtype. */
Tensor* gguf_read_tensor(GGUFContext* ctx, const char* name);
/* The writer (include/core/gguf.h:46,51): tensors are collected and the file is emitted by gguf_close,
 * byte for byte as C-ML emits it (version 3, the infos, zero padding to a multiple of 32, the data back
 * to back; no file when nothing was written; at most 4096 tensors; fp16 / int8 / int16 / int32 keep
 * their type id, every other dtype is labelled F32 as in src/core/gguf.c:47-56). */
GGUFContext* gguf_open_write(const char* filepath);
int gguf_write_tensor(GGUFContext* ctx, const char* name, Tensor* tensor);
/* Additions (C-ML's writer has neither): a block-quantized tensor from its raw GGUF blocks (shape as it
 * is to be read back, numel a multiple of the block size), and key/values: a scalar or string by type
 * id (value points at the scalar, or is the C string), an array of scalars (packed) or of C strings. */
int gguf_write_blocks(GGUFContext* ctx, const char* name, GGUFTensorType type, const int64_t* shape, int ndim, const void* blocks);
int gguf_write_metadata(GGUFContext* ctx, const char* key, int type, const void* value);
int gguf_write_metadata_array(GGUFContext* ctx, const char* key, int elem_type, const void* values, uint64_t count);

/* ---- include/core/quantization.h:16-25: per-tensor affine quantisation -------------------------
 * quantized = clamp(round(value / scale) + zero_point), dequantized = (quantized - zero_point) * scale.
 * params == NULL: symmetric parameters from the tensor's range for int8, the [min, max] mapping onto
 * 0..255 for uint8. Computed on the device, bit-exact with C-ML's loops; fp32 tensors only. */
typedef struct QuantParams {
    float scale;
    int32_t zero_point;
} QuantParams;
QuantParams cml_quantize_compute_params(Tensor* tensor, bool symmetric);
Tensor* cml_quantize_int8(Tensor* tensor, const QuantParams* params, QuantParams* out_params);
Tensor* cml_dequantize_int8(Tensor* tensor, const QuantParams* params);
Tensor* cml_quantize_uint8(Tensor* tensor, const QuantParams* params, QuantParams* out_params);
Tensor* cml_dequantize_uint8(Tensor* tensor, const QuantParams* params);

/* ---- include/core/quantization.h:28-38, include/nn/qlora.h:18-60 -------------------------- */
extern const float CML_NF4_TABLE[16];
Tensor* cml_quantize_nf4(Tensor* tensor, int block_size, float** out_scales, int* out_num_scales);
Tensor* cml_dequantize_nf4(Tensor* nf4_tensor, const float* scales, int num_scales, int block_size, size_t original_numel);

typedef struct CMLNF4Tensor {
    Tensor* packed_data;
    float* scales;
    int num_scales;
    int block_size;
    size_t original_numel;
    int* original_shape;
    int original_ndim;
} CMLNF4Tensor;

typedef struct CMLQLoRALinear {
    int in_features;
    int out_features;
    int rank;
    float alpha;
    float scaling;
    CMLNF4Tensor* base_weight_nf4;
    Tensor* lora_A;
    Tensor* lora_B;
    bool enable_double_quant;
} CMLQLoRALinear;

CMLNF4Tensor* cml_nf4_tensor_create(Tensor* float_tensor, int block_size);
void cml_nf4_tensor_free(CMLNF4Tensor* nf4);
Tensor* cml_nf4_tensor_dequantize(const CMLNF4Tensor* nf4);
CMLQLoRALinear* cml_qlora_linear_create(Tensor* base_weight, int rank, float alpha, int block_size);
void cml_qlora_linear_free(CMLQLoRALinear* qlora);
/* y = x . dequant(W)^T + scaling * (x . A^T) . B^T. The packed base weight is uploaded on the
 * first call and kept on the device; after editing packed_data or scales in place call
 * cml_qlora_linear_invalidate. lora_A / lora_B are re-read on every call. M <= 32 rows use the
 * fp32 decode kernel, larger batches the bf16 tensor-core kernel. */
Tensor* cml_qlora_linear_forward(CMLQLoRALinear* qlora, Tensor* input);
void cml_qlora_linear_invalidate(CMLQLoRALinear* qlora);      /* addition: no C-ML counterpart */
size_t cml_qlora_memory_usage(const CMLQLoRALinear* qlora);
size_t cml_qlora_full_memory_usage(int in_features, int out_features);

/* ---- include/nn/lora.h:16-64: LoRA over an fp32 base weight ------------------------------------
 * y = x W^T + (alpha / rank) (x A^T) B^T. base_weight [out, in] is not owned and must outlive the
 * layer; A [rank, in] starts from C-ML's Box-Muller recipe over rand(), B [out, rank] from zeros.
 * forward, merge (W += scaling B A in place, a frozen copy kept) run on the device; unmerge restores
 * the frozen copy bit for bit. An adapter owns the layers added to it. */
typedef struct CMLLoRALinear {
    int in_features;
    int out_features;
    int rank;
    float alpha;
    float scaling;
    Tensor* base_weight;
    Tensor* lora_A;
    Tensor* lora_B;
    Tensor* frozen_base;
    bool merged;
} CMLLoRALinear;
typedef struct CMLLoRAAdapter {
    char name[64];
    int rank;
    float alpha;
    float scaling;
    int num_layers;
    struct CMLLoRALinear** layers;
    bool merged;
} CMLLoRAAdapter;
CMLLoRALinear* cml_lora_linear_create(Tensor* base_weight, int rank, float alpha);
void cml_lora_linear_free(CMLLoRALinear* lora);
Tensor* cml_lora_linear_forward(CMLLoRALinear* lora, Tensor* input);
int cml_lora_linear_merge(CMLLoRALinear* lora);
int cml_lora_linear_unmerge(CMLLoRALinear* lora);
CMLLoRAAdapter* cml_lora_adapter_create(const char* name, int rank, float alpha);
void cml_lora_adapter_free(CMLLoRAAdapter* adapter);
int cml_lora_adapter_add_layer(CMLLoRAAdapter* adapter, CMLLoRALinear* layer);
int cml_lora_adapter_merge_all(CMLLoRAAdapter* adapter);
int cml_lora_adapter_unmerge_all(CMLLoRAAdapter* adapter);

/* ---- include/nn/llm_ops.h:13-89: KV cache, grouped-query attention, RoPE ------------------------
 * Stand-alone operators on host tensors (arithmetic on the device). A cache made by
 * cml_kv_cache_create holds two dense fp32 host tensors exactly as in C-ML; the caches inside a
 * CMLLLaMAModel are placeholders (key_cache == NULL): that model's keys and values live on the
 * device. */
typedef struct CMLKVCache {
    Tensor* key_cache;      /* [max_seq_len, num_kv_heads, head_dim] */
    Tensor* value_cache;
    int max_seq_len;
    int current_len;
    int num_kv_heads;
    int head_dim;
} CMLKVCache;
CMLKVCache* cml_kv_cache_create(int max_seq_len, int num_kv_heads, int head_dim);
void cml_kv_cache_free(CMLKVCache* cache);
/* new_key / new_value: [seq, num_kv_heads, head_dim]; returns the new length, -1 on overflow. */
int cml_kv_cache_append(CMLKVCache* cache, Tensor* new_key, Tensor* new_value);
void cml_kv_cache_reset(CMLKVCache* cache);
Tensor* cml_kv_cache_get_keys(CMLKVCache* cache);       /* new [current_len, kv_heads, head_dim] copy, NULL when empty */
Tensor* cml_kv_cache_get_values(CMLKVCache* cache);

typedef struct CMLGQAConfig {
    int num_heads;
    int num_kv_heads;
    int head_dim;
    float scale;            /* <= 0: 1/sqrt(head_dim) */
    bool causal;            /* key index > query index (both relative to this call) is masked */
    int window_size;        /* > 0: query index - key index > window_size is masked */
} CMLGQAConfig;
/* Q [batch, seq, heads*head_dim], K, V [batch, kv_len, kv_heads*head_dim], mask NULL or
 * [seq, kv_len] / [batch, seq, kv_len] with 0 = masked; masked scores are -1e9 as in C-ML.
 * Returns a new [batch, seq, heads*head_dim] tensor. */
Tensor* cml_gqa_forward(Tensor* Q, Tensor* K, Tensor* V, const CMLGQAConfig* config, Tensor* mask);
/* Appends K, V (batch 1) to the cache, then attends the whole cached prefix. */
Tensor* cml_gqa_forward_cached(Tensor* Q, Tensor* K, Tensor* V, CMLKVCache* kv_cache, const CMLGQAConfig* config);

/* ---- include/nn/paged_attention.h:14-80 --------------------------------------------------------
 * Paged KV cache: a pool of 16-token blocks shared by up to max_sequences sequences, a stack free
 * list, one block table per sequence. Same structs and return values as C-ML. A block's key_data /
 * value_data are host memory ([block_size, num_kv_heads, head_dim], readable by the caller); the
 * attention runs on a device copy of the pool that cml_paged_gqa_forward brings up to date, so
 * tokens must be written with cml_paged_cache_append. */
#define CML_PAGE_BLOCK_SIZE 16
#define CML_MAX_BLOCKS 4096
#define CML_MAX_SEQUENCES 256
typedef struct CMLPageBlock {
    float* key_data;
    float* value_data;
    int num_tokens;
    int block_id;
    bool in_use;
} CMLPageBlock;
typedef struct CMLBlockTable {
    int* block_ids;
    int num_blocks;
    int capacity;
    int seq_len;
} CMLBlockTable;
typedef struct CMLPagedKVCache {
    CMLPageBlock* blocks;
    int num_blocks;
    int max_blocks;
    int* free_list;
    int free_count;
    CMLBlockTable* sequences;
    int num_sequences;
    int max_sequences;
    int num_kv_heads;
    int head_dim;
    int block_size;
    size_t total_allocated;
    size_t total_freed;
} CMLPagedKVCache;
CMLPagedKVCache* cml_paged_kv_cache_create(int max_blocks, int max_sequences, int num_kv_heads, int head_dim);
void cml_paged_kv_cache_free(CMLPagedKVCache* cache);
int cml_paged_cache_alloc_block(CMLPagedKVCache* cache);              /* block id, -1 when the pool is exhausted */
void cml_paged_cache_free_block(CMLPagedKVCache* cache, int block_id);
int cml_paged_cache_init_sequence(CMLPagedKVCache* cache);            /* sequence id, -1 when all slots are taken */
void cml_paged_cache_free_sequence(CMLPagedKVCache* cache, int seq_id);
/* key, value: [num_kv_heads * head_dim] of one token; a new block is taken when the tail block is full */
int cml_paged_cache_append(CMLPagedKVCache* cache, int seq_id, const float* key, const float* value);
/* Q [1, seq_q, num_heads*head_dim]; query row i sits at position seq_len - seq_q + i of the
 * sequence. Returns a new [1, seq_q, num_heads*head_dim] tensor, NULL on error. */
Tensor* cml_paged_gqa_forward(CMLPagedKVCache* cache, int seq_id, Tensor* Q, const CMLGQAConfig* config);

typedef struct CMLRoPEConfig {
    int dim;
    int max_seq_len;
    float base;             /* <= 0: 10000 */
} CMLRoPEConfig;
/* In place; returns x. [batch, seq, heads, head_dim], [batch, seq, dim] or [seq, dim]. */
Tensor* cml_rope_forward(Tensor* x, int start_pos, const CMLRoPEConfig* config);

/* ---- include/distributed/tensor_parallel.h:12-59 (fp32 building blocks) ----------------------- */
typedef struct CMLColumnParallelLinear {
    Tensor* weight;         /* [out_features / tp_size, in_features] */
    Tensor* bias;           /* [out_features / tp_size] or NULL */
    int in_features;
    int out_features;
    int tp_size;
    int tp_rank;
} CMLColumnParallelLinear;
typedef struct CMLRowParallelLinear {
    Tensor* weight;         /* [out_features, in_features / tp_size] */
    Tensor* bias;           /* [out_features] on rank 0 only, else NULL */
    int in_features;
    int out_features;
    int tp_size;
    int tp_rank;
} CMLRowParallelLinear;
typedef struct CMLTensorParallelConfig {
    int tp_size;
    int tp_rank;
} CMLTensorParallelConfig;
CMLColumnParallelLinear* cml_column_parallel_create(Tensor* full_weight, Tensor* full_bias, int tp_size, int tp_rank);
void cml_column_parallel_free(CMLColumnParallelLinear* cp);
Tensor* cml_column_parallel_forward(CMLColumnParallelLinear* cp, Tensor* input);
CMLRowParallelLinear* cml_row_parallel_create(Tensor* full_weight, Tensor* full_bias, int tp_size, int tp_rank);
void cml_row_parallel_free(CMLRowParallelLinear* rp);
Tensor* cml_row_parallel_forward(CMLRowParallelLinear* rp, Tensor* input);     /* caller sums the ranks' outputs */
Tensor* cml_tp_all_reduce_sum(Tensor** partials, int num_parts);
Tensor* cml_tp_shard_weight(Tensor* weight, int dim, int tp_size, int tp_rank);

/* include/nn/llm_ops.h:123-153: byte-level BPE. encode: one token per byte, then every merge rule in
 * list order joins adjacent tokens that spell its pair (leftmost first); spellings are looked up in
 * the vocabulary (the last of equal spellings wins), unknown ones map to unk_token_id, or 0 when
 * that is unset. decode concatenates the spellings; ids outside the vocabulary contribute nothing.
 * encode returns a malloc'd array (NULL and 0 tokens for an empty text), decode a malloc'd string. */
typedef struct CMLBPEMerge {
    char* pair;            /* spelling of the merged token */
    int new_token_id;      /* its id, -1 when the vocabulary does not hold it */
} CMLBPEMerge;
typedef struct CMLTokenizer {
    char** vocab;
    int vocab_size;
    CMLBPEMerge* merges;
    int num_merges;
    int* token_to_id;      /* internal: spelling -> id table */
    int hash_size;
    int bos_token_id, eos_token_id, pad_token_id, unk_token_id;     /* -1 until cml_tokenizer_set_special */
} CMLTokenizer;
CMLTokenizer* cml_tokenizer_create(char** vocab, int vocab_size, char** merge_pairs, int num_merges);
void cml_tokenizer_free(CMLTokenizer* tok);
int* cml_tokenizer_encode(CMLTokenizer* tok, const char* text, int* num_tokens);
char* cml_tokenizer_decode(CMLTokenizer* tok, const int* tokens, int num_tokens);
void cml_tokenizer_set_special(CMLTokenizer* tok, int bos, int eos, int pad, int unk);
int cml_tokenizer_vocab_size(const CMLTokenizer* tok);

/* ---- include/nn/llama.h:13-106 -------------------------------------------------------------- */
typedef struct CMLLLaMAConfig {
    int vocab_size;
    int hidden_size;
    int intermediate_size;
    int num_layers;
    int num_heads;
    int num_kv_heads;
    int max_seq_len;
    float rope_theta;
    float rms_norm_eps;
    int tensor_parallel_size;
    int tensor_parallel_rank;
} CMLLLaMAConfig;

CMLLLaMAConfig cml_llama_config_7b(void);
CMLLLaMAConfig cml_llama_config_13b(void);
CMLLLaMAConfig cml_llama_config_70b(void);

typedef struct CMLLLaMALayer {
    Tensor* q_proj;
    Tensor* k_proj;
    Tensor* v_proj;
    Tensor* o_proj;
    Tensor* gate_proj;
    Tensor* up_proj;
    Tensor* down_proj;
    Tensor* input_layernorm;
    Tensor* post_attn_layernorm;
    CMLKVCache* kv_cache;
} CMLLLaMALayer;

typedef struct CMLLLaMAModel {
    CMLLLaMAConfig config;
    Tensor* embed_tokens;
    Tensor* norm;
    Tensor* lm_head;
    CMLLLaMALayer** layers;
    int num_layers;
    CMLTokenizer* tokenizer;
    bool weights_loaded;
    int current_seq_len;
} CMLLLaMAModel;

typedef struct CMLGenerationConfig {
    float temperature;
    float top_p;
    int top_k;
    int max_new_tokens;
    int eos_token_id;
    bool do_sample;
} CMLGenerationConfig;

typedef struct CMLGenerationResult {
    int* token_ids;
    int num_tokens;
    char* text;
    float total_time_ms;
    float tokens_per_second;
} CMLGenerationResult;

CMLGenerationConfig cml_generation_default_config(void);
CMLLLaMAModel* cml_llama_create(const CMLLLaMAConfig* config);
void cml_llama_free(CMLLLaMAModel* model);
/* Reads a GGUF v3 file whose projection tensors are Q4_0 or Q8_0 and whose norms / embeddings
 * are F16 (or F32), keeps the blocks quantized, repacks them once and uploads them. Tensor
 * dimensions follow the GGUF convention: dims = (in_features, out_features), i.e. `out` rows of
 * `in` contiguous elements with quantization blocks along `in`. The Tensor* fields of the model
 * are set to small placeholder tensors (shape only) so that callers' NULL checks keep working.
 * With config.tensor_parallel_size > 1 only this rank's shard is uploaded. */
int cml_llama_load_gguf(CMLLLaMAModel* model, const char* filepath);
/* Logits [seq_len, vocab] as a host fp32 tensor the caller frees, one sequence, positions
 * continuing at model->current_seq_len. */
Tensor* cml_llama_forward(CMLLLaMAModel* model, const int* token_ids, int seq_len);
Tensor* cml_llama_layer_forward(CMLLLaMAModel* model, CMLLLaMALayer* layer, Tensor* hidden, int start_pos);
/* src/nn/llama.c:739-851: encode the prompt with model->tokenizer, reset the caches, prefill,
 * then sample / forward one token at a time until max_new_tokens, the EOS id or the sequence
 * limit; the result holds prompt + generated ids, the decoded text, the wall time and generated
 * tokens per second (prefill included, as in C-ML). NULL when the model has no tokenizer: C-ML's
 * GGUF loader never creates one; cml_llama_load_gguf_tokenizer (below) builds it from the file. */
CMLGenerationResult* cml_llama_generate(CMLLLaMAModel* model, const char* prompt, const CMLGenerationConfig* config);
void cml_generation_result_free(CMLGenerationResult* result);
int cml_llama_sample_token(Tensor* logits, const CMLGenerationConfig* config);
void cml_llama_reset(CMLLLaMAModel* model);
void cml_llama_print_config(const CMLLLaMAConfig* config);

/* ---- additions (no C-ML counterpart) ---------------------------------------------------------- */
/* cml_llama_generate encodes and decodes with this library's cml_tokenizer_encode / _decode. A caller
 * with another tokenizer behind model->tokenizer hands its functions over here (NULL, NULL restores
 * the built-in ones): encode returns a malloc'd id array and its length, decode a malloc'd string. */
typedef int* (*CMLTokenizerEncodeFn)(CMLTokenizer* tok, const char* text, int* num_tokens);
typedef char* (*CMLTokenizerDecodeFn)(CMLTokenizer* tok, const int* tokens, int num_tokens);
void cml_llama_set_tokenizer_functions(CMLTokenizerEncodeFn encode, CMLTokenizerDecodeFn decode);
/* GGUF key/value metadata. C-ML's reader steps over every value (src/core/gguf.c:75-103,134-140),
 * so a GGUF file's tokenizer and hyper-parameters are out of its reach; gguf_open_read here keeps
 * them. Types are the file's own ids (include/core/gguf.h:13-27): 0..7 integers and bool, 6 and 12
 * floats, 8 string, 9 array. Lookups return -1 / NULL for a missing key or a value of another kind. */
int gguf_get_num_metadata(GGUFContext* ctx);
const char* gguf_get_metadata_key(GGUFContext* ctx, int index);
int gguf_get_metadata_type(GGUFContext* ctx, const char* key);                      /* -1: no such key */
int gguf_get_metadata_int(GGUFContext* ctx, const char* key, int64_t* out);         /* integer and bool values */
int gguf_get_metadata_float(GGUFContext* ctx, const char* key, double* out);        /* float and integer values */
const char* gguf_get_metadata_string(GGUFContext* ctx, const char* key);
/* Arrays: the element count (-1: not an array) and element type; string elements one by one, scalar
 * elements as one packed little-endian buffer owned by the context. Arrays of arrays are skipped. */
int64_t gguf_get_metadata_array_length(GGUFContext* ctx, const char* key, int* elem_type);
const char* gguf_get_metadata_array_string(GGUFContext* ctx, const char* key, int64_t index);
const void* gguf_get_metadata_array_data(GGUFContext* ctx, const char* key);
/* A CMLTokenizer from tokenizer.ggml.tokens, tokenizer.ggml.merges ("left right" pairs become the
 * merged spelling cml_tokenizer_create expects) and tokenizer.ggml.{bos,eos,padding,unknown}_token_id.
 * NULL when the file has no token list. */
CMLTokenizer* gguf_create_tokenizer(GGUFContext* ctx);
/* Fills a CMLLLaMAConfig from <arch>.block_count / embedding_length / feed_forward_length /
 * attention.head_count(_kv) / context_length / rope.freq_base / attention.layer_norm_rms_epsilon
 * (<arch> = general.architecture, "llama" when absent); the vocabulary size comes from
 * <arch>.vocab_size, else the token list, else the embedding tensor's row count. Fields the file
 * does not give keep cml_llama_config_7b's values. -1 when the file cannot be read or lacks
 * block_count, embedding_length or head_count. */
int cml_llama_config_from_gguf(const char* filepath, CMLLLaMAConfig* config);
/* Replaces model->tokenizer (freed with cml_tokenizer_free) by gguf_create_tokenizer of the file;
 * -1 and the model unchanged when the file has no token list. cml_llama_free releases it. */
int cml_llama_load_gguf_tokenizer(CMLLLaMAModel* model, const char* filepath);
/* Behaviour switches of a model, to be set after cml_llama_create and before the first forward:
 *   CML_B200_REFERENCE_QUIRKS  reproduce two properties of C-ML's forward pass exactly: RoPE
 *       rotates only head 0 (src/nn/llama.c:483-484 passes 2-D tensors to cml_rope_forward) and
 *       the causal mask compares call-relative indices (src/nn/llm_ops.c:290-298), so a cached
 *       decode step attends to cache slot 0 only. Off (default): every head is rotated and the
 *       mask uses absolute positions.
 *   CML_B200_KV_FP32           keep the KV cache in fp32 (default fp16).
 *   CML_B200_ALL_LOGITS_FP32   prompts longer than 32 tokens normally run the bf16 tensor-core
 *       path; with this flag every forward uses the fp32 decode kernels (slow, for parity runs). */
#define CML_B200_REFERENCE_QUIRKS 1
#define CML_B200_KV_FP32 2
#define CML_B200_ALL_LOGITS_FP32 4
int cml_llama_set_options(CMLLLaMAModel* model, int flags, int max_batch);
/* One decode step for `batch` independent sequences (each with its own cache and position),
 * one new token each; logits [batch, vocab]. C-ML's forward is single-sequence only. */
Tensor* cml_llama_forward_batch(CMLLLaMAModel* model, const int* token_ids, int batch);
/* Prefill sequence `seq` of a batch with its prompt (positions continue where that sequence stands).
 * Fills the caches only: no logits are produced (the vocabulary projection is skipped). */
int cml_llama_prefill_sequence(CMLLLaMAModel* model, int seq, const int* token_ids, int seq_len);
/* Greedy decoding kept on the device: feeds each step's arg-max back as the next input for
 * `steps` steps (all `batch` sequences), writes the chosen ids [steps, batch] to out_tokens and
 * the wall time of the loop to *elapsed_ms. The step is captured once as a CUDA graph. */
int cml_llama_decode_greedy(CMLLLaMAModel* model, const int* first_tokens, int batch, int steps, int* out_tokens,
                            float* elapsed_ms);
/* cml_tp_shard_weight (include/distributed/tensor_parallel.h:59) for a weight that stays
 * quantized: the shard of a [rows, cols] array of 32-element GGUF blocks along dim 0 (rows) or
 * dim 1 (columns, on block boundaries) into `out`. -1 when the split is uneven. */
int cml_tp_shard_qblocks(int type, const void* blocks, int rows, int cols, int dim, int tp_size, int tp_rank, void* out);
/* Tensor parallelism over NCCL: every rank creates its model with tensor_parallel_size/rank
 * set, rank 0 obtains an id with cml_llama_tp_unique_id and sends the 128 bytes to the other
 * ranks by any means, then every rank calls cml_llama_tp_init before loading weights. */
int cml_llama_tp_unique_id(void* id128);
int cml_llama_tp_init(CMLLLaMAModel* model, const void* id128, int device);
/* Which all-reduce serves prompt-sized row-parallel projections after cml_llama_tp_init: 1 = the
 * peer-memory form (slices summed by rank inside one launch), 0 = ncclAllReduce, -1 = no such model.
 * The init call times one sum of *probe_floats values each way on every rank (*peer_ms, *nccl_ms:
 * the slowest rank's; zero when the peer form was unavailable or failed its exactness check) and
 * keeps the faster; CML_B200_TP_BULK=1 / =0 in the environment forces the choice. No C-ML
 * counterpart (its all-reduce is always ncclAllReduce, src/distributed/tensor_parallel.c:195-260). */
int cml_llama_tp_prompt_allreduce(CMLLLaMAModel* model, size_t* probe_floats, float* peer_ms, float* nccl_ms);

/* ---- include/nn/serving.h:18-110 ---------------------------------------------------------------
 * Continuous-batching scheduler: request queue, active batch, status and timing bookkeeping, same
 * structs and return values as C-ML. This layer never runs the model itself (as in C-ML). */
#define CML_SERVING_MAX_BATCH 64
#define CML_SERVING_MAX_QUEUE 1024
typedef enum {
    CML_SEQ_STATUS_QUEUED = 0,
    CML_SEQ_STATUS_PREFILL,
    CML_SEQ_STATUS_DECODING,
    CML_SEQ_STATUS_FINISHED,
    CML_SEQ_STATUS_ERROR,
} CMLSequenceStatus;
typedef struct CMLSequenceRequest {
    int request_id;
    int* prompt_tokens;
    int num_prompt_tokens;
    int max_new_tokens;
    float temperature;
    float top_p;
    CMLSequenceStatus status;
    int paged_seq_id;           /* id in the paged KV cache; cml_serving_run_llama keeps the model's batch slot here */
    int* generated_tokens;
    int num_generated;
    int gen_capacity;
    int current_pos;
    double submit_time_ms;
    double first_token_time_ms;
    double finish_time_ms;
} CMLSequenceRequest;
typedef struct CMLServingStats {
    size_t total_requests;
    size_t completed_requests;
    size_t active_sequences;
    size_t total_tokens_generated;
    double avg_time_to_first_token_ms;
    double avg_tokens_per_second;
    double total_time_ms;
} CMLServingStats;
typedef struct CMLServingConfig {
    int max_batch_size;
    int max_queue_size;
    int max_seq_len;
    int max_new_tokens_default;
    float temperature_default;
    float top_p_default;
} CMLServingConfig;
typedef struct CMLServingContext {
    CMLServingConfig config;
    CMLSequenceRequest** queue;         /* circular */
    int queue_head;
    int queue_tail;
    int queue_count;
    int queue_capacity;
    CMLSequenceRequest** active_batch;
    int batch_size;
    CMLPagedKVCache* kv_cache;          /* not owned */
    CMLServingStats stats;
    int next_request_id;
} CMLServingContext;
CMLServingConfig cml_serving_default_config(void);
CMLServingContext* cml_serving_create(const CMLServingConfig* config);
void cml_serving_free(CMLServingContext* ctx);
void cml_serving_set_kv_cache(CMLServingContext* ctx, CMLPagedKVCache* cache);
/* request id (> 0), -1 when the queue is full; the prompt is copied; max_new_tokens 0 = the default */
int cml_serving_submit(CMLServingContext* ctx, const int* prompt_tokens, int num_tokens, int max_new_tokens);
int cml_serving_step(CMLServingContext* ctx);                    /* admits queued requests; returns the active count */
CMLSequenceStatus cml_serving_get_status(CMLServingContext* ctx, int request_id);
const int* cml_serving_get_tokens(CMLServingContext* ctx, int request_id, int* out_count);
int cml_serving_finish_request(CMLServingContext* ctx, int request_id);
CMLServingStats cml_serving_get_stats(const CMLServingContext* ctx);
/* Runs the scheduler over a device-resident LLaMA (no C-ML counterpart): admitted requests are
 * prefilled into free batch slots of the model and all slots take one greedy decode step per
 * iteration through cml_llama_forward_batch, until queue and batch are empty or max_steps (> 0)
 * steps were taken. on_finish (optional) sees each request before it is freed. Returns the number
 * of batched decode steps, -1 on error. The model needs max_batch >= the context's max_batch_size. */
int cml_serving_run_llama(CMLServingContext* ctx, CMLLLaMAModel* model, int eos_token, int max_steps,
                          void (*on_finish)(const CMLSequenceRequest* request, void* user), void* user);

/* ---- include/nn/speculative.h:15-90 ------------------------------------------------------------
 * Draft K tokens with one model, verify them with one call of another, keep the longest run that
 * matches the target's arg-max plus one more token. Same structs, callbacks and return values as
 * C-ML; the decoder is host code. */
#define CML_SPEC_MAX_DRAFT_TOKENS 16
typedef struct CMLSpeculativeConfig {
    int num_draft_tokens;       /* K, 1..CML_SPEC_MAX_DRAFT_TOKENS (default 5) */
    float temperature;
    float top_p;
    int top_k;
    bool do_sample;
} CMLSpeculativeConfig;
typedef struct CMLSpeculativeResult {
    int* accepted_tokens;       /* accepted drafts, then the target's correction or bonus token */
    int num_accepted;           /* entries of accepted_tokens */
    int num_drafted;
    int num_verified;
    float acceptance_rate;      /* accepted drafts / drafted */
    double draft_time_ms;
    double verify_time_ms;
    double total_time_ms;
} CMLSpeculativeResult;
/* logits [seq_len, vocab_size] of the whole sequence; the decoder frees the tensor */
typedef Tensor* (*CMLModelForwardFn)(void* model_ctx, const int* token_ids, int seq_len);
typedef int (*CMLSampleTokenFn)(void* model_ctx, Tensor* logits, float temperature);
typedef struct CMLSpeculativeDecoder {
    CMLSpeculativeConfig config;
    void* draft_model_ctx;
    CMLModelForwardFn draft_forward;
    CMLSampleTokenFn draft_sample;
    void* target_model_ctx;
    CMLModelForwardFn target_forward;
    CMLSampleTokenFn target_sample;
    int vocab_size;
    size_t total_drafted;
    size_t total_accepted;
    size_t total_steps;
} CMLSpeculativeDecoder;
CMLSpeculativeConfig cml_speculative_default_config(void);
CMLSpeculativeDecoder* cml_speculative_create(const CMLSpeculativeConfig* config, int vocab_size);
void cml_speculative_free(CMLSpeculativeDecoder* decoder);
void cml_speculative_set_draft_model(CMLSpeculativeDecoder* dec, void* ctx, CMLModelForwardFn forward_fn, CMLSampleTokenFn sample_fn);
void cml_speculative_set_target_model(CMLSpeculativeDecoder* dec, void* ctx, CMLModelForwardFn forward_fn, CMLSampleTokenFn sample_fn);
CMLSpeculativeResult* cml_speculative_decode_step(CMLSpeculativeDecoder* dec, const int* prefix_tokens, int prefix_len);
void cml_speculative_result_free(CMLSpeculativeResult* result);
float cml_speculative_acceptance_rate(const CMLSpeculativeDecoder* dec);

/* Callbacks that drive a device-resident CMLLLaMAModel (no counterpart in C-ML, whose callers wrap
 * cml_llama_forward themselves and re-run the whole sequence on every call). The context tracks
 * the tokens held by the model's KV cache: a call rolls the cache back to the longest common
 * prefix and forwards only the remaining rows, at least 1 for a draft model and
 * CML_SPEC_MAX_DRAFT_TOKENS + 1 for a target model; rows of the reused prefix come back as zeros.
 * cml_llama_truncate sets the position of sequence `seq` back to new_len (0 <= new_len <= current). */
typedef struct CMLSpeculativeLlama {
    CMLLLaMAModel* model;
    int* cached_tokens;
    int cached_len;
    int capacity;
    int min_rows;
    size_t rows_computed;       /* statistics: rows forwarded / calls */
    size_t calls;
} CMLSpeculativeLlama;
CMLSpeculativeLlama* cml_speculative_llama_create(CMLLLaMAModel* model, bool is_target);
void cml_speculative_llama_free(CMLSpeculativeLlama* ctx);
Tensor* cml_speculative_llama_forward(void* model_ctx, const int* token_ids, int seq_len);
int cml_speculative_llama_sample(void* model_ctx, Tensor* logits, float temperature);
int cml_llama_truncate(CMLLLaMAModel* model, int seq, int new_len);

#ifdef __cplusplus
}
#endif
#endif /* CML_QUANT_API_H */
