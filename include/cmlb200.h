/*
 * cmlb200.h -- the C-ABI boundary between C11 host code and the sm_100a CUDA
 * kernels of the quantized-LLM path (plain pointers and sizes only).
 *
 * Every entry point replaces a piece of C-ML's CPU path; the C-ML location it
 * stands in for is cited as file:line relative to the C-ML source tree.
 * All functions return 0 on success and a negative CMLB200_E* code otherwise;
 * cmlb200_last_error() gives a human-readable reason for the calling thread.
 * Pointers named d_* are device pointers, h_* are host pointers. `stream` is a
 * cudaStream_t passed as void* (NULL = the legacy default stream).
 * There is no CPU fallback: without a CUDA device every compute call fails.
 */
#ifndef CMLB200_H
#define CMLB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CMLB200_OK 0
#define CMLB200_EINVAL (-1)   /* NULL pointer, bad shape, unsupported type (C-ML returns -1/NULL here too) */
#define CMLB200_ECUDA (-2)    /* a CUDA runtime call failed */
#define CMLB200_ENOMEM (-3)
#define CMLB200_ETIMEOUT (-4) /* a bounded device-side wait expired */
#define CMLB200_ENCCL (-5)

/* Weight formats. The first two use the GGUF tensor-type ids
 * (include/core/gguf.h:29-41); NF4 has no GGUF id in C-ML. */
#define CMLB200_Q4_0 2
#define CMLB200_Q8_0 7
#define CMLB200_NF4 100
/* The other block types C-ML reads (src/core/gguf_quant.c:90-311), by GGUF id. A weight of one of
 * these types is the tensor's block stream unchanged: `qs` = rows * (cols / B) blocks, row-major,
 * 16-byte aligned, B = 32 (Q4_1, 20-byte blocks) or 256 (Q4_K 144, Q5_K 176, Q6_K 210 bytes);
 * `scales` = NULL, `block` = B. cmlb200_gemv / cmlb200_gemv_accum take them (M <= 32);
 * cmlb200_gguf_dequantize expands them bit-exactly. */
#define CMLB200_Q4_1 3
#define CMLB200_Q4_K 12
#define CMLB200_Q5_K 13
#define CMLB200_Q6_K 14

/* A quantized [rows, cols] weight (rows = out features N, cols = in features
 * K; y = x . W^T as in src/nn/qlora.c:309-317) in the repacked device layout:
 *   qs     Q8_0: rows*cols int8, row-major.
 *          Q4_0: rows*cols/2 bytes, row-major; the 16 bytes of GGUF block b of
 *                a row sit at byte 16*b of that row, unchanged (byte j = element
 *                j in the low nibble, j+16 in the high nibble).
 *          NF4 : rows*cols/2 bytes exactly as cml_quantize_nf4 packs them
 *                (element 2i = high nibble of byte i, src/core/quantization.c:303-305).
 *   scales Q8_0/Q4_0: rows*(cols/32) fp16, row-major (the `d` of each block).
 *          NF4 : rows*cols/block fp32 absmax values.
 * Both planes must be 16-byte aligned; cols must be a multiple of 32 (and of
 * `block` for NF4) so that every row starts on a 16-byte boundary. */
typedef struct cmlb200_qmat {
    int type;
    int rows;
    int cols;
    int block;      /* 32 for Q4_0/Q8_0, the NF4 block size otherwise */
    void* qs;       /* device */
    void* scales;   /* device */
    int flags;      /* CMLB200_QMAT_* bits */
    void* tiles;    /* device, optional: the same blocks in the tile-major layout (see
                     * cmlb200_repack_tiles); lets cmlb200_gemv use the tensor-core path for M >= 3 */
} cmlb200_qmat;

/* Set when some fp16 block scale is subnormal. C-ML's fp16_to_fp32 widens a subnormal half to
 * half its IEEE value (src/core/gguf_quant.c:35-36); matmul kernels reproduce that only when
 * this flag is set, so the common case pays nothing for it. cmlb200_scales_have_subnormals()
 * computes the flag from a host scale plane (or an array of GGUF blocks' scales). */
#define CMLB200_QMAT_SUBNORMAL_SCALES 1
int cmlb200_scales_have_subnormals(const void* h_scales_f16, size_t count);

const char* cmlb200_last_error(void);

/* ---- device plumbing (no counterpart in C-ML, which runs this path on the host) */
int cmlb200_device_count(int* count);
int cmlb200_set_device(int device);
int cmlb200_malloc(void** d_ptr, size_t bytes);
int cmlb200_free(void* d_ptr);
int cmlb200_host_alloc_pinned(void** h_ptr, size_t bytes);
int cmlb200_host_free_pinned(void* h_ptr);
int cmlb200_memcpy_h2d(void* d_dst, const void* h_src, size_t bytes, void* stream);
int cmlb200_memcpy_d2h(void* h_dst, const void* d_src, size_t bytes, void* stream);
int cmlb200_memcpy_d2d(void* d_dst, const void* d_src, size_t bytes, void* stream);
int cmlb200_memset(void* d_dst, int value, size_t bytes, void* stream);
int cmlb200_stream_create(void** stream);
int cmlb200_stream_destroy(void* stream);
int cmlb200_stream_sync(void* stream);
int cmlb200_device_sync(void);

/* ---- one-time repack (host side; replaces nothing in C-ML -- its loader
 * expands blocks to fp32 instead, src/core/gguf.c:271-295). Sizes in bytes of
 * the two planes for a [rows, cols] matrix of `type`. */
size_t cmlb200_qs_bytes(int type, int rows, int cols, int block);
size_t cmlb200_scale_bytes(int type, int rows, int cols, int block);
/* GGUF blocks (BlockQ4_0 / BlockQ8_0 array in file order,
 * include/core/gguf_quant.h:14-31) -> the two planes; and back. The quantized
 * content is unchanged, so unrepack(repack(b)) == b byte for byte. */
int cmlb200_repack_gguf(int type, const void* h_blocks, int rows, int cols, void* h_qs, void* h_scales);
int cmlb200_unrepack_gguf(int type, const void* h_qs, const void* h_scales, int rows, int cols, void* h_blocks);

/* ---- dequantisation to fp32, bit-exact with C-ML ------------------------- */
/* All six block types C-ML reads are accepted by their GGUF ids: 2 (Q4_0), 3 (Q4_1), 7 (Q8_0),
 * 12 (Q4_K), 13 (Q5_K), 14 (Q6_K; src/core/gguf_quant.c:66-311); numel must be a multiple of
 * the type's block size (32, or 256 for the K types). Only Q4_0 and Q8_0 have matmul kernels.
 * gguf_dequantize(type, src, dst, numel) (src/core/gguf_quant.c:351-391) on
 * raw GGUF blocks resident on the device. Same argument checks: NULL, numel==0,
 * unknown type or numel % 32 != 0 -> CMLB200_EINVAL. */
int cmlb200_gguf_dequantize(int type, const void* d_blocks, float* d_dst, size_t numel, void* stream);
/* The same values from the repacked planes (checks the repack on device). */
int cmlb200_dequant_qmat(const cmlb200_qmat* W, float* d_dst, void* stream);
/* cml_dequantize_nf4 (src/core/quantization.c:314-370):
 * out[e] = CML_NF4_TABLE[idx(e)] * scales[min(e/block, num_scales-1)]. */
int cmlb200_dequantize_nf4(const uint8_t* d_packed, const float* d_scales, int num_scales, int block,
                           size_t numel, float* d_out, void* stream);

/* ---- dequant-fused matmul -------------------------------------------------- */
/* Decode / skinny path, M <= 32: y[M, rows] = x[M, cols] . dequant(W)^T with
 * fp32 activations, fp32 accumulation and fp32 output. Replaces "dequantize,
 * then fp32 matmul": cml_nf4_tensor_dequantize + the triple loop of
 * src/nn/qlora.c:264-317, and gguf_read_tensor's dequantize-at-load followed by
 * UOP_MATMUL / UOP_LINEAR (src/core/gguf.c:271-295, src/ops/ir/execution.c:989-1052,
 * 3090-3134). */
int cmlb200_gemv(const cmlb200_qmat* W, const float* d_x, float* d_y, int M, void* stream);
/* The same product with the SwiGLU of src/nn/llama.c:126-155 fused in:
 * y[M, rows] = silu(x . Wg^T) * (x . Wu^T); Wg and Wu have identical shapes. */
int cmlb200_gemv_swiglu(const cmlb200_qmat* Wg, const cmlb200_qmat* Wu, const float* d_x, float* d_y,
                        int M, void* stream);
/* y += x . W^T (residual add fused; src/nn/llama.c:523-530 and :538-543). */
int cmlb200_gemv_accum(const cmlb200_qmat* W, const float* d_x, float* d_y, int M, void* stream);
/* One quantized Linear on HOST activations, host result out (what C-ML's Linear forward does with
 * host tensors: src/nn/qlora.c:264-317, src/core/gguf.c:271-295 + the fp32 matmul). h_x [M, cols],
 * h_y [M, rows], M <= 32. With page-locked buffers (cmlb200_host_alloc_pinned, cudaHostAlloc,
 * cudaHostRegister) x is read and y is written over the bus by two small kernels chained to the GEMV,
 * no DMA copy; pageable buffers are copied with cudaMemcpyAsync. Synchronises `stream`: y is in h_y on
 * return. Keeps two staging rows per device, grown on demand (the first call allocates). */
int cmlb200_gemv_host(const cmlb200_qmat* W, const float* h_x, float* h_y, int M, void* stream);

/* The same kernels with the activation "digits" (the block-fixed-point form of x the integer-dot
 * GEMV consumes) made explicit, so that one set of digits serves several projections of the same
 * activations (Q/K/V, gate/up) and can be produced by the kernel that makes the activations:
 *   cmlb200_xq_bytes        bytes of digit scratch for M rows of K values
 *   cmlb200_x_digits        x[M,K] fp32 -> digits
 *   cmlb200_rmsnorm_digits  rms_norm (src/nn/llama.c:71-124) writing fp32 (optional) and digits
 *   cmlb200_gemv_xq         y (= | += | swiglu) from digits; M <= 4; epi 0 store, 1 accumulate,
 *                           2 SwiGLU with W2 as the up projection
 *   cmlb200_gemv_rmsnorm    (M <= 8) the same from fp32 x that is RMS-normalised (src/nn/llama.c:71-124)
 *                           inside the GEMV launch: rms_norm followed by a projection
 *                           (src/nn/llama.c:461-470, 535-537, 580-583) in one kernel */
size_t cmlb200_xq_bytes(int M, int K);
int cmlb200_x_digits(const float* d_x, int M, int K, void* d_xq, void* stream);
int cmlb200_rmsnorm_digits(const float* d_x, const uint16_t* d_w_f16, int rows, int dim, float eps, float* d_out_f32, void* d_xq, void* stream);
int cmlb200_gemv_xq(const cmlb200_qmat* W, const cmlb200_qmat* W2, const void* d_xq, float* d_y, int M, int epi, void* stream);
int cmlb200_gemv_rmsnorm(const cmlb200_qmat* W, const cmlb200_qmat* W2, const float* d_x, const uint16_t* d_norm_w_f16, float eps,
                         float* d_y, int M, int epi, void* stream);

/* The decode GEMV for callers that cannot allocate device memory at run time (a serving process
 * that gave the whole GPU to its own arena, a real-time loop that must not take the allocator
 * lock, a sandbox that filters CUDA allocation calls). It has no counterpart in C-ML. Same result
 * as cmlb200_gemv within the 2e-3 bound (not bit for bit: the activations are digitised per 32-block
 * here) for Q4_0 / Q8_0 weights in the planes layout and M <= 4, but the activation
 * scratch is a fixed 512 KiB array inside the library image (resident on every GPU that loads the
 * library until the process exits) and the call performs no cudaMalloc / cudaFree. Limit:
 * M * cols <= 149,796 (e.g. M = 4 with cols = 28672); larger requests fail with CMLB200_EINVAL and
 * a message. The first call on a device looks up the array's device address; make that call
 * before starting any stream capture. All calls on a device share the array: calls whose kernels
 * could overlap on the GPU (different streams) race on it and must be ordered by the caller. */
int cmlb200_gemv_noalloc(const cmlb200_qmat* W, const float* d_x, float* d_y, int M, void* stream);

/* ---- tile-major weights for the tensor-core decode path ----------------------------------
 * The same GGUF blocks regrouped as "units": for row tile t (128 rows, the last one zero
 * padded) and block column b one contiguous unit holds the 128 rows' quants of block b
 * followed by their 128 fp16 scales (Q4_0: 128x16 B + 256 B = 2304 B; Q8_0: 128x16 B for
 * elements 0..15, 128x16 B for elements 16..31, + 256 B = 4352 B); units are ordered [t][b].
 * Content is unchanged: cmlb200_unrepack_tiles restores the file bytes exactly. */
size_t cmlb200_tiles_bytes(int type, int rows, int cols);
int cmlb200_repack_tiles(int type, const void* h_blocks, int rows, int cols, void* h_tiles);
int cmlb200_unrepack_tiles(int type, const void* h_tiles, int rows, int cols, void* h_blocks);
/* y[M, rows] = x . dequant(W)^T (accumulate == 0) or y += ... (accumulate != 0) for M <= 32 on
 * the integer tensor cores; W->qs points at the tile-major buffer, W->scales is ignored,
 * cols must be a multiple of 128. Same C-ML lines replaced as cmlb200_gemv. The activation
 * digits pass through a scratch buffer owned by the library (one per device): calls on
 * different streams of one device must not overlap. */
int cmlb200_gemv_tiles(const cmlb200_qmat* W, const float* d_x, float* d_y, int M, int accumulate, void* stream);
/* Like cmlb200_gemm_status, for the kernel behind cmlb200_gemv_tiles. */
int cmlb200_gemv_tiles_status(int* status, int reset);

/* Prefill path, M >= 1 (any M; built for M >= 64): bf16 activations, weights
 * dequantised to bf16 tiles in shared memory, tcgen05 MMAs accumulating fp32
 * in tensor memory, bf16 output. Same reference lines as cmlb200_gemv.
 * cols must be a multiple of 32 (a last half slab of 32 is zero-extended). */
int cmlb200_gemm_bf16(const cmlb200_qmat* W, const uint16_t* d_x_bf16, uint16_t* d_y_bf16, int M,
                      void* stream);
/* The same product with what happens to the finished values chosen by `mode`:
 *   CMLB200_GEMM_OUT_BF16     d_out bf16 [M, rows] (as cmlb200_gemm_bf16)
 *   CMLB200_GEMM_OUT_F32      d_out fp32 [M, rows]
 *   CMLB200_GEMM_ACC_F32      d_out fp32 [M, rows] += product (the residual adds of src/nn/llama.c:523-530, 538-543)
 *   CMLB200_GEMM_SWIGLU_BF16  d_out bf16 = silu(d_gate_bf16) * product (src/nn/llama.c:126-155 with W the
 *                             up projection and d_gate_bf16 the gate projection's output; may alias d_out) */
#define CMLB200_GEMM_OUT_BF16 0
#define CMLB200_GEMM_OUT_F32 1
#define CMLB200_GEMM_ACC_F32 2
#define CMLB200_GEMM_SWIGLU_BF16 3
int cmlb200_gemm_bf16_ex(const cmlb200_qmat* W, const uint16_t* d_x_bf16, int M, int mode, void* d_out, const uint16_t* d_gate_bf16,
                         void* stream);
/* Same, with the number of K splits chosen by the caller (1 = none). With more than one
 * split the partial sums pass through an fp32 scratch buffer owned by the library. */
int cmlb200_gemm_bf16_splitk(const cmlb200_qmat* W, const uint16_t* d_x_bf16, uint16_t* d_y_bf16, int M,
                             int splits, void* stream);
/* Synchronises the device and reports whether a bounded wait inside the tensor-core kernel
 * expired since the last reset (0 = none). C-ML has no counterpart: its path cannot stall. */
int cmlb200_gemm_status(int* status, int reset);

/* The quantized Linear of src/nn/qlora.c:264-317 for NF4 weights of ANY shape and block size
 * (blocks may straddle rows; the block index is clamped as in src/core/quantization.c:359-364):
 * y[M, rows] = x[M, cols] . dequant(W)^T in fp32, one warp per output value. The vectorised
 * kernels behind cmlb200_gemv / cmlb200_gemm_bf16 need cols % 32 == 0 and a block size that is a
 * multiple of 32 dividing cols; this entry point serves everything else. */
int cmlb200_linear_nf4_general(const uint8_t* d_packed, const float* d_scales, int num_scales, int block, int rows, int cols,
                               const float* d_x, int M, float* d_y, void* stream);

/* ---- NF4 quantisation on the device: cml_quantize_nf4 (src/core/quantization.c:213-312):
 * per-block absmax floored at 1e-10, x/absmax clamped to [-1,1], nearest code with the first
 * minimum winning, even element in the high nibble. d_packed gets (numel+1)/2 bytes, d_scales
 * ceil(numel/block) floats. Bit-identical to the CPU routine. */
int cmlb200_quantize_nf4(const float* d_x, size_t numel, int block, uint8_t* d_packed, float* d_scales, void* stream);

/* ---- the non-matmul pieces of the LLaMA forward pass ------------------------------------------
 * "rows" are the activation rows of one forward call; row r belongs to sequence row_seq[r], sits
 * at absolute position row_pos[r] and may attend to cache slots 0..row_limit[r]. */
/* embed_tokens_lookup (src/nn/llama.c:421-452), fp16 table, out-of-range ids read row 0. */
int cmlb200_embed_f16(const uint16_t* d_table_f16, const int* d_tokens, int rows, int hidden, int vocab, float* d_out, void* stream);
/* rms_norm (src/nn/llama.c:71-124): x * 1/sqrt(mean(x^2)+eps) * w; fp16 weight; writes fp32
 * (d_out_f32) or bf16 (d_out_bf16), whichever is non-NULL. */
int cmlb200_rmsnorm(const float* d_x, const uint16_t* d_w_f16, int rows, int dim, float eps, float* d_out_f32, uint16_t* d_out_bf16, void* stream);
/* cml_rope_forward (src/nn/llm_ops.c:702-805), in place on [rows, width]; all_heads == 0 rotates
 * only the first head_dim columns of each row, which is what C-ML's forward pass does. */
int cmlb200_rope(float* d_x, const int* d_row_pos, int rows, int width, int head_dim, float base, int all_heads, void* stream);
/* cml_kv_cache_append (src/nn/llm_ops.c:118-157) into a [n_seq, max_seq, kvw] cache (fp16 or fp32). */
int cmlb200_kv_append(const float* d_k, const float* d_v, void* d_kcache, void* d_vcache, const int* d_row_seq, const int* d_row_pos, int rows, int kvw, int max_seq, int kv_is_f32, void* stream);
/* cml_gqa_forward (src/nn/llm_ops.c:194-361) over the cache, split over the key range and merged.
 * max_limit = the largest row_limit of the call (sizes the splits); d_scratch needs
 * cmlb200_attention_scratch_floats(rows, heads, head_dim, splits) floats. */
size_t cmlb200_attention_scratch_floats(int rows, int heads, int head_dim, int splits);
int cmlb200_attention(const float* d_q, const void* d_kcache, const void* d_vcache, const int* d_row_seq, const int* d_row_limit, int rows, int heads, int kv_heads, int head_dim, int max_seq, int max_limit, int kv_is_f32, float* d_out, float* d_scratch, int splits, void* stream);
/* The same attention for prompt-sized calls: `rows` query rows of ONE sequence (`seq`) against that
 * sequence's fp16 cache, tiled over 64 rows x 64 keys on the tensor cores (fp16 operands, fp32
 * accumulation) so that keys and values are read once per 64 rows. Row r attends cache slots
 * 0..d_row_limit[r]. head_dim 64 or 128. Writes fp32 and / or bf16 [rows, heads*head_dim]; either
 * output pointer may be NULL. Part of the bf16 prefill pipeline (tolerance 1e-2). */
int cmlb200_attention_prefill(const float* d_q, int q_stride, const void* d_kcache_f16, const void* d_vcache_f16, int seq,
                              const int* d_row_limit, int rows, int heads, int kv_heads, int head_dim, int max_seq,
                              float* d_out_f32, uint16_t* d_out_bf16, void* stream);
/* Fused variants used by the decode step: Q rows `q_stride` floats apart (Q inside a fused q|k|v
 * buffer), attention output optionally also written as activation digits (d_xq, may be NULL); and
 * RoPE on the Q and K parts of such a buffer followed by the K/V cache append in one launch.
 * rotate_heads: 0 none, 1 head 0 of Q and K only (C-ML's behaviour), -1 every head. */
int cmlb200_attention_ex(const float* d_q, int q_stride, const void* d_kcache, const void* d_vcache, const int* d_row_seq, const int* d_row_limit, int rows, int heads, int kv_heads, int head_dim, int max_seq, int max_limit, int kv_is_f32, float* d_out, void* d_xq, float* d_scratch, int splits, void* stream);
int cmlb200_qkv_rope_append(float* d_qkv, int row_stride, const int* d_row_seq, const int* d_row_pos, int rows, int heads, int kv_heads, int head_dim, float base, int rotate_heads, void* d_kcache, void* d_vcache, int max_seq, int kv_is_f32, void* stream);
/* The decode step's attention in one launch, for rows that are one new token per sequence
 * (cml_rope_forward src/nn/llm_ops.c:702-805 on Q and K, cml_kv_cache_append :118-157,
 * cml_gqa_forward :243-372): d_qkv holds [rows][q|k|v] as the fused projection left it, nothing
 * rotated. Every head of Q and K is rotated at row_pos (table from cmlb200_rope_table), K and V of the new token go into the cache,
 * keys 0..row_limit are attended (split over `splits` CTAs per head, merged by the last to finish)
 * and [rows][heads*head_dim] fp32 is written. d_scratch: cmlb200_attention_decode_scratch_bytes
 * bytes, its first 16 KB zero before the first call (the kernel leaves them zero). */
size_t cmlb200_attention_decode_scratch_bytes(int rows, int heads, int head_dim, int splits);
int cmlb200_attention_decode(const float* d_qkv, int row_stride, void* d_kcache, void* d_vcache, const int* d_row_seq,
                             const int* d_row_pos, const int* d_row_limit, int rows, int heads, int kv_heads, int head_dim,
                             int max_seq, int max_limit, int kv_is_f32, const float* d_rope_cs, float* d_out, void* d_scratch,
                             int splits, void* stream);
/* d_cs[rows][head_dim/2][2] = (cos, sin)(row_pos * base^(-2i/head_dim)): the rotation table
 * cmlb200_attention_decode reads; one launch per decode step serves every layer. */
int cmlb200_rope_table(const int* d_row_pos, int rows, int head_dim, float base, float* d_cs, void* stream);
/* Greedy branch of cml_llama_sample_token (src/nn/llama.c:650-660): first index of the maximum. */
int cmlb200_argmax(const float* d_logits, int rows, int vocab, int* d_out, void* stream);
/* The same choice when the vocabulary projection is split over tensor-parallel ranks (C-ML has no
 * counterpart: its lm_head is one matmul, src/nn/llama.c:598-606): every rank reduces its slice
 * [rows, width] to one (value, index + index_offset) pair per row (8 bytes each, fp32 value and
 * int32 index bits); the pairs of all ranks, laid out [rank][row], are merged to the row's first
 * strict maximum. cmlb200_gather_columns puts gathered logit slices [rank][row][width] side by side
 * as [row][ranks * width]. */
int cmlb200_argmax_slice(const float* d_logits, int rows, int width, int index_offset, float* d_pairs, void* stream);
int cmlb200_argmax_merge(const float* d_pairs, int parts, int rows, int* d_out, void* stream);
int cmlb200_gather_columns(const float* d_src, int parts, int rows, int width, float* d_dst, void* stream);
/* Row bookkeeping kept on the device so that a decode step replays as a CUDA graph.
 * mode 0: sequence `seq`, rows consecutive positions from cur_len[seq]; mode 1: rows sequences,
 * one token each at cur_len[b]. relative_mask reproduces C-ML's call-relative causal mask. */
int cmlb200_prepare_rows(const int* d_cur_len, int rows, int mode, int relative_mask, int seq, int* d_row_seq, int* d_row_pos, int* d_row_limit, void* stream);
int cmlb200_advance_rows(int* d_cur_len, int rows, int mode, int seq, void* stream);
/* Element-wise helpers (uop_add src/ops/uops.c:37, silu*mul of src/nn/llama.c:126-155). */
int cmlb200_bf16_to_f32(const uint16_t* d_in, float* d_out, size_t n, void* stream);
int cmlb200_f32_to_bf16(const float* d_in, uint16_t* d_out, size_t n, void* stream);
int cmlb200_add_bf16(float* d_acc, const uint16_t* d_in, size_t n, void* stream);
int cmlb200_add_f32(float* d_acc, const float* d_in, size_t n, void* stream);
int cmlb200_swiglu_bf16(const uint16_t* d_gate, const uint16_t* d_up, uint16_t* d_out, size_t n, void* stream);
int cmlb200_swiglu_f32(const float* d_gate, const float* d_up, float* d_out, size_t n, void* stream);

/* Per-tensor affine 8-bit quantisation (src/core/quantization.c:8-192), bit-exact with C-ML's loops:
 * the value range of x (min, max into d_out[0..1]; d_scratch holds cmlb200_range_scratch_floats()
 * floats), q = clamp(roundf(x / scale) + zero_point) to int8 (or uint8), and back
 * (q - zero_point) * scale. */
size_t cmlb200_range_scratch_floats(void);
int cmlb200_range_f32(const float* d_x, size_t n, float* d_scratch, float* d_out, void* stream);
int cmlb200_quantize_8bit(const float* d_x, size_t n, float scale, int zero_point, int is_unsigned, void* d_q, void* stream);
int cmlb200_dequantize_8bit(const void* d_q, size_t n, float scale, int zero_point, int is_unsigned, float* d_out, void* stream);

/* LoRA term of the quantized Linear (src/nn/qlora.c:336-361): y[M,N] += scaling * (x.A^T).B^T
 * with A [rank,K], B [N,rank]; d_t is M*rank floats of scratch. */
int cmlb200_lora_accum(const float* d_x, const float* d_A, const float* d_B, int M, int K, int N, int rank, float scaling, float* d_t, float* d_y, void* stream);
/* Merging the pair into an fp32 weight (src/nn/lora.c:263-273): W[out, in] += scaling * B . A. */
int cmlb200_lora_merge(float* d_W, const float* d_A, const float* d_B, int out_features, int in_features, int rank, float scaling, void* stream);

/* ---- CUDA graph capture of a launch sequence (used for the decode step) ----------------------- */
int cmlb200_graph_begin(void* stream);
int cmlb200_graph_end(void* stream, void** graph_exec);
int cmlb200_graph_launch(void* graph_exec, void* stream);
int cmlb200_graph_destroy(void* graph_exec);
/* Wall-clock helpers on the device timeline. */
int cmlb200_event_create(void** event);
int cmlb200_event_record(void* event, void* stream);
int cmlb200_event_elapsed_ms(void* start, void* stop, float* ms);
int cmlb200_event_destroy(void* event);

/* Attention of one sequence over a paged KV pool (src/nn/paged_attention.c:332-480). d_q, d_out:
 * [seq_q, heads*head_dim] fp32; d_kpool, d_vpool: [blocks][block_size][kv_heads*head_dim] fp32;
 * d_block_ids: the sequence's block table. Query row i sits at position kv_len - seq_q + i. */
int cmlb200_paged_gqa_f32(const float* d_q, const float* d_kpool, const float* d_vpool, const int* d_block_ids, int block_size,
                          int seq_q, int kv_len, int heads, int kv_heads, int head_dim, float scale, int causal, float* d_out,
                          void* stream);
/* ---- fp32 operators behind the stand-alone C-ML entry points ------------------------------
 * cmlb200_gqa_f32: softmax(Q K^T * scale + masks) V with every option of cml_gqa_forward
 * (src/nn/llm_ops.c:194-372; masked scores are -1e9): q [batch, seq_q, heads*hd], k, v
 * [batch, kv_len, kv_heads*hd], mask NULL or [seq_q, kv_len] (mask_per_batch 0) /
 * [batch, seq_q, kv_len] (1) with 0 = masked. kv_len <= 51200.
 * cmlb200_rope_f32: cml_rope_forward (src/nn/llm_ops.c:702-805) on nvec vectors of last_dim floats,
 * vector v at position start_pos + (v / inner) % seq_len.
 * cmlb200_linear_f32: y[M,N] = x[M,K] . w[N,K]^T (+ bias), the forward of C-ML's fp32
 * column/row-parallel layers (src/distributed/tensor_parallel.c). */
int cmlb200_gqa_f32(const float* d_q, const float* d_k, const float* d_v, const float* d_mask, int mask_per_batch, int batch, int seq_q,
                    int kv_len, int heads, int kv_heads, int head_dim, float scale, int causal, int window, float* d_out, void* stream);
int cmlb200_rope_f32(float* d_x, size_t nvec, int last_dim, int dim, float base, int start_pos, int seq_len, int inner, void* stream);
int cmlb200_linear_f32(const float* d_x, const float* d_w, const float* d_bias, int M, int N, int K, float* d_y, void* stream);

/* ---- tensor-parallel all-reduce over peer memory -------------------------------------------
 * h[0..n) += sum over ranks of partial[0..n) in one launch per rank, for the decode-sized
 * messages after the row-parallel projections (C-ML: cml_tp_all_reduce_sum,
 * src/distributed/tensor_parallel.c:195-260). Each rank owns a workspace of
 * cmlb200_tp_ar_workspace_bytes(max_floats) bytes from cmlb200_malloc, zero-filled once, and
 * maps the other ranks' workspaces through CUDA IPC (ranks are separate processes on GPUs with
 * peer access). ws[r] is rank r's workspace as seen by the caller, ws[rank] its own. n % 4 == 0,
 * n <= max_floats, 2 <= tp <= 8. Every rank makes the same sequence of calls; the ranks' results
 * are bit-identical. Waits are bounded: cmlb200_tp_ar_status reports 1 + the peer a launch gave
 * up on (its h is then untouched), 0 otherwise. */
size_t cmlb200_tp_ar_workspace_bytes(size_t max_floats);
int cmlb200_tp_allreduce_add(float* d_h, const float* d_partial, size_t n, int tp, int rank, void* const* ws, size_t max_floats, void* stream);
int cmlb200_tp_ar_status(const void* own_ws, int* status);
int cmlb200_tp_ar_status_reset(void* own_ws);
/* The same sum for prompt-sized messages (tens of MB): one launch per rank in which every rank sums
 * one slice of the message (in rank order) and hands the summed slice to the others, so a rank
 * sends 2 (tp - 1) / tp of the message instead of tp - 1 times the message. Replaces the
 * ncclAllReduce C-ML issues after a row-parallel projection of a whole prompt
 * (src/distributed/tensor_parallel.c:195-260). A second workspace per rank, of
 * cmlb200_tp_ar_bulk_workspace_bytes(max_floats, tp) bytes, zero-filled once and mapped like the
 * first; tp and max_floats are fixed for its life. n % 4 == 0, n <= max_floats. cmlb200_tp_ar_status
 * on the bulk workspace reports an expired wait; h may then be partly updated and the caller must
 * discard the forward. */
size_t cmlb200_tp_ar_bulk_workspace_bytes(size_t max_floats, int tp);
int cmlb200_tp_allreduce_bulk_add(float* d_h, const float* d_partial, size_t n, int tp, int rank, void* const* ws, size_t max_floats,
                                  void* stream);
/* All tp ranks of that exchange on ONE device as one cooperative launch (d_h[r], d_partial[r],
 * ws[r]: rank r's buffers on the current device): checks the protocol where a single GPU is at
 * hand. Launches that wait on one another must never be separate launches on one GPU. */
int cmlb200_tp_allreduce_bulk_emulate(float* const* d_h, const float* const* d_partial, size_t n, int tp, void* const* ws, size_t max_floats,
                                      void* stream);
/* How many times a launch polls a peer's flag or packet before it gives up (both all-reduce
 * forms). 0 restores the default of 2^22 polls (seconds); the environment variable
 * CMLB200_WAIT_LIMIT sets the initial value. Applies to launches made after the call. C-ML has no
 * counterpart: src/distributed/nccl_backend.c:397-405 marks work complete immediately. */
int cmlb200_set_wait_limit(int polls);
/* The row-parallel projection and its all-reduce in one launch per rank, for M <= 4 and weights
 * the tensor-core decode kernel takes (Q4_0 / Q8_0 planes, cols % 256 == 0):
 * h[M, rows] += sum over ranks of x_rank . dequant(W_rank)^T (src/nn/llama.c:523-530, 538-543 with
 * src/distributed/tensor_parallel.c:195-260). Same workspaces as above (it uses its own part of
 * them); all projections sharing a workspace must have the same `rows`. */
int cmlb200_gemv_tp_allreduce(const cmlb200_qmat* W, const float* d_x, float* d_h, int M, int tp, int rank, void* const* ws,
                              size_t max_floats, void* stream);
int cmlb200_gemv_tp_fused_ok(const cmlb200_qmat* W, int M);
/* 1 when cmlb200_gemv / _accum / _swiglu / _rmsnorm serve 3..32 rows of x for this weight from its
 * planes layout alone (Q4_0, cols % 256 == 0: the 8-row mma.sync kernel), so that no tile-major
 * copy (W->tiles) is needed for batched decode (replaces nothing in C-ML: its decode path is the
 * fp32 matmul of src/ops/ir/execution.c:989-1052 for every batch size). Only type, rows, cols and
 * the alignment of qs and scales are read. */
int cmlb200_gemv_batched_from_planes(const cmlb200_qmat* W);
int cmlb200_ipc_get_handle(void* d_ptr, void* handle64);
int cmlb200_ipc_open(const void* handle64, void** d_ptr);
int cmlb200_ipc_close(void* d_ptr);

#ifdef __cplusplus
}
#endif
#endif /* CMLB200_H */
