"""ctypes binding of lib/libcml_b200.so (the cmlb200 C-ABI plus the C-ML-compatible C11 host
API). Used by tests/ and bench.py only; the product itself is C11 + CUDA. The directory name
contains a hyphen, so import it with `__graft_entry__.load_package()`.

There is no fallback: if the shared library has not been built, importing raises."""
import ctypes as C
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "lib" / "libcml_b200.so"

Q4_0, Q8_0, NF4 = 2, 7, 100

if not LIB_PATH.exists():
    raise ImportError(f"{LIB_PATH} is missing: run `python c-ml_b200/build.py` (needs nvcc). "
                      "There is no CPU or PyTorch fallback for this path.")
lib = C.CDLL(str(LIB_PATH))


class QMat(C.Structure):
    """cmlb200_qmat (include/cmlb200.h)."""
    _fields_ = [("type", C.c_int), ("rows", C.c_int), ("cols", C.c_int), ("block", C.c_int),
                ("qs", C.c_void_p), ("scales", C.c_void_p), ("flags", C.c_int), ("tiles", C.c_void_p)]


def _sig(name, restype, *argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = list(argtypes)
    return fn


vp, sz, ci = C.c_void_p, C.c_size_t, C.c_int
last_error = _sig("cmlb200_last_error", C.c_char_p)
_sig("cmlb200_device_count", ci, C.POINTER(ci))
_sig("cmlb200_set_device", ci, ci)
_sig("cmlb200_malloc", ci, C.POINTER(vp), sz)
_sig("cmlb200_free", ci, vp)
_sig("cmlb200_host_alloc_pinned", ci, C.POINTER(vp), sz)
_sig("cmlb200_host_free_pinned", ci, vp)
_sig("cmlb200_memcpy_h2d", ci, vp, vp, sz, vp)
_sig("cmlb200_memcpy_d2h", ci, vp, vp, sz, vp)
_sig("cmlb200_memcpy_d2d", ci, vp, vp, sz, vp)
_sig("cmlb200_memset", ci, vp, ci, sz, vp)
_sig("cmlb200_stream_create", ci, C.POINTER(vp))
_sig("cmlb200_stream_destroy", ci, vp)
_sig("cmlb200_stream_sync", ci, vp)
_sig("cmlb200_device_sync", ci)
_sig("cmlb200_qs_bytes", sz, ci, ci, ci, ci)
_sig("cmlb200_scale_bytes", sz, ci, ci, ci, ci)
_sig("cmlb200_repack_gguf", ci, ci, vp, ci, ci, vp, vp)
_sig("cmlb200_scales_have_subnormals", ci, vp, sz)
_sig("cmlb200_unrepack_gguf", ci, ci, vp, vp, ci, ci, vp)
_sig("cmlb200_gguf_dequantize", ci, ci, vp, vp, sz, vp)
_sig("cmlb200_dequant_qmat", ci, C.POINTER(QMat), vp, vp)
_sig("cmlb200_dequantize_nf4", ci, vp, vp, ci, ci, sz, vp, vp)
_sig("cmlb200_gemv", ci, C.POINTER(QMat), vp, vp, ci, vp)
_sig("cmlb200_gemv_noalloc", ci, C.POINTER(QMat), vp, vp, ci, vp)
_sig("cmlb200_gemv_accum", ci, C.POINTER(QMat), vp, vp, ci, vp)
_sig("cmlb200_gemv_host", ci, C.POINTER(QMat), vp, vp, ci, vp)
_sig("cmlb200_gemv_swiglu", ci, C.POINTER(QMat), C.POINTER(QMat), vp, vp, ci, vp)
_sig("cmlb200_xq_bytes", sz, ci, ci)
_sig("cmlb200_x_digits", ci, vp, ci, ci, vp, vp)
_sig("cmlb200_rmsnorm_digits", ci, vp, vp, ci, ci, C.c_float, vp, vp, vp)
_sig("cmlb200_gemv_xq", ci, C.POINTER(QMat), C.POINTER(QMat), vp, vp, ci, ci, vp)
_sig("cmlb200_gemv_rmsnorm", ci, C.POINTER(QMat), C.POINTER(QMat), vp, vp, C.c_float, vp, ci, ci, vp)
_sig("cmlb200_attention_scratch_floats", sz, ci, ci, ci, ci)
_sig("cmlb200_attention_ex", ci, vp, ci, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, vp, vp, vp, ci, vp)
_sig("cmlb200_qkv_rope_append", ci, vp, ci, vp, vp, ci, ci, ci, ci, C.c_float, ci, vp, vp, ci, ci, vp)
_sig("cmlb200_attention_decode_scratch_bytes", sz, ci, ci, ci, ci)
_sig("cmlb200_attention_decode", ci, vp, ci, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, vp, vp, vp, ci, vp)
_sig("cmlb200_rope_table", ci, vp, ci, ci, C.c_float, vp, vp)
_sig("cmlb200_attention_prefill", ci, vp, ci, vp, vp, ci, vp, ci, ci, ci, ci, ci, vp, vp, vp)
_sig("cmlb200_argmax", ci, vp, ci, ci, vp, vp)
_sig("cmlb200_embed_f16", ci, vp, vp, ci, ci, ci, vp, vp)
_sig("cmlb200_rmsnorm", ci, vp, vp, ci, ci, C.c_float, vp, vp, vp)
_sig("cmlb200_tiles_bytes", sz, ci, ci, ci)
_sig("cmlb200_repack_tiles", ci, ci, vp, ci, ci, vp)
_sig("cmlb200_unrepack_tiles", ci, ci, vp, ci, ci, vp)
_sig("cmlb200_gemv_tiles", ci, C.POINTER(QMat), vp, vp, ci, ci, vp)
_sig("cmlb200_gemv_tiles_status", ci, C.POINTER(ci), ci)
_sig("cmlb200_gemm_bf16", ci, C.POINTER(QMat), vp, vp, ci, vp)
_sig("cmlb200_gemm_bf16_splitk", ci, C.POINTER(QMat), vp, vp, ci, ci, vp)
_sig("cmlb200_gemm_bf16_ex", ci, C.POINTER(QMat), vp, ci, ci, vp, vp, vp)
_sig("cmlb200_gemm_status", ci, C.POINTER(ci), ci)
_sig("cmlb200_linear_nf4_general", ci, vp, vp, ci, ci, ci, ci, vp, ci, vp, vp)
_sig("cmlb200_tp_ar_workspace_bytes", sz, sz)
_sig("cmlb200_tp_allreduce_add", ci, vp, vp, sz, ci, ci, C.POINTER(vp), sz, vp)
_sig("cmlb200_gemv_tp_allreduce", ci, C.POINTER(QMat), vp, vp, ci, ci, ci, C.POINTER(vp), sz, vp)
_sig("cmlb200_gemv_tp_fused_ok", ci, C.POINTER(QMat), ci)
_sig("cmlb200_tp_ar_status", ci, vp, C.POINTER(ci))
_sig("cmlb200_tp_ar_bulk_workspace_bytes", sz, sz, ci)
_sig("cmlb200_tp_allreduce_bulk_add", ci, vp, vp, sz, ci, ci, C.POINTER(vp), sz, vp)
_sig("cmlb200_tp_allreduce_bulk_emulate", ci, C.POINTER(vp), C.POINTER(vp), sz, ci, C.POINTER(vp), sz, vp)
_sig("cmlb200_tp_ar_status_reset", ci, vp)
_sig("cmlb200_set_wait_limit", ci, ci)


class CmlB200Error(RuntimeError):
    pass


def check(rc: int, what: str = ""):
    """Raise with the library's own message when a C-ABI call failed."""
    if rc != 0:
        raise CmlB200Error(f"{what} failed ({rc}): {last_error().decode(errors='replace')}")
    return rc


def np_ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def repack_gguf(qtype: int, blocks, rows: int, cols: int):
    """Host repack of a numpy uint8 array of GGUF blocks into (qs, scales) numpy planes."""
    import numpy as np
    qs = np.empty(lib.cmlb200_qs_bytes(qtype, rows, cols, 32), np.uint8)
    sc = np.empty(lib.cmlb200_scale_bytes(qtype, rows, cols, 32), np.uint8)
    check(lib.cmlb200_repack_gguf(qtype, np_ptr(blocks), rows, cols, np_ptr(qs), np_ptr(sc)), "repack")
    return qs, sc


def repack_tiles(qtype: int, blocks, rows: int, cols: int):
    """Host repack of GGUF blocks into the tile-major buffer of the tensor-core decode path."""
    import numpy as np
    out = np.empty(lib.cmlb200_tiles_bytes(qtype, rows, cols), np.uint8)
    check(lib.cmlb200_repack_tiles(qtype, np_ptr(blocks), rows, cols, np_ptr(out)), "repack_tiles")
    return out


# ---- the C-ML-compatible C11 host API (include/cml_quant_api.h) ---------------------------------
class Tensor(C.Structure):
    pass


Tensor._fields_ = [("shape", C.POINTER(C.c_int)), ("ndim", C.c_int), ("numel", C.c_size_t), ("dtype", C.c_int),
                   ("device", C.c_int), ("ir_node", C.c_void_p), ("ir_context", C.c_void_p), ("saved_ir_node", C.c_void_p),
                   ("saved_ir_context", C.c_void_p), ("is_executed", C.c_bool), ("data", C.c_void_p), ("owns_data", C.c_bool),
                   ("from_buffer_cache", C.c_bool), ("requires_grad", C.c_bool), ("grad", C.c_void_p), ("ref_count", C.c_int),
                   ("base", C.c_void_p), ("strides", C.POINTER(C.c_size_t)), ("storage_offset", C.c_size_t),
                   ("is_contiguous", C.c_bool), ("buffer_handle", C.c_void_p), ("user_data", C.c_void_p)]


class TensorConfig(C.Structure):
    _fields_ = [("dtype", C.c_int), ("device", C.c_int), ("has_dtype", C.c_bool), ("has_device", C.c_bool)]


class LlamaConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("vocab_size", "hidden_size", "intermediate_size", "num_layers", "num_heads",
                                       "num_kv_heads", "max_seq_len")] + \
               [("rope_theta", C.c_float), ("rms_norm_eps", C.c_float), ("tensor_parallel_size", C.c_int),
                ("tensor_parallel_rank", C.c_int)]


class LlamaModel(C.Structure):
    _fields_ = [("config", LlamaConfig), ("embed_tokens", C.POINTER(Tensor)), ("norm", C.POINTER(Tensor)),
                ("lm_head", C.POINTER(Tensor)), ("layers", C.c_void_p), ("num_layers", C.c_int), ("tokenizer", C.c_void_p),
                ("weights_loaded", C.c_bool), ("current_seq_len", C.c_int)]


class GenerationConfig(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("top_k", C.c_int), ("max_new_tokens", C.c_int),
                ("eos_token_id", C.c_int), ("do_sample", C.c_bool)]


class NF4Tensor(C.Structure):
    _fields_ = [("packed_data", C.POINTER(Tensor)), ("scales", C.POINTER(C.c_float)), ("num_scales", C.c_int),
                ("block_size", C.c_int), ("original_numel", C.c_size_t), ("original_shape", C.POINTER(C.c_int)),
                ("original_ndim", C.c_int)]


class QLoRALinear(C.Structure):
    _fields_ = [("in_features", C.c_int), ("out_features", C.c_int), ("rank", C.c_int), ("alpha", C.c_float),
                ("scaling", C.c_float), ("base_weight_nf4", C.POINTER(NF4Tensor)), ("lora_A", C.POINTER(Tensor)),
                ("lora_B", C.POINTER(Tensor)), ("enable_double_quant", C.c_bool)]


class KVCache(C.Structure):
    _fields_ = [("key_cache", C.POINTER(Tensor)), ("value_cache", C.POINTER(Tensor)), ("max_seq_len", C.c_int),
                ("current_len", C.c_int), ("num_kv_heads", C.c_int), ("head_dim", C.c_int)]


class GQAConfig(C.Structure):
    _fields_ = [("num_heads", C.c_int), ("num_kv_heads", C.c_int), ("head_dim", C.c_int), ("scale", C.c_float),
                ("causal", C.c_bool), ("window_size", C.c_int)]


class PageBlock(C.Structure):
    _fields_ = [("key_data", C.POINTER(C.c_float)), ("value_data", C.POINTER(C.c_float)), ("num_tokens", C.c_int),
                ("block_id", C.c_int), ("in_use", C.c_bool)]


class BlockTable(C.Structure):
    _fields_ = [("block_ids", C.POINTER(C.c_int)), ("num_blocks", C.c_int), ("capacity", C.c_int), ("seq_len", C.c_int)]


class PagedKVCache(C.Structure):
    _fields_ = [("blocks", C.POINTER(PageBlock)), ("num_blocks", C.c_int), ("max_blocks", C.c_int),
                ("free_list", C.POINTER(C.c_int)), ("free_count", C.c_int), ("sequences", C.POINTER(BlockTable)),
                ("num_sequences", C.c_int), ("max_sequences", C.c_int), ("num_kv_heads", C.c_int), ("head_dim", C.c_int),
                ("block_size", C.c_int), ("total_allocated", C.c_size_t), ("total_freed", C.c_size_t)]


class RoPEConfig(C.Structure):
    _fields_ = [("dim", C.c_int), ("max_seq_len", C.c_int), ("base", C.c_float)]


class ParallelLinear(C.Structure):          # CMLColumnParallelLinear and CMLRowParallelLinear share the layout
    _fields_ = [("weight", C.POINTER(Tensor)), ("bias", C.POINTER(Tensor)), ("in_features", C.c_int), ("out_features", C.c_int),
                ("tp_size", C.c_int), ("tp_rank", C.c_int)]


TP = C.POINTER(Tensor)
MP = C.POINTER(LlamaModel)
KP = C.POINTER(KVCache)
PLP = C.POINTER(ParallelLinear)
_sig("cml_kv_cache_create", KP, ci, ci, ci)
_sig("cml_kv_cache_free", None, KP)
_sig("cml_kv_cache_append", ci, KP, TP, TP)
_sig("cml_kv_cache_reset", None, KP)
_sig("cml_kv_cache_get_keys", TP, KP)
_sig("cml_kv_cache_get_values", TP, KP)
_sig("cml_gqa_forward", TP, TP, TP, TP, C.POINTER(GQAConfig), TP)
_sig("cml_gqa_forward_cached", TP, TP, TP, TP, KP, C.POINTER(GQAConfig))
_sig("cml_rope_forward", TP, TP, ci, C.POINTER(RoPEConfig))
PKP = C.POINTER(PagedKVCache)
_sig("cml_paged_kv_cache_create", PKP, ci, ci, ci, ci)
_sig("cml_paged_kv_cache_free", None, PKP)
_sig("cml_paged_cache_alloc_block", ci, PKP)
_sig("cml_paged_cache_free_block", None, PKP, ci)
_sig("cml_paged_cache_init_sequence", ci, PKP)
_sig("cml_paged_cache_free_sequence", None, PKP, ci)
_sig("cml_paged_cache_append", ci, PKP, ci, vp, vp)
_sig("cml_paged_gqa_forward", TP, PKP, ci, TP, C.POINTER(GQAConfig))
class SpeculativeConfig(C.Structure):
    _fields_ = [("num_draft_tokens", C.c_int), ("temperature", C.c_float), ("top_p", C.c_float), ("top_k", C.c_int), ("do_sample", C.c_bool)]


class SpeculativeResult(C.Structure):
    _fields_ = [("accepted_tokens", C.POINTER(C.c_int)), ("num_accepted", C.c_int), ("num_drafted", C.c_int), ("num_verified", C.c_int),
                ("acceptance_rate", C.c_float), ("draft_time_ms", C.c_double), ("verify_time_ms", C.c_double), ("total_time_ms", C.c_double)]


ModelForwardFn = C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.POINTER(C.c_int), C.c_int)
SampleTokenFn = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_float)


class SpeculativeDecoder(C.Structure):
    _fields_ = [("config", SpeculativeConfig), ("draft_model_ctx", C.c_void_p), ("draft_forward", ModelForwardFn), ("draft_sample", SampleTokenFn),
                ("target_model_ctx", C.c_void_p), ("target_forward", ModelForwardFn), ("target_sample", SampleTokenFn), ("vocab_size", C.c_int),
                ("total_drafted", C.c_size_t), ("total_accepted", C.c_size_t), ("total_steps", C.c_size_t)]


class SpeculativeLlama(C.Structure):
    _fields_ = [("model", MP), ("cached_tokens", C.POINTER(C.c_int)), ("cached_len", C.c_int), ("capacity", C.c_int), ("min_rows", C.c_int),
                ("rows_computed", C.c_size_t), ("calls", C.c_size_t)]


SDP, SRP, SLP = C.POINTER(SpeculativeDecoder), C.POINTER(SpeculativeResult), C.POINTER(SpeculativeLlama)
_sig("cml_speculative_default_config", SpeculativeConfig)
_sig("cml_speculative_create", SDP, C.POINTER(SpeculativeConfig), ci)
_sig("cml_speculative_free", None, SDP)
_sig("cml_speculative_set_draft_model", None, SDP, vp, vp, vp)
_sig("cml_speculative_set_target_model", None, SDP, vp, vp, vp)
_sig("cml_speculative_decode_step", SRP, SDP, vp, ci)
_sig("cml_speculative_result_free", None, SRP)
_sig("cml_speculative_acceptance_rate", C.c_float, SDP)
_sig("cml_speculative_llama_create", SLP, MP, C.c_bool)
_sig("cml_speculative_llama_free", None, SLP)
_sig("cml_speculative_llama_forward", TP, vp, vp, ci)
_sig("cml_speculative_llama_sample", ci, vp, TP, C.c_float)
_sig("cml_llama_truncate", ci, MP, ci, ci)
class SequenceRequest(C.Structure):
    _fields_ = [("request_id", C.c_int), ("prompt_tokens", C.POINTER(C.c_int)), ("num_prompt_tokens", C.c_int), ("max_new_tokens", C.c_int),
                ("temperature", C.c_float), ("top_p", C.c_float), ("status", C.c_int), ("paged_seq_id", C.c_int),
                ("generated_tokens", C.POINTER(C.c_int)), ("num_generated", C.c_int), ("gen_capacity", C.c_int), ("current_pos", C.c_int),
                ("submit_time_ms", C.c_double), ("first_token_time_ms", C.c_double), ("finish_time_ms", C.c_double)]


class ServingStats(C.Structure):
    _fields_ = [("total_requests", C.c_size_t), ("completed_requests", C.c_size_t), ("active_sequences", C.c_size_t),
                ("total_tokens_generated", C.c_size_t), ("avg_time_to_first_token_ms", C.c_double), ("avg_tokens_per_second", C.c_double),
                ("total_time_ms", C.c_double)]


class ServingConfig(C.Structure):
    _fields_ = [("max_batch_size", C.c_int), ("max_queue_size", C.c_int), ("max_seq_len", C.c_int), ("max_new_tokens_default", C.c_int),
                ("temperature_default", C.c_float), ("top_p_default", C.c_float)]


FinishFn = C.CFUNCTYPE(None, C.POINTER(SequenceRequest), C.c_void_p)
_sig("cml_serving_default_config", ServingConfig)
_sig("cml_serving_create", vp, C.POINTER(ServingConfig))
_sig("cml_serving_free", None, vp)
_sig("cml_serving_submit", ci, vp, vp, ci, ci)
_sig("cml_serving_step", ci, vp)
_sig("cml_serving_get_status", ci, vp, ci)
_sig("cml_serving_get_tokens", C.POINTER(C.c_int), vp, ci, C.POINTER(C.c_int))
_sig("cml_serving_finish_request", ci, vp, ci)
_sig("cml_serving_get_stats", ServingStats, vp)
_sig("cml_serving_run_llama", ci, vp, MP, ci, ci, vp, vp)
_sig("cml_column_parallel_create", PLP, TP, TP, ci, ci)
_sig("cml_column_parallel_free", None, PLP)
_sig("cml_column_parallel_forward", TP, PLP, TP)
_sig("cml_row_parallel_create", PLP, TP, TP, ci, ci)
_sig("cml_row_parallel_free", None, PLP)
_sig("cml_row_parallel_forward", TP, PLP, TP)
_sig("cml_tp_all_reduce_sum", TP, C.POINTER(TP), ci)
_sig("cml_tp_shard_weight", TP, TP, ci, ci, ci)
_sig("cml_llama_layer_forward", TP, MP, vp, TP, ci)
_sig("cml_set_log_level", None, ci)
_sig("tensor_from_data", TP, vp, C.POINTER(ci), ci, C.POINTER(TensorConfig))
_sig("tensor_zeros", TP, C.POINTER(ci), ci, C.POINTER(TensorConfig))
_sig("tensor_free", None, TP)
_sig("tensor_data_ptr", vp, TP)
_sig("gguf_type_is_quantized", C.c_bool, ci)
_sig("gguf_quant_block_size", ci, ci)
_sig("gguf_quant_type_size", sz, ci)
_sig("gguf_dequantize", ci, ci, vp, vp, sz)
_sig("gguf_open_read", vp, C.c_char_p)
_sig("gguf_close", None, vp)
_sig("gguf_get_num_tensors", ci, vp)
_sig("gguf_get_tensor_name", C.c_char_p, vp, ci)
_sig("gguf_read_tensor", TP, vp, C.c_char_p)
_sig("cml_quantize_nf4", TP, TP, ci, C.POINTER(C.POINTER(C.c_float)), C.POINTER(ci))
_sig("cml_dequantize_nf4", TP, TP, C.POINTER(C.c_float), ci, ci, sz)
_sig("cml_nf4_tensor_create", C.POINTER(NF4Tensor), TP, ci)
_sig("cml_nf4_tensor_free", None, C.POINTER(NF4Tensor))
_sig("cml_nf4_tensor_dequantize", TP, C.POINTER(NF4Tensor))
_sig("cml_qlora_linear_create", C.POINTER(QLoRALinear), TP, ci, C.c_float, ci)
_sig("cml_qlora_linear_free", None, C.POINTER(QLoRALinear))
_sig("cml_qlora_linear_forward", TP, C.POINTER(QLoRALinear), TP)
_sig("cml_qlora_linear_invalidate", None, C.POINTER(QLoRALinear))
_sig("cml_qlora_memory_usage", sz, C.POINTER(QLoRALinear))
_sig("cml_qlora_full_memory_usage", sz, ci, ci)
_sig("cml_llama_config_7b", LlamaConfig)
_sig("cml_llama_config_13b", LlamaConfig)
_sig("cml_llama_config_70b", LlamaConfig)
_sig("cml_generation_default_config", GenerationConfig)
_sig("cml_llama_create", MP, C.POINTER(LlamaConfig))
_sig("cml_llama_free", None, MP)
_sig("cml_llama_load_gguf", ci, MP, C.c_char_p)
_sig("cml_llama_forward", TP, MP, vp, ci)
_sig("cml_llama_forward_batch", TP, MP, vp, ci)
_sig("cml_llama_prefill_sequence", ci, MP, ci, vp, ci)
_sig("cml_llama_decode_greedy", ci, MP, vp, ci, ci, vp, C.POINTER(C.c_float))
_sig("cml_llama_generate", vp, MP, C.c_char_p, C.POINTER(GenerationConfig))
_sig("cml_generation_result_free", None, vp)
_sig("cml_llama_sample_token", ci, TP, C.POINTER(GenerationConfig))
_sig("cml_llama_reset", None, MP)
_sig("cml_llama_print_config", None, C.POINTER(LlamaConfig))
_sig("cml_llama_set_options", ci, MP, ci, ci)
_sig("cml_tp_shard_qblocks", ci, ci, vp, ci, ci, ci, ci, ci, vp)
_sig("cml_llama_tp_unique_id", ci, vp)
_sig("cml_llama_tp_init", ci, MP, vp, ci)
_sig("cml_llama_tp_prompt_allreduce", ci, MP, C.POINTER(sz), C.POINTER(C.c_float), C.POINTER(C.c_float))
class Tokenizer(C.Structure):
    _fields_ = [("vocab", C.POINTER(C.c_char_p)), ("vocab_size", C.c_int), ("merges", C.c_void_p), ("num_merges", C.c_int),
                ("token_to_id", C.c_void_p), ("hash_size", C.c_int), ("bos_token_id", C.c_int), ("eos_token_id", C.c_int),
                ("pad_token_id", C.c_int), ("unk_token_id", C.c_int)]


TKP = C.POINTER(Tokenizer)
_sig("cml_tokenizer_create", TKP, C.POINTER(C.c_char_p), ci, C.POINTER(C.c_char_p), ci)
_sig("cml_tokenizer_free", None, TKP)
_sig("cml_tokenizer_encode", C.POINTER(C.c_int), TKP, C.c_char_p, C.POINTER(C.c_int))
_sig("cml_tokenizer_decode", vp, TKP, vp, ci)
_sig("cml_tokenizer_set_special", None, TKP, ci, ci, ci, ci)
_sig("cml_tokenizer_vocab_size", ci, TKP)
_sig("gguf_get_num_metadata", ci, vp)
_sig("gguf_get_metadata_key", C.c_char_p, vp, ci)
_sig("gguf_get_metadata_type", ci, vp, C.c_char_p)
_sig("gguf_get_metadata_int", ci, vp, C.c_char_p, C.POINTER(C.c_int64))
_sig("gguf_get_metadata_float", ci, vp, C.c_char_p, C.POINTER(C.c_double))
_sig("gguf_get_metadata_string", C.c_char_p, vp, C.c_char_p)
_sig("gguf_get_metadata_array_length", C.c_int64, vp, C.c_char_p, C.POINTER(ci))
_sig("gguf_get_metadata_array_string", C.c_char_p, vp, C.c_char_p, C.c_int64)
_sig("gguf_get_metadata_array_data", vp, vp, C.c_char_p)
_sig("gguf_create_tokenizer", TKP, vp)
_sig("cml_llama_config_from_gguf", ci, C.c_char_p, C.POINTER(LlamaConfig))
_sig("cml_llama_load_gguf_tokenizer", ci, MP, C.c_char_p)
class LoRALinear(C.Structure):
    _fields_ = [("in_features", C.c_int), ("out_features", C.c_int), ("rank", C.c_int), ("alpha", C.c_float), ("scaling", C.c_float),
                ("base_weight", C.POINTER(Tensor)), ("lora_A", C.POINTER(Tensor)), ("lora_B", C.POINTER(Tensor)),
                ("frozen_base", C.POINTER(Tensor)), ("merged", C.c_bool)]


class LoRAAdapter(C.Structure):
    _fields_ = [("name", C.c_char * 64), ("rank", C.c_int), ("alpha", C.c_float), ("scaling", C.c_float), ("num_layers", C.c_int),
                ("layers", C.POINTER(C.POINTER(LoRALinear))), ("merged", C.c_bool)]


LP, AP = C.POINTER(LoRALinear), C.POINTER(LoRAAdapter)
_sig("cml_lora_linear_create", LP, TP, ci, C.c_float)
_sig("cml_lora_linear_free", None, LP)
_sig("cml_lora_linear_forward", TP, LP, TP)
_sig("cml_lora_linear_merge", ci, LP)
_sig("cml_lora_linear_unmerge", ci, LP)
_sig("cml_lora_adapter_create", AP, C.c_char_p, ci, C.c_float)
_sig("cml_lora_adapter_free", None, AP)
_sig("cml_lora_adapter_add_layer", ci, AP, LP)
_sig("cml_lora_adapter_merge_all", ci, AP)
_sig("cml_lora_adapter_unmerge_all", ci, AP)
_sig("cmlb200_lora_merge", ci, vp, vp, vp, ci, ci, ci, C.c_float, vp)
class QuantParams(C.Structure):
    _fields_ = [("scale", C.c_float), ("zero_point", C.c_int32)]


_sig("cml_quantize_compute_params", QuantParams, TP, C.c_bool)
_sig("cml_quantize_int8", TP, TP, C.POINTER(QuantParams), C.POINTER(QuantParams))
_sig("cml_dequantize_int8", TP, TP, C.POINTER(QuantParams))
_sig("cml_quantize_uint8", TP, TP, C.POINTER(QuantParams), C.POINTER(QuantParams))
_sig("cml_dequantize_uint8", TP, TP, C.POINTER(QuantParams))
_sig("gguf_open_write", vp, C.c_char_p)
_sig("gguf_write_tensor", ci, vp, C.c_char_p, TP)
_sig("gguf_write_blocks", ci, vp, C.c_char_p, ci, C.POINTER(C.c_int64), ci, vp)
_sig("gguf_write_metadata", ci, vp, C.c_char_p, ci, vp)
_sig("gguf_write_metadata_array", ci, vp, C.c_char_p, ci, vp, C.c_uint64)
_sig("cml_init", ci)
_sig("cml_cleanup", ci)
_sig("tensor_manual_seed", None, C.c_uint64)
_sig("tensor_get_seed", C.c_uint64)
REFERENCE_QUIRKS, KV_FP32, ALL_LOGITS_FP32 = 1, 2, 4


def tensor_to_numpy(tp, free=True):
    """Copy a host Tensor* returned by the library into a numpy array (fp32 / uint8 / fp16)."""
    import numpy as np
    t = tp.contents
    shape = [t.shape[i] for i in range(t.ndim)]
    np_dtype = {0: np.float32, 8: np.uint8, 7: np.int8, 5: np.float16, 2: np.int32}[t.dtype]
    n = int(np.prod(shape))
    arr = np.frombuffer((C.c_char * (n * np.dtype(np_dtype).itemsize)).from_address(t.data), dtype=np_dtype).reshape(shape).copy()
    if free:
        lib.tensor_free(tp)
    return arr


def numpy_to_tensor(a):
    """A host Tensor* owning a copy of `a` (fp32, fp16, int32, uint8 or int8); release with lib.tensor_free."""
    import numpy as np
    a = np.ascontiguousarray(a)
    dt = {np.dtype(np.float32): 0, np.dtype(np.uint8): 8, np.dtype(np.int8): 7, np.dtype(np.int32): 2, np.dtype(np.float16): 5}[a.dtype]
    cfg = TensorConfig(dt, 0, True, True)
    shape = (C.c_int * a.ndim)(*a.shape)
    return lib.tensor_from_data(np_ptr(a), shape, a.ndim, C.byref(cfg))
