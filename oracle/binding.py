"""TEST INFRASTRUCTURE: ctypes access to the two CPU checkers.

  orc  -> oracle/libcml_oracle.so        this repo's C restatement (always buildable with gcc)
  ref  -> oracle/_ref/libref_driver.so   the compiled C-ML reference, None where it was not built

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may import this module."""
import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
vp, sz, ci, cf = C.c_void_p, C.c_size_t, C.c_int, C.c_float


def build_oracle():
    so = HERE / "libcml_oracle.so"
    src = HERE / "cml_oracle.c"
    if not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["gcc", "-std=c11", "-O2", "-fPIC", "-shared", "-o", str(so), str(src), "-lm"], check=True)
    return so


def reference_root():
    """Where the C-ML source tree is: $CML_REFERENCE_ROOT, else a `reference` directory beside
    this repository. None when neither exists (the prebuilt oracle/_ref/ is then used as it is)."""
    import os
    for cand in (os.environ.get("CML_REFERENCE_ROOT"), HERE.parent.parent / "reference"):
        if cand and Path(cand, "src").is_dir() and Path(cand, "include").is_dir():
            return str(cand)
    return None


def build_ref(root=None):
    """Compile the C-ML reference where its source tree is present; no-op elsewhere."""
    root = root or reference_root()
    if root:
        subprocess.run(["make", "-s", "-j8", "-C", str(HERE), "ref", f"REF={root}"], check=True)
    so = HERE / "_ref" / "libref_driver.so"
    return so if so.exists() else None


def build_reference_tests(root=None):
    """C-ML's own test programs for the path, compiled unchanged against this repo's headers and linked
    to its library (which must be built): oracle/_ref/tests/<name>. No-op without the source tree."""
    root = root or reference_root()
    if root:
        subprocess.run(["make", "-s", "-j8", "-C", str(HERE), "reftests", f"REF={root}"], check=True)
    d = HERE / "_ref" / "tests"
    return sorted(d.iterdir()) if d.is_dir() else []


def p(a):
    return a.ctypes.data_as(vp)


def _sig(lib, name, restype, *argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = list(argtypes)


class OrcLlamaStruct(C.Structure):
    _fields_ = [(n, ci) for n in ("vocab", "hidden", "inter", "layers", "heads", "kv_heads", "max_seq")] + \
               [("rope_theta", cf), ("eps", cf)] + \
               [(n, vp) for n in ("embed", "final_norm", "lm_head", "wq", "wk", "wv", "wo", "wgate", "wup", "wdown",
                                  "norm1", "norm2", "kcache", "vcache")] + \
               [("cur_len", ci), ("rope_all_heads", ci), ("mask_absolute", ci)]


class RefLlamaCfg(C.Structure):
    _fields_ = [(n, ci) for n in ("vocab", "hidden", "inter", "layers", "heads", "kv_heads", "max_seq")] + \
               [("rope_theta", cf), ("eps", cf)]


def load_orc():
    lib = C.CDLL(str(build_oracle()))
    _sig(lib, "orc_fp16_to_fp32", cf, C.c_uint16)
    _sig(lib, "orc_fp32_to_fp16", C.c_uint16, cf)
    _sig(lib, "orc_gguf_dequantize", ci, ci, vp, vp, sz)
    _sig(lib, "orc_quantize_q4_0", None, vp, vp, sz)
    _sig(lib, "orc_quantize_q8_0", None, vp, vp, sz)
    _sig(lib, "orc_nf4_quantize", ci, vp, sz, ci, vp, vp)
    _sig(lib, "orc_nf4_dequantize", ci, vp, vp, ci, ci, sz, vp)
    _sig(lib, "orc_linear_nt", None, vp, vp, ci, ci, ci, vp)
    _sig(lib, "orc_matmul_nn", None, vp, vp, ci, ci, ci, vp)
    _sig(lib, "orc_qlora_forward", ci, vp, ci, ci, ci, vp, vp, ci, ci, vp, vp, ci, cf, vp)
    _sig(lib, "orc_rmsnorm", None, vp, vp, ci, ci, cf, vp)
    _sig(lib, "orc_rope", None, vp, ci, ci, ci, ci, cf, ci)
    _sig(lib, "orc_gqa", ci, vp, vp, vp, ci, ci, ci, ci, ci, ci, vp)
    _sig(lib, "orc_paged_gqa", ci, vp, vp, vp, ci, ci, ci, ci, ci, cf, ci, vp)
    _sig(lib, "orc_lora_forward", None, vp, ci, ci, ci, vp, vp, vp, ci, cf, ci, vp, vp)
    _sig(lib, "orc_lora_merge", None, vp, vp, vp, ci, ci, ci, cf)
    _sig(lib, "orc_quant_params", None, vp, C.c_size_t, ci, vp)
    _sig(lib, "orc_quantize8", None, vp, C.c_size_t, cf, C.c_int32, ci, vp)
    _sig(lib, "orc_dequantize8", None, vp, C.c_size_t, cf, C.c_int32, ci, vp)
    _sig(lib, "orc_llama_forward", ci, C.POINTER(OrcLlamaStruct), vp, ci, vp)
    _sig(lib, "orc_argmax_first", ci, vp, ci)
    _sig(lib, "orc_tp_shard", ci, vp, ci, ci, ci, ci, ci, vp)
    _sig(lib, "orc_tp_allreduce_sum", None, vp, ci, sz, vp)
    return lib


_ref_cache = []


def load_ref():
    """The compiled reference driver, or None when oracle/_ref/ has not been built."""
    if _ref_cache:
        return _ref_cache[0]
    so = HERE / "_ref" / "libref_driver.so"
    lib = None
    if so.exists():
        lib = C.CDLL(str(so))
        _sig(lib, "ref_init", ci)
        _sig(lib, "ref_gguf_dequantize", ci, ci, vp, vp, sz)
        _sig(lib, "ref_gguf_type_is_quantized", ci, ci)
        _sig(lib, "ref_gguf_quant_block_size", ci, ci)
        _sig(lib, "ref_gguf_quant_type_size", sz, ci)
        _sig(lib, "ref_nf4_table", C.POINTER(cf * 16))
        _sig(lib, "ref_nf4_quantize", ci, vp, sz, ci, vp, vp)
        _sig(lib, "ref_nf4_dequantize", ci, vp, vp, ci, ci, sz, vp)
        _sig(lib, "ref_linear", ci, vp, vp, ci, ci, ci, vp)
        _sig(lib, "ref_weight_create", vp, vp, ci, ci)
        _sig(lib, "ref_weight_free", None, vp)
        _sig(lib, "ref_linear_resident", ci, vp, vp, ci, vp)
        _sig(lib, "ref_qlora_forward", ci, vp, ci, ci, ci, vp, vp, vp, ci, ci, cf, vp, vp, vp)
        _sig(lib, "ref_llama_create", vp, C.POINTER(RefLlamaCfg), vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp)
        _sig(lib, "ref_llama_forward", ci, vp, vp, ci, vp)
        _sig(lib, "ref_llama_reset", None, vp)
        _sig(lib, "ref_llama_cur_len", ci, vp)
        _sig(lib, "ref_llama_free", None, vp)
        _sig(lib, "ref_sample_greedy", ci, vp, ci, ci)
        _sig(lib, "ref_sample_token", ci, vp, ci, ci, cf, cf, ci, ci, C.c_uint)
        _sig(lib, "ref_rope_2d", ci, vp, ci, ci, ci, ci, cf)
        _sig(lib, "ref_gqa", ci, vp, vp, vp, ci, ci, ci, ci, ci, vp)
        _sig(lib, "ref_paged_gqa", ci, vp, vp, vp, ci, ci, ci, ci, ci, cf, ci, ci, ci, vp)
        _sig(lib, "ref_speculative_step", ci, vp, vp, ci, ci, vp, ci, ci, vp, vp, vp)
        _sig(lib, "ref_tp_column_then_row", ci, vp, ci, ci, vp, ci, vp, ci, ci, vp)
        _sig(lib, "ref_tokenizer_encode", ci, C.c_char_p, ci, C.c_char_p, ci, ci, C.c_char_p, vp, ci)
        _sig(lib, "ref_tokenizer_decode", ci, C.c_char_p, ci, vp, ci, vp, ci)
        _sig(lib, "ref_lora", ci, vp, ci, ci, ci, vp, ci, cf, C.c_uint, vp, vp, vp, vp, vp, vp)
        _sig(lib, "ref_quant_params", ci, vp, ci, ci, vp)
        _sig(lib, "ref_gguf_write", ci, C.c_char_p, vp, ci, ci, vp, ci, vp, ci)
        _sig(lib, "ref_quant8", ci, vp, ci, ci, ci, cf, ci, vp, vp, vp)
        lib.ref_init()
    _ref_cache.append(lib)
    return lib


# ---- numpy conveniences over the restatement ---------------------------------------------
def dequant_blocks(orc, qtype, blocks, numel):
    out = np.empty(numel, np.float32)
    rc = orc.orc_gguf_dequantize(qtype, p(blocks), p(out), numel)
    assert rc == 0
    return out


def dequant_nf4(orc, packed, scales, block, numel):
    out = np.empty(numel, np.float32)
    assert orc.orc_nf4_dequantize(p(packed), p(scales), len(scales), block, numel, p(out)) == 0
    return out


def linear_nt(orc, x, W):
    x = np.ascontiguousarray(x, np.float32)
    W = np.ascontiguousarray(W, np.float32)
    M, K = x.shape
    N = W.shape[0]
    y = np.empty((M, N), np.float32)
    orc.orc_linear_nt(p(x), p(W), M, N, K, p(y))
    return y


def ptr_array(arrs):
    """A C array of float pointers (keeps nothing alive: the caller owns `arrs`)."""
    return (vp * len(arrs))(*[a.ctypes.data for a in arrs])
