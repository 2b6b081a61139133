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
_sig("cmlb200_gemv_accum", ci, C.POINTER(QMat), vp, vp, ci, vp)
_sig("cmlb200_gemv_swiglu", ci, C.POINTER(QMat), C.POINTER(QMat), vp, vp, ci, vp)
_sig("cmlb200_tiles_bytes", sz, ci, ci, ci)
_sig("cmlb200_repack_tiles", ci, ci, vp, ci, ci, vp)
_sig("cmlb200_unrepack_tiles", ci, ci, vp, ci, ci, vp)
_sig("cmlb200_gemv_tiles", ci, C.POINTER(QMat), vp, vp, ci, ci, vp)
_sig("cmlb200_gemv_tiles_status", ci, C.POINTER(ci), ci)
_sig("cmlb200_gemm_bf16", ci, C.POINTER(QMat), vp, vp, ci, vp)
_sig("cmlb200_gemm_bf16_splitk", ci, C.POINTER(QMat), vp, vp, ci, ci, vp)
_sig("cmlb200_gemm_status", ci, C.POINTER(ci), ci)


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
