"""LoRA layer, the parts that need no device: the adapter initialisation drawn from rand() exactly as
C-ML draws it (src/nn/lora.c:50-72; vector from the compiled reference), shapes, ownership,
argument errors and adapter bookkeeping (include/nn/lora.h)."""
import ctypes as C
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

libc = C.CDLL(None)
libc.srand.argtypes = [C.c_uint]


@pytest.fixture(scope="module")
def pkg():
    return entry.load_package()


def test_create_draws_the_adapter_c_ml_would(pkg, golden):
    M, K, N, r, seed = (int(v) for v in golden["lora_cfg"])
    W = pkg.numpy_to_tensor(np.ascontiguousarray(golden["lora_W"]))
    libc.srand(seed)
    lo = pkg.lib.cml_lora_linear_create(W, r, float(golden["lora_alpha"][0]))
    assert lo
    l = lo.contents
    assert (l.in_features, l.out_features, l.rank, l.merged) == (K, N, r, False)
    assert l.scaling == golden["lora_alpha"][0] / r and not l.frozen_base
    A = pkg.tensor_to_numpy(l.lora_A, free=False)
    B = pkg.tensor_to_numpy(l.lora_B, free=False)
    assert A.shape == (r, K) and B.shape == (N, r) and not B.any()
    # same libm here and where the vector was made; one ulp of slack for another build of it
    assert np.allclose(A, golden["lora_A_init"], rtol=2e-7, atol=0)
    assert pkg.lib.cml_lora_linear_unmerge(lo) == -1                      # not merged
    pkg.lib.cml_lora_linear_free(lo)
    pkg.lib.tensor_free(W)


def test_argument_errors_and_adapter_bookkeeping(pkg):
    lib = pkg.lib
    assert not lib.cml_lora_linear_create(None, 2, 1.0)
    W3 = pkg.numpy_to_tensor(np.zeros((2, 3, 4), np.float32))
    assert not lib.cml_lora_linear_create(W3, 2, 1.0)                     # not 2-D
    W = pkg.numpy_to_tensor(np.zeros((3, 4), np.float32))
    assert not lib.cml_lora_linear_create(W, 0, 1.0)
    assert lib.cml_lora_linear_merge(None) == -1 and lib.cml_lora_linear_unmerge(None) == -1
    assert not lib.cml_lora_linear_forward(None, W)
    assert not lib.cml_lora_adapter_create(None, 2, 4.0) and not lib.cml_lora_adapter_create(b"x", 0, 4.0)
    ad = lib.cml_lora_adapter_create(b"a-name-that-is-much-longer-than-the-sixty-three-characters-the-struct-keeps-for-it", 2, 4.0)
    assert ad and len(ad.contents.name) == 63 and ad.contents.scaling == 2.0 and ad.contents.num_layers == 0
    l1, l2 = lib.cml_lora_linear_create(W, 2, 4.0), lib.cml_lora_linear_create(W, 2, 4.0)
    assert lib.cml_lora_adapter_add_layer(ad, l1) == 0 and lib.cml_lora_adapter_add_layer(ad, l2) == 0
    assert ad.contents.num_layers == 2 and lib.cml_lora_adapter_add_layer(ad, None) == -1
    assert lib.cml_lora_adapter_unmerge_all(ad) == -1                     # not merged
    assert lib.cml_lora_adapter_merge_all(None) == -1
    lib.cml_lora_adapter_free(ad)                                         # frees both layers, not W
    lib.cml_lora_adapter_free(None)
    lib.cml_lora_linear_free(None)
    lib.tensor_free(W)
    lib.tensor_free(W3)


def test_quantisation_argument_errors_need_no_device(pkg):
    """src/core/quantization.c:40-48, 82-90: NULL tensors and parameters are refused before any device work."""
    lib = pkg.lib
    assert not lib.cml_quantize_int8(None, None, None) and not lib.cml_quantize_uint8(None, None, None)
    assert not lib.cml_dequantize_int8(None, None) and not lib.cml_dequantize_uint8(None, None)
    p0 = lib.cml_quantize_compute_params(None, False)
    assert (p0.scale, p0.zero_point) == (1.0, 0)
    u = pkg.numpy_to_tensor(np.zeros(4, np.uint8))
    assert not lib.cml_dequantize_uint8(u, None)
    lib.tensor_free(u)
