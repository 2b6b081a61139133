"""GPU parity of the LoRA layer over an fp32 weight (C-ML src/nn/lora.c:105-320): forward with the
pair applied on the fly, merge into the weight, forward on the merged weight, unmerge, and the
adapter's merge_all / unmerge_all, against vectors from the compiled reference and an fp64 product."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
TOL = 2e-3


def rel(got, want):
    return float(np.abs(got - want).max() / np.abs(want).max())


def set_tensor(pkg, tp, a):
    t = tp.contents
    C.memmove(t.data, np.ascontiguousarray(a, np.float32).ctypes.data, a.size * 4)


def test_forward_merge_unmerge_match_the_reference(pkg, golden, torch_dev):
    lib = pkg.lib
    M, K, N, r, _ = (int(v) for v in golden["lora_cfg"])
    W0 = np.ascontiguousarray(golden["lora_W"])
    W = pkg.numpy_to_tensor(W0.copy())
    x = pkg.numpy_to_tensor(np.ascontiguousarray(golden["lora_x"]))
    lo = lib.cml_lora_linear_create(W, r, float(golden["lora_alpha"][0]))
    assert lo
    # B starts from zeros: the layer is the base Linear
    y0 = pkg.tensor_to_numpy(lib.cml_lora_linear_forward(lo, x))
    base = golden["lora_x"].astype(np.float64) @ W0.T.astype(np.float64)
    assert y0.shape == (M, N) and rel(y0, base) <= 1e-5
    set_tensor(pkg, lo.contents.lora_A, golden["lora_A"])
    set_tensor(pkg, lo.contents.lora_B, golden["lora_B"])
    y = pkg.tensor_to_numpy(lib.cml_lora_linear_forward(lo, x))
    assert rel(y, golden["lora_y"]) <= 1e-5
    assert lib.cml_lora_linear_merge(lo) == 0 and lo.contents.merged and lo.contents.frozen_base
    assert lib.cml_lora_linear_merge(lo) == -1                                   # already merged
    Wm = pkg.tensor_to_numpy(W, free=False)
    assert np.abs(Wm - golden["lora_W_merged"]).max() <= 1e-6 * np.abs(golden["lora_W_merged"]).max()
    ym = pkg.tensor_to_numpy(lib.cml_lora_linear_forward(lo, x))                 # the pair is inside W now
    assert rel(ym, golden["lora_y_merged"]) <= 1e-5 and rel(ym, y) <= 1e-5
    assert lib.cml_lora_linear_unmerge(lo) == 0 and not lo.contents.merged and not lo.contents.frozen_base
    assert np.array_equal(pkg.tensor_to_numpy(W, free=False), W0)                # bit for bit
    bad = pkg.numpy_to_tensor(np.zeros((2, K + 1), np.float32))
    assert not lib.cml_lora_linear_forward(lo, bad)                              # in_features mismatch
    lib.tensor_free(bad)
    lib.cml_lora_linear_free(lo)
    lib.tensor_free(x)
    lib.tensor_free(W)


@pytest.mark.parametrize("M,K,N,r", [(1, 64, 48, 1), (7, 300, 129, 8), (33, 1024, 512, 16)])
def test_random_shapes_against_fp64_and_adapter(pkg, torch_dev, M, K, N, r):
    lib = pkg.lib
    rng = np.random.default_rng(M + K)
    Ws = [rng.standard_normal((N, K)).astype(np.float32) for _ in range(2)]
    Wt = [pkg.numpy_to_tensor(w.copy()) for w in Ws]
    xn = rng.standard_normal((M, K)).astype(np.float32)
    x = pkg.numpy_to_tensor(xn)
    ad = lib.cml_lora_adapter_create(b"pair", r, 2.0 * r)
    layers, AB = [], []
    for w in Wt:
        lo = lib.cml_lora_linear_create(w, r, 2.0 * r)
        A = (rng.standard_normal((r, K)) * 0.1).astype(np.float32)
        B = (rng.standard_normal((N, r)) * 0.1).astype(np.float32)
        set_tensor(pkg, lo.contents.lora_A, A)
        set_tensor(pkg, lo.contents.lora_B, B)
        assert lib.cml_lora_adapter_add_layer(ad, lo) == 0
        layers.append(lo)
        AB.append((A, B))
    want = [xn.astype(np.float64) @ w.T.astype(np.float64) + 2.0 * (xn.astype(np.float64) @ A.T.astype(np.float64)) @ B.T.astype(np.float64)
            for w, (A, B) in zip(Ws, AB)]
    for lo, wv in zip(layers, want):
        assert rel(pkg.tensor_to_numpy(lib.cml_lora_linear_forward(lo, x)), wv) <= TOL * 1e-2
    assert lib.cml_lora_adapter_merge_all(ad) == 0 and ad.contents.merged
    assert lib.cml_lora_adapter_merge_all(ad) == -1
    for lo, w, wv, (A, B) in zip(layers, Wt, want, AB):
        merged = pkg.tensor_to_numpy(w, free=False)
        wm = Ws[layers.index(lo)].astype(np.float64) + 2.0 * B.astype(np.float64) @ A.astype(np.float64)
        assert np.abs(merged - wm).max() <= 1e-6 * np.abs(wm).max()
        assert rel(pkg.tensor_to_numpy(lib.cml_lora_linear_forward(lo, x)), wv) <= TOL * 1e-2
    assert lib.cml_lora_adapter_unmerge_all(ad) == 0 and not ad.contents.merged
    for w, w0 in zip(Wt, Ws):
        assert np.array_equal(pkg.tensor_to_numpy(w, free=False), w0)
    lib.cml_lora_adapter_free(ad)
    lib.tensor_free(x)
    for w in Wt:
        lib.tensor_free(w)
