"""GPU parity of the per-tensor int8 / uint8 quantisation (C-ML src/core/quantization.c:8-192):
parameters, quantised bytes and dequantised floats bit for bit against vectors from the compiled
reference, including ties of roundf, values that clamp, and quotients outside the int32 range
(where the compiled reference yields INT_MIN and wraps the zero-point addition)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def params_of(v):
    return float(v[:1].view(np.float32)[0]), int(v[1])


def test_parameters_and_round_trips_match_the_reference(pkg, golden, torch_dev):
    lib = pkg.lib
    x = pkg.numpy_to_tensor(np.ascontiguousarray(golden["q8_x"]).reshape(50, 100))
    for sym in (0, 1):
        p = lib.cml_quantize_compute_params(x, bool(sym))
        assert (p.scale, p.zero_point) == params_of(golden[f"q8_params_sym{sym}"])
    for name, uns, given in (("i8_auto", 0, None), ("u8_auto", 1, None), ("i8_given", 0, (0.1, 3)), ("u8_given", 1, (0.05, 128))):
        quant = lib.cml_quantize_uint8 if uns else lib.cml_quantize_int8
        dequant = lib.cml_dequantize_uint8 if uns else lib.cml_dequantize_int8
        used = pkg.QuantParams(0.0, 0)
        pin = C.byref(pkg.QuantParams(float(np.float32(given[0])), given[1])) if given else None
        q = quant(x, pin, C.byref(used))
        assert q
        assert (used.scale, used.zero_point) == params_of(golden[f"q8_{name}_params"])
        qa = pkg.tensor_to_numpy(q, free=False)
        assert qa.shape == (50, 100) and qa.dtype == (np.uint8 if uns else np.int8)
        assert np.array_equal(qa.reshape(-1).view(np.uint8), golden[f"q8_{name}_q"])
        d = dequant(q, C.byref(used))
        assert d
        da = pkg.tensor_to_numpy(d)
        assert np.array_equal(da.reshape(-1).view(np.uint32), golden[f"q8_{name}_deq"].view(np.uint32))
        # a tensor of the other signedness is refused
        assert not (lib.cml_dequantize_int8 if uns else lib.cml_dequantize_uint8)(q, C.byref(used))
        lib.tensor_free(q)
    lib.tensor_free(x)


def test_quotients_outside_int32_follow_the_compiled_reference(pkg, golden, torch_dev):
    lib = pkg.lib
    x = pkg.numpy_to_tensor(np.ascontiguousarray(golden["q8_x_outliers"]))
    for name in ("i8_out", "i8_out_neg", "u8_out"):
        uns, zp = (int(v) for v in golden[f"q8_{name}_cfg"])
        pin = pkg.QuantParams(float(golden[f"q8_{name}_scale"][0]), zp)
        q = (lib.cml_quantize_uint8 if uns else lib.cml_quantize_int8)(x, C.byref(pin), None)
        assert q
        assert np.array_equal(pkg.tensor_to_numpy(q).reshape(-1).view(np.uint8), golden[f"q8_{name}_q"]), name
    lib.tensor_free(x)


def test_large_tensor_and_argument_errors(pkg, torch_dev):
    lib = pkg.lib
    rng = np.random.default_rng(8)
    a = rng.standard_normal((1 << 22) + 3).astype(np.float32)
    a[12345], a[-1] = -7.5, 9.25
    x = pkg.numpy_to_tensor(a)
    p = lib.cml_quantize_compute_params(x, True)
    assert p.scale == float(np.float32(9.25) / np.float32(127.0)) and p.zero_point == 0
    p = lib.cml_quantize_compute_params(x, False)
    sc = (np.float32(9.25) - np.float32(-7.5)) / np.float32(255.0)
    assert p.scale == float(sc) and p.zero_point == int(np.round(np.float32(7.5) / sc)) - 128
    used = pkg.QuantParams(0.0, 0)
    q = lib.cml_quantize_int8(x, None, C.byref(used))
    want = np.clip(np.trunc(np.abs(a / np.float32(used.scale)) + np.float32(0.5)) * np.sign(a), -128, 127).astype(np.int8)
    got = pkg.tensor_to_numpy(q, free=False).reshape(-1)
    assert (got != want).sum() <= 4                       # numpy's fp32 division may differ in the last place on a tie
    d = pkg.tensor_to_numpy(lib.cml_dequantize_int8(q, C.byref(used)))
    assert np.abs(d - a).max() <= used.scale * 0.5001
    lib.tensor_free(q)
    lib.tensor_free(x)
    assert not lib.cml_quantize_int8(None, None, None) and not lib.cml_dequantize_int8(None, None)
    u = pkg.numpy_to_tensor(np.zeros(4, np.uint8))
    assert not lib.cml_quantize_int8(u, None, None)       # fp32 tensors only
    assert not lib.cml_dequantize_uint8(u, None)
    p0 = lib.cml_quantize_compute_params(None, True)
    assert (p0.scale, p0.zero_point) == (1.0, 0)
    lib.tensor_free(u)
