"""GPU tests of the C-ML-compatible host entry points that wrap single kernels: gguf_dequantize,
gguf_read_tensor, cml_quantize_nf4 / cml_dequantize_nf4 and the quantized Linear forward."""
import ctypes as C

import numpy as np
import pytest

from conftest import rel_err, rel_err_inf

pytestmark = pytest.mark.gpu


def test_gguf_dequantize_host_pointers_bit_exact(pkg, synth, ob, orc, torch_dev):
    rng = np.random.default_rng(31)
    for qtype, gen in ((7, synth.q8_0_blocks), (2, synth.q4_0_blocks)):
        blocks = gen(rng, 16, 256)
        out = np.empty(16 * 256, np.float32)
        assert pkg.lib.gguf_dequantize(qtype, pkg.np_ptr(blocks), pkg.np_ptr(out), out.size) == 0
        assert np.array_equal(out.view(np.uint32), ob.dequant_blocks(orc, qtype, blocks, out.size).view(np.uint32))
        assert pkg.lib.gguf_dequantize(qtype, pkg.np_ptr(blocks), pkg.np_ptr(out), 48) == -1
        assert pkg.lib.gguf_dequantize(qtype, None, pkg.np_ptr(out), 32) == -1
    assert pkg.lib.gguf_dequantize(12, pkg.np_ptr(blocks), pkg.np_ptr(out), 128) == -1     # Q4_K blocks hold 256 elements
    assert pkg.lib.gguf_dequantize(6, pkg.np_ptr(blocks), pkg.np_ptr(out), 256) == -1       # not a type C-ML reads
    assert pkg.lib.gguf_type_is_quantized(2) and pkg.lib.gguf_type_is_quantized(14) and not pkg.lib.gguf_type_is_quantized(0)
    assert pkg.lib.gguf_quant_block_size(7) == 32 and pkg.lib.gguf_quant_block_size(12) == 256 and pkg.lib.gguf_quant_block_size(1) == 0
    assert pkg.lib.gguf_quant_type_size(2) == 18 and pkg.lib.gguf_quant_type_size(7) == 34


def test_gguf_reader_returns_dequantized_tensors(pkg, synth, ob, orc, torch_dev, tmp_path):
    rng = np.random.default_rng(32)
    blocks = synth.q4_0_blocks(rng, 8, 64)
    vec = rng.standard_normal(64).astype(np.float32)
    path = tmp_path / "t.gguf"
    synth.write_gguf(path, [("w", (64, 8), 2, blocks.tobytes()), ("v", (64,), 0, vec.tobytes())])
    ctx = pkg.lib.gguf_open_read(str(path).encode())
    assert ctx and pkg.lib.gguf_get_num_tensors(ctx) == 2 and pkg.lib.gguf_get_tensor_name(ctx, 0) == b"w"
    w = pkg.tensor_to_numpy(pkg.lib.gguf_read_tensor(ctx, b"w"))
    assert w.shape == (64, 8)                      # dims in file order, element stream unchanged (as C-ML reads it)
    assert np.array_equal(w.reshape(-1).view(np.uint32), ob.dequant_blocks(orc, 2, blocks, 512).view(np.uint32))
    assert np.array_equal(pkg.tensor_to_numpy(pkg.lib.gguf_read_tensor(ctx, b"v")), vec)
    assert not pkg.lib.gguf_read_tensor(ctx, b"missing")
    pkg.lib.gguf_close(ctx)
    assert not pkg.lib.gguf_open_read(b"/nonexistent.gguf")
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"NOPE" + b"\0" * 64)
    assert not pkg.lib.gguf_open_read(str(bad).encode())
    trunc = tmp_path / "trunc.gguf"
    trunc.write_bytes(path.read_bytes()[:60])
    assert not pkg.lib.gguf_open_read(str(trunc).encode())


@pytest.mark.parametrize("numel,block", [(12 * 128, 64), (131, 64), (4096, 32)])
def test_nf4_quantize_bit_exact(pkg, ob, orc, golden, torch_dev, numel, block):
    rng = np.random.default_rng(33)
    x = (rng.standard_normal(numel) * 0.05).astype(np.float32)
    x[:block] = 0.0
    t = pkg.numpy_to_tensor(x)
    sc, ns = C.POINTER(C.c_float)(), C.c_int()
    p = pkg.lib.cml_quantize_nf4(t, block, C.byref(sc), C.byref(ns))
    assert p
    packed = pkg.tensor_to_numpy(p)
    scales = np.ctypeslib.as_array(sc, (ns.value,)).copy()
    wp, ws = np.zeros((numel + 1) // 2, np.uint8), np.zeros((numel + block - 1) // block, np.float32)
    assert orc.orc_nf4_quantize(ob.p(x), numel, block, ob.p(wp), ob.p(ws)) == ns.value
    assert np.array_equal(packed, wp) and np.array_equal(scales.view(np.uint32), ws.view(np.uint32))
    d = pkg.lib.cml_dequantize_nf4(pkg.numpy_to_tensor(packed), sc, ns.value, block, numel)
    assert np.array_equal(pkg.tensor_to_numpy(d).view(np.uint32), ob.dequant_nf4(orc, wp, ws, block, numel).view(np.uint32))
    assert not pkg.lib.cml_quantize_nf4(None, block, C.byref(sc), C.byref(ns))
    assert not pkg.lib.cml_quantize_nf4(t, 0, C.byref(sc), C.byref(ns))
    pkg.lib.tensor_free(t)


def test_nf4_golden_vectors(pkg, golden, torch_dev):
    """Stored output of the compiled reference's cml_quantize_nf4 on the golden weight."""
    W = golden["nf4_W"]
    t = pkg.numpy_to_tensor(W.reshape(-1))
    sc, ns = C.POINTER(C.c_float)(), C.c_int()
    p = pkg.lib.cml_quantize_nf4(t, 64, C.byref(sc), C.byref(ns))
    assert np.array_equal(pkg.tensor_to_numpy(p), golden["nf4_packed"])
    assert np.array_equal(np.ctypeslib.as_array(sc, (ns.value,)).view(np.uint32), golden["nf4_scales"].view(np.uint32))
    pkg.lib.tensor_free(t)


@pytest.mark.parametrize("M", [3, 40])
def test_qlora_linear_forward(pkg, ob, orc, torch_dev, M):
    """y = x.dequant(W)^T + scaling * x.A^T.B^T (C-ML tests/test_qlora.c:153-518): shape, B = 0
    equals the base product, non-zero B changes it; M = 40 takes the bf16 tensor-core path."""
    rng = np.random.default_rng(34)
    N, K, r, block = 96, 256, 4, 64
    W = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    wt = pkg.numpy_to_tensor(W)
    q = pkg.lib.cml_qlora_linear_create(wt, r, 8.0, block)
    assert q and q.contents.scaling == 2.0 and (q.contents.in_features, q.contents.out_features) == (K, N)
    nf4 = q.contents.base_weight_nf4.contents
    packed = pkg.tensor_to_numpy(nf4.packed_data, free=False)
    scales = np.ctypeslib.as_array(nf4.scales, (nf4.num_scales,)).copy()
    A = pkg.tensor_to_numpy(q.contents.lora_A, free=False)
    assert np.all(pkg.tensor_to_numpy(q.contents.lora_B, free=False) == 0)
    x = rng.standard_normal((M, K)).astype(np.float32)
    xt = pkg.numpy_to_tensor(x)
    tol, xin = (2e-3, x) if M <= 32 else (1e-2, x)
    want0 = np.empty((M, N), np.float32)
    Bz = np.zeros((N, r), np.float32)
    assert orc.orc_qlora_forward(ob.p(xin), M, K, N, ob.p(packed), ob.p(scales), len(scales), block, ob.p(A), ob.p(Bz), r, 2.0, ob.p(want0)) == 0
    y0 = pkg.tensor_to_numpy(pkg.lib.cml_qlora_linear_forward(q, xt))
    assert y0.shape == (M, N) and rel_err_inf(y0, want0) <= tol
    B = (rng.standard_normal((N, r)) * 0.1).astype(np.float32)
    C.memmove(q.contents.lora_B.contents.data, B.ctypes.data, B.nbytes)
    want1 = np.empty((M, N), np.float32)
    assert orc.orc_qlora_forward(ob.p(xin), M, K, N, ob.p(packed), ob.p(scales), len(scales), block, ob.p(A), ob.p(B), r, 2.0, ob.p(want1)) == 0
    y1 = pkg.tensor_to_numpy(pkg.lib.cml_qlora_linear_forward(q, xt))
    assert rel_err_inf(y1, want1) <= tol and not np.allclose(y0, y1)
    assert pkg.lib.cml_qlora_memory_usage(q) < 0.5 * pkg.lib.cml_qlora_full_memory_usage(K, N)
    bad = pkg.numpy_to_tensor(rng.standard_normal((2, K + 64)).astype(np.float32))
    assert not pkg.lib.cml_qlora_linear_forward(q, bad)
    assert not pkg.lib.cml_qlora_linear_forward(None, xt)
    for t in (xt, bad, wt):
        pkg.lib.tensor_free(t)
    pkg.lib.cml_qlora_linear_free(q)


@pytest.mark.parametrize("gid,bs,bb", [(3, 32, 20), (12, 256, 144), (13, 256, 176), (14, 256, 210)])
def test_other_block_types_bit_exact_on_device(pkg, ob, orc, golden, torch_dev, tmp_path, gid, bs, bb):
    """Q4_1 / Q4_K / Q5_K / Q6_K through gguf_dequantize and gguf_read_tensor: the stored outputs of
    the compiled reference, then random bytes (any scale pattern) against the oracle."""
    blocks = np.ascontiguousarray(golden[f"gguf{gid}_blocks"])
    numel = blocks.size // bb * bs
    out = np.empty(numel, np.float32)
    assert pkg.lib.gguf_dequantize(gid, pkg.np_ptr(blocks), pkg.np_ptr(out), numel) == 0
    assert np.array_equal(out.view(np.uint32), golden[f"gguf{gid}_dequant_bits"])
    rng = np.random.default_rng(50 + gid)
    fresh = rng.integers(0, 256, 300 * bb, dtype=np.uint8)
    out = np.empty(300 * bs, np.float32)
    assert pkg.lib.gguf_dequantize(gid, pkg.np_ptr(fresh), pkg.np_ptr(out), out.size) == 0
    want = ob.dequant_blocks(orc, gid, fresh, out.size)
    both_nan = np.isnan(out) & np.isnan(want)          # NaN scales: a NaN on both sides, payload aside
    assert np.array_equal(out.view(np.uint32)[~both_nan], want.view(np.uint32)[~both_nan])
    # a file holding such a tensor can be read now
    import __graft_entry__ as entry
    synth = entry.load_synth()
    path = tmp_path / f"t{gid}.gguf"
    synth.write_gguf(path, [("w", (bs, 300), gid, fresh.tobytes())])
    ctx = pkg.lib.gguf_open_read(str(path).encode())
    assert ctx
    t = pkg.lib.gguf_read_tensor(ctx, b"w")
    assert t
    got = pkg.tensor_to_numpy(t)
    pkg.lib.gguf_close(ctx)
    assert np.array_equal(got.reshape(-1).view(np.uint32)[~both_nan], out.view(np.uint32)[~both_nan])


@pytest.mark.parametrize("tag", ["b16", "b4", "straddle"])
def test_qlora_forward_small_blocks_match_reference(pkg, golden, torch_dev, tag):
    """C-ML's own QLoRA test shapes (tests/test_qlora.c:174,332,453: block 16 and 4 on tiny weights)
    and a block that straddles rows: stored outputs of the compiled reference's
    cml_qlora_linear_forward. These shapes run the element-wise NF4 kernel."""
    n_out, n_in, block, rank, M = (int(v) for v in golden[f"qlora_{tag}_cfg"])
    W, x, A, B = (np.ascontiguousarray(golden[f"qlora_{tag}_{k}"]) for k in ("W", "x", "A", "B"))
    wt = pkg.numpy_to_tensor(W)
    q = pkg.lib.cml_qlora_linear_create(wt, rank, 4.0, block)
    assert q
    C.memmove(q.contents.lora_A.contents.data, A.ctypes.data, A.nbytes)
    C.memmove(q.contents.lora_B.contents.data, B.ctypes.data, B.nbytes)
    xt = pkg.numpy_to_tensor(x)
    y = pkg.tensor_to_numpy(pkg.lib.cml_qlora_linear_forward(q, xt))
    assert y.shape == (M, n_out) and rel_err_inf(y, golden[f"qlora_{tag}_y"]) <= 2e-3
    pkg.lib.tensor_free(xt)
    pkg.lib.tensor_free(wt)
    pkg.lib.cml_qlora_linear_free(q)


def test_nf4_tensor_dequantize_direct(pkg, ob, orc, torch_dev):
    """cml_nf4_tensor_create / cml_nf4_tensor_dequantize (src/nn/qlora.c:10-132): the dequantised
    tensor has the original shape and the oracle's bits."""
    rng = np.random.default_rng(35)
    W = (rng.standard_normal((24, 160)) * 0.07).astype(np.float32)
    wt = pkg.numpy_to_tensor(W)
    nf = pkg.lib.cml_nf4_tensor_create(wt, 32)
    assert nf and nf.contents.block_size == 32 and nf.contents.original_numel == W.size and nf.contents.num_scales == W.size // 32
    packed = pkg.tensor_to_numpy(nf.contents.packed_data, free=False)
    scales = np.ctypeslib.as_array(nf.contents.scales, (nf.contents.num_scales,)).copy()
    got = pkg.tensor_to_numpy(pkg.lib.cml_nf4_tensor_dequantize(nf))
    assert got.shape == W.shape
    assert np.array_equal(got.reshape(-1).view(np.uint32), ob.dequant_nf4(orc, packed, scales, 32, W.size).view(np.uint32))
    assert np.abs(got - W).max() <= 0.2 * np.abs(W).max()
    assert not pkg.lib.cml_nf4_tensor_dequantize(None)
    pkg.lib.cml_nf4_tensor_free(nf)
    pkg.lib.tensor_free(wt)
