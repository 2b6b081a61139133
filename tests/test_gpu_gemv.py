"""GPU parity of the decode dequant-GEMV (fp32 activations, fp32 accumulate) against the
oracle: max relative error <= 2e-3 (the tolerance the path is specified with), measured
element-wise with a floor of 1e-3 * max|y|."""
import numpy as np
import pytest
import torch

from conftest import rel_err, rel_err_inf
from gpu_util import make_block_stream, make_weight, stream_ptr, to_dev

pytestmark = pytest.mark.gpu
# M <= 4 rounds x to 24 bits relative to each 32-block maximum: as good as fp32 accumulation
DIGIT_TOL = 1e-5
TOL = 2e-3


def _run(pkg, fn, W, x, N, dev, y0=None, W2=None):
    M = x.shape[0]
    d_x = to_dev(x, dev)
    d_y = torch.zeros((M, N), dtype=torch.float32, device=dev) if y0 is None else to_dev(y0, dev)
    if W2 is None:
        pkg.check(fn(W.q, d_x.data_ptr(), d_y.data_ptr(), M, stream_ptr()), "gemv")
    else:
        pkg.check(fn(W.q, W2.q, d_x.data_ptr(), d_y.data_ptr(), M, stream_ptr()), "gemv_swiglu")
    torch.cuda.synchronize()
    return d_y.cpu().numpy()


@pytest.mark.parametrize("kind", ["q8_0", "q4_0", "nf4"])
@pytest.mark.parametrize("M", [1, 2, 3, 8, 32])
def test_gemv_matches_oracle(pkg, synth, ob, orc, torch_dev, kind, M):
    rng = np.random.default_rng(100 + M)
    N, K = 515, 1024                                  # ragged N: not a multiple of the row group
    W, Wf = make_weight(pkg, synth, ob, orc, torch_dev, rng, kind, N, K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    got = _run(pkg, pkg.lib.cmlb200_gemv, W, x, N, torch_dev)
    want = ob.linear_nt(orc, x, Wf)
    assert rel_err(got, want) <= TOL


@pytest.mark.parametrize("kind,N,K", [("q8_0", 4096, 4096), ("q4_0", 11008, 4096), ("q4_0", 4096, 11008), ("nf4", 4096, 4096)])
def test_gemv_config_shapes_sampled_rows(pkg, synth, ob, orc, torch_dev, kind, N, K):
    """Full benchmark shapes; the oracle checks 96 sampled output rows (it is a scalar loop)."""
    rng = np.random.default_rng(7)
    W, Wf = make_weight(pkg, synth, ob, orc, torch_dev, rng, kind, N, K)
    x = rng.standard_normal((1, K)).astype(np.float32)
    got = _run(pkg, pkg.lib.cmlb200_gemv, W, x, N, torch_dev)
    rows = rng.choice(N, 96, replace=False)
    want = ob.linear_nt(orc, x, Wf[rows])
    scale = np.abs(x @ Wf.T).max()
    assert np.abs(got[:, rows] - want).max() / scale <= DIGIT_TOL
    assert rel_err(got[:, rows], want) <= TOL


def test_gemv_linearity_at_full_size(pkg, synth, ob, orc, torch_dev):
    """Size-independent property at the full Q4_0 config: W.(a*x1 + x2) = a*W.x1 + W.x2."""
    rng = np.random.default_rng(8)
    N, K = 11008, 4096
    W, _ = make_weight(pkg, synth, ob, orc, torch_dev, rng, "q4_0", N, K)
    x1 = rng.standard_normal((1, K)).astype(np.float32)
    x2 = rng.standard_normal((1, K)).astype(np.float32)
    y1 = _run(pkg, pkg.lib.cmlb200_gemv, W, x1, N, torch_dev)
    y2 = _run(pkg, pkg.lib.cmlb200_gemv, W, x2, N, torch_dev)
    y3 = _run(pkg, pkg.lib.cmlb200_gemv, W, (np.float32(0.5) * x1 + x2), N, torch_dev)
    assert rel_err_inf(y3, 0.5 * y1 + y2) <= DIGIT_TOL
    # batching is row-independent: M=8 output rows equal eight M=1 calls
    X = rng.standard_normal((8, K)).astype(np.float32)
    Y = _run(pkg, pkg.lib.cmlb200_gemv, W, X, N, torch_dev)
    for m in (0, 3, 7):
        assert rel_err_inf(Y[m:m + 1], _run(pkg, pkg.lib.cmlb200_gemv, W, X[m:m + 1], N, torch_dev)) <= DIGIT_TOL


@pytest.mark.parametrize("kind", ["q4_0", "q8_0"])
def test_gemv_accumulate_and_swiglu_epilogues(pkg, synth, ob, orc, torch_dev, kind):
    rng = np.random.default_rng(9)
    N, K, M = 300, 512, 2
    Wg, Wgf = make_weight(pkg, synth, ob, orc, torch_dev, rng, kind, N, K)
    Wu, Wuf = make_weight(pkg, synth, ob, orc, torch_dev, rng, kind, N, K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    y0 = rng.standard_normal((M, N)).astype(np.float32)
    acc = _run(pkg, pkg.lib.cmlb200_gemv_accum, Wg, x, N, torch_dev, y0=y0)
    assert rel_err(acc, y0 + ob.linear_nt(orc, x, Wgf)) <= TOL
    g, u = ob.linear_nt(orc, x, Wgf), ob.linear_nt(orc, x, Wuf)
    want = (g / (1.0 + np.exp(-g.astype(np.float64)))).astype(np.float32) * u
    got = _run(pkg, pkg.lib.cmlb200_gemv_swiglu, Wg, x, N, torch_dev, W2=Wu)
    assert rel_err(got, want) <= TOL


def test_gemv_long_k_segments(pkg, synth, ob, orc, torch_dev):
    """K larger than one shared-memory activation segment (the 70B down-projection has K = 28672)."""
    rng = np.random.default_rng(10)
    N, K = 64, 28672
    W, Wf = make_weight(pkg, synth, ob, orc, torch_dev, rng, "q4_0", N, K)
    for M in (1, 4):
        x = rng.standard_normal((M, K)).astype(np.float32)
        assert rel_err(_run(pkg, pkg.lib.cmlb200_gemv, W, x, N, torch_dev), ob.linear_nt(orc, x, Wf)) <= TOL


def test_gemv_matches_stored_reference_output(pkg, golden, torch_dev):
    """The stored uop_linear output of the compiled reference on dequantised Q4_0 / Q8_0 weights."""
    from gpu_util import DevQMat
    for name, qtype in (("q8_0", 7), ("q4_0", 2)):
        blocks = golden[f"{name}_blocks"].reshape(-1, 34 if qtype == 7 else 18).copy()
        finite = np.isfinite(golden[f"{name}_dequant_bits"].view(np.float32).reshape(-1, 32)).all(1)
        blocks[~finite, :2] = 0                       # the generator zeroed non-finite weights
        W = DevQMat.from_gguf(pkg, torch_dev, qtype, np.ascontiguousarray(blocks.reshape(-1)), 8, 256)
        got = _run(pkg, pkg.lib.cmlb200_gemv, W, golden[f"{name}_x"], 8, torch_dev)
        assert rel_err_inf(got, golden[f"{name}_linear_y"]) <= DIGIT_TOL


@pytest.mark.parametrize("kind", ["q4_0", "q8_0"])
def test_gemv_with_subnormal_scales_follows_reference_quirk(pkg, synth, ob, orc, torch_dev, kind):
    """Blocks whose fp16 scale is subnormal widen to half the IEEE value in C-ML; the matmul
    kernels follow when the weight carries CMLB200_QMAT_SUBNORMAL_SCALES."""
    from gpu_util import DevQMat
    rng = np.random.default_rng(21)
    N, K = 64, 256
    qtype, bb = (7, 34) if kind == "q8_0" else (2, 18)
    blocks = (synth.q8_0_blocks if kind == "q8_0" else synth.q4_0_blocks)(rng, N, K).reshape(-1, bb)
    blocks[:, :2] = rng.integers(1, 0x0400, len(blocks), dtype=np.uint16).view(np.uint8).reshape(-1, 2)  # all subnormal
    blocks = np.ascontiguousarray(blocks.reshape(-1))
    W = DevQMat.from_gguf(pkg, torch_dev, qtype, blocks, N, K)
    assert W.q.flags == 1
    Wf = ob.dequant_blocks(orc, qtype, blocks, N * K).reshape(N, K)
    for M in (1, 2, 8):
        x = rng.standard_normal((M, K)).astype(np.float32)
        assert rel_err(_run(pkg, pkg.lib.cmlb200_gemv, W, x, N, torch_dev), ob.linear_nt(orc, x, Wf)) <= TOL


@pytest.mark.parametrize("kind", ["q4_0", "q8_0"])
@pytest.mark.parametrize("K", [512, 1056])                 # tensor-core kernel (K % 256 == 0) and register kernel
def test_gemv_digit_entry_points_and_fused_rmsnorm(pkg, synth, ob, orc, torch_dev, kind, K):
    """x_digits + gemv_xq, rmsnorm_digits + gemv_xq and gemv_rmsnorm agree with the oracle's
    rms_norm followed by its linear."""
    rng = np.random.default_rng(11)
    N, eps = 301, 1e-5
    Wg, Wgf = make_weight(pkg, synth, ob, orc, torch_dev, rng, kind, N, K)
    Wu, Wuf = make_weight(pkg, synth, ob, orc, torch_dev, rng, kind, N, K)
    nw = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float16)
    for M in (1, 2, 3):
        x = (3.0 * rng.standard_normal((M, K))).astype(np.float32)
        normed = np.zeros_like(x)
        nwf = nw.astype(np.float32)
        orc.orc_rmsnorm(x.ctypes.data, nwf.ctypes.data, M, K, eps, normed.ctypes.data)
        d_x, d_nw = to_dev(x, torch_dev), to_dev(nw.view(np.uint16), torch_dev)
        d_xq = torch.zeros(pkg.lib.cmlb200_xq_bytes(M, K), dtype=torch.uint8, device=torch_dev)
        d_y = torch.zeros((M, N), dtype=torch.float32, device=torch_dev)
        # plain digits
        pkg.check(pkg.lib.cmlb200_x_digits(d_x.data_ptr(), M, K, d_xq.data_ptr(), stream_ptr()), "x_digits")
        pkg.check(pkg.lib.cmlb200_gemv_xq(Wg.q, None, d_xq.data_ptr(), d_y.data_ptr(), M, 0, stream_ptr()), "gemv_xq")
        assert rel_err(d_y.cpu().numpy(), ob.linear_nt(orc, x, Wgf)) <= TOL
        # digits out of RMSNorm, fp32 copy of the normalised rows on the side
        d_n = torch.zeros_like(d_x)
        pkg.check(pkg.lib.cmlb200_rmsnorm_digits(d_x.data_ptr(), d_nw.data_ptr(), M, K, eps, d_n.data_ptr(), d_xq.data_ptr(), stream_ptr()), "rmsnorm_digits")
        assert rel_err(d_n.cpu().numpy(), normed) <= 1e-5
        y0 = rng.standard_normal((M, N)).astype(np.float32)
        d_y.copy_(to_dev(y0, torch_dev))
        pkg.check(pkg.lib.cmlb200_gemv_xq(Wg.q, None, d_xq.data_ptr(), d_y.data_ptr(), M, 1, stream_ptr()), "gemv_xq accum")
        want = ob.linear_nt(orc, normed, Wgf)
        assert rel_err(d_y.cpu().numpy(), y0 + want) <= TOL
        # normalisation inside the GEMV launch: store and SwiGLU
        pkg.check(pkg.lib.cmlb200_gemv_rmsnorm(Wg.q, None, d_x.data_ptr(), d_nw.data_ptr(), eps, d_y.data_ptr(), M, 0, stream_ptr()), "gemv_rmsnorm")
        assert rel_err(d_y.cpu().numpy(), want) <= TOL
        pkg.check(pkg.lib.cmlb200_gemv_rmsnorm(Wg.q, Wu.q, d_x.data_ptr(), d_nw.data_ptr(), eps, d_y.data_ptr(), M, 2, stream_ptr()), "gemv_rmsnorm swiglu")
        u = ob.linear_nt(orc, normed, Wuf)
        assert rel_err(d_y.cpu().numpy(), (want / (1.0 + np.exp(-want.astype(np.float64)))).astype(np.float32) * u) <= TOL


@pytest.mark.parametrize("kind", ["q4_0", "q8_0"])
@pytest.mark.parametrize("N,K", [(5, 256), (16, 512), (33, 4096), (301, 2816)])
def test_gemv_tensor_core_kernel_edges(pkg, synth, ob, orc, torch_dev, kind, N, K):
    """Shapes around the tensor-core decode kernel's tiling: fewer rows than one 16-row item, a single
    8-block unit (most warps idle), K that leaves the last warps without a unit, every M up to 8
    (4 + 2 + 1 rows per launch), all three epilogues."""
    rng = np.random.default_rng(12)
    Wg, Wgf = make_weight(pkg, synth, ob, orc, torch_dev, rng, kind, N, K)
    Wu, Wuf = make_weight(pkg, synth, ob, orc, torch_dev, rng, kind, N, K)
    for M in (1, 2, 3, 4, 5, 7, 8):
        x = rng.standard_normal((M, K)).astype(np.float32)
        x[0, :32] = 0.0                                   # an all-zero block
        x[M - 1, 40] = 1e4                                # one huge element in a slice
        g, u = ob.linear_nt(orc, x, Wgf), ob.linear_nt(orc, x, Wuf)
        assert rel_err(_run(pkg, pkg.lib.cmlb200_gemv, Wg, x, N, torch_dev), g) <= TOL
        y0 = rng.standard_normal((M, N)).astype(np.float32)
        assert rel_err(_run(pkg, pkg.lib.cmlb200_gemv_accum, Wg, x, N, torch_dev, y0=y0), y0 + g) <= TOL
        with np.errstate(over="ignore"):                  # exp(-g) may overflow to inf for the huge element: silu -> 0
            want = (g / (1.0 + np.exp(-g.astype(np.float64)))).astype(np.float32) * u
        assert rel_err(_run(pkg, pkg.lib.cmlb200_gemv_swiglu, Wg, x, N, torch_dev, W2=Wu), want) <= TOL


@pytest.mark.parametrize("N,K", [(40, 256), (301, 2816), (48, 4352), (9700, 4096), (333, 11008)])
def test_gemv_eight_row_kernel(pkg, synth, ob, orc, torch_dev, N, K):
    """Q4_0 with 5..8 rows of x per launch (plane-major digit columns): a single unit, idle warps in
    the only phase, a second phase with one unit, more than four items per CTA, three phases; row
    counts that are not a multiple of 16; all three epilogues, RMSNorm inside the launch, and M
    above 8 (several launches)."""
    rng = np.random.default_rng(13)
    eps = 1e-5
    Wg, Wgf = make_weight(pkg, synth, ob, orc, torch_dev, rng, "q4_0", N, K)
    Wu, Wuf = make_weight(pkg, synth, ob, orc, torch_dev, rng, "q4_0", N, K)
    nw = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float16)
    for M in (5, 6, 8, 13, 32):
        x = rng.standard_normal((M, K)).astype(np.float32)
        x[0, :32] = 0.0                                   # an all-zero block
        x[M - 1, 40] = 1e4                                # one huge element in a slice
        g, u = ob.linear_nt(orc, x, Wgf), ob.linear_nt(orc, x, Wuf)
        assert rel_err(_run(pkg, pkg.lib.cmlb200_gemv, Wg, x, N, torch_dev), g) <= TOL
        y0 = rng.standard_normal((M, N)).astype(np.float32)
        assert rel_err(_run(pkg, pkg.lib.cmlb200_gemv_accum, Wg, x, N, torch_dev, y0=y0), y0 + g) <= TOL
        with np.errstate(over="ignore"):
            want = (g / (1.0 + np.exp(-g.astype(np.float64)))).astype(np.float32) * u
        assert rel_err(_run(pkg, pkg.lib.cmlb200_gemv_swiglu, Wg, x, N, torch_dev, W2=Wu), want) <= TOL
        if M > 8:
            continue
        x = (3.0 * rng.standard_normal((M, K))).astype(np.float32)
        normed, nwf = np.zeros_like(x), nw.astype(np.float32)
        orc.orc_rmsnorm(x.ctypes.data, nwf.ctypes.data, M, K, eps, normed.ctypes.data)
        d_x, d_nw = to_dev(x, torch_dev), to_dev(nw.view(np.uint16), torch_dev)
        d_y = torch.zeros((M, N), dtype=torch.float32, device=torch_dev)
        g, u = ob.linear_nt(orc, normed, Wgf), ob.linear_nt(orc, normed, Wuf)
        pkg.check(pkg.lib.cmlb200_gemv_rmsnorm(Wg.q, None, d_x.data_ptr(), d_nw.data_ptr(), eps, d_y.data_ptr(), M, 0, stream_ptr()), "gemv_rmsnorm")
        assert rel_err(d_y.cpu().numpy(), g) <= TOL
        pkg.check(pkg.lib.cmlb200_gemv_rmsnorm(Wg.q, Wu.q, d_x.data_ptr(), d_nw.data_ptr(), eps, d_y.data_ptr(), M, 2, stream_ptr()), "gemv_rmsnorm swiglu")
        assert rel_err(d_y.cpu().numpy(), (g / (1.0 + np.exp(-g.astype(np.float64)))).astype(np.float32) * u) <= TOL


@pytest.mark.parametrize("gtype", [3, 12, 13, 14])
@pytest.mark.parametrize("M", [1, 3, 8, 13])
def test_gemv_other_gguf_block_types(pkg, synth, ob, orc, torch_dev, gtype, M):
    """Q4_1, Q4_K, Q5_K, Q6_K weights straight from the block stream (C-ML's own nibble order for
    the K types), against the oracle's dequantise-then-multiply."""
    rng = np.random.default_rng(500 + 10 * gtype + M)
    N, K = 301, 1536 if gtype != 3 else 1504          # ragged N; Q4_1: K a multiple of 32 only
    W, Wf = make_block_stream(pkg, synth, ob, orc, torch_dev, rng, gtype, N, K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    got = _run(pkg, pkg.lib.cmlb200_gemv, W, x, N, torch_dev)
    want = ob.linear_nt(orc, x, Wf)
    assert rel_err(got, want) <= TOL
    y0 = rng.standard_normal((M, N)).astype(np.float32)
    acc = _run(pkg, pkg.lib.cmlb200_gemv_accum, W, x, N, torch_dev, y0=y0)
    assert rel_err(acc, y0 + want) <= TOL


@pytest.mark.parametrize("gtype,N,K", [(12, 4096, 4096), (14, 4096, 11008)])
def test_gemv_other_block_types_long_k_sampled_rows(pkg, synth, ob, orc, torch_dev, gtype, N, K):
    """LLaMA-7B widths: K longer than one staged segment of x at M = 8."""
    rng = np.random.default_rng(40 + gtype)
    W, Wf = make_block_stream(pkg, synth, ob, orc, torch_dev, rng, gtype, N, K)
    x = rng.standard_normal((8, K)).astype(np.float32)
    got = _run(pkg, pkg.lib.cmlb200_gemv, W, x, N, torch_dev)
    rows = rng.choice(N, 64, replace=False)
    assert rel_err(got[:, rows], ob.linear_nt(orc, x, Wf[rows])) <= TOL


def test_gemv_other_block_types_reject_swiglu_and_partial_blocks(pkg, synth, ob, orc, torch_dev):
    rng = np.random.default_rng(3)
    W, _ = make_block_stream(pkg, synth, ob, orc, torch_dev, rng, 12, 16, 512)
    x = to_dev(rng.standard_normal((1, 512)).astype(np.float32), torch_dev)
    y = torch.zeros((1, 16), dtype=torch.float32, device=torch_dev)
    assert pkg.lib.cmlb200_gemv_swiglu(W.q, W.q, x.data_ptr(), y.data_ptr(), 1, stream_ptr()) != 0
    bad = pkg.QMat(12, 16, 384, 256, W.qs.data_ptr(), None, 0, None)       # 384 is not a whole number of 256-blocks
    assert pkg.lib.cmlb200_gemv(bad, x.data_ptr(), y.data_ptr(), 1, stream_ptr()) != 0


@pytest.mark.parametrize("kind,N,K", [("q4_0", 11008, 4096), ("q8_0", 1000, 1056), ("nf4", 384, 1024), ("q4_0", 200, 512)])
@pytest.mark.parametrize("M", [1, 3, 8])
def test_gemv_host_buffers(pkg, synth, ob, orc, torch_dev, kind, N, K, M):
    """cmlb200_gemv_host: host activations in, host result out, with page-locked buffers (read and
    written by kernels over the bus) and with pageable ones (DMA copies). Both must give the bits
    of cmlb200_gemv on device buffers, and those match the oracle within the fp32 bound."""
    import torch
    rng = np.random.default_rng(1200 + M + K)
    W, Wf = make_weight(pkg, synth, ob, orc, torch_dev, rng, kind, N, K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    d_x = to_dev(x, torch_dev)
    d_y = torch.zeros((M, N), dtype=torch.float32, device=torch_dev)
    pkg.check(pkg.lib.cmlb200_gemv(W.q, d_x.data_ptr(), d_y.data_ptr(), M, stream_ptr()), "gemv")
    torch.cuda.synchronize()
    dev_result = d_y.cpu().numpy()
    assert rel_err(dev_result, ob.linear_nt(orc, x, Wf)) <= TOL
    xp = torch.from_numpy(x).pin_memory()
    yp = torch.zeros((M, N), dtype=torch.float32).pin_memory()
    for _ in range(2):                                   # the second call reuses the staging rows
        yp.zero_()
        pkg.check(pkg.lib.cmlb200_gemv_host(W.q, xp.data_ptr(), yp.data_ptr(), M, stream_ptr()), "gemv_host pinned")
        assert np.array_equal(yp.numpy(), dev_result)
    y_pageable = np.zeros((M, N), np.float32)
    pkg.check(pkg.lib.cmlb200_gemv_host(W.q, x.ctypes.data, y_pageable.ctypes.data, M, stream_ptr()), "gemv_host pageable")
    assert np.array_equal(y_pageable, dev_result)
    # an odd offset into the page-locked buffer: scalar staging
    if N % 4 == 0:
        yo = torch.zeros(M * N + 1, dtype=torch.float32).pin_memory()
        pkg.check(pkg.lib.cmlb200_gemv_host(W.q, xp.data_ptr(), yo.data_ptr() + 4, M, stream_ptr()), "gemv_host offset")
        assert np.array_equal(yo.numpy()[1:].reshape(M, N), dev_result)
    assert pkg.lib.cmlb200_gemv_host(W.q, None, yp.data_ptr(), M, stream_ptr()) == -1
    assert pkg.lib.cmlb200_gemv_host(W.q, xp.data_ptr(), yp.data_ptr(), 33, stream_ptr()) == -1
