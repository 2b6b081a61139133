"""GPU parity of the tensor-core decode path (cmlb200_gemv_tiles: tcgen05 kind::i8 over
tile-major weights) against the oracle, tolerance 2e-3 as for every fp32-accumulate path."""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import rel_err, rel_err_inf
from gpu_util import stream_ptr, to_dev

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _weight(pkg, synth, ob, orc, dev, rng, kind, N, K):
    qtype = pkg.Q8_0 if kind == "q8_0" else pkg.Q4_0
    blocks = (synth.q8_0_blocks if kind == "q8_0" else synth.q4_0_blocks)(rng, N, K)
    tiles = to_dev(pkg.repack_tiles(qtype, blocks, N, K), dev)
    Wf = ob.dequant_blocks(orc, qtype, blocks, N * K).reshape(N, K)
    return pkg.QMat(qtype, N, K, 32, tiles.data_ptr(), None, 0, None), tiles, Wf


def _status(pkg):
    st = C.c_int(-1)
    pkg.check(pkg.lib.cmlb200_gemv_tiles_status(C.byref(st), 1))
    return st.value


def _run(pkg, W, x, N, dev, y0=None):
    M = x.shape[0]
    d_x = to_dev(x, dev)
    d_y = torch.full((M, N), 7.0, dtype=torch.float32, device=dev) if y0 is None else to_dev(y0, dev)
    pkg.check(pkg.lib.cmlb200_gemv_tiles(W, d_x.data_ptr(), d_y.data_ptr(), M, 0 if y0 is None else 1, stream_ptr()), "gemv_tiles")
    assert _status(pkg) == 0, "a bounded wait inside the tensor-core GEMV expired"
    return d_y.cpu().numpy()


@pytest.mark.parametrize("kind", ["q4_0", "q8_0"])
@pytest.mark.parametrize("M", [1, 2, 3, 5, 8, 10, 11, 32])
def test_gemv_tiles_matches_oracle(pkg, synth, ob, orc, torch_dev, kind, M):
    rng = np.random.default_rng(500 + M)
    N, K = 300, 1024                                   # ragged N: three row tiles, the last one partial
    W, keep, Wf = _weight(pkg, synth, ob, orc, torch_dev, rng, kind, N, K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    got = _run(pkg, W, x, N, torch_dev)
    assert rel_err(got, ob.linear_nt(orc, x, Wf)) <= TOL


@pytest.mark.parametrize("kind", ["q4_0", "q8_0"])
def test_gemv_tiles_small_and_accumulate(pkg, synth, ob, orc, torch_dev, kind):
    rng = np.random.default_rng(600)
    for N, K in ((1, 128), (128, 128), (129, 256)):
        W, keep, Wf = _weight(pkg, synth, ob, orc, torch_dev, rng, kind, N, K)
        x = rng.standard_normal((2, K)).astype(np.float32)
        assert rel_err(_run(pkg, W, x, N, torch_dev), ob.linear_nt(orc, x, Wf)) <= TOL
        y0 = rng.standard_normal((2, N)).astype(np.float32)
        assert rel_err(_run(pkg, W, x, N, torch_dev, y0=y0), y0 + ob.linear_nt(orc, x, Wf)) <= TOL


@pytest.mark.parametrize("kind,N,K", [("q8_0", 4096, 4096), ("q4_0", 11008, 4096), ("q4_0", 4096, 11008), ("q4_0", 32000, 4096)])
def test_gemv_tiles_config_shapes(pkg, synth, ob, orc, torch_dev, kind, N, K):
    """Benchmark shapes: sampled rows against the oracle, all rows against an fp64 matmul."""
    rng = np.random.default_rng(700)
    W, keep, Wf = _weight(pkg, synth, ob, orc, torch_dev, rng, kind, N, K)
    for M in (1, 8):
        x = rng.standard_normal((M, K)).astype(np.float32)
        got = _run(pkg, W, x, N, torch_dev)
        rows = rng.choice(N, 64, replace=False)
        assert rel_err(got[:, rows], ob.linear_nt(orc, x, Wf[rows])) <= TOL
        full = x.astype(np.float64) @ Wf.T.astype(np.float64)
        assert rel_err_inf(got, full) <= 1e-5


def test_gemv_tiles_x_edge_values(pkg, synth, ob, orc, torch_dev):
    """Activation blocks that are all zero, contain one huge element, or are tiny."""
    rng = np.random.default_rng(800)
    N, K = 256, 512
    W, keep, Wf = _weight(pkg, synth, ob, orc, torch_dev, rng, "q4_0", N, K)
    x = rng.standard_normal((3, K)).astype(np.float32)
    x[0, :64] = 0.0
    x[1, 100] = 1e6
    x[2] *= 1e-20
    got = _run(pkg, W, x, N, torch_dev)
    want = ob.linear_nt(orc, x, Wf)
    for m in range(3):
        assert rel_err(got[m], want[m]) <= TOL
