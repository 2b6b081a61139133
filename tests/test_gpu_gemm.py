"""GPU parity of the tcgen05 prefill dequant-GEMM (bf16 activations/outputs, fp32 accumulate
in tensor memory). Tolerance 1e-2 relative to max|y| (bf16 tensor-core prefill), as the path
is specified; the oracle is fed the fp32 values of the bf16-rounded activations."""
import numpy as np
import pytest
import torch

from conftest import rel_err_inf
from gpu_util import gemm_status, make_weight, stream_ptr, to_dev

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _gemm(pkg, synth, W, x, N, dev, splits=0):
    M = x.shape[0]
    xb, _ = synth.bf16_round(x)
    d_x = to_dev(xb.reshape(x.shape), dev)
    d_y = torch.zeros((M, N), dtype=torch.uint16, device=dev)
    if splits:
        pkg.check(pkg.lib.cmlb200_gemm_bf16_splitk(W.q, d_x.data_ptr(), d_y.data_ptr(), M, splits, stream_ptr()), "gemm")
    else:
        pkg.check(pkg.lib.cmlb200_gemm_bf16(W.q, d_x.data_ptr(), d_y.data_ptr(), M, stream_ptr()), "gemm")
    assert gemm_status(pkg) == 0, "a bounded wait inside the tensor-core kernel expired"
    return synth.bf16_to_f32(d_y.cpu().numpy())


@pytest.mark.parametrize("kind", ["nf4", "q4_0", "q8_0"])
@pytest.mark.parametrize("M", [1, 16, 64, 100, 256, 300, 513, 1000])
def test_gemm_matches_oracle(pkg, synth, ob, orc, torch_dev, kind, M):
    rng = np.random.default_rng(200 + M)
    N, K = 200, 512                                    # ragged N (tile is 128 rows)
    W, Wf = make_weight(pkg, synth, ob, orc, torch_dev, rng, kind, N, K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    _, xr = synth.bf16_round(x)
    got = _gemm(pkg, synth, W, x, N, torch_dev)
    want = ob.linear_nt(orc, xr.reshape(x.shape), Wf)
    assert rel_err_inf(got, want) <= TOL


@pytest.mark.parametrize("splits", [1, 2, 4])
def test_gemm_split_k_agrees(pkg, synth, ob, orc, torch_dev, splits):
    rng = np.random.default_rng(300)
    N, K, M = 256, 2048, 64
    W, Wf = make_weight(pkg, synth, ob, orc, torch_dev, rng, "nf4", N, K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    _, xr = synth.bf16_round(x)
    got = _gemm(pkg, synth, W, x, N, torch_dev, splits=splits)
    assert rel_err_inf(got, ob.linear_nt(orc, xr.reshape(x.shape), Wf)) <= TOL


@pytest.mark.parametrize("M", [64, 512, 2048])
def test_gemm_nf4_config_shape_sampled(pkg, synth, ob, orc, torch_dev, M):
    """NF4 4096 x 4096, block 64 at the benchmark's M values; the oracle checks sampled rows and
    columns (its full triple loop would take minutes)."""
    rng = np.random.default_rng(400 + M)
    N = K = 4096
    W, Wf = make_weight(pkg, synth, ob, orc, torch_dev, rng, "nf4", N, K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    _, xr = synth.bf16_round(x)
    got = _gemm(pkg, synth, W, x, N, torch_dev)
    ms = rng.choice(M, 16, replace=False)
    ns = rng.choice(N, 256, replace=False)
    want = ob.linear_nt(orc, xr.reshape(x.shape)[ms], Wf[ns])
    assert np.abs(got[np.ix_(ms, ns)] - want).max() / np.abs(want).max() <= TOL
    # whole-output check against an fp64 matmul of the same dequantised weights
    full = xr.reshape(x.shape).astype(np.float64) @ Wf.T.astype(np.float64)
    assert rel_err_inf(got, full) <= TOL


@pytest.mark.parametrize("kind,N,K,M", [("q4_0", 11008, 4096, 512), ("nf4", 4096, 4096, 2000), ("q4_0", 4096, 11008, 2048), ("nf4", 4096, 4096, 4096)])
def test_gemm_large_shapes_repeated(pkg, synth, ob, orc, torch_dev, kind, N, K, M):
    """LLaMA-sized weights with 512 to 4096 activation rows, incl. a ragged last tile; every output
    against an fp64 product, three launches in a row (cold and warm caches: a pipeline race would show
    as whole output columns off by a K slab's worth)."""
    rng = np.random.default_rng(900 + M)
    W, Wf = make_weight(pkg, synth, ob, orc, torch_dev, rng, kind, N, K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    _, xr = synth.bf16_round(x)
    full = xr.reshape(x.shape).astype(np.float64) @ Wf.T.astype(np.float64)
    for _ in range(3):
        assert rel_err_inf(_gemm(pkg, synth, W, x, N, torch_dev), full) <= TOL


@pytest.mark.parametrize("kind,K", [("q4_0", 1376), ("q8_0", 96), ("nf4", 1376), ("q4_0", 32)])
@pytest.mark.parametrize("M", [40, 300])
def test_gemm_k_tail_of_half_a_slab(pkg, synth, ob, orc, torch_dev, kind, K, M):
    """cols % 64 == 32 (LLaMA-7B's FFN width split over 8 ranks is 1376): the last 64-wide slab is
    half real, half zero; rows of an odd number of blocks start on odd scale indices."""
    rng = np.random.default_rng(500 + K + M)
    N = 200
    W, Wf = make_weight(pkg, synth, ob, orc, torch_dev, rng, kind, N, K, block=32)
    x = rng.standard_normal((M, K)).astype(np.float32)
    _, xr = synth.bf16_round(x)
    got = _gemm(pkg, synth, W, x, N, torch_dev)
    assert rel_err_inf(got, ob.linear_nt(orc, xr.reshape(x.shape), Wf)) <= TOL
    if K >= 256:
        got2 = _gemm(pkg, synth, W, x, N, torch_dev, splits=3)
        assert rel_err_inf(got2, ob.linear_nt(orc, xr.reshape(x.shape), Wf)) <= TOL


@pytest.mark.parametrize("M", [48, 300])
def test_gemm_output_modes(pkg, synth, ob, orc, torch_dev, M):
    """The epilogues the LLaMA prefill uses: fp32 output, accumulation onto an fp32 residual, and
    SwiGLU of an earlier gate output (in place), with and without the split-K reduction (M = 48
    takes it on this shape)."""
    rng = np.random.default_rng(700 + M)
    N, K = 384, 1024
    W, Wf = make_weight(pkg, synth, ob, orc, torch_dev, rng, "q4_0", N, K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    xb, xr = synth.bf16_round(x)
    want = ob.linear_nt(orc, xr.reshape(x.shape), Wf)
    d_x = to_dev(xb.reshape(x.shape), torch_dev)
    out32 = torch.zeros((M, N), dtype=torch.float32, device=torch_dev)
    pkg.check(pkg.lib.cmlb200_gemm_bf16_ex(W.q, d_x.data_ptr(), M, 1, out32.data_ptr(), None, stream_ptr()), "out_f32")
    torch.cuda.synchronize()
    assert rel_err_inf(out32.cpu().numpy(), want) <= TOL
    h0 = rng.standard_normal((M, N)).astype(np.float32)
    h = to_dev(h0, torch_dev)
    pkg.check(pkg.lib.cmlb200_gemm_bf16_ex(W.q, d_x.data_ptr(), M, 2, h.data_ptr(), None, stream_ptr()), "acc_f32")
    torch.cuda.synchronize()
    assert np.abs(h.cpu().numpy() - (h0 + want)).max() <= TOL * np.abs(want).max()
    gate = rng.standard_normal((M, N)).astype(np.float32)
    gb, gr = synth.bf16_round(gate)
    gr = gr.reshape(gate.shape)
    buf = to_dev(gb.reshape(gate.shape), torch_dev)
    pkg.check(pkg.lib.cmlb200_gemm_bf16_ex(W.q, d_x.data_ptr(), M, 3, buf.data_ptr(), buf.data_ptr(), stream_ptr()), "swiglu")
    torch.cuda.synchronize()
    ref = (gr / (1.0 + np.exp(-gr.astype(np.float64)))) * want
    assert np.abs(synth.bf16_to_f32(buf.cpu().numpy()) - ref).max() <= TOL * np.abs(ref).max()
    assert gemm_status(pkg) == 0
    assert pkg.lib.cmlb200_gemm_bf16_ex(W.q, d_x.data_ptr(), M, 3, buf.data_ptr(), None, stream_ptr()) == -1      # SwiGLU needs the gate
    assert pkg.lib.cmlb200_gemm_bf16_ex(W.q, d_x.data_ptr(), M, 7, buf.data_ptr(), None, stream_ptr()) == -1

