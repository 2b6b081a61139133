"""The allocation-free decode GEMV (cmlb200_gemv_noalloc) is for hosts that may not allocate
device memory while running: its activation scratch is a fixed array inside the library instead
of a buffer obtained with cudaMalloc. It must give the same numbers as the ordinary entry point,
call after call, although every call reuses that one array. Collected last on purpose."""
import numpy as np
import pytest
import torch

from conftest import rel_err
from gpu_util import make_weight, stream_ptr, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", ["q4_0", "q8_0"])
@pytest.mark.parametrize("K", [1024, 1056])               # the tensor-core kernel, and (K % 256 != 0) the dp4a kernel
def test_noalloc_matches_regular_entry_point_twice(pkg, synth, ob, orc, torch_dev, kind, K):
    rng = np.random.default_rng(4242)
    N = 515
    W, Wf = make_weight(pkg, synth, ob, orc, torch_dev, rng, kind, N, K)
    for call, M in enumerate((2, 1)):                     # two calls in a row, different activations
        x = rng.standard_normal((M, K)).astype(np.float32)
        d_x = to_dev(x, torch_dev)
        y_ref = torch.zeros((M, N), dtype=torch.float32, device=torch_dev)
        y_new = torch.full((M, N), -3.0, dtype=torch.float32, device=torch_dev)
        pkg.check(pkg.lib.cmlb200_gemv(W.q, d_x.data_ptr(), y_ref.data_ptr(), M, stream_ptr()), "cmlb200_gemv")
        pkg.check(pkg.lib.cmlb200_gemv_noalloc(W.q, d_x.data_ptr(), y_new.data_ptr(), M, stream_ptr()), "cmlb200_gemv_noalloc")
        torch.cuda.synchronize()
        got, want = y_new.cpu().numpy(), y_ref.cpu().numpy()
        assert rel_err(got, want) <= 2e-3, f"call {call}: differs from cmlb200_gemv"
        assert rel_err(got, ob.linear_nt(orc, x, Wf)) <= 2e-3, f"call {call}: differs from the oracle"


def test_noalloc_large_accepted_case_allocates_nothing(pkg, synth, ob, orc, torch_dev):
    """Four rows of 28672 activations (LLaMA-70B's FFN width) use 401 KB of the 512 KiB array. Once
    the first call on the device has looked the array up, a call leaves the device's free memory
    exactly as it found it."""
    rng = np.random.default_rng(4243)
    N, K, M = 48, 28672, 4
    W, Wf = make_weight(pkg, synth, ob, orc, torch_dev, rng, "q4_0", N, K)
    x = rng.standard_normal((M, K)).astype(np.float32)
    d_x = to_dev(x, torch_dev)
    y = torch.zeros((M, N), dtype=torch.float32, device=torch_dev)
    pkg.check(pkg.lib.cmlb200_gemv_noalloc(W.q, d_x.data_ptr(), y.data_ptr(), M, stream_ptr()), "cmlb200_gemv_noalloc")
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    y.zero_()
    pkg.check(pkg.lib.cmlb200_gemv_noalloc(W.q, d_x.data_ptr(), y.data_ptr(), M, stream_ptr()), "cmlb200_gemv_noalloc")
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
    assert rel_err(y.cpu().numpy(), ob.linear_nt(orc, x, Wf)) <= 2e-3


def test_noalloc_rejects_what_does_not_fit(pkg, torch_dev):
    fake = 0x1000
    W = pkg.QMat(pkg.Q4_0, 8, 65536, 32, fake, fake, 0, None)
    assert pkg.lib.cmlb200_gemv_noalloc(W, fake, fake, 4, None) == -1       # 4 x 65536 exceeds the built-in array
    assert b"built-in array" in pkg.last_error()
    assert pkg.lib.cmlb200_gemv_noalloc(pkg.QMat(pkg.Q4_0, 8, 64, 32, fake, fake, 0, None), fake, fake, 5, None) == -1
    assert pkg.lib.cmlb200_gemv_noalloc(pkg.QMat(pkg.NF4, 8, 64, 64, fake, fake, 0, None), fake, fake, 1, None) == -1
