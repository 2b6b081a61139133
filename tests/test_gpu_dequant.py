"""GPU parity, bit-exact: dequantised weights must equal C-ML's CPU routines bit for bit."""
import numpy as np
import pytest
import torch

from gpu_util import DevQMat, stream_ptr, to_dev

pytestmark = pytest.mark.gpu


def _all_scale_blocks(rng, qtype):
    """65536 blocks, one per fp16 bit pattern as the scale (subnormals, inf, NaN included)."""
    bb, qb = (34, 32) if qtype == 7 else (18, 16)
    blk = np.zeros((65536, bb), np.uint8)
    blk[:, :2] = np.arange(65536, dtype=np.uint16).view(np.uint8).reshape(-1, 2)
    blk[:, 2:] = rng.integers(0, 256, (65536, qb), dtype=np.uint8)
    return np.ascontiguousarray(blk.reshape(-1))


def _same_bits(a, b):
    a, b = a.view(np.uint32), b.view(np.uint32)
    nan = np.isnan(a.view(np.float32)) & np.isnan(b.view(np.float32))
    return np.array_equal(a[~nan], b[~nan])


@pytest.mark.parametrize("qtype", [7, 2])
def test_raw_block_dequant_bit_exact_every_scale(pkg, ob, orc, torch_dev, qtype):
    rng = np.random.default_rng(11)
    blocks = _all_scale_blocks(rng, qtype)
    numel = 65536 * 32
    want = ob.dequant_blocks(orc, qtype, blocks, numel)
    d_blk = to_dev(blocks, torch_dev)
    d_out = torch.empty(numel, dtype=torch.float32, device=torch_dev)
    pkg.check(pkg.lib.cmlb200_gguf_dequantize(qtype, d_blk.data_ptr(), d_out.data_ptr(), numel, stream_ptr()))
    torch.cuda.synchronize()
    assert _same_bits(d_out.cpu().numpy(), want)


@pytest.mark.parametrize("qtype", [7, 2])
def test_repacked_dequant_bit_exact(pkg, ob, orc, torch_dev, qtype):
    rng = np.random.default_rng(12)
    blocks = _all_scale_blocks(rng, qtype)
    rows, cols = 512, 4096
    want = ob.dequant_blocks(orc, qtype, blocks, rows * cols)
    W = DevQMat.from_gguf(pkg, torch_dev, qtype, blocks, rows, cols)
    d_out = torch.empty(rows * cols, dtype=torch.float32, device=torch_dev)
    pkg.check(pkg.lib.cmlb200_dequant_qmat(W.q, d_out.data_ptr(), stream_ptr()))
    torch.cuda.synchronize()
    assert _same_bits(d_out.cpu().numpy(), want)


@pytest.mark.parametrize("name,qtype", [("q8_0", 7), ("q4_0", 2)])
def test_dequant_matches_stored_reference_output(pkg, golden, torch_dev, name, qtype):
    blocks = golden[f"{name}_blocks"]
    d_blk = to_dev(blocks, torch_dev)
    d_out = torch.empty(8 * 256, dtype=torch.float32, device=torch_dev)
    pkg.check(pkg.lib.cmlb200_gguf_dequantize(qtype, d_blk.data_ptr(), d_out.data_ptr(), 8 * 256, stream_ptr()))
    torch.cuda.synchronize()
    assert _same_bits(d_out.cpu().numpy(), golden[f"{name}_dequant_bits"].view(np.float32))


@pytest.mark.parametrize("numel,block", [(4096 * 64, 64), (131, 64), (64 * 33 + 1, 32), (2, 64)])
def test_nf4_dequant_bit_exact(pkg, ob, orc, torch_dev, numel, block):
    rng = np.random.default_rng(13)
    packed = rng.integers(0, 256, (numel + 1) // 2, dtype=np.uint8)
    ns = (numel + block - 1) // block
    scales = rng.uniform(0.01, 0.1, ns).astype(np.float32)
    scales[0] = 1e-10
    want = ob.dequant_nf4(orc, packed, scales, block, numel)
    d_p, d_s = to_dev(packed, torch_dev), to_dev(scales, torch_dev)
    d_out = torch.empty(numel, dtype=torch.float32, device=torch_dev)
    pkg.check(pkg.lib.cmlb200_dequantize_nf4(d_p.data_ptr(), d_s.data_ptr(), ns, block, numel, d_out.data_ptr(), stream_ptr()))
    torch.cuda.synchronize()
    assert np.array_equal(d_out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    # fewer scales than blocks: the block index clamps to the last scale (quantization.c:359)
    if ns > 1:
        want2 = ob.dequant_nf4(orc, packed, scales[:ns - 1].copy(), block, numel)
        pkg.check(pkg.lib.cmlb200_dequantize_nf4(d_p.data_ptr(), d_s.data_ptr(), ns - 1, block, numel, d_out.data_ptr(), stream_ptr()))
        torch.cuda.synchronize()
        assert np.array_equal(d_out.cpu().numpy().view(np.uint32), want2.view(np.uint32))


def test_nf4_golden_dequant(pkg, golden, torch_dev):
    packed, scales = golden["nf4_packed"], golden["nf4_scales"]
    n = packed.size * 2
    d_out = torch.empty(n, dtype=torch.float32, device=torch_dev)
    d_p, d_s = to_dev(packed, torch_dev), to_dev(scales, torch_dev)
    pkg.check(pkg.lib.cmlb200_dequantize_nf4(d_p.data_ptr(), d_s.data_ptr(), len(scales), 64, n, d_out.data_ptr(), stream_ptr()))
    torch.cuda.synchronize()
    assert np.array_equal(d_out.cpu().numpy().view(np.uint32), golden["nf4_dequant_bits"])


def test_full_size_dequant_checksum(pkg, ob, orc, synth, torch_dev):
    """Config-sized Q4_0 weight (11008 x 4096): the device and oracle outputs agree on a
    position-weighted checksum and on 64 random rows compared bit for bit."""
    rng = np.random.default_rng(14)
    rows, cols = 11008, 4096
    blocks = synth.q4_0_blocks(rng, rows, cols)
    W = DevQMat.from_gguf(pkg, torch_dev, 2, blocks, rows, cols)
    d_out = torch.empty(rows * cols, dtype=torch.float32, device=torch_dev)
    pkg.check(pkg.lib.cmlb200_dequant_qmat(W.q, d_out.data_ptr(), stream_ptr()))
    torch.cuda.synchronize()
    got = d_out.cpu().numpy().reshape(rows, cols)
    want = ob.dequant_blocks(orc, 2, blocks, rows * cols).reshape(rows, cols)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
