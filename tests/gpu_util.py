"""Helpers for the GPU parity tests: torch owns device memory and the stream; every compute
call goes through the C-ABI with raw pointers."""
import ctypes as C

import numpy as np
import torch


def to_dev(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def stream_ptr():
    return torch.cuda.current_stream().cuda_stream


class DevQMat:
    """A quantized weight uploaded in the repacked device layout."""

    def __init__(self, pkg, dev, qtype, rows, cols, qs, scales, block=32, tiles=None):
        self.qs = to_dev(qs, dev)
        self.scales = to_dev(scales, dev)
        self.tiles = to_dev(tiles, dev) if tiles is not None else None
        flags = 0
        if qtype != pkg.NF4:
            sc = np.ascontiguousarray(scales)
            flags = pkg.lib.cmlb200_scales_have_subnormals(pkg.np_ptr(sc), sc.size // 2)
        self.q = pkg.QMat(qtype, rows, cols, block, self.qs.data_ptr(), self.scales.data_ptr(), flags,
                          self.tiles.data_ptr() if self.tiles is not None else None)

    @classmethod
    def from_gguf(cls, pkg, dev, qtype, blocks, rows, cols):
        qs, sc = pkg.repack_gguf(qtype, blocks, rows, cols)
        tiles = pkg.repack_tiles(qtype, blocks, rows, cols) if cols % 128 == 0 else None
        return cls(pkg, dev, qtype, rows, cols, qs, sc, tiles=tiles)

    @classmethod
    def from_nf4(cls, pkg, dev, packed, scales, rows, cols, block):
        return cls(pkg, dev, pkg.NF4, rows, cols, packed, scales, block)


class DevBlockStream:
    """A Q4_1 / Q4_K / Q5_K / Q6_K weight: the GGUF block stream uploaded unchanged."""

    def __init__(self, pkg, dev, gtype, rows, cols, blocks):
        self.qs = to_dev(blocks, dev)
        self.q = pkg.QMat(gtype, rows, cols, 32 if gtype == 3 else 256, self.qs.data_ptr(), None, 0, None)


def make_block_stream(pkg, synth, ob, orc, dev, rng, gtype, N, K, std=0.02):
    blocks = synth.gguf_blocks(rng, gtype, N, K, std)
    return DevBlockStream(pkg, dev, gtype, N, K, blocks), ob.dequant_blocks(orc, gtype, blocks, N * K).reshape(N, K)


def make_weight(pkg, synth, ob, orc, dev, rng, kind, N, K, block=64):
    """Returns (DevQMat, dequantised fp32 [N,K] from the oracle)."""
    if kind == "nf4":
        packed, scales = synth.nf4_weight(rng, N, K, block)
        Wf = ob.dequant_nf4(orc, packed, scales, block, N * K).reshape(N, K)
        return DevQMat.from_nf4(pkg, dev, packed, scales, N, K, block), Wf
    qtype = pkg.Q8_0 if kind == "q8_0" else pkg.Q4_0
    blocks = (synth.q8_0_blocks if kind == "q8_0" else synth.q4_0_blocks)(rng, N, K)
    Wf = ob.dequant_blocks(orc, qtype, blocks, N * K).reshape(N, K)
    return DevQMat.from_gguf(pkg, dev, qtype, blocks, N, K), Wf


def gemm_status(pkg, reset=True):
    st = C.c_int(-1)
    pkg.check(pkg.lib.cmlb200_gemm_status(C.byref(st), 1 if reset else 0), "cmlb200_gemm_status")
    return st.value
