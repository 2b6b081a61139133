"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs
(numpy only; shared by tests/ and bench.py). Nothing here computes results."""
import numpy as np


def q8_0_blocks(rng, rows, cols, d_lo=1e-3, d_hi=1e-2):
    """GGUF Q8_0 blocks, file order: int8 uniform in [-127,127], fp16 d uniform in [d_lo,d_hi]."""
    nb = rows * cols // 32
    blk = np.empty((nb, 34), np.uint8)
    blk[:, :2] = rng.uniform(d_lo, d_hi, nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    blk[:, 2:] = rng.integers(-127, 128, (nb, 32), dtype=np.int8).view(np.uint8)
    return blk.reshape(-1)


def q4_0_blocks(rng, rows, cols, d_lo=1e-3, d_hi=2e-2):
    """GGUF Q4_0 blocks: nibbles uniform 0..15, fp16 d uniform in [d_lo,d_hi]."""
    nb = rows * cols // 32
    blk = np.empty((nb, 18), np.uint8)
    blk[:, :2] = rng.uniform(d_lo, d_hi, nb).astype(np.float16).view(np.uint8).reshape(nb, 2)
    blk[:, 2:] = rng.integers(0, 256, (nb, 16), dtype=np.uint8)
    return blk.reshape(-1)


def nf4_weight(rng, rows, cols, block=64, s_lo=0.01, s_hi=0.1):
    """NF4 packed bytes (indices uniform 0..15) and fp32 absmax per block of the flat index."""
    packed = rng.integers(0, 256, rows * cols // 2, dtype=np.uint8)
    scales = rng.uniform(s_lo, s_hi, rows * cols // block).astype(np.float32)
    return packed, scales


def bf16_round(a):
    """fp32 -> nearest-even bf16, returned both as uint16 bit patterns and as fp32 values."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r, (r.astype(np.uint32) << 16).view(np.float32)


def bf16_to_f32(u16):
    return (np.ascontiguousarray(u16, np.uint16).astype(np.uint32) << 16).view(np.float32)
