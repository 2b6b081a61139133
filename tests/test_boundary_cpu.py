"""CPU-side checks of the drop-in boundary: the C-ABI library loads, exports every symbol the
public headers declare, rejects bad arguments without touching a GPU, and the host repack is
a byte-exact bijection."""
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]


def _declared_functions():
    names = []
    for h in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        text = re.sub(r"//[^\n]*", "", text)
        for m in re.finditer(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{}()]*(?:\([^()]*\)[^;{}()]*)*\)\s*;", text):
            name = m.group(1)
            if name not in ("defined", "sizeof", "__attribute__"):
                names.append(name)
    return sorted(set(names))


def test_library_exports_every_declared_symbol(pkg):
    names = _declared_functions()
    assert len(names) >= 25
    missing = [n for n in names if not hasattr(pkg.lib, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


@pytest.mark.parametrize("qtype,bb", [(7, 34), (2, 18)])
def test_repack_is_a_bijection(pkg, synth, qtype, bb):
    rng = np.random.default_rng(5)
    rows, cols = 37, 96                       # ragged row count, three blocks per row
    blocks = (synth.q8_0_blocks if qtype == 7 else synth.q4_0_blocks)(rng, rows, cols)
    qs, sc = pkg.repack_gguf(qtype, blocks, rows, cols)
    assert qs.size == rows * cols * (1 if qtype == 7 else 0.5) and sc.size == rows * (cols // 32) * 2
    back = np.zeros_like(blocks)
    pkg.check(pkg.lib.cmlb200_unrepack_gguf(qtype, pkg.np_ptr(qs), pkg.np_ptr(sc), rows, cols, pkg.np_ptr(back)))
    assert np.array_equal(back, blocks)
    b2 = blocks.reshape(-1, bb)
    assert np.array_equal(sc.reshape(-1, 2), b2[:, :2]) and np.array_equal(qs.reshape(-1, bb - 2), b2[:, 2:])


def test_repack_rejects_bad_arguments(pkg):
    buf = np.zeros(1024, np.uint8)
    p = pkg.np_ptr(buf)
    assert pkg.lib.cmlb200_repack_gguf(7, None, 1, 32, p, p) == -1
    assert pkg.lib.cmlb200_repack_gguf(7, p, 1, 33, p, p) == -1          # cols % 32
    assert pkg.lib.cmlb200_repack_gguf(100, p, 1, 32, p, p) == -1        # NF4 is not a GGUF block type
    assert b"cols" in pkg.last_error() or b"type" in pkg.last_error()
    assert pkg.lib.cmlb200_qs_bytes(2, 4, 64, 32) == 128 and pkg.lib.cmlb200_scale_bytes(2, 4, 64, 32) == 16
    assert pkg.lib.cmlb200_qs_bytes(100, 4, 64, 64) == 128 and pkg.lib.cmlb200_scale_bytes(100, 4, 64, 64) == 16
    assert pkg.lib.cmlb200_qs_bytes(55, 4, 64, 32) == 0


def test_compute_entry_points_validate_before_launching(pkg):
    """Argument checks mirror C-ML's (-1 / NULL on NULL pointers, numel == 0, unknown type,
    numel % block != 0) and run before any CUDA call, so they hold without a GPU."""
    lib = pkg.lib
    fake = 0x1000
    assert lib.cmlb200_gguf_dequantize(7, None, fake, 32, None) == -1
    assert lib.cmlb200_gguf_dequantize(7, fake, fake, 0, None) == -1
    assert lib.cmlb200_gguf_dequantize(12, fake, fake, 256, None) == -1
    assert lib.cmlb200_gguf_dequantize(2, fake, fake, 48, None) == -1
    assert lib.cmlb200_dequantize_nf4(fake, fake, 0, 64, 64, fake, None) == -1
    W = pkg.QMat(pkg.Q4_0, 8, 48, 32, fake, fake)            # cols not a multiple of 32
    assert lib.cmlb200_gemv(W, fake, fake, 1, None) == -1
    W = pkg.QMat(pkg.Q4_0, 8, 64, 32, fake, fake)
    assert lib.cmlb200_gemv(W, fake, fake, 33, None) == -1     # outside the decode range
    assert lib.cmlb200_gemv(W, None, fake, 1, None) == -1
    W = pkg.QMat(pkg.NF4, 8, 64, 48, fake, fake)             # NF4 block must divide cols
    assert lib.cmlb200_gemv(W, fake, fake, 1, None) == -1
    W = pkg.QMat(pkg.Q4_0, 8, 96, 32, fake, fake)            # tensor-core path wants cols % 64 == 0
    assert lib.cmlb200_gemm_bf16(W, fake, fake, 64, None) == -1
    assert lib.cmlb200_gemm_bf16(pkg.QMat(pkg.Q4_0, 8, 128, 32, fake, fake), fake, fake, 0, None) == -1


@pytest.mark.parametrize("qtype", [7, 2])
def test_tile_major_repack_is_a_bijection(pkg, synth, qtype):
    rng = np.random.default_rng(6)
    rows, cols = 200, 256                     # two row tiles, the second partial
    blocks = (synth.q8_0_blocks if qtype == 7 else synth.q4_0_blocks)(rng, rows, cols)
    tiles = pkg.repack_tiles(qtype, blocks, rows, cols)
    unit = 4352 if qtype == 7 else 2304
    assert tiles.size == unit * 2 * (cols // 32)
    back = np.zeros_like(blocks)
    pkg.check(pkg.lib.cmlb200_unrepack_tiles(qtype, pkg.np_ptr(tiles), rows, cols, pkg.np_ptr(back)))
    assert np.array_equal(back, blocks)
    assert pkg.lib.cmlb200_repack_tiles(qtype, pkg.np_ptr(blocks), rows, 48, pkg.np_ptr(tiles)) == -1
    assert pkg.lib.cmlb200_tiles_bytes(100, rows, cols) == 0
