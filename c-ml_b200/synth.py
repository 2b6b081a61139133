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


GGUF_BLOCK = {2: (32, 18), 3: (32, 20), 7: (32, 34), 12: (256, 144), 13: (256, 176), 14: (256, 210)}   # type -> (elements, bytes)


def gguf_blocks(rng, gtype, rows, cols, std=0.02):
    """Random GGUF blocks of type Q4_1 (3), Q4_K (12), Q5_K (13) or Q6_K (14) in C-ML's layouts
    (src/core/gguf_quant.c:90-311) whose dequantised weights have mean about 0 and roughly `std`:
    uniform quants, small integer sub-block scales, fp16 d / dmin / m chosen to centre the values."""
    if gtype == 2: return q4_0_blocks(rng, rows, cols, std / 6, std / 3)
    if gtype == 7: return q8_0_blocks(rng, rows, cols, std / 100, std / 50)
    be, bb = GGUF_BLOCK[gtype]
    nb = rows * cols // be
    blk = rng.integers(0, 256, (nb, bb), dtype=np.uint8)
    f16 = lambda a: np.asarray(a, np.float16).view(np.uint8).reshape(nb, 2)
    if gtype == 3:                                   # w = q * d + m, q uniform 0..15
        d = rng.uniform(0.5, 1.0, nb) * std / 4.6
        blk[:, 0:2] = f16(d)
        blk[:, 2:4] = f16(-7.5 * d * rng.uniform(0.9, 1.1, nb))
    elif gtype in (12, 13):                          # w = q * (d * sc) - dmin * mn, q uniform 0..15 (0..31)
        qmax = 15 if gtype == 12 else 31
        sc = rng.integers(2, 8 if gtype == 12 else 4, (nb, 8))
        mn = np.clip(np.rint(qmax / 2 * sc + rng.integers(-2, 3, (nb, 8))), 0, 63).astype(np.int64)
        s = np.zeros((nb, 12), np.int64)             # get_scale_min_k4's packing
        s[:, 0:4] = sc[:, 0:4] | ((sc[:, 4:8] >> 4) << 6)
        s[:, 4:8] = mn[:, 0:4] | ((mn[:, 4:8] >> 4) << 6)
        s[:, 8:12] = (sc[:, 4:8] & 15) | ((mn[:, 4:8] & 15) << 4)
        d = rng.uniform(0.5, 1.0, nb) * std / (5.0 * (qmax + 1) / 3.46)
        blk[:, 0:2] = f16(d)
        blk[:, 2:4] = f16(d)
        blk[:, 4:16] = s.astype(np.uint8)
    else:                                            # w = d * scale8 * (q - 32), q uniform 0..63
        blk[:, 192:208] = rng.integers(-24, 25, (nb, 16)).astype(np.int8).view(np.uint8)
        blk[:, 208:210] = f16(rng.uniform(0.5, 1.0, nb) * std / (14.0 * 18.5))
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


# ---- GGUF v3 writer for synthetic models (little-endian; tensor data 32-byte aligned) ------------
_GGUF_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<B", 10: "<Q", 11: "<q", 12: "<d"}


def _gguf_value(vtype, value):
    """One GGUF metadata value: scalars by type id, 8 = string (bytes or str), 9 = (elem_type, items)."""
    import struct
    if vtype == 8:
        raw = value.encode() if isinstance(value, str) else bytes(value)
        return struct.pack("<Q", len(raw)) + raw
    if vtype == 9:
        et, items = value
        return struct.pack("<IQ", et, len(items)) + b"".join(_gguf_value(et, v) for v in items)
    return struct.pack(_GGUF_SCALAR[vtype], value)


def write_gguf(path, tensors, metadata=None):
    """tensors: list of (name, dims, gguf_type, raw_bytes). dims are written in the given order
    (for weights: (in_features, out_features), the GGUF convention). metadata: list of
    (key, value_type, value) written after general.architecture = "llama"."""
    import struct
    infos, blobs, off = [], [], 0
    for name, dims, gtype, raw in tensors:
        raw = bytes(raw)
        infos.append((name.encode(), dims, gtype, off))
        pad = (-len(raw)) % 32
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    out = bytearray()
    metadata = list(metadata or [])
    out += struct.pack("<IIQQ", 0x46475547, 3, len(tensors), 1 + len(metadata))
    key = b"general.architecture"
    out += struct.pack("<Q", len(key)) + key + struct.pack("<I", 8) + struct.pack("<Q", 5) + b"llama"
    for k, vtype, value in metadata:
        k = k.encode() if isinstance(k, str) else bytes(k)
        out += struct.pack("<Q", len(k)) + k + struct.pack("<I", vtype) + _gguf_value(vtype, value)
    for name, dims, gtype, o in infos:
        out += struct.pack("<Q", len(name)) + name + struct.pack("<I", len(dims))
        for d in dims:
            out += struct.pack("<Q", d)
        out += struct.pack("<IQ", gtype, o)
    out += b"\0" * ((-len(out)) % 32)
    with open(path, "wb") as f:
        f.write(out)
        for b in blobs:
            f.write(b)


def make_llama(rng, cfg, quantize, qtype=2, wscale=0.05):
    """Random LLaMA weights quantized with `quantize(fp32 [out,in]) -> GGUF block bytes`.
    Returns (gguf tensor list, dict of quantized block arrays + fp16 vectors)."""
    V, H, I, L = cfg["vocab"], cfg["hidden"], cfg["inter"], cfg["layers"]
    hd = H // cfg["heads"]
    QW, KVW = cfg["heads"] * hd, cfg["kv_heads"] * hd
    tensors, store = [], {}

    def proj(name, out_f, in_f):
        w = (rng.standard_normal((out_f, in_f)) * wscale).astype(np.float32)
        blocks = quantize(w)
        store[name] = (blocks, out_f, in_f)
        tensors.append((name, (in_f, out_f), qtype, blocks.tobytes()))

    def vec(name, n, base=1.0, rows=None):
        shape = (rows, n) if rows else (n,)
        v = (base + 0.1 * rng.standard_normal(shape)).astype(np.float16) if base else (rng.standard_normal(shape) * 0.5).astype(np.float16)
        store[name] = v
        tensors.append((name, tuple(reversed(shape)), 1, v.tobytes()))

    vec("token_embd.weight", H, base=0.0, rows=V)
    for l in range(L):
        vec(f"blk.{l}.attn_norm.weight", H)
        proj(f"blk.{l}.attn_q.weight", QW, H)
        proj(f"blk.{l}.attn_k.weight", KVW, H)
        proj(f"blk.{l}.attn_v.weight", KVW, H)
        proj(f"blk.{l}.attn_output.weight", H, QW)
        vec(f"blk.{l}.ffn_norm.weight", H)
        proj(f"blk.{l}.ffn_gate.weight", I, H)
        proj(f"blk.{l}.ffn_up.weight", I, H)
        proj(f"blk.{l}.ffn_down.weight", H, I)
    vec("output_norm.weight", H)
    proj("output.weight", V, H)
    return tensors, store


def write_random_llama_gguf(path, rng, cfg, qtype=2, weight_std=0.02, alias_layers=False):
    """A LLaMA-shaped GGUF with random Q4_0/Q8_0 blocks (uniform quants, fp16 scales chosen so
    that the dequantised weights have roughly `weight_std`), fp16 norms near 1 and fp16
    embeddings. Generated tensor by tensor straight into the file, so 7B-sized models need no
    fp32 staging; every layer reuses the random bytes drawn for layer 0. By default the file
    still holds each layer separately; with alias_layers the tensor infos of layers 1.. point at
    layer 0's data (GGUF addresses tensors by offset, so this is a valid file of a fraction of
    the size; the loader still uploads every layer as its own device copy). Returns the number
    of bytes written."""
    import struct
    V, H, I, L = cfg["vocab"], cfg["hidden"], cfg["inter"], cfg["layers"]
    hd = H // cfg["heads"]
    QW, KVW = cfg["heads"] * hd, cfg["kv_heads"] * hd
    bb, qstd = (18, 4.6) if qtype == 2 else (34, 73.0)
    d0 = weight_std / qstd
    spec = [("token_embd.weight", (H, V), 1)]
    for l in range(L):
        spec += [(f"blk.{l}.attn_norm.weight", (H,), 1), (f"blk.{l}.attn_q.weight", (H, QW), qtype),
                 (f"blk.{l}.attn_k.weight", (H, KVW), qtype), (f"blk.{l}.attn_v.weight", (H, KVW), qtype),
                 (f"blk.{l}.attn_output.weight", (QW, H), qtype), (f"blk.{l}.ffn_norm.weight", (H,), 1),
                 (f"blk.{l}.ffn_gate.weight", (H, I), qtype), (f"blk.{l}.ffn_up.weight", (H, I), qtype),
                 (f"blk.{l}.ffn_down.weight", (I, H), qtype)]
    spec += [("output_norm.weight", (H,), 1), ("output.weight", (H, V), qtype)]

    def nbytes(dims, t):
        n = int(np.prod(dims))
        return n * 2 if t == 1 else n // 32 * bb

    def kind_of(name, dims, t):
        return (name.split(".", 2)[2] if name.startswith("blk.") else name, dims, t)

    head = bytearray(struct.pack("<IIQQ", 0x46475547, 3, len(spec), 0))
    off = 0
    placed = {}         # alias_layers: data offset of the first tensor of each kind
    stored = []         # the tensors whose bytes go into the file, in order
    for name, dims, t in spec:
        nb = name.encode()
        head += struct.pack("<Q", len(nb)) + nb + struct.pack("<I", len(dims))
        for d in dims:
            head += struct.pack("<Q", d)
        kind = kind_of(name, dims, t)
        if alias_layers and kind in placed:
            head += struct.pack("<IQ", t, placed[kind])
            continue
        placed[kind] = off
        stored.append((name, dims, t))
        head += struct.pack("<IQ", t, off)
        off += (nbytes(dims, t) + 31) // 32 * 32
    head += b"\0" * ((-len(head)) % 32)
    cache = {}          # layers share their random bytes: one draw per (tensor kind, shape)
    with open(path, "wb") as f:
        f.write(head)
        for name, dims, t in stored:
            n = int(np.prod(dims))
            kind = kind_of(name, dims, t)
            if kind in cache:
                raw = cache[kind]
            elif t == 1:
                if len(dims) == 1:
                    raw = (1.0 + 0.05 * rng.standard_normal(n)).astype(np.float16).tobytes()
                else:
                    raw = (0.5 * rng.standard_normal(n, dtype=np.float32)).astype(np.float16).tobytes()
            else:
                nblk = n // 32
                blk = np.empty((nblk, bb), np.uint8)
                blk[:, :2] = rng.uniform(0.5 * d0, 1.5 * d0, nblk).astype(np.float16).view(np.uint8).reshape(nblk, 2)
                blk[:, 2:] = rng.integers(0, 256, (nblk, bb - 2), dtype=np.uint8)
                raw = blk.tobytes()
            cache[kind] = raw
            f.write(raw)
            f.write(b"\0" * ((-len(raw)) % 32))
    return len(head) + off
