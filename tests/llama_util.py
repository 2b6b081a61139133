"""Builds a synthetic quantized LLaMA (GGUF file for the device path, dequantised fp32 arrays in
C-ML's [in,out] orientation for the oracle) and drives the oracle's forward pass."""
import ctypes as C

import numpy as np

TINY = dict(vocab=256, hidden=256, inter=512, layers=2, heads=4, kv_heads=2, max_seq=96)


def build(entry, rng, cfg, path, qtype=2, wscale=0.05, metadata=None):
    synth, ob = entry.load_synth(), entry.load_oracle_binding()
    orc = ob.load_orc()

    def quantize(w):
        if qtype not in (2, 7):                            # Q4_1 / K types: random blocks of the same spread (no quantiser for them)
            return synth.gguf_blocks(rng, qtype, w.shape[0], w.shape[1], wscale)
        nb = w.size // 32
        blocks = np.zeros(nb * (18 if qtype == 2 else 34), np.uint8)
        (orc.orc_quantize_q4_0 if qtype == 2 else orc.orc_quantize_q8_0)(ob.p(np.ascontiguousarray(w)), ob.p(blocks), nb)
        return blocks

    tensors, store = synth.make_llama(rng, cfg, quantize, qtype, wscale)
    synth.write_gguf(path, tensors, metadata=metadata)
    return store


class OracleLlama:
    """orc_llama_forward over the dequantised weights of `store`."""

    def __init__(self, entry, cfg, store, qtype=2, rope_all_heads=0, mask_absolute=0):
        self.ob = ob = entry.load_oracle_binding()
        self.orc = ob.load_orc()
        self.cfg = cfg
        L = cfg["layers"]
        kvw = cfg["kv_heads"] * (cfg["hidden"] // cfg["heads"])

        def deq_t(name):
            blocks, out_f, in_f = store[name]
            w = ob.dequant_blocks(self.orc, qtype, blocks, out_f * in_f).reshape(out_f, in_f)
            return np.ascontiguousarray(w.T)               # C-ML keeps projections as [in, out]

        f32 = lambda name: np.ascontiguousarray(store[name].astype(np.float32))
        self.keep = dict(embed=f32("token_embd.weight"), fnorm=f32("output_norm.weight"), head=deq_t("output.weight"))
        names = dict(wq="attn_q", wk="attn_k", wv="attn_v", wo="attn_output", wg="ffn_gate", wu="ffn_up", wd="ffn_down")
        for k, n in names.items():
            self.keep[k] = [deq_t(f"blk.{l}.{n}.weight") for l in range(L)]
        self.keep["n1"] = [f32(f"blk.{l}.attn_norm.weight") for l in range(L)]
        self.keep["n2"] = [f32(f"blk.{l}.ffn_norm.weight") for l in range(L)]
        self.keep["kc"] = np.zeros((L, cfg["max_seq"], kvw), np.float32)
        self.keep["vc"] = np.zeros((L, cfg["max_seq"], kvw), np.float32)
        arrs = {k: ob.ptr_array(self.keep[k]) for k in ("wq", "wk", "wv", "wo", "wg", "wu", "wd", "n1", "n2")}
        self.keep["arrs"] = arrs
        a = lambda x: C.cast(x, C.c_void_p)
        self.m = ob.OrcLlamaStruct(cfg["vocab"], cfg["hidden"], cfg["inter"], L, cfg["heads"], cfg["kv_heads"], cfg["max_seq"],
                                   10000.0, 1e-5, self.keep["embed"].ctypes.data, self.keep["fnorm"].ctypes.data,
                                   self.keep["head"].ctypes.data, a(arrs["wq"]), a(arrs["wk"]), a(arrs["wv"]), a(arrs["wo"]),
                                   a(arrs["wg"]), a(arrs["wu"]), a(arrs["wd"]), a(arrs["n1"]), a(arrs["n2"]),
                                   self.keep["kc"].ctypes.data, self.keep["vc"].ctypes.data, 0, rope_all_heads, mask_absolute)

    def forward(self, tokens):
        tokens = np.ascontiguousarray(tokens, np.int32)
        out = np.empty((len(tokens), self.cfg["vocab"]), np.float32)
        rc = self.orc.orc_llama_forward(C.byref(self.m), self.ob.p(tokens), len(tokens), self.ob.p(out))
        return out if rc == 0 else None


def device_model(pkg, cfg, path, flags=0, max_batch=1, tp=0, rank=0):
    c = pkg.LlamaConfig(cfg["vocab"], cfg["hidden"], cfg["inter"], cfg["layers"], cfg["heads"], cfg["kv_heads"], cfg["max_seq"],
                        10000.0, 1e-5, tp, rank)
    m = pkg.lib.cml_llama_create(C.byref(c))
    assert m
    assert pkg.lib.cml_llama_set_options(m, flags, max_batch) == 0
    assert pkg.lib.cml_llama_load_gguf(m, str(path).encode()) == 0
    return m


def dev_forward(pkg, m, tokens):
    tokens = np.ascontiguousarray(tokens, np.int32)
    t = pkg.lib.cml_llama_forward(m, pkg.np_ptr(tokens), len(tokens))
    return pkg.tensor_to_numpy(t) if t else None
