"""Regenerates tests/golden/golden.npz by running the COMPILED C-ML REFERENCE
(oracle/_ref/, built by oracle/Makefile from the C-ML source tree) on small seeded inputs.
Run it only where the C-ML source tree is available:  python tests/golden/make_golden.py
The stored vectors pin the oracle (and through it the CUDA path) on machines that do not
have the reference, e.g. the GPU box."""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402


def main():
    ob = entry.load_oracle_binding()
    ob.build_ref()
    ref = ob.load_ref()
    assert ref is not None, "oracle/_ref/ is not built (needs the C-ML source tree)"
    synth = entry.load_synth()
    p = ob.p
    rng = np.random.default_rng(20240601)
    out = {}

    # --- block dequantisation: random blocks plus every special fp16 scale class
    for name, qtype, bb in (("q8_0", 7, 34), ("q4_0", 2, 18)):
        rows, cols = 8, 256
        blocks = (synth.q8_0_blocks if qtype == 7 else synth.q4_0_blocks)(rng, rows, cols).reshape(-1, bb)
        special = np.array([0x0000, 0x8000, 0x0001, 0x03FF, 0x0400, 0x7BFF, 0x7C00, 0xFC00, 0x3C00, 0xBC00,
                            0x0200, 0x8001, 0x1400, 0x2E66, 0x211F, 0x7E00], np.uint16)
        blocks[:16, :2] = special.view(np.uint8).reshape(16, 2)
        blocks = np.ascontiguousarray(blocks.reshape(-1))
        deq = np.empty(rows * cols, np.float32)
        assert ref.ref_gguf_dequantize(qtype, p(blocks), p(deq), rows * cols) == 0
        out[f"{name}_blocks"] = blocks
        out[f"{name}_dequant_bits"] = deq.view(np.uint32)
        x = rng.standard_normal((3, cols)).astype(np.float32)
        y = np.empty((3, rows), np.float32)
        Wf = deq.reshape(rows, cols).copy()
        Wf[~np.isfinite(Wf)] = 0.0
        assert ref.ref_linear(p(x), p(Wf), 3, rows, cols, p(y)) == 0
        out[f"{name}_x"] = x
        out[f"{name}_linear_y"] = y

    # --- NF4 quantise / dequantise / QLoRA forward
    n_out, n_in, block, rank = 12, 128, 64, 4
    W = (rng.standard_normal((n_out, n_in)) * 0.05).astype(np.float32)
    W[0, :64] = 0.0                      # an all-zero block exercises the 1e-10 absmax floor
    packed = np.zeros(n_out * n_in // 2, np.uint8)
    scales = np.zeros(n_out * n_in // block, np.float32)
    assert ref.ref_nf4_quantize(p(W), W.size, block, p(packed), p(scales)) == len(scales)
    deq = np.empty(W.size, np.float32)
    assert ref.ref_nf4_dequantize(p(packed), p(scales), len(scales), block, W.size, p(deq)) == 0
    x = rng.standard_normal((5, n_in)).astype(np.float32)
    A = (rng.standard_normal((rank, n_in)) * 0.1).astype(np.float32)
    B = (rng.standard_normal((n_out, rank)) * 0.1).astype(np.float32)
    y0 = np.empty((5, n_out), np.float32)
    y1 = np.empty((5, n_out), np.float32)
    assert ref.ref_qlora_forward(p(x), 5, n_in, n_out, p(W), None, None, block, rank, 8.0, p(A), None, p(y0)) == 0
    assert ref.ref_qlora_forward(p(x), 5, n_in, n_out, p(W), None, None, block, rank, 8.0, p(A), p(B), p(y1)) == 0
    out.update(nf4_W=W, nf4_packed=packed, nf4_scales=scales, nf4_dequant_bits=deq.view(np.uint32), nf4_x=x,
               nf4_A=A, nf4_B=B, nf4_y_noB=y0, nf4_y_withB=y1,
               nf4_table_bits=np.array(ref.ref_nf4_table().contents, np.float32).view(np.uint32))
    # odd length: padding nibble and the clamped last block
    odd = (rng.standard_normal(131) * 0.3).astype(np.float32)
    op = np.zeros(66, np.uint8)
    osc = np.zeros(3, np.float32)
    assert ref.ref_nf4_quantize(p(odd), 131, 64, p(op), p(osc)) == 3
    od = np.empty(131, np.float32)
    assert ref.ref_nf4_dequantize(p(op), p(osc), 3, 64, 131, p(od)) == 0
    out.update(nf4_odd_x=odd, nf4_odd_packed=op, nf4_odd_scales=osc, nf4_odd_dequant_bits=od.view(np.uint32))

    # --- RoPE (2-D input, as llama.c passes it) and GQA
    seq, heads, kvh, hd = 5, 4, 2, 16
    q = rng.standard_normal((seq, heads * hd)).astype(np.float32)
    qr = q.copy()
    assert ref.ref_rope_2d(p(qr), seq, heads * hd, hd, 3, 10000.0) == 0
    k = rng.standard_normal((seq + 3, kvh * hd)).astype(np.float32)
    v = rng.standard_normal((seq + 3, kvh * hd)).astype(np.float32)
    att = np.empty((seq, heads * hd), np.float32)
    assert ref.ref_gqa(p(q), p(k), p(v), seq, seq + 3, heads, kvh, hd, p(att)) == 0
    out.update(rope_in=q, rope_out=qr, gqa_k=k, gqa_v=v, gqa_out=att)

    # --- tiny LLaMA: prefill 6 tokens, then 3 single-token steps (reference orientation [in,out])
    cfg = dict(vocab=48, hidden=32, inter=64, layers=2, heads=4, kv_heads=2, max_seq=16)
    hdm = cfg["hidden"] // cfg["heads"]
    qw, kvw = cfg["heads"] * hdm, cfg["kv_heads"] * hdm
    w = lambda *s: (rng.standard_normal(s) * 0.08).astype(np.float32)
    Wt = dict(embed=w(cfg["vocab"], cfg["hidden"]), final_norm=(1 + 0.1 * rng.standard_normal(cfg["hidden"])).astype(np.float32),
              lm_head=w(cfg["hidden"], cfg["vocab"]))
    per = {k2: [] for k2 in ("wq", "wk", "wv", "wo", "wg", "wu", "wd", "n1", "n2")}
    for _ in range(cfg["layers"]):
        per["wq"].append(w(cfg["hidden"], qw)); per["wk"].append(w(cfg["hidden"], kvw)); per["wv"].append(w(cfg["hidden"], kvw))
        per["wo"].append(w(qw, cfg["hidden"])); per["wg"].append(w(cfg["hidden"], cfg["inter"]))
        per["wu"].append(w(cfg["hidden"], cfg["inter"])); per["wd"].append(w(cfg["inter"], cfg["hidden"]))
        per["n1"].append((1 + 0.1 * rng.standard_normal(cfg["hidden"])).astype(np.float32))
        per["n2"].append((1 + 0.1 * rng.standard_normal(cfg["hidden"])).astype(np.float32))
    rc = ob.RefLlamaCfg(cfg["vocab"], cfg["hidden"], cfg["inter"], cfg["layers"], cfg["heads"], cfg["kv_heads"],
                        cfg["max_seq"], 10000.0, 1e-5)
    import ctypes as C
    model = ref.ref_llama_create(C.byref(rc), p(Wt["embed"]), p(Wt["final_norm"]), p(Wt["lm_head"]),
                                 *[ob.ptr_array(per[k2]) for k2 in ("wq", "wk", "wv", "wo", "wg", "wu", "wd", "n1", "n2")])
    assert model
    tokens = rng.integers(0, cfg["vocab"], 9).astype(np.int32)
    logits = [np.empty((6, cfg["vocab"]), np.float32)]
    assert ref.ref_llama_forward(model, p(tokens[:6]), 6, p(logits[0])) == 0
    for i in range(3):
        lg = np.empty((1, cfg["vocab"]), np.float32)
        assert ref.ref_llama_forward(model, p(tokens[6 + i:7 + i]), 1, p(lg)) == 0
        logits.append(lg)
    out["llama_cfg"] = np.array([cfg[k2] for k2 in ("vocab", "hidden", "inter", "layers", "heads", "kv_heads", "max_seq")], np.int32)
    out["llama_tokens"] = tokens
    out["llama_logits"] = np.concatenate(logits, 0)
    out["llama_greedy_last"] = np.array([ref.ref_sample_greedy(p(logits[0]), 6, cfg["vocab"])], np.int32)
    for k2, v2 in Wt.items():
        out[f"llama_{k2}"] = v2
    for k2, v2 in per.items():
        out[f"llama_{k2}"] = np.stack(v2)

    # --- tensor parallel: column-parallel then row-parallel then all-reduce, tp = 1, 2, 4
    M, K, N1, N = 3, 32, 64, 16
    x = rng.standard_normal((M, K)).astype(np.float32)
    W1 = w(N1, K)
    W2 = w(N, N1)
    out.update(tp_x=x, tp_W1=W1, tp_W2=W2)
    for tp in (1, 2, 4):
        y = np.empty((M, N), np.float32)
        assert ref.ref_tp_column_then_row(p(x), M, K, p(W1), N1, p(W2), N, tp, p(y)) == 0
        out[f"tp_y_{tp}"] = y

    # ---- everything below draws from generators of its own, so that adding a section never changes
    # the arrays above.
    # --- the other block types the reference reads (GGUF ids 3, 12, 13, 14): random bytes with sane
    # fp16 scale fields, plus the special fp16 classes in the first blocks
    rng2 = np.random.default_rng(20240602)
    special = np.array([0x0000, 0x8000, 0x0001, 0x03FF, 0x0400, 0x7BFF, 0x3C00, 0xBC00, 0x0200, 0x8001, 0x1400, 0x2E66], np.uint16)
    for gid, bb, bs, half_at in ((3, 20, 32, (0, 2)), (12, 144, 256, (0, 2)), (13, 176, 256, (0, 2)), (14, 210, 256, (208,))):
        nb = 40
        blocks = rng2.integers(0, 256, (nb, bb), dtype=np.uint8)
        for off in half_at:
            h = rng2.uniform(-2e-2, 2e-2, nb).astype(np.float16)
            blocks[:, off:off + 2] = h.view(np.uint8).reshape(nb, 2)
            blocks[:len(special), off:off + 2] = np.roll(special, off).view(np.uint8).reshape(-1, 2)
        blocks = np.ascontiguousarray(blocks.reshape(-1))
        deq = np.empty(nb * bs, np.float32)
        assert ref.ref_gguf_dequantize(gid, p(blocks), p(deq), deq.size) == 0
        out[f"gguf{gid}_blocks"] = blocks
        out[f"gguf{gid}_dequant_bits"] = deq.view(np.uint32)

    # --- the sampling branch of cml_llama_sample_token: (temperature, top_p, top_k, do_sample, seed) -> id
    rng3 = np.random.default_rng(20240603)
    slog = (rng3.standard_normal((2, 200)) * 3).astype(np.float32)
    slog[1, 17] = slog[1, 40] = slog[1].max() + 1.0          # a tie at the top
    cases = [(0.8, 0.9, 40, 1, s) for s in range(12)] + [(1.5, 1.0, 0, 1, s) for s in range(6)] + \
            [(0.3, 0.5, 5, 1, s) for s in range(6)] + [(1.0, 0.0, 3, 1, 7), (0.0, 0.9, 40, 1, 1), (0.8, 0.9, 40, 0, 1), (1.0, 0.95, 1000, 1, 3)]
    ids = [ref.ref_sample_token(p(slog), 2, 200, t, tp_, tk, ds, sd) for (t, tp_, tk, ds, sd) in cases]
    out.update(sample_logits=slog, sample_cases=np.array(cases, np.float64), sample_ids=np.array(ids, np.int32))

    # --- quantized Linear on shapes outside the vectorised kernels: the block sizes and sizes the
    # reference's own tests use (block 16 and 4 on tiny weights) and a block that straddles rows
    rng4 = np.random.default_rng(20240604)
    for tag, (n_out2, n_in2, block2, rank2, M2) in (("b16", (8, 16, 16, 2, 3)), ("b4", (4, 8, 4, 2, 2)), ("straddle", (5, 24, 16, 3, 4))):
        W2 = (rng4.standard_normal((n_out2, n_in2)) * 0.1).astype(np.float32)
        x2 = rng4.standard_normal((M2, n_in2)).astype(np.float32)
        A2 = (rng4.standard_normal((rank2, n_in2)) * 0.1).astype(np.float32)
        B2 = (rng4.standard_normal((n_out2, rank2)) * 0.1).astype(np.float32)
        y2 = np.empty((M2, n_out2), np.float32)
        assert ref.ref_qlora_forward(p(x2), M2, n_in2, n_out2, p(W2), None, None, block2, rank2, 4.0, p(A2), p(B2), p(y2)) == 0
        out.update({f"qlora_{tag}_W": W2, f"qlora_{tag}_x": x2, f"qlora_{tag}_A": A2, f"qlora_{tag}_B": B2, f"qlora_{tag}_y": y2,
                    f"qlora_{tag}_cfg": np.array([n_out2, n_in2, block2, rank2, M2], np.int32)})

    # --- paged KV cache + cml_paged_gqa_forward: (seq_q, kv_len, heads, kv_heads, hd, scale, causal, spoil)
    rng5 = np.random.default_rng(20240605)
    pcases = [(1, 37, 4, 2, 16, 0.0, 1, 20), (5, 21, 4, 4, 8, 0.0, 1, 0), (3, 16, 6, 2, 32, 0.25, 0, 5), (4, 4, 2, 1, 16, 0.0, 1, 0)]
    for i, (sq, kvl, hh, kh, hd2, sc2, cz, spoil) in enumerate(pcases):
        pq = rng5.standard_normal((sq, hh * hd2)).astype(np.float32)
        pk = rng5.standard_normal((kvl, kh * hd2)).astype(np.float32)
        pv = rng5.standard_normal((kvl, kh * hd2)).astype(np.float32)
        po = np.empty((sq, hh * hd2), np.float32)
        nb = ref.ref_paged_gqa(p(pq), p(pk), p(pv), sq, kvl, hh, kh, hd2, sc2, cz, 8, spoil, p(po))
        assert nb == (kvl + 15) // 16, nb
        out.update({f"paged{i}_q": pq, f"paged{i}_k": pk, f"paged{i}_v": pv, f"paged{i}_out": po,
                    f"paged{i}_cfg": np.array([sq, kvl, hh, kh, hd2, cz, spoil], np.int32), f"paged{i}_scale": np.array([sc2], np.float32)})

    # --- cml_speculative_decode_step over table-driven stand-in models (see oracle/ref_driver.c):
    # all drafts accepted, first draft rejected, a miss in the middle, a draft model that gives up
    rng6 = np.random.default_rng(20240606)
    vocab6 = 23
    tgt = rng6.permutation(vocab6).astype(np.int32)
    scases = []
    for name, K6, nmiss, fail in (("all", 5, 0, 0), ("first", 4, 1, 0), ("mid", 6, 1, 0), ("giveup", 5, 0, 9), ("k1", 1, 0, 0), ("k16", 16, 3, 0)):
        drf = tgt.copy()
        prefix6 = rng6.integers(0, vocab6, 7).astype(np.int32)
        # walk the target chain from the prefix's last token and break the draft table along it
        chain = [int(prefix6[-1])]
        for _ in range(K6 + 1):
            chain.append(int(tgt[chain[-1]]))
        if nmiss:
            at = {"first": 0, "mid": 3, "k16": 9}[name]
            drf[chain[at]] = (tgt[chain[at]] + 2) % vocab6
        toks = np.full(K6 + 1, -1, np.int32)
        meta = np.zeros(6, np.int32)
        rates = np.zeros(2, np.float32)
        assert ref.ref_speculative_step(p(drf), p(tgt), vocab6, fail, p(prefix6), len(prefix6), K6, p(toks), p(meta), p(rates)) == 0
        out.update({f"spec_{name}_draft": drf, f"spec_{name}_prefix": prefix6, f"spec_{name}_tokens": toks, f"spec_{name}_meta": meta,
                    f"spec_{name}_rates": rates, f"spec_{name}_cfg": np.array([K6, fail], np.int32)})
        scases.append(name)
    out["spec_target"] = tgt

    # ---- byte-level BPE tokenizer (src/nn/llm_ops.c:1140-1389) ----------------------------------
    # vocabulary: single bytes of a small alphabet (one byte >= 0x80), then spellings made by
    # joining two earlier entries (the merge rules, in that order); a few merged spellings are left
    # out of the vocabulary (-> unknown id), two spellings appear twice (the later id must win).
    trng = np.random.default_rng(77)
    alphabet = [bytes([c]) for c in b"abcde "] + [b"\xc3"]
    vocab = list(alphabet)
    merges = []
    while len(merges) < 40:
        a, b = vocab[trng.integers(len(vocab))], vocab[trng.integers(len(vocab))]
        s = a + b
        if len(s) > 9:
            continue
        merges.append(s)
        if len(merges) % 9 != 0:
            vocab.append(s)                                  # every ninth merged spelling stays unknown
    vocab.append(vocab[3])
    vocab.append(merges[4])                                  # duplicates
    texts = [b"a", b"ab", b"zzz", b"hello world"]
    for n in (2, 3, 5, 17, 64, 200, 400):
        for _ in range(3):
            texts.append(b"".join(alphabet[i] for i in trng.integers(len(alphabet), size=n)))
    texts.append(b"a" * 50)
    texts.append((merges[0] + merges[1]) * 20 + b"z" + merges[2] * 7)
    vblob = b"".join(v + b"\0" for v in vocab)
    mblob = b"".join(m + b"\0" for m in merges)
    ids_all, counts, unks = [], [], []
    for k, txt in enumerate(texts):
        unk = [-1, 2, len(vocab) - 1][k % 3]
        buf = np.zeros(len(txt) + 1, np.int32)
        n = ref.ref_tokenizer_encode(vblob, len(vocab), mblob, len(merges), unk, txt, p(buf), len(buf))
        assert 0 < n <= len(txt)
        ids_all.append(buf[:n].copy()); counts.append(n); unks.append(unk)
    dec_ids = np.concatenate([ids_all[5], np.array([-3, len(vocab) + 5], np.int32), ids_all[9]])      # two ids outside the vocabulary
    dbuf = np.zeros(4096, np.uint8)
    dn = ref.ref_tokenizer_decode(vblob, len(vocab), p(dec_ids), len(dec_ids), p(dbuf), len(dbuf))
    assert dn >= 0
    out.update({"tok_vocab_blob": np.frombuffer(vblob, np.uint8), "tok_vocab_n": np.array([len(vocab)], np.int32),
                "tok_merges_blob": np.frombuffer(mblob, np.uint8), "tok_merges_n": np.array([len(merges)], np.int32),
                "tok_texts_blob": np.frombuffer(b"".join(x + b"\0" for x in texts), np.uint8),
                "tok_ids": np.concatenate(ids_all), "tok_counts": np.array(counts, np.int32), "tok_unk": np.array(unks, np.int32),
                "tok_decode_ids": dec_ids, "tok_decode_text": dbuf[:dn].copy()})

    # ---- LoRA over an fp32 weight (src/nn/lora.c) ------------------------------------------------
    lrng = np.random.default_rng(91)
    Ml, Kl, Nl, rl, alphal, seedl = 5, 96, 40, 4, 8.0, 4242
    lW = lrng.standard_normal((Nl, Kl)).astype(np.float32)
    lx = lrng.standard_normal((Ml, Kl)).astype(np.float32)
    lA = (lrng.standard_normal((rl, Kl)) * 0.2).astype(np.float32)
    lB = (lrng.standard_normal((Nl, rl)) * 0.2).astype(np.float32)
    a_init = np.zeros((rl, Kl), np.float32)
    ly, lwm, lym = np.zeros((Ml, Nl), np.float32), np.zeros((Nl, Kl), np.float32), np.zeros((Ml, Nl), np.float32)
    assert ref.ref_lora(p(lx), Ml, Kl, Nl, p(lW), rl, alphal, seedl, p(lA), p(lB), p(a_init), p(ly), p(lwm), p(lym)) == 0
    out.update({"lora_cfg": np.array([Ml, Kl, Nl, rl, seedl], np.int32), "lora_alpha": np.array([alphal], np.float32), "lora_W": lW,
                "lora_x": lx, "lora_A": lA, "lora_B": lB, "lora_A_init": a_init, "lora_y": ly, "lora_W_merged": lwm, "lora_y_merged": lym})

    # ---- per-tensor int8 / uint8 quantisation (src/core/quantization.c:8-192) -------------------
    qrng = np.random.default_rng(17)
    qx = (qrng.standard_normal(5000) * 3.0).astype(np.float32)
    qx[:8] = [0.0, -0.0, 0.5 * 0.1, 1.5 * 0.1, -2.5 * 0.1, 40.0, -40.0, 12.7]        # ties of round-half-away and values that clamp
    out["q8_x"] = qx
    # values whose quotient leaves the int32 range: C-ML's cast is undefined there; the compiled x86 code
    # yields INT_MIN ("integer indefinite") and wraps the zero-point addition, which the device code reproduces
    qo = np.array([1e9, -1e9, 3e10, -3e10, 2.1e8, -2.1e8, 1.0, np.inf, -np.inf], np.float32)
    out["q8_x_outliers"] = qo
    for name, uns, sc, zp in (("i8_out", 0, 0.1, 3), ("i8_out_neg", 0, 0.1, -5), ("u8_out", 1, 0.05, 128)):
        qq, pr, dq = np.zeros(len(qo), np.uint8), np.zeros(2, np.int32), np.zeros(len(qo), np.float32)
        assert ref.ref_quant8(p(qo), len(qo), uns, 1, sc, zp, p(qq), p(pr), p(dq)) == 0
        out.update({f"q8_{name}_q": qq, f"q8_{name}_cfg": np.array([uns, zp], np.int32), f"q8_{name}_scale": np.array([sc], np.float32)})
    for sym in (0, 1):
        pr = np.zeros(2, np.int32)
        assert ref.ref_quant_params(p(qx), len(qx), sym, p(pr)) == 0
        out[f"q8_params_sym{sym}"] = pr
    for name, uns, use, sc, zp in (("i8_auto", 0, 0, 0.0, 0), ("u8_auto", 1, 0, 0.0, 0), ("i8_given", 0, 1, 0.1, 3), ("u8_given", 1, 1, 0.05, 128)):
        qq, pr, dq = np.zeros(len(qx), np.uint8), np.zeros(2, np.int32), np.zeros(len(qx), np.float32)
        assert ref.ref_quant8(p(qx), len(qx), uns, use, sc, zp, p(qq), p(pr), p(dq)) == 0
        out.update({f"q8_{name}_q": qq, f"q8_{name}_params": pr, f"q8_{name}_deq": dq})

    # ---- GGUF writer (src/core/gguf.c:181-232, 312-340): the bytes of a three-tensor file ----------
    import tempfile
    wr = np.random.default_rng(33)
    wa = wr.standard_normal((3, 5)).astype(np.float32)
    wb = wr.integers(-1000, 1000, 7).astype(np.int32)
    wc = wr.standard_normal(9).astype(np.float16).view(np.uint16)
    with tempfile.TemporaryDirectory() as td:
        fp = str(Path(td) / "ref.gguf")
        assert ref.ref_gguf_write(fp.encode(), p(wa), 3, 5, p(wb), len(wb), p(wc), len(wc)) == 0
        out.update({"ggufw_a": wa, "ggufw_b": wb, "ggufw_c": wc, "ggufw_file": np.frombuffer(Path(fp).read_bytes(), np.uint8)})

    np.savez_compressed(ROOT / "tests" / "golden" / "golden.npz", **out)
    print("wrote golden.npz with", len(out), "arrays,", sum(v.nbytes for v in out.values()), "bytes")


if __name__ == "__main__":
    main()
