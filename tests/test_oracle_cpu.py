"""The oracle (oracle/cml_oracle.c) pinned against (a) stored outputs of the compiled C-ML
reference (tests/golden/golden.npz), (b) the compiled reference itself where oracle/_ref/ is
present, (c) the single-block known answers of C-ML's tests/test_gguf_quant.c."""
import ctypes as C

import numpy as np
import pytest

from conftest import rel_err_inf


def _dq(ob, orc, qtype, blocks, numel):
    return ob.dequant_blocks(orc, qtype, np.ascontiguousarray(blocks), numel)


@pytest.mark.parametrize("name,qtype", [("q8_0", 7), ("q4_0", 2)])
def test_block_dequant_matches_golden_bits(ob, orc, golden, name, qtype):
    blocks = golden[f"{name}_blocks"]
    got = _dq(ob, orc, qtype, blocks, 8 * 256)
    assert np.array_equal(got.view(np.uint32), golden[f"{name}_dequant_bits"])


def test_known_answer_q8_0_all_ones(ob, orc):
    # C-ML tests/test_gguf_quant.c:71-95: d = 1.0, every quant 1 -> 1.0
    blk = np.zeros(34, np.uint8)
    blk[:2] = np.array([0x3C00], np.uint16).view(np.uint8)
    blk[2:] = 1
    assert np.all(_dq(ob, orc, 7, blk, 32) == 1.0)


def test_known_answer_q4_0_nibbles(ob, orc):
    # C-ML tests/test_gguf_quant.c:97-140: nibbles 0x88 -> 0, 0x99 with d = 2.0 -> 2.0
    blk = np.zeros(18, np.uint8)
    blk[:2] = np.array([0x3C00], np.uint16).view(np.uint8)
    blk[2:] = 0x88
    assert np.all(_dq(ob, orc, 2, blk, 32) == 0.0)
    blk[:2] = np.array([0x4000], np.uint16).view(np.uint8)
    blk[2:] = 0x99
    assert np.all(_dq(ob, orc, 2, blk, 32) == 2.0)


def test_dequantize_error_contract(ob, orc):
    # src/core/gguf_quant.c:351-363: NULL, numel == 0, unknown type, numel % 32 != 0 -> -1
    buf = np.zeros(64, np.uint8)
    out = np.zeros(64, np.float32)
    assert orc.orc_gguf_dequantize(7, None, ob.p(out), 32) == -1
    assert orc.orc_gguf_dequantize(7, ob.p(buf), None, 32) == -1
    assert orc.orc_gguf_dequantize(7, ob.p(buf), ob.p(out), 0) == -1
    assert orc.orc_gguf_dequantize(99, ob.p(buf), ob.p(out), 32) == -1
    assert orc.orc_gguf_dequantize(2, ob.p(buf), ob.p(out), 33) == -1


def test_fp16_widening_all_patterns(orc):
    """C-ML's fp16_to_fp32 (src/core/gguf_quant.c:14-58) is IEEE-exact for normals, zeros,
    infinities and NaNs, but its subnormal branch counts one shift too many (:35-36), so a
    subnormal half widens to HALF its IEEE value. Parity means reproducing that."""
    h = np.arange(65536, dtype=np.uint16)
    ieee = h.view(np.float16).astype(np.float32)
    sub = ((h & 0x7C00) == 0) & ((h & 0x03FF) != 0)
    want = np.where(sub, ieee * np.float32(0.5), ieee).astype(np.float32).view(np.uint32)
    got = np.array([orc.orc_fp16_to_fp32(int(v)) for v in h[::7]], np.float32).view(np.uint32)
    nan = np.isnan(h[::7].view(np.float16))
    assert np.array_equal(got[~nan], want[::7][~nan])
    assert np.all(np.isnan(got.view(np.float32)[nan]))


def test_fp16_rounding_round_trip(orc):
    rng = np.random.default_rng(3)
    x = np.concatenate([rng.uniform(-70000, 70000, 2000), rng.uniform(-1e-4, 1e-4, 2000), [0.0, 65504.0, 65520.0, 6e-8, 2.98e-8]]).astype(np.float32)
    got = np.array([orc.orc_fp32_to_fp16(float(v)) for v in x], np.uint16)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, want)


def test_nf4_quantize_dequantize_golden(ob, orc, golden):
    W = golden["nf4_W"]
    packed = np.zeros(W.size // 2, np.uint8)
    scales = np.zeros(W.size // 64, np.float32)
    assert orc.orc_nf4_quantize(ob.p(W), W.size, 64, ob.p(packed), ob.p(scales)) == len(scales)
    assert np.array_equal(packed, golden["nf4_packed"])
    assert np.array_equal(scales.view(np.uint32), golden["nf4_scales"].view(np.uint32))
    assert scales[0] == np.float32(1e-10)          # all-zero block: absmax floor (quantization.c:266)
    deq = ob.dequant_nf4(orc, packed, scales, 64, W.size)
    assert np.array_equal(deq.view(np.uint32), golden["nf4_dequant_bits"])


def test_nf4_odd_length_golden(ob, orc, golden):
    x = golden["nf4_odd_x"]
    packed = np.zeros(66, np.uint8)
    scales = np.zeros(3, np.float32)
    assert orc.orc_nf4_quantize(ob.p(x), 131, 64, ob.p(packed), ob.p(scales)) == 3
    assert np.array_equal(packed, golden["nf4_odd_packed"])
    deq = ob.dequant_nf4(orc, packed, scales, 64, 131)
    assert np.array_equal(deq.view(np.uint32), golden["nf4_odd_dequant_bits"])


def test_nf4_table_properties(ob, golden):
    # C-ML tests/test_qlora.c:109-150: monotone, ends at -1 / +1, entry 7 is zero
    t = (C.c_float * 16).in_dll(C.CDLL(str(ob.HERE / "libcml_oracle.so")), "ORC_NF4_TABLE")
    t = np.array(t, np.float32)
    assert np.array_equal(t.view(np.uint32), golden["nf4_table_bits"])
    assert np.all(np.diff(t) > 0) and t[0] == -1.0 and t[15] == 1.0 and t[7] == 0.0


def test_nf4_round_trip_error_bounds(ob, orc):
    # C-ML tests/test_qlora.c:26-106: max error < 0.15, rmse < 0.08 on a 128-element ramp
    x = np.linspace(-1, 1, 128).astype(np.float32)
    packed = np.zeros(64, np.uint8)
    scales = np.zeros(2, np.float32)
    orc.orc_nf4_quantize(ob.p(x), 128, 64, ob.p(packed), ob.p(scales))
    d = ob.dequant_nf4(orc, packed, scales, 64, 128)
    assert np.abs(d - x).max() < 0.15 and np.sqrt(np.mean((d - x) ** 2)) < 0.08


@pytest.mark.parametrize("name,qtype", [("q8_0", 7), ("q4_0", 2)])
def test_linear_matches_golden(ob, orc, golden, name, qtype):
    W = golden[f"{name}_dequant_bits"].view(np.float32).reshape(8, 256).copy()
    W[~np.isfinite(W)] = 0.0
    y = ob.linear_nt(orc, golden[f"{name}_x"], W)
    assert rel_err_inf(y, golden[f"{name}_linear_y"]) < 1e-5


def test_qlora_forward_matches_golden(ob, orc, golden):
    x, A, B = golden["nf4_x"], golden["nf4_A"], golden["nf4_B"]
    packed, scales = golden["nf4_packed"], golden["nf4_scales"]
    for Bm, want in ((None, golden["nf4_y_noB"]), (B, golden["nf4_y_withB"])):
        y = np.empty((5, 12), np.float32)
        Bz = np.zeros_like(B) if Bm is None else Bm
        assert orc.orc_qlora_forward(ob.p(x), 5, 128, 12, ob.p(packed), ob.p(scales), len(scales), 64,
                                     ob.p(A), ob.p(Bz), 4, 2.0, ob.p(y)) == 0
        assert rel_err_inf(y, want) < 1e-5
    assert not np.allclose(golden["nf4_y_noB"], golden["nf4_y_withB"])   # tests/test_qlora.c:435-518


def test_rope_matches_golden_and_quirk(ob, orc, golden):
    x = golden["rope_in"].copy()
    orc.orc_rope(ob.p(x), 5, 64, 16, 3, 10000.0, 0)
    assert np.abs(x - golden["rope_out"]).max() < 1e-5
    assert np.array_equal(x[:, 16:], golden["rope_in"][:, 16:])      # heads 1.. are left unrotated
    y = golden["rope_in"].copy()
    orc.orc_rope(ob.p(y), 5, 64, 16, 3, 10000.0, 1)
    assert not np.allclose(y[:, 16:], golden["rope_in"][:, 16:])


def test_gqa_matches_golden(ob, orc, golden):
    q, k, v = golden["rope_in"], golden["gqa_k"], golden["gqa_v"]
    out = np.empty((5, 64), np.float32)
    assert orc.orc_gqa(ob.p(q), ob.p(k), ob.p(v), 5, 8, 4, 2, 16, 0, ob.p(out)) == 0
    assert np.abs(out - golden["gqa_out"]).max() < 1e-5
    assert orc.orc_gqa(ob.p(q), ob.p(k), ob.p(v), 5, 8, 3, 2, 16, 0, ob.p(out)) == -1   # heads % kv_heads


def _orc_llama(ob, golden, **flags):
    cfg = [int(v) for v in golden["llama_cfg"]]
    layers, hidden, max_seq, kvh, heads = cfg[3], cfg[1], cfg[6], cfg[5], cfg[4]
    kvw = kvh * (hidden // heads)
    keep = {k: [np.ascontiguousarray(a) for a in golden[f"llama_{k}"]] for k in ("wq", "wk", "wv", "wo", "wg", "wu", "wd", "n1", "n2")}
    keep["embed"] = np.ascontiguousarray(golden["llama_embed"])
    keep["final_norm"] = np.ascontiguousarray(golden["llama_final_norm"])
    keep["lm_head"] = np.ascontiguousarray(golden["llama_lm_head"])
    keep["kc"] = np.zeros((layers, max_seq, kvw), np.float32)
    keep["vc"] = np.zeros((layers, max_seq, kvw), np.float32)
    arrs = {k: ob.ptr_array(keep[k]) for k in ("wq", "wk", "wv", "wo", "wg", "wu", "wd", "n1", "n2")}
    keep["arrs"] = arrs
    addr = lambda a: C.cast(a, C.c_void_p)
    m = ob.OrcLlamaStruct(*cfg, 10000.0, 1e-5, keep["embed"].ctypes.data, keep["final_norm"].ctypes.data,
                          keep["lm_head"].ctypes.data, addr(arrs["wq"]), addr(arrs["wk"]), addr(arrs["wv"]),
                          addr(arrs["wo"]), addr(arrs["wg"]), addr(arrs["wu"]), addr(arrs["wd"]), addr(arrs["n1"]),
                          addr(arrs["n2"]), keep["kc"].ctypes.data, keep["vc"].ctypes.data, 0,
                          flags.get("rope_all_heads", 0), flags.get("mask_absolute", 0))
    return m, keep, cfg


def test_llama_forward_matches_golden(ob, orc, golden):
    m, keep, cfg = _orc_llama(ob, golden)
    tokens = golden["llama_tokens"]
    vocab = cfg[0]
    got = [np.empty((6, vocab), np.float32)]
    assert orc.orc_llama_forward(C.byref(m), ob.p(tokens[:6]), 6, ob.p(got[0])) == 0
    for i in range(3):
        lg = np.empty((1, vocab), np.float32)
        assert orc.orc_llama_forward(C.byref(m), ob.p(tokens[6 + i:7 + i]), 1, ob.p(lg)) == 0
        got.append(lg)
    got = np.concatenate(got, 0)
    assert m.cur_len == 9
    assert rel_err_inf(got, golden["llama_logits"]) < 2e-5
    assert orc.orc_argmax_first(ob.p(np.ascontiguousarray(got[5])), vocab) == int(golden["llama_greedy_last"][0])
    # cache overflow -> -1 (src/nn/llm_ops.c:133-137)
    big = np.zeros(8, np.int32)
    assert orc.orc_llama_forward(C.byref(m), ob.p(big), 8, ob.p(np.empty((8, vocab), np.float32))) == -1


def test_llama_position_correct_mode_differs_in_decode_only(ob, orc, golden):
    # With the reference's relative-index mask a cached decode step attends to slot 0 only;
    # the position-correct mode must agree on prefill-from-zero and differ afterwards.
    tokens = golden["llama_tokens"]
    vocab = int(golden["llama_cfg"][0])
    a, keep_a, _ = _orc_llama(ob, golden)
    b, keep_b, _ = _orc_llama(ob, golden, mask_absolute=1)
    la, lb = np.empty((6, vocab), np.float32), np.empty((6, vocab), np.float32)
    orc.orc_llama_forward(C.byref(a), ob.p(tokens[:6]), 6, ob.p(la))
    orc.orc_llama_forward(C.byref(b), ob.p(tokens[:6]), 6, ob.p(lb))
    assert np.array_equal(la, lb)
    la1, lb1 = np.empty((1, vocab), np.float32), np.empty((1, vocab), np.float32)
    orc.orc_llama_forward(C.byref(a), ob.p(tokens[6:7]), 1, ob.p(la1))
    orc.orc_llama_forward(C.byref(b), ob.p(tokens[6:7]), 1, ob.p(lb1))
    assert not np.allclose(la1, lb1)


@pytest.mark.parametrize("tp", [1, 2, 4])
def test_tensor_parallel_matches_golden(ob, orc, golden, tp):
    x, W1, W2 = golden["tp_x"], golden["tp_W1"], golden["tp_W2"]
    M, K = x.shape
    N1, N = W1.shape[0], W2.shape[0]
    parts = []
    for r in range(tp):
        w1 = np.empty((N1 // tp, K), np.float32)
        w2 = np.empty((N, N1 // tp), np.float32)
        assert orc.orc_tp_shard(ob.p(W1), N1, K, 0, tp, r, ob.p(w1)) == 0
        assert orc.orc_tp_shard(ob.p(W2), N, N1, 1, tp, r, ob.p(w2)) == 0
        parts.append(ob.linear_nt(orc, ob.linear_nt(orc, x, w1), w2))
    y = np.empty((M, N), np.float32)
    orc.orc_tp_allreduce_sum(ob.ptr_array(parts), tp, M * N, ob.p(y))
    assert rel_err_inf(y, golden[f"tp_y_{tp}"]) < 1e-5
    assert orc.orc_tp_shard(ob.p(W1), N1, K, 0, 3, 0, ob.p(np.empty(1, np.float32))) == -1   # uneven split


# ---- against the compiled reference itself, where it exists -----------------------------------
def test_oracle_equals_compiled_reference_on_fresh_inputs(ob, orc, ref, synth):
    if ref is None:
        pytest.skip("oracle/_ref/ not built on this machine (the stored golden vectors cover it)")
    rng = np.random.default_rng(99)
    for qtype, gen, bb in ((7, synth.q8_0_blocks, 34), (2, synth.q4_0_blocks, 18)):
        blocks = gen(rng, 64, 512).reshape(-1, bb)
        blocks[:, :2] = rng.integers(0, 65536, len(blocks), dtype=np.uint16).view(np.uint8).reshape(-1, 2)  # any fp16 pattern
        blocks = np.ascontiguousarray(blocks.reshape(-1))
        a = ob.dequant_blocks(orc, qtype, blocks, 64 * 512)
        b = np.empty_like(a)
        assert ref.ref_gguf_dequantize(qtype, ob.p(blocks), ob.p(b), a.size) == 0
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
        assert ref.ref_gguf_quant_block_size(qtype) == 32 and ref.ref_gguf_quant_type_size(qtype) == bb
    x = (rng.standard_normal(64 * 300 + 5) * 0.2).astype(np.float32)
    n = x.size
    pa, pb = np.zeros((n + 1) // 2, np.uint8), np.zeros((n + 1) // 2, np.uint8)
    sa, sb = np.zeros((n + 63) // 64, np.float32), np.zeros((n + 63) // 64, np.float32)
    assert orc.orc_nf4_quantize(ob.p(x), n, 64, ob.p(pa), ob.p(sa)) == ref.ref_nf4_quantize(ob.p(x), n, 64, ob.p(pb), ob.p(sb))
    assert np.array_equal(pa, pb) and np.array_equal(sa, sb)
    da, db = ob.dequant_nf4(orc, pa, sa, 64, n), np.empty(n, np.float32)
    assert ref.ref_nf4_dequantize(ob.p(pa), ob.p(sa), len(sa), 64, n, ob.p(db)) == 0
    assert np.array_equal(da.view(np.uint32), db.view(np.uint32))


@pytest.mark.parametrize("gid,bs,bb", [(3, 32, 20), (12, 256, 144), (13, 256, 176), (14, 256, 210)])
def test_other_block_types_match_golden_bits(ob, orc, ref, golden, gid, bs, bb):
    """Q4_1, Q4_K, Q5_K, Q6_K (C-ML src/core/gguf_quant.c:90-311, its own nibble order for the K
    types) against stored outputs of the compiled reference, and against it directly when built."""
    blocks = np.ascontiguousarray(golden[f"gguf{gid}_blocks"])
    numel = blocks.size // bb * bs
    got = _dq(ob, orc, gid, blocks, numel)
    assert np.array_equal(got.view(np.uint32), golden[f"gguf{gid}_dequant_bits"])
    out = np.zeros(numel, np.float32)
    assert orc.orc_gguf_dequantize(gid, ob.p(blocks), ob.p(out), bs // 2) == -1          # not a whole block
    if ref is not None:
        rng = np.random.default_rng(gid)
        fresh = rng.integers(0, 256, 64 * bb, dtype=np.uint8)
        a, b = _dq(ob, orc, gid, fresh, 64 * bs), np.empty(64 * bs, np.float32)
        assert ref.ref_gguf_dequantize(gid, ob.p(fresh), ob.p(b), b.size) == 0
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))                     # any bytes, NaN scales included
        assert ref.ref_gguf_quant_block_size(gid) == bs and ref.ref_gguf_quant_type_size(gid) == bb


@pytest.mark.parametrize("tag", ["b16", "b4", "straddle"])
def test_qlora_small_block_shapes_match_golden(ob, orc, golden, tag):
    """The quantized Linear at the block sizes C-ML's own tests use (tests/test_qlora.c:174,332,453:
    16 and 4) and with a block that straddles two weight rows."""
    n_out, n_in, block, rank, M = (int(v) for v in golden[f"qlora_{tag}_cfg"])
    W, x, A, B = (np.ascontiguousarray(golden[f"qlora_{tag}_{k}"]) for k in ("W", "x", "A", "B"))
    ns = (W.size + block - 1) // block
    packed, scales = np.zeros((W.size + 1) // 2, np.uint8), np.zeros(ns, np.float32)
    assert orc.orc_nf4_quantize(ob.p(W), W.size, block, ob.p(packed), ob.p(scales)) == ns
    y = np.empty((M, n_out), np.float32)
    assert orc.orc_qlora_forward(ob.p(x), M, n_in, n_out, ob.p(packed), ob.p(scales), ns, block, ob.p(A), ob.p(B), rank, 4.0 / rank, ob.p(y)) == 0
    assert rel_err_inf(y, golden[f"qlora_{tag}_y"]) < 1e-5


def test_paged_attention_matches_golden_and_reference(ob, orc, golden):
    """cml_paged_gqa_forward: causal mask anchored at the end of the cached sequence, explicit and
    default scale, block tables that are not the identity (src/nn/paged_attention.c:332-480)."""
    ref = ob.load_ref()
    for i in range(4):
        sq, kvl, hh, kh, hd, cz, spoil = (int(x) for x in golden[f"paged{i}_cfg"])
        sc = float(golden[f"paged{i}_scale"][0])
        q, k, v = golden[f"paged{i}_q"], golden[f"paged{i}_k"], golden[f"paged{i}_v"]
        out = np.empty_like(golden[f"paged{i}_out"])
        assert orc.orc_paged_gqa(ob.p(q), ob.p(k), ob.p(v), sq, kvl, hh, kh, hd, sc, cz, ob.p(out)) == 0
        assert np.abs(out - golden[f"paged{i}_out"]).max() < 1e-5
        if ref is not None:
            live = np.empty_like(out)
            assert ref.ref_paged_gqa(ob.p(q), ob.p(k), ob.p(v), sq, kvl, hh, kh, hd, sc, cz, 8, spoil, ob.p(live)) == (kvl + 15) // 16
            assert np.array_equal(live, golden[f"paged{i}_out"])
    # causal with the query anchored at the end: one query row over kv_len keys sees all of them
    q, k, v = golden["paged0_q"], golden["paged0_k"], golden["paged0_v"]
    a, b = np.empty_like(q), np.empty_like(q)
    assert orc.orc_paged_gqa(ob.p(q), ob.p(k), ob.p(v), 1, 37, 4, 2, 16, 0.0, 1, ob.p(a)) == 0
    assert orc.orc_paged_gqa(ob.p(q), ob.p(k), ob.p(v), 1, 37, 4, 2, 16, 0.0, 0, ob.p(b)) == 0
    assert np.array_equal(a, b)
    assert orc.orc_paged_gqa(ob.p(q), ob.p(k), ob.p(v), 1, 37, 3, 2, 16, 0.0, 1, ob.p(a)) == -1


def test_lora_restatement_matches_reference_vectors(ob, orc, golden):
    """orc_lora_forward / orc_lora_merge against the compiled reference's outputs (src/nn/lora.c)."""
    M, K, N, r, _ = (int(v) for v in golden["lora_cfg"])
    scaling = float(golden["lora_alpha"][0]) / r
    x, W, A, B = (np.ascontiguousarray(golden[k]) for k in ("lora_x", "lora_W", "lora_A", "lora_B"))
    t, y = np.zeros((M, r), np.float32), np.zeros((M, N), np.float32)
    orc.orc_lora_forward(ob.p(x), M, K, N, ob.p(W), ob.p(A), ob.p(B), r, scaling, 0, ob.p(t), ob.p(y))
    assert np.abs(y - golden["lora_y"]).max() <= 1e-5 * np.abs(golden["lora_y"]).max()
    Wm = W.copy()
    orc.orc_lora_merge(ob.p(Wm), ob.p(A), ob.p(B), N, K, r, scaling)
    assert np.abs(Wm - golden["lora_W_merged"]).max() <= 1e-6 * np.abs(Wm).max()
    orc.orc_lora_forward(ob.p(x), M, K, N, ob.p(Wm), ob.p(A), ob.p(B), r, scaling, 1, ob.p(t), ob.p(y))
    assert np.abs(y - golden["lora_y_merged"]).max() <= 1e-5 * np.abs(golden["lora_y_merged"]).max()


def test_quant8_restatement_matches_reference_vectors(ob, orc, golden):
    """orc_quant_params / orc_quantize8 / orc_dequantize8 bit for bit against the compiled reference
    (src/core/quantization.c:8-192), the out-of-range quotients included."""
    x = np.ascontiguousarray(golden["q8_x"])
    pr = np.zeros(2, np.int32)
    for mode, key in ((0, "q8_params_sym1"), (1, "q8_params_sym0"), (0, "q8_i8_auto_params"), (2, "q8_u8_auto_params")):
        orc.orc_quant_params(ob.p(x), x.size, mode, ob.p(pr))
        assert np.array_equal(pr, golden[key]), key
    for name, uns in (("i8_auto", 0), ("u8_auto", 1), ("i8_given", 0), ("u8_given", 1)):
        prm = golden[f"q8_{name}_params"]
        scale, zp = float(prm[:1].view(np.float32)[0]), int(prm[1])
        q, d = np.zeros(x.size, np.uint8), np.zeros(x.size, np.float32)
        orc.orc_quantize8(ob.p(x), x.size, scale, zp, uns, ob.p(q))
        assert np.array_equal(q, golden[f"q8_{name}_q"]), name
        orc.orc_dequantize8(ob.p(q), x.size, scale, zp, uns, ob.p(d))
        assert np.array_equal(d.view(np.uint32), golden[f"q8_{name}_deq"].view(np.uint32)), name
    xo = np.ascontiguousarray(golden["q8_x_outliers"])
    for name in ("i8_out", "i8_out_neg", "u8_out"):
        uns, zp = (int(v) for v in golden[f"q8_{name}_cfg"])
        q = np.zeros(xo.size, np.uint8)
        orc.orc_quantize8(ob.p(xo), xo.size, float(golden[f"q8_{name}_scale"][0]), zp, uns, ob.p(q))
        assert np.array_equal(q, golden[f"q8_{name}_q"]), name
