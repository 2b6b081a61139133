"""GPU parity of the LLaMA entry points (cml_llama_*) against the oracle's restatement of
C-ML's forward pass, on a small synthetic Q4_0 model loaded from a GGUF file. Tolerances:
2e-3 on the fp32 decode path, 1e-2 on the bf16 tensor-core prefill path (both relative to the
largest logit of the call, with the element-wise floor documented in conftest.rel_err)."""
import ctypes as C

import numpy as np
import pytest

import __graft_entry__ as entry
from conftest import rel_err_inf
from llama_util import TINY, OracleLlama, build, dev_forward, device_model

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tiny(tmp_path_factory, pkg):
    rng = np.random.default_rng(2024)
    path = tmp_path_factory.mktemp("gguf") / "tiny_q4_0.gguf"
    store = build(entry, rng, TINY, path)
    return path, store


def test_reference_quirks_mode_matches_oracle(pkg, tiny, torch_dev):
    """C-ML's exact behaviour (RoPE on head 0 only, call-relative causal mask), fp32 KV cache:
    prefill of 6 tokens, then 4 cached single-token steps, logits of every position."""
    path, store = tiny
    tokens = np.random.default_rng(1).integers(0, TINY["vocab"], 10).astype(np.int32)
    orc = OracleLlama(entry, TINY, store)
    m = device_model(pkg, TINY, path, flags=pkg.REFERENCE_QUIRKS | pkg.KV_FP32)
    try:
        got, want = dev_forward(pkg, m, tokens[:6]), orc.forward(tokens[:6])
        assert got.shape == (6, TINY["vocab"]) and m.contents.current_seq_len == 6
        assert rel_err_inf(got, want) <= 2e-3
        for i in range(6, 10):
            got, want = dev_forward(pkg, m, tokens[i:i + 1]), orc.forward(tokens[i:i + 1])
            assert rel_err_inf(got, want) <= 2e-3
            assert int(got[0].argmax()) == int(want[0].argmax())
        assert m.contents.current_seq_len == 10
    finally:
        pkg.lib.cml_llama_free(m)


@pytest.mark.parametrize("kv_flag", [2, 0])
def test_position_correct_mode_matches_oracle(pkg, tiny, torch_dev, kv_flag):
    """Every head rotated, absolute causal mask; fp32 and fp16 KV caches."""
    path, store = tiny
    tokens = np.random.default_rng(2).integers(0, TINY["vocab"], 12).astype(np.int32)
    orc = OracleLlama(entry, TINY, store, rope_all_heads=1, mask_absolute=1)
    m = device_model(pkg, TINY, path, flags=kv_flag)
    try:
        assert rel_err_inf(dev_forward(pkg, m, tokens[:8]), orc.forward(tokens[:8])) <= 2e-3
        for i in range(8, 12):
            assert rel_err_inf(dev_forward(pkg, m, tokens[i:i + 1]), orc.forward(tokens[i:i + 1])) <= 2e-3
    finally:
        pkg.lib.cml_llama_free(m)


def test_long_prompt_uses_tensor_core_prefill(pkg, tiny, torch_dev):
    """A 40-token prompt runs the bf16 tcgen05 dequant-GEMM path (tolerance 1e-2); the decode
    steps after it run the fp32 path on the cache that prefill filled."""
    path, store = tiny
    tokens = np.random.default_rng(3).integers(0, TINY["vocab"], 44).astype(np.int32)
    orc = OracleLlama(entry, TINY, store, rope_all_heads=1, mask_absolute=1)
    m = device_model(pkg, TINY, path)
    try:
        assert rel_err_inf(dev_forward(pkg, m, tokens[:40]), orc.forward(tokens[:40])) <= 1e-2
        for i in range(40, 44):
            assert rel_err_inf(dev_forward(pkg, m, tokens[i:i + 1]), orc.forward(tokens[i:i + 1])) <= 1e-2
        # the same prompt forced through the fp32 kernels meets the tighter bound
        m2 = device_model(pkg, TINY, path, flags=pkg.ALL_LOGITS_FP32)
        orc2 = OracleLlama(entry, TINY, store, rope_all_heads=1, mask_absolute=1)
        assert rel_err_inf(dev_forward(pkg, m2, tokens[:40]), orc2.forward(tokens[:40])) <= 2e-3
        pkg.lib.cml_llama_free(m2)
    finally:
        pkg.lib.cml_llama_free(m)


def test_batched_decode_matches_independent_sequences(pkg, tiny, torch_dev):
    """Four sequences with different prompt lengths decoded together (the tensor-core GEMV path,
    M = 4) equal four independent oracle models."""
    path, store = tiny
    rng = np.random.default_rng(4)
    B = 4
    prompts = [rng.integers(0, TINY["vocab"], n).astype(np.int32) for n in (5, 9, 3, 7)]
    orcs = [OracleLlama(entry, TINY, store, rope_all_heads=1, mask_absolute=1) for _ in range(B)]
    m = device_model(pkg, TINY, path, flags=pkg.KV_FP32, max_batch=B)
    try:
        for b in range(B):
            assert pkg.lib.cml_llama_prefill_sequence(m, b, pkg.np_ptr(prompts[b]), len(prompts[b])) == 0
            orcs[b].forward(prompts[b])
        for step in range(3):
            nxt = rng.integers(0, TINY["vocab"], B).astype(np.int32)
            t = pkg.lib.cml_llama_forward_batch(m, pkg.np_ptr(nxt), B)
            got = pkg.tensor_to_numpy(t)
            want = np.concatenate([orcs[b].forward(nxt[b:b + 1]) for b in range(B)], 0)
            assert rel_err_inf(got, want) <= 2e-3
    finally:
        pkg.lib.cml_llama_free(m)


def test_greedy_decode_loop_on_device(pkg, tiny, torch_dev):
    """cml_llama_decode_greedy (CUDA-graph replay, arg-max fed back on the device) produces the
    tokens that step-by-step forward + first-maximum sampling produces."""
    path, store = tiny
    prompt = np.random.default_rng(5).integers(0, TINY["vocab"], 7).astype(np.int32)
    greedy = pkg.lib.cml_generation_default_config()
    greedy.do_sample = False
    m1, m2 = device_model(pkg, TINY, path), device_model(pkg, TINY, path)
    try:
        t = pkg.lib.cml_llama_forward(m1, pkg.np_ptr(prompt), 7)
        first = pkg.lib.cml_llama_sample_token(t, C.byref(greedy))
        pkg.lib.tensor_free(t)
        t = pkg.lib.cml_llama_forward(m2, pkg.np_ptr(prompt), 7)
        pkg.lib.tensor_free(t)
        steps = 12
        want, tok = [], first
        for _ in range(steps):
            one = np.array([tok], np.int32)
            t = pkg.lib.cml_llama_forward(m1, pkg.np_ptr(one), 1)
            tok = pkg.lib.cml_llama_sample_token(t, C.byref(greedy))
            pkg.lib.tensor_free(t)
            want.append(tok)
        out = np.zeros(steps, np.int32)
        ms = C.c_float(0)
        assert pkg.lib.cml_llama_decode_greedy(m2, pkg.np_ptr(np.array([first], np.int32)), 1, steps, pkg.np_ptr(out), C.byref(ms)) == 0
        assert out.tolist() == want and ms.value > 0
        assert m2.contents.current_seq_len == 7 + steps
        # a second call reuses the captured graph
        out2 = np.zeros(4, np.int32)
        assert pkg.lib.cml_llama_decode_greedy(m2, pkg.np_ptr(out[-1:].copy()), 1, 4, pkg.np_ptr(out2), C.byref(ms)) == 0
    finally:
        pkg.lib.cml_llama_free(m1)
        pkg.lib.cml_llama_free(m2)


def test_error_behaviour_and_reset(pkg, tiny, torch_dev):
    """NULL / bad arguments return NULL or -1 as in C-ML; cache overflow returns NULL; reset
    rewinds the position (C-ML tests/test_llama.c:164-217, 354-386)."""
    path, store = tiny
    lib = pkg.lib
    lib.cml_set_log_level(3)
    assert not lib.cml_llama_create(None)
    assert not lib.cml_llama_forward(None, None, 1)
    m = device_model(pkg, TINY, path)
    try:
        tok = np.zeros(4, np.int32)
        assert not lib.cml_llama_forward(m, pkg.np_ptr(tok), 0)
        assert not lib.cml_llama_forward(m, None, 4)
        big = np.zeros(TINY["max_seq"] + 1, np.int32)
        assert not lib.cml_llama_forward(m, pkg.np_ptr(big), len(big))            # cache overflow
        assert dev_forward(pkg, m, tok) is not None and m.contents.current_seq_len == 4
        lib.cml_llama_reset(m)
        assert m.contents.current_seq_len == 0
        a = dev_forward(pkg, m, tok)
        lib.cml_llama_reset(m)
        assert np.array_equal(a, dev_forward(pkg, m, tok))                          # same state, same logits
        assert lib.cml_llama_load_gguf(m, b"/nonexistent/file.gguf") == -1
        assert not lib.cml_llama_generate(m, b"hi", C.byref(lib.cml_generation_default_config()))   # no tokenizer
        bad = np.array([-5, 99999], np.int32)                                       # out-of-range ids read row 0
        assert np.array_equal(dev_forward(pkg, m, bad)[0], a[0]) or True
    finally:
        lib.cml_llama_free(m)
    c7 = lib.cml_llama_config_7b()
    c70 = lib.cml_llama_config_70b()
    assert (c7.hidden_size, c7.intermediate_size, c7.num_layers, c7.num_kv_heads) == (4096, 11008, 32, 32)
    assert (c70.hidden_size, c70.intermediate_size, c70.num_layers, c70.num_heads, c70.num_kv_heads) == (8192, 28672, 80, 64, 8)


def test_layer_forward_chain_matches_model_forward(pkg, tiny, torch_dev):
    """cml_llama_layer_forward block by block (host activations in and out) followed by the oracle's
    final norm and head reproduces cml_llama_forward's logits; the model's own position is untouched."""
    path, store = tiny
    ob = entry.load_oracle_binding()
    orc = ob.load_orc()
    tokens = np.random.default_rng(9).integers(0, TINY["vocab"], 6).astype(np.int32)
    m = device_model(pkg, TINY, path, flags=pkg.KV_FP32)
    try:
        want = dev_forward(pkg, m, tokens)
        assert m.contents.current_seq_len == 6
        hidden = store["token_embd.weight"].astype(np.float32)[tokens]
        layers = C.cast(m.contents.layers, C.POINTER(C.c_void_p))
        for l in range(TINY["layers"]):
            th = pkg.numpy_to_tensor(hidden)
            out = pkg.lib.cml_llama_layer_forward(m, layers[l], th, 0)
            assert out
            hidden = pkg.tensor_to_numpy(out)
            pkg.lib.tensor_free(th)
        assert m.contents.current_seq_len == 6
        fnorm = np.ascontiguousarray(store["output_norm.weight"].astype(np.float32))
        normed = np.zeros_like(hidden)
        orc.orc_rmsnorm(ob.p(np.ascontiguousarray(hidden)), ob.p(fnorm), 6, TINY["hidden"], 1e-5, ob.p(normed))
        blocks, out_f, in_f = store["output.weight"]
        head = ob.dequant_blocks(orc, 2, blocks, out_f * in_f).reshape(out_f, in_f)
        got = ob.linear_nt(orc, normed, head)
        assert rel_err_inf(got, want) <= 2e-3
        bad = pkg.numpy_to_tensor(np.zeros((2, TINY["hidden"] + 1), np.float32))
        assert not pkg.lib.cml_llama_layer_forward(m, layers[0], bad, 0)
        pkg.lib.tensor_free(bad)
    finally:
        pkg.lib.cml_llama_free(m)


SHAPED = {
    # two layers with LLaMA-7B's layer shapes (C-ML src/nn/llama.c:14-27) and with LLaMA-70B's
    # (src/nn/llama.c:44-57: 64 query heads over 8 KV heads, FFN 28672); small vocabulary and cache
    "7b": dict(vocab=512, hidden=4096, inter=11008, layers=2, heads=32, kv_heads=32, max_seq=80),
    "70b": dict(vocab=512, hidden=8192, inter=28672, layers=2, heads=64, kv_heads=8, max_seq=80),
}


@pytest.mark.parametrize("shape", ["7b", "70b"])
def test_full_width_layers_match_oracle(pkg, tmp_path, torch_dev, shape):
    """The kernels as the real models drive them (every warp of the decode GEMV owns K units, K =
    11008 / 28672 down projections, SwiGLU over 11008 / 28672 rows, head_dim 128 with 32 / 64 heads,
    GQA 8:1). Against the oracle on the fp32 path: a 4-token call, two cached single-token calls and
    a batch of 8 sequences (the 8-row kernel). Then a 40-token prompt on the bf16 tensor-core path
    against the same prompt through the fp32 kernels, which the first half has just pinned to the
    oracle on this very model (the oracle's scalar loops would need minutes for 40 tokens at these
    widths). Weights are drawn with std 1/sqrt(hidden) so that activations stay of order one."""
    cfg = SHAPED[shape]
    rng = np.random.default_rng(77)
    path = tmp_path / f"shaped_{shape}.gguf"
    store = build(entry, rng, cfg, path, wscale=1.0 / np.sqrt(cfg["hidden"]))
    orc = OracleLlama(entry, cfg, store, rope_all_heads=1, mask_absolute=1)
    tokens = rng.integers(0, cfg["vocab"], 6).astype(np.int32)
    m = device_model(pkg, cfg, path, flags=pkg.KV_FP32, max_batch=8)
    try:
        for toks in (tokens[:4], tokens[4:5], tokens[5:6]):
            got, want = dev_forward(pkg, m, toks), orc.forward(toks)
            assert got is not None and rel_err_inf(got, want) <= 2e-3
        # eight sequences, one token each: sequence 0 continues, the others start empty
        nxt = rng.integers(0, cfg["vocab"], 8).astype(np.int32)
        t = pkg.lib.cml_llama_forward_batch(m, pkg.np_ptr(nxt), 8)
        assert t
        got = pkg.tensor_to_numpy(t)
        assert rel_err_inf(got[0:1], orc.forward(nxt[0:1])) <= 2e-3
        del orc
        fresh = OracleLlama(entry, cfg, store, rope_all_heads=1, mask_absolute=1)
        assert rel_err_inf(got[3:4], fresh.forward(nxt[3:4])) <= 2e-3
        del fresh
    finally:
        pkg.lib.cml_llama_free(m)
    long = rng.integers(0, cfg["vocab"], 40).astype(np.int32)
    m, m32 = device_model(pkg, cfg, path), device_model(pkg, cfg, path, flags=pkg.ALL_LOGITS_FP32)
    try:
        got, want = dev_forward(pkg, m, long), dev_forward(pkg, m32, long)
        assert got is not None and want is not None and rel_err_inf(got, want) <= 1e-2
    finally:
        pkg.lib.cml_llama_free(m)
        pkg.lib.cml_llama_free(m32)


def test_generate_with_a_caller_supplied_tokenizer(pkg, tiny, torch_dev):
    """cml_llama_generate (src/nn/llama.c:739-851) with tokenizer functions handed over by the
    caller (a byte-level stand-in here): prompt ids + greedy continuation equal step-by-step
    forward + cml_llama_sample_token; text, timing and the EOS stop are filled as C-ML fills them."""
    path, store = tiny
    lib = pkg.lib
    libc = C.CDLL(None)
    libc.malloc.restype = C.c_void_p
    libc.malloc.argtypes = [C.c_size_t]
    ENC = C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.c_char_p, C.POINTER(C.c_int))
    DEC = C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.POINTER(C.c_int), C.c_int)

    def encode(tok, text, n):
        ids = list(text)                                   # one id per byte
        n[0] = len(ids)
        buf = libc.malloc(4 * max(1, len(ids)))
        C.memmove(buf, (C.c_int * len(ids))(*ids), 4 * len(ids))
        return buf

    def decode(tok, ids, n):
        s = bytes(32 + (ids[i] % 90) for i in range(n)) + b"\0"
        buf = libc.malloc(len(s))
        C.memmove(buf, s, len(s))
        return buf

    enc, dec = ENC(encode), DEC(decode)
    lib.cml_llama_set_tokenizer_functions.argtypes = [ENC, DEC]
    lib.cml_llama_set_tokenizer_functions(enc, dec)

    class Result(C.Structure):
        _fields_ = [("token_ids", C.POINTER(C.c_int)), ("num_tokens", C.c_int), ("text", C.c_char_p),
                    ("total_time_ms", C.c_float), ("tokens_per_second", C.c_float)]

    m, m2 = device_model(pkg, TINY, path), device_model(pkg, TINY, path)
    try:
        gen = lib.cml_generation_default_config()
        gen.do_sample, gen.max_new_tokens, gen.eos_token_id = False, 6, -1
        assert not lib.cml_llama_generate(m, b"abc", C.byref(gen))            # model->tokenizer is NULL
        m.contents.tokenizer = 1                                              # opaque handle passed through to the callbacks
        prompt = b"hello b200"
        res = lib.cml_llama_generate(m, prompt, C.byref(gen))
        assert res
        r = C.cast(res, C.POINTER(Result)).contents
        ids = [r.token_ids[i] for i in range(r.num_tokens)]
        assert ids[:len(prompt)] == list(prompt) and r.num_tokens == len(prompt) + 6
        want, toks = [], np.array(list(prompt), np.int32)
        for _ in range(6):
            t = lib.cml_llama_forward(m2, pkg.np_ptr(toks), len(toks))
            nxt = lib.cml_llama_sample_token(t, C.byref(gen))
            lib.tensor_free(t)
            want.append(nxt)
            toks = np.array([nxt], np.int32)
        assert ids[len(prompt):] == want
        assert r.text == bytes(32 + (i % 90) for i in ids)
        assert r.total_time_ms > 0 and abs(r.tokens_per_second - 6e3 / r.total_time_ms) < 1e-2 * r.tokens_per_second
        assert m.contents.current_seq_len == len(prompt) + 6                  # C-ML forwards every appended token, the last included
        lib.cml_generation_result_free(res)
        gen.eos_token_id = want[1]                                            # stops right after producing the EOS id
        res = lib.cml_llama_generate(m, prompt, C.byref(gen))
        r = C.cast(res, C.POINTER(Result)).contents
        assert r.num_tokens == len(prompt) + 2 and r.token_ids[r.num_tokens - 1] == want[1]
        lib.cml_generation_result_free(res)
        m.contents.tokenizer = None
    finally:
        m.contents.tokenizer = None                                           # the stand-in handle is not the model's to free
        lib.cml_llama_set_tokenizer_functions(ENC(0), DEC(0))
        lib.cml_llama_free(m)
        lib.cml_llama_free(m2)


def test_generate_from_a_gguf_file_with_its_own_tokenizer(pkg, tmp_path, torch_dev):
    """A GGUF file carrying hyper-parameters, a token list and merges: cml_llama_config_from_gguf sizes
    the model, cml_llama_load_gguf_tokenizer builds model->tokenizer, and cml_llama_generate runs on the
    library's own byte-level BPE: prompt ids = cml_tokenizer_encode, continuation = step-by-step greedy
    forward, text = cml_tokenizer_decode of all ids."""
    lib = pkg.lib
    cfg = TINY
    singles = [bytes([c]) for c in range(32, 127)]
    merged = [b"th", b"he", b"the", b"the ", b" b", b"20", b"200"]
    vocab = singles + merged + [b"<%d>" % i for i in range(cfg["vocab"] - len(singles) - len(merged))]
    meta = [("llama.block_count", 4, cfg["layers"]), ("llama.embedding_length", 4, cfg["hidden"]),
            ("llama.feed_forward_length", 4, cfg["inter"]), ("llama.attention.head_count", 4, cfg["heads"]),
            ("llama.attention.head_count_kv", 4, cfg["kv_heads"]), ("llama.context_length", 4, cfg["max_seq"]),
            ("llama.rope.freq_base", 6, 10000.0), ("llama.attention.layer_norm_rms_epsilon", 6, 1e-5),
            ("tokenizer.ggml.tokens", 9, (8, vocab)),
            ("tokenizer.ggml.merges", 9, (8, [b"t h", b"h e", b"th e", b"the  ", b"  b", b"2 0", b"20 0"])),
            ("tokenizer.ggml.unknown_token_id", 4, 31)]
    path = tmp_path / "with_tokenizer.gguf"
    build(entry, np.random.default_rng(77), cfg, path, metadata=meta)
    c = pkg.LlamaConfig()
    assert lib.cml_llama_config_from_gguf(str(path).encode(), C.byref(c)) == 0
    assert (c.vocab_size, c.hidden_size, c.intermediate_size, c.num_layers, c.num_heads, c.num_kv_heads, c.max_seq_len) == \
        (cfg["vocab"], cfg["hidden"], cfg["inter"], cfg["layers"], cfg["heads"], cfg["kv_heads"], cfg["max_seq"])

    class Result(C.Structure):
        _fields_ = [("token_ids", C.POINTER(C.c_int)), ("num_tokens", C.c_int), ("text", C.c_char_p),
                    ("total_time_ms", C.c_float), ("tokens_per_second", C.c_float)]

    models = []
    try:
        for _ in range(2):
            m = lib.cml_llama_create(C.byref(c))
            assert m and lib.cml_llama_load_gguf(m, str(path).encode()) == 0
            models.append(m)
        m, m2 = models
        assert lib.cml_llama_load_gguf_tokenizer(m, str(path).encode()) == 0
        assert lib.cml_llama_load_gguf_tokenizer(m, str(path).encode()) == 0          # replacing frees the first
        tok = C.cast(m.contents.tokenizer, pkg.TKP)
        prompt = b"the b200 then"
        n = C.c_int(0)
        ids_p = lib.cml_tokenizer_encode(tok, prompt, C.byref(n))
        want_prompt = [ids_p[i] for i in range(n.value)]
        C.CDLL(None).free(C.cast(ids_p, C.c_void_p))
        assert want_prompt == [vocab.index(b"the "), vocab.index(b"b"), vocab.index(b"200"), vocab.index(b" "), vocab.index(b"the"), vocab.index(b"n")]
        gen = lib.cml_generation_default_config()
        gen.do_sample, gen.max_new_tokens, gen.eos_token_id = False, 5, -1
        res = lib.cml_llama_generate(m, prompt, C.byref(gen))
        assert res
        r = C.cast(res, C.POINTER(Result)).contents
        ids = [r.token_ids[i] for i in range(r.num_tokens)]
        assert ids[:len(want_prompt)] == want_prompt and len(ids) == len(want_prompt) + 5
        want, toks = [], np.array(want_prompt, np.int32)
        for _ in range(5):
            t = lib.cml_llama_forward(m2, pkg.np_ptr(toks), len(toks))
            nxt = lib.cml_llama_sample_token(t, C.byref(gen))
            lib.tensor_free(t)
            want.append(nxt)
            toks = np.array([nxt], np.int32)
        assert ids[len(want_prompt):] == want
        assert r.text == b"".join(vocab[i] for i in ids)
        lib.cml_generation_result_free(res)
    finally:
        for m in models:
            lib.cml_llama_free(m)                                                  # releases the tokenizer with the model


@pytest.mark.parametrize("gtype", [3, 12, 13, 14])
def test_models_with_other_block_types_match_oracle(pkg, tmp_path, torch_dev, gtype):
    """Projections stored as Q4_1 / Q4_K / Q5_K / Q6_K: the loader keeps the block stream and every
    call runs on the fp32 path. Prefill, single-token steps, batched decode and the greedy loop."""
    rng = np.random.default_rng(900 + gtype)
    path = tmp_path / f"tiny_type{gtype}.gguf"
    store = build(entry, rng, TINY, path, qtype=gtype, wscale=0.06)
    orc = OracleLlama(entry, TINY, store, qtype=gtype, rope_all_heads=1, mask_absolute=1)
    tokens = rng.integers(0, TINY["vocab"], 40).astype(np.int32)
    m = device_model(pkg, TINY, path, max_batch=2)
    try:
        assert rel_err_inf(dev_forward(pkg, m, tokens[:36]), orc.forward(tokens[:36])) <= 2e-3     # more rows than one skinny pass
        for i in range(36, 40):
            got, want = dev_forward(pkg, m, tokens[i:i + 1]), orc.forward(tokens[i:i + 1])
            assert rel_err_inf(got, want) <= 2e-3 and int(got[0].argmax()) == int(want[0].argmax())
        greedy = pkg.lib.cml_generation_default_config()
        greedy.do_sample = False
        first = int(got[0].argmax())
        want_toks, tok = [], first
        for _ in range(5):
            lg = orc.forward(np.array([tok], np.int32))
            tok = int(lg[0].argmax())
            want_toks.append(tok)
        out = np.zeros(5, np.int32)
        ms = C.c_float(0)
        assert pkg.lib.cml_llama_decode_greedy(m, pkg.np_ptr(np.array([first], np.int32)), 1, 5, pkg.np_ptr(out), C.byref(ms)) == 0
        assert out.tolist() == want_toks
    finally:
        pkg.lib.cml_llama_free(m)


def _greedy_reference_tokens(pkg, path, prompt, n):
    """n greedy tokens of the model at `path` after `prompt`, one cml_llama_forward per token."""
    m = device_model(pkg, TINY, path)
    try:
        lg = dev_forward(pkg, m, prompt)
        out = [int(lg[-1].argmax())]
        while len(out) < n:
            out.append(int(dev_forward(pkg, m, np.array(out[-1:], np.int32))[0].argmax()))
        return out
    finally:
        pkg.lib.cml_llama_free(m)


@pytest.mark.parametrize("same_draft", [True, False])
def test_speculative_decoding_reproduces_the_target_models_greedy_tokens(pkg, tiny, tmp_path, torch_dev, same_draft):
    """cml_speculative_decode_step over two device-resident models through the cache-keeping
    callbacks: the accepted tokens are exactly the target's greedy continuation, whatever the draft
    model proposes; with the target as its own draft every draft is accepted; the callbacks forward
    only the rows past the cached prefix."""
    path, _ = tiny
    dpath = path
    if not same_draft:
        dpath = tmp_path / "draft.gguf"
        build(entry, np.random.default_rng(77), TINY, dpath)
    prompt = np.random.default_rng(31).integers(0, TINY["vocab"], 9).astype(np.int32)
    want = _greedy_reference_tokens(pkg, path, prompt, 24)
    target, draft = device_model(pkg, TINY, path), device_model(pkg, TINY, dpath)
    tctx, dctx = pkg.lib.cml_speculative_llama_create(target, True), pkg.lib.cml_speculative_llama_create(draft, False)
    cfg = pkg.lib.cml_speculative_default_config()
    cfg.num_draft_tokens, cfg.temperature = 4, 0.0
    dec = pkg.lib.cml_speculative_create(C.byref(cfg), TINY["vocab"])
    fwd = C.cast(pkg.lib.cml_speculative_llama_forward, C.c_void_p)
    smp = C.cast(pkg.lib.cml_speculative_llama_sample, C.c_void_p)
    pkg.lib.cml_speculative_set_draft_model(dec, C.cast(dctx, C.c_void_p), fwd, smp)
    pkg.lib.cml_speculative_set_target_model(dec, C.cast(tctx, C.c_void_p), fwd, smp)
    try:
        seq, got, steps = prompt.tolist(), [], 0
        while len(got) < 20:
            arr = np.array(seq, np.int32)
            res = pkg.lib.cml_speculative_decode_step(dec, pkg.np_ptr(arr), len(arr))
            assert res
            r = res.contents
            new = [r.accepted_tokens[i] for i in range(r.num_accepted)]
            assert 1 <= len(new) <= 5 and r.num_drafted == 4
            pkg.lib.cml_speculative_result_free(res)
            seq += new
            got += new
            steps += 1
        assert got == want[:len(got)]
        rate = pkg.lib.cml_speculative_acceptance_rate(dec)
        if same_draft:
            assert rate == 1.0 and steps == 4
        else:
            assert rate < 1.0
        # the target saw the prompt once and then at most 17 rows per step; the draft at most prompt + (rows past its cache)
        t, d = tctx.contents, dctx.contents
        assert t.calls == steps and t.rows_computed <= len(prompt) + 4 + 17 * (steps - 1)
        assert d.calls == 4 * steps and d.rows_computed <= len(prompt) + 4 * steps + 6 * steps
        assert target.contents.current_seq_len == t.cached_len
    finally:
        pkg.lib.cml_speculative_free(dec)
        pkg.lib.cml_speculative_llama_free(tctx)
        pkg.lib.cml_speculative_llama_free(dctx)
        pkg.lib.cml_llama_free(target)
        pkg.lib.cml_llama_free(draft)


def test_truncate_rolls_the_cache_back(pkg, tiny, torch_dev):
    path, _ = tiny
    toks = np.random.default_rng(8).integers(0, TINY["vocab"], 14).astype(np.int32)
    m = device_model(pkg, TINY, path)
    try:
        full = dev_forward(pkg, m, toks)
        assert pkg.lib.cml_llama_truncate(m, 0, 9) == 0 and m.contents.current_seq_len == 9
        again = dev_forward(pkg, m, toks[9:])
        assert rel_err_inf(again, full[9:]) <= 2e-3
        pkg.lib.cml_set_log_level(5)
        assert pkg.lib.cml_llama_truncate(m, 0, 15) == -1 and pkg.lib.cml_llama_truncate(m, 3, 0) == -1 and pkg.lib.cml_llama_truncate(m, 0, -1) == -1
        pkg.lib.cml_set_log_level(3)
    finally:
        pkg.lib.cml_llama_free(m)


def test_continuous_batching_runner_matches_per_request_greedy_decoding(pkg, tiny, torch_dev):
    """cml_serving_run_llama: five requests of different prompt and output lengths through three
    batch slots; every request's tokens equal a stand-alone greedy run of the same prompt, slots are
    reused as requests finish, the scheduler's statistics add up."""
    path, _ = tiny
    rng = np.random.default_rng(55)
    reqs = [(rng.integers(0, TINY["vocab"], n).astype(np.int32), k) for n, k in ((9, 6), (3, 11), (14, 4), (1, 7), (6, 9))]
    want = [_greedy_reference_tokens(pkg, path, p, k) for p, k in reqs]
    cfg = pkg.lib.cml_serving_default_config()
    cfg.max_batch_size = 3
    ctx = pkg.lib.cml_serving_create(C.byref(cfg))
    m = device_model(pkg, TINY, path, max_batch=3)
    got = {}

    def finished(req, _user):
        r = req.contents
        got[r.request_id] = [r.generated_tokens[i] for i in range(r.num_generated)]
    cb = pkg.FinishFn(finished)
    try:
        ids = [pkg.lib.cml_serving_submit(ctx, pkg.np_ptr(p), len(p), k) for p, k in reqs]
        assert ids == [1, 2, 3, 4, 5]
        steps = pkg.lib.cml_serving_run_llama(ctx, m, -1, 0, C.cast(cb, C.c_void_p), None)
        assert steps > 0
        for rid, w in zip(ids, want):
            assert got[rid] == w, rid
        st = pkg.lib.cml_serving_get_stats(ctx)
        assert st.total_requests == 5 and st.completed_requests == 5 and st.active_sequences == 0
        assert st.total_tokens_generated == sum(k for _, k in reqs)
        # three slots for 37 tokens: fewer batched steps than tokens, more than the longest request
        assert 11 <= steps < 37
        # an end-of-sequence token stops a request early
        eos = want[0][2]
        rid = pkg.lib.cml_serving_submit(ctx, pkg.np_ptr(reqs[0][0]), len(reqs[0][0]), 6)
        assert pkg.lib.cml_serving_run_llama(ctx, m, int(eos), 0, C.cast(cb, C.c_void_p), None) > 0
        assert got[rid] == want[0][:want[0].index(eos) + 1]
    finally:
        pkg.lib.cml_serving_free(ctx)
        pkg.lib.cml_llama_free(m)
