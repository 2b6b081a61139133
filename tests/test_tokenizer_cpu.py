"""The byte-level BPE tokenizer and the GGUF key/value reader (host code, no GPU): encode / decode
against vectors produced by the compiled C-ML tokenizer (tests/golden/make_golden.py; C-ML
src/nn/llm_ops.c:1140-1389), against the compiled reference itself on random cases where it is
built, the known answers of C-ML's tests/test_llm_ops.c:550-665, and a synthetic GGUF file with a
token list, merges, special ids and hyper-parameters read back through the library."""
import ctypes as C
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

libc = C.CDLL(None)
libc.free.argtypes = [C.c_void_p]


@pytest.fixture(scope="module")
def pkg():
    return entry.load_package()


def split_blob(blob, n):
    parts = bytes(blob).split(b"\0")
    assert len(parts) >= n
    return parts[:n]


def make_tok(pkg, vocab, merges):
    va = (C.c_char_p * len(vocab))(*vocab)
    ma = (C.c_char_p * max(1, len(merges)))(*merges) if merges else None
    tok = pkg.lib.cml_tokenizer_create(va, len(vocab), ma, len(merges))
    assert tok
    return tok


def encode(pkg, tok, text):
    n = C.c_int(-7)
    ids = pkg.lib.cml_tokenizer_encode(tok, text, C.byref(n))
    if not ids:
        return None, n.value
    out = [ids[i] for i in range(n.value)]
    libc.free(C.cast(ids, C.c_void_p))
    return out, n.value


def decode(pkg, tok, ids):
    arr = np.asarray(ids, np.int32)
    s = pkg.lib.cml_tokenizer_decode(tok, arr.ctypes.data, len(arr))
    if not s:
        return None
    out = C.string_at(s)
    libc.free(s)
    return out


def test_encode_decode_match_the_reference_vectors(pkg, golden):
    nv, nm = int(golden["tok_vocab_n"][0]), int(golden["tok_merges_n"][0])
    vocab = split_blob(golden["tok_vocab_blob"], nv)
    merges = split_blob(golden["tok_merges_blob"], nm)
    counts, unks = golden["tok_counts"], golden["tok_unk"]
    texts = split_blob(golden["tok_texts_blob"], len(counts))
    tok = make_tok(pkg, vocab, merges)
    assert tok.contents.vocab_size == nv and tok.contents.num_merges == nm
    assert tok.contents.bos_token_id == -1 and tok.contents.unk_token_id == -1
    off = 0
    for txt, n, unk in zip(texts, counts, unks):
        pkg.lib.cml_tokenizer_set_special(tok, -1, -1, -1, int(unk))
        ids, got_n = encode(pkg, tok, txt)
        want = golden["tok_ids"][off:off + n].tolist()
        assert got_n == n and ids == want, txt
        off += n
    assert decode(pkg, tok, golden["tok_decode_ids"]) == bytes(golden["tok_decode_text"])
    pkg.lib.cml_tokenizer_free(tok)


def test_known_answers_and_edge_cases(pkg):
    tok = make_tok(pkg, [b"h", b"e", b"l", b"o"], [])
    assert encode(pkg, tok, b"hello") == ([0, 1, 2, 2, 3], 5)
    assert decode(pkg, tok, [0, 1, 2, 2, 3]) == b"hello"
    assert encode(pkg, tok, b"") == (None, 0)                       # empty text: no array, zero tokens
    assert encode(pkg, tok, b"hex") == ([0, 1, 0], 3)               # unknown spelling, unk unset -> id 0
    pkg.lib.cml_tokenizer_set_special(tok, 0, 1, 2, 3)
    t = tok.contents
    assert (t.bos_token_id, t.eos_token_id, t.pad_token_id, t.unk_token_id) == (0, 1, 2, 3)
    assert encode(pkg, tok, b"hex") == ([0, 1, 3], 3)
    assert pkg.lib.cml_tokenizer_vocab_size(tok) == 4 and pkg.lib.cml_tokenizer_vocab_size(None) == 0
    assert decode(pkg, tok, [9, -1]) == b""                         # ids outside the vocabulary contribute nothing
    assert decode(pkg, tok, []) is None
    pkg.lib.cml_tokenizer_free(tok)
    tok = make_tok(pkg, [b"a", b"b", b"ab"], [b"ab"])
    ids, n = encode(pkg, tok, b"abab")
    assert n == 2 and ids == [2, 2] and decode(pkg, tok, ids) == b"abab"
    pkg.lib.cml_tokenizer_free(tok)
    # the joined token meets its left neighbour again under the same rule: "aa" on "aaaa" -> [aa][aa];
    # rule order decides, not length: ["bc", "ab"] on "abc" -> [a][bc]
    tok = make_tok(pkg, [b"a", b"aa", b"b", b"c", b"bc", b"ab"], [b"aa", b"bc", b"ab"])
    assert encode(pkg, tok, b"aaaa")[0] == [1, 1]
    assert encode(pkg, tok, b"aaa")[0] == [1, 0]
    assert encode(pkg, tok, b"abc")[0] == [0, 4]
    pkg.lib.cml_tokenizer_free(tok)
    assert not pkg.lib.cml_tokenizer_create(None, 3, None, 0)
    va = (C.c_char_p * 1)(b"x")
    assert not pkg.lib.cml_tokenizer_create(va, 0, None, 0)
    pkg.lib.cml_tokenizer_free(None)


def test_random_cases_against_the_compiled_reference(pkg):
    """Where the reference library is built (not on a GPU box): a few hundred random vocabularies,
    merge lists and texts, including long runs of one byte and spellings missing from the vocabulary."""
    sys.path.insert(0, str(ROOT / "oracle"))
    import binding
    try:
        ref = binding.load_ref()
    except Exception as e:                                           # noqa: BLE001
        pytest.skip(f"compiled reference not available: {e}")
    rng = np.random.default_rng(5)
    for case in range(150):
        alpha = [bytes([c]) for c in rng.choice(np.arange(97, 123), size=int(rng.integers(2, 6)), replace=False)]
        vocab, merges = list(alpha), []
        for _ in range(int(rng.integers(0, 25))):
            s = vocab[rng.integers(len(vocab))] + vocab[rng.integers(len(vocab))]
            if len(s) > 12:
                continue
            merges.append(s)
            if rng.random() < 0.8:
                vocab.append(s)
        if rng.random() < 0.3:
            vocab.append(vocab[rng.integers(len(vocab))])
        n = int(rng.choice([1, 2, 7, 40, 300]))
        pool = alpha + [b"z"] if rng.random() < 0.3 else alpha
        text = b"".join(pool[i] for i in rng.integers(len(pool), size=n))
        unk = int(rng.integers(-1, len(vocab)))
        buf = np.zeros(n + 1, np.int32)
        vb = b"".join(v + b"\0" for v in vocab)
        mb = b"".join(m + b"\0" for m in merges) or b"\0"
        want_n = ref.ref_tokenizer_encode(vb, len(vocab), mb, len(merges), unk, text, buf.ctypes.data, len(buf))
        tok = make_tok(pkg, vocab, merges)
        pkg.lib.cml_tokenizer_set_special(tok, -1, -1, -1, unk)
        ids, got_n = encode(pkg, tok, text)
        assert got_n == want_n and ids == buf[:want_n].tolist(), (case, text, merges)
        pkg.lib.cml_tokenizer_free(tok)


def test_gguf_metadata_tokenizer_and_config(pkg, tmp_path):
    synth = entry.load_synth()
    vocab = [b"<unk>", b"<s>", b"</s>", b"a", b"b", b" ", b"ab", b"ab ", b" a"]
    meta = [
        ("llama.block_count", 4, 3), ("llama.embedding_length", 4, 256), ("llama.feed_forward_length", 4, 704),
        ("llama.attention.head_count", 4, 8), ("llama.attention.head_count_kv", 4, 2), ("llama.context_length", 10, 384),
        ("llama.rope.freq_base", 6, 50000.0), ("llama.attention.layer_norm_rms_epsilon", 6, 1e-6),
        ("general.name", 8, "tiny"), ("general.quantized", 7, 1), ("some.i16", 3, -12), ("some.f64", 12, 2.5),
        ("tokenizer.ggml.model", 8, "gpt2"),
        ("tokenizer.ggml.tokens", 9, (8, vocab)),
        ("tokenizer.ggml.scores", 9, (6, [0.0] * len(vocab))),
        ("tokenizer.ggml.token_type", 9, (5, list(range(len(vocab))))),
        ("tokenizer.ggml.merges", 9, (8, [b"a b", b"ab  ", b"  a"])),
        ("tokenizer.ggml.bos_token_id", 4, 1), ("tokenizer.ggml.eos_token_id", 4, 2), ("tokenizer.ggml.unknown_token_id", 4, 0),
        ("nested", 9, (9, [(4, [1, 2]), (8, [b"x"])])),
    ]
    path = tmp_path / "meta.gguf"
    emb = np.zeros((len(vocab), 256), np.float32)
    synth.write_gguf(str(path), [("token_embd.weight", (len(vocab), 256), 0, emb.tobytes())], metadata=meta)
    lib = pkg.lib
    g = lib.gguf_open_read(str(path).encode())
    assert g
    assert lib.gguf_get_num_metadata(g) == len(meta) + 1 and lib.gguf_get_metadata_key(g, 0) == b"general.architecture"
    assert lib.gguf_get_num_tensors(g) == 1                                  # the tensor infos still parse after the values
    v, f, et = C.c_int64(0), C.c_double(0), C.c_int(-1)
    assert lib.gguf_get_metadata_int(g, b"llama.block_count", C.byref(v)) == 0 and v.value == 3
    assert lib.gguf_get_metadata_int(g, b"some.i16", C.byref(v)) == 0 and v.value == -12
    assert lib.gguf_get_metadata_int(g, b"llama.context_length", C.byref(v)) == 0 and v.value == 384
    assert lib.gguf_get_metadata_int(g, b"general.quantized", C.byref(v)) == 0 and v.value == 1
    assert lib.gguf_get_metadata_int(g, b"llama.rope.freq_base", C.byref(v)) == -1      # a float is not an integer
    assert lib.gguf_get_metadata_int(g, b"missing", C.byref(v)) == -1 and lib.gguf_get_metadata_type(g, b"missing") == -1
    assert lib.gguf_get_metadata_float(g, b"llama.rope.freq_base", C.byref(f)) == 0 and f.value == 50000.0
    assert lib.gguf_get_metadata_float(g, b"some.f64", C.byref(f)) == 0 and f.value == 2.5
    assert lib.gguf_get_metadata_float(g, b"llama.block_count", C.byref(f)) == 0 and f.value == 3.0
    assert lib.gguf_get_metadata_string(g, b"general.name") == b"tiny" and lib.gguf_get_metadata_string(g, b"llama.block_count") is None
    assert lib.gguf_get_metadata_type(g, b"tokenizer.ggml.tokens") == 9
    assert lib.gguf_get_metadata_array_length(g, b"tokenizer.ggml.tokens", C.byref(et)) == len(vocab) and et.value == 8
    assert lib.gguf_get_metadata_array_string(g, b"tokenizer.ggml.tokens", 7) == b"ab "
    assert lib.gguf_get_metadata_array_string(g, b"tokenizer.ggml.tokens", len(vocab)) is None
    assert lib.gguf_get_metadata_array_length(g, b"tokenizer.ggml.token_type", C.byref(et)) == len(vocab) and et.value == 5
    data = lib.gguf_get_metadata_array_data(g, b"tokenizer.ggml.token_type")
    assert list((C.c_int32 * len(vocab)).from_address(data)) == list(range(len(vocab)))
    assert lib.gguf_get_metadata_array_length(g, b"nested", C.byref(et)) == 2 and et.value == 9
    assert lib.gguf_get_metadata_array_data(g, b"nested") is None
    assert lib.gguf_get_metadata_array_length(g, b"general.name", None) == -1
    tok = lib.gguf_create_tokenizer(g)
    lib.gguf_close(g)
    assert tok
    t = tok.contents
    assert t.vocab_size == len(vocab) and t.num_merges == 3
    assert (t.bos_token_id, t.eos_token_id, t.pad_token_id, t.unk_token_id) == (1, 2, -1, 0)
    assert encode(pkg, tok, b"ab ab")[0] == [7, 6]                           # "a b" -> ab, "ab  " -> "ab " (the left part may end the pair with a space)
    assert encode(pkg, tok, b"b a")[0] == [4, 8]                             # "  a": a pair whose left part is a space
    assert encode(pkg, tok, b"abq")[0] == [6, 0]
    lib.cml_tokenizer_free(tok)
    cfg = pkg.LlamaConfig()
    assert lib.cml_llama_config_from_gguf(str(path).encode(), C.byref(cfg)) == 0
    assert (cfg.vocab_size, cfg.hidden_size, cfg.intermediate_size, cfg.num_layers, cfg.num_heads, cfg.num_kv_heads, cfg.max_seq_len) == \
        (len(vocab), 256, 704, 3, 8, 2, 384)
    assert cfg.rope_theta == 50000.0 and abs(cfg.rms_norm_eps - 1e-6) < 1e-12
    # a file without hyper-parameters or token list
    bare = tmp_path / "bare.gguf"
    synth.write_gguf(str(bare), [("token_embd.weight", (len(vocab), 256), 0, emb.tobytes())])
    assert lib.cml_llama_config_from_gguf(str(bare).encode(), C.byref(cfg)) == -1
    g = lib.gguf_open_read(str(bare).encode())
    assert g and not lib.gguf_create_tokenizer(g)
    lib.gguf_close(g)
    # truncated inside the metadata: the open fails, as C-ML's does
    raw = path.read_bytes()
    cut = tmp_path / "cut.gguf"
    cut.write_bytes(raw[:200])
    assert not lib.gguf_open_read(str(cut).encode())


def test_gguf_reader_survives_truncated_and_mutated_files(pkg, tmp_path):
    """Every truncation of a small GGUF file and 1,500 random byte mutations of it: the reader either
    refuses the file or returns a context that can be queried, turned into a tokenizer and closed.
    Counts taken from the file are checked against the bytes left before anything is allocated or
    looped over (a mutated array length used to make the value skipper seek 2^60 times)."""
    synth = entry.load_synth()
    lib = pkg.lib
    vocab = [b"<unk>", b"a", b"b", b"ab"]
    meta = [("llama.block_count", 4, 3), ("general.name", 8, "tiny"), ("tokenizer.ggml.tokens", 9, (8, vocab)),
            ("tokenizer.ggml.token_type", 9, (5, [1, 2, 3, 4])), ("tokenizer.ggml.merges", 9, (8, [b"a b"])),
            ("nested", 9, (9, [(4, [1, 2]), (8, [b"x"])])), ("f", 12, 2.5)]
    path = tmp_path / "m.gguf"
    synth.write_gguf(str(path), [("token_embd.weight", (4, 8), 0, np.zeros((4, 8), np.float32).tobytes())], metadata=meta)
    raw = path.read_bytes()
    cut = tmp_path / "c.gguf"
    lib.cml_set_log_level.argtypes = [C.c_int]
    lib.cml_set_log_level(5)                                        # the refusals are expected: keep them off the log

    def probe(data):
        cut.write_bytes(data)
        g = lib.gguf_open_read(str(cut).encode())
        if not g:
            return 0
        for i in range(lib.gguf_get_num_metadata(g)):
            key = lib.gguf_get_metadata_key(g, i)
            assert key is not None
            lib.gguf_get_metadata_type(g, key)
            lib.gguf_get_metadata_array_length(g, key, None)
        tok = lib.gguf_create_tokenizer(g)
        if tok:
            n = C.c_int(0)
            ids = lib.cml_tokenizer_encode(tok, b"abab", C.byref(n))
            if ids:
                libc.free(C.cast(ids, C.c_void_p))
            lib.cml_tokenizer_free(tok)
        lib.gguf_close(g)
        lib.cml_llama_config_from_gguf(str(cut).encode(), C.byref(pkg.LlamaConfig()))
        return 1
    try:
        opened = sum(probe(raw[:k]) for k in range(len(raw)))
        assert 0 < opened < len(raw)                                # cuts inside the tensor data still open, cuts before it do not
        rng = np.random.default_rng(0)
        for _ in range(1500):
            b = bytearray(raw)
            for _ in range(int(rng.integers(1, 4))):
                b[int(rng.integers(0, len(b) - 130))] = int(rng.integers(0, 256))
            probe(bytes(b))
        assert probe(raw) == 1
    finally:
        lib.cml_set_log_level(3)


def test_gguf_writer_emits_c_ml_bytes_and_reads_back(pkg, golden, tmp_path):
    """gguf_open_write / gguf_write_tensor / gguf_close produce, for the same three tensors, the file
    C-ML's writer produces (src/core/gguf.c:181-232, 312-340; bytes from the compiled reference); the
    additions (key/values, block-quantized tensors) read back through gguf_open_read."""
    lib = pkg.lib
    path = tmp_path / "mine.gguf"
    g = lib.gguf_open_write(str(path).encode())
    assert g
    tensors = [pkg.numpy_to_tensor(np.ascontiguousarray(golden["ggufw_a"])), pkg.numpy_to_tensor(np.ascontiguousarray(golden["ggufw_b"])),
               pkg.numpy_to_tensor(np.ascontiguousarray(golden["ggufw_c"]).view(np.float16))]
    for name, t in zip((b"w.f32", b"v.i32", b"h.f16"), tensors):
        assert lib.gguf_write_tensor(g, name, t) == 0
    assert lib.gguf_write_tensor(g, None, tensors[0]) == -1 and lib.gguf_write_tensor(g, b"x", None) == -1
    assert lib.gguf_get_num_tensors(g) == 0                                   # a write context lists nothing
    lib.gguf_close(g)
    assert path.read_bytes() == bytes(golden["ggufw_file"])
    # nothing written -> no file (src/core/gguf.c:184)
    empty = tmp_path / "empty.gguf"
    lib.gguf_close(lib.gguf_open_write(str(empty).encode()))
    assert not empty.exists()
    # a model-like file from C: key/values, a string array, a Q4_0 tensor, an fp32 tensor
    synth = entry.load_synth()
    rng = np.random.default_rng(3)
    blocks = synth.q4_0_blocks(rng, 8, 64)
    full = tmp_path / "full.gguf"
    g = lib.gguf_open_write(str(full).encode())
    u32, f32 = C.c_uint32(7), C.c_float(1e-5)
    assert lib.gguf_write_metadata(g, b"llama.block_count", 4, C.byref(u32)) == 0
    assert lib.gguf_write_metadata(g, b"llama.attention.layer_norm_rms_epsilon", 6, C.byref(f32)) == 0
    assert lib.gguf_write_metadata(g, b"general.name", 8, b"from-c") == 0
    toks = (C.c_char_p * 3)(b"a", b"b", b"ab")
    assert lib.gguf_write_metadata_array(g, b"tokenizer.ggml.tokens", 8, toks, 3) == 0
    types = (C.c_int32 * 3)(1, 1, 2)
    assert lib.gguf_write_metadata_array(g, b"tokenizer.ggml.token_type", 5, types, 3) == 0
    assert lib.gguf_write_metadata(g, b"bad", 9, C.byref(u32)) == -1 and lib.gguf_write_metadata(g, None, 4, C.byref(u32)) == -1
    shape = (C.c_int64 * 2)(8, 64)
    assert lib.gguf_write_blocks(g, b"blk.0.attn_q.weight", 2, shape, 2, blocks.ctypes.data) == 0
    assert lib.gguf_write_blocks(g, b"odd", 2, (C.c_int64 * 1)(33), 1, blocks.ctypes.data) == -1      # not a whole number of blocks
    assert lib.gguf_write_blocks(g, b"f32", 0, shape, 2, blocks.ctypes.data) == -1                    # not a block type
    assert lib.gguf_write_tensor(g, b"norm.weight", tensors[0]) == 0
    lib.gguf_close(g)
    r = lib.gguf_open_read(str(full).encode())
    assert r and lib.gguf_get_num_tensors(r) == 2 and lib.gguf_get_num_metadata(r) == 5
    assert lib.gguf_get_tensor_name(r, 0) == b"blk.0.attn_q.weight" and lib.gguf_get_tensor_name(r, 1) == b"norm.weight"
    v, f = C.c_int64(0), C.c_double(0)
    assert lib.gguf_get_metadata_int(r, b"llama.block_count", C.byref(v)) == 0 and v.value == 7
    assert lib.gguf_get_metadata_float(r, b"llama.attention.layer_norm_rms_epsilon", C.byref(f)) == 0 and f.value == float(np.float32(1e-5))
    assert lib.gguf_get_metadata_string(r, b"general.name") == b"from-c"
    assert lib.gguf_get_metadata_array_string(r, b"tokenizer.ggml.tokens", 2) == b"ab"
    tok = lib.gguf_create_tokenizer(r)
    assert tok and encode(pkg, tok, b"abb")[0] == [0, 1, 1]                   # no merges in the file: bytes only
    lib.cml_tokenizer_free(tok)
    back = lib.gguf_read_tensor(r, b"norm.weight")                            # not quantized: no device involved
    assert back and np.array_equal(pkg.tensor_to_numpy(back), golden["ggufw_a"])
    lib.gguf_close(r)
    # the block payload sits, unpadded, right behind the aligned start of the data section
    raw = full.read_bytes()
    at = raw.find(blocks.tobytes())
    assert at > 0 and at % 32 == 0 and raw[at + blocks.nbytes:at + blocks.nbytes + 60] == golden["ggufw_a"].tobytes()
    for t in tensors:
        lib.tensor_free(t)


def test_gguf_tensor_reads_are_bounded_by_the_file(pkg, tmp_path):
    """A tensor is read when its bytes lie inside the file (padded tail, unpadded tail) and refused when
    they reach past its end, before anything is allocated for it."""
    synth = entry.load_synth()
    lib = pkg.lib
    rng = np.random.default_rng(0)
    a = rng.standard_normal((7, 9)).astype(np.float32)
    b = rng.standard_normal(5).astype(np.float32)
    path = tmp_path / "s.gguf"
    synth.write_gguf(str(path), [("a", (7, 9), 0, a.tobytes()), ("q", (4, 64), 2, synth.q4_0_blocks(rng, 4, 64).tobytes()),
                                 ("b", (5,), 0, b.tobytes())])
    raw = path.read_bytes()
    end = raw.rfind(b.tobytes()) + b.nbytes
    lib.cml_set_log_level.argtypes = [C.c_int]
    lib.cml_set_log_level(5)
    try:
        for data, last_ok in ((raw, True), (raw[:end], True), (raw[:end - 1], False)):
            path.write_bytes(data)
            g = lib.gguf_open_read(str(path).encode())
            assert g
            t = lib.gguf_read_tensor(g, b"a")
            assert t and np.array_equal(pkg.tensor_to_numpy(t), a)
            t = lib.gguf_read_tensor(g, b"b")
            assert bool(t) == last_ok
            if t:
                assert np.array_equal(pkg.tensor_to_numpy(t), b)
            assert not lib.gguf_read_tensor(g, b"missing")
            lib.gguf_close(g)
    finally:
        lib.cml_set_log_level(3)
