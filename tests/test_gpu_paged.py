"""GPU parity of the paged KV cache + cml_paged_gqa_forward (include/nn/paged_attention.h in the
C-ML tree) against the stored outputs of the compiled reference and against the oracle."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _forward(pkg, cache, seq, q, heads, kvh, hd, scale=0.0, causal=True):
    tq = pkg.numpy_to_tensor(q[None])
    cfg = pkg.GQAConfig(heads, kvh, hd, scale, causal, 0)
    t = pkg.lib.cml_paged_gqa_forward(cache, seq, tq, C.byref(cfg))
    pkg.lib.tensor_free(tq)
    return pkg.tensor_to_numpy(t)[0] if t else None


def _append(pkg, cache, seq, k, v):
    for t in range(len(k)):
        assert pkg.lib.cml_paged_cache_append(cache, seq, pkg.np_ptr(np.ascontiguousarray(k[t])), pkg.np_ptr(np.ascontiguousarray(v[t]))) == 0


def test_paged_attention_matches_the_reference_outputs(pkg, golden, torch_dev):
    for i in range(4):
        sq, kvl, hh, kh, hd, cz, spoil = (int(x) for x in golden[f"paged{i}_cfg"])
        sc = float(golden[f"paged{i}_scale"][0])
        q, k, v = golden[f"paged{i}_q"], golden[f"paged{i}_k"], golden[f"paged{i}_v"]
        cache = pkg.lib.cml_paged_kv_cache_create(8, 4, kh, hd)
        try:
            other = -1
            if spoil:                                         # the block table must not be the identity
                other = pkg.lib.cml_paged_cache_init_sequence(cache)
                _append(pkg, cache, other, np.repeat(k[:1], spoil, 0), np.repeat(v[:1], spoil, 0))
            s = pkg.lib.cml_paged_cache_init_sequence(cache)
            _append(pkg, cache, s, k[:kvl // 2], v[:kvl // 2])
            if other >= 0:
                pkg.lib.cml_paged_cache_free_sequence(cache, other)
            _append(pkg, cache, s, k[kvl // 2:], v[kvl // 2:])
            got = _forward(pkg, cache, s, q, hh, kh, hd, sc, bool(cz))
            assert got.shape == (sq, hh * hd)
            assert np.abs(got - golden[f"paged{i}_out"]).max() <= 2e-5
            bt = cache.contents.sequences[s]
            assert bt.seq_len == kvl and bt.num_blocks == (kvl + 15) // 16
        finally:
            pkg.lib.cml_paged_kv_cache_free(cache)


def test_paged_decode_loop_uploads_only_new_tokens_and_reuses_blocks(pkg, ob, orc, torch_dev):
    """One token appended per step with a forward after each (the decode pattern), LLaMA-sized heads;
    then the sequence is freed, its blocks go to a new sequence, and nothing of the old one leaks."""
    rng = np.random.default_rng(11)
    heads, kvh, hd, n = 8, 2, 128, 70
    k = rng.standard_normal((n, kvh * hd)).astype(np.float32)
    v = rng.standard_normal((n, kvh * hd)).astype(np.float32)
    cache = pkg.lib.cml_paged_kv_cache_create(6, 2, kvh, hd)
    try:
        s = pkg.lib.cml_paged_cache_init_sequence(cache)
        for t in range(n):
            _append(pkg, cache, s, k[t:t + 1], v[t:t + 1])
            if t % 9 == 0 or t == n - 1:
                q = rng.standard_normal((1, heads * hd)).astype(np.float32)
                want = np.empty_like(q)
                assert orc.orc_paged_gqa(ob.p(q), ob.p(k), ob.p(v), 1, t + 1, heads, kvh, hd, 0.0, 1, ob.p(want)) == 0
                assert np.abs(_forward(pkg, cache, s, q, heads, kvh, hd) - want).max() <= 2e-5
        # a 7-row query block at the end of the sequence (chunked prefill / speculative verification)
        q = rng.standard_normal((7, heads * hd)).astype(np.float32)
        want = np.empty_like(q)
        assert orc.orc_paged_gqa(ob.p(q), ob.p(k), ob.p(v), 7, n, heads, kvh, hd, 0.0, 1, ob.p(want)) == 0
        assert np.abs(_forward(pkg, cache, s, q, heads, kvh, hd) - want).max() <= 2e-5
        assert cache.contents.free_count == 1
        pkg.lib.cml_paged_cache_free_sequence(cache, s)
        assert cache.contents.free_count == 6
        s2 = pkg.lib.cml_paged_cache_init_sequence(cache)
        k2, v2 = -k[:20].copy(), v[:20][::-1].copy()
        _append(pkg, cache, s2, k2, v2)
        q = rng.standard_normal((2, heads * hd)).astype(np.float32)
        want = np.empty_like(q)
        assert orc.orc_paged_gqa(ob.p(q), ob.p(k2), ob.p(v2), 2, 20, heads, kvh, hd, 0.0, 0, ob.p(want)) == 0
        assert np.abs(_forward(pkg, cache, s2, q, heads, kvh, hd, causal=False) - want).max() <= 2e-5
    finally:
        pkg.lib.cml_paged_kv_cache_free(cache)


def test_paged_forward_error_returns(pkg, torch_dev):
    cache = pkg.lib.cml_paged_kv_cache_create(2, 2, 2, 8)
    pkg.lib.cml_set_log_level(5)
    try:
        s = pkg.lib.cml_paged_cache_init_sequence(cache)
        q = np.zeros((1, 4 * 8), np.float32)
        assert _forward(pkg, cache, s, q, 4, 2, 8) is None                      # no cached tokens
        _append(pkg, cache, s, np.ones((1, 16), np.float32), np.ones((1, 16), np.float32))
        assert _forward(pkg, cache, s, q, 3, 2, 8) is None                      # heads % kv_heads
        assert _forward(pkg, cache, s, q, 4, 1, 8) is None                      # config does not match the cache
        assert _forward(pkg, cache, 1, q, 4, 2, 8) is None                      # sequence not initialised
        got = _forward(pkg, cache, s, q, 4, 2, 8)
        assert got is not None and np.allclose(got, 1.0)                         # one key: the output is its value
        for _ in range(31):
            _append(pkg, cache, s, np.ones((1, 16), np.float32), np.ones((1, 16), np.float32))
        one = np.ones(16, np.float32)
        assert pkg.lib.cml_paged_cache_append(cache, s, pkg.np_ptr(one), pkg.np_ptr(one)) == -1    # pool exhausted
    finally:
        pkg.lib.cml_set_log_level(3)
        pkg.lib.cml_paged_kv_cache_free(cache)
