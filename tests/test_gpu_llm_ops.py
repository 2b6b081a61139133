"""The stand-alone KV-cache / GQA / RoPE / tensor-parallel entry points (C-ML include/nn/llm_ops.h:13-89,
include/distributed/tensor_parallel.h:12-59) against float64 evaluations of C-ML's formulas
(src/nn/llm_ops.c:194-444, 702-805; src/distributed/tensor_parallel.c) and the oracle's RoPE / GQA."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _t(pkg, a):
    t = pkg.numpy_to_tensor(np.ascontiguousarray(a, np.float32))
    assert t
    return t


def _np(pkg, t):
    return pkg.tensor_to_numpy(t, free=False)


def _gqa_ref(q, k, v, H, KH, D, scale, causal, window, mask):
    B, SQ, _ = q.shape
    KV = k.shape[1]
    out = np.zeros((B, SQ, H * D))
    for b in range(B):
        for h in range(H):
            kh = h // (H // KH)
            qq = q[b, :, h * D:(h + 1) * D].astype(np.float64)
            kk = k[b, :, kh * D:(kh + 1) * D].astype(np.float64)
            vv = v[b, :, kh * D:(kh + 1) * D].astype(np.float64)
            s = qq @ kk.T * scale
            i, j = np.arange(SQ)[:, None], np.arange(KV)[None, :]
            if causal:
                s[j > i] = -1e9
            if window > 0:
                s[(i - j) > window] = -1e9
            if mask is not None:
                m = mask if mask.ndim == 2 else mask[b]
                s[m == 0] = -1e9
            p = np.exp(s - s.max(1, keepdims=True))
            p /= p.sum(1, keepdims=True)
            out[b, :, h * D:(h + 1) * D] = p @ vv
    return out


@pytest.mark.parametrize("H,KH,D", [(8, 2, 64), (4, 4, 32), (6, 3, 128)])
def test_gqa_forward_options(pkg, torch_dev, H, KH, D):
    rng = np.random.default_rng(41)
    B, SQ, KV = 2, 7, 19
    q = rng.standard_normal((B, SQ, H * D)).astype(np.float32)
    k = rng.standard_normal((B, KV, KH * D)).astype(np.float32)
    v = rng.standard_normal((B, KV, KH * D)).astype(np.float32)
    m2 = (rng.random((SQ, KV)) > 0.3).astype(np.float32)
    m2[3] = 0.0                                              # a fully masked row: C-ML's -1e9 gives a uniform average
    m3 = (rng.random((B, SQ, KV)) > 0.3).astype(np.float32)
    tq, tk, tv = _t(pkg, q), _t(pkg, k), _t(pkg, v)
    for scale, causal, window, mask in [(0.0, False, 0, None), (0.0, True, 0, None), (0.25, True, 3, None), (0.0, False, 0, m2),
                                        (0.0, True, 0, m3)]:
        cfg = pkg.GQAConfig(H, KH, D, scale, causal, window)
        tm = _t(pkg, mask) if mask is not None else None
        out = pkg.lib.cml_gqa_forward(tq, tk, tv, C.byref(cfg), tm)
        assert out
        got = _np(pkg, out)
        want = _gqa_ref(q, k, v, H, KH, D, scale if scale > 0 else 1.0 / np.sqrt(D), causal, window, mask)
        assert got.shape == (B, SQ, H * D)
        assert np.abs(got - want).max() <= 2e-5 * max(1.0, np.abs(want).max())
        pkg.lib.tensor_free(out)
        if tm:
            pkg.lib.tensor_free(tm)
    bad = pkg.GQAConfig(5, 2, D, 0.0, False, 0)
    assert not pkg.lib.cml_gqa_forward(tq, tk, tv, C.byref(bad), None)       # heads not divisible by kv heads
    for t in (tq, tk, tv):
        pkg.lib.tensor_free(t)


def test_kv_cache_and_cached_attention(pkg, torch_dev):
    rng = np.random.default_rng(42)
    H, KH, D, MAXS = 4, 2, 32, 12
    cache = pkg.lib.cml_kv_cache_create(MAXS, KH, D)
    assert cache and cache.contents.current_len == 0 and not pkg.lib.cml_kv_cache_get_keys(cache)
    cfg = pkg.GQAConfig(H, KH, D, 0.0, True, 0)
    ks, vs = [], []
    for step, n in enumerate((5, 1, 1)):
        q = rng.standard_normal((1, n, H * D)).astype(np.float32)
        k = rng.standard_normal((1, n, KH * D)).astype(np.float32)
        v = rng.standard_normal((1, n, KH * D)).astype(np.float32)
        ks.append(k[0]); vs.append(v[0])
        tq, tk, tv = _t(pkg, q), _t(pkg, k), _t(pkg, v)
        out = pkg.lib.cml_gqa_forward_cached(tq, tk, tv, cache, C.byref(cfg))
        assert out
        K, V = np.concatenate(ks)[None], np.concatenate(vs)[None]
        assert cache.contents.current_len == K.shape[1]
        # the causal mask is relative to this call's query index, as in C-ML
        want = _gqa_ref(q, K, V, H, KH, D, 1.0 / np.sqrt(D), True, 0, None)
        assert np.abs(_np(pkg, out) - want).max() <= 2e-5
        for t in (out, tq, tk, tv):
            pkg.lib.tensor_free(t)
    tkeys = pkg.lib.cml_kv_cache_get_keys(cache)
    assert np.array_equal(_np(pkg, tkeys).reshape(7, KH * D), np.concatenate(ks))
    pkg.lib.tensor_free(tkeys)
    big = _t(pkg, np.zeros((6, KH, D), np.float32))
    assert pkg.lib.cml_kv_cache_append(cache, big, big) == -1                  # 7 + 6 > 12
    pkg.lib.tensor_free(big)
    pkg.lib.cml_kv_cache_reset(cache)
    assert cache.contents.current_len == 0
    pkg.lib.cml_kv_cache_free(cache)


@pytest.mark.parametrize("shape", [(2, 5, 3, 16), (2, 5, 24), (6, 16)])
def test_rope_forward_shapes(pkg, ob, orc, torch_dev, shape):
    rng = np.random.default_rng(43)
    x = rng.standard_normal(shape).astype(np.float32)
    dim, base, start = 16, 10000.0, 9
    t = _t(pkg, x)
    cfg = pkg.RoPEConfig(dim, 64, base)
    r = pkg.lib.cml_rope_forward(t, start, C.byref(cfg))
    assert r and C.addressof(r.contents) == C.addressof(t.contents)             # in place, same tensor back
    got = _np(pkg, t)
    last = shape[-1]
    half = min(dim, last) // 2
    want = x.astype(np.float64).copy().reshape(-1, last)
    if len(shape) == 4:
        pos = start + (np.arange(want.shape[0]) // shape[2]) % shape[1]
    elif len(shape) == 3:
        pos = start + np.arange(want.shape[0]) % shape[1]
    else:
        pos = start + np.arange(want.shape[0])
    i = np.arange(half)
    th = pos[:, None] * (1.0 / np.power(base, 2.0 * i / dim))[None, :]
    x0, x1 = want[:, 0:2 * half:2].copy(), want[:, 1:2 * half:2].copy()
    want[:, 0:2 * half:2] = x0 * np.cos(th) - x1 * np.sin(th)
    want[:, 1:2 * half:2] = x0 * np.sin(th) + x1 * np.cos(th)
    assert np.abs(got.reshape(-1, last) - want).max() <= 1e-5
    pkg.lib.tensor_free(t)


def test_tensor_parallel_building_blocks(pkg, torch_dev):
    """Column-parallel then row-parallel over 4 ranks equals the unsharded two-layer product
    (C-ML tests/test_tensor_parallel.c:330-430), bias sharded / kept on rank 0, uneven splits refused."""
    rng = np.random.default_rng(44)
    tp, B, K, N1, N2 = 4, 3, 24, 32, 20
    x = rng.standard_normal((B, K)).astype(np.float32)
    w1 = rng.standard_normal((N1, K)).astype(np.float32); b1 = rng.standard_normal(N1).astype(np.float32)
    w2 = rng.standard_normal((N2, N1)).astype(np.float32); b2 = rng.standard_normal(N2).astype(np.float32)
    tx, tw1, tb1, tw2, tb2 = (_t(pkg, a) for a in (x, w1, b1, w2, b2))
    partials = []
    for r in range(tp):
        cp = pkg.lib.cml_column_parallel_create(tw1, tb1, tp, r)
        rp = pkg.lib.cml_row_parallel_create(tw2, tb2, tp, r)
        assert cp and rp
        assert tuple(cp.contents.weight.contents.shape[i] for i in range(2)) == (N1 // tp, K)
        assert tuple(rp.contents.weight.contents.shape[i] for i in range(2)) == (N2, N1 // tp)
        assert bool(rp.contents.bias) == (r == 0)
        h = pkg.lib.cml_column_parallel_forward(cp, tx)
        assert h
        hn = _np(pkg, h)
        assert np.abs(hn - (x.astype(np.float64) @ w1[r * 8:(r + 1) * 8].T + b1[r * 8:(r + 1) * 8])).max() <= 1e-4
        y = pkg.lib.cml_row_parallel_forward(rp, h)
        assert y
        partials.append(y)
        pkg.lib.tensor_free(h)
        pkg.lib.cml_column_parallel_free(cp)
        pkg.lib.cml_row_parallel_free(rp)
    arr = (pkg.TP * tp)(*partials)
    total = pkg.lib.cml_tp_all_reduce_sum(arr, tp)
    assert total
    want = (x.astype(np.float64) @ w1.T + b1) @ w2.T + b2
    assert np.abs(_np(pkg, total) - want).max() <= 1e-3 * np.abs(want).max()
    for t in partials + [total]:
        pkg.lib.tensor_free(t)
    assert not pkg.lib.cml_column_parallel_create(tw1, None, 5, 0)             # 32 rows over 5 ranks
    assert not pkg.lib.cml_tp_shard_weight(tw1, 2, 2, 0)                        # bad dim
    sh = pkg.lib.cml_tp_shard_weight(tw1, 1, 3, 2)                              # columns 16..23
    assert np.array_equal(_np(pkg, sh), w1[:, 16:24])
    pkg.lib.tensor_free(sh)
    for t in (tx, tw1, tb1, tw2, tb2):
        pkg.lib.tensor_free(t)


@pytest.mark.parametrize("vocab", [32000, 1001, 7])
def test_argmax_first_strict_maximum(pkg, ob, orc, torch_dev, vocab):
    """Greedy branch of cml_llama_sample_token (src/nn/llama.c:650-660): the first index of the
    strictly greatest logit; ties go to the lowest index, NaN never wins, rows are independent."""
    import torch
    rng = np.random.default_rng(vocab)
    rows = 5
    lg = rng.standard_normal((rows, vocab)).astype(np.float32)
    lg[1, [vocab - 1, vocab // 2, 3 % vocab]] = 9.0                # a three-way tie
    lg[2, :] = -np.inf                                             # nothing beats the first element
    lg[3, 0] = np.nan
    lg[3, vocab - 1] = 50.0
    lg[4, vocab - 1] = 77.0                                        # the winner in the last slice
    d = torch.from_numpy(lg).to(torch_dev)
    out = torch.full((rows,), -1, dtype=torch.int32, device=torch_dev)
    pkg.check(pkg.lib.cmlb200_argmax(d.data_ptr(), rows, vocab, out.data_ptr(), None), "cmlb200_argmax")
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    want = [orc.orc_argmax_first(ob.p(np.ascontiguousarray(lg[r])), vocab) for r in (0, 1, 2, 4)]
    assert [int(got[r]) for r in (0, 1, 2, 4)] == want
    assert int(got[1]) == min(vocab - 1, vocab // 2, 3 % vocab) and int(got[2]) == 0 and int(got[3]) == vocab - 1


@pytest.mark.parametrize("hidden", [4096, 8192, 100])
def test_embedding_gather(pkg, torch_dev, hidden):
    """embed_tokens_lookup (src/nn/llama.c:421-452): fp16 rows widened to fp32, out-of-range ids read row 0."""
    import torch
    rng = np.random.default_rng(hidden)
    vocab = 50
    table = rng.standard_normal((vocab, hidden)).astype(np.float16)
    toks = np.array([3, 49, 0, -1, 50, 7], np.int32)
    d_t, d_k = torch.from_numpy(table).to(torch_dev), torch.from_numpy(toks).to(torch_dev)
    out = torch.zeros((len(toks), hidden), dtype=torch.float32, device=torch_dev)
    pkg.check(pkg.lib.cmlb200_embed_f16(d_t.data_ptr(), d_k.data_ptr(), len(toks), hidden, vocab, out.data_ptr(), None), "cmlb200_embed_f16")
    torch.cuda.synchronize()
    idx = np.where((toks < 0) | (toks >= vocab), 0, toks)
    assert np.array_equal(out.cpu().numpy(), table[idx].astype(np.float32))



@pytest.mark.parametrize("dim", [4096, 8192, 1376, 100, 8200])
def test_rmsnorm_fp32_and_bf16_outputs(pkg, ob, orc, synth, torch_dev, dim):
    """RMSNorm (src/nn/llama.c:71-124) with an fp16 weight: the vectorised single-pass kernel (dim % 4 == 0,
    up to 8192) and the general one, fp32 output against the oracle and bf16 output as its rounding."""
    import torch
    rng = np.random.default_rng(dim)
    rows = 5
    x = (rng.standard_normal((rows, dim)) * rng.uniform(0.1, 4.0, (rows, 1))).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float16)
    want = np.empty_like(x)
    orc.orc_rmsnorm(ob.p(x), ob.p(w.astype(np.float32)), rows, dim, 1e-5, ob.p(want))
    d_x, d_w = torch.from_numpy(x).to(torch_dev), torch.from_numpy(w).to(torch_dev)
    o32 = torch.zeros((rows, dim), dtype=torch.float32, device=torch_dev)
    o16 = torch.zeros((rows, dim), dtype=torch.bfloat16, device=torch_dev)
    pkg.check(pkg.lib.cmlb200_rmsnorm(d_x.data_ptr(), d_w.data_ptr(), rows, dim, 1e-5, o32.data_ptr(), None, None), "cmlb200_rmsnorm")
    pkg.check(pkg.lib.cmlb200_rmsnorm(d_x.data_ptr(), d_w.data_ptr(), rows, dim, 1e-5, None, o16.data_ptr(), None), "cmlb200_rmsnorm")
    torch.cuda.synchronize()
    got = o32.cpu().numpy()
    assert np.abs(got - want).max() <= 2e-6 * np.abs(want).max()
    _, rounded = synth.bf16_round(got)
    assert np.array_equal(o16.float().cpu().numpy(), rounded)
