"""The one-launch decode attention (RoPE + cache append + split attention + merge) against the
three-launch path it replaces and against a float64 computation of the same formulas
(C-ML src/nn/llm_ops.c:702-805 RoPE, :118-157 cache append, :243-372 GQA)."""
import numpy as np
import pytest
import torch

from gpu_util import stream_ptr, to_dev

pytestmark = pytest.mark.gpu


def _reference(qkv, kc, vc, seqs, pos, heads, kvh, hd, base):
    rows = qkv.shape[0]
    qw, kvw = heads * hd, kvh * hd
    out = np.zeros((rows, qw))
    i = np.arange(hd // 2)
    freq = 1.0 / np.power(float(base), 2.0 * i / hd)
    for r in range(rows):
        th = pos[r] * freq
        c, s = np.cos(th), np.sin(th)
        def rot(v):
            v = v.reshape(-1, hd // 2, 2).astype(np.float64)
            return np.stack([v[..., 0] * c - v[..., 1] * s, v[..., 0] * s + v[..., 1] * c], -1).reshape(-1, hd)
        q = rot(qkv[r, :qw])
        k_new = rot(qkv[r, qw:qw + kvw]).astype(kc.dtype).astype(np.float64)
        v_new = qkv[r, qw + kvw:].reshape(kvh, hd).astype(vc.dtype).astype(np.float64)
        K = kc[seqs[r], :pos[r] + 1].astype(np.float64).reshape(pos[r] + 1, kvh, hd).copy()
        V = vc[seqs[r], :pos[r] + 1].astype(np.float64).reshape(pos[r] + 1, kvh, hd).copy()
        K[pos[r]], V[pos[r]] = k_new, v_new
        for h in range(heads):
            kh = h // (heads // kvh)
            sc = K[:, kh] @ q[h] / np.sqrt(hd)
            p = np.exp(sc - sc.max()); p /= p.sum()
            out[r, h * hd:(h + 1) * hd] = p @ V[:, kh]
    return out


@pytest.mark.parametrize("kv_f32", [0, 1])
@pytest.mark.parametrize("heads,kvh,hd", [(8, 8, 128), (8, 2, 64), (4, 4, 32)])
def test_attention_decode_matches_unfused_path_and_formulas(pkg, torch_dev, kv_f32, heads, kvh, hd):
    rng = np.random.default_rng(31)
    rows, nseq, max_seq, base = 3, 4, 300, 10000.0
    qw, kvw = heads * hd, kvh * hd
    stride = qw + 2 * kvw
    kvt = np.float32 if kv_f32 else np.float16
    kc = rng.standard_normal((nseq, max_seq, kvw)).astype(kvt)
    vc = rng.standard_normal((nseq, max_seq, kvw)).astype(kvt)
    seqs = np.array([2, 0, 3], np.int32)
    pos = np.array([0, 77, 290], np.int32)                     # first token, mid chunk, several splits
    qkv = rng.standard_normal((rows, stride)).astype(np.float32)
    want = _reference(qkv, kc, vc, seqs, pos, heads, kvh, hd, base)
    max_limit, splits = int(pos.max()), 5
    d_seq, d_pos = to_dev(seqs, torch_dev), to_dev(pos, torch_dev)

    # one launch
    d_qkv, d_kc, d_vc = to_dev(qkv, torch_dev), to_dev(kc, torch_dev), to_dev(vc, torch_dev)
    d_out = torch.zeros((rows, qw), dtype=torch.float32, device=torch_dev)
    scratch = torch.zeros(pkg.lib.cmlb200_attention_decode_scratch_bytes(rows, heads, hd, splits), dtype=torch.uint8, device=torch_dev)
    d_cs = torch.zeros((rows, hd // 2, 2), dtype=torch.float32, device=torch_dev)
    pkg.check(pkg.lib.cmlb200_rope_table(d_pos.data_ptr(), rows, hd, base, d_cs.data_ptr(), stream_ptr()), "rope_table")
    for _ in range(2):                                         # twice: the arrival counters must come back to zero
        pkg.check(pkg.lib.cmlb200_attention_decode(d_qkv.data_ptr(), stride, d_kc.data_ptr(), d_vc.data_ptr(), d_seq.data_ptr(),
                                                   d_pos.data_ptr(), d_pos.data_ptr(), rows, heads, kvh, hd, max_seq, max_limit, kv_f32,
                                                   d_cs.data_ptr(), d_out.data_ptr(), scratch.data_ptr(), splits, stream_ptr()), "attention_decode")
    torch.cuda.synchronize()
    got = d_out.cpu().numpy()
    assert np.abs(got - want).max() / np.abs(want).max() <= 2e-3
    assert int(scratch[:16384].view(torch.int32).abs().sum()) == 0

    # three launches on fresh copies
    e_qkv, e_kc, e_vc = to_dev(qkv, torch_dev), to_dev(kc, torch_dev), to_dev(vc, torch_dev)
    e_out = torch.zeros_like(d_out)
    sc2 = torch.zeros(pkg.lib.cmlb200_attention_scratch_floats(rows, heads, hd, splits), dtype=torch.float32, device=torch_dev)
    pkg.check(pkg.lib.cmlb200_qkv_rope_append(e_qkv.data_ptr(), stride, d_seq.data_ptr(), d_pos.data_ptr(), rows, heads, kvh, hd, base, -1,
                                              e_kc.data_ptr(), e_vc.data_ptr(), max_seq, kv_f32, stream_ptr()), "qkv_rope_append")
    pkg.check(pkg.lib.cmlb200_attention_ex(e_qkv.data_ptr(), stride, e_kc.data_ptr(), e_vc.data_ptr(), d_seq.data_ptr(), d_pos.data_ptr(),
                                           rows, heads, kvh, hd, max_seq, max_limit, kv_f32, e_out.data_ptr(), None, sc2.data_ptr(), splits,
                                           stream_ptr()), "attention_ex")
    torch.cuda.synchronize()
    assert np.abs(got - e_out.cpu().numpy()).max() / np.abs(want).max() <= 1e-5
    # same cache contents (the rotation may contract its multiply-adds differently in the two kernels)
    assert torch.equal(d_vc, e_vc)
    assert torch.allclose(d_kc.float(), e_kc.float(), rtol=0, atol=2e-6 if kv_f32 else 0)


@pytest.mark.parametrize("heads,kvh,hd", [(8, 2, 128), (4, 4, 64)])
@pytest.mark.parametrize("start", [0, 37])
def test_attention_prefill_tiles_match_formulas(pkg, torch_dev, heads, kvh, hd, start):
    """The tiled tensor-core attention of prompt-sized calls (64 query rows x 64 keys per step, fp16
    operands) against a float64 softmax(Q K^T / sqrt(d)) V over the same fp16 cache: 150 rows (a
    ragged last tile) at absolute positions start .. start+149 of sequence 1, every row limited to
    its own position; fp32 and bf16 outputs. Tolerance: the bf16 prefill pipeline's 1e-2."""
    rng = np.random.default_rng(41 + start)
    rows, nseq, max_seq, seq = 150, 3, 256, 1
    qw, kvw = heads * hd, kvh * hd
    stride = qw + 2 * kvw                                      # Q sits inside a q|k|v row, as the projection leaves it
    kc = rng.standard_normal((nseq, max_seq, kvw)).astype(np.float16)
    vc = rng.standard_normal((nseq, max_seq, kvw)).astype(np.float16)
    qkv = rng.standard_normal((rows, stride)).astype(np.float32)
    limit = (start + np.arange(rows)).astype(np.int32)
    want = np.zeros((rows, qw))
    for r in range(rows):
        K = kc[seq, :limit[r] + 1].astype(np.float64).reshape(-1, kvh, hd)
        V = vc[seq, :limit[r] + 1].astype(np.float64).reshape(-1, kvh, hd)
        for h in range(heads):
            kh = h // (heads // kvh)
            sc = K[:, kh] @ qkv[r, h * hd:(h + 1) * hd].astype(np.float64) / np.sqrt(hd)
            pr = np.exp(sc - sc.max()); pr /= pr.sum()
            want[r, h * hd:(h + 1) * hd] = pr @ V[:, kh]
    d_q, d_kc, d_vc, d_lim = to_dev(qkv, torch_dev), to_dev(kc, torch_dev), to_dev(vc, torch_dev), to_dev(limit, torch_dev)
    o32 = torch.zeros((rows, qw), dtype=torch.float32, device=torch_dev)
    o16 = torch.zeros((rows, qw), dtype=torch.uint16, device=torch_dev)
    pkg.check(pkg.lib.cmlb200_attention_prefill(d_q.data_ptr(), stride, d_kc.data_ptr(), d_vc.data_ptr(), seq, d_lim.data_ptr(), rows, heads, kvh, hd,
                                                max_seq, o32.data_ptr(), o16.data_ptr(), stream_ptr()), "attention_prefill")
    torch.cuda.synchronize()
    got = o32.cpu().numpy()
    assert np.abs(got - want).max() / np.abs(want).max() <= 1e-2
    got16 = (o16.cpu().numpy().astype(np.uint32) << 16).view(np.float32)
    assert np.abs(got16 - want).max() / np.abs(want).max() <= 1e-2
    assert pkg.lib.cmlb200_attention_prefill(d_q.data_ptr(), stride, d_kc.data_ptr(), d_vc.data_ptr(), seq, d_lim.data_ptr(), rows, heads, kvh, 32,
                                             max_seq, o32.data_ptr(), None, stream_ptr()) == -1          # head_dim 32 stays on the general kernel

