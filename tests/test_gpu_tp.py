"""Tensor-parallel LLaMA on 2, 4 and 8 GPUs of one box: Q/K/V and gate/up sharded by rows,
attention-out and FFN-down by columns, the partial sums of the two row-parallel projections added
over all ranks (C-ML src/distributed/tensor_parallel.c:25-101, 195-260;
tests/test_tensor_parallel.c:330-430). Every rank must produce the oracle's logits, and all ranks
the same bits. Cases that need more GPUs than the box has are skipped.

Also here, on ONE GPU: the bounded waits of the peer-memory all-reduce forms are made to run
out (a peer workspace that nobody writes) and must leave a status word behind, not a hang; and the
prompt-sized all-reduce runs with all its ranks inside one cooperative launch against the sum in
rank order."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
pytestmark = pytest.mark.gpu

WORKER = r'''
import os, sys, ctypes as C
import numpy as np
import torch, torch.distributed as dist
root, work, case = sys.argv[1], sys.argv[2], sys.argv[3]
sys.path.insert(0, root); sys.path.insert(0, os.path.join(root, "tests"))
import nvidia.nccl
os.environ.setdefault("CML_NCCL_LIB", os.path.join(list(nvidia.nccl.__path__)[0], "lib", "libnccl.so.2"))
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
import __graft_entry__ as entry
import llama_util
pkg = entry.load_package()
dist.init_process_group("gloo")
rank, tp = dist.get_rank(), dist.get_world_size()
torch.cuda.set_device(rank)
# "wide": LLaMA-7B's widths on two layers. At 8 ranks the FFN shard is 11008 / 8 = 1376 columns
# (a multiple of 32 but not of 64 or 256), hidden 4096 gives every CTA of the fused projection +
# all-reduce launch more than one item, and 8 KV heads leave one per rank.
cfg = llama_util.TINY if case == "tiny" else dict(vocab=256, hidden=4096, inter=11008, layers=2, heads=32, kv_heads=8, max_seq=96)
path = os.path.join(work, "tp_model.gguf")
# weights of std 1/sqrt(hidden) keep the activations of the wide model of order one
store = llama_util.build(entry, np.random.default_rng(5), cfg, path if rank == 0 else os.path.join(work, f"scratch{rank}.gguf"),
                         wscale=0.05 if case == "tiny" else 1.0 / np.sqrt(cfg["hidden"]))
dist.barrier()
ident = torch.zeros(128, dtype=torch.uint8)
if rank == 0:
    buf = (C.c_uint8 * 128)()
    assert pkg.lib.cml_llama_tp_unique_id(buf) == 0
    ident = torch.tensor(list(buf), dtype=torch.uint8)
dist.broadcast(ident, 0)
idb = (C.c_uint8 * 128)(*ident.tolist())
c = pkg.LlamaConfig(cfg["vocab"], cfg["hidden"], cfg["inter"], cfg["layers"], cfg["heads"], cfg["kv_heads"], cfg["max_seq"],
                    10000.0, 1e-5, tp, rank)
m = pkg.lib.cml_llama_create(C.byref(c))
assert m
assert pkg.lib.cml_llama_set_options(m, pkg.KV_FP32, 4) == 0
assert pkg.lib.cml_llama_tp_init(m, idb, rank) == 0
assert pkg.lib.cml_llama_load_gguf(m, path.encode()) == 0

def same_on_all_ranks(a, what):
    got = [None] * tp
    dist.all_gather_object(got, a.tobytes())
    assert all(g == got[0] for g in got), "ranks disagree on " + what

oracle = llama_util.OracleLlama(entry, cfg, store, rope_all_heads=1, mask_absolute=1)
rng = np.random.default_rng(6)
prompt = rng.integers(0, cfg["vocab"], 9).astype(np.int32)
worst = 0.0
late = case == "tiny" and os.environ.get("CML_B200_TP_NCCL_ONLY") != "1"
if late and rank == tp - 1:
    import time
    time.sleep(6.0)        # longer than the peer kernels' bounded waits: the ranks must line up at the head of the call
for toks in (prompt, np.array([7], np.int32), np.array([11], np.int32)):     # a 9-token call, then two cached single-token calls
    got = llama_util.dev_forward(pkg, m, toks)
    want = oracle.forward(toks)
    assert got is not None and want is not None
    worst = max(worst, float(np.abs(got - want).max() / np.abs(want).max()))
    same_on_all_ranks(got, "the logits")
assert worst < 2e-3, worst
# one token for each of four sequences in one call (the projection + all-reduce launch takes four rows)
# against the same calls on an unsharded copy of the model on this GPU
c1 = pkg.LlamaConfig(cfg["vocab"], cfg["hidden"], cfg["inter"], cfg["layers"], cfg["heads"], cfg["kv_heads"], cfg["max_seq"],
                     10000.0, 1e-5, 0, 0)
m1 = pkg.lib.cml_llama_create(C.byref(c1))
assert m1 and pkg.lib.cml_llama_set_options(m1, pkg.KV_FP32, 4) == 0 and pkg.lib.cml_llama_load_gguf(m1, path.encode()) == 0
for toks in (prompt, np.array([7], np.int32), np.array([11], np.int32)):
    assert llama_util.dev_forward(pkg, m1, toks) is not None
for B in (4, 3, 2):
    toks = rng.integers(0, cfg["vocab"], B).astype(np.int32)
    t_tp = pkg.lib.cml_llama_forward_batch(m, pkg.np_ptr(toks), B)
    t_1 = pkg.lib.cml_llama_forward_batch(m1, pkg.np_ptr(toks), B)
    assert t_tp and t_1
    a, b = pkg.tensor_to_numpy(t_tp), pkg.tensor_to_numpy(t_1)
    err = float(np.abs(a - b).max() / np.abs(b).max())
    assert err < 2e-3, (B, err)
    same_on_all_ranks(a, "the batched logits")
# the greedy device loop (captured graph with the all-reduce launches inside) against the unsharded copy
first = np.array([3], np.int32)
o_tp, o_1 = np.zeros(6, np.int32), np.zeros(6, np.int32)
ms = C.c_float(0)
assert pkg.lib.cml_llama_decode_greedy(m, pkg.np_ptr(first), 1, 6, pkg.np_ptr(o_tp), C.byref(ms)) == 0
assert pkg.lib.cml_llama_decode_greedy(m1, pkg.np_ptr(first), 1, 6, pkg.np_ptr(o_1), C.byref(ms)) == 0
assert o_tp.tolist() == o_1.tolist(), (o_tp, o_1)
same_on_all_ranks(o_tp, "the greedy tokens")
# a 40-token prompt: the bf16 tensor-core path, the row-parallel projections summed over peer memory by slices
# (CML_B200_TP_BULK=1) or by ncclAllReduce (CML_B200_TP_NCCL_ONLY=1)
pkg.lib.cml_llama_reset(m)
long = rng.integers(0, cfg["vocab"], 40).astype(np.int32)
if late and rank == 0:
    import time
    time.sleep(6.0)        # the same for the prompt-sized form, with the other rank late
got = llama_util.dev_forward(pkg, m, long)
oracle2 = llama_util.OracleLlama(entry, cfg, store, rope_all_heads=1, mask_absolute=1)
want = oracle2.forward(long)
assert got is not None
err = float(np.abs(got - want).max() / np.abs(want).max())
assert err < 1e-2, err
same_on_all_ranks(got, "the prefill logits")
pkg.lib.cml_llama_free(m1)
dist.barrier()
pkg.lib.cml_llama_free(m)
dist.destroy_process_group()
print(f"rank {rank} ok {worst:.2e}")
'''


@pytest.mark.parametrize("case,ranks,nccl_only", [("tiny", 2, "0"), ("tiny", 2, "1"), ("wide", 2, "0"), ("wide", 4, "0"), ("wide", 8, "0"), ("wide", 8, "1")])
def test_tensor_parallel_matches_oracle(tmp_path, case, ranks, nccl_only):
    """nccl_only "0": decode-sized rows go through the peer-memory all-reduce (inside the GEMV launch
    where the weight allows) and prompts through its sliced form (forced on: left alone, the start-up
    timing picks between it and NCCL), "1": NCCL for every size."""
    import torch
    if torch.cuda.device_count() < ranks:
        pytest.skip(f"needs {ranks} GPUs")
    script = tmp_path / "tp_worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", CML_B200_TP_NCCL_ONLY=nccl_only, CML_B200_TP_BULK="1")
    port = 29500 + ranks * 10 + int(nccl_only) + (5 if case == "wide" else 0)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(ranks), "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(script), str(ROOT), str(tmp_path), case]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env, cwd=str(ROOT))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    for k in range(ranks):
        assert f"rank {k} ok" in r.stdout


# ---- bounded waits, on one GPU -------------------------------------------------------------------
def _workspaces(pkg, torch, dev, max_floats):
    import ctypes as C
    nbytes = pkg.lib.cmlb200_tp_ar_workspace_bytes(max_floats)
    ws = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(2)]
    arr = (C.c_void_p * 2)(ws[0].data_ptr(), ws[1].data_ptr())
    return ws, arr


def _status(pkg, ws_t):
    import ctypes as C
    st = C.c_int(-1)
    pkg.check(pkg.lib.cmlb200_tp_ar_status(ws_t.data_ptr(), C.byref(st)))
    return st.value


def test_allreduce_wait_expires_with_a_status_and_recovers(pkg, torch_dev):
    """The stand-alone all-reduce kernel with two "ranks" whose workspaces both live on this GPU and
    whose launches run one after the other. A launch whose peer has not published yet gives up
    after the (shortened) poll limit: it returns, raises status 1 + peer and leaves h alone. Because
    an expired launch has still delivered its own share, the other rank's launch of the same
    sequence number then completes, and so does the first rank's next one after the same dance:
    the protocol recovers without a reset."""
    import torch
    lib = pkg.lib
    n, max_floats = 4096, 8192
    ws, arr = _workspaces(pkg, torch, torch_dev, max_floats)
    rng = np.random.default_rng(3)
    part = [torch.from_numpy(rng.standard_normal(n).astype(np.float32)).to(torch_dev) for _ in range(2)]
    h0 = [torch.from_numpy(rng.standard_normal(n).astype(np.float32)).to(torch_dev) for _ in range(2)]
    h = [t.clone() for t in h0]
    call = lambda r: pkg.check(lib.cmlb200_tp_allreduce_add(h[r].data_ptr(), part[r].data_ptr(), n, 2, r, arr, max_floats, None))
    pkg.check(lib.cmlb200_set_wait_limit(2000))
    try:
        call(0)                                              # nobody has written rank 1's share
        torch.cuda.synchronize()
        assert _status(pkg, ws[0]) == 2 and torch.equal(h[0], h0[0])
        pkg.check(lib.cmlb200_tp_ar_status_reset(ws[0].data_ptr()))
        call(1)                                              # rank 0's share of this all-reduce is there
        torch.cuda.synchronize()
        assert _status(pkg, ws[1]) == 0
        want = h0[1] + (part[0] + part[1])
        assert torch.allclose(h[1], want, rtol=0, atol=1e-6)
        call(1)                                              # next all-reduce: rank 0 has not joined yet
        torch.cuda.synchronize()
        assert _status(pkg, ws[1]) == 1
        call(0)
        torch.cuda.synchronize()
        assert _status(pkg, ws[0]) == 0
        assert torch.allclose(h[0], h0[0] + (part[0] + part[1]), rtol=0, atol=1e-6)
    finally:
        pkg.check(lib.cmlb200_set_wait_limit(0))


def test_fused_projection_allreduce_wait_expires_with_a_status(pkg, synth, ob, orc, torch_dev):
    """The same for the all-reduce inside the row-parallel GEMV launch: no packets from the peer ->
    the launch returns, status 1 + peer, the residual untouched; once the peer's packets of that
    sequence number exist the next launch adds both shares."""
    import torch
    from gpu_util import make_weight, to_dev
    lib = pkg.lib
    N, K, M = 512, 1024, 2
    max_floats = 2 * M * N
    ws, arr = _workspaces(pkg, torch, torch_dev, max_floats)
    rng = np.random.default_rng(4)
    W, Wf, x = [], [], []
    for r in range(2):
        w, wf = make_weight(pkg, synth, ob, orc, torch_dev, rng, "q4_0", N, K)
        W.append(w); Wf.append(wf)
        x.append(rng.standard_normal((M, K)).astype(np.float32))
    assert lib.cmlb200_gemv_tp_fused_ok(W[0].q, M) == 1
    d_x = [to_dev(v, torch_dev) for v in x]
    h0 = rng.standard_normal((M, N)).astype(np.float32)
    h = [to_dev(h0, torch_dev) for _ in range(2)]
    call = lambda r: pkg.check(lib.cmlb200_gemv_tp_allreduce(W[r].q, d_x[r].data_ptr(), h[r].data_ptr(), M, 2, r, arr, max_floats, None))
    pkg.check(lib.cmlb200_set_wait_limit(2000))
    try:
        call(0)
        torch.cuda.synchronize()
        assert _status(pkg, ws[0]) == 2 and np.array_equal(h[0].cpu().numpy(), h0)
        pkg.check(lib.cmlb200_tp_ar_status_reset(ws[0].data_ptr()))
        call(1)                                              # rank 0's packets of sequence 1 are in rank 1's inbox
        torch.cuda.synchronize()
        assert _status(pkg, ws[1]) == 0
        want = h0 + ob.linear_nt(orc, x[0], Wf[0]) + ob.linear_nt(orc, x[1], Wf[1])
        assert np.abs(h[1].cpu().numpy() - want).max() <= 2e-3 * np.abs(want).max() * 1e-2
    finally:
        pkg.check(lib.cmlb200_set_wait_limit(0))


def test_bulk_allreduce_wait_expires_with_a_status(pkg, torch_dev):
    """The prompt-sized form, rank 0 of 2 launched alone: its wait for the peer's slice runs out, the
    launch returns, the status names the peer and h is as it was."""
    import ctypes as C
    import torch
    lib = pkg.lib
    n, max_floats = 1 << 16, 1 << 17
    nbytes = lib.cmlb200_tp_ar_bulk_workspace_bytes(max_floats, 2)
    ws = [torch.zeros(nbytes, dtype=torch.uint8, device=torch_dev) for _ in range(2)]
    arr = (C.c_void_p * 2)(ws[0].data_ptr(), ws[1].data_ptr())
    part = torch.ones(n, dtype=torch.float32, device=torch_dev)
    h = torch.full((n,), 3.0, dtype=torch.float32, device=torch_dev)
    pkg.check(lib.cmlb200_set_wait_limit(2000))
    try:
        pkg.check(lib.cmlb200_tp_allreduce_bulk_add(h.data_ptr(), part.data_ptr(), n, 2, 0, arr, max_floats, None))
        torch.cuda.synchronize()
        assert _status(pkg, ws[0]) == 2
        assert torch.equal(h, torch.full_like(h, 3.0))
    finally:
        pkg.check(lib.cmlb200_set_wait_limit(0))
    assert lib.cmlb200_tp_allreduce_bulk_add(h.data_ptr(), part.data_ptr(), n + 2, 2, 0, arr, max_floats, None) == -1   # n % 4
    assert lib.cmlb200_tp_allreduce_bulk_add(h.data_ptr(), part.data_ptr(), 2 * max_floats, 2, 0, arr, max_floats, None) == -1


@pytest.mark.parametrize("tp", [2, 3, 4, 8])
def test_bulk_allreduce_all_ranks_in_one_launch(pkg, torch_dev, tp):
    """All ranks of the prompt-sized all-reduce as one cooperative launch on this GPU: after every call
    each rank's h is h + (((p0 + p1) + p2) + ...) bit for bit, for message sizes that split evenly,
    raggedly, into less than one float4 per rank, and up to the workspace limit; consecutive calls
    alternate the inboxes."""
    import ctypes as C
    import torch
    lib = pkg.lib
    max_floats = 3 << 20
    nbytes = lib.cmlb200_tp_ar_bulk_workspace_bytes(max_floats, tp)
    ws = [torch.zeros(nbytes, dtype=torch.uint8, device=torch_dev) for _ in range(tp)]
    arr = (C.c_void_p * tp)(*[w.data_ptr() for w in ws])
    rng = np.random.default_rng(40 + tp)
    for n in (4, 8, 4 * 1001, 1 << 20, max_floats - 4, max_floats, 4 * 77):
        parts = [rng.standard_normal(n).astype(np.float32) for _ in range(tp)]
        h0 = [rng.standard_normal(n).astype(np.float32) for _ in range(tp)]
        d_p = [torch.from_numpy(a).to(torch_dev) for a in parts]
        d_h = [torch.from_numpy(a).to(torch_dev) for a in h0]
        pa = (C.c_void_p * tp)(*[a.data_ptr() for a in d_p])
        ha = (C.c_void_p * tp)(*[a.data_ptr() for a in d_h])
        pkg.check(lib.cmlb200_tp_allreduce_bulk_emulate(ha, pa, n, tp, arr, max_floats, None))
        torch.cuda.synchronize()
        total = np.zeros(n, np.float32)
        for a in parts:
            total = total + a
        for r in range(tp):
            assert _status(pkg, ws[r]) == 0
            assert np.array_equal(d_h[r].cpu().numpy(), h0[r] + total), (n, r)
