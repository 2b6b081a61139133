"""Tensor-parallel LLaMA on two GPUs of one box: Q/K/V and gate/up sharded by rows, attention-out
and FFN-down by columns, NCCL all-reduce after the two row-parallel projections (C-ML
src/distributed/tensor_parallel.c:25-101, 195-260; tests/test_tensor_parallel.c:330-430). Both
ranks must produce the oracle's logits. Needs two GPUs; skipped with fewer."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
pytestmark = pytest.mark.gpu

WORKER = r'''
import os, sys, ctypes as C
import numpy as np
import torch, torch.distributed as dist
root, work = sys.argv[1], sys.argv[2]
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
cfg = llama_util.TINY
path = os.path.join(work, "tiny_tp.gguf")
store = llama_util.build(entry, np.random.default_rng(5), cfg, path if rank == 0 else os.path.join(work, f"scratch{rank}.gguf"))
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
oracle = llama_util.OracleLlama(entry, cfg, store, rope_all_heads=1, mask_absolute=1)
rng = np.random.default_rng(6)
prompt = rng.integers(0, cfg["vocab"], 9).astype(np.int32)
worst = 0.0
for toks in (prompt, np.array([7], np.int32), np.array([11], np.int32)):     # a 9-token call, then two cached single-token calls
    got = llama_util.dev_forward(pkg, m, toks)
    want = oracle.forward(toks)
    assert got is not None and want is not None
    err = float(np.abs(got - want).max() / np.abs(want).max())
    worst = max(worst, err)
    both = [None, None]
    dist.all_gather_object(both, got.tobytes())
    assert both[0] == both[1], "ranks disagree on the logits"
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
    both = [None, None]
    dist.all_gather_object(both, a.tobytes())
    assert both[0] == both[1], "ranks disagree on the batched logits"
pkg.lib.cml_llama_free(m1)
dist.barrier()
pkg.lib.cml_llama_free(m)
dist.destroy_process_group()
print(f"rank {rank} ok {worst:.2e}")
'''


@pytest.mark.parametrize("nccl_only", ["0", "1"])           # peer-memory all-reduce, then NCCL for every size
def test_two_gpu_tensor_parallel_matches_oracle(tmp_path, nccl_only):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "tp_worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", CML_B200_TP_NCCL_ONLY=nccl_only)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "2954" + nccl_only, str(script), str(ROOT), str(tmp_path)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(ROOT))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout
