"""World-size-2 checks of the tensor-parallel host logic on CPU (gloo): sharding quantized
weights the way the loader does, column-parallel -> row-parallel -> all-reduce equals the
unsharded product (C-ML tests/test_tensor_parallel.c:330-430, 503-537), and the benchmark's
reference arm under a 2-rank launch (rank 0 prints one JSON line, the other rank exits 0)."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]

WORKER = r'''
import os, sys
import numpy as np
import torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
import __graft_entry__ as entry
pkg, synth, ob = entry.load_package(), entry.load_synth(), entry.load_oracle_binding()
orc = ob.load_orc()
dist.init_process_group("gloo")
rank, tp = dist.get_rank(), dist.get_world_size()
rng = np.random.default_rng(77)                      # same weights on every rank
M, K, N1, N = 3, 256, 512, 128
b1 = synth.q4_0_blocks(rng, N1, K)                   # column-parallel: rows split
b2 = synth.q4_0_blocks(rng, N, N1)                   # row-parallel: columns split
x = rng.standard_normal((M, K)).astype(np.float32)
s1 = np.zeros(b1.size // tp, np.uint8); s2 = np.zeros(b2.size // tp, np.uint8)
assert pkg.lib.cml_tp_shard_qblocks(2, pkg.np_ptr(b1), N1, K, 0, tp, rank, pkg.np_ptr(s1)) == 0
assert pkg.lib.cml_tp_shard_qblocks(2, pkg.np_ptr(b2), N, N1, 1, tp, rank, pkg.np_ptr(s2)) == 0
W1 = ob.dequant_blocks(orc, 2, s1, (N1 // tp) * K).reshape(N1 // tp, K)
W2 = ob.dequant_blocks(orc, 2, s2, N * (N1 // tp)).reshape(N, N1 // tp)
part = torch.from_numpy(ob.linear_nt(orc, ob.linear_nt(orc, x, W1), W2))
dist.all_reduce(part)                                # sum of the row-parallel partial outputs
F1 = ob.dequant_blocks(orc, 2, b1, N1 * K).reshape(N1, K)
F2 = ob.dequant_blocks(orc, 2, b2, N * N1).reshape(N, N1)
want = ob.linear_nt(orc, ob.linear_nt(orc, x, F1), F2)
err = np.abs(part.numpy() - want).max() / np.abs(want).max()
assert err < 1e-5, err
# the shards are exactly the reference's slices of the dequantised weight
assert np.array_equal(W1, F1[rank * (N1 // tp):(rank + 1) * (N1 // tp)])
assert np.array_equal(W2, F2[:, rank * (N1 // tp):(rank + 1) * (N1 // tp)])
dist.barrier()
dist.destroy_process_group()
import sys
sys.stdout.write("rank %d ok\n" % rank)   # one write: the two ranks share a pipe
sys.stdout.flush()
'''


def _torchrun(args, timeout=600):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29533"] + args
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=str(ROOT))


def test_shard_then_allreduce_equals_unsharded_world2(tmp_path, pkg):
    script = tmp_path / "tp_worker.py"
    script.write_text(WORKER)
    r = _torchrun([str(script), str(ROOT)])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout


def test_shard_rejects_uneven_splits(pkg, synth):
    rng = np.random.default_rng(1)
    b = synth.q4_0_blocks(rng, 6, 96)
    out = np.zeros(b.size, np.uint8)
    assert pkg.lib.cml_tp_shard_qblocks(2, pkg.np_ptr(b), 6, 96, 0, 4, 0, pkg.np_ptr(out)) == -1      # 6 rows / 4
    assert pkg.lib.cml_tp_shard_qblocks(2, pkg.np_ptr(b), 6, 96, 1, 2, 0, pkg.np_ptr(out)) == -1      # 48 columns: not whole blocks
    assert pkg.lib.cml_tp_shard_qblocks(2, pkg.np_ptr(b), 6, 96, 1, 3, 3, pkg.np_ptr(out)) == -1      # rank out of range
    assert pkg.lib.cml_tp_shard_qblocks(2, pkg.np_ptr(b), 6, 96, 2, 2, 0, pkg.np_ptr(out)) == -1      # bad dim
    assert pkg.lib.cml_tp_shard_qblocks(2, pkg.np_ptr(b), 6, 96, 1, 3, 1, pkg.np_ptr(out)) == 0
    got = out[:6 * 18].reshape(6, 18)
    assert np.array_equal(got, b.reshape(6, 3, 18)[:, 1, :])


def test_reference_arm_under_two_rank_launch():
    r = _torchrun(["bench.py", "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"])
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["cpu_baseline"]["kind"] in ("reference", "port") and d["value"] > 0
