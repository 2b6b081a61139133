#!/usr/bin/env python
"""Benchmark of the quantized-LLM hot path on B200.

Headline workload (N = 1): the Q4_0 dequant-GEMV of LLaMA-7B's FFN-up shape, weight
11008 x 4096 in GGUF Q4_0 blocks, fp32 activation vector (M = 1), fp32 output. One "step" is
16 sweeps over 24 distinct weight copies (24 x 25.4 MB > the 126 MB L2), one GEMV launch per copy,
so every launch streams its weight from HBM. metric = achieved HBM GB/s computed from the
ALGORITHMIC bytes of a launch (packed weight + x + y).

The same line carries, under "legs", the other configurations of the path, each with its own
roofline block: Q8_0 4096 x 4096 M=1, Q4_0 M=8 / M=32, the NF4 prefill GEMM 4096 x 4096 at
M = 64 / 512 / 2048 (tensor-core bound), LLaMA-7B Q4_0 decode (batch 1 and 8) and LLaMA-70B Q4_0
decode / prefill (batch 1 and 16), the latter tensor parallel over all ranks when N > 1.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

With N > 1 (under torchrun) every rank runs the GEMV sweep on its own GPU ("replicas only": a
standalone GEMV has nothing to exchange) and rank 0 prints the aggregate; the LLaMA legs shard
their weights over the N ranks. `--impl reference` times C-ML's own CPU path (dequantize once,
then its fp32 linear per call) on the host cores, scalar and, where an OpenBLAS is found, through
C-ML's CML_BLAS_LIB hook.
"""
import argparse
import ctypes as C
import glob
import json
import os
import re
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

N_ROWS, K_COLS = 11008, 4096
COPIES = 24                       # 24 x 25.36 MB = 609 MB of distinct weights per sweep (> L2)
SWEEPS_PER_STEP = 16              # one step = 16 sweeps = 384 GEMV launches (9.8 GB of weights)
SEED = 1234
# Identical in both arms: what is computed, on which synthetic input.
CONFIG = {"workload": "Q4_0 dequant-GEMV 11008x4096 (LLaMA-7B FFN-up), M=1, fp32 activations, fp32 accumulate, fp32 output",
          "weight": "GGUF Q4_0 blocks: nibbles uniform 0..15, fp16 scale uniform [1e-3, 2e-2]",
          "activation": "fp32 ~N(0,1), 4096 values", "seed": SEED}
LLAMA_7B = dict(vocab=32000, hidden=4096, inter=11008, layers=32, heads=32, kv_heads=32, max_seq=1024)
LLAMA_70B = dict(vocab=32000, hidden=8192, inter=28672, layers=80, heads=64, kv_heads=8, max_seq=1280)


def alg_bytes(M, rows=N_ROWS, cols=K_COLS, block_bytes=18, block_elems=32):
    """Algorithmic bytes of one GEMV launch: packed weight (18 B per 32 Q4_0 weights, 34 B per 32
    Q8_0 weights, 144 / 210 B per 256 Q4_K / Q6_K weights) + x + y."""
    return rows * cols // block_elems * block_bytes + M * cols * 4 + M * rows * 4


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d["bf16_tflops_sustained"]), "source": "measured (MEASURED_PEAKS.json)"}
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def captured_traffic(summary_name):
    """DRAM bytes per launch of a kernel, as written in its ncu summary under profiles/ (a line
    `dram_bytes_per_launch: <n>`); None when that kernel has no capture."""
    p = ROOT / "profiles" / summary_name
    if p.exists():
        m = re.search(r"dram_bytes_per_launch:\s*([0-9]+)", p.read_text())
        if m:
            return int(m.group(1))
    return None


class ClockSampler:
    """Samples the SM clock and the throttle reasons through NVML every 20 ms while the timed
    region runs (read-only queries; nothing on the GPU is changed)."""

    def __init__(self, index):
        self.index, self.sm, self.reasons, self.max_mhz = index, [], set(), None
        self._stop = threading.Event()
        self.thread = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()
        except Exception:
            self.thread = None

    def _run(self):
        nv = self.nv
        names = {nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                 nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                 nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                 nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap"}
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.02)

    def stop(self):
        if not self.thread:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"], "samples": 0}
        self._stop.set()
        self.thread.join(timeout=2)
        return {"sm_mhz": float(np.median(self.sm)) if self.sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.sm)}


# ------------------------------------------------------------------------------------------------
# CPU legs: C-ML's own code on the host cores. They run in a child process so that the BLAS hook
# (an environment variable C-ML reads when it first multiplies) can be chosen per leg and so that
# the reference arm never loads this repository's CUDA library.
def find_openblas():
    """numpy's bundled ILP64 OpenBLAS, the library C-ML's CML_BLAS_LIB hook accepts
    (src/backend/blas.c:189-200); None when there is none."""
    hits = sorted(glob.glob(os.path.join(os.path.dirname(np.__file__), "..", "numpy.libs", "libscipy_openblas64_*.so")))
    return os.path.realpath(hits[0]) if hits else None


def cpu_gemv_child(calls, steps, warmup):
    """One CPU arm of the headline workload: dequantize the Q4_0 blocks once (C-ML's loader does
    that), then time `calls` fp32 linear calls per step over the resident fp32 weight."""
    ob = entry.load_oracle_binding()
    synth = entry.load_synth()
    ref = ob.load_ref()
    rng = np.random.default_rng(SEED)
    blocks = synth.q4_0_blocks(rng, N_ROWS, K_COLS)
    x = rng.standard_normal((1, K_COLS)).astype(np.float32)
    W = np.empty(N_ROWS * K_COLS, np.float32)
    y = np.empty((1, N_ROWS), np.float32)
    t0 = time.perf_counter()
    if ref is not None:
        kind = "reference"
        assert ref.ref_gguf_dequantize(2, ob.p(blocks), ob.p(W), W.size) == 0
        t_deq = time.perf_counter() - t0
        wt = ref.ref_weight_create(ob.p(W), N_ROWS, K_COLS)
        lin = lambda: ref.ref_linear_resident(ob.p(x), wt, 1, ob.p(y))
    else:
        kind = "port"
        orc = ob.load_orc()
        assert orc.orc_gguf_dequantize(2, ob.p(blocks), ob.p(W), W.size) == 0
        t_deq = time.perf_counter() - t0
        lin = lambda: orc.orc_linear_nt(ob.p(x), ob.p(W), 1, N_ROWS, K_COLS, ob.p(y))
    lin()
    step_s = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        for _ in range(calls):
            lin()
        if i >= warmup:
            step_s.append(time.perf_counter() - t0)
    per_call = float(np.mean(step_s)) / calls
    blas = os.environ.get("CML_BLAS_LIB")
    return {"value": alg_bytes(1) / per_call / 1e9, "unit": "GB/s", "kind": kind,
            "cores": (os.cpu_count() if blas else 1), "host_cores_available": os.cpu_count(),
            "blas": os.path.basename(blas) if blas else None, "ms_per_call": 1e3 * per_call,
            "ms_per_step": 1e3 * float(np.mean(step_s)), "dequantize_once_ms": 1e3 * t_deq,
            "checksum": float(np.abs(y).sum()),
            "sample": f"{steps} steps x {calls} calls of C-ML's fp32 linear, M=1, over the resident dequantized 11008x4096 weight "
                      f"({'BLAS sgemm through CML_BLAS_LIB, all host threads' if blas else 'scalar path: no BLAS library loaded, one thread'})"}


def cpu_llama_child(steps):
    """C-ML's cml_llama_forward on the host: a 2-layer model with LLaMA-7B's layer shapes and fp32
    weights (what its loader leaves in memory), a 4-token prompt and then `steps` cached
    single-token calls; plus the vocabulary projection alone. The 32-layer figure is extrapolated:
    32 x (time of one layer) + head."""
    ob = entry.load_oracle_binding()
    ref = ob.load_ref()
    if ref is None:
        return {"unavailable": "oracle/_ref is not built"}
    cfg = dict(LLAMA_7B, layers=2, max_seq=64)
    rng = np.random.default_rng(SEED + 1)
    hd = cfg["hidden"] // cfg["heads"]
    qw = kvw = cfg["heads"] * hd
    f = lambda *s: ((rng.random(s, dtype=np.float32) - 0.5) * 0.04)
    big = f(cfg["vocab"], cfg["hidden"])                       # serves as embedding table and (same bytes) as the head
    wq, wo, wg, wd = f(cfg["hidden"], qw), f(qw, cfg["hidden"]), f(cfg["hidden"], cfg["inter"]), f(cfg["inter"], cfg["hidden"])
    n = np.ones(cfg["hidden"], np.float32)
    L = cfg["layers"]
    rc = ob.RefLlamaCfg(cfg["vocab"], cfg["hidden"], cfg["inter"], L, cfg["heads"], cfg["kv_heads"], cfg["max_seq"], 10000.0, 1e-5)
    arr = lambda a: ob.ptr_array([a] * L)
    keep = [arr(wq), arr(wq), arr(wq), arr(wo), arr(wg), arr(wg), arr(wd), arr(n), arr(n)]
    model = ref.ref_llama_create(C.byref(rc), ob.p(big), ob.p(n), ob.p(big), *keep)
    assert model
    toks = rng.integers(0, cfg["vocab"], 4 + steps).astype(np.int32)
    lg = np.empty((4, cfg["vocab"]), np.float32)
    assert ref.ref_llama_forward(model, ob.p(toks[:4]), 4, ob.p(lg)) == 0
    ts = []
    one = np.empty((1, cfg["vocab"]), np.float32)
    for i in range(steps):
        t0 = time.perf_counter()
        assert ref.ref_llama_forward(model, ob.p(toks[4 + i:5 + i]), 1, ob.p(one)) == 0
        ts.append(time.perf_counter() - t0)
    # the head alone: [vocab, hidden] fp32 linear, M = 1
    wt = ref.ref_weight_create(ob.p(big), cfg["vocab"], cfg["hidden"])
    xv = rng.standard_normal((1, cfg["hidden"])).astype(np.float32)
    ref.ref_linear_resident(ob.p(xv), wt, 1, ob.p(one))
    t0 = time.perf_counter()
    for _ in range(3):
        ref.ref_linear_resident(ob.p(xv), wt, 1, ob.p(one))
    t_head = (time.perf_counter() - t0) / 3
    t2 = float(np.median(ts))
    t_layer = max(0.0, (t2 - t_head) / L)
    t_full = 32 * t_layer + t_head
    blas = os.environ.get("CML_BLAS_LIB")
    return {"value": 1.0 / t_full, "unit": "tok/s", "kind": "reference", "extrapolated": True,
            "cores": (os.cpu_count() if blas else 1), "host_cores_available": os.cpu_count(),
            "blas": os.path.basename(blas) if blas else None,
            "ms_per_step_2_layers": 1e3 * t2, "ms_first_step": 1e3 * ts[0], "ms_head": 1e3 * t_head, "ms_per_layer": 1e3 * t_layer,
            "sample": f"cml_llama_forward, fp32 weights, 2 layers of LLaMA-7B shape + 32000-row head, batch 1, {steps} cached decode steps "
                      f"(median); 7B figure = 32 x layer + head"}


def run_cpu_leg(which, blas, **kw):
    """Runs one CPU leg in a child process (python bench.py --cpu-leg ...) and returns its dict."""
    env = dict(os.environ)
    env.pop("CML_BLAS_LIB", None)
    if blas:
        env["CML_BLAS_LIB"] = blas
    cmd = [sys.executable, str(ROOT / "bench.py"), "--cpu-leg", which] + [f"--{k.replace('_', '-')}={v}" for k, v in kw.items()]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env, timeout=900)
    for line in reversed(r.stdout.strip().splitlines()):
        if line.startswith("{"):
            return json.loads(line)
    return {"unavailable": f"child exited {r.returncode}: {(r.stderr or r.stdout)[-300:]}"}


def cpu_baselines(calls=3, steps=2, warmup=1, llama_steps=4, with_llama=True):
    """Scalar and BLAS variants of the GEMV leg (and of the LLaMA decode leg). The headline CPU
    figure is the faster GEMV variant: "all the host threads it can use"."""
    blas = find_openblas()
    out = {"gemv_scalar": run_cpu_leg("gemv", None, calls=calls, steps=steps, warmup=warmup)}
    if blas:
        out["gemv_blas"] = run_cpu_leg("gemv", blas, calls=max(calls, 10), steps=steps, warmup=warmup)
    if with_llama:
        out["llama7b_decode_scalar"] = run_cpu_leg("llama", None, llama_steps=llama_steps)
        if blas:
            out["llama7b_decode_blas"] = run_cpu_leg("llama", blas, llama_steps=2 * llama_steps)
    best = max((v for k, v in out.items() if k.startswith("gemv") and "value" in v), key=lambda v: v["value"])
    head = dict(best)
    head["variants"] = out
    return head


def run_reference(args, rank):
    """The reference arm: the unmodified C-ML CPU path for the headline workload. Rank 0 only."""
    if rank != 0:
        return
    base = cpu_baselines(calls=3, steps=args.steps, warmup=args.warmup, with_llama=not args.skip_llama)
    v = base["value"]
    line = {"impl": "reference", "metric": "q4_0_dequant_gemv_hbm_gbs", "value": v, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": CONFIG, "cpu_baseline": base,
            "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
def llama_leg(pkg, synth, torch, dist, dev, rank, world, cfg, tag, prompt_len, new_tokens, batches, peaks):
    """LLaMA decode / prefill through cml_llama_*: random Q4_0 weights (fp16 norms and embeddings)
    written as a GGUF file and loaded through cml_llama_load_gguf (tensor parallel over all ranks
    when world > 1), a random prompt per sequence prefilled with cml_llama_prefill_sequence, then
    greedy tokens generated on the device (fp16 KV cache). Times are the maximum over ranks."""
    import tempfile
    out = {}
    path = os.path.join(tempfile.gettempdir(), f"cmlb200_{tag}_{os.environ.get('MASTER_PORT', str(os.getpid()))}.gguf")
    if rank == 0:
        out["gguf_bytes"] = synth.write_random_llama_gguf(path, np.random.default_rng(99), cfg, alias_layers=True)
    if world > 1:
        dist.barrier()
    try:
        idb = None
        if world > 1:
            ident = torch.zeros(128, dtype=torch.uint8, device=dev)
            if rank == 0:
                buf = (C.c_uint8 * 128)()
                assert pkg.lib.cml_llama_tp_unique_id(buf) == 0
                ident = torch.tensor(list(buf), dtype=torch.uint8, device=dev)
            dist.broadcast(ident, 0)
            idb = (C.c_uint8 * 128)(*ident.cpu().tolist())
        hd = cfg["hidden"] // cfg["heads"]
        wbytes = cfg["layers"] * (cfg["hidden"] * hd * (cfg["heads"] + 2 * cfg["kv_heads"]) + cfg["hidden"] * cfg["heads"] * hd +
                                  3 * cfg["hidden"] * cfg["inter"]) * 18 // 32
        head_bytes = cfg["vocab"] * cfg["hidden"] * 18 // 32
        wflops = 2 * (wbytes + head_bytes) * 32 // 18                    # per token through every projection
        c = pkg.LlamaConfig(cfg["vocab"], cfg["hidden"], cfg["inter"], cfg["layers"], cfg["heads"], cfg["kv_heads"],
                            cfg["max_seq"], 10000.0, 1e-5, world if world > 1 else 0, rank if world > 1 else 0)
        m = pkg.lib.cml_llama_create(C.byref(c))
        assert m and pkg.lib.cml_llama_set_options(m, 0, max(batches)) == 0
        if world > 1:
            assert pkg.lib.cml_llama_tp_init(m, idb, dev.index) == 0, "cml_llama_tp_init failed"
            nf, pm, nm = C.c_size_t(0), C.c_float(0), C.c_float(0)
            which = pkg.lib.cml_llama_tp_prompt_allreduce(m, C.byref(nf), C.byref(pm), C.byref(nm))
            out["prompt_allreduce"] = {"used": "peer_memory" if which == 1 else "nccl", "probe_bytes": nf.value * 4,
                                       "peer_memory_ms": pm.value, "nccl_plus_add_ms": nm.value}
        t0 = time.perf_counter()
        assert pkg.lib.cml_llama_load_gguf(m, path.encode()) == 0, "cml_llama_load_gguf failed"
        out["load_s"] = time.perf_counter() - t0
        prng = np.random.default_rng(7)
        # warm-up outside the timed region: first-use set-up of every kernel and of NCCL
        warm = prng.integers(0, cfg["vocab"], min(64, prompt_len)).astype(np.int32)
        assert pkg.lib.cml_llama_prefill_sequence(m, 0, pkg.np_ptr(warm), len(warm)) == 0
        for B in batches:
            prompts = prng.integers(0, cfg["vocab"], (B, prompt_len)).astype(np.int32)
            first = prng.integers(0, cfg["vocab"], B).astype(np.int32)
            toks = np.zeros((new_tokens, B), np.int32)
            ms = C.c_float(0)
            # untimed pass with the same geometry (batch, final position): the decode loop's first call
            # captures its CUDA graph, host work that would otherwise sit inside the timed loop
            pkg.lib.cml_llama_reset(m)
            assert pkg.lib.cml_llama_prefill_sequence(m, 0, pkg.np_ptr(prompts[0]), prompt_len) == 0
            assert pkg.lib.cml_llama_decode_greedy(m, pkg.np_ptr(first), B, new_tokens, pkg.np_ptr(toks), C.byref(ms)) == 0
            pkg.lib.cml_llama_reset(m)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            t0 = time.perf_counter()
            for b in range(B):
                assert pkg.lib.cml_llama_prefill_sequence(m, b, pkg.np_ptr(prompts[b]), prompt_len) == 0
            torch.cuda.synchronize()
            prefill_s = time.perf_counter() - t0
            assert pkg.lib.cml_llama_decode_greedy(m, pkg.np_ptr(first), B, new_tokens, pkg.np_ptr(toks), C.byref(ms)) == 0
            t = torch.tensor([ms.value, prefill_s], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dec_ms, pre_s = float(t[0]), float(t[1])
            step_ms = dec_ms / new_tokens
            # bytes one decode step must read per GPU: this rank's weight shard, the head, the caches
            kv_bytes = 2 * cfg["layers"] * B * (prompt_len + new_tokens / 2) * cfg["kv_heads"] * hd * 2
            step_bytes = wbytes / world + (head_bytes / world if cfg["vocab"] % world == 0 else head_bytes) + kv_bytes / world
            out[f"decode_tok_s_b{B}"] = B * new_tokens / (dec_ms * 1e-3)
            out[f"decode_ms_per_step_b{B}"] = step_ms
            out[f"decode_roofline_b{B}"] = {"bound": "hbm", "achieved": step_bytes / (step_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                            "frac": step_bytes / (step_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "traffic": None,
                                            "algorithmic_bytes_per_step_per_gpu": step_bytes}
            out[f"prefill_tok_s_b{B}"] = B * prompt_len / pre_s
            tf = wflops * B * prompt_len / world / pre_s / 1e12
            out[f"prefill_roofline_b{B}"] = {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                                             "frac": tf / peaks["bf16_tflops_sustained"], "traffic": None,
                                             "note": "projection flops only (2 x weights per token), per GPU, wall clock of the prefill calls"}
        pkg.lib.cml_llama_free(m)
        torch.cuda.empty_cache()
    finally:
        if world > 1:
            dist.barrier()
        if rank == 0 and os.path.exists(path):
            os.remove(path)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU legs (profiling runs)")
    ap.add_argument("--copies", type=int, default=COPIES)
    ap.add_argument("--skip-llama", action="store_true", help="skip the LLaMA legs")
    ap.add_argument("--skip-70b", action="store_true", help="skip the LLaMA-70B leg")
    ap.add_argument("--profile", default=None, choices=["gemv", "gemv8", "gemm", "llama"],
                    help="small run for ncu: plain launches (no CUDA graph) of one kernel family only")
    ap.add_argument("--profile-m", type=int, default=1, help="rows of x of the --profile run")
    ap.add_argument("--profile-batch", type=int, default=1, help="batch size of --profile llama")
    ap.add_argument("--only-gemm", action="store_true", help="run the NF4 prefill-GEMM leg alone")
    ap.add_argument("--cpu-leg", default=None, choices=["gemv", "llama"], help=argparse.SUPPRESS)
    ap.add_argument("--calls", type=int, default=3, help=argparse.SUPPRESS)
    ap.add_argument("--llama-steps", type=int, default=4, help=argparse.SUPPRESS)
    args = ap.parse_args()

    if args.cpu_leg:                                   # child process of run_cpu_leg
        print(json.dumps(cpu_gemv_child(args.calls, args.steps, args.warmup) if args.cpu_leg == "gemv" else cpu_llama_child(args.llama_steps)))
        return
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return run_reference(args, rank)

    import torch
    import torch.distributed as dist
    pkg, synth = entry.load_package(), entry.load_synth()
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU fallback"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        if not os.environ.get("CML_NCCL_LIB"):      # the library's dlopen should find the NCCL torch itself uses
            try:
                import nvidia.nccl
                cand = os.path.join(list(nvidia.nccl.__path__)[0], "lib", "libnccl.so.2")
                if os.path.exists(cand):
                    os.environ["CML_NCCL_LIB"] = cand
            except ImportError:
                pass
    peaks = measured_peaks()
    stream = torch.cuda.Stream(device=dev)
    sp = stream.cuda_stream

    if args.profile == "llama":
        cfg = dict(LLAMA_7B, layers=4)
        print(json.dumps({"profile_run": True, **llama_leg(pkg, synth, torch, dist, dev, 0, 1, cfg, "llama7b_4layers", 512, 6, (args.profile_batch,), peaks)}))
        return

    def make_weights(qtype, rows, cols, copies, rng, tiles=False):
        ws, keep = [], []
        gen = synth.q4_0_blocks if qtype == pkg.Q4_0 else synth.q8_0_blocks
        for _ in range(copies):
            blocks = gen(rng, rows, cols)
            qs, sc = pkg.repack_gguf(qtype, blocks, rows, cols)
            d_qs, d_sc = torch.from_numpy(qs).to(dev), torch.from_numpy(sc).to(dev)
            d_t = torch.from_numpy(pkg.repack_tiles(qtype, blocks, rows, cols)).to(dev) if tiles else None
            keep.append((d_qs, d_sc, d_t))
            ws.append(pkg.QMat(qtype, rows, cols, 32, d_qs.data_ptr(), d_sc.data_ptr(), 0, d_t.data_ptr() if tiles else None))
        return ws, keep

    def timed_graph(enqueue_sweep, steps, warmup, sweeps=SWEEPS_PER_STEP):
        """One step (`sweeps` sweeps over all weight copies) is captured once into a CUDA graph and
        replayed, so the figure is device time, not Python launch overhead. Returns ms for `steps`."""
        with torch.cuda.stream(stream):
            enqueue_sweep()                               # first-use initialisation outside capture
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
                for _ in range(sweeps):
                    enqueue_sweep()
            for _ in range(warmup):
                graph.replay()
            stream.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                graph.replay()
            e1.record(stream)
            e1.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    gemv = pkg.lib.cmlb200_gemv

    def gemv_leg(weights, rows, cols, M, steps, warmup, block_bytes, rng, block_elems=32):
        x = torch.from_numpy(rng.standard_normal((M, cols)).astype(np.float32)).to(dev)
        y = torch.empty((M, rows), dtype=torch.float32, device=dev)

        def sweep():
            for W in weights:
                pkg.check(gemv(W, x.data_ptr(), y.data_ptr(), M, sp), "cmlb200_gemv")
        ms = timed_graph(sweep, steps, warmup)
        per_launch_s = ms * 1e-3 / (steps * len(weights) * SWEEPS_PER_STEP)
        ab = alg_bytes(M, rows, cols, block_bytes, block_elems)
        gbs = ab / per_launch_s / 1e9
        return {"us_per_call": per_launch_s * 1e6, "value": gbs, "unit": "GB/s", "pct_of_8TBps": 100.0 * gbs / 8000.0,
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                             "traffic": None, "algorithmic_bytes_per_launch": ab}}, ms

    rng = np.random.default_rng(SEED + rank)
    copies = args.copies

    if args.profile in ("gemv", "gemv8"):
        M = args.profile_m
        weights, keep = make_weights(pkg.Q4_0, N_ROWS, K_COLS, copies, rng)
        x = torch.from_numpy(rng.standard_normal((M, K_COLS)).astype(np.float32)).to(dev)
        y = torch.empty((M, N_ROWS), dtype=torch.float32, device=dev)
        with torch.cuda.stream(stream):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for i in range(args.warmup + args.steps):
                if i == args.warmup:
                    stream.synchronize()
                    e0.record(stream)
                for W in weights:
                    pkg.check(gemv(W, x.data_ptr(), y.data_ptr(), M, sp), "cmlb200_gemv")
            e1.record(stream)
            e1.synchronize()
        print(json.dumps({"profile_run": True, "M": M, "launches": (args.steps + args.warmup) * copies,
                          "us_per_call_including_host_overhead": 1e3 * e0.elapsed_time(e1) / (args.steps * copies)}))
        return

    # ---- NF4 prefill GEMM 4096 x 4096, block 64, bf16 activations (tcgen05)
    def nf4_gemm_leg(Ms, steps, warmup, ncopies=16, plain=False):
        out = {}
        N = K = 4096
        ws, keep = [], []
        for _ in range(ncopies):
            packed, scales = synth.nf4_weight(rng, N, K, 64)
            d_p, d_s = torch.from_numpy(packed).to(dev), torch.from_numpy(scales).to(dev)
            keep.append((d_p, d_s))
            ws.append(pkg.QMat(pkg.NF4, N, K, 64, d_p.data_ptr(), d_s.data_ptr(), 0, None))
        for M in Ms:
            xb, _ = synth.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
            x = torch.from_numpy(xb.reshape(M, K)).to(dev)
            y = torch.empty((M, N), dtype=torch.uint16, device=dev)

            def sweep():
                for W in ws:
                    pkg.check(pkg.lib.cmlb200_gemm_bf16(W, x.data_ptr(), y.data_ptr(), M, sp), "cmlb200_gemm_bf16")
            if plain:
                with torch.cuda.stream(stream):
                    for _ in range(warmup + steps):
                        sweep()
                    stream.synchronize()
                continue
            ms = timed_graph(sweep, steps, warmup, sweeps=4)
            per = ms * 1e-3 / (steps * ncopies * 4)
            flops = 2.0 * M * N * K
            byts = N * K // 2 + N * K // 64 * 4 + 2 * M * (K + N)
            tf = flops / per / 1e12
            t_hbm, t_tc = byts / (peaks["hbm_gbs"] * 1e9), flops / (peaks["bf16_tflops"] * 1e12)
            bound = "tensor" if t_tc >= t_hbm else "hbm"
            rl = {"bound": bound, "unit": "TFLOP/s" if bound == "tensor" else "GB/s", "traffic": None,
                  "achieved": tf if bound == "tensor" else byts / per / 1e9,
                  "peak": peaks["bf16_tflops"] if bound == "tensor" else peaks["hbm_gbs"]}
            rl["frac"] = rl["achieved"] / rl["peak"]
            rl["frac_of_sustained_bf16"] = tf / peaks["bf16_tflops_sustained"]
            rl["roofline_time_us"] = 1e6 * max(t_hbm, t_tc)
            out[f"M{M}"] = {"us_per_call": per * 1e6, "tflops": tf, "roofline": rl}
        return out

    if args.only_gemm:
        print(json.dumps({"only_gemm": True, "nf4_gemm_4096x4096_bf16": nf4_gemm_leg((64, 512, 2048), max(2, args.steps // 8), 3)}))
        return
    if args.profile == "gemm":
        nf4_gemm_leg((args.profile_m,), args.steps, args.warmup, ncopies=4, plain=True)
        print(json.dumps({"profile_run": True, "M": args.profile_m, "launches": (args.steps + args.warmup) * 4}))
        return

    # ---- headline: Q4_0 11008 x 4096, M = 1
    weights, keep = make_weights(pkg.Q4_0, N_ROWS, K_COLS, copies, rng, tiles=False)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    head, ms = gemv_leg(weights, N_ROWS, K_COLS, 1, args.steps, args.warmup, 18, rng)
    clocks = sampler.stop() if rank == 0 else None
    timed_launches = args.steps * copies * SWEEPS_PER_STEP
    gbs_one = head["value"]
    legs = {}
    few = max(2, args.steps // 8)
    for M in (8, 32):
        legs[f"q4_0_11008x4096_M{M}"], _ = gemv_leg(weights, N_ROWS, K_COLS, M, few, 3, 18, rng)

    # ---- e2e: the call a C-ML user makes: host activations in, host result out, every launch
    x_host = torch.from_numpy(rng.standard_normal((1, K_COLS)).astype(np.float32)).pin_memory()
    y_host = torch.empty((1, N_ROWS), dtype=torch.float32).pin_memory()
    x_dev = torch.empty((1, K_COLS), dtype=torch.float32, device=dev)
    y_dev = torch.empty((1, N_ROWS), dtype=torch.float32, device=dev)
    xb, yb = K_COLS * 4, N_ROWS * 4

    def e2e_one(W):                  # the library's host-buffer call: x over the bus, GEMV, y over the bus, synchronised
        pkg.check(pkg.lib.cmlb200_gemv_host(W, x_host.data_ptr(), y_host.data_ptr(), 1, sp), "cmlb200_gemv_host")

    def e2e_dma(W):                  # the same with explicit DMA copies around the device call
        pkg.check(pkg.lib.cmlb200_memcpy_h2d(x_dev.data_ptr(), x_host.data_ptr(), xb, sp))
        pkg.check(gemv(W, x_dev.data_ptr(), y_dev.data_ptr(), 1, sp))
        pkg.check(pkg.lib.cmlb200_memcpy_d2h(y_host.data_ptr(), y_dev.data_ptr(), yb, sp))
        pkg.check(pkg.lib.cmlb200_stream_sync(sp))
    e2e_steps = max(2, args.steps // 4)

    def e2e_time(one):
        for _ in range(3):
            for W in weights:
                one(W)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            for W in weights:
                one(W)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([dt], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        return alg_bytes(1) * copies * e2e_steps / dt / 1e9 * world
    e2e_dma_gbs = e2e_time(e2e_dma)
    e2e_gbs = e2e_time(e2e_one)
    # the host call must have produced the device call's result
    e2e_dma(weights[0])
    want = y_host.clone()
    y_host.zero_()
    e2e_one(weights[0])
    assert torch.equal(want, y_host), "cmlb200_gemv_host disagrees with cmlb200_gemv"
    del weights, keep
    torch.cuda.empty_cache()

    failures = []
    if rank == 0 and world == 1:
        # ---- Q8_0 4096 x 4096, M = 1 (the CPU-runnable configuration of the metric)
        w8, keep8 = make_weights(pkg.Q8_0, 4096, 4096, 24, rng)
        legs["q8_0_4096x4096_M1"], _ = gemv_leg(w8, 4096, 4096, 1, few, 3, 34, rng)
        del w8, keep8
        torch.cuda.empty_cache()
        # ---- the other GGUF block types, straight from the block stream (CUDA-core kernel)
        for gtype, tag in ((12, "q4_k"), (14, "q6_k")):
            be, bb = synth.GGUF_BLOCK[gtype]
            wk, keepk = [], []
            for _ in range(24):
                d_b = torch.from_numpy(synth.gguf_blocks(rng, gtype, 4096, 4096)).to(dev)
                keepk.append(d_b)
                wk.append(pkg.QMat(gtype, 4096, 4096, be, d_b.data_ptr(), None, 0, None))
            legs[f"{tag}_4096x4096_M1"], _ = gemv_leg(wk, 4096, 4096, 1, few, 3, bb, rng, block_elems=be)
            del wk, keepk
            torch.cuda.empty_cache()
        legs["nf4_gemm_4096x4096_bf16"] = nf4_gemm_leg((64, 512, 2048), few, 3)
        torch.cuda.empty_cache()
    if not args.skip_llama:
        plan = [("llama7b_q4_0", LLAMA_7B, 512, 128, (1, 8))]
        if not args.skip_70b:
            plan.append(("llama70b_q4_0", LLAMA_70B, 1024, 128, (1, 16)))
        for tag, cfg, plen, ntok, batches in plan:
            try:
                res = llama_leg(pkg, synth, torch, dist, dev, rank, world, cfg, tag, plen, ntok, batches, peaks)
                res["parallelism"] = f"tp{world}" if world > 1 else "single GPU"
                res["prompt_len"], res["new_tokens"] = plen, ntok
                legs[tag] = res
            except Exception as exc:                     # reported, and the run exits non-zero
                legs[tag] = {"error": repr(exc)[:300]}
                failures.append(tag)

    if rank == 0:
        cpu = None if (args.no_cpu_baseline or world > 1) else cpu_baselines(with_llama=not args.skip_llama)
        head["roofline"]["traffic"] = captured_traffic("gemv_mma_q4_0_11008x4096_m1.md")
        head["roofline"]["peak_source"] = peaks["source"]
        head["roofline"]["us_per_launch"] = head["us_per_call"]
        line = {
            "metric": "q4_0_dequant_gemv_hbm_gbs", "value": gbs_one * world, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": CONFIG,
            "detail": {"launches_per_step": copies * SWEEPS_PER_STEP, "distinct_weight_copies": copies,
                       "l2_policy": f"inputs larger than L2: {copies} x 25.4 MB of distinct weights per sweep",
                       "parallelism": "replicas only (GEMV); LLaMA legs tensor parallel" if world > 1 else "single GPU",
                       "pct_of_8TBps": 100.0 * gbs_one / 8000.0},
            "roofline": head["roofline"],
            "legs": legs,
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_gbs, "unit": "GB/s", "h2d_bytes_per_step": xb * copies, "d2h_bytes_per_step": yb * copies,
                    "note": "cmlb200_gemv_host per call: page-locked host fp32 activations read over the bus by a staging kernel, GEMV, "
                            "result written over the bus into the page-locked host buffer, stream synchronised; weights resident",
                    "with_dma_copies": e2e_dma_gbs},
            "gpu_launches": timed_launches,       # one kernel per call (activation digits are made inside it)
            "clocks": clocks,
        }
        if world > 1:
            for tag in ("llama70b_q4_0", "llama7b_q4_0"):
                if tag in legs and "error" not in legs[tag]:
                    line["tp"] = {"model": tag, "n_gpus": world, **{k: v for k, v in legs[tag].items() if k.startswith(("decode_tok_s", "prefill_tok_s", "decode_ms", "prompt_allreduce"))}}
                    break
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    if failures:
        sys.exit(f"bench.py: these legs failed: {failures}")


if __name__ == "__main__":
    main()
