#!/usr/bin/env python
"""Benchmark of the quantized-LLM hot path on B200.

Headline workload (N = 1): the Q4_0 dequant-GEMV of LLaMA-7B's FFN-up shape, weight
11008 x 4096 in GGUF Q4_0 blocks, fp32 activation vector (M = 1), fp32 output. One "step" is one
sweep over R distinct weight copies (R x 25.4 MB > the 126 MB L2), one GEMV launch per copy,
so every launch streams its weight from HBM. metric = achieved HBM GB/s computed from the
ALGORITHMIC bytes of a launch (packed weight + x + y).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

With N > 1 (under torchrun) every rank runs the same sweep on its own GPU ("replicas only":
a standalone GEMV has nothing to exchange) and rank 0 prints the aggregate.
`--impl reference` times C-ML's own CPU path (dequantize, then its fp32 linear) on the host.
"""
import argparse
import ctypes as C
import json
import os
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
EXTRA_M = (8, 32)


def alg_bytes(M, rows=N_ROWS, cols=K_COLS):
    """Algorithmic bytes of one Q4_0 GEMV launch: packed weight (18 B per 32 weights) + x + y."""
    return rows * cols // 32 * 18 + M * cols * 4 + M * rows * 4


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return float(d["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


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


def cpu_reference_leg(budget_s=12.0):
    """C-ML's own CPU path for one 11008 x 4096 Q4_0 weight, M = 1, on the host cores: its
    loader dequantizes the blocks to fp32 once (timed separately), after which every forward is
    its fp32 linear over the resident fp32 weight (timed as the per-call cost)."""
    ob = entry.load_oracle_binding()
    synth = entry.load_synth()
    ref = ob.load_ref()
    rng = np.random.default_rng(1234)
    blocks = synth.q4_0_blocks(rng, N_ROWS, K_COLS)
    x = rng.standard_normal((1, K_COLS)).astype(np.float32)
    W = np.empty(N_ROWS * K_COLS, np.float32)
    y = np.empty((1, N_ROWS), np.float32)
    if ref is not None:
        kind = "reference"
        t0 = time.perf_counter()
        assert ref.ref_gguf_dequantize(2, ob.p(blocks), ob.p(W), W.size) == 0
        t_deq = time.perf_counter() - t0
        wt = ref.ref_weight_create(ob.p(W), N_ROWS, K_COLS)
        lin = lambda: ref.ref_linear_resident(ob.p(x), wt, 1, ob.p(y))
    else:
        kind = "port"
        orc = ob.load_orc()
        t0 = time.perf_counter()
        assert orc.orc_gguf_dequantize(2, ob.p(blocks), ob.p(W), W.size) == 0
        t_deq = time.perf_counter() - t0
        wt = None
        lin = lambda: orc.orc_linear_nt(ob.p(x), ob.p(W), 1, N_ROWS, K_COLS, ob.p(y))
    lin()
    t_lin, reps = 0.0, 0
    t_end = time.perf_counter() + budget_s
    while reps < 3 or (time.perf_counter() < t_end and reps < 500):
        t0 = time.perf_counter(); lin(); t_lin += time.perf_counter() - t0; reps += 1
    if wt:
        ref.ref_weight_free(wt)
    per_call = t_lin / reps
    return {"value": alg_bytes(1) / per_call / 1e9, "unit": "GB/s", "cores": 1, "kind": kind,
            "sample": f"{reps} x fp32 linear M=1 over the resident dequantized 11008x4096 weight "
                      f"({1e3 * per_call:.2f} ms per call, scalar path, no BLAS library on the host); "
                      f"one-time gguf_dequantize of the Q4_0 blocks took {1e3 * t_deq:.1f} ms",
            "host_cores_available": os.cpu_count(), "ms_per_call": 1e3 * per_call}


LLAMA_7B = dict(vocab=32000, hidden=4096, inter=11008, layers=32, heads=32, kv_heads=32, max_seq=1024)


def llama_leg(pkg, synth, prompt_len=512, new_tokens=128, batches=(1, 8), cfg=LLAMA_7B, tag="llama7b_q4_0"):
    """LLaMA-7B-architecture decode on one GPU: random Q4_0 weights (fp16 norms and embeddings)
    written as a GGUF file and loaded through cml_llama_load_gguf, a random 512-token prompt per
    sequence, then 128 greedy tokens generated on the device (fp16 KV cache)."""
    import tempfile
    out = {}
    rng = np.random.default_rng(99)
    with tempfile.TemporaryDirectory(prefix="cmlb200_") as tmp:
        path = os.path.join(tmp, "model.gguf")
        t0 = time.perf_counter()
        nbytes = synth.write_random_llama_gguf(path, rng, cfg)
        out[f"{tag}_gguf_bytes"] = nbytes
        out[f"{tag}_generate_s"] = time.perf_counter() - t0
        for B in batches:
            c = pkg.LlamaConfig(cfg["vocab"], cfg["hidden"], cfg["inter"], cfg["layers"], cfg["heads"], cfg["kv_heads"],
                                cfg["max_seq"], 10000.0, 1e-5, 0, 0)
            m = pkg.lib.cml_llama_create(C.byref(c))
            assert m and pkg.lib.cml_llama_set_options(m, 0, B) == 0
            t0 = time.perf_counter()
            assert pkg.lib.cml_llama_load_gguf(m, path.encode()) == 0, "cml_llama_load_gguf failed"
            out[f"{tag}_load_s_b{B}"] = time.perf_counter() - t0
            prompts = rng.integers(0, cfg["vocab"], (B, prompt_len)).astype(np.int32)
            t0 = time.perf_counter()
            for b in range(B):
                assert pkg.lib.cml_llama_prefill_sequence(m, b, pkg.np_ptr(prompts[b]), prompt_len) == 0
            out[f"{tag}_prefill_tok_s_b{B}"] = B * prompt_len / (time.perf_counter() - t0)
            first = rng.integers(0, cfg["vocab"], B).astype(np.int32)
            toks = np.zeros((new_tokens, B), np.int32)
            ms = C.c_float(0)
            assert pkg.lib.cml_llama_decode_greedy(m, pkg.np_ptr(first), B, new_tokens, pkg.np_ptr(toks), C.byref(ms)) == 0
            out[f"{tag}_decode_tok_s_b{B}"] = B * new_tokens / (ms.value * 1e-3)
            out[f"{tag}_decode_ms_per_step_b{B}"] = ms.value / new_tokens
            pkg.lib.cml_llama_free(m)
    return out


def llama_tp_leg(pkg, synth, dist, torch, dev, rank, world, prompt_len=512, new_tokens=128, cfg=LLAMA_7B, tag="llama7b_q4_0"):
    """The same LLaMA-7B-architecture decode with the weights sharded over all ranks (Q/K/V and
    gate/up by rows, attention-out and FFN-down by columns, NCCL all-reduce after the two
    row-parallel projections): batch 1, 512-token prompt, 128 greedy tokens. Every rank runs it;
    the step time is the maximum over ranks."""
    import tempfile
    out = {}
    rng = np.random.default_rng(99)
    path = os.path.join(tempfile.gettempdir(), f"cmlb200_tp_{os.environ.get('MASTER_PORT', '0')}.gguf")
    if rank == 0:
        synth.write_random_llama_gguf(path, rng, cfg)
    dist.barrier()
    try:
        ident = torch.zeros(128, dtype=torch.uint8, device=dev)
        if rank == 0:
            buf = (C.c_uint8 * 128)()
            assert pkg.lib.cml_llama_tp_unique_id(buf) == 0
            ident = torch.tensor(list(buf), dtype=torch.uint8, device=dev)
        dist.broadcast(ident, 0)
        idb = (C.c_uint8 * 128)(*ident.cpu().tolist())
        c = pkg.LlamaConfig(cfg["vocab"], cfg["hidden"], cfg["inter"], cfg["layers"], cfg["heads"], cfg["kv_heads"],
                            cfg["max_seq"], 10000.0, 1e-5, world, rank)
        m = pkg.lib.cml_llama_create(C.byref(c))
        assert m and pkg.lib.cml_llama_set_options(m, 0, 1) == 0
        assert pkg.lib.cml_llama_tp_init(m, idb, dev.index) == 0, "cml_llama_tp_init failed"
        assert pkg.lib.cml_llama_load_gguf(m, path.encode()) == 0, "cml_llama_load_gguf failed"
        prng = np.random.default_rng(7)
        prompt = prng.integers(0, cfg["vocab"], prompt_len).astype(np.int32)
        t0 = time.perf_counter()
        assert pkg.lib.cml_llama_prefill_sequence(m, 0, pkg.np_ptr(prompt), prompt_len) == 0
        torch.cuda.synchronize()
        prefill_s = time.perf_counter() - t0
        first = np.array([5], np.int32)
        toks = np.zeros((new_tokens, 1), np.int32)
        ms = C.c_float(0)
        assert pkg.lib.cml_llama_decode_greedy(m, pkg.np_ptr(first), 1, new_tokens, pkg.np_ptr(toks), C.byref(ms)) == 0
        t = torch.tensor([ms.value, prefill_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[f"{tag}_tp{world}_decode_tok_s_b1"] = new_tokens / (float(t[0]) * 1e-3)
        out[f"{tag}_tp{world}_decode_ms_per_step_b1"] = float(t[0]) / new_tokens
        out[f"{tag}_tp{world}_prefill_tok_s_b1"] = prompt_len / float(t[1])
        pkg.lib.cml_llama_free(m)
    finally:
        dist.barrier()
        if rank == 0 and os.path.exists(path):
            os.remove(path)
    return out


def run_reference(args, rank, world):
    if rank != 0:
        return
    steps_t = []
    base = None
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        base = cpu_reference_leg(budget_s=0.0)       # one bounded sample (3 calls) per step
        if i >= args.warmup:
            steps_t.append(time.perf_counter() - t0)
    v = base["value"]
    line = {"impl": "reference", "metric": "q4_0_dequant_gemv_hbm_gbs", "value": v, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * float(np.mean(steps_t)),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "Q4_0 dequant-GEMV 11008x4096, M=1 (C-ML CPU path: gguf_dequantize + fp32 linear)"},
            "cpu_baseline": base, "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU leg (profiling runs)")
    ap.add_argument("--copies", type=int, default=COPIES)
    ap.add_argument("--skip-llama", action="store_true", help="skip the LLaMA-7B decode leg")
    ap.add_argument("--profile-llama", action="store_true",
                    help="small run for ncu: 4-layer LLaMA-7B-shaped model, 512-token prefill, 6 decode steps")
    ap.add_argument("--profile-m", type=int, default=1, choices=[1, 8, 32], help="rows of x of the --profile run")
    ap.add_argument("--profile-batch", type=int, default=1, help="batch size of the --profile-llama run")
    ap.add_argument("--profile", action="store_true",
                    help="small run for ncu: plain launches (no CUDA graph), one sweep per step, headline kernel only")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return run_reference(args, rank, world)

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

    if args.profile_llama:
        cfg = dict(LLAMA_7B, layers=4)
        print(json.dumps({"profile_run": True, **llama_leg(pkg, synth, new_tokens=6, batches=(args.profile_batch,), cfg=cfg, tag="llama7b_4layers")}))
        return

    rng = np.random.default_rng(1234 + rank)
    copies = args.copies
    stream = torch.cuda.Stream(device=dev)
    sp = stream.cuda_stream
    weights, keep = [], []
    for c in range(copies):
        blocks = synth.q4_0_blocks(rng, N_ROWS, K_COLS)
        qs, sc = pkg.repack_gguf(pkg.Q4_0, blocks, N_ROWS, K_COLS)
        d_qs, d_sc = torch.from_numpy(qs).to(dev), torch.from_numpy(sc).to(dev)
        d_t = torch.from_numpy(pkg.repack_tiles(pkg.Q4_0, blocks, N_ROWS, K_COLS)).to(dev)
        keep.append((d_qs, d_sc, d_t))
        weights.append(pkg.QMat(pkg.Q4_0, N_ROWS, K_COLS, 32, d_qs.data_ptr(), d_sc.data_ptr(), 0, d_t.data_ptr()))
    x_host = {M: torch.from_numpy(rng.standard_normal((M, K_COLS)).astype(np.float32)).pin_memory() for M in (1,) + EXTRA_M}
    x_dev = {M: x_host[M].to(dev) for M in x_host}
    y_dev = {M: torch.empty((M, N_ROWS), dtype=torch.float32, device=dev) for M in x_host}
    y_host = {M: torch.empty((M, N_ROWS), dtype=torch.float32).pin_memory() for M in x_host}
    gemv = pkg.lib.cmlb200_gemv       # M <= 4: gemv_mma_kernel; above (Q4_0): x_planes_kernel + gemv_mma8_kernel per 8 rows

    def sweep(M, sweeps=SWEEPS_PER_STEP):
        xp, yp = x_dev[M].data_ptr(), y_dev[M].data_ptr()
        for _ in range(sweeps):
            for W in weights:
                pkg.check(gemv(W, xp, yp, M, sp), "cmlb200_gemv")

    def timed_plain(M, steps, warmup):
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                sweep(M, 1)
            stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                sweep(M, 1)
            e1.record(stream)
            e1.synchronize()
        return e0.elapsed_time(e1)

    if args.profile:
        ms = timed_plain(args.profile_m, args.steps, args.warmup)
        print(json.dumps({"profile_run": True, "M": args.profile_m, "launches": (args.steps + args.warmup) * copies,
                          "us_per_launch_including_host_overhead": 1e3 * ms / (args.steps * copies)}))
        return

    def timed(M, steps, warmup):
        """One step (SWEEPS_PER_STEP sweeps over all weight copies) is captured once into a CUDA
        graph and replayed, so the figure is device time, not Python launch overhead."""
        with torch.cuda.stream(stream):
            sweep(M, 1)                                   # first-use initialisation outside capture
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
                sweep(M)
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

    def e2e_timed(M, steps, warmup):
        """The call a C-ML user makes: host activations in, host result out, every launch.
        The weight stays resident (it is loaded once, as cml_llama_load_gguf does)."""
        xb = M * K_COLS * 4
        yb = M * N_ROWS * 4
        def one(W):
            pkg.check(pkg.lib.cmlb200_memcpy_h2d(x_dev[M].data_ptr(), x_host[M].data_ptr(), xb, sp))
            pkg.check(gemv(W, x_dev[M].data_ptr(), y_dev[M].data_ptr(), M, sp))
            pkg.check(pkg.lib.cmlb200_memcpy_d2h(y_host[M].data_ptr(), y_dev[M].data_ptr(), yb, sp))
            pkg.check(pkg.lib.cmlb200_stream_sync(sp))
        for _ in range(warmup):
            for W in weights:
                one(W)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            for W in weights:
                one(W)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([dt], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        return dt, xb * copies, yb * copies

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = timed(1, args.steps, args.warmup)
    timed_launches = args.steps * copies * SWEEPS_PER_STEP
    clocks = sampler.stop() if rank == 0 else None

    per_launch_s = ms * 1e-3 / timed_launches
    gbs_one = alg_bytes(1) / per_launch_s / 1e9
    value = gbs_one * world
    extra = {}
    for M in EXTRA_M:
        sM = max(1, args.steps // 8)
        msM = timed(M, sM, 3)
        extra[f"M{M}_gbs"] = alg_bytes(M) / (msM * 1e-3 / (sM * copies * SWEEPS_PER_STEP)) / 1e9 * world
    e2e_dt, h2d, d2h = e2e_timed(1, max(2, args.steps // 4), 3)
    e2e_gbs = alg_bytes(1) * copies * max(2, args.steps // 4) / e2e_dt / 1e9 * world

    if rank == 0 and world == 1 and not args.skip_llama:
        del weights, keep
        torch.cuda.empty_cache()
        try:
            extra.update(llama_leg(pkg, synth))
        except Exception as exc:                     # the GEMV headline stands on its own
            extra["llama7b_q4_0_error"] = repr(exc)[:300]
    if world > 1 and not args.skip_llama:
        del weights, keep
        torch.cuda.empty_cache()
        try:
            tp_out = llama_tp_leg(pkg, synth, dist, torch, dev, rank, world)
            if rank == 0:
                extra.update(tp_out)
        except Exception as exc:
            extra[f"llama7b_q4_0_tp{world}_error"] = repr(exc)[:300]

    if rank == 0:
        peak, peak_kind = measured_peaks()
        cpu = None if (args.no_cpu_baseline or world > 1) else cpu_reference_leg()
        line = {
            "metric": "q4_0_dequant_gemv_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "Q4_0 dequant-GEMV 11008x4096 (LLaMA-7B FFN-up), M=1, fp32 activations",
                       "launches_per_step": copies * SWEEPS_PER_STEP, "distinct_weight_copies": copies,
                       "l2_policy": f"inputs larger than L2: {copies} x 25.4 MB of distinct weights per step",
                       "parallelism": "replicas only" if world > 1 else "single GPU",
                       "pct_of_8TBps": 100.0 * gbs_one / 8000.0},
            "extra": extra,
            "roofline": {"bound": "hbm", "achieved": gbs_one, "peak": peak, "unit": "GB/s", "frac": gbs_one / peak,
                         "peak_source": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs)" if peak_kind == "measured" else "fallback 6650",
                         "traffic": 25412864,   # dram__bytes_read+write per launch, ncu capture in profiles/
                         "algorithmic_bytes_per_launch": alg_bytes(1), "us_per_launch": per_launch_s * 1e6},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_gbs, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "note": "host fp32 activations -> H2D -> GEMV -> D2H host result, synchronised per call; weights resident"},
            "gpu_launches": timed_launches,       # one kernel per call (activation digits are made inside it)
            "clocks": clocks,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
