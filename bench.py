#!/usr/bin/env python
"""Benchmark of the quantized decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload `decode_b1`: greedy batch-1 decode of a BitNet-b1.58-2B-4T-shaped model with
seeded synthetic ternary weights (30 layers, hidden 2560, FFN 6912, 20/5 heads, INT8 LM head
128256 x 2560, INT8 KV cache), 64-token prompt prefilled, then K generated tokens. One step = one
generated token; every step streams ~852 MB of weights (far larger than the 126 MB L2), so no
explicit L2 flush is needed between steps.

  value  tokens/s with the token fed back on the device (tenzo_ext_decode_greedy): inputs resident
         in HBM, CUDA-event timed on the engine's stream.
  e2e    tokens/s through tenzo_generate_step (the reference's own public call): host token in,
         host token out every step, wall clock between synchronisations.
  roofline  the TL1 GEMV: the model's 120 weight matrices (521 MB, HBM-cold) run back to back,
         CUDA-event timed; achieved = algorithmic bytes / time against the measured HBM peak.
  cpu_baseline  the reference's own CPU engine (compiled from its sources into oracle/_ref) on this
         box's host cores, same model, same prompt, bounded sample.

Other workloads (`gemv`, `gemm`, `attn`, `decode_batch`) measure BASELINE configs 0, 0 at 256 sequences, 2 and 3.
With N > 1 every rank decodes its own independent sequence(s) (no data-path collective).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PROMPT_LEN = 64
SEED = 0
NCU_DRAM_RATIO = 4482816 / 4461568  # measured DRAM bytes per algorithmic byte of the TL1 kernel (profiles/tl1_mma_kernel_gemv_6912x2560.md)


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled while the timed region runs (read-only query)."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.rows = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "25",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 9 for n, v in zip(names, r[5:9]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's own CPU engine, compiled into oracle/_ref
# ------------------------------------------------------------------------------------------------
def cpu_reference_decode(model, prompt, n_warm, n_steps):
    """Times n_steps greedy tokens on the host cores. Returns (tok/s, kind, cores, tokens)."""
    sys.path.insert(0, str(ROOT / "tests"))
    from helpers import OracleEngine, RefEngine
    from oracle import oracle_py as ora
    cores = os.cpu_count() or 1
    os.environ.setdefault("OMP_NUM_THREADS", str(cores))
    os.environ.setdefault("OMP_PLACES", "cores")          # the reference's own recipe (its Makefile:87)
    os.environ.setdefault("OMP_PROC_BIND", "spread")
    if ora.ref_available("fast"):
        eng, kind = RefEngine(model, max_seq_len=512, kind="fast"), "reference"
    else:
        eng, kind = OracleEngine(model, max_seq_len=512), "port"
    for t in prompt[:-1]:
        eng.prefill(int(t))
    cur = int(prompt[-1])
    for _ in range(n_warm):
        cur = eng.generate(cur, temperature=0.0, rep=1.0)
    toks = []
    t0 = time.perf_counter()
    for _ in range(n_steps):
        cur = eng.generate(cur, temperature=0.0, rep=1.0)
        toks.append(cur)
    dt = time.perf_counter() - t0
    eng.close()
    return n_steps / dt, kind, cores, toks, dt


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from tenzo_b200 import synth
    cfg = dict(synth.BITNET_2B, max_seq_len=512)
    model = synth.SyntheticModel(cfg, seed=SEED)
    prompt = synth.prompt_tokens(SEED, PROMPT_LEN, cfg["vocab_size"])
    tps, kind, cores, _, dt = cpu_reference_decode(model, prompt, args.warmup, args.steps)
    sample = f"{PROMPT_LEN - 1} prefill + {args.warmup} warm-up + {args.steps} timed greedy tokens, one sequence"
    line = {
        "impl": "reference", "metric": "decode_tokens_per_second_batch1", "value": tps, "unit": "tok/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1000.0 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "decode_b1: BitNet-2B-shaped greedy decode, 64-token prompt", "where": "host CPU cores"},
        "cpu_baseline": {"value": tps, "unit": "tok/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": tps, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# ours
# ------------------------------------------------------------------------------------------------
def dist_setup(n):
    import torch
    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def barrier_sync(world):
    import torch
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x: float, world) -> float:
    if world == 1:
        return x
    import torch
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gemv_stack_roofline(engine, model, iters, peak):
    """CUDA-event time of the model's own TL1 matrices run back to back (HBM-cold: 521 MB > L2)."""
    lib = engine.lib
    lib.tenzo_ext_bench_gemv_stack.restype = C.c_float
    lib.tenzo_ext_bench_gemv_stack.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_ulonglong)]
    n_launch = C.c_ulonglong(0)
    lib.tenzo_ext_bench_gemv_stack(engine.get_raw_handle(), 2, C.byref(n_launch))             # warm-up
    ms = lib.tenzo_ext_bench_gemv_stack(engine.get_raw_handle(), iters, C.byref(n_launch))
    if ms <= 0:
        raise RuntimeError("tenzo_ext_bench_gemv_stack failed: " + engine.last_error())
    c = model.cfg
    per_stack = 0
    for name, (n, k) in model.shapes.items():
        per_stack += n * k // 4 + 4 * n
    # activation reads: one fp32 vector per launch (q|k|v share one, gate|up share one)
    per_stack += 4 * (3 * c["hidden_size"] + c["ffn_dim"])
    per_stack *= c["num_layers"]
    launches = int(n_launch.value)
    bytes_per_launch = per_stack * iters / launches
    sec_per_launch = ms * 1e-3 / launches
    achieved = bytes_per_launch / sec_per_launch / 1e9
    return {"bound": "hbm", "kernel": "tl1_mma_kernel", "achieved": achieved, "peak": peak[0], "peak_source": peak[1],
            "unit": "GB/s", "frac": achieved / peak[0], "traffic": NCU_DRAM_RATIO * bytes_per_launch,
            "traffic_source": "ncu dram__bytes_read+write of the 6912x2560 launch with the next-matrix L2 prefetch off (4 482 816 B for "
                              "4 461 568 B algorithmic), scaled to this launch mix; with the prefetch on, ncu's cache flush between replays "
                              "counts the next matrix a second time (8.9 MB)",
            "bytes_per_launch": bytes_per_launch,
            "us_per_launch": sec_per_launch * 1e6, "launches_timed": launches}


def run_decode_b1(args):
    import torch
    from tenzo_b200 import abi, synth
    from tenzo_b200.engine import Engine
    rank, world, local = dist_setup(args.gpus)
    cfg = dict(synth.BITNET_2B, max_seq_len=512)
    model = synth.SyntheticModel(cfg, seed=SEED)
    prompt = synth.prompt_tokens(SEED, PROMPT_LEN, cfg["vocab_size"])
    eng = Engine(model.config_struct(kv_mode=args.kv_mode)).load_synthetic(model)
    greedy = abi.TenzoSampling(0.0, 0.9, 40, 1.0)

    def prefill():
        eng.reset()
        for t in prompt[:-1]:
            eng.prefill_token(int(t))

    # ---- value: device-resident loop -----------------------------------------------------------
    prefill()
    cur = int(prompt[-1])
    warm = eng.decode_greedy([cur], max(3, args.warmup))
    cur = int(warm[-1, 0])
    sampler = ClockSampler(local).start() if rank == 0 else None
    barrier_sync(world)
    l0 = eng.kernel_launches()
    toks_dev = eng.decode_greedy([cur], args.steps)
    dev_ms = eng.last_device_ms()
    barrier_sync(world)
    launches = eng.kernel_launches() - l0
    dev_ms = max_over_ranks(dev_ms, world)
    clocks = sampler.stop() if sampler else None

    # ---- e2e: the reference-facing call, host token in / out every step -----------------------------
    prefill()
    cur = int(prompt[-1])
    for _ in range(max(3, args.warmup)):
        cur = eng.generate_step(cur, greedy)
    barrier_sync(world)
    t0 = time.perf_counter()
    toks_e2e = []
    for _ in range(args.steps):
        cur = eng.generate_step(cur, greedy)
        toks_e2e.append(cur)
    eng.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier_sync(world)
    e2e_s = max_over_ranks(e2e_s, world)
    same_stream = bool(np.array_equal(np.asarray(toks_e2e), toks_dev[:, 0]))

    # ---- prompt processing: token by token (the reference's loop) against one chunk through the batched path -----
    eng.reset()
    t0 = time.perf_counter()
    for t in prompt[:-1]:
        eng.prefill_token(int(t))
    eng.synchronize()
    pf_tokens_s = time.perf_counter() - t0
    first_after_tokens = int(eng.decode_greedy([int(prompt[-1])], 1)[0, 0])
    eng.reset()
    eng.prefill_chunk(prompt[:-1])                  # warm-up (buffers, function attributes)
    eng.reset()
    t0 = time.perf_counter()
    eng.prefill_chunk(prompt[:-1])
    eng.synchronize()
    pf_chunk_s = time.perf_counter() - t0
    first_after_chunk = int(eng.decode_greedy([int(prompt[-1])], 1)[0, 0])

    roof = cpu = None
    if rank == 0:
        roof = gemv_stack_roofline(eng, model, 20, measured_peaks())
    eng.close()
    torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        n_cpu = min(args.steps, 128)
        tps, kind, cores, toks_cpu, dt = cpu_reference_decode(model, prompt, 0, n_cpu + max(3, args.warmup))
        cpu = {"value": tps, "unit": "tok/s", "cores": cores, "kind": kind,
               "sample": f"{PROMPT_LEN - 1} prefill + {n_cpu + max(3, args.warmup)} greedy tokens of the same model and prompt, one sequence, {dt:.1f} s"}
    if rank == 0:
        total = args.steps * world
        line = {
            "metric": "decode_tokens_per_second_batch1", "value": total / (dev_ms * 1e-3), "unit": "tok/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": "decode_b1: BitNet-2B-shaped greedy decode (30L, 2560/6912, 20q/5kv, INT8 LM head 128256x2560, INT8 KV), "
                                   "64-token prompt, one sequence per GPU", "l2": "inputs larger than L2 (852 MB of weights per step)",
                       "parallelism": "replicas only" if world > 1 else "single GPU", "bytes_per_token": model.weight_bytes_per_token(),
                       "kv_mode": args.kv_mode},
            "e2e": {"value": total / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 4,
                    "same_tokens_as_device_loop": same_stream},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roof, "cpu_baseline": cpu,
            "prefill": {"prompt_tokens": PROMPT_LEN - 1, "token_by_token_ms": 1e3 * pf_tokens_s, "chunked_ms": 1e3 * pf_chunk_s,
                        "same_next_token": first_after_chunk == first_after_tokens},
            "hbm_frac_whole_token": model.weight_bytes_per_token() / (dev_ms * 1e-3 / args.steps) / 1e9 / measured_peaks()[0],
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode_b1")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--pdl", type=int, default=1)
    ap.add_argument("--heads-per-cta", type=int, default=0)
    ap.add_argument("--gemm-rows", type=int, default=13824, help="gemm workload: output rows of the TL1 matrix (multiple of 128)")
    ap.add_argument("--gemm-k", type=int, default=2560, help="gemm workload: K of the TL1 matrix (multiple of 128)")
    ap.add_argument("--kv-mode", default="int8_fused", choices=["int8_fused", "paged_int8"], help="decode workloads: KV cache mode")
    ap.add_argument("--no-prefetch", action="store_true", help="gemv/gemm workloads: do not ask L2 for the next matrix (for DRAM-traffic captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.workload == "decode_b1":
        return run_decode_b1(args)
    from tenzo_b200 import bench_extra
    return bench_extra.run(args)


if __name__ == "__main__":
    main()
