#!/usr/bin/env python
"""Benchmark of the quantized decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload `decode_b1`: greedy batch-1 decode of a BitNet-b1.58-2B-4T-shaped model with
seeded synthetic ternary weights (30 layers, hidden 2560, FFN 6912, 20/5 heads, INT8 LM head
128256 x 2560, INT8 KV cache), 64-token prompt prefilled, then K generated tokens. One step = one
generated token; every step streams ~852 MB of weights (far larger than the 126 MB L2), so no
explicit L2 flush is needed between steps. The K-step decode is repeated from the same state until
at least a second has been timed; the median repetition is reported (the fastest beside it).

  value     tokens/s with the token fed back on the device (tenzo_ext_decode_greedy): inputs resident
            in HBM, CUDA-event timed on the engine's stream.
  e2e       tokens/s through tenzo_generate_step (the reference's own public call): host token in,
            host token out every step, wall clock between synchronisations.
  roofline  the kernel that is the step: one persistent launch per token that reads every weight byte
            once; achieved = algorithmic bytes per token / CUDA-event time per launch against the
            measured HBM peak. `phases` breaks the launch down (GPU timer, per phase kind) and
            `tl1` gives the TL1 matrix-vector phases on their own.
  batched   the other half of the metric: global batch 256, context 4096, sharded over the launched
            ranks (strong scaling), with the attention kernel's own roofline.
  cpu_baseline  the reference's own CPU engine (compiled from its sources into oracle/_ref) on this
            box's host cores, same model, same prompt, bounded sample.

Other workloads (`gemv`, `gemm`, `attn`, `decode_batch`, `decode_tp`): single TL1 matrix-vector product, its
256-sequence form, attention alone, batched decode alone, tensor-parallel decode.
With N > 1 every rank decodes its own independent sequence (no data-path collective) for `value`.
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
WORKLOAD = ("decode_b1: BitNet-2B-shaped greedy decode (30L, 2560/6912, 20q/5kv, INT8 LM head 128256x2560, INT8 KV), "
            "64-token prompt, one sequence per GPU")
BATCHED_GLOBAL, BATCHED_CONTEXT, BATCHED_STEPS = 256, 4096, 64


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
        self.idx, self.proc, self.rows, self.t_mark = gpu_index, None, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def mark(self):
        """Samples from here on are 'under load' (the timed region starts)."""
        self.t_mark = time.perf_counter()

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = [r for t, r in self.rows if len(r) >= 9 and (self.t_mark is None or t >= self.t_mark)]
        sm = [float(r[1]) for r in rows if r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in rows if r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in rows for n, v in zip(names, r[5:9]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's own CPU engine, compiled into oracle/_ref
# ------------------------------------------------------------------------------------------------
def physical_cores() -> int:
    """Physical cores this process may run on (distinct (package, core) pairs among the allowed CPUs)."""
    allowed = os.sched_getaffinity(0) if hasattr(os, "sched_getaffinity") else set(range(os.cpu_count() or 1))
    pairs, cpu, phys = set(), None, 0
    try:
        for line in open("/proc/cpuinfo"):
            k, _, v = line.partition(":")
            k, v = k.strip(), v.strip()
            if k == "processor":
                cpu = int(v)
            elif k == "physical id":
                phys = int(v)
            elif k == "core id" and cpu in allowed:
                pairs.add((phys, int(v)))
    except OSError:
        pass
    return len(pairs) or len(allowed) or 1


def use_host_threads() -> int:
    """Give the OpenMP runtime every physical core, whatever the launcher put in the environment (torch.distributed.run
    pre-sets OMP_NUM_THREADS=1 for more than one rank), and return the thread count the runtime then reports."""
    n = physical_cores()
    os.environ["OMP_NUM_THREADS"] = str(n)
    os.environ["OMP_PLACES"] = "cores"                # the reference's own recipe (its Makefile:87)
    os.environ["OMP_PROC_BIND"] = "spread"
    try:
        omp = C.CDLL("libgomp.so.1")
        omp.omp_set_num_threads(n)                    # in case the runtime was initialised before the assignment above
        return int(omp.omp_get_max_threads())
    except OSError:
        return n


def cpu_reference_decode(model, prompt, n_warm, n_steps, context=None):
    """Times n_steps greedy tokens of one sequence on the host cores. `context`: start from a cache preset to that many
    (seeded random int8) tokens instead of prefilling the prompt. Returns (tok/s, kind, threads, tokens, seconds)."""
    sys.path.insert(0, str(ROOT / "tests"))
    from helpers import OracleEngine, RefEngine
    from oracle import oracle_py as ora
    threads = use_host_threads()
    max_seq = (context or 0) + len(prompt) + n_warm + n_steps + 8
    if context and ora.ref_available("kernels_fast"):
        eng, kind = RefEngine(model, max_seq_len=max_seq, kind="kernels_fast"), "reference"
        L, c = eng.L, model.cfg
        kv = L.refk_engine_kv(eng.h)
        rows = c["num_layers"] * c["num_kv_heads"] * max_seq
        rng = np.random.default_rng(11)
        for getter in (L.refk_kv_k, L.refk_kv_v):
            ora.view(getter(kv), rows * c["head_dim"], np.int8)[:] = rng.integers(-127, 128, rows * c["head_dim"], dtype=np.int8)
        for getter in (L.refk_kv_k_scales, L.refk_kv_v_scales):
            ora.view(getter(kv), rows, np.float32)[:] = (0.01 + 0.02 * rng.random(rows)).astype(np.float32)
        L.refk_kv_set_len(kv, int(context))
    elif ora.ref_available("fast"):
        eng, kind = RefEngine(model, max_seq_len=max_seq, kind="fast"), "reference"
    else:
        eng, kind = OracleEngine(model, max_seq_len=max_seq), "port"
    if not (context and kind == "reference" and ora.ref_available("kernels_fast")):
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
    return n_steps / dt, kind, threads, toks, dt


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from tenzo_b200 import synth
    cfg = dict(synth.BITNET_2B, max_seq_len=512)
    model = synth.SyntheticModel(cfg, seed=SEED)
    prompt = synth.prompt_tokens(SEED, PROMPT_LEN, cfg["vocab_size"])
    warm = max(3, args.warmup)
    tps, kind, threads, _, dt = cpu_reference_decode(model, prompt, warm, args.steps)
    sample = f"{PROMPT_LEN - 1} prefill + {warm} warm-up + {args.steps} timed greedy tokens, one sequence"
    line = {
        "impl": "reference", "metric": "decode_tokens_per_second_batch1", "value": tps, "unit": "tok/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": warm, "ms_per_step": 1000.0 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": WORKLOAD, "where": f"host CPU, {threads} OpenMP threads; the reference has no batch dimension and no GPU path"},
        "cpu_baseline": {"value": tps, "unit": "tok/s", "cores": threads, "kind": kind, "sample": sample},
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
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
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


def tl1_bytes_per_token(model) -> int:
    """Algorithmic bytes of the TL1 matrix-vector products of one token: packed weights + fp32 vector in and out."""
    c = model.cfg
    per_layer = sum(n * k // 4 + 4 * n for n, k in model.shapes.values()) + 4 * (3 * c["hidden_size"] + c["ffn_dim"])
    return per_layer * c["num_layers"]


def gemv_stack_roofline(engine, model, iters, peak):
    """Kernel-chain engines: CUDA-event time of the model's own TL1 matrices run back to back (HBM-cold: 521 MB > L2)."""
    lib = engine.lib
    lib.tenzo_ext_bench_gemv_stack.restype = C.c_float
    lib.tenzo_ext_bench_gemv_stack.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_ulonglong)]
    n_launch = C.c_ulonglong(0)
    lib.tenzo_ext_bench_gemv_stack(engine.get_raw_handle(), 2, C.byref(n_launch))             # warm-up
    ms = lib.tenzo_ext_bench_gemv_stack(engine.get_raw_handle(), iters, C.byref(n_launch))
    if ms <= 0:
        raise RuntimeError("tenzo_ext_bench_gemv_stack failed: " + engine.last_error())
    launches = int(n_launch.value)
    bytes_per_launch = tl1_bytes_per_token(model) * iters / launches
    sec_per_launch = ms * 1e-3 / launches
    achieved = bytes_per_launch / sec_per_launch / 1e9
    return {"bound": "hbm", "kernel": "tl1_mma_kernel", "achieved": achieved, "peak": peak[0], "peak_source": peak[1],
            "unit": "GB/s", "frac": achieved / peak[0], "traffic": 1.005 * bytes_per_launch,
            "traffic_source": "ncu dram__bytes_read+write of the 6912x2560 launch with the next-matrix L2 prefetch off: 1.005 x algorithmic",
            "bytes_per_launch": bytes_per_launch, "us_per_launch": sec_per_launch * 1e6, "launches_timed": launches}


PHASE_NAMES = ["norm_quant_qkv", "attention", "out_proj", "gate_up", "down", "final_norm_lm_head", "argmax_exit"]


def persistent_roofline(model, ms_per_token, context_mid, phases_ns, n_tokens, peak):
    """The persistent kernel IS the step: one launch per token, every weight byte read once."""
    c = model.cfg
    kv_bytes = c["num_layers"] * c["num_kv_heads"] * context_mid * (2 * c["head_dim"] + 8)
    bytes_per_launch = model.weight_bytes_per_token() + kv_bytes
    achieved = bytes_per_launch / (ms_per_token * 1e-3) / 1e9
    roof = {"bound": "hbm", "kernel": "decode_persistent_kernel", "achieved": achieved, "peak": peak[0], "peak_source": peak[1],
            "unit": "GB/s", "frac": achieved / peak[0], "traffic": None,
            "traffic_source": "no ncu capture of this kernel yet; weights are streamed once by bulk copies, no re-reads by construction",
            "bytes_per_launch": bytes_per_launch, "us_per_launch": ms_per_token * 1e3, "launches_timed": n_tokens}
    if phases_ns:
        us = [v / 1e3 / n_tokens for v in phases_ns[:7]]
        roof["phases_us_per_token"] = dict(zip(PHASE_NAMES, [round(v, 2) for v in us]))
        tl1_us = us[0] + us[2] + us[3] + us[4]
        tl1_bytes = tl1_bytes_per_token(model)
        roof["tl1"] = {"us_per_token": tl1_us, "bytes_per_token": tl1_bytes, "achieved": tl1_bytes / (tl1_us * 1e-6) / 1e9,
                       "frac": tl1_bytes / (tl1_us * 1e-6) / 1e9 / peak[0],
                       "what": "the four TL1 matrix-vector phases per layer (grid barrier, RMS sum in the reference's order, quantiser, "
                               "product), GPU global timer at the barriers"}
        lm_bytes = c["vocab_size"] * c["hidden_size"] + 4 * c["vocab_size"]
        roof["lm_head"] = {"us_per_token": us[5], "achieved": lm_bytes / (us[5] * 1e-6) / 1e9 if us[5] > 0 else None}
    return roof


def attention_roofline(B, ctx, steps, peak, mode=0):
    """The attention kernel alone at the batched block's shape (B sequences x ctx keys, 20q/5kv heads), CUDA events.
    mode 0: the reference's operation order (bit-identical); mode 1: tolerance mode (split over keys, tensor cores)."""
    import torch
    from tenzo_b200 import kernels
    nq, nkv = 20, 5
    g = torch.Generator(device="cuda").manual_seed(2)
    ck = torch.randint(-127, 128, (B, 1, nkv, ctx, 128), generator=g, device="cuda", dtype=torch.int8)
    cv = torch.randint(-127, 128, (B, 1, nkv, ctx, 128), generator=g, device="cuda", dtype=torch.int8)
    sk = 0.01 + 0.02 * torch.rand(B, 1, nkv, ctx, generator=g, device="cuda")
    sv = 0.01 + 0.02 * torch.rand(B, 1, nkv, ctx, generator=g, device="cuda")
    q = torch.randn(B, nq * 128, generator=g, device="cuda")
    k = torch.randn(B, nkv * 128, generator=g, device="cuda")
    v = torch.randn(B, nkv * 128, generator=g, device="cuda")
    pos = torch.full((B,), ctx - 1, dtype=torch.int32, device="cuda")
    ws = torch.empty(kernels.attention_workspace_bytes(B, nq, nkv, ctx), dtype=torch.uint8, device="cuda") if mode == 1 else None
    run = lambda: kernels.attention_int8(q, k, v, ck, cv, sk, sv, pos, layer=0, n_q=nq, n_kv=nkv, max_seq=ctx, max_len=ctx, mode=mode, workspace=ws)
    for _ in range(3):
        run()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    bytes_per = B * nkv * ctx * (2 * 128 + 8) + B * nq * 128 * 8
    gbs = bytes_per / (ms * 1e-3) / 1e9
    del ck, cv, sk, sv
    torch.cuda.empty_cache()
    return {"bound": "hbm", "kernel": "attn_fast_kernel (+ append, merge)" if mode == 1 else "attn_kernel", "achieved": gbs, "peak": peak[0],
            "peak_source": peak[1], "unit": "GB/s", "frac": gbs / peak[0],
            "traffic": bytes_per * (265.2 / 259.5) if mode == 0 else bytes_per * (265.6 / 259.5),
            "traffic_source": "ncu at 24 sequences x 8192 keys: 1.02 x algorithmic, scaled by the keys read" if mode == 0 else
                              "ncu at 24 sequences x 8192 keys: 259.8 MB read + 5.8 MB of partial outputs written for 259.5 MB algorithmic, scaled by the keys read",
            "bytes_per_launch": bytes_per, "us_per_launch": ms * 1e3, "launches_timed": steps,
            "l2": f"{bytes_per / 1e6:.0f} MB of KV per launch, larger than L2" if bytes_per > 130e6 else "smaller than L2: an upper bound"}


def run_batched_block(args, model, rank, world):
    """Global batch 256 x context 4096 sharded over the launched ranks (no data-path collective), 64 steps; once with the
    attention that is bit-identical to the reference (the headline) and once in tolerance mode."""
    import torch
    from tenzo_b200 import synth
    from tenzo_b200.engine import Engine
    from tenzo_b200.sharding import shard_sequences
    _, B = shard_sequences(BATCHED_GLOBAL, world, rank)
    ctx, steps, warm = BATCHED_CONTEXT, BATCHED_STEPS, 3
    peak = measured_peaks()
    out = {}
    for mode in (0, 1):
        if mode == 1 and args.kv_mode != "int8_fused":
            continue
        eng = Engine(model.config_struct(max_seq_len=(ctx + steps + warm + 8 + 3) // 4 * 4, kv_mode=args.kv_mode), batch=B,
                     attention_mode=mode).load_synthetic(model)
        eng.kv_fill_random(ctx, seed=rank)
        first = synth.prompt_tokens(1000 + rank, B, model.cfg["vocab_size"])
        w = eng.decode_greedy(first, warm)
        barrier_sync(world)
        l0 = eng.kernel_launches()
        eng.decode_greedy(w[-1], steps)
        ms = eng.last_device_ms()
        launches = eng.kernel_launches() - l0
        barrier_sync(world)
        ms = max_over_ranks(ms, world)
        eng.close()
        torch.cuda.empty_cache()
        roof = attention_roofline(B, ctx, 10, peak, mode) if rank == 0 else None
        block = {"tok_s": BATCHED_GLOBAL * steps / (ms * 1e-3), "ms_per_step": ms / steps, "gpu_launches": int(launches), "roofline": roof,
                 "attention": "reference operation order, bit-identical to the CPU engine" if mode == 0 else
                              "tolerance mode: keys split over CTAs, fp16 tensor-core products, about 1e-4 relative on the attention output"}
        if roof:
            kv_bytes_step = B * model.cfg["num_layers"] * model.cfg["num_kv_heads"] * ctx * 264
            block["attention_share_of_step"] = roof["us_per_launch"] * 1e-3 * model.cfg["num_layers"] / (ms / steps)
            block["hbm_frac_whole_step"] = (kv_bytes_step + model.weight_bytes_per_token()) / (ms / steps * 1e-3) / 1e9 / peak[0]
        out[mode] = block
    block = dict(out[0])
    block.update({"global_batch": BATCHED_GLOBAL, "context": ctx, "steps": steps, "warmup": warm, "seqs_per_gpu": B, "n_gpus": world,
                  "scaling": "strong", "parallelism": f"dp{world}: sequences sharded over the ranks, weights replicated, no data-path collective"})
    if 1 in out:
        block["tolerance_mode"] = out[1]
    return block


def run_decode_b1(args):
    import torch
    from tenzo_b200 import abi, synth
    from tenzo_b200.engine import Engine
    rank, world, local = dist_setup(args.gpus)
    sampler = ClockSampler(local).start() if rank == 0 else None      # before warm-up, so that the timed region has samples
    tp_parity = None
    if world > 1:
        from tenzo_b200 import tp
        tp_parity = tp.parity_check()                                   # the ranks the launcher started, before any timing
    cfg = dict(synth.BITNET_2B, max_seq_len=512)
    model = synth.SyntheticModel(cfg, seed=SEED)
    prompt = synth.prompt_tokens(SEED, PROMPT_LEN, cfg["vocab_size"])
    eng = Engine(model.config_struct(kv_mode=args.kv_mode), persistent=args.persistent).load_synthetic(model)
    greedy = abi.TenzoSampling(0.0, 0.9, 40, 1.0)
    warm = max(3, args.warmup)

    for t in prompt[:-1]:
        eng.prefill_token(int(t))
    start_len = eng.seq_len()

    # ---- value: device-resident loop, K steps repeated from the same state until a second has been timed --------
    first = int(prompt[-1])
    eng.decode_greedy([first], warm)
    eng.persistent_phase_ns(reset=True)
    if sampler:
        sampler.mark()
    barrier_sync(world)
    l0 = eng.kernel_launches()
    rep_ms, toks_dev, total_ms = [], None, 0.0
    while total_ms < 1000.0 or len(rep_ms) < 3:
        eng.set_seq_len(0, start_len)
        toks_dev = eng.decode_greedy([first], args.steps)
        rep_ms.append(eng.last_device_ms())
        total_ms += rep_ms[-1]
        if len(rep_ms) >= 400:
            break
    barrier_sync(world)
    launches = eng.kernel_launches() - l0
    phases = eng.persistent_phase_ns(reset=True)
    dev_ms = max_over_ranks(statistics.median(rep_ms), world)
    dev_ms_min = max_over_ranks(min(rep_ms), world)
    clocks = sampler.stop() if sampler else None

    # ---- e2e: the reference-facing call, host token in / out every step ------------------------------------------
    e2e_reps, toks_e2e, total_s = [], None, 0.0
    while total_s < 1.0 or len(e2e_reps) < 3:
        eng.set_seq_len(0, start_len)
        cur = first
        barrier_sync(world)
        t0 = time.perf_counter()
        toks_e2e = []
        for _ in range(args.steps):
            cur = eng.generate_step(cur, greedy)
            toks_e2e.append(cur)
        eng.synchronize()
        e2e_reps.append(time.perf_counter() - t0)
        total_s += e2e_reps[-1]
        if len(e2e_reps) >= 400:
            break
    e2e_s = max_over_ranks(statistics.median(e2e_reps), world)
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
    peak = measured_peaks()
    if rank == 0:
        if phases is not None:
            n_tok = len(rep_ms) * args.steps
            roof = persistent_roofline(model, dev_ms / args.steps, start_len + args.steps / 2, phases, n_tok, peak)
        else:
            roof = gemv_stack_roofline(eng, model, 20, peak)
    eng.close()
    torch.cuda.empty_cache()

    batched = None if args.no_batched else run_batched_block(args, model, rank, world)

    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        n_cpu = min(args.steps, 128)
        tps, kind, threads, toks_cpu, dt = cpu_reference_decode(model, prompt, warm, n_cpu)
        cpu = {"value": tps, "unit": "tok/s", "cores": threads, "kind": kind,
               "sample": f"{PROMPT_LEN - 1} prefill + {warm} warm-up + {n_cpu} timed greedy tokens of the same model and prompt, one sequence, {dt:.1f} s",
               "same_tokens_as_gpu": bool(kind == "port" and list(toks_cpu) == toks_dev[:n_cpu, 0].tolist()) if kind == "port" else None}
        if batched is not None:
            tps_c, kind_c, threads_c, _, dt_c = cpu_reference_decode(model, prompt, 2, 12, context=BATCHED_CONTEXT)
            batched["cpu_baseline"] = {"value": tps_c, "unit": "tok/s", "cores": threads_c, "kind": kind_c,
                                       "sample": f"ONE sequence (the reference has no batch dimension) at context {BATCHED_CONTEXT} "
                                                 f"(cache preset to seeded random int8 rows), 2 warm-up + 12 timed greedy tokens, {dt_c:.1f} s"}
    if rank == 0:
        total = args.steps * world
        line = {
            "metric": "decode_tokens_per_second_batch1", "value": total / (dev_ms * 1e-3), "unit": "tok/s",
            "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": WORKLOAD, "l2": "inputs larger than L2 (852 MB of weights per step)",
                       "parallelism": "replicas only" if world > 1 else "single GPU", "bytes_per_token": model.weight_bytes_per_token(),
                       "kv_mode": args.kv_mode, "step_kernel": "persistent" if phases is not None else "kernel chain",
                       "timed": f"{len(rep_ms)} repetitions of {args.steps} steps from the same state, median (fastest: "
                                f"{total / (dev_ms_min * 1e-3):.1f} tok/s)"},
            "e2e": {"value": total / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 4,
                    "same_tokens_as_device_loop": same_stream, "repetitions": len(e2e_reps)},
            "gpu_launches": int(launches), "clocks": clocks, "roofline": roof, "cpu_baseline": cpu,
            "prefill": {"prompt_tokens": PROMPT_LEN - 1, "token_by_token_ms": 1e3 * pf_tokens_s, "chunked_ms": 1e3 * pf_chunk_s,
                        "same_next_token": first_after_chunk == first_after_tokens},
            "hbm_frac_whole_token": model.weight_bytes_per_token() / (dev_ms * 1e-3 / args.steps) / 1e9 / peak[0],
            "batched": batched,
        }
        if tp_parity is not None:
            line["tp_parity"], line["tp_ranks"] = bool(tp_parity), world
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
    ap.add_argument("--no-batched", action="store_true", help="decode_b1: skip the batch-256 block")
    ap.add_argument("--persistent", type=int, default=-1, help="decode_b1: 1 = one persistent kernel per token, 0 = kernel chain, -1 = default")
    ap.add_argument("--attention-mode", type=int, default=0, help="decode_batch workload: 0 = exact-order attention, 1 = tolerance mode")
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--pdl", type=int, default=1)
    ap.add_argument("--heads-per-cta", type=int, default=0)
    ap.add_argument("--gemm-rows", type=int, default=13824, help="gemm workload: output rows of the TL1 matrix (multiple of 128)")
    ap.add_argument("--gemm-k", type=int, default=2560, help="gemm workload: K of the TL1 matrix (multiple of 128)")
    ap.add_argument("--gemm-epilogue", choices=["model", "store", "residual", "glu"], default="model",
                    help="gemm workload: epilogue of the call; 'model' = what the 2B layer uses for the shape (13824 rows: ReLU^2*GLU of the "
                         "gate|up halves; 2560 rows: + residual; else plain store)")
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
