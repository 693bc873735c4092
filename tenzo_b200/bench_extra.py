"""Secondary benchmark workloads (single kernels and the batched configurations), reached through `bench.py --workload`.

  gemv          one TL1 bitlinear GEMV 6912 x 2560 at batch 1, cycled over 64 distinct
                seeded matrices (283 MB, larger than L2) captured in one CUDA graph.
  gemm          its batched form: TL1 bitlinear GEMM 13824 x 2560 (gate|up of the 2B shape) for 256
                sequences on tcgen05, cycled over 16 distinct matrices (141 MB, larger than L2).
  lm_head       the INT8 LM head 128256 x 2560 + greedy argmax for one sequence (final RMSNorm + absmax quantiser fused),
                alternating between two distinct tables (657 MB, larger than L2).
  attn          fused INT8-KV GQA decode attention alone, batch 64, 20/5 heads, ctx 8192.
  decode_batch  batched greedy decode of the BitNet-2B shape, KV prefilled on the device.

  decode_tp     greedy decode of the synthetic 8B shape (32 layers, 4096/14336, 32q/8kv, vocab 128256), batch 32,
                context 2048, tensor-parallel over the launched ranks (row splits + NCCL all-gathers; tenzo_b200/tp.py).

Each prints one JSON line in the same format as the default workload.
"""
from __future__ import annotations

import json
import os

import numpy as np

from . import synth


def _peak():
    from pathlib import Path
    p = Path(__file__).resolve().parents[1] / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def _random_tl1_device(n_bytes: int, seed: int):
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    table = torch.from_numpy(synth._BYTE81).cuda()
    return table[torch.randint(0, 81, (n_bytes,), generator=g, device="cuda", dtype=torch.int64)].contiguous()


def run_gemv(args):
    import torch
    from . import kernels
    N, K, n_mat = 6912, 2560, 64
    ws = [_random_tl1_device(N * K // 4, 100 + i) for i in range(n_mat)]
    x = torch.randn(1, K, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    out = torch.empty(1, N, device="cuda")
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for w in ws[:2]:
            kernels.tl1_gemv(x, w, N // 64, K, [0.016], out=out, use_pdl=bool(args.pdl))
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i, w in enumerate(ws):      # each launch asks L2 for the next matrix, as the decode engine does
                kernels.tl1_gemv(x, w, N // 64, K, [0.016], out=out, use_pdl=bool(args.pdl), prefetch=None if args.no_prefetch else ws[(i + 1) % n_mat])
        for _ in range(max(3, args.warmup)):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        stream.synchronize()
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
    ms = e0.elapsed_time(e1)
    launches = args.steps * n_mat
    bytes_per = N * K // 4 + 4 * K + 4 * N
    gbs = bytes_per * launches / (ms * 1e-3) / 1e9
    peak = _peak()
    cpu = None if getattr(args, "no_cpu_baseline", False) else _cpu_gemv_baseline(N, K)
    print(json.dumps({
        "cpu_baseline": cpu,
        "metric": "tl1_gemv_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic", "config": {"workload": f"gemv: TL1 bitlinear {N}x{K}, batch 1, {n_mat} distinct matrices per step "
                                                    f"({n_mat * N * K // 4 / 1e6:.0f} MB > L2), one graph per step", "pdl": int(args.pdl)},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "kernel": "tl1_mma_kernel", "achieved": gbs, "peak": peak[0], "peak_source": peak[1], "unit": "GB/s",
                     "frac": gbs / peak[0], "traffic": 4482816.0, "traffic_source": "ncu dram__bytes_read+write per launch of this workload run with "
                     "--no-prefetch; with the next-matrix L2 prefetch on, ncu's cache flush between replays counts that matrix twice (8.9 MB)",
                     "bytes_per_launch": bytes_per, "us_per_launch": ms * 1e3 / launches},
    }), flush=True)


def _cpu_gemv_baseline(N, K):
    """The reference's build_lut + compute_from_lut (src/runtime/TenzoEngine.cpp:22-146, through oracle/_ref) on the host
    cores over 32 distinct seeded matrices (more than the host's last-level cache), bounded sample."""
    import sys
    import time
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    for pth in (str(root), str(root / "tests")):
        if pth not in sys.path:
            sys.path.insert(0, pth)
    import bench
    from oracle import oracle_py as ora
    threads = bench.use_host_threads()
    rng = np.random.default_rng(4)
    mats = [synth.random_tl1_packed(rng, N, K) for _ in range(32)]
    x = rng.standard_normal(K).astype(np.float32)
    out, acc = np.zeros(N, np.float32), np.zeros(N, np.int32)
    P = ora.ptr
    kind = "kernels_fast" if ora.ref_available("kernels_fast") else ("kernels" if ora.ref_available("kernels") else None)
    if kind:
        L = ora.load_ref(kind)
        one = lambda w: L.refk_bitlinear_tl1(P(x, ora.c_f32p), P(w.view(np.int8), ora.c_i8p), N, K, 0.016, P(out, ora.c_f32p), P(acc, ora.c_i32p))
    else:
        O = ora.load_oracle()
        one = lambda w: O.ora_bitlinear_tl1(P(x, ora.c_f32p), P(w, ora.c_u8p), N, K, 0.016, P(out, ora.c_f32p), P(acc, ora.c_i32p))
    one(mats[0])
    n, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < 3.0:
        one(mats[n % len(mats)])
        n += 1
    dt = time.perf_counter() - t0
    return {"value": n * (N * K // 4 + 4 * K + 4 * N) / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "reference" if kind else "port",
            "sample": f"{n} calls of the reference's TL1 product {N}x{K} cycling over 32 distinct matrices, {dt:.1f} s; {dt / n * 1e6:.0f} us per call"}


def run_lm_head(args):
    """compute_logits' int8 branch + the greedy scan (src/runtime/TenzoEngine.cpp:1634-1638, :1661-1719, :1745-1755)."""
    import torch
    from . import kernels
    V, H, n_mat, per_graph = 128256, 2560, 2, 8
    g = torch.Generator(device="cuda").manual_seed(7)
    ws = [torch.randint(-127, 128, (V, H), generator=g, device="cuda", dtype=torch.int8) for _ in range(n_mat)]
    scales = (torch.rand(V, generator=g, device="cuda") * 0.01 + 0.001).contiguous()
    norm_w = (1.0 + 0.1 * torch.randn(H, generator=g, device="cuda")).contiguous()
    x = torch.randn(1, H, generator=g, device="cuda")
    arg = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for w in ws:
            kernels.lm_head_i8_static(x, w, scales, norm_w=norm_w, argmax=arg, use_pdl=bool(args.pdl))
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(per_graph):
                kernels.lm_head_i8_static(x, ws[i % n_mat], scales, norm_w=norm_w, argmax=arg, use_pdl=bool(args.pdl))
        for _ in range(max(3, args.warmup)):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        stream.synchronize()
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
    ms = e0.elapsed_time(e1)
    calls = args.steps * per_graph
    bytes_per = V * H + 4 * V
    gbs = bytes_per * calls / (ms * 1e-3) / 1e9
    peak = _peak()
    cpu = None if getattr(args, "no_cpu_baseline", False) else _cpu_lm_head_baseline(V, H)
    print(json.dumps({
        "cpu_baseline": cpu,
        "metric": "lm_head_int8_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic", "config": {"workload": f"lm_head: INT8 LM head {V}x{H} + greedy argmax, one sequence, {per_graph} calls per step "
                                                    f"alternating between {n_mat} tables ({n_mat * V * H / 1e6:.0f} MB > L2)", "pdl": int(args.pdl)},
        "gpu_launches": 2 * calls,
        "roofline": {"bound": "hbm", "kernel": "lm_head_kernel<1> (+ argmax_finish_kernel)", "achieved": gbs, "peak": peak[0], "peak_source": peak[1],
                     "unit": "GB/s", "frac": gbs / peak[0], "traffic": 329044224.0,
                     "traffic_source": "ncu dram__bytes_read.sum of one launch inside the decode step: 1.00 x algorithmic",
                     "bytes_per_launch": bytes_per, "us_per_launch": ms * 1e3 / calls},
    }), flush=True)


def _cpu_lm_head_baseline(V, H):
    """The restated int8 LM head (oracle: TenzoEngine.cpp:1688-1718) on the host cores, alternating between two tables
    (more than the host's last-level cache), bounded sample. The reference has no kernel-level entry for it."""
    import sys
    import time
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    for pth in (str(root), str(root / "tests")):
        if pth not in sys.path:
            sys.path.insert(0, pth)
    import bench
    from oracle import oracle_py as ora
    threads = bench.use_host_threads()
    rng = np.random.default_rng(5)
    ws = [rng.integers(-127, 128, (V, H), dtype=np.int8) for _ in range(2)]
    scales = (rng.random(V) * 0.01 + 0.001).astype(np.float32)
    x8 = rng.integers(-127, 128, H, dtype=np.int8)
    logits = np.zeros(V, np.float32)
    O, P = ora.load_oracle(), ora.ptr
    one = lambda w: O.ora_lm_head_i8(P(x8, ora.c_i8p), 0.01, P(w, ora.c_i8p), P(scales, ora.c_f32p), V, H, P(logits, ora.c_f32p), None)
    one(ws[0])
    n, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < 3.0:
        one(ws[n % 2])
        n += 1
    dt = time.perf_counter() - t0
    return {"value": n * (V * H + 4 * V) / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{n} calls of the restated int8 LM head {V}x{H} alternating between 2 tables, {dt:.1f} s; {dt / n * 1e3:.1f} ms per call"}


def _peak_tensor():
    from pathlib import Path
    p = Path(__file__).resolve().parents[1] / "MEASURED_PEAKS.json"
    if p.exists():
        return 2.0 * float(json.loads(p.read_text())["bf16_tflops"]), "2 x measured bf16 burst (int8 is twice bf16 on this part; no int8 GEMM peak was measured)"
    return 2.0 * 1590.0, "2 x fallback bf16"


def _int8_library_peak():
    """A library int8 GEMM (torch._int_mm, 8192^3, best of 10, CUDA events) as the tensor peak this GPU gives int8 - a
    measurement of the denominator, like the bf16 figure of the peaks file; nothing on the decode path calls it."""
    import torch
    n = 8192
    a = torch.randint(-127, 128, (n, n), device="cuda", dtype=torch.int8)
    b = torch.randint(-127, 128, (n, n), device="cuda", dtype=torch.int8)
    try:
        torch._int_mm(a, b)
    except Exception:
        return None
    best = None
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        torch._int_mm(a, b)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        best = ms if best is None or ms < best else best
    return 2.0 * n ** 3 / (best * 1e-3) / 1e12


def run_gemm(args):
    import torch
    from . import kernels
    N, K = args.gemm_rows, args.gemm_k
    n_mat = max(16, min(128, (160 << 20) // (N * K // 4) + 1))     # distinct matrices per step: more bytes than L2 holds
    B = args.batch
    epi = getattr(args, "gemm_epilogue", "model")
    if epi == "model":                                   # what the 2B layer does with a matrix of this height
        epi = "glu" if N == 13824 else "residual" if N == 2560 else "store"
    epilogue = {"store": kernels.EPI_STORE, "residual": kernels.EPI_RESIDUAL, "glu": kernels.EPI_RELU2_GLU}[epi]
    ws = [_random_tl1_device(N * K // 4, 200 + i) for i in range(n_mat)]
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(B, K, device="cuda", generator=g)
    norm_w = 1.0 + 0.1 * torch.randn(K, device="cuda", generator=g)      # every TL1 product of the layer has an RMSNorm in front
    n_out = N // 2 if epi == "glu" else N
    out = torch.empty(B, n_out, device="cuda")
    resid = torch.randn(B, n_out, device="cuda", generator=g) if epi == "residual" else None
    call = dict(epilogue=epilogue, resid=resid, norm_w=norm_w, do_norm=True, out=out, use_pdl=bool(args.pdl))
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for w in ws[:2]:
            kernels.tl1_gemv(x, w, N // 64, K, [0.016], **call)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i, w in enumerate(ws):
                kernels.tl1_gemv(x, w, N // 64, K, [0.016], prefetch=None if args.no_prefetch else ws[(i + 1) % n_mat], **call)
        for _ in range(max(3, args.warmup)):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        stream.synchronize()
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
    ms = e0.elapsed_time(e1)
    calls = args.steps * n_mat
    tops = 2.0 * N * K * B * calls / (ms * 1e-3) / 1e12
    peak = _peak_tensor()
    lib_int8 = _int8_library_peak()
    if lib_int8:
        peak = (lib_int8, "measured: torch._int_mm 8192^3 int8 -> int32, best of 10")
    print(json.dumps({
        "metric": "tl1_gemm_tops", "value": tops, "unit": "TOP/s", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8 x s8 -> s32",
        "data": "synthetic", "config": {"workload": f"gemm: TL1 bitlinear {N}x{K} for {B} sequences (RMSNorm + absmax quantiser, tcgen05 GEMM, {epi} epilogue), "
                                                    f"{n_mat} distinct matrices per step ({n_mat * N * K // 4 / 1e6:.0f} MB > L2)", "pdl": int(args.pdl)},
        "gpu_launches": 2 * calls,
        "roofline": {"bound": "tensor", "kernel": "act_quant_kernel + tl1_umma_kernel", "achieved": tops, "peak": peak[0], "peak_source": peak[1],
                     "unit": "TOP/s", "frac": tops / peak[0], "traffic": None, "ops_per_launch": 2.0 * N * K * B, "us_per_launch": ms * 1e3 / calls},
    }), flush=True)


def run_attn(args):
    import torch
    from . import kernels
    B, nq, nkv, T = args.batch if args.batch != 256 else 64, 20, 5, args.context if args.context != 4096 else 8192
    g = torch.Generator(device="cuda").manual_seed(2)
    ck = torch.randint(-127, 128, (B, 1, nkv, T, 128), generator=g, device="cuda", dtype=torch.int8)
    cv = torch.randint(-127, 128, (B, 1, nkv, T, 128), generator=g, device="cuda", dtype=torch.int8)
    sk = 0.01 + 0.02 * torch.rand(B, 1, nkv, T, generator=g, device="cuda")
    sv = 0.01 + 0.02 * torch.rand(B, 1, nkv, T, generator=g, device="cuda")
    q = torch.randn(B, nq * 128, generator=g, device="cuda")
    k = torch.randn(B, nkv * 128, generator=g, device="cuda")
    v = torch.randn(B, nkv * 128, generator=g, device="cuda")
    pos = torch.full((B,), T - 1, dtype=torch.int32, device="cuda")

    def timed(mode):
        ws = torch.empty(kernels.attention_workspace_bytes(B, nq, nkv, T), dtype=torch.uint8, device="cuda") if mode == 1 else None
        run = lambda: kernels.attention_int8(q, k, v, ck, cv, sk, sv, pos, layer=0, n_q=nq, n_kv=nkv, max_seq=T, max_len=T,
                                             heads_per_cta=args.heads_per_cta, mode=mode, workspace=ws)
        for _ in range(max(3, args.warmup)):
            run()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            run()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.steps

    bytes_per = B * nkv * T * (2 * 128 + 8) + B * nq * 128 * 8
    peak = _peak()
    ms_fast = timed(1)
    want = kernels.attention_int8(q, k, v, ck, cv, sk, sv, pos, layer=0, n_q=nq, n_kv=nkv, max_seq=T, max_len=T, append=False)
    got = kernels.attention_int8(q, k, v, ck, cv, sk, sv, pos, layer=0, n_q=nq, n_kv=nkv, max_seq=T, max_len=T, append=False, mode=1)
    fast_err = float((got - want).abs().max() / want.abs().max())
    ms = timed(0)
    gbs = bytes_per / (ms * 1e-3) / 1e9
    cpu = _cpu_attention_baseline(nq, nkv, T) if not getattr(args, "no_cpu_baseline", False) else None
    print(json.dumps({
        "metric": "attention_int8_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 x int8", "data": "synthetic",
        "config": {"workload": f"attn: fused INT8-KV GQA decode attention, batch {B}, {nq}q/{nkv}kv heads, context {T}",
                   "l2": f"KV {bytes_per / 1e6:.0f} MB per step, larger than L2"},
        "gpu_launches": args.steps,
        "roofline": {"bound": "hbm", "kernel": "attn_kernel", "achieved": gbs, "peak": peak[0], "peak_source": peak[1], "unit": "GB/s",
                     "frac": gbs / peak[0], "traffic": bytes_per * (265.2 / 259.5),
                     "traffic_source": "ncu at 24 sequences: 260.2 MB read + 5.0 MB written for 259.5 MB algorithmic, scaled by the sequence count",
                     "bytes_per_launch": bytes_per, "us_per_launch": ms * 1e3},
        "tolerance_mode": {"ms_per_step": ms_fast, "achieved": bytes_per / (ms_fast * 1e-3) / 1e9, "unit": "GB/s",
                           "frac": bytes_per / (ms_fast * 1e-3) / 1e9 / peak[0], "kernel": "fa_append_kernel + attn_fast_kernel + attn_fast_merge_kernel",
                           "max_rel_err_vs_exact": fast_err, "tolerance": 1e-3},
        "cpu_baseline": cpu,
    }), flush=True)


def _cpu_attention_baseline(nq, nkv, T):
    """The reference's own attention (FusedKVCache::forward_attention_raw through oracle/_ref) for ONE sequence at this
    context on the host cores: sequences per second, bounded sample."""
    import sys
    import time
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    for pth in (str(root), str(root / "tests")):
        if pth not in sys.path:
            sys.path.insert(0, pth)
    import bench
    from oracle import oracle_py as ora
    threads = bench.use_host_threads()
    kind = "kernels_fast" if ora.ref_available("kernels_fast") else ("kernels" if ora.ref_available("kernels") else None)
    rng = np.random.default_rng(3)
    q = rng.standard_normal(nq * 128).astype(np.float32)
    k = rng.standard_normal(nkv * 128).astype(np.float32)
    v = rng.standard_normal(nkv * 128).astype(np.float32)
    out = np.zeros(nq * 128, np.float32)
    P = ora.ptr
    if kind:
        L = ora.load_ref(kind)
        kv = L.refk_kv_create(1, nq, nkv, 128, T)
        rows = nkv * T
        ora.view(L.refk_kv_k(kv), rows * 128, np.int8)[:] = rng.integers(-127, 128, rows * 128, dtype=np.int8)
        ora.view(L.refk_kv_v(kv), rows * 128, np.int8)[:] = rng.integers(-127, 128, rows * 128, dtype=np.int8)
        ora.view(L.refk_kv_k_scales(kv), rows, np.float32)[:] = (0.01 + 0.02 * rng.random(rows)).astype(np.float32)
        ora.view(L.refk_kv_v_scales(kv), rows, np.float32)[:] = (0.01 + 0.02 * rng.random(rows)).astype(np.float32)

        def one():
            L.refk_kv_set_len(kv, T - 1)
            L.refk_kv_attention(kv, 0, P(q.copy(), ora.c_f32p), P(k.copy(), ora.c_f32p), P(v.copy(), ora.c_f32p), P(out, ora.c_f32p))
    else:
        O = ora.load_oracle()
        ck, cv = rng.integers(-127, 128, nkv * T * 128, dtype=np.int8), rng.integers(-127, 128, nkv * T * 128, dtype=np.int8)
        sk, sv = (0.01 + 0.02 * rng.random(nkv * T)).astype(np.float32), (0.01 + 0.02 * rng.random(nkv * T)).astype(np.float32)

        def one():
            O.ora_attention_int8(0, T - 1, nq, nkv, 128, T, 10000.0, P(q.copy(), ora.c_f32p), P(k.copy(), ora.c_f32p), P(v.copy(), ora.c_f32p),
                                 P(out, ora.c_f32p), P(ck, ora.c_i8p), P(cv, ora.c_i8p), P(sk, ora.c_f32p), P(sv, ora.c_f32p))
    one()
    n, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < 3.0:
        one()
        n += 1
    dt = time.perf_counter() - t0
    bytes_seq = nkv * T * 264
    return {"value": n * bytes_seq / dt / 1e9, "unit": "GB/s", "cores": threads, "kind": "reference" if kind else "port",
            "sample": f"{n} calls of the reference's attention for ONE sequence at context {T} ({bytes_seq / 1e6:.1f} MB of KV each), {dt:.1f} s; "
                      f"{n / dt:.1f} sequences/s"}


def run_decode_batch(args):
    import torch
    from .engine import Engine
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))))
    from .sharding import shard_sequences
    _, B = shard_sequences(args.batch, world, rank)     # sequences are sharded across ranks, no data-path collective
    ctx = args.context
    cfg = dict(synth.BITNET_2B, max_seq_len=(ctx + args.steps + max(3, args.warmup) + 8 + 3) // 4 * 4)
    model = synth.SyntheticModel(cfg, seed=0)
    eng = Engine(model.config_struct(kv_mode=args.kv_mode), batch=B, attention_mode=args.attention_mode).load_synthetic(model)
    eng.kv_fill_random(ctx, seed=rank)
    first = synth.prompt_tokens(1000 + rank, B, cfg["vocab_size"])
    warm = eng.decode_greedy(first, max(3, args.warmup))
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    l0 = eng.kernel_launches()
    eng.decode_greedy(warm[-1], args.steps)
    ms = eng.last_device_ms()
    launches = eng.kernel_launches() - l0
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank == 0:
        print(json.dumps({
            "metric": "decode_tokens_per_second_batched", "value": args.batch * args.steps / (ms * 1e-3), "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": f"decode_batch: BitNet-2B shape, global batch {args.batch}, context {ctx} (device-filled KV), "
                                   f"{B} sequences per GPU", "parallelism": f"dp{world}", "kv_mode": args.kv_mode,
                       "attention_mode": args.attention_mode},
            "gpu_launches": int(launches),
        }), flush=True)
    eng.close()
    if world > 1:
        dist.destroy_process_group()


def run_decode_tp(args):
    import torch
    from . import tp
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    B = 32 if args.batch == 256 else args.batch
    ctx = 2048 if args.context == 4096 else args.context
    warm = max(3, args.warmup)
    cfg = dict(synth.SYNTH_8B)
    dec = tp.TensorParallelDecoder(cfg, B, ctx + args.steps + warm + 8).load_random(seed=0, context=ctx)
    first = torch.from_numpy(synth.prompt_tokens(2000, B, cfg["vocab_size"])).cuda()
    dec.step(first)
    for _ in range(warm - 1):
        dec.step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        dec.step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank == 0:
        print(json.dumps({
            "metric": "decode_tokens_per_second_batched", "value": B * args.steps / (ms * 1e-3), "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": f"decode_tp: synthetic 8B shape (32L, 4096/14336, 32q/8kv, vocab 128256), batch {B}, context {ctx} "
                                   f"(device-filled KV), device-generated random shards", "parallelism": f"tp{world}",
                       "collectives_per_step": dec.collectives_per_step, "cuda_graph": bool(dec.use_graph)},
            "gpu_launches": int(dec.kernels_per_step * args.steps),
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run(args):
    fn = {"gemv": run_gemv, "lm_head": run_lm_head, "gemm": run_gemm, "attn": run_attn, "decode_batch": run_decode_batch, "decode_tp": run_decode_tp}.get(args.workload)
    if fn is None:
        raise SystemExit(f"unknown workload {args.workload!r}")
    return fn(args)
