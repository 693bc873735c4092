"""The artefacts of tests/test_boundary_build.py, run: the consumer written against the reference's tenzo.hpp drives this
library through a checkpoint on disk, and the reference's own engine - compiled against this repository's CUDARuntime.h -
decodes with device = "cuda". Both must give the CPU engine's greedy stream."""
import subprocess
from pathlib import Path

import numpy as np
import pytest
from helpers import RefEngine, best_cpu_engine, greedy_stream, ora, synth, write_checkpoint

pytestmark = pytest.mark.gpu
REFDIR = Path(__file__).resolve().parents[1] / "oracle" / "_ref"


def test_consumer_of_the_reference_cpp_wrapper(cuda_lib, tmp_path):
    exe = REFDIR / "hpp_consumer"
    if not exe.exists():
        pytest.skip("oracle/_ref/hpp_consumer was not built (needs the reference checkout at build time)")
    cfg = dict(synth.TINY)
    m = synth.SyntheticModel(cfg, seed=3)
    emb = write_checkpoint(m, tmp_path / "weights.bin", tmp_path / "model.mlir")
    prompt = synth.prompt_tokens(3, 8, cfg["vocab_size"])
    n_gen = 12
    # the loader re-quantises the fp32 embedding it reads; the model above is already its fixed point (test_loader_host.py)
    cpu = best_cpu_engine(m)
    want = greedy_stream(cpu, prompt, n_gen)
    cpu.close()
    args = [str(exe), str(tmp_path / "weights.bin"), str(tmp_path / "model.mlir"), cfg["hidden_size"], cfg["num_q_heads"], cfg["num_kv_heads"],
            cfg["num_layers"], cfg["ffn_dim"], cfg["vocab_size"], cfg["max_seq_len"], n_gen, *prompt.tolist()]
    r = subprocess.run([str(a) for a in args], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [int(t) for t in r.stdout.split()] == want.tolist()


def test_reference_engine_with_device_cuda_runs_on_this_backend(cuda_lib):
    if not ora.ref_available("cuda"):
        pytest.skip("oracle/_ref/libtenzo_ref_cuda.so was not built (needs the reference checkout at build time)")
    m = synth.SyntheticModel(synth.TINY, seed=3)
    prompt = synth.prompt_tokens(5, 7, synth.TINY["vocab_size"])
    cpu = best_cpu_engine(m)
    want = greedy_stream(cpu, prompt, 10)
    want_logits = cpu.buffer("logits", synth.TINY["vocab_size"])
    cpu.close()
    before = cuda_lib.tenzo_hal_call_count()
    eng = RefEngine(m, kind="cuda", device=b"cuda")
    got = greedy_stream(eng, prompt, 10)
    got_logits = eng.buffer("logits", synth.TINY["vocab_size"])
    eng.close()
    calls = cuda_lib.tenzo_hal_call_count() - before
    # per token and layer: 4 norms + 7 TL1 products through tenzo::CUDARuntime (TenzoEngine.cpp:1374-1411)
    assert calls == (len(prompt) - 1 + 10) * synth.TINY["num_layers"] * 11, calls
    assert np.array_equal(got, want)
    assert np.array_equal(got_logits, want_logits)
