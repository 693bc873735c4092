"""Whole-engine parity through the tenzo.h ABI: greedy token streams, logits, KV cache contents,
teacher-forced single layers, the batched extension, the backend class and error behaviour.
fp32 buffers are compared with `==`: the engine reproduces the reference's operation order."""
import ctypes as C
import hashlib

import numpy as np
import pytest
from helpers import OracleEngine, best_cpu_engine, greedy_stream, ora, rel_err, synth

pytestmark = pytest.mark.gpu
FP_TOL = 1e-3


def gpu_engine(model, **kw):
    from tenzo_b200.engine import Engine
    cfg_keys = ("max_seq_len", "kv_mode")
    return Engine(model.config_struct(**{k: v for k, v in kw.items() if k in cfg_keys}),
                  **{k: v for k, v in kw.items() if k not in cfg_keys}).load_synthetic(model)


class GpuAsCpuApi:
    """Adapter so greedy_stream() can drive the CUDA engine exactly as it drives the CPU ones."""

    def __init__(self, e):
        self.e = e

    def prefill(self, tok):
        self.e.prefill_token(tok)

    def generate(self, tok, temperature=0.0, rep=1.0, **_):
        from tenzo_b200 import abi
        return self.e.generate_step(tok, abi.TenzoSampling(temperature, 0.9, 40, rep))


@pytest.mark.parametrize("graph,pdl", [(0, 0), (1, 0), (1, 1)])
def test_tiny_stream_matches_reference_fixture(cuda_lib, golden, graph, pdl):
    g = golden["engine_tiny"]
    m = synth.SyntheticModel(synth.TINY, seed=3)
    assert hashlib.sha256(m.lm_w.tobytes()).hexdigest() == str(g["lm_sha"])
    with gpu_engine(m, use_graph=graph, use_pdl=pdl) as e:
        toks = greedy_stream(GpuAsCpuApi(e), g["prompt"], 32)
        assert np.array_equal(toks, g["tokens"]), "greedy stream diverged from the reference"
        assert np.array_equal(e.read_buffer(15), g["logits"]), "logits differ"
        assert np.array_equal(e.read_buffer(0), g["x"]), "residual stream differs"
        assert e.get_seq_len() == 15 + 32
        assert e.kernel_launches() > 0


def test_medium_model_stream_logits_and_cache(cuda_lib):
    cfg = dict(synth.TINY, hidden_size=512, num_q_heads=4, num_kv_heads=1, ffn_dim=1408, num_layers=4, vocab_size=4096,
               max_seq_len=320)
    m = synth.SyntheticModel(cfg, seed=21)
    cpu = best_cpu_engine(m)
    prompt = synth.prompt_tokens(21, 270, cfg["vocab_size"])   # crosses the 256-key attention chunk
    ref = greedy_stream(cpu, prompt, 32)
    with gpu_engine(m) as e:
        got = greedy_stream(GpuAsCpuApi(e), prompt, 32)
        assert np.array_equal(got, ref)
        assert np.array_equal(e.read_buffer(15), cpu.buffer("logits", cfg["vocab_size"]))
        k, v, sk, sv = e.kv_export(0, 3, 301)
        if isinstance(cpu, OracleEngine):
            pk, pv, psk, psv = (C.POINTER(C.c_int8)(), C.POINTER(C.c_int8)(), C.POINTER(C.c_float)(), C.POINTER(C.c_float)())
            cpu.O.ora_engine_kv(cpu.e, C.byref(pk), C.byref(pv), C.byref(psk), C.byref(psv))
            rk = ora.view(pk, 4 * 320 * 128, np.int8).reshape(4, 1, 320, 128)[3, :, :301]
        else:
            kvp = cpu.L.refk_engine_kv(cpu.h)
            rk = ora.view(cpu.L.refk_kv_k(kvp), 4 * 320 * 128, np.int8).reshape(4, 1, 320, 128)[3, :, :301]
        assert np.array_equal(k, rk), "cached int8 keys differ"
    cpu.close()


def test_teacher_forced_layer_is_exact_where_the_reference_is(cuda_lib):
    """Same fp32 residual stream into layer 0 on both sides, BitNet-2B layer shape: every buffer equal."""
    cfg = dict(synth.TINY, hidden_size=2560, num_q_heads=20, num_kv_heads=5, ffn_dim=6912, num_layers=1, vocab_size=512)
    m = synth.SyntheticModel(cfg, seed=22)
    cpu = best_cpu_engine(m)
    x = np.random.default_rng(22).standard_normal(2560).astype(np.float32)
    cpu.set_buffer("x", x)
    (cpu.L.refk_engine_forward_layer if hasattr(cpu, "L") else cpu.O.ora_engine_forward_layer)(cpu.h if hasattr(cpu, "L") else cpu.e, 0)
    with gpu_engine(m) as e:
        e.write_x(x)
        e.run_layer(0)
        for which, name, n in ((8, "h1", 2560), (12, "act", 6912), (0, "x", 2560), (5, "attn_out", 2560)):
            assert np.array_equal(e.read_buffer(which), cpu.buffer(name, n)), f"{name}: rel err {rel_err(e.read_buffer(which), cpu.buffer(name, n)):.2e}"
        assert np.array_equal(e.read_buffer(4), cpu.buffer("v", 640))
    cpu.close()


def test_bitnet_2b_shape_first_32_tokens(cuda_lib, golden):
    """The north-star check: BitNet-2B-shaped model, 64-token prompt, first 32 greedy tokens equal
    the reference's; also the device-resident decode loop produces the same stream."""
    g = golden["engine_2b"]
    cfg = dict(synth.BITNET_2B, max_seq_len=256)
    m = synth.SyntheticModel(cfg, seed=0)
    assert hashlib.sha256(m.lm_w.tobytes()).hexdigest() == str(g["lm_sha"])
    assert hashlib.sha256(m.layers[29]["down_w"].tobytes()).hexdigest() == str(g["l29down_sha"])
    with gpu_engine(m) as e:
        toks = greedy_stream(GpuAsCpuApi(e), g["prompt"], 32)
        assert np.array_equal(toks, g["tokens"]), f"first mismatch at {int(np.argmax(toks != g['tokens']))}"
        lg = e.read_buffer(15)
        assert np.array_equal(lg[g["top_idx"]], g["top_val"])
        assert hashlib.sha256(lg.tobytes()).hexdigest() == str(g["logits_sha"]), "128256 logits are not bit-identical"
        e.reset()
        for t in g["prompt"][:-1]:
            e.prefill_token(int(t))
        dev_loop = e.decode_greedy([int(g["prompt"][-1])], 32)[:, 0]
        assert np.array_equal(dev_loop, g["tokens"])


def test_batched_engine_equals_independent_sequences(cuda_lib):
    cfg = dict(synth.TINY, hidden_size=512, num_q_heads=4, num_kv_heads=2, ffn_dim=704, num_layers=2, vocab_size=2000)
    m = synth.SyntheticModel(cfg, seed=23)
    B, npre, ngen = 3, 9, 12
    prompts = np.stack([synth.prompt_tokens(100 + b, npre, cfg["vocab_size"]) for b in range(B)])
    singles = []
    for b in range(B):
        with gpu_engine(m) as e:
            singles.append(greedy_stream(GpuAsCpuApi(e), prompts[b], ngen))
    with gpu_engine(m, batch=B) as e:
        for t in range(npre - 1):
            e.prefill_tokens(prompts[:, t])
        cur, outs = prompts[:, -1].copy(), []
        for _ in range(ngen):
            cur = e.generate_steps(cur)
            outs.append(cur.copy())
        assert np.array_equal(np.stack(outs, axis=1), np.stack(singles))
        assert [e.seq_len(b) for b in range(B)] == [npre - 1 + ngen] * B
    cpu = best_cpu_engine(m)
    assert np.array_equal(greedy_stream(cpu, prompts[1], ngen), singles[1])
    cpu.close()


def test_batched_engine_on_the_tensor_core_paths_matches_the_cpu_engine(cuda_lib):
    """32 sequences: the TL1 layers run as tcgen05 GEMMs, the LM head as a tcgen05 GEMM, attention reads K through
    TMA tiles (32 x 2 kv heads = 64 items). Every sequence's greedy stream and the last step's logits must equal the
    CPU engine's for that sequence alone; both the stepwise call and the device-resident greedy loop are checked."""
    cfg = dict(synth.TINY, hidden_size=512, num_q_heads=4, num_kv_heads=2, ffn_dim=768, num_layers=2, vocab_size=2048, max_seq_len=96)
    m = synth.SyntheticModel(cfg, seed=29)
    B, npre, ngen = 32, 70, 10                       # context crosses the 64-key tile boundary
    prompts = np.stack([synth.prompt_tokens(300 + b, npre, cfg["vocab_size"]) for b in range(B)])
    want, want_logits = [], []
    for b in (0, 7, 31):
        cpu = best_cpu_engine(m, max_seq_len=96)
        want.append(greedy_stream(cpu, prompts[b], ngen))
        want_logits.append(cpu.buffer("logits", cfg["vocab_size"]))
        cpu.close()
    with gpu_engine(m, batch=B, max_seq_len=96) as e:
        for t in range(npre - 1):
            e.prefill_tokens(prompts[:, t])
        cur, outs = prompts[:, -1].copy(), []
        for _ in range(ngen):
            cur = e.generate_steps(cur)
            outs.append(cur.copy())
        got = np.stack(outs, axis=1)
        for i, b in enumerate((0, 7, 31)):
            assert np.array_equal(got[b], want[i]), f"sequence {b}"
            assert np.array_equal(e.read_buffer(15, seq=b, count=cfg["vocab_size"]), want_logits[i]), f"logits of sequence {b}"
    with gpu_engine(m, batch=B, max_seq_len=96) as e:
        for t in range(npre - 1):
            e.prefill_tokens(prompts[:, t])
        assert np.array_equal(e.decode_greedy(prompts[:, -1], ngen).T, got)


def test_batch_256_engine_matches_the_cpu_engine(cuda_lib):
    """256 sequences at once (the largest tcgen05 tile: 256 accumulator columns) for a few steps; three of the
    sequences are replayed alone on the CPU engine."""
    cfg = dict(synth.TINY, hidden_size=256, num_q_heads=2, num_kv_heads=1, ffn_dim=384, num_layers=2, vocab_size=2048, max_seq_len=32)
    m = synth.SyntheticModel(cfg, seed=37)
    B, npre, ngen = 256, 5, 6
    prompts = np.stack([synth.prompt_tokens(700 + b, npre, cfg["vocab_size"]) for b in range(B)])
    with gpu_engine(m, batch=B, max_seq_len=32) as e:
        for t in range(npre - 1):
            e.prefill_tokens(prompts[:, t])
        got = e.decode_greedy(prompts[:, -1], ngen).T
    for b in (0, 129, 255):
        cpu = best_cpu_engine(m, max_seq_len=32)
        assert np.array_equal(got[b], greedy_stream(cpu, prompts[b], ngen)), f"sequence {b}"
        cpu.close()


def test_long_decode_crosses_every_attention_bucket(cuda_lib):
    """1100 greedy tokens of a tiny model: the step graph is re-captured for the 512-, 1024- and 2048-key attention
    buckets and the device-resident loop hands over between them; the stream must equal the CPU engine's throughout,
    and no kernel may have given up a bounded wait."""
    cfg = dict(synth.TINY, max_seq_len=1200)
    m = synth.SyntheticModel(cfg, seed=31)
    prompt = synth.prompt_tokens(8, 6, cfg["vocab_size"])
    cpu = best_cpu_engine(m, max_seq_len=1200)
    want = greedy_stream(cpu, prompt, 1100)
    cpu.close()
    with gpu_engine(m, max_seq_len=1200) as e:
        for t in prompt[:-1]:
            e.prefill_token(int(t))
        got = e.decode_greedy([int(prompt[-1])], 1100)[:, 0]
        assert np.array_equal(got, want), f"first difference at step {int(np.argmax(got != want))}"
        assert e.seq_len() == len(prompt) - 1 + 1100
    assert cuda_lib.tenzo_cuda_tl1_gemv_take_timeouts() == 0 and cuda_lib.tenzo_cuda_attention_take_timeouts() == 0


def test_rope_theta_extension_against_oracle(cuda_lib):
    m = synth.SyntheticModel(synth.TINY, seed=24)
    o = OracleEngine(m, rope_theta=500000.0)
    prompt = synth.prompt_tokens(24, 20, 1024)
    ref = greedy_stream(o, prompt, 16)
    with gpu_engine(m, rope_theta=500000.0) as e:
        assert np.array_equal(greedy_stream(GpuAsCpuApi(e), prompt, 16), ref)
    o.close()


def test_sampling_paths(cuda_lib, golden):
    """Greedy with a repetition penalty follows the reference (fixture); the stochastic path only
    ever returns one of the top-k tokens."""
    from tenzo_b200 import abi
    g, s = golden["engine_tiny"], golden["sampler"]
    m = synth.SyntheticModel(synth.TINY, seed=3)
    with gpu_engine(m) as e:
        toks = greedy_stream(GpuAsCpuApi(e), g["prompt"], 32)
        nxt = e.generate_step(int(toks[-1]), abi.TenzoSampling(0.0, 0.9, 40, 1.3), s["past"])
        assert nxt == int(s["next_penalised"])
        e.set_seq_len(0, e.get_seq_len() - 1)               # the penalty was applied to the logits in place (as in the reference)
        draws = set()
        for _ in range(20):
            draws.add(e.generate_step(int(toks[-1]), abi.TenzoSampling(0.8, 0.95, 5, 1.0)))
            e.set_seq_len(0, e.get_seq_len() - 1)
        top5 = set(np.argsort(e.read_buffer(15))[-5:].tolist())      # logits of the last (unpenalised) step
        assert draws <= top5


def test_error_behaviour(cuda_lib):
    from tenzo_b200 import abi
    from tenzo_b200.engine import Engine
    m = synth.SyntheticModel(synth.TINY, seed=25)
    lib = cuda_lib
    with gpu_engine(m, max_seq_len=4) as e:
        assert e.set_layer_weights(99, m.layer_struct(0)) == abi.ERR_INVALID
        assert lib.tenzo_prefill_token(e.get_raw_handle(), 10 ** 6) == abi.ERR_INVALID      # token outside the vocabulary
        assert lib.tenzo_set_lm_head_f32(e.get_raw_handle(), m.final_norm.ctypes.data_as(abi.c_f32p), 4, 4) == abi.ERR_UNSUPPORTED
        assert lib.tenzo_load_model(e.get_raw_handle(), b"/nonexistent/w.bin", b"/nonexistent/m.mlir") == abi.ERR_IO
        for t in range(4):
            e.prefill_token(t)
        assert lib.tenzo_prefill_token(e.get_raw_handle(), 1) == abi.ERR_INVALID            # cache full
        assert lib.tenzo_generate_step(e.get_raw_handle(), 1, None, None, 0) == -1
        e.reset()
        assert e.get_seq_len() == 0
        e.prefill_token(1)
    bad = m.config_struct()
    bad.kv_mode = b"tl1_fused"
    with pytest.raises(RuntimeError):
        Engine(bad)
    bad = m.config_struct()
    bad.head_dim = 64
    with pytest.raises(RuntimeError):
        Engine(bad)


def test_backend_class_host_pointer_calls(cuda_lib):
    """tenzo::CUDARuntime::execute* with host pointers, as forward_layer_cuda calls them
    (TenzoEngine.cpp:1374-1411), against the CPU kernels."""
    from gpu_helpers import cpu_bitlinear, cpu_rms_norm
    from tenzo_b200 import abi
    lib = cuda_lib
    assert lib.tenzo_hal_initialize() == 1
    rng = np.random.default_rng(26)
    N, K = 6912, 2560
    w = synth.random_tl1_packed(rng, N, K)
    x = rng.standard_normal(K).astype(np.float32)
    out = np.zeros(N, np.float32)
    assert lib.tenzo_hal_bitlinear_tl1_host(x.ctypes.data_as(abi.c_f32p), w.ctypes.data_as(abi.c_u8p), out.ctypes.data_as(abi.c_f32p), 1, K, N, 0.016) == 1
    assert np.array_equal(out, cpu_bitlinear(x, w, N, K, 0.016)[0])
    nw = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    y = np.zeros(K, np.float32)
    assert lib.tenzo_hal_rmsnorm_host(x.ctypes.data_as(abi.c_f32p), nw.ctypes.data_as(abi.c_f32p), y.ctypes.data_as(abi.c_f32p), K, 1e-5) == 1
    assert np.array_equal(y, cpu_rms_norm(x, nw)), "the backend class's RMSNorm is the engine's kernel: same bits as the CPU's"
    A, Bm = rng.standard_normal((5, 70)).astype(np.float32), rng.standard_normal((70, 33)).astype(np.float32)
    Cm = np.zeros((5, 33), np.float32)
    assert lib.tenzo_hal_gemm_f32_host(A.ctypes.data_as(abi.c_f32p), Bm.ctypes.data_as(abi.c_f32p), Cm.ctypes.data_as(abi.c_f32p), 5, 70, 33) == 1
    assert rel_err(Cm, A @ Bm) < 1e-5
    assert lib.tenzo_hal_bitlinear_tl1_host(x.ctypes.data_as(abi.c_f32p), w.ctypes.data_as(abi.c_u8p), out.ctypes.data_as(abi.c_f32p), 1, 3, N, 1.0) == 0


@pytest.mark.parametrize("with_manifest", [True, False])
def test_load_model_from_files_matches_the_cpu_engine(tmp_path, with_manifest):
    """tenzo_load_model on a checkpoint in the reference's format (writer pinned to the reference's own loader in
    tests/test_loader_host.py): device-side embedding quantisation and TL1 repack, then the same greedy stream as the
    CPU engine fed the same tensors through its setters. A short file loads with the reference's fallbacks, an
    unreadable one reports TENZO_ERROR_IO."""
    from helpers import loader_quantised_embedding, write_checkpoint
    from tenzo_b200 import abi
    from tenzo_b200.engine import Engine
    cfg = dict(synth.BITNET_2B, num_layers=2, vocab_size=768, max_seq_len=48)
    model = synth.SyntheticModel(cfg, seed=11)
    w, m = tmp_path / "weights.bin", tmp_path / "model.mlir"
    emb = write_checkpoint(model, w, m, with_manifest=with_manifest, gap=48)
    if not with_manifest:
        for lw in model.layers:
            for name in model.shapes:
                lw[name + "_scale"] = np.float32(1.0)
    model.lm_w, model.lm_scales = loader_quantised_embedding(emb)
    prompt = synth.prompt_tokens(4, 5, cfg["vocab_size"])
    cpu = best_cpu_engine(model, max_seq_len=48)
    want = greedy_stream(cpu, prompt, 8)
    cpu.close()
    with Engine(model.config_struct(max_seq_len=48)) as e:
        e.load_model(str(w), str(m))
        for t in prompt[:-1]:
            e.prefill_token(int(t))
        cur, got = int(prompt[-1]), []
        for _ in range(8):
            cur = e.generate_step(cur, abi.TenzoSampling(0.0, 0.9, 40, 1.0))
            got.append(cur)
        assert np.array_equal(np.asarray(got, np.int32), want)
        short = tmp_path / "short.bin"
        short.write_bytes(w.read_bytes()[: cfg["vocab_size"] * cfg["hidden_size"] * 4 + 1000])
        e.load_model(str(short), str(m))                   # tensors past the end become ones / zero weights, as in the reference
        assert e.lib.tenzo_load_model(e.get_raw_handle(), str(tmp_path / "missing.bin").encode(), str(m).encode()) == abi.ERR_IO


def test_chunked_prefill_equals_token_by_token(cuda_lib):
    """tenzo_ext_prefill_chunk (prompt rows through the GEMM path, K/V appended, causal attention as independent queries)
    leaves the same KV cache bytes and scales as token-by-token prefill and the same greedy continuation, which is also
    the CPU engine's. Chunks of 1, 15 (per-sequence kernels), 16+ (tensor cores) and a chunk that starts mid-sequence."""
    cfg = dict(synth.TINY, hidden_size=512, num_q_heads=4, num_kv_heads=2, ffn_dim=768, num_layers=2, vocab_size=2048, max_seq_len=400)
    m = synth.SyntheticModel(cfg, seed=41)
    prompt = synth.prompt_tokens(12, 301, cfg["vocab_size"])
    cpu = best_cpu_engine(m, max_seq_len=400)
    want = greedy_stream(cpu, prompt, 12)
    cpu.close()
    with gpu_engine(m, max_seq_len=400) as ref:
        for t in prompt[:-1]:
            ref.prefill_token(int(t))
        kv_ref = [ref.kv_export(0, l, 300) for l in range(cfg["num_layers"])]
        assert np.array_equal(ref.decode_greedy([int(prompt[-1])], 12)[:, 0], want)
    for chunks in ([300], [1, 15, 16, 100, 168], [37, 263]):
        with gpu_engine(m, max_seq_len=400) as e:
            at = 0
            for c in chunks:
                e.prefill_chunk(prompt[at:at + c])
                at += c
            assert at == 300 and e.seq_len() == 300
            for l in range(cfg["num_layers"]):
                for got, ref_part in zip(e.kv_export(0, l, 300), kv_ref[l]):
                    assert np.array_equal(got, ref_part), f"layer {l}, chunks {chunks}"
            assert np.array_equal(e.decode_greedy([int(prompt[-1])], 12)[:, 0], want), f"chunks {chunks}"


def test_stochastic_streams_equal_the_reference_on_the_same_rand_sequence(cuda_lib):
    """The reference draws from libc's process-global rand() (TenzoEngine.cpp:1800) and so does this library: seed it,
    run 64 sampled steps (temperature, top-k, top-p, repetition penalty over the running history) on the compiled
    reference, seed it again, run the same on the GPU engine - the logits are bit-identical, so the streams must be."""
    if not ora.ref_available("kernels"):
        pytest.skip("needs the compiled reference (oracle/_ref)")
    from helpers import RefEngine
    from tenzo_b200 import abi
    libc = C.CDLL("libc.so.6")
    m = synth.SyntheticModel(synth.TINY, seed=3)
    prompt = synth.prompt_tokens(11, 9, synth.TINY["vocab_size"])
    for temperature, top_p, top_k, rep in ((0.7, 0.9, 40, 1.15), (1.3, 1.0, 64, 1.0), (0.4, 0.5, 5, 1.3)):
        ref = RefEngine(m)
        for t in prompt[:-1]:
            ref.prefill(int(t))
        libc.srand(1234)
        cur, want, hist = int(prompt[-1]), [], [int(t) for t in prompt]
        for _ in range(64):
            cur = ref.generate(cur, temperature=temperature, top_p=top_p, top_k=top_k, rep=rep, past=hist)
            want.append(cur)
            hist.append(cur)
        ref.close()
        with gpu_engine(m) as e:
            for t in prompt[:-1]:
                e.prefill_token(int(t))
            libc.srand(1234)
            cur, got, hist = int(prompt[-1]), [], [int(t) for t in prompt]
            for _ in range(64):
                cur = e.generate_step(cur, abi.TenzoSampling(temperature, top_p, top_k, rep), past_tokens=hist)
                got.append(cur)
                hist.append(cur)
        assert got == want, (temperature, top_p, top_k, rep, int(np.argmax(np.asarray(got) != np.asarray(want))))
