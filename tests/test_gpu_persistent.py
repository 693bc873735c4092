"""The persistent single-sequence kernel (tenzo_ext_options_t.persistent = 1: one cooperative launch per token) against the
reference fixtures and the kernel chain: it is the same arithmetic, so everything is compared with `==`."""
import numpy as np
import pytest
from helpers import best_cpu_engine, greedy_stream, synth

pytestmark = pytest.mark.gpu
BUFS = {0: "x", 2: "q", 3: "k", 4: "v", 5: "attn_out", 8: "h1", 12: "act"}


def test_tiny_stream_matches_reference_fixture(cuda_lib, golden):
    from tenzo_b200 import abi
    from tenzo_b200.engine import Engine
    g = golden["engine_tiny"]
    m = synth.SyntheticModel(synth.TINY, seed=3)
    prompt = g["prompt"]
    with Engine(m.config_struct(), persistent=1).load_synthetic(m) as e:
        for t in prompt[:-1]:
            e.prefill_token(int(t))
        assert e.persistent_phase_ns(reset=False) is not None, "the persistent kernel was not used"
        cur, got = int(prompt[-1]), []
        for _ in range(len(g["tokens"])):
            cur = e.generate_step(cur, abi.TenzoSampling(0.0, 0.9, 40, 1.0))
            got.append(cur)
        assert got == g["tokens"].tolist()
        assert np.array_equal(e.read_buffer(15), g["logits"]) and np.array_equal(e.read_buffer(0), g["x"])


def test_medium_model_equals_kernel_chain_and_cpu_engine(cuda_lib):
    """Context past 128 and 256 keys (two value chunks, the attention bucket changes): buffers after selected steps,
    every layer's cache bytes and the greedy stream equal the kernel chain's; the stream equals the CPU engine's."""
    from tenzo_b200 import abi
    from tenzo_b200.engine import Engine
    cfg = dict(hidden_size=512, num_q_heads=4, num_kv_heads=2, head_dim=128, num_layers=3, ffn_dim=1536, vocab_size=4096, max_seq_len=1024)
    m = synth.SyntheticModel(cfg, seed=5)
    prompt = synth.prompt_tokens(5, 271, cfg["vocab_size"])
    greedy = abi.TenzoSampling(0.0, 0.9, 40, 1.0)
    with Engine(m.config_struct(), persistent=0).load_synthetic(m) as a, Engine(m.config_struct(), persistent=1).load_synthetic(m) as b:
        for i, t in enumerate(prompt[:-1]):
            a.prefill_token(int(t))
            b.prefill_token(int(t))
            if i in (0, 1, 127, 128, 255, 256, 269):
                for w, name in BUFS.items():
                    assert np.array_equal(a.read_buffer(w), b.read_buffer(w)), f"token {i}: {name} differs"
        ca = cb = int(prompt[-1])
        for i in range(6):
            ca, cb = a.generate_step(ca, greedy), b.generate_step(cb, greedy)
            assert ca == cb
            assert np.array_equal(a.read_buffer(15), b.read_buffer(15)), "logits differ"
        T = a.seq_len()
        assert T == b.seq_len()
        for l in range(cfg["num_layers"]):
            for x, y in zip(a.kv_export(0, l, T), b.kv_export(0, l, T)):
                assert np.array_equal(x, y)
        ta, tb = a.decode_greedy([ca], 12), b.decode_greedy([cb], 12)
        assert np.array_equal(ta, tb)
    cpu = best_cpu_engine(m, 1024)
    want = greedy_stream(cpu, prompt[:40], 8)
    cpu.close()
    with Engine(m.config_struct(), persistent=1).load_synthetic(m) as e:
        for t in prompt[:39]:
            e.prefill_token(int(t))
        got = e.decode_greedy([int(prompt[39])], 8)[:, 0]
    assert got.tolist() == want.tolist()


def test_bitnet_2b_shape_first_32_tokens(cuda_lib, golden):
    from tenzo_b200.engine import Engine
    g = golden["engine_2b"]
    cfg = dict(synth.BITNET_2B, max_seq_len=256)
    m = synth.SyntheticModel(cfg, seed=0)
    prompt = g["prompt"]
    with Engine(m.config_struct(), persistent=1).load_synthetic(m) as e:
        for t in prompt[:-1]:
            e.prefill_token(int(t))
        got = e.decode_greedy([int(prompt[-1])], 32)[:, 0]
    assert got.tolist() == g["tokens"][:32].tolist()
