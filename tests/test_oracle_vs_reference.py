"""The C oracle against the compiled reference itself, on fresh seeded inputs (CPU only).

Skipped where oracle/_ref was not built (the reference checkout is needed to build it); the
golden-vector tests cover the same ground there.
"""
import numpy as np
import pytest
from helpers import OracleEngine, RefEngine, greedy_stream, ora, synth

pytestmark = pytest.mark.skipif(not ora.ref_available("kernels"), reason="compiled reference (oracle/_ref) not present")
P = ora.ptr


@pytest.mark.parametrize("N,K", [(64, 2), (64, 126), (128, 128), (192, 258), (640, 2560)])
def test_bitlinear_bit_exact(N, K):
    O, R = ora.load_oracle(), ora.load_ref("kernels")
    rng = np.random.default_rng([31, N, K])
    w = synth.random_tl1_packed(rng, N, K)
    for trial in range(3):
        x = (rng.standard_normal(K) * (10.0 ** rng.integers(-3, 3))).astype(np.float32)
        if trial == 2:
            x[:] = 0.0   # all-zero activation: the 1e-6 floor path
        o1, a1, o2, a2 = np.zeros(N, np.float32), np.zeros(N, np.int32), np.zeros(N, np.float32), np.zeros(N, np.int32)
        i1 = O.ora_bitlinear_tl1(P(x, ora.c_f32p), P(w, ora.c_u8p), N, K, 0.0161, P(o1, ora.c_f32p), P(a1, ora.c_i32p))
        i2 = R.refk_bitlinear_tl1(P(x, ora.c_f32p), P(w.view(np.int8), ora.c_i8p), N, K, 0.0161, P(o2, ora.c_f32p), P(a2, ora.c_i32p))
        assert i1 == i2 and np.array_equal(a1, a2) and np.array_equal(o1, o2)


def test_lut_bytes_identical():
    O, R = ora.load_oracle(), ora.load_ref("kernels")
    rng = np.random.default_rng(32)
    x = rng.standard_normal(514).astype(np.float32)
    l1, l2 = np.zeros(257 * 32, np.int8), np.zeros(257 * 32, np.uint8)
    assert O.ora_build_lut(P(x, ora.c_f32p), 514, P(l1, ora.c_i8p)) == R.refk_build_lut(P(x, ora.c_f32p), 514, P(l2, ora.c_u8p))
    assert np.array_equal(l1.view(np.uint8), l2)


@pytest.mark.parametrize("cfg", [synth.TINY, dict(synth.TINY, hidden_size=512, num_q_heads=4, num_kv_heads=2, ffn_dim=704,
                                                  num_layers=3, vocab_size=2000)])
def test_engine_stream_and_every_buffer(cfg):
    m = synth.SyntheticModel(cfg, seed=9)
    r, o = RefEngine(m), OracleEngine(m)
    prompt = synth.prompt_tokens(9, 12, cfg["vocab_size"])
    assert np.array_equal(greedy_stream(r, prompt, 24), greedy_stream(o, prompt, 24))
    sizes = dict(x=cfg["hidden_size"], norm_x=cfg["hidden_size"], q=cfg["hidden_size"], attn_out=cfg["hidden_size"],
                 h1=cfg["hidden_size"], act=cfg["ffn_dim"], ffn_norm=cfg["ffn_dim"], down=cfg["hidden_size"],
                 logits=cfg["vocab_size"])
    for name, n in sizes.items():
        assert np.array_equal(r.buffer(name, n), o.buffer(name, n)), name
    assert r.seq_len() == o.seq_len() == 11 + 24
    r.close()
    o.close()


def test_penalised_greedy_matches():
    m = synth.SyntheticModel(synth.TINY, seed=10)
    r, o = RefEngine(m), OracleEngine(m)
    past, cur_r, cur_o = [5, 6, 7], 7, 7
    for _ in range(12):
        cur_r = r.generate(cur_r, temperature=0.0, rep=1.4, past=past)
        cur_o = o.generate(cur_o, temperature=0.0, rep=1.4, past=past)
        assert cur_r == cur_o
        past.append(cur_r)
    r.close()
    o.close()


def test_paged_attention_bit_exact_with_scattered_blocks():
    """PagedKVCache::forward_attention_raw against the restatement, blocks placed out of order."""
    O, R = ora.load_oracle(), ora.load_ref("kernels")
    L, nq, nkv, hd, blocks, layer = 2, 8, 2, 128, 12, 1
    rng = np.random.default_rng(41)
    order = rng.permutation(blocks).astype(np.int32)
    kv = R.refk_paged_create(L, nq, nkv, hd, blocks)
    rows = blocks * L * nkv * 16
    pk, pv = np.zeros(rows * hd, np.int8), np.zeros(rows * hd, np.int8)
    psk, psv = np.ones(rows, np.float32), np.ones(rows, np.float32)
    steps = 70
    for t in range(steps):
        if t % 16 == 0:
            R.refk_paged_push_block(kv, int(order[t // 16]))
        q = (rng.standard_normal(nq * hd) * (4.0 if t % 7 == 0 else 1.0)).astype(np.float32)   # peaked rows: weights under 1e-7
        k = rng.standard_normal(nkv * hd).astype(np.float32)
        v = rng.standard_normal(nkv * hd).astype(np.float32)
        o1, o2 = np.zeros(nq * hd, np.float32), np.zeros(nq * hd, np.float32)
        q1, k1, v1 = q.copy(), k.copy(), v.copy()
        R.refk_paged_set_len(kv, t)
        R.refk_paged_attention(kv, layer, P(q1, ora.c_f32p), P(k1, ora.c_f32p), P(v1, ora.c_f32p), P(o1, ora.c_f32p))
        q2, k2, v2 = q.copy(), k.copy(), v.copy()
        O.ora_attention_paged_int8(layer, t, nq, nkv, hd, L, 10000.0, P(q2, ora.c_f32p), P(k2, ora.c_f32p), P(v2, ora.c_f32p),
                                   P(o2, ora.c_f32p), P(pk, ora.c_i8p), P(pv, ora.c_i8p), P(psk, ora.c_f32p), P(psv, ora.c_f32p),
                                   P(order, ora.c_i32p))
        assert np.array_equal(o1, o2), t
        assert np.array_equal(q1, q2) and np.array_equal(k1, k2)
    assert np.array_equal(ora.view(R.refk_paged_k(kv), rows * hd, np.int8), pk)
    assert np.array_equal(ora.view(R.refk_paged_v(kv), rows * hd, np.int8), pv)
    assert np.array_equal(ora.view(R.refk_paged_k_scales(kv), rows, np.float32), psk)
    assert np.array_equal(ora.view(R.refk_paged_v_scales(kv), rows, np.float32), psv)
    R.refk_paged_destroy(kv)


def test_paged_engine_stream_matches_and_differs_from_fused():
    cfg = dict(synth.TINY, max_seq_len=96)
    m = synth.SyntheticModel(cfg, seed=9)
    r, o = RefEngine(m, kv_mode="paged_int8"), OracleEngine(m, kv_mode="paged_int8")
    prompt = synth.prompt_tokens(9, 20, cfg["vocab_size"])
    assert np.array_equal(greedy_stream(r, prompt, 40), greedy_stream(o, prompt, 40))
    for name, n in dict(x=cfg["hidden_size"], attn_out=cfg["hidden_size"], logits=cfg["vocab_size"]).items():
        assert np.array_equal(r.buffer(name, n), o.buffer(name, n)), name
    assert r.seq_len() == o.seq_len() == 19 + 40
    tab = np.zeros(16, np.int32)
    n = ora.load_ref("kernels").refk_paged_table(ora.load_ref("kernels").refk_engine_paged_kv(r.h), P(tab, ora.c_i32p), 16)
    assert n == 4 and list(tab[:4]) == [0, 1, 2, 3]          # the reference's allocator hands out 0, 1, 2, ...
    f = OracleEngine(m)                                       # the two KV modes are different arithmetic: ulps apart
    greedy_stream(f, prompt, 40)
    assert not np.array_equal(f.buffer("attn_out", cfg["hidden_size"]), o.buffer("attn_out", cfg["hidden_size"]))
    for e in (r, o, f):
        e.close()
