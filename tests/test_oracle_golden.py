"""The C oracle against the golden vectors produced by the compiled reference (CPU only).

These fixtures are the pin: the oracle must reproduce the reference's integers exactly and its
floats exactly too, because it restates the same scalar arithmetic with the same compiler.
"""
import ctypes as C
import hashlib

import numpy as np
import pytest
from helpers import OracleEngine, greedy_stream, ora, synth

O = ora.load_oracle()
P = ora.ptr


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def gemv_weights(g, name):
    N, K = (int(v) for v in g[f"{name}_shape"])
    if f"{name}_w" in g.files:
        return g[f"{name}_w"], N, K
    rng = np.random.default_rng([11, N, K])
    w = synth.random_tl1_packed(rng, N, K)
    assert sha(w) == str(g[f"{name}_wsha"]), "seeded weight generator drifted from the fixture"
    return w, N, K


@pytest.mark.parametrize("name", ["k2", "k64", "ragged", "mid", "cfg0", "down"])
def test_tl1_gemv_matches_reference_vectors(golden, name):
    g = golden["tl1_gemv"]
    w, N, K = gemv_weights(g, name)
    x = g[f"{name}_x"]
    out, acc = np.zeros(N, np.float32), np.zeros(N, np.int32)
    inv = O.ora_bitlinear_tl1(P(x, ora.c_f32p), P(w, ora.c_u8p), N, K, float(g[f"{name}_scale"]), P(out, ora.c_f32p), P(acc, ora.c_i32p))
    assert np.float32(inv) == g[f"{name}_inv"]
    assert np.array_equal(acc, g[f"{name}_acc"])
    assert np.array_equal(out, g[f"{name}_out"])
    # the table lookup is a plain integer dot product in disguise: check that too
    a = np.zeros(K, np.int8)
    O.ora_act_quant31(P(x, ora.c_f32p), K, P(a, ora.c_i8p))
    assert np.array_equal(synth.unpack_tl1(w, N, K).astype(np.int32) @ a.astype(np.int32), acc)


@pytest.mark.parametrize("dim", [64, 100, 2560, 6912])
def test_rmsnorm_and_quantiser(golden, dim):
    g = golden["rmsnorm_quant"]
    x, w = g[f"d{dim}_x"], g[f"d{dim}_w"]
    y = np.zeros(dim, np.float32)
    O.ora_rms_norm(P(x, ora.c_f32p), P(w, ora.c_f32p), P(y, ora.c_f32p), dim, 1e-5)
    assert np.array_equal(y, g[f"d{dim}_y"])
    a = np.zeros(dim, np.int8)
    inv = O.ora_act_quant31(P(y, ora.c_f32p), dim, P(a, ora.c_i8p))
    assert np.array_equal(a, g[f"d{dim}_a"]) and np.float32(inv) == g[f"d{dim}_inv"]
    assert np.abs(a).max() == 31


def attention_inputs(g):
    L, nq, nkv, hd, ms, steps = (int(v) for v in g["dims"])
    rng = np.random.default_rng(13)
    q = rng.standard_normal((steps, nq * hd)).astype(np.float32)
    k = rng.standard_normal((steps, nkv * hd)).astype(np.float32)
    v = rng.standard_normal((steps, nkv * hd)).astype(np.float32)
    assert sha(np.concatenate([q, k, v], axis=1)) == str(g["qkv_sha"]), "seeded generator drifted from the fixture"
    return (L, nq, nkv, hd, ms, steps), q, k, v


def test_attention_sequence(golden):
    g = golden["attention"]
    (L, nq, nkv, hd, ms, steps), q, k, v = attention_inputs(g)
    ck = np.zeros(L * nkv * ms * hd, np.int8)
    cv = np.zeros_like(ck)
    sk = np.zeros(L * nkv * ms, np.float32)
    sv = np.zeros_like(sk)
    keep = {int(t): i for i, t in enumerate(g["keep"])}
    for t in range(steps):
        qq, kk, vv, o = q[t].copy(), k[t].copy(), v[t].copy(), np.zeros(nq * hd, np.float32)
        O.ora_attention_int8(1, t, nq, nkv, hd, ms, 10000.0, P(qq, ora.c_f32p), P(kk, ora.c_f32p), P(vv, ora.c_f32p),
                             P(o, ora.c_f32p), P(ck, ora.c_i8p), P(cv, ora.c_i8p), P(sk, ora.c_f32p), P(sv, ora.c_f32p))
        if t in keep:
            assert np.array_equal(o, g["outs"][keep[t]]), f"attention output differs at position {t}"
    assert np.array_equal(ck.reshape(L, nkv, ms, hd)[1, :, :steps], g["cache_k"])
    assert np.array_equal(cv.reshape(L, nkv, ms, hd)[1, :, :steps], g["cache_v"])
    assert np.array_equal(sk.reshape(L, nkv, ms)[1, :, :steps], g["scale_k"])
    assert np.array_equal(sv.reshape(L, nkv, ms)[1, :, :steps], g["scale_v"])
    assert not ck.reshape(L, nkv, ms, hd)[0].any(), "layer 0 of the cache must stay untouched"


def paged_attention_inputs(g):
    L, nq, nkv, hd, blocks, steps, layer = (int(v) for v in g["dims"])
    rng = np.random.default_rng(15)
    order = rng.permutation(blocks).astype(np.int32)
    q = rng.standard_normal((steps, nq * hd)).astype(np.float32)
    q[::7] *= 4.0
    k = rng.standard_normal((steps, nkv * hd)).astype(np.float32)
    v = rng.standard_normal((steps, nkv * hd)).astype(np.float32)
    assert sha(np.concatenate([q, k, v], axis=1)) == str(g["qkv_sha"]) and np.array_equal(order, g["order"])
    return (L, nq, nkv, hd, blocks, steps, layer), order, q, k, v


def test_paged_attention_sequence(golden):
    g = golden["attention_paged"]
    (L, nq, nkv, hd, blocks, steps, layer), order, q, k, v = paged_attention_inputs(g)
    rows = blocks * L * nkv * 16
    pk, pv = np.zeros(rows * hd, np.int8), np.zeros(rows * hd, np.int8)
    psk, psv = np.ones(rows, np.float32), np.ones(rows, np.float32)      # the reference presets scales to 1
    keep = {int(t): i for i, t in enumerate(g["keep"])}
    for t in range(steps):
        qq, kk, vv, o = q[t].copy(), k[t].copy(), v[t].copy(), np.zeros(nq * hd, np.float32)
        O.ora_attention_paged_int8(layer, t, nq, nkv, hd, L, 10000.0, P(qq, ora.c_f32p), P(kk, ora.c_f32p), P(vv, ora.c_f32p),
                                   P(o, ora.c_f32p), P(pk, ora.c_i8p), P(pv, ora.c_i8p), P(psk, ora.c_f32p), P(psv, ora.c_f32p),
                                   P(order, ora.c_i32p))
        if t in keep:
            assert np.array_equal(o, g["outs"][keep[t]]), f"paged attention output differs at position {t}"
    assert np.array_equal(pk.reshape(g["pool_k"].shape), g["pool_k"]) and np.array_equal(pv.reshape(g["pool_v"].shape), g["pool_v"])
    assert np.array_equal(psk.reshape(g["scale_k"].shape), g["scale_k"]) and np.array_equal(psv.reshape(g["scale_v"].shape), g["scale_v"])


def test_paged_engine_tiny_stream(golden):
    g = golden["engine_paged"]
    e = OracleEngine(synth.SyntheticModel(synth.TINY, seed=3), kv_mode="paged_int8")
    assert np.array_equal(greedy_stream(e, g["tiny_prompt"], 32), g["tiny_tokens"])
    assert np.array_equal(e.buffer("logits", 1024), g["tiny_logits"])
    assert np.array_equal(e.buffer("attn_out", 256), g["tiny_attn_out"])
    e.close()


def test_lm_head(golden):
    g = golden["lm_head"]
    w, s, x, fn = g["w"], g["s"], g["x"], g["final_norm"]
    V, H = w.shape
    y, x8 = np.zeros(H, np.float32), np.zeros(H, np.int8)
    O.ora_rms_norm(P(x, ora.c_f32p), P(fn, ora.c_f32p), P(y, ora.c_f32p), H, 1e-5)
    sx = O.ora_act_quant127(P(y, ora.c_f32p), H, P(x8, ora.c_i8p))
    assert np.array_equal(x8, g["x8"])
    lg = np.zeros(V, np.float32)
    O.ora_lm_head_i8(P(x8, ora.c_i8p), sx, P(w, ora.c_i8p), P(s, ora.c_f32p), V, H, P(lg, ora.c_f32p), None)
    assert np.array_equal(lg, g["logits"])


def test_engine_tiny_stream_and_sampler(golden):
    g = golden["engine_tiny"]
    m = synth.SyntheticModel(synth.TINY, seed=3)
    assert sha(m.lm_w) == str(g["lm_sha"]) and sha(m.layers[0]["q_w"]) == str(g["l0q_sha"])
    e = OracleEngine(m)
    toks = greedy_stream(e, g["prompt"], 32)
    assert np.array_equal(toks, g["tokens"])
    assert np.array_equal(e.buffer("logits", 1024), g["logits"])
    assert np.array_equal(e.buffer("x", 256), g["x"])
    assert e.seq_len() == 16 - 1 + 32
    s = golden["sampler"]
    nxt = e.generate(int(toks[-1]), temperature=0.0, rep=1.3, past=s["past"])
    assert nxt == int(s["next_penalised"])
    assert np.array_equal(e.buffer("logits", 1024), s["logits_after"])
    e.close()


def test_pack_roundtrip_and_checkpoint_rows():
    rng = np.random.default_rng(21)
    N, K = 192, 70
    t = rng.integers(-1, 2, (N, K)).astype(np.int8)
    p = np.zeros(N * K // 4, np.uint8)
    O.ora_tl1_pack(P(t, ora.c_i8p), N, K, P(p, ora.c_u8p))
    assert np.array_equal(p, synth.pack_tl1(t))
    back = np.zeros_like(t)
    O.ora_tl1_unpack(P(p, ora.c_u8p), N, K, P(back, ora.c_i8p))
    assert np.array_equal(back, t)
    assert set(np.unique(p & 15)) <= {0, 1, 2, 4, 5, 6, 8, 9, 10}
    # checkpoint form: [N/4][K], row r in bits 2*(r%4)
    raw = np.zeros((N // 4, K), np.uint8)
    for r in range(N):
        raw[r // 4] |= ((t[r] + 1).astype(np.uint8) << (2 * (r % 4)))
    p2 = np.zeros_like(p)
    O.ora_tl1_pack_from_rows2bit(P(raw, ora.c_u8p), N, K, P(p2, ora.c_u8p))
    assert np.array_equal(p2, p)


def test_sampler_stochastic_path_is_a_distribution():
    rng = np.random.default_rng(5)
    lg = rng.standard_normal(1000).astype(np.float32) * 3
    order = np.argsort(lg)[::-1]
    seen = set()
    for u in np.linspace(0.0, 1.0, 41):
        l = lg.copy()
        seen.add(O.ora_sample(P(l, ora.c_f32p), 1000, 0.7, 0.9, 40, 1.0, None, 0, float(u)))
    assert seen <= set(order[:40].tolist()) and int(order[0]) in seen
    l = lg.copy()
    assert O.ora_sample(P(l, ora.c_f32p), 1000, 0.7, 0.9, 1, 1.0, None, 0, 0.999) == int(order[0])
