"""Generate tests/golden/*.npz from the UNMODIFIED reference engine compiled by `make -C oracle ref`.

Run where the reference checkout exists:  python tests/golden/make_golden.py
The reference's own tests hold no golden vectors for the quantized decode path, so these
fixtures are outputs of the reference itself on seeded inputs. They travel with the repository;
the compiled reference does not have to.
"""
from __future__ import annotations

import hashlib
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
from helpers import RefEngine, greedy_stream, ora, synth  # noqa: E402

R = ora.load_ref("kernels")
P = ora.ptr


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def gemv_cases():
    out = {}
    cases = [("k2", 64, 2), ("k64", 64, 64), ("ragged", 128, 130), ("mid", 256, 384), ("cfg0", 6912, 2560), ("down", 2560, 6912)]
    for name, N, K in cases:
        rng = np.random.default_rng([11, N, K])
        w = synth.random_tl1_packed(rng, N, K)
        x = rng.standard_normal(K).astype(np.float32)
        scale = synth.weight_scale(rng)
        o = np.zeros(N, np.float32)
        acc = np.zeros(N, np.int32)
        inv = R.refk_bitlinear_tl1(P(x, ora.c_f32p), P(w.view(np.int8), ora.c_i8p), N, K, float(scale), P(o, ora.c_f32p), P(acc, ora.c_i32p))
        out[f"{name}_x"] = x
        out[f"{name}_scale"] = np.float32(scale)
        out[f"{name}_inv"] = np.float32(inv)
        out[f"{name}_acc"] = acc
        out[f"{name}_out"] = o
        out[f"{name}_shape"] = np.array([N, K])
        if N * K <= 256 * 384:
            out[f"{name}_w"] = w
        else:
            out[f"{name}_wsha"] = np.array(sha(w))
    np.savez_compressed(HERE / "tl1_gemv.npz", **out)


def norm_cases():
    out = {}
    for dim in (64, 100, 2560, 6912):
        rng = np.random.default_rng([12, dim])
        x = (3.0 * rng.standard_normal(dim)).astype(np.float32)
        w = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
        y = np.zeros(dim, np.float32)
        R.refk_rms_norm(P(x, ora.c_f32p), P(w, ora.c_f32p), P(y, ora.c_f32p), dim, 1e-5)
        lut = np.zeros(dim // 2 * 32, np.uint8)
        inv = R.refk_build_lut(P(y, ora.c_f32p), dim, P(lut, ora.c_u8p))
        # a0 = T[w0=+1,w1=0] = lut[2 | 1<<2 = 6], a1 = T[w0=0,w1=+1] = lut[1 | 2<<2 = 9]
        t = lut.view(np.int8).reshape(dim // 2, 32)
        a = np.stack([t[:, 6], t[:, 9]], axis=1).reshape(-1)
        out[f"d{dim}_x"], out[f"d{dim}_w"], out[f"d{dim}_y"] = x, w, y
        out[f"d{dim}_a"], out[f"d{dim}_inv"] = a, np.float32(inv)
    np.savez_compressed(HERE / "rmsnorm_quant.npz", **out)


def attention_case():
    L, nq, nkv, hd, ms = 2, 8, 2, 128, 320
    kv = R.refk_kv_create(L, nq, nkv, hd, ms)
    rng = np.random.default_rng(13)
    steps = 300
    q = rng.standard_normal((steps, nq * hd)).astype(np.float32)
    k = rng.standard_normal((steps, nkv * hd)).astype(np.float32)
    v = rng.standard_normal((steps, nkv * hd)).astype(np.float32)
    outs = np.zeros((steps, nq * hd), np.float32)
    for t in range(steps):
        qq, kk, vv = q[t].copy(), k[t].copy(), v[t].copy()
        R.refk_kv_set_len(kv, t)
        R.refk_kv_attention(kv, 1, P(qq, ora.c_f32p), P(kk, ora.c_f32p), P(vv, ora.c_f32p), P(outs[t], ora.c_f32p))
    n = L * nkv * ms
    ck = ora.view(R.refk_kv_k(kv), n * hd, np.int8).reshape(L, nkv, ms, hd)[1, :, :steps].copy()
    cv = ora.view(R.refk_kv_v(kv), n * hd, np.int8).reshape(L, nkv, ms, hd)[1, :, :steps].copy()
    sk = ora.view(R.refk_kv_k_scales(kv), n, np.float32).reshape(L, nkv, ms)[1, :, :steps].copy()
    sv = ora.view(R.refk_kv_v_scales(kv), n, np.float32).reshape(L, nkv, ms)[1, :, :steps].copy()
    keep = [0, 1, 2, 31, 127, 255, 256, 257, 299]
    # q, k, v are regenerated from the seed by the tests (qkv_sha guards against a generator change)
    np.savez_compressed(HERE / "attention.npz", qkv_sha=np.array(sha(np.concatenate([q, k, v], axis=1))), cache_k=ck, cache_v=cv, scale_k=sk, scale_v=sv,
                        keep=np.array(keep), outs=outs[keep], dims=np.array([L, nq, nkv, hd, ms, steps]))
    R.refk_kv_destroy(kv)


def engine_cases():
    # tiny: everything stored
    m = synth.SyntheticModel(synth.TINY, seed=3)
    r = RefEngine(m)
    prompt = synth.prompt_tokens(3, 16, synth.TINY["vocab_size"])
    toks = greedy_stream(r, prompt, 32)
    np.savez_compressed(HERE / "engine_tiny.npz", prompt=prompt, tokens=toks, logits=r.buffer("logits", 1024),
                        x=r.buffer("x", 256), lm_sha=np.array(sha(m.lm_w)), l0q_sha=np.array(sha(m.layers[0]["q_w"])))
    # one sampled (penalised greedy) continuation
    past = np.concatenate([prompt, toks])
    nxt = r.generate(int(toks[-1]), temperature=0.0, rep=1.3, past=past)
    np.savez_compressed(HERE / "sampler.npz", past=past, next_penalised=np.int32(nxt), logits_after=r.buffer("logits", 1024))
    r.close()
    # BitNet-2B shape: 64-token prompt, first 32 greedy tokens (the north-star stream check)
    cfg = dict(synth.BITNET_2B, max_seq_len=256)
    m = synth.SyntheticModel(cfg, seed=0)
    r = RefEngine(m)
    prompt = synth.prompt_tokens(0, 64, cfg["vocab_size"])
    toks = greedy_stream(r, prompt, 32)
    lg = r.buffer("logits", cfg["vocab_size"])
    top = np.argsort(lg)[-16:][::-1]
    np.savez_compressed(HERE / "engine_2b.npz", prompt=prompt, tokens=toks, top_idx=top.astype(np.int32), top_val=lg[top],
                        logits_sha=np.array(sha(lg)), lm_sha=np.array(sha(m.lm_w)), l29down_sha=np.array(sha(m.layers[29]["down_w"])))
    r.close()


def paged_cases():
    """kv_mode "paged_int8": PagedKVCache::forward_attention_raw with the blocks placed out of order, and whole-engine streams."""
    L, nq, nkv, hd, blocks, layer, steps = 2, 8, 2, 128, 20, 1, 300
    rng = np.random.default_rng(15)
    order = rng.permutation(blocks).astype(np.int32)
    kv = R.refk_paged_create(L, nq, nkv, hd, blocks)
    q = rng.standard_normal((steps, nq * hd)).astype(np.float32)
    q[::7] *= 4.0                                   # peaked softmax rows: some weights fall under the 1e-7 cut
    k = rng.standard_normal((steps, nkv * hd)).astype(np.float32)
    v = rng.standard_normal((steps, nkv * hd)).astype(np.float32)
    outs = np.zeros((steps, nq * hd), np.float32)
    for t in range(steps):
        if t % 16 == 0:
            R.refk_paged_push_block(kv, int(order[t // 16]))
        qq, kk, vv = q[t].copy(), k[t].copy(), v[t].copy()
        R.refk_paged_set_len(kv, t)
        R.refk_paged_attention(kv, layer, P(qq, ora.c_f32p), P(kk, ora.c_f32p), P(vv, ora.c_f32p), P(outs[t], ora.c_f32p))
    rows = blocks * L * nkv * 16
    keep = [0, 1, 15, 16, 17, 127, 128, 255, 256, 299]
    np.savez_compressed(HERE / "attention_paged.npz", qkv_sha=np.array(sha(np.concatenate([q, k, v], axis=1))), order=order,
                        pool_k=ora.view(R.refk_paged_k(kv), rows * hd, np.int8).reshape(blocks, L, nkv, 16, hd).copy(),
                        pool_v=ora.view(R.refk_paged_v(kv), rows * hd, np.int8).reshape(blocks, L, nkv, 16, hd).copy(),
                        scale_k=ora.view(R.refk_paged_k_scales(kv), rows, np.float32).reshape(blocks, L, nkv, 16).copy(),
                        scale_v=ora.view(R.refk_paged_v_scales(kv), rows, np.float32).reshape(blocks, L, nkv, 16).copy(),
                        keep=np.array(keep), outs=outs[keep], dims=np.array([L, nq, nkv, hd, blocks, steps, layer]))
    R.refk_paged_destroy(kv)
    # whole engine, tiny shape and BitNet-2B shape (same models and prompts as engine_cases)
    out = {}
    m = synth.SyntheticModel(synth.TINY, seed=3)
    r = RefEngine(m, kv_mode="paged_int8")
    prompt = synth.prompt_tokens(3, 16, synth.TINY["vocab_size"])
    out["tiny_prompt"], out["tiny_tokens"] = prompt, greedy_stream(r, prompt, 32)
    out["tiny_logits"], out["tiny_attn_out"] = r.buffer("logits", 1024), r.buffer("attn_out", 256)
    r.close()
    cfg = dict(synth.BITNET_2B, max_seq_len=256)
    m = synth.SyntheticModel(cfg, seed=0)
    r = RefEngine(m, kv_mode="paged_int8")
    prompt = synth.prompt_tokens(0, 64, cfg["vocab_size"])
    out["b2_prompt"], out["b2_tokens"] = prompt, greedy_stream(r, prompt, 32)
    lg = r.buffer("logits", cfg["vocab_size"])
    top = np.argsort(lg)[-16:][::-1]
    out["b2_top_idx"], out["b2_top_val"], out["b2_logits_sha"] = top.astype(np.int32), lg[top], np.array(sha(lg))
    out["b2_attn_out_sha"] = np.array(sha(r.buffer("attn_out", cfg["hidden_size"])))
    r.close()
    np.savez_compressed(HERE / "engine_paged.npz", **out)


def lm_head_case():
    rng = np.random.default_rng(14)
    V, H = 500, 256
    lat = (0.05 * rng.standard_normal((V, H))).astype(np.float32)
    w, s = synth.quantize_rows_i8(lat)
    x = rng.standard_normal(H).astype(np.float32)
    fn = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    cfg = dict(synth.TINY, hidden_size=H, num_q_heads=2, vocab_size=V)
    m = synth.SyntheticModel(cfg, seed=5)
    m.lm_w, m.lm_scales, m.final_norm = w, s, fn
    r = RefEngine(m)
    r.set_buffer("x", x)
    R.refk_engine_logits(r.h)
    np.savez_compressed(HERE / "lm_head.npz", w=w, s=s, x=x, final_norm=fn, logits=r.buffer("logits", V),
                        x8=ora.view(R.refk_engine_x_i8(r.h), H, np.int8).copy())
    r.close()


if __name__ == "__main__":
    groups = dict(gemv=gemv_cases, norm=norm_cases, attention=attention_case, lm_head=lm_head_case, engine=engine_cases, paged=paged_cases)
    for name in (sys.argv[1:] or list(groups)):      # no arguments: everything; else only the named groups
        groups[name]()
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size)
