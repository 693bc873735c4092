"""kv_mode "paged_int8" on the GPU: the attention kernel through a block table and the engine with block pools,
against the reference's PagedKVCache (golden vectors from the compiled reference, the C restatement elsewhere).
Floats are compared with `==`; the paged cache's arithmetic is not the contiguous cache's, so these outputs differ
from the int8_fused ones by design."""
import hashlib

import numpy as np
import pytest
import torch
from gpu_helpers import dev, host
from helpers import best_cpu_engine, greedy_stream, ora, synth
from test_gpu_engine import GpuAsCpuApi, gpu_engine
from test_gpu_norm_attn_lm import rope_tables
from test_oracle_golden import paged_attention_inputs

pytestmark = pytest.mark.gpu
P = ora.ptr


def oracle_paged(O, layer, pos, nq, nkv, L, q, k, v, pk, pv, psk, psv, table):
    qq, kk, vv, o = q.copy(), k.copy(), v.copy(), np.zeros(nq * 128, np.float32)
    O.ora_attention_paged_int8(layer, pos, nq, nkv, 128, L, 10000.0, P(qq, ora.c_f32p), P(kk, ora.c_f32p), P(vv, ora.c_f32p),
                               P(o, ora.c_f32p), P(pk, ora.c_i8p), P(pv, ora.c_i8p), P(psk, ora.c_f32p), P(psv, ora.c_f32p),
                               P(table, ora.c_i32p))
    return o


def test_paged_attention_token_by_token_against_reference_vectors(cuda_lib, golden):
    """300 tokens appended one by one through a scattered block table: the reference's outputs at the kept positions,
    the restatement's at every position, and the reference's pools at the end."""
    from tenzo_b200 import kernels
    O = ora.load_oracle()
    g = golden["attention_paged"]
    (L, nq, nkv, hd, blocks, steps, layer), order, q, k, v = paged_attention_inputs(g)
    rows = blocks * L * nkv * 16
    pk = torch.zeros(blocks, L, nkv, 16, hd, dtype=torch.int8, device="cuda")
    pv = torch.zeros_like(pk)
    psk = torch.ones(blocks, L, nkv, 16, dtype=torch.float32, device="cuda")
    psv = torch.ones_like(psk)
    opk, opv = np.zeros(rows * hd, np.int8), np.zeros(rows * hd, np.int8)
    opsk, opsv = np.ones(rows, np.float32), np.ones(rows, np.float32)
    cs, sn = rope_tables(blocks * 16, 10000.0)
    dcs, dsn, table = dev(cs), dev(sn), dev(order[None].copy())
    keep = {int(t): i for i, t in enumerate(g["keep"])}
    for t in range(steps):
        out = kernels.attention_int8(dev(q[t][None]), dev(k[t][None]), dev(v[t][None]), pk, pv, psk, psv,
                                     torch.tensor([t], dtype=torch.int32, device="cuda"), layer=layer, n_q=nq, n_kv=nkv,
                                     max_seq=blocks * 16, rope_cos=dcs, rope_sin=dsn, max_len=t + 1, block_table=table, n_layers=L)
        o = oracle_paged(O, layer, t, nq, nkv, L, q[t], k[t], v[t], opk, opv, opsk, opsv, order)
        assert np.array_equal(host(out)[0], o), f"position {t}"
        if t in keep:
            assert np.array_equal(host(out)[0], g["outs"][keep[t]]), f"reference output, position {t}"
    assert np.array_equal(host(pk), g["pool_k"]) and np.array_equal(host(pv), g["pool_v"])
    assert np.array_equal(host(psk), g["scale_k"]) and np.array_equal(host(psv), g["scale_v"])
    assert cuda_lib.tenzo_cuda_attention_take_timeouts() == 0


@pytest.mark.parametrize("nq,nkv", [(8, 2), (8, 1), (4, 4)])
@pytest.mark.parametrize("heads_per_cta", [0, 1, 2, 4, 8])
@pytest.mark.parametrize("tiles", [2, 1])
def test_paged_attention_many_sequences_share_one_pool(cuda_lib, nq, nkv, heads_per_cta, tiles):
    """Ragged lengths, interleaved blocks of several sequences in one pool, every heads-per-CTA variant, with and
    without the append; keys read per lane through the table (tiles = 2) and as TMA tiles of four blocks (tiles = 1)."""
    from tenzo_b200 import kernels
    if tiles == 1 and heads_per_cta == 8 and nq // nkv == 8:
        pytest.skip("eight heads per CTA exist only with per-lane loads")
    O = ora.load_oracle()
    L, layer, per_seq = 3, 2, 41
    lens = [1, 15, 16, 17, 63, 64, 65, 128, 129, 257, 300, 640]
    B = len(lens)
    blocks = B * per_seq
    rng = np.random.default_rng([61, nq, nkv])
    table = rng.permutation(blocks).astype(np.int32).reshape(B, per_seq)
    pk = rng.integers(-127, 128, (blocks, L, nkv, 16, 128)).astype(np.int8)
    pv = rng.integers(-127, 128, (blocks, L, nkv, 16, 128)).astype(np.int8)
    psk = (0.01 + 0.02 * rng.random((blocks, L, nkv, 16))).astype(np.float32)
    psv = (0.01 + 0.02 * rng.random((blocks, L, nkv, 16))).astype(np.float32)
    q = rng.standard_normal((B, nq * 128)).astype(np.float32)
    q[::2] *= 3.0                                    # peaked rows: weights under the 1e-7 cut
    k = rng.standard_normal((B, nkv * 128)).astype(np.float32)
    v = rng.standard_normal((B, nkv * 128)).astype(np.float32)
    cs, sn = rope_tables(per_seq * 16, 10000.0)
    pos = np.array([n - 1 for n in lens], np.int32)
    dpk, dpv, dsk, dsv = dev(pk), dev(pv), dev(psk), dev(psv)
    common = dict(layer=layer, n_q=nq, n_kv=nkv, max_seq=per_seq * 16, rope_cos=dev(cs), rope_sin=dev(sn), heads_per_cta=heads_per_cta,
                  block_table=dev(table), n_layers=L, tiles=tiles)
    out = kernels.attention_int8(dev(q), dev(k), dev(v), dpk, dpv, dsk, dsv, dev(pos), **common)
    torch.cuda.synchronize()
    opk, opv, osk, osv = pk.reshape(-1).copy(), pv.reshape(-1).copy(), psk.reshape(-1).copy(), psv.reshape(-1).copy()
    for b in range(B):
        o = oracle_paged(O, layer, int(pos[b]), nq, nkv, L, q[b], k[b], v[b], opk, opv, osk, osv, table[b])
        assert np.array_equal(host(out)[b], o), f"sequence {b} (length {lens[b]})"
    assert np.array_equal(host(dpk).reshape(-1), opk) and np.array_equal(host(dpv).reshape(-1), opv)
    assert np.array_equal(host(dsk).reshape(-1), osk) and np.array_equal(host(dsv).reshape(-1), osv)
    # the pools now hold every sequence's new token: the same queries without the append must give the same outputs
    again = kernels.attention_int8(dev(q), None, None, dpk, dpv, dsk, dsv, dev(pos), append=False, **common)
    assert np.array_equal(host(again), host(out))
    assert np.array_equal(host(dpk).reshape(-1), opk) and np.array_equal(host(dsv).reshape(-1), osv)
    assert cuda_lib.tenzo_cuda_attention_take_timeouts() == 0


def test_paged_attention_tma_tiles_long_context(cuda_lib):
    """Contexts long enough that a scoring warp refills its two-stage ring several times (12 warps x 64 keys x 2 stages =
    1536 keys), blocks scattered over the pool, GQA group 4."""
    from tenzo_b200 import kernels
    O = ora.load_oracle()
    nq, nkv, L, layer, per_seq = 8, 2, 2, 0, 200
    lens = [1, 1536, 1537, 2000, 3100, 3137]
    B = len(lens)
    blocks = B * per_seq
    rng = np.random.default_rng(62)
    table = rng.permutation(blocks).astype(np.int32).reshape(B, per_seq)
    pk = rng.integers(-127, 128, (blocks, L, nkv, 16, 128)).astype(np.int8)
    pv = rng.integers(-127, 128, (blocks, L, nkv, 16, 128)).astype(np.int8)
    psk = (0.01 + 0.02 * rng.random((blocks, L, nkv, 16))).astype(np.float32)
    psv = (0.01 + 0.02 * rng.random((blocks, L, nkv, 16))).astype(np.float32)
    q = rng.standard_normal((B, nq * 128)).astype(np.float32)
    k = rng.standard_normal((B, nkv * 128)).astype(np.float32)
    v = rng.standard_normal((B, nkv * 128)).astype(np.float32)
    cs, sn = rope_tables(per_seq * 16, 10000.0)
    pos = np.array([n - 1 for n in lens], np.int32)
    outs = {}
    for tiles in (1, 2):
        dpk, dpv, dsk, dsv = dev(pk), dev(pv), dev(psk), dev(psv)
        outs[tiles] = host(kernels.attention_int8(dev(q), dev(k), dev(v), dpk, dpv, dsk, dsv, dev(pos), layer=layer, n_q=nq, n_kv=nkv,
                                                  max_seq=per_seq * 16, rope_cos=dev(cs), rope_sin=dev(sn), block_table=dev(table),
                                                  n_layers=L, tiles=tiles))
    assert np.array_equal(outs[1], outs[2])
    opk, opv, osk, osv = pk.reshape(-1).copy(), pv.reshape(-1).copy(), psk.reshape(-1).copy(), psv.reshape(-1).copy()
    for b in range(B):
        o = oracle_paged(O, layer, int(pos[b]), nq, nkv, L, q[b], k[b], v[b], opk, opv, osk, osv, table[b])
        assert np.array_equal(outs[1][b], o), f"sequence {b} (length {lens[b]})"
    assert np.array_equal(host(dpk).reshape(-1), opk) and np.array_equal(host(dsk).reshape(-1), osk)
    assert cuda_lib.tenzo_cuda_attention_take_timeouts() == 0


def paged_engine(model, **kw):
    return gpu_engine(model, kv_mode="paged_int8", **kw)


@pytest.mark.parametrize("graph,pdl", [(0, 0), (1, 1)])
def test_paged_engine_tiny_stream_matches_reference_fixture(cuda_lib, golden, graph, pdl):
    g = golden["engine_paged"]
    m = synth.SyntheticModel(synth.TINY, seed=3)
    with paged_engine(m, use_graph=graph, use_pdl=pdl) as e:
        toks = greedy_stream(GpuAsCpuApi(e), g["tiny_prompt"], 32)
        assert np.array_equal(toks, g["tiny_tokens"])
        assert np.array_equal(e.read_buffer(15), g["tiny_logits"]) and np.array_equal(e.read_buffer(5), g["tiny_attn_out"])
        assert e.get_seq_len() == 15 + 32
        e.reset()                                          # blocks go back to the free list; the same stream comes out again
        assert e.get_seq_len() == 0
        for t in g["tiny_prompt"][:-1]:
            e.prefill_token(int(t))
        assert np.array_equal(e.decode_greedy([int(g["tiny_prompt"][-1])], 32)[:, 0], g["tiny_tokens"])


def test_paged_engine_bitnet_2b_shape_first_32_tokens(cuda_lib, golden):
    """BitNet-2B shape in paged_int8 mode: the reference's own 32 greedy tokens and bit-identical logits. The int8_fused
    stream of the same model and prompt is a different one (the two caches round differently), so this cannot pass by
    running the contiguous cache's arithmetic through a block table."""
    g, fused = golden["engine_paged"], golden["engine_2b"]
    assert not np.array_equal(g["b2_tokens"], fused["tokens"])
    m = synth.SyntheticModel(dict(synth.BITNET_2B, max_seq_len=256), seed=0)
    with paged_engine(m, max_seq_len=256) as e:
        toks = greedy_stream(GpuAsCpuApi(e), g["b2_prompt"], 32)
        assert np.array_equal(toks, g["b2_tokens"]), f"first mismatch at {int(np.argmax(toks != g['b2_tokens']))}"
        lg = e.read_buffer(15)
        assert np.array_equal(lg[g["b2_top_idx"]], g["b2_top_val"])
        assert hashlib.sha256(lg.tobytes()).hexdigest() == str(g["b2_logits_sha"])
        assert hashlib.sha256(e.read_buffer(5).tobytes()).hexdigest() == str(g["b2_attn_out_sha"])


def test_paged_engine_batched_and_chunked_prefill(cuda_lib):
    """Sequences that share the block pool (their blocks interleave) against one CPU engine per sequence, through the
    tensor-core paths (32 sequences); chunked prefill in paged mode against token-by-token prefill; KV export and import
    through the block table."""
    cfg = dict(synth.TINY, hidden_size=512, num_q_heads=4, num_kv_heads=2, ffn_dim=768, num_layers=2, vocab_size=2048, max_seq_len=128)
    m = synth.SyntheticModel(cfg, seed=43)
    B, npre, ngen = 32, 20, 20
    prompts = np.stack([synth.prompt_tokens(300 + b, npre, cfg["vocab_size"]) for b in range(B)])
    with paged_engine(m, batch=B, max_seq_len=128) as e:
        for t in range(npre - 1):
            e.prefill_tokens(prompts[:, t])
        got = e.decode_greedy(prompts[:, -1], ngen).T                      # [B][ngen]
        assert [e.seq_len(b) for b in range(B)] == [npre - 1 + ngen] * B
        exported = e.kv_export(5, 1, npre - 1 + ngen)
    for b in (0, 5, 31):
        cpu = best_cpu_engine(m, max_seq_len=128, kv_mode="paged_int8")
        assert np.array_equal(greedy_stream(cpu, prompts[b], ngen), got[b]), f"sequence {b}"
        cpu.close()
    prompt = prompts[5]
    with paged_engine(m, max_seq_len=128) as one:
        for t in prompt[:-1]:
            one.prefill_token(int(t))
        kv_tok = one.kv_export(0, 1, npre - 1)
        assert np.array_equal(one.decode_greedy([int(prompt[-1])], ngen)[:, 0], got[5])
        for a, b_ in zip(one.kv_export(0, 1, npre - 1 + ngen), exported):
            assert np.array_equal(a, b_), "a sequence's cache does not depend on which blocks it got"
    for chunks in ([19], [3, 16]):
        with paged_engine(m, max_seq_len=128) as e:
            at = 0
            for c in chunks:
                e.prefill_chunk(prompt[at:at + c])
                at += c
            for a, b_ in zip(e.kv_export(0, 1, npre - 1), kv_tok):
                assert np.array_equal(a, b_), f"chunks {chunks}"
            assert np.array_equal(e.decode_greedy([int(prompt[-1])], ngen)[:, 0], got[5]), f"chunks {chunks}"
    # import: a fresh engine given sequence 5's cache continues as sequence 5 did
    with paged_engine(m, max_seq_len=128) as src, paged_engine(m, batch=2, max_seq_len=128) as dst:
        for t in prompt[:-1]:
            src.prefill_token(int(t))
        for l in range(cfg["num_layers"]):
            for s in range(2):
                dst.kv_import(s, l, *src.kv_export(0, l, npre - 1))
        for s in range(2):
            dst.set_seq_len(s, npre - 1)
        out = dst.decode_greedy([int(prompt[-1])] * 2, ngen)
        assert np.array_equal(out[:, 0], got[5]) and np.array_equal(out[:, 1], got[5])


def test_paged_engine_refuses_tokens_past_max_seq_len_and_unknown_kv_modes(cuda_lib):
    from tenzo_b200.engine import Engine
    m = synth.SyntheticModel(synth.TINY, seed=3)
    with paged_engine(m, max_seq_len=32) as e:
        for t in range(32):
            e.prefill_token(t)
        with pytest.raises(RuntimeError):
            e.prefill_token(1)
    with pytest.raises(RuntimeError):
        Engine(m.config_struct(kv_mode="tl1_fused"))
