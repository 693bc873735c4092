"""Tolerance-mode attention (tenzo_attention_args.mode = 1) against the CPU oracle and the exact-order kernel.

The exact kernel is compared with `==` elsewhere; this mode is free to reorder, so its outputs are held to the
tolerance the specification gives floating-point outputs: 1e-3 relative, normalised by the output's largest
magnitude (measured: about 1e-4). What must still be exact: the int8 row and the scale it appends to the cache
(FusedKVCache append, src/runtime/TenzoEngine.cpp:507-533 of the reference), whatever the mode."""
import numpy as np
import pytest
import torch
from gpu_helpers import dev, host
from helpers import ora, rel_err

pytestmark = pytest.mark.gpu
P = ora.ptr
FP_TOL = 1e-3


def rope_tables(max_seq, theta=10000.0):
    O = ora.load_oracle()
    cs, sn = np.zeros((max_seq, 64), np.float32), np.zeros((max_seq, 64), np.float32)
    for p in range(max_seq):
        O.ora_rope_table(p, 128, theta, P(cs[p], ora.c_f32p), P(sn[p], ora.c_f32p))
    return cs, sn


def random_cache(B, nkv, ms, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    ck = torch.randint(-127, 128, (B, 1, nkv, ms, 128), generator=g, device="cuda", dtype=torch.int8)
    cv = torch.randint(-127, 128, (B, 1, nkv, ms, 128), generator=g, device="cuda", dtype=torch.int8)
    sk = 0.01 + 0.02 * torch.rand(B, 1, nkv, ms, generator=g, device="cuda")
    sv = 0.01 + 0.02 * torch.rand(B, 1, nkv, ms, generator=g, device="cuda")
    return ck, cv, sk, sv


@pytest.mark.parametrize("B,nq,nkv,lens_cycle,ms,split", [
    (3, 20, 5, [1, 256, 700], 768, 0),                      # group of 4, ragged
    (5, 8, 8, [1, 2, 31, 32, 33], 64, 0),                   # no grouping, lengths around one 32-key block
    (6, 16, 2, [127, 128, 129, 255, 257, 300], 384, 128),   # group of 8, finest split, lengths around the split
    (2, 4, 2, [2048, 1000], 2048, 256),                     # group of 2, several splits
])
def test_against_the_oracle_with_rotation_and_append(cuda_lib, B, nq, nkv, lens_cycle, ms, split):
    from tenzo_b200 import kernels
    O = ora.load_oracle()
    lens = [lens_cycle[i % len(lens_cycle)] for i in range(B)]
    dck, dcv, dsk, dsv = random_cache(B, nkv, ms, 77)
    ck, cv, sk, sv = host(dck), host(dcv), host(dsk), host(dsv)
    rng = np.random.default_rng(53)
    q = rng.standard_normal((B, nq * 128)).astype(np.float32)
    k = rng.standard_normal((B, nkv * 128)).astype(np.float32)
    v = rng.standard_normal((B, nkv * 128)).astype(np.float32)
    cs, sn = rope_tables(ms)
    pos = np.array([n - 1 for n in lens], np.int32)
    out = kernels.attention_int8(dev(q), dev(k), dev(v), dck, dcv, dsk, dsv, dev(pos), layer=0, n_q=nq, n_kv=nkv, max_seq=ms,
                                 rope_cos=dev(cs), rope_sin=dev(sn), mode=1, split_keys=split)
    torch.cuda.synchronize()
    assert cuda_lib.tenzo_cuda_attention_take_timeouts() == 0
    got, gck, gcv, gsk, gsv = host(out), host(dck), host(dcv), host(dsk), host(dsv)
    assert np.isfinite(got).all()
    for b in range(B):
        ock, ocv, osk, osv = ck[b].reshape(-1).copy(), cv[b].reshape(-1).copy(), sk[b].reshape(-1).copy(), sv[b].reshape(-1).copy()
        qq, kk, vv, o = q[b].copy(), k[b].copy(), v[b].copy(), np.zeros(nq * 128, np.float32)
        O.ora_attention_int8(0, int(pos[b]), nq, nkv, 128, ms, 10000.0, P(qq, ora.c_f32p), P(kk, ora.c_f32p), P(vv, ora.c_f32p),
                             P(o, ora.c_f32p), P(ock, ora.c_i8p), P(ocv, ora.c_i8p), P(osk, ora.c_f32p), P(osv, ora.c_f32p))
        assert rel_err(got[b], o) < FP_TOL, f"sequence {b} (length {lens[b]}): rel err {rel_err(got[b], o):.2e}"
        # the appended row and its scales: bit for bit
        assert np.array_equal(gck[b].reshape(-1), ock) and np.array_equal(gcv[b].reshape(-1), ocv)
        assert np.array_equal(gsk[b].reshape(-1), osk) and np.array_equal(gsv[b].reshape(-1), osv)


def test_full_benchmark_shape_against_the_exact_kernel(cuda_lib):
    """Batch 64, 20/5 heads, context 8192 (the attention benchmark's shape), ragged: every sequence within tolerance of
    the exact-order kernel, which other tests pin to the oracle bit for bit; every split choice agrees."""
    from tenzo_b200 import kernels
    B, nq, nkv, ms = 64, 20, 5, 8192
    dck, dcv, dsk, dsv = random_cache(B, nkv, ms, 5)
    g = torch.Generator(device="cuda").manual_seed(6)
    q = torch.randn(B, nq * 128, generator=g, device="cuda")
    pos = torch.tensor([ms - 1 - 97 * (b % 11) for b in range(B)], dtype=torch.int32, device="cuda")
    want = kernels.attention_int8(q, None, None, dck, dcv, dsk, dsv, pos, layer=0, n_q=nq, n_kv=nkv, max_seq=ms, max_len=ms, append=False)
    for split in (0, 512, 8192):
        got = kernels.attention_int8(q, None, None, dck, dcv, dsk, dsv, pos, layer=0, n_q=nq, n_kv=nkv, max_seq=ms, max_len=ms,
                                     append=False, mode=1, split_keys=split)
        torch.cuda.synchronize()
        for b in range(B):
            e = rel_err(host(got[b]), host(want[b]))
            assert e < FP_TOL, f"split {split}, sequence {b}: rel err {e:.2e}"
    assert cuda_lib.tenzo_cuda_attention_take_timeouts() == 0


def test_large_scores_and_tiny_weights(cuda_lib):
    """Peaked softmax (scores tens of units apart) and keys whose weight underflows: no NaN, still within tolerance."""
    from tenzo_b200 import kernels
    B, nq, nkv, ms = 2, 4, 1, 512
    dck, dcv, dsk, dsv = random_cache(B, nkv, ms, 9)
    dsk *= 8.0                                            # scores of order +-12
    g = torch.Generator(device="cuda").manual_seed(10)
    q = 3.0 * torch.randn(B, nq * 128, generator=g, device="cuda")
    pos = torch.tensor([511, 300], dtype=torch.int32, device="cuda")
    want = kernels.attention_int8(q, None, None, dck, dcv, dsk, dsv, pos, layer=0, n_q=nq, n_kv=nkv, max_seq=ms, max_len=ms, append=False)
    got = kernels.attention_int8(q, None, None, dck, dcv, dsk, dsv, pos, layer=0, n_q=nq, n_kv=nkv, max_seq=ms, max_len=ms, append=False,
                                 mode=1, split_keys=128)
    torch.cuda.synchronize()
    assert torch.isfinite(got).all()
    for b in range(B):
        assert rel_err(host(got[b]), host(want[b])) < FP_TOL


def test_mode_is_refused_where_it_does_not_apply(cuda_lib):
    from tenzo_b200 import kernels
    B, nq, nkv, ms = 1, 4, 1, 66                          # max_seq not a multiple of 4: the scale copies need 16-byte rows
    dck, dcv, dsk, dsv = random_cache(B, nkv, ms, 1)
    q = torch.zeros(B, nq * 128, device="cuda")
    pos = torch.tensor([10], dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="rc=-5"):
        kernels.attention_int8(q, None, None, dck, dcv, dsk, dsv, pos, layer=0, n_q=nq, n_kv=nkv, max_seq=ms, append=False, mode=1)


def test_engine_in_tolerance_mode_stays_close_to_the_exact_engine(cuda_lib):
    """A one-layer model through both engines (batch 3, six tokens): the cache bytes are upstream of every attention
    output and must be identical; the attention output is within the tolerance. Deeper models are not compared: the
    +-31 activation quantiser in front of every product turns a last-digit difference into a flipped level now and then,
    and a synthetic ternary network amplifies that (measured 5 % on the second layer's attention output)."""
    from tenzo_b200.engine import Engine
    from helpers import synth
    cfg = dict(hidden_size=512, num_q_heads=4, num_kv_heads=2, head_dim=128, num_layers=1, ffn_dim=1536, vocab_size=4096, max_seq_len=256)
    m = synth.SyntheticModel(cfg, seed=5)
    B = 3
    prompts = np.stack([synth.prompt_tokens(40 + b, 6, cfg["vocab_size"]) for b in range(B)])
    with Engine(m.config_struct(), batch=B).load_synthetic(m) as a, Engine(m.config_struct(), batch=B, attention_mode=1).load_synthetic(m) as b:
        for t in range(5):
            a.prefill_tokens(prompts[:, t])
            b.prefill_tokens(prompts[:, t])
        a.generate_steps(prompts[:, 5])
        b.generate_steps(prompts[:, 5])
        for s in range(B):
            for x, y in zip(a.kv_export(s, 0, 6), b.kv_export(s, 0, 6)):
                assert np.array_equal(x, y)
            assert rel_err(b.read_buffer(5, seq=s), a.read_buffer(5, seq=s)) < FP_TOL
            assert np.isfinite(b.read_buffer(15, seq=s)).all()
