"""TL1 GEMV on the GPU through the C ABI against the CPU oracle: int32 accumulators, quantised
activations and the fp32 epilogue must be bit-identical on identical fp32 inputs."""
import hashlib

import numpy as np
import pytest
import torch
from gpu_helpers import cpu_bitlinear, cpu_rms_norm, dev, host
from helpers import ora, rel_err, synth

pytestmark = pytest.mark.gpu
P = ora.ptr


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.mark.parametrize("name", ["k2", "k64", "ragged", "mid", "cfg0", "down"])
def test_against_reference_golden_vectors(cuda_lib, golden, name):
    from tenzo_b200 import kernels
    g = golden["tl1_gemv"]
    N, K = (int(v) for v in g[f"{name}_shape"])
    if f"{name}_w" in g.files:
        w = g[f"{name}_w"]
    else:
        w = synth.random_tl1_packed(np.random.default_rng([11, N, K]), N, K)
        assert sha(w) == str(g[f"{name}_wsha"])
    r = kernels.tl1_gemv(dev(g[f"{name}_x"][None]), dev(w), N // 64, K, [float(g[f"{name}_scale"])], want_acc=True, want_act=True)
    torch.cuda.synchronize()
    assert np.array_equal(host(r["acc"])[0], g[f"{name}_acc"]), "int32 accumulators differ"
    assert np.float32(host(r["inv"])[0]) == g[f"{name}_inv"]
    assert np.array_equal(host(r["out"])[0], g[f"{name}_out"]), "fp32 outputs differ"


@pytest.mark.parametrize("N,K", [(64, 2), (64, 4), (64, 126), (64, 128), (128, 130), (192, 258), (256, 384), (640, 2560),
                                 (2560, 2560), (6912, 2560), (2560, 6912), (4096, 4096), (128, 16384)])
@pytest.mark.parametrize("batch", [1, 3])
def test_bit_exact_on_seeded_inputs(cuda_lib, N, K, batch):
    from tenzo_b200 import kernels
    rng = np.random.default_rng([41, N, K, batch])
    w = synth.random_tl1_packed(rng, N, K)
    x = (rng.standard_normal((batch, K)) * np.float32(10.0) ** rng.integers(-2, 3, (batch, 1))).astype(np.float32)
    scale = float(synth.weight_scale(rng))
    r = kernels.tl1_gemv(dev(x), dev(w), N // 64, K, [scale], want_acc=True, want_act=True)
    torch.cuda.synchronize()
    O = ora.load_oracle()
    for b in range(batch):
        out, acc, inv = cpu_bitlinear(x[b], w, N, K, scale)
        a = np.zeros(K, np.int8)
        O.ora_act_quant31(P(x[b], ora.c_f32p), K, P(a, ora.c_i8p))
        assert np.array_equal(host(r["a"])[b], a), "quantised activations differ"
        assert np.float32(host(r["inv"])[b]) == inv
        assert np.array_equal(host(r["acc"])[b], acc), "int32 accumulators differ"
        assert np.array_equal(host(r["out"])[b], out), "fp32 outputs differ"


def test_edge_activations(cuda_lib):
    """All-zero input (1e-6 floor), a single spike, exact .5 rounding ties, saturating +-31."""
    from tenzo_b200 import kernels
    N, K = 128, 256
    rng = np.random.default_rng(42)
    w = synth.random_tl1_packed(rng, N, K)
    xs = np.zeros((4, K), np.float32)
    xs[1, 17] = -3.0
    xs[2] = np.float32(31.0) * np.sign(rng.standard_normal(K)).astype(np.float32)
    xs[3] = (np.arange(K) % 63 - 31).astype(np.float32) + np.float32(0.5) * (np.arange(K) % 2)
    xs[3, 0] = 31.0
    r = kernels.tl1_gemv(dev(xs), dev(w), N // 64, K, [0.5], want_acc=True)
    torch.cuda.synchronize()
    for b in range(4):
        out, acc, _ = cpu_bitlinear(xs[b], w, N, K, 0.5)
        assert np.array_equal(host(r["acc"])[b], acc) and np.array_equal(host(r["out"])[b], out)
    assert not host(r["acc"])[0].any()


def test_fused_qkv_segments_and_norm(cuda_lib):
    """The q|k|v launch: three scale segments, RMSNorm fused in front (TenzoEngine.cpp:1542-1572)."""
    from tenzo_b200 import kernels
    h, qd, kvd = 2560, 2560, 640
    rng = np.random.default_rng(43)
    ws = [synth.random_tl1_packed(rng, n, h) for n in (qd, kvd, kvd)]
    scales = [0.011, 0.017, 0.023]
    x = (2.5 * rng.standard_normal((2, h))).astype(np.float32)
    nw = (1 + 0.1 * rng.standard_normal(h)).astype(np.float32)
    wcat = np.concatenate(ws)
    nb = (qd + 2 * kvd) // 64
    # teacher-forced: normalise on the CPU, quantise + multiply on the GPU -> exact
    y = np.stack([cpu_rms_norm(x[b], nw) for b in range(2)])
    r = kernels.tl1_gemv(dev(y), dev(wcat), nb, h, scales, [qd // 64, (qd + kvd) // 64, nb], want_acc=True)
    # fused: normalise on the GPU too
    rf = kernels.tl1_gemv(dev(x), dev(wcat), nb, h, scales, [qd // 64, (qd + kvd) // 64, nb], norm_w=dev(nw), do_norm=True)
    torch.cuda.synchronize()
    for b in range(2):
        ref = np.concatenate([cpu_bitlinear(y[b], w, n, h, s)[0] for w, n, s in zip(ws, (qd, kvd, kvd), scales)])
        acc = np.concatenate([cpu_bitlinear(y[b], w, n, h, s)[1] for w, n, s in zip(ws, (qd, kvd, kvd), scales)])
        assert np.array_equal(host(r["acc"])[b], acc)
        assert np.array_equal(host(r["out"])[b], ref)
        assert np.array_equal(host(rf["out"])[b], ref)   # fused norm reproduces the reference's sum order: exact too


def test_residual_and_glu_epilogues(cuda_lib):
    from tenzo_b200 import kernels
    h, f = 512, 704
    rng = np.random.default_rng(44)
    O = ora.load_oracle()
    x = rng.standard_normal((2, h)).astype(np.float32)
    res = rng.standard_normal((2, h)).astype(np.float32)
    wo = synth.random_tl1_packed(rng, h, h)
    r = kernels.tl1_gemv(dev(x), dev(wo), h // 64, h, [0.02], epilogue=kernels.EPI_RESIDUAL, resid=dev(res))
    wg, wu = synth.random_tl1_packed(rng, f, h), synth.random_tl1_packed(rng, f, h)
    g = kernels.tl1_gemv(dev(x), dev(np.concatenate([wg, wu])), 2 * f // 64, h, [0.02, 0.03], [f // 64, 2 * f // 64, 2 * f // 64],
                         epilogue=kernels.EPI_RELU2_GLU)
    torch.cuda.synchronize()
    for b in range(2):
        o = cpu_bitlinear(x[b], wo, h, h, 0.02)[0]
        assert np.array_equal(host(r["out"])[b], res[b] + o)                     # TenzoEngine.cpp:1590
        gate, up = cpu_bitlinear(x[b], wg, f, h, 0.02)[0], cpu_bitlinear(x[b], wu, f, h, 0.03)[0]
        act = np.zeros(f, np.float32)
        O.ora_relu2_glu(P(gate, ora.c_f32p), P(up, ora.c_f32p), P(act, ora.c_f32p), f)
        assert np.array_equal(host(g["out"])[b], act)                            # :1616-1620


def test_properties_at_full_size(cuda_lib):
    """Size-independent checks on the 6912 x 2560 shape: sign symmetry, column-sum identity, and
    back-to-back launches do not leak into each other."""
    from tenzo_b200 import kernels
    N, K = 6912, 2560
    rng = np.random.default_rng(45)
    w = synth.random_tl1_packed(rng, N, K)
    x = rng.standard_normal((1, K)).astype(np.float32)
    dw = dev(w)
    a = kernels.tl1_gemv(dev(x), dw, N // 64, K, [1.0], want_acc=True, want_act=True)
    b = kernels.tl1_gemv(dev(-x), dw, N // 64, K, [1.0], want_acc=True)
    c = kernels.tl1_gemv(dev(x), dw, N // 64, K, [1.0], want_acc=True)
    torch.cuda.synchronize()
    assert np.array_equal(host(a["acc"]), -host(b["acc"]))          # round-half-away is odd-symmetric
    assert np.array_equal(host(a["acc"]), host(c["acc"]))
    colsum = synth.unpack_tl1(w, N, K).astype(np.int64).sum(axis=0)
    assert int(host(a["acc"]).astype(np.int64).sum()) == int(colsum @ host(a["a"])[0].astype(np.int64))


def test_argument_errors(cuda_lib):
    from tenzo_b200 import kernels
    x, w = torch.zeros(1, 64, device="cuda"), torch.zeros(64 * 64 // 4, dtype=torch.uint8, device="cuda")
    with pytest.raises(RuntimeError):
        kernels.tl1_gemv(x, w, 1, 63, [1.0])           # odd K
    with pytest.raises(RuntimeError):
        kernels.tl1_gemv(x, w[1:], 1, 64, [1.0])       # misaligned weights
    with pytest.raises(RuntimeError):
        kernels.tl1_gemv(x, w, 1, 64, [1.0], epilogue=kernels.EPI_RESIDUAL)   # residual missing


@pytest.mark.parametrize("N,K,batch", [(128, 128, 16), (192, 256, 40), (640, 2560, 64), (2560, 6912, 256), (256, 384, 300), (128, 16384, 17)])
def test_tensor_core_path_bit_exact(cuda_lib, N, K, batch):
    """16 or more sequences with K a multiple of 128 run on tcgen05 (codes 0..2 as u8, activations s8,
    int32 accumulators in tensor memory): accumulators, quantised activations and outputs equal the oracle's."""
    from tenzo_b200 import kernels
    rng = np.random.default_rng([45, N, K, batch])
    w = synth.random_tl1_packed(rng, N, K)
    x = (rng.standard_normal((batch, K)) * np.float32(10.0) ** rng.integers(-2, 3, (batch, 1))).astype(np.float32)
    scale = float(synth.weight_scale(rng))
    r = kernels.tl1_gemv(dev(x), dev(w), N // 64, K, [scale], want_acc=True, want_act=True)
    torch.cuda.synchronize()
    assert cuda_lib.tenzo_cuda_tl1_gemv_take_timeouts() == 0
    O = ora.load_oracle()
    check = range(batch) if N * K * batch <= 640 * 2560 * 64 else [0, 1, 15, 16, batch // 2, batch - 2, batch - 1]
    for b in check:
        out, acc, inv = cpu_bitlinear(x[b], w, N, K, scale)
        a = np.zeros(K, np.int8)
        O.ora_act_quant31(P(x[b], ora.c_f32p), K, P(a, ora.c_i8p))
        assert np.array_equal(host(r["a"])[b], a), "quantised activations differ"
        assert np.float32(host(r["inv"])[b]) == inv
        assert np.array_equal(host(r["acc"])[b], acc), f"int32 accumulators differ (sequence {b})"
        assert np.array_equal(host(r["out"])[b], out), "fp32 outputs differ"


@pytest.mark.parametrize("h,B", [(512, 48), (2048, 48), (2048, 144), (512, 240), (2048, 256)])
def test_tensor_core_path_epilogues_match_single_sequence_path(cuda_lib, h, B):
    """Segment scales + fused norm, residual and ReLU^2*GLU epilogues against the same launches made one sequence at a
    time (already pinned to the oracle above). At h = 2048 every one of them splits K across a cluster of four CTAs.
    48, 144 and 240 sequences leave an odd number of 16-sequence column blocks (a store unit of one block, ranks of a
    cluster owning different numbers of blocks); above 128 sequences the kernel runs with four ring slots instead of
    eight or twelve and one chunk per expand iteration."""
    from tenzo_b200 import kernels
    f = 704
    rng = np.random.default_rng([46, h, B])
    x = rng.standard_normal((B, h)).astype(np.float32)
    res = rng.standard_normal((B, h)).astype(np.float32)
    nw = (1 + 0.1 * rng.standard_normal(h)).astype(np.float32)
    wo = dev(synth.random_tl1_packed(rng, h, h))
    wgu = dev(np.concatenate([synth.random_tl1_packed(rng, f, h), synth.random_tl1_packed(rng, f, h)]))
    wqkv = dev(np.concatenate([synth.random_tl1_packed(rng, n, h) for n in (512, 128, 128)]))   # 12 row blocks
    dx, dres, dnw = dev(x), dev(res), dev(nw)

    def launches(xs, rs):
        o = kernels.tl1_gemv(xs, wo, h // 64, h, [0.02], epilogue=kernels.EPI_RESIDUAL, resid=rs, norm_w=dnw, do_norm=True)["out"]
        g = kernels.tl1_gemv(xs, wgu, 2 * f // 64, h, [0.02, 0.03], [f // 64, 2 * f // 64, 2 * f // 64], epilogue=kernels.EPI_RELU2_GLU)["out"]
        q = kernels.tl1_gemv(xs, wqkv, 12, h, [0.011, 0.017, 0.023], [8, 10, 12], norm_w=dnw, do_norm=True)["out"]
        return o, g, q

    big = launches(dx, dres)
    torch.cuda.synchronize()
    for b in sorted({0, 7, 16, 33, 47, B // 2, B - 17, B - 1}):
        one = launches(dx[b:b + 1].contiguous(), dres[b:b + 1].contiguous())
        torch.cuda.synchronize()
        for got, want, name in zip(big, one, ("residual", "glu", "qkv")):
            assert np.array_equal(host(got)[b], host(want)[0]), f"{name} epilogue differs at sequence {b}"
    assert cuda_lib.tenzo_cuda_tl1_gemv_take_timeouts() == 0


def test_many_row_tiles_without_a_cluster_and_more_than_128_sequences(cuda_lib):
    """150 row blocks (more tiles than half the SMs: one CTA per tile, no cluster) at 160 sequences: plain store and
    GLU against the one-sequence path."""
    from tenzo_b200 import kernels
    N, K, B = 9600, 256, 160
    rng = np.random.default_rng(48)
    w = dev(synth.random_tl1_packed(rng, N, K))
    x = dev(rng.standard_normal((B, K)).astype(np.float32))
    assert cuda_lib.tenzo_cuda_tl1_gemm_ksplit(N // 64, K, B, kernels.EPI_STORE) == 1

    def launches(xs):
        s = kernels.tl1_gemv(xs, w, N // 64, K, [0.02])["out"]
        g = kernels.tl1_gemv(xs, w, N // 64, K, [0.02, 0.03], [N // 128, N // 64, N // 64], epilogue=kernels.EPI_RELU2_GLU)["out"]
        return s, g

    big = launches(x)
    torch.cuda.synchronize()
    for b in [0, 15, 16, 127, 128, 143, 159]:
        one = launches(x[b:b + 1].contiguous())
        torch.cuda.synchronize()
        for got, want, name in zip(big, one, ("store", "glu")):
            assert np.array_equal(host(got)[b], host(want)[0]), f"{name} differs at sequence {b}"
    assert cuda_lib.tenzo_cuda_tl1_gemv_take_timeouts() == 0


@pytest.mark.parametrize("batch", [3, 17])
def test_quantiser_paths_agree_on_misaligned_rows(cuda_lib, batch):
    """The batched quantiser keeps 16-byte-aligned rows in registers and walks others element by element: the same
    numbers through an aligned and a 4-byte-shifted buffer give the same quantised activations, scales and products
    (3 sequences: packed mma.sync fragments; 17: the int8 matrix of the tcgen05 path)."""
    from tenzo_b200 import kernels
    N, K = 256, 384
    rng = np.random.default_rng([49, batch])
    w = dev(synth.random_tl1_packed(rng, N, K))
    x = rng.standard_normal((batch, K)).astype(np.float32)
    nw = dev((1 + 0.1 * rng.standard_normal(K)).astype(np.float32))
    aligned = dev(x)
    raw = torch.zeros(batch * K + 1, dtype=torch.float32, device="cuda")
    shifted = raw[1:].view(batch, K)
    shifted.copy_(aligned)
    assert aligned.data_ptr() % 16 == 0 and shifted.data_ptr() % 16 == 4
    a = kernels.tl1_gemv(aligned, w, N // 64, K, [0.02], norm_w=nw, do_norm=True, want_acc=True, want_act=True)
    b = kernels.tl1_gemv(shifted, w, N // 64, K, [0.02], norm_w=nw, do_norm=True, want_acc=True, want_act=True)
    torch.cuda.synchronize()
    for k in ("a", "inv", "acc", "out"):
        assert np.array_equal(host(a[k]), host(b[k])), f"{k} differs between the two quantiser paths"


@pytest.mark.parametrize("world", [4, 8])
def test_tensor_parallel_shard_shapes_match_the_single_sequence_path(cuda_lib, world):
    """The row slices a rank of a 4- or 8-way tensor-parallel 8B-shaped layer multiplies (out, gate|up, down, q|k|v at 32
    sequences: few row tiles, K split over clusters of up to eight CTAs, as few as four 128-byte chunks per CTA) against
    the same launches made one sequence at a time."""
    from tenzo_b200 import kernels
    rng = np.random.default_rng([50, world])
    B, h, f = 32, 4096, 14336
    for name, N, K, epi in (("out", h // world, h, kernels.EPI_RESIDUAL), ("gate|up", 2 * f // world, h, kernels.EPI_RELU2_GLU),
                            ("down", h // world, f, kernels.EPI_RESIDUAL), ("qkv", (32 + 8 + 8) * 128 // world, h, kernels.EPI_STORE)):
        w = dev(synth.random_tl1_packed(rng, N, K))
        x = dev(rng.standard_normal((B, K)).astype(np.float32))
        nw = dev((1 + 0.1 * rng.standard_normal(K)).astype(np.float32))
        n_out = N // 2 if epi == kernels.EPI_RELU2_GLU else N
        res = dev(rng.standard_normal((B, n_out)).astype(np.float32)) if epi == kernels.EPI_RESIDUAL else None
        nb = N // 64
        seg = [nb // 2, nb, nb] if epi == kernels.EPI_RELU2_GLU else [nb, nb, nb]

        def run(xs, rs):
            return kernels.tl1_gemv(xs, w, nb, K, [0.02, 0.03], seg, epilogue=epi, resid=rs, norm_w=nw, do_norm=True)["out"]

        big = run(x, res)
        torch.cuda.synchronize()
        for b in (0, 15, 16, 31):
            one = run(x[b:b + 1].contiguous(), res[b:b + 1].contiguous() if res is not None else None)
            torch.cuda.synchronize()
            assert torch.equal(big[b], one[0]), f"{name} slice of a {world}-rank layer differs at sequence {b}"
    assert cuda_lib.tenzo_cuda_tl1_gemv_take_timeouts() == 0
