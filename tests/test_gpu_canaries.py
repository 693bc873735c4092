"""Out-of-bounds writes, checked without a memory checker: every output, cache and workspace buffer a kernel is given
sits between two 256-byte guard regions that must come back untouched (gpu_helpers.Guarded). Shapes are the awkward ones:
K of 2, 4, 126 and 130 columns (ragged last set: the product loop reads stale shared memory there, so it matters that its
WRITES stay in bounds), batch tails around the 8-, 16- and 32-sequence tile sizes, ragged attention lengths, a vocabulary
that is not a multiple of anything. Results are also compared with a plain run."""
import numpy as np
import pytest
import torch
from gpu_helpers import Guarded, dev
from helpers import synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("K", [2, 4, 126, 130, 2560])
@pytest.mark.parametrize("batch", [1, 3, 9, 17, 33])
@pytest.mark.parametrize("epilogue", [0, 1, 2])
def test_tl1_product_writes_stay_inside_its_buffers(cuda_lib, K, batch, epilogue):
    from tenzo_b200 import kernels
    rng = np.random.default_rng(K * 100 + batch)
    N = 128
    w = dev(synth.random_tl1_packed(rng, N, K))
    x = dev(rng.standard_normal((batch, K)).astype(np.float32))
    n_out = N // 2 if epilogue == 2 else N
    resid = dev(rng.standard_normal((batch, n_out)).astype(np.float32)) if epilogue == 1 else None
    nw = dev((1 + 0.1 * rng.standard_normal(K)).astype(np.float32))
    want = kernels.tl1_gemv(x, w, N // 64, K, [0.016, 0.02], [1, 2, 2], epilogue=epilogue, resid=resid, norm_w=nw, do_norm=True)["out"]
    g = Guarded()
    out = g.empty((batch, n_out), torch.float32)
    ws = g.empty((cuda_lib.tenzo_cuda_tl1_gemv_workspace_bytes(batch, K),), torch.uint8) if batch > 1 else None
    kernels.tl1_gemv(x, w, N // 64, K, [0.016, 0.02], [1, 2, 2], epilogue=epilogue, resid=resid, norm_w=nw, do_norm=True, out=out, workspace=ws)
    g.check()
    assert torch.equal(out, want)


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("B,lens", [(1, [1]), (3, [1, 256, 700]), (70, [1, 2, 63, 64, 65, 127, 128, 129, 255, 257])])
def test_attention_writes_stay_inside_its_buffers(cuda_lib, mode, B, lens):
    from tenzo_b200 import kernels
    nq, nkv, ms = 8, 2, 704
    lens = [lens[i % len(lens)] for i in range(B)]
    gen = torch.Generator(device="cuda").manual_seed(B)
    g = Guarded()
    ck = g.empty((B, 1, nkv, ms, 128), torch.int8, torch.randint(-127, 128, (B, 1, nkv, ms, 128), generator=gen, device="cuda", dtype=torch.int8))
    cv = g.empty((B, 1, nkv, ms, 128), torch.int8, torch.randint(-127, 128, (B, 1, nkv, ms, 128), generator=gen, device="cuda", dtype=torch.int8))
    sk = g.empty((B, 1, nkv, ms), torch.float32, 0.01 + 0.02 * torch.rand(B, 1, nkv, ms, generator=gen, device="cuda"))
    sv = g.empty((B, 1, nkv, ms), torch.float32, 0.01 + 0.02 * torch.rand(B, 1, nkv, ms, generator=gen, device="cuda"))
    out = g.empty((B, nq * 128), torch.float32)
    ws = g.empty((kernels.attention_workspace_bytes(B, nq, nkv, ms),), torch.uint8) if mode == 1 else None
    q = torch.randn(B, nq * 128, generator=gen, device="cuda")
    k = torch.randn(B, nkv * 128, generator=gen, device="cuda")
    v = torch.randn(B, nkv * 128, generator=gen, device="cuda")
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device="cuda")
    before = [t.clone() for t in (ck, cv, sk, sv)]
    kernels.attention_int8(q, k, v, ck, cv, sk, sv, pos, layer=0, n_q=nq, n_kv=nkv, max_seq=ms, max_len=ms, out=out, mode=mode, workspace=ws)
    g.check()
    assert cuda_lib.tenzo_cuda_attention_take_timeouts() == 0
    assert bool(torch.isfinite(out).all())
    # inside the caches only the appended rows changed
    for b in range(B):
        keep = torch.ones(ms, dtype=torch.bool, device="cuda")
        keep[lens[b] - 1] = False
        for now, was in zip((ck, cv), before[:2]):
            assert torch.equal(now[b, 0][:, keep], was[b, 0][:, keep])
        for now, was in zip((sk, sv), before[2:]):
            assert torch.equal(now[b, 0][:, keep], was[b, 0][:, keep])


@pytest.mark.parametrize("batch", [1, 3, 17])
def test_lm_head_writes_stay_inside_its_buffers(cuda_lib, batch):
    from tenzo_b200 import kernels
    rng = np.random.default_rng(batch)
    V, H = 1004, 256
    w = dev(rng.integers(-127, 128, (V, H), dtype=np.int8))
    s = dev((0.001 + 0.001 * rng.random(V)).astype(np.float32))
    x = dev(rng.standard_normal((batch, H)).astype(np.float32))
    want, _, want_arg = kernels.lm_head_i8(x, w, s)
    g = Guarded()
    logits = g.empty((batch, V), torch.float32)
    got, _, arg = kernels.lm_head_i8(x, w, s, logits=logits)
    g.check()
    assert torch.equal(got, want) and torch.equal(arg, want_arg)
