"""The allocation-free LM-head entry point (tenzo_cuda_lm_head_i8_static) against the ordinary one.

It exists for callers that must not allocate device memory while serving (all memory already
committed to a KV pool, or a host application that forbids cudaMalloc after start-up): its argmax
scratch is a fixed array inside the library. Called twice in a row, through the C ABI, it must give
exactly the logits and argmax of tenzo_cuda_lm_head_i8 — the shared array keeps the previous call's
contents, so the second call checks that nothing stale leaks through. This file sorts last so a
run that stops at the first failure has already covered every other test."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_lm_head_matches_allocating_entry_point(cuda_lib):
    from tenzo_b200 import kernels
    rng = np.random.default_rng(77)
    V, H = 128256, 2560
    w = torch.from_numpy(rng.integers(-127, 128, (V, H), dtype=np.int8)).cuda()
    s = torch.from_numpy((0.001 + 0.001 * rng.random(V)).astype(np.float32)).cuda()
    nw = torch.from_numpy((1 + 0.1 * rng.standard_normal(H)).astype(np.float32)).cuda()
    assert cuda_lib.tenzo_cuda_lm_head_static_max_batch() == 32
    # 32 fills the built-in array exactly; 17 and 32 are sizes at which the allocating entry point switches to its
    # tensor-core kernel while this one must stay on the warp-per-row kernel; the last call is a smaller batch over
    # the earlier calls' leftovers
    for call, batch in enumerate((3, 32, 17, 1)):
        x = torch.from_numpy(rng.standard_normal((batch, H)).astype(np.float32)).cuda()
        want_logits, _, want_arg = kernels.lm_head_i8(x, w, s, norm_w=nw)
        logits = torch.full((batch, V), float("nan"), dtype=torch.float32, device="cuda")
        arg = torch.full((batch,), -1, dtype=torch.int32, device="cuda")
        before = torch.cuda.memory_allocated()
        kernels.lm_head_i8_static(x, w, s, norm_w=nw, logits=logits, argmax=arg)
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        assert torch.equal(logits, want_logits), f"call {call}: logits differ"
        assert torch.equal(arg, want_arg), f"call {call}: argmax differs"
        assert torch.equal(arg.long(), want_logits.argmax(dim=1)), f"call {call}: argmax is not the maximum"


def test_static_scratch_rejects_oversized_batch(cuda_lib):
    from tenzo_b200 import kernels
    x = torch.zeros(33, 64, device="cuda")
    w = torch.zeros(128, 64, dtype=torch.int8, device="cuda")
    s = torch.ones(128, device="cuda")
    with pytest.raises(RuntimeError, match="rc=-5"):
        kernels.lm_head_i8_static(x, w, s, do_norm=False, logits=torch.empty(33, 128, device="cuda"),
                                  argmax=torch.empty(33, dtype=torch.int32, device="cuda"))
