"""The give-up path of the kernels' bounded waits, exercised without a fault or a hang: a self-test kernel lets a wait on a
copy that is never issued run out, which raises the same flag a real give-up raises. The flag must reach the host
(tenzo_cuda_tl1_gemv_take_timeouts), clear on reading, and turn the next engine call that checks it into an error with a
message - after which the engine works again."""
import numpy as np
import pytest
import torch
from helpers import synth

pytestmark = pytest.mark.gpu


def test_flag_reaches_the_host_and_clears(cuda_lib):
    assert cuda_lib.tenzo_cuda_tl1_gemv_take_timeouts() == 0
    assert cuda_lib.tenzo_cuda_selftest_wait_expiry(None) == 0
    torch.cuda.synchronize()
    assert cuda_lib.tenzo_cuda_tl1_gemv_take_timeouts() == 1
    assert cuda_lib.tenzo_cuda_tl1_gemv_take_timeouts() == 0


def test_engine_reports_the_failure_and_recovers(cuda_lib):
    from tenzo_b200.engine import Engine
    m = synth.SyntheticModel(synth.TINY, seed=3)
    prompt = synth.prompt_tokens(3, 5, synth.TINY["vocab_size"])
    with Engine(m.config_struct()).load_synthetic(m) as e:
        for t in prompt[:-1]:
            e.prefill_token(int(t))
        want = e.decode_greedy([int(prompt[-1])], 4)
        e.set_seq_len(0, len(prompt) - 1)
        assert cuda_lib.tenzo_cuda_selftest_wait_expiry(None) == 0
        with pytest.raises(RuntimeError, match="gave up waiting"):
            e.decode_greedy([int(prompt[-1])], 4)
        e.set_seq_len(0, len(prompt) - 1)
        assert np.array_equal(e.decode_greedy([int(prompt[-1])], 4), want)
