"""The host half of the sampler (tenzo_ext_sample_pairs, no GPU): feeding it only the logits at or above the k-th
largest gives the same token as feeding it the whole vector, ties at the threshold included."""
import ctypes as C

import numpy as np

from tenzo_b200 import abi, load_library


def sample(L, vals, idxs, params, r):
    v = np.ascontiguousarray(vals, np.float32)
    i = None if idxs is None else np.ascontiguousarray(idxs, np.int32)
    return L.tenzo_ext_sample_pairs(v.ctypes.data_as(abi.c_f32p), None if i is None else i.ctypes.data_as(abi.c_i32p), len(v), C.byref(params), r)


def test_candidates_above_the_threshold_reproduce_the_full_scan():
    L = load_library()
    rng = np.random.default_rng(17)
    for trial in range(300):
        V = int(rng.integers(70, 3000))
        levels = int(rng.integers(3, 200))                       # few distinct values: many ties, also at the threshold
        logits = (rng.integers(-levels, levels, V) * np.float32(0.25)).astype(np.float32)
        k = int(rng.integers(1, 65))
        p = abi.TenzoSampling(float(rng.choice([0.0, 0.3, 0.8, 1.5])), float(rng.choice([0.5, 0.9, 1.0])), k, 1.0)
        kk = 1 if p.temperature <= 0 else k
        thr = np.sort(logits)[::-1][kk - 1]
        idx = np.nonzero(logits >= thr)[0]
        for r in (0.0, 0.37, 0.999, 1.0):
            assert sample(L, logits, None, p, r) == sample(L, logits[idx], idx, p, r), (trial, V, k, r)


def test_first_maximum_and_top_k_membership():
    L = load_library()
    logits = np.array([0.5, 2.0, -1.0, 2.0, 1.5, 2.0], np.float32)
    assert sample(L, logits, None, abi.TenzoSampling(0.0, 0.9, 40, 1.0), 0.5) == 1               # greedy: first maximum
    # k = 2: the streaming heap (TenzoEngine.cpp:1760-1768) ends with (2.0, 1) and (2.0, 3) - index 5 arrives when the
    # heap minimum already equals it and is not strictly greater - and lists the larger pair first
    assert sample(L, logits, None, abi.TenzoSampling(1.0, 1.0, 2, 1.0), 0.0) == 3
    assert sample(L, logits, None, abi.TenzoSampling(1.0, 1.0, 2, 1.0), 1.0) == 1


def test_host_sampler_equals_the_oracle_sampler_on_the_same_draw():
    """tenzo_ext_sample_pairs against the C restatement of the reference's sampler (TenzoEngine.cpp:1757-1806; itself pinned
    to the compiled reference in test_oracle_vs_reference.py) on 300 random logit vectors - ties, every top-k and top-p
    regime - with the uniform draw passed in, including a NaN logit in the greedy branch."""
    from oracle import oracle_py as ora
    L, O = load_library(), ora.load_oracle()
    rng = np.random.default_rng(23)
    for trial in range(300):
        V = int(rng.integers(70, 4000))
        if trial % 3 == 0:
            logits = (rng.integers(-40, 40, V) * np.float32(0.25)).astype(np.float32)        # many ties
        else:
            logits = (rng.standard_normal(V) * 3).astype(np.float32)
        p = abi.TenzoSampling(float(rng.choice([0.0, 0.3, 0.7, 1.5])), float(rng.choice([0.3, 0.9, 1.0])), int(rng.integers(1, 80)), 1.0)
        for r in (0.0, float(rng.random()), 0.999, 1.0):
            want = O.ora_sample(ora.ptr(logits.copy(), ora.c_f32p), V, p.temperature, p.top_p, p.top_k, 1.0, None, 0, r)
            assert sample(L, logits, None, p, r) == want, (trial, V, p.temperature, p.top_p, p.top_k, r)
    greedy = abi.TenzoSampling(0.0, 0.9, 40, 1.0)
    for logits in (np.array([np.nan, 1.0, 2.0], np.float32), np.array([1.0, np.nan, 2.0, 2.0], np.float32), np.full(5, np.nan, np.float32)):
        want = O.ora_sample(ora.ptr(logits.copy(), ora.c_f32p), len(logits), 0.0, 0.9, 40, 1.0, None, 0, 0.5)
        assert sample(L, logits, None, greedy, 0.5) == want
