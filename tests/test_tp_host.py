"""Host-side pieces of the tensor-parallel decoder on CPU: the partition plan, the first-maximum combine and the
column all-gather, the last one across two gloo ranks."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from tenzo_b200 import synth, tp

ROOT = Path(__file__).resolve().parents[1]


def test_plan_covers_every_row_once():
    cfg = synth.SYNTH_8B
    for world in (1, 2, 4, 8):
        plans = [tp.plan(cfg, world, r) for r in range(world)]
        for field, total in (("q_heads", cfg["num_q_heads"]), ("kv_heads", cfg["num_kv_heads"]), ("hidden_rows", cfg["hidden_size"]),
                             ("ffn_rows", cfg["ffn_dim"]), ("vocab_rows", cfg["vocab_size"])):
            spans = [getattr(p, field) for p in plans]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == total
            assert all(spans[i][0] + spans[i][1] == spans[i + 1][0] for i in range(world - 1))
        assert all(p.hidden_rows[1] % 64 == 0 and p.ffn_rows[1] % 64 == 0 for p in plans)
        assert all(p.q_heads[0] == p.kv_heads[0] * (cfg["num_q_heads"] // cfg["num_kv_heads"]) for p in plans)   # q heads sit with their kv head
    with pytest.raises(ValueError):
        tp.plan(synth.BITNET_2B, 2, 0)        # 5 kv heads do not split in two
    with pytest.raises(ValueError):
        tp.plan(cfg, 4, 4)


def test_tl1_row_slices_are_whole_blocks():
    rng = np.random.default_rng(3)
    n, k = 256, 128
    tern = rng.integers(-1, 2, (n, k)).astype(np.int8)
    packed = synth.pack_tl1(tern)
    part = tp._tl1_rows(packed, n, k, 64, 128)
    assert np.array_equal(synth.unpack_tl1(part, 128, k), tern[64:192])


def test_combine_argmax_keeps_first_maximum():
    vals = torch.tensor([[1.0, 5.0, 2.0], [3.0, 5.0, 2.0], [3.0, 4.0, 2.0]])
    idxs = torch.tensor([[10, 11, 12], [110, 111, 112], [210, 211, 212]])
    assert tp.combine_argmax(vals, idxs).tolist() == [110, 11, 12]


def test_all_gather_cols_two_gloo_ranks(tmp_path):
    code = """
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, %r)
from tenzo_b200 import tp
dist.init_process_group("gloo")
r, w = dist.get_rank(), dist.get_world_size()
B, S = 3, 4
loc = (torch.arange(B * S, dtype=torch.float32).view(B, S) + 100 * r)
full, scratch = torch.empty(B, w * S), torch.empty(w * B * S)
tp.all_gather_cols(loc, full, scratch, w)
want = torch.cat([torch.arange(B * S, dtype=torch.float32).view(B, S) + 100 * q for q in range(w)], dim=1)
assert torch.equal(full, want), (full, want)
dist.destroy_process_group()
print("GATHER_OK")
""" % str(ROOT)
    script = tmp_path / "w.py"
    script.write_text(code)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29541", str(script)], capture_output=True, text=True, timeout=300,
                       env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0 and r.stdout.count("GATHER_OK") == 2, (r.stdout[-1500:], r.stderr[-2500:])
