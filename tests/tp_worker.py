"""Worker for tests/test_gpu_tp.py: one process per GPU (launched by torch.distributed.run, or alone for world 1).
Runs the tensor-parallel decoder next to the single-GPU engine on the same seeded model and prints TP_OK when the
token streams and the logits of the last step are identical."""
import os
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def main():
    import torch
    import torch.distributed as dist
    from tenzo_b200 import synth, tp
    from tenzo_b200.engine import Engine
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    use_graph = int(os.environ.get("TP_GRAPH", "1"))
    cfg = dict(synth.SYNTH_8B, num_layers=2, vocab_size=16384, max_seq_len=64)
    B, prompt_len, steps = 32, 3, 6
    model = synth.SyntheticModel(cfg, seed=5)
    prompts = np.stack([synth.prompt_tokens(100 + b, prompt_len, cfg["vocab_size"]) for b in range(B)])     # [B, prompt_len]

    say = lambda m: print(f"[rank {rank}] {m}", file=sys.stderr, flush=True)
    say("model built")
    eng = Engine(model.config_struct(), batch=B).load_synthetic(model)
    for t in range(prompt_len - 1):
        eng.prefill_tokens(prompts[:, t])
    want = eng.decode_greedy(prompts[:, -1], steps - 1)                   # [steps - 1, B]
    last = eng.generate_steps(want[-1])                                   # the last step also leaves its logits behind
    want = np.concatenate([want, np.asarray(last)[None]])
    want_logits = np.stack([eng.read_buffer(15, seq=b, count=cfg["vocab_size"]) for b in (0, B - 1)])
    eng.close()

    say("single-GPU reference done")
    dec = tp.TensorParallelDecoder(model, B, cfg["max_seq_len"], use_graph=bool(use_graph))
    say("shards loaded")
    for t in range(prompt_len - 1):
        dec.step(prompts[:, t])
        torch.cuda.synchronize()
        say(f"prompt step {t} done")
    got = []
    nxt = dec.step(prompts[:, -1])
    got.append(nxt.cpu().numpy().copy())
    for _ in range(steps - 1):
        nxt = dec.step()
        got.append(nxt.cpu().numpy().copy())
    got = np.stack(got)
    say("decode done")
    v0, vn = dec.p.vocab_rows
    mine = dec.logits_slice().cpu().numpy()
    ok = np.array_equal(got, want) and np.array_equal(mine[0], want_logits[0, v0:v0 + vn]) and np.array_equal(mine[B - 1], want_logits[1, v0:v0 + vn])
    if not ok:
        print(f"rank {rank}: MISMATCH tokens equal={np.array_equal(got, want)} first diff step={np.argwhere(got != want)[:1].tolist()}", flush=True)
    if world > 1:
        flag = torch.tensor([1 if ok else 0], device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        ok = bool(flag.item())
        dist.destroy_process_group()
    if rank == 0:
        print("TP_OK" if ok else "TP_FAIL", flush=True)
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
