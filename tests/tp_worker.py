"""Worker for tests/test_gpu_tp.py: one process per GPU (launched by torch.distributed.run, or alone for world 1).
Runs tenzo_b200.tp.parity_check (the tensor-parallel decoder next to the single-GPU engine on the same seeded model) and
prints TP_OK when the token streams and the logits of the last step are identical on every rank."""
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def main():
    import torch
    import torch.distributed as dist
    from tenzo_b200 import tp
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ok = tp.parity_check(use_graph=bool(int(os.environ.get("TP_GRAPH", "1"))),
                         say=lambda m: print(f"[rank {rank}] {m}", file=sys.stderr, flush=True))
    if world > 1:
        dist.destroy_process_group()
    if rank == 0:
        print("TP_OK" if ok else "TP_FAIL", flush=True)
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
