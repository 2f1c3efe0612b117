"""Run by tests/test_replicas_cpu.py under torch.distributed.run with two ranks: exercises bench.py's replica plumbing
(gloo barrier, max and sum over ranks) without a GPU."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench  # noqa: E402

ranks = bench.Ranks(2)
ranks.barrier()
slowest = ranks.max(10.0 + ranks.rank)       # every rank's time; the slowest decides
total = ranks.sum(100.0 * (ranks.rank + 1))  # every replica's tokens
batch = bench.encoder_batch(1000, 4, 5 + ranks.rank)
if ranks.rank == 0:
    print(json.dumps({"world": ranks.world, "slowest": slowest, "total": total, "first_len": int(len(batch[0]))}), flush=True)
ranks.close()
