"""world_size-2 checks (gloo, CPU) of the benchmark's multi-rank logic: the path shards by batch with no
data-path collective, so the only cross-rank step is taking the slowest rank's time."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    import bench
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ms, e2e = bench.max_over_ranks([2.0 + rank, 5.0 - rank], world, "cpu")
    out[rank] = (ms, e2e, bench.whole_job_rate(world, 4, ms))
    dist.barrier()
    dist.destroy_process_group()


def test_slowest_rank_sets_the_whole_job_rate():
    world = 2
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_worker, args=(world, 29531, out), nprocs=world, join=True)
        assert out[0] == out[1]
        ms, e2e, rate = out[0]
        assert ms == 3.0 and e2e == 5.0            # max over ranks of each time
        assert rate == world * 4 / 3.0e-3          # both replicas' tokens over the slowest rank's step time
