"""The multi-GPU path of the 0.8B model is replicas only: ranks share nothing but the timing
reduction.  Two gloo ranks on the CPU check that reduction (max time, summed tokens)."""

import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank(rank, world, port, out):
    sys.path.insert(0, ROOT)
    import bench
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ms, tokens = bench.aggregate(100.0 + 50.0 * rank, 512 * (rank + 1), world, torch.device("cpu"))
    assert bench.dist_env()[:2] == (rank, world)
    out[rank] = (ms, tokens)
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_report_slowest_time_and_total_tokens():
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_rank, args=(2, 29731, out), nprocs=2, join=True)
    assert out[0] == out[1] == (150.0, 1536.0)


def test_single_rank_is_passthrough():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.aggregate(12.5, 512, 1, torch.device("cpu")) == (12.5, 512)
    assert bench.measured_peak_gbs()[0] > 1000
