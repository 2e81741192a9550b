"""The N > 1 path of the benchmark on CPU: two gloo ranks shard the sequences (no data-path collective), time their
own shard and agree on the slowest rank's time, from which rank 0 reports the whole-job value."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    import bench
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q_lens, ctx_lens, bt, pages, ids = bench.shard_batch(rank)
        # weak scaling: the same number of rows and sequences on every rank, different sequences
        sig = torch.tensor([int(q_lens.sum()), len(q_lens), int(ctx_lens.sum()), int(ids[:64].sum())], dtype=torch.int64)
        gathered = [torch.zeros_like(sig) for _ in range(world)]
        dist.all_gather(gathered, sig)
        rows = {int(g[0]) for g in gathered}
        seqs = {int(g[1]) for g in gathered}
        assert len(rows) == 1 and len(seqs) == 1
        assert len({(int(g[2]), int(g[3])) for g in gathered}) == world, "ranks must not share sequences"
        # the block table of a rank only names pages of its own pool
        assert bt.max() < pages and bt.min() >= 0
        # every rank reports the slowest rank's time, and the whole-job value follows from it
        ms_local = 100.0 + 25.0 * rank
        ms = bench.reduce_max_ms(ms_local, world)
        assert ms == 100.0 + 25.0 * (world - 1)
        value = bench.whole_job_value(int(q_lens.sum()), world, ms)
        assert abs(value - int(q_lens.sum()) * world / (ms * 1e-3)) < 1e-6
        dist.barrier()
        with open(os.path.join(out_dir, f"rank{rank}.ok"), "w") as f:
            f.write(repr(value))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(240)
def test_two_ranks_shard_and_agree_on_time(tmp_path):
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    vals = [open(tmp_path / f"rank{r}.ok").read() for r in range(world)]
    assert vals[0] == vals[1]


def test_single_rank_needs_no_process_group():
    import bench
    assert bench.reduce_max_ms(12.5, 1) == 12.5
    assert bench.whole_job_value(1052, 1, 100.0) == pytest.approx(10520.0)
