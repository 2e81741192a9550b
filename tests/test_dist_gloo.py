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
        q_lens, ctx_lens, bt, pages, ids, part_imb = bench.shard_batch(rank)
        assert 1.0 <= part_imb < 1.05
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
        rows_job = bench.reduce_sum(int(q_lens.sum()), world)
        assert rows_job == int(q_lens.sum()) * world
        assert abs(bench.reduce_sum(ms_local, world) / world - (100.0 + 12.5 * (world - 1))) < 1e-9
        value = bench.whole_job_value(int(q_lens.sum()), world, ms)
        assert abs(value - rows_job / (ms * 1e-3)) < 1e-6
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


@pytest.mark.parametrize("workload", ["c4", "verify"])
def test_partition_is_disjoint_complete_and_balanced(workload):
    """the host partitioner deals the whole batch of a workload into 8 shards: every sequence in exactly one shard, the
    same number of sequences of every row class per shard, and the cost (kv_len + rows) within 5 % of the mean"""
    sys.path.insert(0, os.path.join(ROOT, "exllamav3-rs_b200"))
    import bench
    from exl3b200.partition import imbalance, partition_sequences, sequence_cost
    q, ctx = bench.global_batch(workload)
    parts = partition_sequences(q, ctx, 8)
    allidx = np.concatenate(parts)
    assert sorted(allidx.tolist()) == list(range(len(q)))
    for ql in set(q.tolist()):
        counts = {int((q[p] == ql).sum()) for p in parts}
        assert max(counts) - min(counts) <= 1
    assert len({int(q[p].sum()) for p in parts}) == 1, "equal packed rows per shard"
    cost = sequence_cost(q, ctx)
    loads = np.array([cost[p].sum() for p in parts], np.float64)
    assert loads.max() / loads.mean() < 1.05 and loads.min() / loads.mean() > 0.95
    assert imbalance(q, ctx, parts) == pytest.approx(loads.max() / loads.mean())
    # shard_batch(rank) is shard `rank` of that partition
    for rank in (0, 5):
        ql, cl, bt, pages, ids, _ = bench.shard_batch(rank, workload)
        assert ql.tolist() == q[parts[rank]].tolist() and cl.tolist() == ctx[parts[rank]].tolist()
        assert len(ids) == int(ql.sum()) and bt.shape[0] == len(ql)


def test_partition_uneven_counts():
    """a batch whose classes do not divide by the shard count: counts differ by at most one and nothing is lost"""
    sys.path.insert(0, os.path.join(ROOT, "exllamav3-rs_b200"))
    from exl3b200.partition import partition_sequences
    r = np.random.default_rng(3)
    q = np.concatenate([np.ones(13, np.int32), np.full(5, 256, np.int32), np.full(3, 8, np.int32)])
    ctx = r.integers(1, 5000, len(q)).astype(np.int32)
    parts = partition_sequences(q, ctx, 4)
    assert sorted(np.concatenate(parts).tolist()) == list(range(len(q)))
    for ql in (1, 256, 8):
        counts = [int((q[p] == ql).sum()) for p in parts]
        assert max(counts) - min(counts) <= 1
