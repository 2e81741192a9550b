"""Sequence partitioner for the multi-GPU decode step: the sequences of one continuous batch are dealt to the GPUs of a
box, each GPU holding a weight replica and its own paged pool; no collective runs on the step.

The reference is single-GPU; what this takes its shape from is its admission loop (src/generator.rs:1163-1200), which
fills one batch from the queue by row budget and page budget.  Here the unit is the whole batch and the budget is the
time of the slowest GPU, so the split balances the cost of a step instead of the sequence count: a sequence costs its
rows (the GEMM and row-op work, which every packed row pays 64 layers deep) plus its context (the attention's KV walk).
"""
import numpy as np


def sequence_cost(q_lens, ctx_lens):
    """Cost of a sequence in token units: kv_len + rows, with kv_len = cached tokens + this step's rows."""
    return np.asarray(ctx_lens, np.int64) + 2 * np.asarray(q_lens, np.int64)


def partition_sequences(q_lens, ctx_lens, n_parts):
    """Deal the sequences to `n_parts` shards.  Returns a list of index arrays (each sorted ascending), disjoint, covering
    every sequence.

    Sequences of one row class (same q_len: decode rows, verify batches, prefill chunks) are dealt separately, longest
    context first, each to the shard with the least accumulated cost that still has the fewest members of that class.
    Every shard therefore gets the same number (+-1) of prefill chunks and of decode rows, so packed row counts agree to
    within one sequence of each class; within a class the contexts are balanced by the longest-processing-time rule and
    then by pairwise swaps that lower the most expensive shard.
    """
    q_lens = np.asarray(q_lens, np.int64)
    ctx_lens = np.asarray(ctx_lens, np.int64)
    cost = sequence_cost(q_lens, ctx_lens)
    load = np.zeros(n_parts, np.int64)
    parts = [[] for _ in range(n_parts)]
    for ql in sorted(set(q_lens.tolist()), reverse=True):
        members = np.nonzero(q_lens == ql)[0]
        members = members[np.argsort(-cost[members], kind="stable")]
        count = np.zeros(n_parts, np.int64)
        for i in members:
            fewest = np.nonzero(count == count.min())[0]
            p = int(fewest[np.argmin(load[fewest])])
            parts[p].append(int(i)); load[p] += cost[i]; count[p] += 1
    # refinement: while it lowers the largest shard, swap a sequence of the most expensive shard with a cheaper one of the
    # same row class from another shard (class counts and packed rows per shard stay as dealt)
    for _ in range(10 * len(q_lens)):
        hi = int(np.argmax(load))
        best = None
        for i in parts[hi]:
            for p in range(n_parts):
                if p == hi:
                    continue
                for j in parts[p]:
                    d = cost[i] - cost[j]
                    if q_lens[i] != q_lens[j] or d <= 0:
                        continue
                    new_max = max(load[hi] - d, load[p] + d)
                    if new_max < load[hi] and (best is None or new_max < best[0]):
                        best = (new_max, i, p, j)
        if best is None:
            break
        _, i, p, j = best
        d = cost[i] - cost[j]
        parts[hi].remove(i); parts[hi].append(j); parts[p].remove(j); parts[p].append(i)
        load[hi] -= d; load[p] += d
    return [np.array(sorted(p), np.int64) for p in parts]


def imbalance(q_lens, ctx_lens, parts):
    """Largest shard cost over the mean shard cost (1.0 = perfectly balanced)."""
    cost = sequence_cost(q_lens, ctx_lens)
    loads = np.array([cost[p].sum() for p in parts], np.float64)
    return float(loads.max() / loads.mean())
