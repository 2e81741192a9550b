#!/usr/bin/env python
"""Benchmark of the ragged continuous-batching decode step (27B-class dense model, EXL3 4 bpw, paged KV).

    python bench.py --gpus N --steps K --warmup W              # this library, one rank per GPU (torchrun for N > 1)
    python bench.py --impl reference --steps K --warmup W      # CPU restatement of the same ops on the host cores
    python bench.py --workload verify ...                      # the speculative-verify step (32 sequences x 8 draft rows, 4-bit KV)
    python bench.py --op gemm|gemm_sweep|attn ...              # op-level measurements

Workload "c4" (default): one seeded batch of 256 sequences - 224 decoding one token, 32 prefill chunks of 256 tokens,
contexts uniform in [512, 16384] - is dealt into 8 shards by the host partitioner (exl3b200/partition.py: the same number
of prefill chunks and decode rows per shard, contexts balanced within each class); rank r of N runs shard r.  Every GPU
holds a weight replica (64 layers, hidden 5120, 40 q / 8 kv heads, head_dim 128, MLP 17408, vocab 151936, seeded random
EXL3 codes) and its own paged pool; no collective runs on the step.  N = 8 is the whole 256-sequence batch (8416 packed
rows); on fewer GPUs the fp16 KV of 256 sequences (about 567 GB) does not fit, so N ranks run N of the 8 shards (weak
scaling).  Workload "verify": 32 sequences that each verify 8 draft tokens, contexts log-uniform in [1024, 32768], 4-bit
quantised KV, dealt into 8 shards of 4 sequences (32 packed rows per GPU) the same way.
Prints ONE JSON line on rank 0.
"""
import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "exllamav3-rs_b200"))

CFG = dict(n_layers=64, hidden=5120, nq=40, nkv=8, hd=128, inter=17408, vocab=151936, K=4, cb=1)
N_SHARDS = 8
WORKLOADS = {
    # name: (sequences, [(count, q_len)], context sampler, kv_bits, description)
    "c4": dict(classes=[(224, 1), (32, 256)], ctx=("uniform", 512, 16384), kv_bits=0,
               name=("27B-class dense decode step, 4 bpw EXL3, fp16 paged KV: 256 sequences (224 decode rows + 32 prefill chunks "
                     "of 256) dealt to 8 GPUs = per GPU 28 decode rows + 4 chunks (1052 packed rows, 32 sequences), contexts U[512,16384]")),
    "verify": dict(classes=[(32, 8)], ctx=("loguniform", 1024, 32768), kv_bits=4,
                   name=("speculative-verify step on the 27B-class 4 bpw model: 32 sequences x 8 draft rows dealt to 8 GPUs = per "
                         "GPU 4 sequences (32 packed rows), contexts log-U[1024,32768], 4-bit quantised paged KV")),
}


def global_batch(workload, seed=1234):
    """The whole batch of a workload: (q_lens, ctx_lens) of all sequences, seeded."""
    w = WORKLOADS[workload]
    r = np.random.default_rng(seed)
    q_lens = np.concatenate([np.full(c, q, np.int32) for c, q in w["classes"]])
    kind, lo, hi = w["ctx"]
    if kind == "uniform":
        ctx = r.integers(lo, hi + 1, len(q_lens)).astype(np.int32)
    else:
        ctx = np.exp(r.uniform(np.log(lo), np.log(hi), len(q_lens))).astype(np.int32)
    return q_lens, ctx


def shard_batch(rank, workload="c4", seed=1234):
    """Sequences of shard `rank` of the 8-way partition: (q_lens, ctx_lens, block_table, pages, ids, imbalance of the
    partition).  Pages are assigned by a seeded permutation of the shard's own pool."""
    from exl3b200.partition import imbalance, partition_sequences
    gq, gctx = global_batch(workload, seed)
    parts = partition_sequences(gq, gctx, N_SHARDS)
    idx = parts[rank % N_SHARDS]
    q_lens, ctx = gq[idx], gctx[idx]
    r = np.random.default_rng(seed + 1 + rank)
    need = (ctx + q_lens + 255) // 256
    pps = int(need.max())
    pages = int(need.sum()) + 1
    perm = r.permutation(pages).astype(np.int32)
    bt = np.zeros((len(idx), pps), np.int32)
    o = 0
    for b in range(len(idx)):
        bt[b, :need[b]] = perm[o:o + need[b]]
        o += need[b]
    ids = r.integers(0, CFG["vocab"], int(q_lens.sum())).astype(np.int64)
    return q_lens, ctx, bt, pages, ids, imbalance(gq, gctx, parts)


def reduce_max_ms(ms_local, world, device="cpu"):
    """Device time of a multi-rank run: the slowest rank's.  One all_reduce(MAX) over the job's process group (NCCL on
    GPUs, gloo in the CPU tests); the data path itself has no collective: sequences never leave their rank."""
    if world <= 1:
        return float(ms_local)
    import torch
    import torch.distributed as dist
    t = torch.tensor([float(ms_local)], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def reduce_sum(x, world, device="cpu"):
    """Sum of a per-rank scalar over the job (1 rank: the value itself)."""
    if world <= 1:
        return float(x)
    import torch
    import torch.distributed as dist
    t = torch.tensor([float(x)], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def whole_job_value(rows_per_rank, world, ms_per_step):
    """Tokens/s of the whole job under weak scaling: every rank processes `rows_per_rank` rows per step."""
    return rows_per_rank * world / (ms_per_step * 1e-3)


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz, self._halt = index, [], set(), None, threading.Event()

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                     nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                     nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                     nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap"}
            while not self._halt.is_set():
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
                time.sleep(0.05)
        except Exception as e:  # NVML missing: report that rather than invent numbers
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


CPU_SAMPLE = {
    "c4": ("ONE layer of the 64 (full widths, 4 bpw) over a 1/16-scale cut of a GPU's shard: 2 decode sequences + one prefill "
           "chunk of 64 rows (66 packed rows, 3 sequences), contexts in [512, 2048], composed from oracle/ ops; tokens/s = "
           "66 rows / (64 layers x the measured time of one layer): an extrapolated sample, not the 1052-row step"),
    "verify": ("ONE layer of the 64 (full widths, 4 bpw) over one verify sequence of 8 draft rows with a 4-bit quantised KV "
               "context of 2048 tokens, composed from oracle/ ops; tokens/s = 8 rows / (64 layers x the measured time of one "
               "layer): an extrapolated sample"),
}


def host_threads(world=1):
    """Threads the CPU legs may use: the cores this process may run on (torchrun pins OMP_NUM_THREADS to 1, which is
    not a property of the machine)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return max(1, n // max(world, 1))


class CpuSample:
    """Bounded CPU sample of a workload's step: ONE layer of the model (full widths) over a small cut of a shard, composed
    from the oracle's ops.  Each call of layer() runs that layer once and returns its wall time."""

    def __init__(self, workload, threads):
        from oracle import oracle as O
        from oracle import oracle_model
        O.set_num_threads(threads)
        self.threads = O.num_threads()
        self._step = oracle_model.step
        r = np.random.default_rng(7)
        c = CFG
        kv_bits = WORKLOADS[workload]["kv_bits"]
        if workload == "c4":
            q_lens = np.array([1, 1, 64], np.int32)
            ctx = r.integers(512, 2049, len(q_lens)).astype(np.int32)
        else:
            q_lens = np.array([8], np.int32)
            ctx = np.array([2048], np.int32)
        nseq, self.rows = len(q_lens), int(q_lens.sum())

        def lin(k, n):
            return dict(trellis=r.integers(-32768, 32768, size=(k // 16, n // 16, 16 * c["K"]), dtype=np.int16),
                        suh=(r.integers(0, 2, k) * 2 - 1).astype(np.float16),
                        svh=((r.integers(0, 2, n) * 2 - 1) / np.sqrt(k)).astype(np.float16), K=c["K"], cb=c["cb"])

        need = (ctx + q_lens + 255) // 256
        pages = int(need.sum()) + 1
        bt = np.zeros((nseq, int(need.max())), np.int32)
        o = 0
        for b in range(nseq):
            bt[b, :need[b]] = np.arange(o, o + need[b]); o += need[b]
        hid, nq, nkv, hd = c["hidden"], c["nq"], c["nkv"], c["hd"]
        layer = dict(q_proj=lin(hid, nq * hd), k_proj=lin(hid, nkv * hd), v_proj=lin(hid, nkv * hd), o_proj=lin(nq * hd, hid),
                     gate_proj=lin(hid, c["inter"]), up_proj=lin(hid, c["inter"]), down_proj=lin(c["inter"], hid),
                     attn_norm=np.ones(hid, np.float16), mlp_norm=np.ones(hid, np.float16),
                     q_norm=np.ones(hd, np.float16), k_norm=np.ones(hd, np.float16))
        if kv_bits == 0:
            layer["k_cache"] = (0.5 * r.standard_normal((pages, 256, nkv, hd))).astype(np.float16)
            layer["v_cache"] = (0.5 * r.standard_normal((pages, 256, nkv, hd))).astype(np.float16)
        else:
            groups = nkv * hd // 32
            for nm in ("qk", "qv"):
                layer[nm] = r.integers(-2 ** 31, 2 ** 31 - 1, size=(pages, 256, groups * kv_bits), dtype=np.int64).astype(np.int32)
            for nm in ("sk", "sv"):
                layer[nm] = (r.random((pages, 256, groups)) * 0.05 + 0.01).astype(np.float16)
        small_vocab = 1024     # the head is excluded from the sample (one layer only); a tiny head keeps the call valid
        self.m = dict(cfg=dict(c, vocab=small_vocab, kv_bits=kv_bits), embed=r.standard_normal((small_vocab, hid)).astype(np.float16),
                      final_norm=np.ones(hid, np.float16), inv_freq=(1.0 / (1e6 ** (np.arange(0, hd, 2) / hd))).astype(np.float32),
                      lm_head=dict(lin(hid, small_vocab)), layers=[layer])
        self.ids = r.integers(0, small_vocab, self.rows).astype(np.int64)
        self.q_lens, self.ctx, self.bt = q_lens, ctx, bt

    def layer(self):
        t0 = time.perf_counter()
        self._step(self.m, self.ids, self.q_lens, self.ctx, self.bt)
        return time.perf_counter() - t0


def cpu_sample(workload, steps, warmup, threads, budget_s=60.0):
    """Runs up to `warmup` + `steps` one-layer samples inside `budget_s` seconds of wall time (at least one timed sample).
    Returns (tokens_per_s of the 64-layer model, seconds per layer, threads, timed samples, warm-up samples)."""
    cs = CpuSample(workload, threads)
    t_begin = time.perf_counter()
    done_w = 0
    for _ in range(warmup):
        if done_w >= 1 and time.perf_counter() - t_begin > budget_s / 4:
            break
        cs.layer(); done_w += 1
    times = []
    for _ in range(max(steps, 1)):
        if times and time.perf_counter() - t_begin > budget_s:
            break
        times.append(cs.layer())
    t_layer = float(np.mean(times))
    return cs.rows / (CFG["n_layers"] * t_layer), t_layer, cs.threads, len(times), done_w


def run_reference(args):
    """The reference arm: the reference's CUDA ops have no CPU path of their own for this step, so the arm times the CPU
    restatement of them (oracle/) on all host cores.  A timed step is ONE layer over the cut described in
    cpu_baseline.sample; `steps` and `ms_per_step` are what was actually run, `value` extrapolates that layer to the 64
    of the model."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tps, t_layer, threads, n_timed, n_warm = cpu_sample(args.workload, args.steps, min(args.warmup, 1), host_threads(1))
    line = {"impl": "reference", "metric": "ragged decode-step tokens/s", "value": tps, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": n_timed, "warmup": n_warm, "ms_per_step": 1e3 * t_layer,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
            "config": {"workload": WORKLOADS[args.workload]["name"], "same_config": False,
                       "timed_step": "one layer of 64 over the sample named in cpu_baseline.sample; value = sample rows / (64 x ms_per_step)"},
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": CPU_SAMPLE[args.workload]},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops_sustained", 1400.0), "measured"
    return 6650.0, 1400.0, "fallback"


def time_gemm_op(ctx, torch, lins, x, y, reps=1):
    """Average device time of exl3_gemm over the given tensors in turn (each call reads weights no earlier call of the
    last len(lins) - 1 touched: L2-cold when their total size exceeds L2).  The calls are captured once into a CUDA graph
    on the context's side stream and the graph is replayed between two events on that stream, so that host launch cost
    (two launches and a tensor-map encode per call, more than a 26 us kernel leaves room for) stays out of the kernel's
    time.  Returns (seconds per call, launches per call)."""
    import exl3b200
    side = torch.cuda.ExternalStream(exl3b200.lib().exl3_side_stream(ctx.handle))
    torch.cuda.synchronize()
    for l in lins[:3]:
        ctx.exl3_gemm(x, l.trellis, y, l.suh, None, l.svh, mcg=True, stream=side)
    exl3b200.lib().exl3_sync_side_stream(ctx.handle)
    g0 = ctx.launch_count()
    gr = exl3b200.CudaGraph(ctx)
    gr.capture_begin()
    for l in lins:
        ctx.exl3_gemm(x, l.trellis, y, l.suh, None, l.svh, mcg=True, stream=side)
    gr.capture_end()
    launches = (ctx.launch_count() - g0) // len(lins)
    gr.replay()
    exl3b200.lib().exl3_sync_side_stream(ctx.handle)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(side)
    for _ in range(reps):
        gr.replay()
    e1.record(side)
    exl3b200.lib().exl3_sync_side_stream(ctx.handle)
    ctx.poll_status()
    return e0.elapsed_time(e1) * 1e-3 / (reps * len(lins)), launches


def gemm_alg_bytes(m, k, n, K):
    """Algorithmic bytes of one exl3_gemm: codes + sign vectors + activations in + fp16 out."""
    return k * n * K / 8 + 2 * (k + n) + 2 * m * k + 2 * m * n


# DRAM bytes of one gemm_tc_kernel launch at M = 1052 on 5120 x 17408, 4 bpw (dram__bytes_read.sum + dram__bytes_write.sum of
# one ncu capture); the figure belongs to the commit named with it and is not re-measured by the run
NCU_TRAFFIC_TC_M1052 = {"bytes": 63079680 + 12018944, "source": "ncu capture of gemm_tc_kernel<4,1,2,256> at M=1052 (summary under profiles/)"}


def run_ours(args):
    import torch
    import torch.distributed as dist
    import exl3b200
    from exl3b200.step import SyntheticModel

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = f"cuda:{local}"
    wl = WORKLOADS[args.workload]
    ctx = exl3b200.Ctx(local, workspace_bytes=1 << 30)
    q_lens, ctx_lens, bt, pages, ids, part_imbalance = shard_batch(rank, args.workload)
    rows, bsz = int(q_lens.sum()), len(q_lens)
    model = SyntheticModel(pages=pages, kv_bits=wl["kv_bits"], seed=100 + rank, device=dev, **CFG)
    model.fill_kv(seed=200 + rank)
    torch.cuda.synchronize()

    # host-side (pinned) step inputs for the end-to-end leg, device-resident copies for the kernel-only leg
    h_ids = torch.from_numpy(ids).pin_memory(); h_q = torch.from_numpy(q_lens).pin_memory()
    h_sl = torch.from_numpy(ctx_lens).pin_memory(); h_bt = torch.from_numpy(bt).pin_memory()
    d_ids, d_q, d_sl, d_bt = h_ids.to(dev), h_q.to(dev), h_sl.to(dev), h_bt.to(dev)
    max_q = int(q_lens.max())
    stream = torch.cuda.current_stream()

    # The step is captured once into a CUDA graph on the context's side stream (the reference's CudaGraph,
    # src/ffi.rs:403-451, does the same for its decode loop) and replayed: the device buffers the step reads are
    # fixed, their contents change per step.  --no-graph launches the kernels of a step one by one instead.
    for _ in range(2):
        model.step(ctx, d_ids, d_q, d_sl, d_bt, max_q)
    torch.cuda.synchronize()
    graph, tok_static, launches_captured = None, torch.empty(bsz, dtype=torch.int64, device=dev), None
    if not args.no_graph:
        graph = exl3b200.CudaGraph(ctx)
        stream = torch.cuda.ExternalStream(graph.side_stream(), device=dev)
        l0 = ctx.launch_count()
        graph.capture_begin()
        model.step(ctx, d_ids, d_q, d_sl, d_bt, max_q, stream=graph.side_stream(), tokens_out=tok_static)
        graph.capture_end()
        launches_captured = ctx.launch_count() - l0

    def step_resident():
        if graph is not None:
            graph.replay()
            return tok_static
        return model.step(ctx, d_ids, d_q, d_sl, d_bt, max_q, tokens_out=tok_static)[0]

    def step_e2e():
        with torch.cuda.stream(stream):
            d_ids.copy_(h_ids, non_blocking=True); d_q.copy_(h_q, non_blocking=True)
            d_sl.copy_(h_sl, non_blocking=True); d_bt.copy_(h_bt, non_blocking=True)
            tok = step_resident()
            return tok.cpu()                   # device -> host read of the sampled tokens (synchronises)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        """(slowest rank's device time, mean over ranks) of `steps` calls, in ms"""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        return reduce_max_ms(ms, world, dev), reduce_sum(ms, world, dev) / world

    for _ in range(max(args.warmup, 3)):
        step_resident()
    ctx.poll_status()
    sampler = ClockSampler(local)
    sampler.start()
    l0 = ctx.launch_count()
    # a profiler started with `--profile-from-start off` sees exactly the timed steps (no effect otherwise)
    torch.cuda.cudart().cudaProfilerStart()
    ms_total, ms_mean = timed(step_resident, args.steps)
    torch.cuda.cudart().cudaProfilerStop()
    launches = launches_captured if graph is not None else (ctx.launch_count() - l0) // max(args.steps, 1)
    clocks = sampler.stop()
    step_e2e()
    ms_e2e, _ = timed(step_e2e, args.steps)
    ctx.poll_status()
    # per-stage device times of the same step, launched kernel by kernel with events at the stage boundaries (outside the
    # timed regions; the graph replay above has no stage boundaries to time)
    stages = None
    if rank == 0:
        ctx.stage_profile(True)
        for _ in range(2):
            model.step(ctx, d_ids, d_q, d_sl, d_bt, max_q, tokens_out=tok_static)
        torch.cuda.synchronize()
        stages, _ = ctx.stage_times(reset=True)
        ctx.stage_profile(False)
        stages = {k: round(v, 3) for k, v in stages.items()}

    ms_step = ms_total / args.steps
    rows_job = reduce_sum(rows, world, dev)             # every shard has the same row count; summed for the record
    seqs_job = reduce_sum(bsz, world, dev)
    value = rows_job / (ms_step * 1e-3)
    e2e_value = rows_job / (ms_e2e / args.steps * 1e-3)
    h2d = int(ids.nbytes + q_lens.nbytes + ctx_lens.nbytes + bt.nbytes)

    hbm_peak, tf_peak, which = peaks()
    roof, roof_decode = None, None
    if rank == 0:
        # ---- roofline of the dominant kernel: the EXL3 GEMM at the step's row count, timed on L2-cold weights (the 64
        # layers' gate_proj tensors in turn; 44.6 MB each, 2.9 GB in total)
        k, n, K = CFG["hidden"], CFG["inter"], CFG["K"]
        lins = [L["gate_proj"] for L in model.layers]
        x = (torch.randn(max(rows, 16), k, device=dev) * 0.1).to(torch.float16)
        y = torch.empty(max(rows, 16), n, dtype=torch.float16, device=dev)
        t_op, launches_op = time_gemm_op(ctx, torch, lins, x[:rows], y[:rows])
        kv_bytes_tok = CFG["nkv"] * CFG["hd"] * 2 * (2 if wl["kv_bits"] == 0 else wl["kv_bits"] / 8 + 2 / 32)
        step_bytes = model.weight_bytes() + float((ctx_lens + q_lens).sum()) * kv_bytes_tok * CFG["n_layers"]
        step_hbm = step_bytes / (ms_step * 1e-3) / 1e9
        if rows > 64:
            flops = 2.0 * rows * k * n
            ach = flops / t_op / 1e12
            roof = {"bound": "tensor", "kernel": "exl3_gemm (gate_proj 5120x17408, M=%d)" % rows, "achieved": ach,
                    "peak": tf_peak, "unit": "TFLOP/s", "frac": ach / tf_peak,
                    "traffic": NCU_TRAFFIC_TC_M1052["bytes"], "traffic_source": NCU_TRAFFIC_TC_M1052["source"],
                    "algorithmic_bytes": gemm_alg_bytes(rows, k, n, K), "peak_source": which, "launches_per_op": launches_op,
                    "op_ms": t_op * 1e3, "step_hbm_gbs": step_hbm, "step_hbm_frac": step_hbm / hbm_peak}
        else:
            byts = gemm_alg_bytes(rows, k, n, K)
            ach = byts / t_op / 1e9
            roof = {"bound": "hbm", "kernel": "exl3_gemm (gate_proj 5120x17408, M=%d)" % rows, "achieved": ach, "peak": hbm_peak,
                    "unit": "GB/s", "frac": ach / hbm_peak, "traffic": None, "algorithmic_bytes": byts, "peak_source": which,
                    "launches_per_op": launches_op, "op_ms": t_op * 1e3, "step_hbm_gbs": step_hbm,
                    "step_hbm_frac": step_hbm / hbm_peak}
        # ---- the decode regime of the same op (the metric's "EXL3 GEMM HBM GB/s vs peak"): M = 16 and M = 1
        pts = {}
        for m in (16, 1):
            t_m, _ = time_gemm_op(ctx, torch, lins, x[:m], y[:m], reps=2)
            pts[m] = (t_m, gemm_alg_bytes(m, k, n, K))
        roof_decode = {"bound": "hbm", "kernel": "exl3_gemm (gate_proj 5120x17408, 4 bpw, M=16)", "achieved": pts[16][1] / pts[16][0] / 1e9,
                       "peak": hbm_peak, "unit": "GB/s", "frac": pts[16][1] / pts[16][0] / 1e9 / hbm_peak, "traffic": None,
                       "algorithmic_bytes": pts[16][1], "op_us": pts[16][0] * 1e6, "peak_source": which,
                       "m1": {"op_us": pts[1][0] * 1e6, "achieved": pts[1][1] / pts[1][0] / 1e9, "frac": pts[1][1] / pts[1][0] / 1e9 / hbm_peak}}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        tps, t_layer, threads, n_timed, _ = cpu_sample(args.workload, 3, 1, host_threads(1), budget_s=25.0)
        cpu = {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": CPU_SAMPLE[args.workload] + " (%d timed layers, %.2f s per layer)" % (n_timed, t_layer)}
    if rank == 0:
        line = {"metric": "ragged decode-step tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
                "config": {"workload": wl["name"], "rows_per_gpu": rows, "sequences_per_gpu": bsz, "shards_run": world,
                           "shards_total": N_SHARDS, "partition_cost_imbalance": part_imbalance,
                           "rank_time_imbalance": ms_total / ms_mean if ms_mean > 0 else None,
                           "generated_tokens_per_s": seqs_job / (ms_step * 1e-3),
                           "l2": "inputs larger than L2 (11 GB of weights and the KV pool are streamed every step)"},
                "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                        "d2h_bytes_per_step": bsz * 8},
                "gpu_launches": int(launches), "launch_mode": "cuda graph replay" if graph is not None else "stream launches",
                "stage_ms": stages, "clocks": clocks, "roofline": roof, "roofline_decode": roof_decode, "cpu_baseline": cpu}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_ops(args):
    """Op-level measurements (not the headline line): --op gemm (one shape), gemm_sweep (K=5120, N=17408 sweep of
    bits x M), attn (paged attention alone: 64 sequences, contexts log-uniform in [128, 32768], 40 q / 8 kv heads).
    Every timed launch reads weights / KV that were not touched by the previous launch (a ring of tensors larger
    than L2).  One JSON line per measurement."""
    import torch
    import exl3b200
    torch.cuda.set_device(0)
    ctx = exl3b200.Ctx(0, workspace_bytes=1 << 30)
    hbm_peak, tf_peak, which = peaks()
    stream = torch.cuda.current_stream()
    g = torch.Generator(device="cuda"); g.manual_seed(5)

    side = torch.cuda.ExternalStream(exl3b200.lib().exl3_side_stream(ctx.handle))

    def time_calls(fns, reps):
        """Average device time per call.  The calls are captured once into a CUDA graph on the context's side stream and
        the graph is replayed between two events, so host-side launch cost does not enter the number."""
        torch.cuda.synchronize()
        for f in fns[:2]:
            f(side)
        exl3b200.lib().exl3_sync_side_stream(ctx.handle)
        gr = exl3b200.CudaGraph(ctx)
        gr.capture_begin()
        for f in fns:
            f(side)
        gr.capture_end()
        gr.replay()
        exl3b200.lib().exl3_sync_side_stream(ctx.handle)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(side)
        for _ in range(reps):
            gr.replay()
        e1.record(side)
        exl3b200.lib().exl3_sync_side_stream(ctx.handle)
        return e0.elapsed_time(e1) * 1e-3 / (reps * len(fns))

    def gemm_point(m, k, n, K, reps, cb=1):
        ring = max(2, min(8, int(300e6 // (k * n * K / 8)) + 1))        # > 126 MB of L2 between reuses
        ws = [torch.randint(-32768, 32768, (k // 16, n // 16, 16 * K), dtype=torch.int16, device="cuda", generator=g)
              for _ in range(ring)]
        suh = (torch.randint(0, 2, (k,), device="cuda", generator=g) * 2 - 1).to(torch.float16)
        svh = (torch.randint(0, 2, (n,), device="cuda", generator=g) * 2 - 1).to(torch.float16)
        a = torch.randn(m, k, device="cuda", generator=g).to(torch.float16)
        c = torch.empty(m, n, dtype=torch.float16, device="cuda")
        fns = [(lambda st, w=w: ctx.exl3_gemm(a, w, c, suh, None, svh, mcg=cb == 1, mul1=cb == 2, stream=st)) for w in ws]
        t = time_calls(fns, reps)
        byts = k * n * K / 8 + 2 * (k + n) + 2 * m * k + 2 * m * n
        fl = 2.0 * m * k * n
        return {"op": "exl3_gemm", "m": m, "k": k, "n": n, "bits": K, "us": t * 1e6, "GBps": byts / t / 1e9,
                "hbm_frac": byts / t / 1e9 / hbm_peak, "TFLOPs": fl / t / 1e12, "tensor_frac": fl / t / 1e12 / tf_peak,
                "peaks": which}

    if args.op == "gemm":
        print(json.dumps(gemm_point(args.m, args.k, args.n, args.bits, args.reps)))
    elif args.op == "gemm_sweep":
        for K in (2, 3, 4, 5, 8):
            for m in (1, 4, 16, 64, 256, 2048):
                print(json.dumps(gemm_point(m, 5120, 17408, K, args.reps)))
    elif args.op == "attn":
        r = np.random.default_rng(3)
        bsz, nq, nkv, hd, q_len = args.seqs, 40, 8, 128, args.m
        ctx_lens = np.exp(r.uniform(np.log(128), np.log(32768), bsz)).astype(np.int32)
        need = (ctx_lens + q_len + 255) // 256
        pages = int(need.sum()) + 1
        perm = r.permutation(pages).astype(np.int32)
        bt = np.zeros((bsz, int(need.max())), np.int32)
        o = 0
        for b in range(bsz):
            bt[b, :need[b]] = perm[o:o + need[b]]; o += need[b]
        kc = (torch.randn(pages, 256, nkv, hd, device="cuda", generator=g) * 0.5).to(torch.float16)
        vc = (torch.randn(pages, 256, nkv, hd, device="cuda", generator=g) * 0.5).to(torch.float16)
        q = torch.randn(bsz, q_len, nq, hd, device="cuda", generator=g).to(torch.float16)
        kn = (torch.randn(bsz, q_len, nkv, hd, device="cuda", generator=g) * 0.5).to(torch.float16)
        out = torch.empty_like(q)
        dbt, dsl = torch.from_numpy(bt).cuda(), torch.from_numpy(ctx_lens).cuda()
        if args.kv_bits:
            # quantised pools with random codes and small positive scales (timing only: every bit pattern is a valid code)
            del kc, vc
            groups, bits = nkv * hd // 32, args.kv_bits
            qk = torch.randint(-2 ** 31, 2 ** 31 - 1, (pages, 256, groups * bits), dtype=torch.int32, device="cuda", generator=g)
            qv = torch.randint(-2 ** 31, 2 ** 31 - 1, (pages, 256, groups * bits), dtype=torch.int32, device="cuda", generator=g)
            sk = (torch.rand(pages, 256, groups, device="cuda", generator=g) * 0.05 + 0.01).to(torch.float16)
            sv = (torch.rand(pages, 256, groups, device="cuda", generator=g) * 0.05 + 0.01).to(torch.float16)
            t = time_calls([lambda st: ctx.bighead_attn_paged_q(q, kn, kn, qk, sk, qv, sv, dbt, dsl, out, nkv, stream=st)], args.reps)
            byts = float((ctx_lens + q_len).sum()) * nkv * hd * 2 * (bits / 8 + 2 / 32)
            kc = qk
        else:
            t = time_calls([lambda st: ctx.bighead_attn_paged(q, kn, kn, kc, vc, dbt, dsl, out, stream=st)], args.reps)
            byts = float((ctx_lens + q_len).sum()) * nkv * hd * 2 * 2
        flops = float((4.0 * q_len * nq * hd * (ctx_lens + (q_len + 1) / 2)).sum())       # QK^T and PV under the causal mask
        print(json.dumps({"op": "bighead_attn_paged_q" if args.kv_bits else "bighead_attn_paged", "kv_bits": args.kv_bits or 16, "seqs": bsz, "q_len": q_len, "mean_ctx": float(ctx_lens.mean()),
                          "kv_bytes": byts, "us": t * 1e6, "GBps": byts / t / 1e9, "hbm_frac": byts / t / 1e9 / hbm_peak,
                          "TFLOPs": flops / t / 1e12,
                          "note": "KV pool %.1f GB" % (kc.numel() * 4 / 1e9), "peaks": which}))
    ctx.poll_status()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default=None, choices=["gemm", "gemm_sweep", "attn"])
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--k", type=int, default=5120)
    ap.add_argument("--n", type=int, default=17408)
    ap.add_argument("--bits", type=int, default=4)
    ap.add_argument("--seqs", type=int, default=64)
    ap.add_argument("--kv-bits", type=int, default=0, help="--op attn: quantised KV pools with this many bits (0 = fp16 pools)")
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch the step's kernels one by one instead of replaying a CUDA graph")
    args = ap.parse_args()
    if args.op:
        run_ops(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
