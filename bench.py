#!/usr/bin/env python
"""Benchmark of the ragged continuous-batching decode step (27B-class dense model, EXL3 4 bpw, paged fp16 KV).

    python bench.py --gpus N --steps K --warmup W              # this library, one rank per GPU (torchrun for N > 1)
    python bench.py --impl reference --steps K --warmup W      # CPU restatement of the same ops on the host cores

Workload (per GPU, weak scaling: sequences are partitioned across GPUs, a weight replica and a paged pool per GPU, no
collective on the step): 32 sequences = 28 decoding one token + 4 prefill chunks of 256 tokens, contexts uniform in
[512, 16384], 64 layers, hidden 5120, 40 q / 8 kv heads, head_dim 128, MLP 17408, vocab 151936, all weights seeded
random EXL3 codes.  The 256-sequence batch of the full configuration is this shard times 8 GPUs; on fewer GPUs the
fp16 KV of 256 sequences (about 567 GB) does not fit, so every GPU always holds 32 sequences.
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
SEQ_PER_GPU, N_PREFILL, CHUNK = 32, 4, 256
CTX_LO, CTX_HI = 512, 16384


def shard_batch(rank, seed=1234):
    """Per-rank sequences: (q_lens, ctx_lens, block_table, pages, ids)."""
    r = np.random.default_rng(seed + rank)
    q_lens = np.array([1] * (SEQ_PER_GPU - N_PREFILL) + [CHUNK] * N_PREFILL, np.int32)
    ctx = r.integers(CTX_LO, CTX_HI + 1, SEQ_PER_GPU).astype(np.int32)
    need = (ctx + q_lens + 255) // 256
    pps = int(need.max())
    pages = int(need.sum()) + 1
    perm = r.permutation(pages).astype(np.int32)
    bt = np.zeros((SEQ_PER_GPU, pps), np.int32)
    o = 0
    for b in range(SEQ_PER_GPU):
        bt[b, :need[b]] = perm[o:o + need[b]]
        o += need[b]
    ids = r.integers(0, CFG["vocab"], int(q_lens.sum())).astype(np.int64)
    return q_lens, ctx, bt, pages, ids


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


CPU_SAMPLE = ("one layer of the 64 (full widths, 4 bpw) over a 1/16-scale cut of a GPU's shard: 2 decode sequences + one "
              "prefill chunk of 64 rows (66 packed rows, 3 sequences), contexts in [512, 2048], composed from oracle/ ops; "
              "step time extrapolated as 64 x layer time")


def cpu_sample(steps=3, warmup=1):
    """Bounded CPU sample of the same step: ONE layer of the model (full widths) over 2 decode sequences and one prefill
    chunk of 64 rows (the shard's 28 : 1024 row mix at 1/16 scale) with contexts in [512, 2048], composed from the
    oracle's ops; a whole step is 64 such layers plus the head, so tokens/s is rows / (64 * t_layer).
    Returns (tokens_per_s, seconds_per_layer, threads)."""
    from oracle import oracle as O
    from oracle import oracle_model
    r = np.random.default_rng(7)
    c = CFG
    q_lens = np.array([1, 1, 64], np.int32)
    nseq, rows = len(q_lens), int(q_lens.sum())

    def lin(k, n):
        return dict(trellis=r.integers(-32768, 32768, size=(k // 16, n // 16, 16 * c["K"]), dtype=np.int16),
                    suh=(r.integers(0, 2, k) * 2 - 1).astype(np.float16),
                    svh=((r.integers(0, 2, n) * 2 - 1) / np.sqrt(k)).astype(np.float16), K=c["K"], cb=c["cb"])

    ctx = r.integers(512, 2049, nseq).astype(np.int32)
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
                 q_norm=np.ones(hd, np.float16), k_norm=np.ones(hd, np.float16),
                 k_cache=(0.5 * r.standard_normal((pages, 256, nkv, hd))).astype(np.float16),
                 v_cache=(0.5 * r.standard_normal((pages, 256, nkv, hd))).astype(np.float16))
    small_vocab = 1024     # the head is excluded from the sample (one layer only); a tiny head keeps the call valid
    m = dict(cfg=dict(c, vocab=small_vocab, kv_bits=0), embed=r.standard_normal((small_vocab, hid)).astype(np.float16),
             final_norm=np.ones(hid, np.float16), inv_freq=(1.0 / (1e6 ** (np.arange(0, hd, 2) / hd))).astype(np.float32),
             lm_head=dict(lin(hid, small_vocab)), layers=[layer])
    ids = r.integers(0, small_vocab, rows).astype(np.int64)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        oracle_model.step(m, ids, q_lens, ctx, bt)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    t_layer = float(np.mean(times))
    return rows / (c["n_layers"] * t_layer), t_layer, O.num_threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tps, t_layer, threads = cpu_sample(steps=max(1, min(args.steps, 5)), warmup=min(args.warmup, 1))
    sample = CPU_SAMPLE
    line = {"impl": "reference", "metric": "ragged decode-step tokens/s", "value": tps, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 64e3 * t_layer,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
            "config": {"workload": WORKLOAD_NAME},
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


WORKLOAD_NAME = ("27B-class dense decode step, 4 bpw EXL3, fp16 paged KV: per GPU 28 decode rows + 4 prefill chunks of 256 "
                 "(1052 packed rows, 32 sequences), contexts U[512,16384]")


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops_sustained", 1400.0), "measured"
    return 6650.0, 1400.0, "fallback"


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
    ctx = exl3b200.Ctx(local, workspace_bytes=1 << 30)
    q_lens, ctx_lens, bt, pages, ids = shard_batch(rank)
    rows, bsz = int(q_lens.sum()), len(q_lens)
    model = SyntheticModel(pages=pages, kv_bits=0, seed=100 + rank, device=dev, **CFG)
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
    # fixed, their contents change per step.  --no-graph launches the ~1200 kernels of a step one by one instead.
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
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        return reduce_max_ms(e0.elapsed_time(e1), world, dev)

    for _ in range(max(args.warmup, 3)):
        step_resident()
    ctx.poll_status()
    sampler = ClockSampler(local)
    sampler.start()
    l0 = ctx.launch_count()
    # a profiler started with `--profile-from-start off` sees exactly the timed steps (no effect otherwise)
    torch.cuda.cudart().cudaProfilerStart()
    ms_total = timed(step_resident, args.steps)
    torch.cuda.cudart().cudaProfilerStop()
    launches = launches_captured if graph is not None else (ctx.launch_count() - l0) // max(args.steps, 1)
    clocks = sampler.stop()
    step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    ctx.poll_status()

    ms_step = ms_total / args.steps
    value = whole_job_value(rows, world, ms_step)
    e2e_value = whole_job_value(rows, world, ms_e2e / args.steps)
    h2d = int(ids.nbytes + q_lens.nbytes + ctx_lens.nbytes + bt.nbytes)

    # ---- roofline of the dominant kernel: the EXL3 GEMM at the step's row count, timed on L2-cold weights (the 64
    # layers' gate_proj tensors in turn; 44.6 MB each, 2.9 GB in total)
    hbm_peak, tf_peak, which = peaks()
    roof = None
    if rank == 0:
        x = (torch.randn(rows, CFG["hidden"], device=dev) * 0.1).to(torch.float16)
        y = torch.empty(rows, CFG["inter"], dtype=torch.float16, device=dev)
        lins = [L["gate_proj"] for L in model.layers]
        for l in lins[:3]:
            ctx.exl3_gemm(x, l.trellis, y, l.suh, None, l.svh, mcg=True)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        g0 = ctx.launch_count()
        cur = torch.cuda.current_stream()
        e0.record(cur)
        for l in lins:
            ctx.exl3_gemm(x, l.trellis, y, l.suh, None, l.svh, mcg=True)
        e1.record(cur)
        torch.cuda.synchronize()
        t_op = e0.elapsed_time(e1) * 1e-3 / len(lins)
        flops = 2.0 * rows * CFG["hidden"] * CFG["inter"]
        ach = flops / t_op / 1e12
        kv_bytes = float((ctx_lens + q_lens).sum()) * CFG["nkv"] * CFG["hd"] * 2 * 2 * CFG["n_layers"]
        step_bytes = model.weight_bytes() + kv_bytes
        roof = {"bound": "tensor", "kernel": "exl3_gemm (gate_proj 5120x17408, M=%d)" % rows, "achieved": ach,
                "peak": tf_peak, "unit": "TFLOP/s", "frac": ach / tf_peak,
                # DRAM bytes of one gemm_tc_kernel launch at this shape (dram__bytes_read.sum + dram__bytes_write.sum of the
                # ncu capture summarised in profiles/gemm_tc_kernel_m1052_k5120_n17408_4bpw.md): the 44.6 MB of codes once,
                # the transformed activations, and the part of the output that leaves L2
                "traffic": 57940224 + 10788096, "peak_source": which,
                "launches_per_op": (ctx.launch_count() - g0) // len(lins), "op_ms": t_op * 1e3,
                "step_hbm_gbs": step_bytes / (ms_step * 1e-3) / 1e9, "step_hbm_frac": step_bytes / (ms_step * 1e-3) / 1e9 / hbm_peak}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        tps, t_layer, threads = cpu_sample()
        cpu = {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
               "sample": CPU_SAMPLE + " (%.2f s per layer)" % t_layer}
    if rank == 0:
        line = {"metric": "ragged decode-step tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
                "config": {"workload": WORKLOAD_NAME, "rows_per_gpu": rows, "sequences_per_gpu": bsz,
                           "generated_tokens_per_s": bsz * world / (ms_step * 1e-3),
                           "l2": "inputs larger than L2 (11 GB of weights and the KV pool are streamed every step)"},
                "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                        "d2h_bytes_per_step": bsz * 8},
                "gpu_launches": int(launches), "launch_mode": "cuda graph replay" if graph is not None else "stream launches",
                "clocks": clocks, "roofline": roof, "cpu_baseline": cpu}
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
