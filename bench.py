"""Benchmark of the block-scaled quantize -> dense GEMM path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = group_wise_quant(A) + group_wise_quant(B) + dense_gemm, MXFP8, on
the large square configuration M = N = K = 8192 (A ~ N(0,1), B ~ N(0,0.02),
seeded synthetic data, which is also what the reference's own benchmark uses).
With N > 1 ranks (torchrun, one per GPU) every rank owns one 8192-column shard
of a weight that is N x 8192 columns wide (column-parallel, no data-path
collective): weak scaling.  Prints ONE JSON line on rank 0.

``--impl reference`` times the reference's CPU path of the same step (torch
quantise + float32 dequantise-then-matmul, all host threads) on a bounded
sample of the workload and extrapolates it to the whole step.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M = N_LOCAL = K = 8192
MODE = "w8a8-mxfp8"
NOMINAL_FP8_TFLOPS = 4500.0


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken during the timed region."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=self.file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        clocks, maxes, power, reasons = [], [], [], set()
        for line in self.file.read().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                clocks.append(float(f[1]))
                maxes.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        self.file.close()
        os.unlink(self.file.name)
        if clocks:
            clocks.sort()
            out.update(sm_mhz=clocks[len(clocks) // 2], sm_max_mhz=max(maxes), reasons=sorted(reasons),
                       samples=len(clocks), power_w_max=max(power))
        return out


def _dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ----------------------------------------------------------------------------- CPU arm


def cpu_reference_step(sample_m: int, sample_n: int, threads: int):
    """One bounded sample of the step on the host: quantise an [sample_m, K]
    block of A and an [sample_n, K] block of B, dequantise both and multiply
    them in float32.  Returns the measured times of the three parts."""
    from oracle.cpu_path import dequant_mxfp8_torch, quant_mxfp8_torch

    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(2027)
    a = torch.randn([sample_m, K], generator=g).to(torch.bfloat16)
    b = (torch.randn([sample_n, K], generator=g) * 0.02).to(torch.bfloat16)
    t0 = time.perf_counter()
    aq, sfa = quant_mxfp8_torch(a)
    bq, sfb = quant_mxfp8_torch(b)
    t1 = time.perf_counter()
    ad, bd = dequant_mxfp8_torch(aq, sfa), dequant_mxfp8_torch(bq, sfb)
    t2 = time.perf_counter()
    out = torch.matmul(ad, bd.T).to(torch.bfloat16)
    t3 = time.perf_counter()
    return t1 - t0, t2 - t1, t3 - t2, float(out[0, 0])


def cpu_baseline(steps: int, warmup: int, sample_m: int = 512, sample_n: int = 2048):
    """Times the sample `steps` times and extrapolates to the whole step:
    quantise and dequantise scale with the elements, the matmul with the flops."""
    threads = os.cpu_count() or 1
    for _ in range(warmup):
        cpu_reference_step(sample_m, sample_n, threads)
    tq = td = tm = 0.0
    t_begin = time.perf_counter()
    for _ in range(steps):
        q, d, mm, _ = cpu_reference_step(sample_m, sample_n, threads)
        tq += q
        td += d
        tm += mm
    wall = time.perf_counter() - t_begin
    elem_ratio = (M + N_LOCAL) * K / ((sample_m + sample_n) * K)
    flop_ratio = (2.0 * M * N_LOCAL * K) / (2.0 * sample_m * sample_n * K)
    full = (tq + td) / steps * elem_ratio + tm / steps * flop_ratio
    tflops = 2.0 * M * N_LOCAL * K / full / 1e12
    sample = (f"{sample_m}x{K} block of A and {sample_n}x{K} block of B quantised (torch, MXFP8), "
              f"dequantised and multiplied in float32; quantise and dequantise times scaled by elements "
              f"and the matmul time by flops to the full {M}x{N_LOCAL}x{K} step")
    return {"value": tflops, "unit": "TFLOPS", "cores": threads, "kind": "port", "sample": sample,
            "ms_per_sample_step": 1e3 * wall / steps}


def run_reference(args):
    rank, world, _ = _dist_env()
    if rank != 0:
        return
    base = cpu_baseline(max(args.steps, 1), args.warmup)
    line = {
        "impl": "reference", "metric": "mxfp8_dense_gemm_tflops_quant_incl", "value": base["value"],
        "unit": "TFLOPS", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": base["ms_per_sample_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"C2 MXFP8 dense GEMM M=N=K={M}, quant(A)+quant(B)+GEMM per step",
                   "arm": "reference CPU path (torch quantise + float32 dequantise-then-matmul), rank 0 only"},
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- GPU arm


def run_ours(args):
    import halops_b200 as hq

    rank, world, local = _dist_env()
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    peaks = _peaks()
    g = torch.Generator(device=dev).manual_seed(2026 + 1)
    a = torch.randn([M, K], generator=g, device=dev).to(torch.bfloat16)
    # rank r owns columns [r * N_LOCAL, (r + 1) * N_LOCAL) of the global weight
    gw = torch.Generator(device=dev).manual_seed(4052 + rank)
    b = (torch.randn([N_LOCAL, K], generator=gw, device=dev) * 0.02).to(torch.bfloat16)
    out = torch.empty([M, N_LOCAL], dtype=torch.bfloat16, device=dev)
    aq = torch.empty([M, K], dtype=torch.float8_e4m3fn, device=dev)
    bq = torch.empty([N_LOCAL, K], dtype=torch.float8_e4m3fn, device=dev)
    sfa = torch.empty([M, K // 32], dtype=torch.uint8, device=dev)
    sfb = torch.empty([N_LOCAL, K // 32], dtype=torch.uint8, device=dev)

    def step():
        hq.group_wise_quant(a, MODE, True, True, aq, sfa)
        hq.group_wise_quant(b, MODE, True, True, bq, sfb)
        hq.dense_gemm(aq, bq, sfa, sfb, out, None, None, -1, MODE, True)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    assert hq.device_status(dev) == 0

    # ---- timed region: K steps, device time by CUDA events on the launching stream
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    steps = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for i in range(steps):
        ev[i][0].record()
        hq.group_wise_quant(a, MODE, True, True, aq, sfa)
        hq.group_wise_quant(b, MODE, True, True, bq, sfb)
        ev[i][1].record()
        hq.dense_gemm(aq, bq, sfa, sfb, out, None, None, -1, MODE, True)
        ev[i][2].record()
    stop.record()
    barrier()
    total_ms = start.elapsed_time(stop)
    quant_ms = sum(e[0].elapsed_time(e[1]) for e in ev) / steps
    gemm_ms = sum(e[1].elapsed_time(e[2]) for e in ev) / steps
    clocks = sampler.stop() if rank == 0 else None
    assert hq.device_status(dev) == 0

    # ---- GEMM alone and quantizer alone (explains the headline; same buffers, > L2 working set)
    def timed(fn, reps):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fn()
        torch.cuda.synchronize()
        s.record()
        for _ in range(reps):
            fn()
        e.record()
        torch.cuda.synchronize()
        return s.elapsed_time(e) / reps

    if args.kernels_only:
        # profiling aid: only the timed steps above run (keeps a profiler's launch list short)
        if rank == 0:
            print(json.dumps({"kernels_only": True, "ms_per_step": total_ms / steps, "gemm_ms": gemm_ms,
                              "quant_ms": quant_ms}), flush=True)
        if dist is not None:
            dist.destroy_process_group()
        return
    gemm_only_ms = timed(lambda: hq.dense_gemm(aq, bq, sfa, sfb, out, None, None, -1, MODE, False), max(steps, 5))
    quant_only_ms = timed(lambda: hq.group_wise_quant(a, MODE, True, False, aq, sfa), max(steps, 5))

    # ---- end to end through the public API with host buffers
    a_host = a.cpu().pin_memory()
    b_host = b.cpu().pin_memory()
    out_host = torch.empty([M, N_LOCAL], dtype=torch.bfloat16).pin_memory()
    # Every step copies its own inputs in and its own result out; consecutive steps overlap on
    # three streams (copy in / kernels / copy out) with two sets of device buffers, as a serving
    # loop would: PCIe carries 268 MB in and 134 MB out per step, in both directions at once.
    a_dev = [torch.empty_like(a) for _ in range(2)]
    b_dev = [torch.empty_like(b) for _ in range(2)]
    out_dev = [torch.empty_like(out) for _ in range(2)]
    s_in, s_run, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]        # inputs of the step are on the device
    ev_in_free = [torch.cuda.Event() for _ in range(2)]   # the quantizers have read them
    ev_run = [torch.cuda.Event() for _ in range(2)]       # the GEMM has written out_dev
    ev_out = [torch.cuda.Event() for _ in range(2)]       # the result is in host memory

    def e2e_step(i):
        j = i & 1
        s_in.wait_event(ev_in_free[j])
        with torch.cuda.stream(s_in):
            a_dev[j].copy_(a_host, non_blocking=True)
            b_dev[j].copy_(b_host, non_blocking=True)
            ev_in[j].record(s_in)
        s_run.wait_event(ev_in[j])
        s_run.wait_event(ev_out[j])
        with torch.cuda.stream(s_run):
            xq, xs = hq.group_wise_quant(a_dev[j], MODE, True, True, aq, sfa)
            wq, ws = hq.group_wise_quant(b_dev[j], MODE, True, True, bq, sfb)
            ev_in_free[j].record(s_run)
            hq.dense_gemm(xq, wq, xs, ws, out_dev[j], None, None, -1, MODE, True)
            ev_run[j].record(s_run)
        s_out.wait_event(ev_run[j])
        with torch.cuda.stream(s_out):
            out_host.copy_(out_dev[j], non_blocking=True)
            ev_out[j].record(s_out)

    e2e_steps = max(4, min(steps, 10))
    e2e_step(0)
    e2e_step(1)
    torch.cuda.synchronize(dev)
    barrier()
    cur = torch.cuda.current_stream(dev)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record(cur)
    for st in (s_in, s_run, s_out):
        st.wait_event(s)
    for i in range(e2e_steps):
        e2e_step(i)
    for st in (s_in, s_run, s_out):
        cur.wait_stream(st)
    e.record(cur)
    barrier()
    e2e_ms = s.elapsed_time(e) / e2e_steps
    # the bytes that came back are the GEMM's (same operands as the device-resident steps above)
    torch.cuda.synchronize(dev)
    assert torch.equal(out_host, out.cpu()), "end-to-end result differs from the device-resident one"

    # ---- max over ranks
    times = torch.tensor([total_ms, gemm_ms, quant_ms, gemm_only_ms, quant_only_ms, e2e_ms], device=dev,
                         dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, gemm_ms, quant_ms, gemm_only_ms, quant_only_ms, e2e_ms = times.tolist()

    flops_rank = 2.0 * M * N_LOCAL * K
    ms_per_step = total_ms / steps
    value = world * flops_rank / (ms_per_step * 1e-3) / 1e12
    gemm_tflops = flops_rank / (gemm_ms * 1e-3) / 1e12
    timed_seconds = total_ms * 1e-3
    fp8_peak = 2.0 * (peaks["bf16"] if timed_seconds < 1.0 else peaks["bf16_sustained"])
    pair_tile = "pair=1" in hq.describe_tile(M, N_LOCAL, K, MODE, device=local)
    quant_bytes = M * K * (2 + 1 + 1 / 32)

    if rank == 0:
        base = cpu_baseline(steps=2, warmup=1) if world == 1 and not args.no_cpu_baseline else None
        line = {
            "metric": "mxfp8_dense_gemm_tflops_quant_incl", "value": value, "unit": "TFLOPS", "n_gpus": world,
            "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32 accumulate -> bf16",
            "data": "synthetic",
            "config": {
                "workload": f"C2 MXFP8 dense GEMM M=N=K={M} per GPU: group_wise_quant(A) + group_wise_quant(B) + "
                            "dense_gemm per step; N>1: column-parallel, one 8192-column weight shard per rank",
                "cache": "inputs larger than L2 (A and B bf16 128 MiB each, e4m3 64 MiB each, output 128 MiB)",
                "tile": hq.describe_tile(M, N_LOCAL, K, MODE, device=local),
            },
            "gemm_only": {"tflops_in_step": gemm_tflops, "ms_in_step": gemm_ms,
                          "tflops_alone": flops_rank / (gemm_only_ms * 1e-3) / 1e12, "ms_alone": gemm_only_ms,
                          "frac_of_nominal_fp8": gemm_tflops / NOMINAL_FP8_TFLOPS},
            "quant": {"ms_both_in_step": quant_ms, "ms_one_operand_alone": quant_only_ms,
                      "gbs_alone": quant_bytes / (quant_only_ms * 1e-3) / 1e9,
                      "frac_of_hbm": quant_bytes / (quant_only_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                      "bytes_per_element": 3.03125},
            "roofline": {"kernel": ("gemm_pair_kernel<256, mxfp8> (256x256x128 2-CTA tile)" if pair_tile else
                                    "gemm_kernel<256, mxfp8> (128x256x128 single-CTA tile)"),
                         "bound": "tensor", "achieved": gemm_tflops,
                         "peak": fp8_peak, "unit": "TFLOP/s", "frac": gemm_tflops / fp8_peak,
                         # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this
                         # workload (ncu captures summarised in profiles/gemm_pair_kernel_mxfp8_256x256_c2_ncu.md
                         # and profiles/gemm_kernel_mxfp8_128x256_c2_ncu.md)
                         "traffic": 478.3e6 if pair_tile else 605.2e6,
                         "algorithmic_bytes": 64 * 2**20 * 2 + 4 * 2**20 + 128 * 2**20,
                         "peak_source": f"2 x {peaks['source']} cuBLAS bf16 "
                                        f"({'burst' if timed_seconds < 1.0 else 'sustained'}) as the dense fp8 peak"},
            "e2e": {"value": world * flops_rank / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOPS",
                    "h2d_bytes_per_step": 2 * M * K * 2, "d2h_bytes_per_step": M * N_LOCAL * 2,
                    "ms_per_step": e2e_ms,
                    "overlap": "consecutive steps pipelined over 3 streams (copy in, kernels, copy out), 2 buffer sets"},
            "gpu_launches": 3 * steps,
            "clocks": clocks,
        }
        if base is not None:
            line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


# ----------------------------------------------------------------------------- config 5 (N-sharded, strong scaling)


def run_c5(args):
    """Config 5: M=16384, N=57344, K=8192 MXFP8, weight rows (output columns) split
    over the ranks; the activation is replicated and quantised on every rank.  Strong
    scaling: the whole job is fixed, each rank computes N/world columns.  Reports the
    aggregate TFLOPS of quantise + GEMM, of the GEMM alone, and with the NCCL all-gather
    of the bf16 output added (max over ranks, CUDA events)."""
    import halops_b200 as hq
    from halops_b200.dist import ColumnParallelDenseGemm, shard_bounds

    rank, world, local = _dist_env()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)
    m, n, k = 16384, 57344, 8192
    start, rows = shard_bounds(n, world, rank)
    g = torch.Generator(device=dev).manual_seed(2031)
    x = torch.randn([m, k], generator=g, device=dev).to(torch.bfloat16)
    gw = torch.Generator(device=dev).manual_seed(7000 + rank)
    w = (torch.randn([rows, k], generator=gw, device=dev) * 0.02).to(torch.bfloat16)
    layer = ColumnParallelDenseGemm(w, mode=MODE)
    out = torch.empty([m, rows], dtype=torch.bfloat16, device=dev)
    xq = torch.empty([m, k], dtype=torch.float8_e4m3fn, device=dev)
    sfa = torch.empty([m, k // 32], dtype=torch.uint8, device=dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, reps):
        for _ in range(3):
            fn()
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(reps):
            fn()
        e.record()
        barrier()
        t = torch.tensor([s.elapsed_time(e) / reps], device=dev, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def gemm_only():
        layer.local_quantized(xq, sfa, out)

    def quant_gemm():
        hq.group_wise_quant(x, MODE, True, True, xq, sfa)
        layer.local_quantized(xq, sfa, out)

    def quant_gemm_gather():
        quant_gemm()
        layer.gather(out)

    hq.group_wise_quant(x, MODE, True, True, xq, sfa)
    reps = max(3, min(args.steps, 10))
    t_gemm = timed(gemm_only, reps)
    t_step = timed(quant_gemm, reps)
    t_gather = timed(quant_gemm_gather, reps) if world > 1 else t_step
    assert hq.device_status(dev) == 0
    flops = 2.0 * m * n * k
    if rank == 0:
        print(json.dumps({
            "metric": "mxfp8_dense_gemm_tflops_quant_incl", "value": flops / (t_step * 1e-3) / 1e12, "unit": "TFLOPS",
            "n_gpus": world, "steps": reps, "warmup": 3, "ms_per_step": t_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32 accumulate -> bf16",
            "data": "synthetic",
            "config": {"workload": f"C5 N-sharded MXFP8 GEMM M={m} N={n} K={k}, {rows} weight rows per rank; "
                                   "step = group_wise_quant(activation) + dense_gemm on the rank's shard "
                                   "(weights quantised once at load)",
                       "tile": hq.describe_tile(m, rows, k, MODE, device=local)},
            "gemm_only": {"tflops": flops / (t_gemm * 1e-3) / 1e12, "ms": t_gemm},
            "with_allgather": {"tflops": flops / (t_gather * 1e-3) / 1e12, "ms": t_gather,
                               "gathered_bytes_per_rank": m * (n - rows) * 2},
        }), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


# ----------------------------------------------------------------------------- shape sweep


SWEEP = (
    # (label, mode, M, N, K, A distribution, B scale)
    [("C1", "w8a8-mxfp8", 128, 256, 512, "normal", 1.0),
     ("C2", "w8a8-mxfp8", 8192, 8192, 8192, "normal", 0.02)]
    + [(f"C3 m={m}", "w8a8-mxfp8", m, n, k, "student_t", 0.02)
       for (n, k) in ((7168, 2048), (24576, 1536)) for m in (1, 8, 32, 64, 128)]
    + [("C4", "w4a4-nvfp4", 4096, 14336, 4096, "normal", 1.0),
       ("C5 shard of 8", "w8a8-mxfp8", 16384, 7168, 8192, "normal", 0.02),
       ("ref CI 8192x4096x4096", "w8a8-mxfp8", 8192, 4096, 4096, "normal", 1.0),
       ("ref CI 8192x4096x4096", "w4a4-nvfp4", 8192, 4096, 4096, "normal", 1.0),
       ("ref CI 128x256x512", "w4a4-nvfp4", 128, 256, 512, "normal", 1.0),
       ("ref README 1024x4096x8192", "w8a8-mxfp8", 1024, 4096, 8192, "normal", 1.0)]
)


def run_sweep(args):
    """GEMM-only and quantizer-only medians for every benchmark configuration and the
    reference's published shapes, measured the way the reference's benchmark does
    (cold L2: a 256 MiB buffer is zeroed before every timed call; 10 warm-up, 30 timed).
    One JSON object per line; not the driver's contract line."""
    import halops_b200 as hq

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = _peaks()
    flush = torch.empty([256 << 20], dtype=torch.uint8, device=dev)

    def median_us(fn, warm=10, reps=30):
        for _ in range(warm):
            fn()
        ts = []
        for _ in range(reps):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e) * 1e3)
        ts.sort()
        return ts[len(ts) // 2]

    for label, mode, m, n, k, dist, bscale in SWEEP:
        g = torch.Generator(device=dev).manual_seed(2026)
        a = torch.randn([m, k], generator=g, device=dev)
        if dist == "student_t":
            a = a / torch.sqrt(torch.randn([3, m, k], generator=g, device=dev).pow(2).sum(0) / 3)
        a = a.to(torch.bfloat16)
        b = (torch.randn([n, k], generator=g, device=dev) * bscale).to(torch.bfloat16)
        aq, sfa = hq.group_wise_quant(a, mode=mode)
        bq, sfb = hq.group_wise_quant(b, mode=mode)
        out = torch.empty([m, n], dtype=torch.bfloat16, device=dev)
        alpha = torch.ones([1], dtype=torch.float32, device=dev) if mode == "w4a4-nvfp4" else None
        gemm_us = median_us(lambda: hq.dense_gemm(aq, bq, sfa, sfb, out, None, alpha, -1, mode, False))
        qa_us = median_us(lambda: hq.group_wise_quant(a, mode=mode, use_pdl=False))
        qb_us = median_us(lambda: hq.group_wise_quant(b, mode=mode, use_pdl=False))
        assert hq.device_status(dev) == 0
        fp8 = mode == "w8a8-mxfp8"
        group = 32 if fp8 else 16
        bpe = 1.0 if fp8 else 0.5
        gemm_bytes = bpe * (m * k + n * k) + ((m + 127) // 128 * 128 + n) * k / group + 2.0 * m * n
        q_bpe = 2 + bpe + 1.0 / group
        flops = 2.0 * m * n * k
        print(json.dumps({
            "config": label, "mode": mode, "m": m, "n": n, "k": k,
            "tile": hq.describe_tile(m, n, k, mode).split("-> ")[1],
            "gemm_us": round(gemm_us, 2), "gemm_tflops": round(flops / gemm_us / 1e6, 1),
            "gemm_gbs": round(gemm_bytes / gemm_us / 1e3, 1),
            "gemm_frac_of_hbm": round(gemm_bytes / gemm_us / 1e3 / peaks["hbm_gbs"], 3),
            "quant_a_us": round(qa_us, 2), "quant_b_us": round(qb_us, 2),
            "quant_b_gbs": round(n * k * q_bpe / qb_us / 1e3, 1),
            "quant_incl_tflops": round(flops / (gemm_us + qa_us + qb_us) / 1e6, 1),
        }), flush=True)
    run_sweep_next_rows(median_us, dev, peaks)


def run_sweep_next_rows(median_us, dev, peaks):
    """Rows beyond the dense path: rms_norm_quant and the non-Identity epilogues."""
    import halops_b200 as hq

    for m, k in ((3072, 8192), (16384, 4096), (128, 4096)):
        g = torch.Generator(device=dev).manual_seed(9)
        x = (torch.randn([m, k], generator=g, device=dev) * 3).to(torch.bfloat16)
        w = (torch.rand([k], generator=g, device=dev) + 0.5).to(torch.bfloat16)
        us = median_us(lambda: hq.rms_norm_quant(x, w, 1e-6, True, False))
        nbytes = m * k * 3.03125 + k * 2
        print(json.dumps({"config": "rms_norm_quant", "m": m, "k": k, "us": round(us, 2),
                          "gbs": round(nbytes / us / 1e3, 1),
                          "frac_of_hbm": round(nbytes / us / 1e3 / peaks["hbm_gbs"], 3)}), flush=True)
    m, n, k = 4096, 7168, 2048
    g = torch.Generator(device=dev).manual_seed(10)
    a = torch.randn([m, k], generator=g, device=dev).to(torch.bfloat16)
    b = (torch.randn([n, k], generator=g, device=dev) * 0.05).to(torch.bfloat16)
    bias = torch.rand([n], generator=g, device=dev).to(torch.bfloat16)
    aq, sfa = hq.group_wise_quant(a)
    bq, sfb = hq.group_wise_quant(hq.interleave_gate_up(b).contiguous())
    out = torch.empty([m, n], dtype=torch.bfloat16, device=dev)
    q = torch.empty([m, n // 2], dtype=torch.float8_e4m3fn, device=dev)
    sf = torch.zeros([m * n // 64], dtype=torch.uint8, device=dev)
    flops = 2.0 * m * n * k
    for label, fn in (
        ("identity", lambda: hq.dense_gemm(aq, bq, sfa, sfb, out, None, None, -1, MODE, False)),
        ("bias", lambda: hq.dense_gemm(aq, bq, sfa, sfb, out, bias, None, -1, MODE, False)),
        ("sigmoid+bias", lambda: hq.dense_gemm(aq, bq, sfa, sfb, out, bias, None, -1, MODE, False,
                                                 hq.EpilogueOp.Sigmoid)),
        ("situ_quant", lambda: hq.dense_gemm(aq, bq, sfa, sfb, q, None, None, -1, MODE, False,
                                               hq.EpilogueOp.SituQuant, sf, 4.0, 25.0)),
    ):
        us = median_us(fn)
        print(json.dumps({"config": f"epilogue {label}", "m": m, "n": n, "k": k, "us": round(us, 2),
                          "tflops": round(flops / us / 1e6, 1)}), flush=True)
    assert hq.device_status(dev) == 0
    run_sweep_grouped(median_us, dev)
    run_sweep_low_latency(median_us, dev, peaks)


def run_sweep_grouped(median_us, dev):
    """Batch / MoE grouped GEMMs on the shapes of the reference's CI baselines
    (ci/baselines/gemm/group_*.json: 4 experts x 128 rows, N=256, K=512 and 10 experts x
    4096 rows, N=K=4096) plus a decode-like masked case with partly filled slots."""
    import halops_b200 as hq

    for mode in ("w8a8-mxfp8", "w4a4-nvfp4", "w4a8-mxfp4"):
        for experts, rows, n, k in ((4, 128, 256, 512), (10, 4096, 4096, 4096)):
            m = experts * rows
            g = torch.Generator(device=dev).manual_seed(12)
            x = torch.randn([m, k], generator=g, device=dev).to(torch.bfloat16)
            w = (torch.randn([experts * n, k], generator=g, device=dev) * 0.05).to(torch.bfloat16)
            # "w4a8-mxfp4" (grouped entries only): MXFP8 activations x MXFP4 weights
            xq, sfa = hq.group_wise_quant(x, mode="w8a8-mxfp8" if mode == "w4a8-mxfp4" else mode)
            wq, sfb = hq.group_wise_quant(w, mode="w4a4-mxfp4" if mode == "w4a8-mxfp4" else mode)
            wq, sfb = wq.view(experts, n, -1), sfb.view(experts, n, -1)
            del x, w
            alpha = torch.ones([experts], dtype=torch.float32, device=dev) if mode == "w4a4-nvfp4" else None
            out = torch.empty([m, n], dtype=torch.bfloat16, device=dev)
            out_b = torch.empty([rows, experts * n], dtype=torch.bfloat16, device=dev)
            full = torch.full([experts], rows, dtype=torch.int32, device=dev)
            half = torch.full([experts], rows // 2, dtype=torch.int32, device=dev)
            ids = (torch.arange(m, device=dev, dtype=torch.int32) // rows).contiguous()
            cases = (
                ("group_masked", 1.0, lambda: hq.group_masked_gemm(xq, wq, sfa, sfb, full, out, None, alpha, rows, -1, mode)),
                ("group_masked half-filled", 0.5,
                 lambda: hq.group_masked_gemm(xq, wq, sfa, sfb, half, out, None, alpha, rows, -1, mode)),
                ("group_contiguous", 1.0,
                 lambda: hq.group_contiguous_gemm(xq, wq, sfa, sfb, ids, out, None, alpha, -1, mode)),
                ("batch", 1.0, lambda: hq.batch_gemm(xq.view(experts, rows, -1), wq, sfa, sfb, out_b, None, alpha,
                                                     -1, mode, use_pdl=False)),
            )
            for label, filled, fn in cases[:3] if mode == "w4a8-mxfp4" else cases:
                us = median_us(fn)
                print(json.dumps({"config": label, "mode": mode, "experts": experts, "rows_per_expert": rows,
                                  "n": n, "k": k, "us": round(us, 2),
                                  "tflops": round(2.0 * m * n * k * filled / us / 1e6, 1)}), flush=True)
            assert hq.device_status(dev) == 0


def run_sweep_low_latency(median_us, dev, peaks):
    """low_latency_mma_gemm (M <= 16, plain scales) next to dense_gemm on the same operands."""
    import halops_b200 as hq

    for m, n, k in ((1, 4096, 4096), (8, 8192, 1024), (16, 7168, 2048), (16, 24576, 1536), (8, 32768, 1024)):
        g = torch.Generator(device=dev).manual_seed(13)
        x = torch.randn([m, k], generator=g, device=dev).to(torch.bfloat16)
        w = (torch.randn([n, k], generator=g, device=dev) * 0.02).to(torch.bfloat16)
        xq, sfa = hq.group_wise_quant(x, use_swizzle=False)
        wq, sfb = hq.group_wise_quant(w, use_swizzle=False)
        _, sfa_sw = hq.group_wise_quant(x)
        _, sfb_sw = hq.group_wise_quant(w)
        out = torch.empty([m, n], dtype=torch.bfloat16, device=dev)
        ll_us = median_us(lambda: hq.low_latency_mma_gemm(xq, wq, sfa, sfb, out, use_pdl=False))
        dense_us = median_us(lambda: hq.dense_gemm(xq, wq, sfa_sw, sfb_sw, out, None, None, -1, MODE, False))
        nbytes = n * k * (1 + 1 / 32)
        print(json.dumps({"config": "low_latency_mma_gemm", "m": m, "n": n, "k": k, "us": round(ll_us, 2),
                          "weight_gbs": round(nbytes / ll_us / 1e3, 1),
                          "frac_of_hbm": round(nbytes / ll_us / 1e3 / peaks["hbm_gbs"], 3),
                          "dense_gemm_us": round(dense_us, 2)}), flush=True)
    assert hq.device_status(dev) == 0


def run_shape(args):
    """One dense GEMM shape, GEMM only: MODE,M,N,K.  Prints one JSON line (cold-L2 median);
    with --kernels-only just 3 warm-up and 3 measured launches, for profiler captures."""
    import halops_b200 as hq

    mode, m, n, k = args.shape.split(",")
    m, n, k = int(m), int(n), int(k)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(2026)
    a = torch.randn([m, k], generator=g, device=dev).to(torch.bfloat16)
    b = (torch.randn([n, k], generator=g, device=dev) * 0.02).to(torch.bfloat16)
    aq, sfa = hq.group_wise_quant(a, mode=mode)
    bq, sfb = hq.group_wise_quant(b, mode=mode)
    out = torch.empty([m, n], dtype=torch.bfloat16, device=dev)
    alpha = torch.ones([1], dtype=torch.float32, device=dev) if mode == "w4a4-nvfp4" else None
    flush = torch.empty([256 << 20], dtype=torch.uint8, device=dev)
    reps = 3 if args.kernels_only else 30
    for _ in range(3):
        hq.dense_gemm(aq, bq, sfa, sfb, out, None, alpha, -1, mode, False)
    ts = []
    for _ in range(reps):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        hq.dense_gemm(aq, bq, sfa, sfb, out, None, alpha, -1, mode, False)
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e) * 1e3)
    assert hq.device_status(dev) == 0
    ts.sort()
    us = ts[len(ts) // 2]
    print(json.dumps({"shape": args.shape, "tile": hq.describe_tile(m, n, k, mode).split("-> ")[1],
                      "gemm_us": round(us, 2), "gemm_tflops": round(2.0 * m * n * k / us / 1e6, 1)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kernels-only", action="store_true",
                    help="run only warm-up and the timed steps (for profiler captures)")
    ap.add_argument("--sweep", action="store_true",
                    help="time every benchmark configuration (GEMM only / quantizer only, cold L2) instead")
    ap.add_argument("--c5", action="store_true",
                    help="run config 5 (M=16384, N=57344, K=8192 split over the ranks, strong scaling) instead")
    ap.add_argument("--shape", default=None, metavar="MODE,M,N,K",
                    help="time one dense GEMM shape (GEMM only, cold L2) instead, e.g. w8a8-mxfp8,16,24576,1536")
    args = ap.parse_args()
    if args.shape:
        run_shape(args)
    elif args.sweep:
        run_sweep(args)
    elif args.c5:
        run_c5(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
