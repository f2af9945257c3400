"""Benchmark of the block-scaled quantize -> dense GEMM path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

The workload is the N-sharded configuration: MXFP8 dense GEMM with M = 16384,
N = 57344, K = 8192 (activation ~ N(0,1), weight ~ N(0,0.02), seeded synthetic
data, which is also what the reference's own benchmark uses).  The weight rows
(output columns) are split over the ranks (torchrun, one per GPU); the weight is
quantised once at load, the activation is replicated.  One step =
group_wise_quant(activation) + dense_gemm on the rank's shard: strong scaling,
no data-path collective.  The optional NCCL all-gather of the bf16 output,
overlapped with the GEMM block by block, is timed beside it.  With one GPU the
line also carries the large square configuration (M = N = K = 8192, both
operands quantised inside the step) as the ``c2`` record.  Prints ONE JSON line
on rank 0.

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

M5, N5, K5 = 16384, 57344, 8192      # the N-sharded configuration
M2 = N2 = K2 = 8192                  # the large square configuration
WEIGHT_BLOCK = 7168                  # weight rows generated per seed: an eighth of N5
MODE = "w8a8-mxfp8"
NOMINAL_FP8_TFLOPS = 4500.0
METRIC = "mxfp8_dense_gemm_tflops_quant_incl"
WORKLOAD = (f"C5 N-sharded MXFP8 dense GEMM M={M5} N={N5} K={K5}, weight rows split over the GPUs; step = "
            "group_wise_quant(activation) + dense_gemm on the rank's shard (weight quantised once at load)")
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the 2-CTA 256x256 kernel
# on 16384 x 7168 x 8192 (ncu, one launch); a rank's launch covers N5 / world / 7168 such
# column blocks, whose tiles are walked one block of 8 row tiles x all columns at a time,
# so the traffic grows in proportion
TRAFFIC_PER_7168_COLUMNS = 897.6e6
TRAFFIC_SOURCE = ("ncu capture of one launch of this kernel on 16384 x 7168 x 8192 (677.5 MB read + 220.1 MB "
                  "written), times the number of 7168-column blocks of the rank's shard")


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples of one GPU (named by its UUID, so that a
    remapped CUDA_VISIBLE_DEVICES cannot point the query at another GPU) taken during a
    timed region.  Read-only."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: torch.device):
        try:
            uuid = str(torch.cuda.get_device_properties(device).uuid)
            self.gpu_id = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:
            self.gpu_id = str(device.index)
        self.proc = None
        self.file = None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_id}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
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


class SmClock:
    """Instantaneous SM clock of one GPU through NVML (read-only), for per-row clock notes
    of the sweep, whose timed loops are too short for a sampling process."""

    def __init__(self, device: torch.device):
        self.handle = None
        try:
            import pynvml

            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device).uuid)
            uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
        except Exception:
            self.handle = None

    def mhz(self):
        if self.handle is None:
            return None
        try:
            return float(self.nvml.nvmlDeviceGetClockInfo(self.handle, self.nvml.NVML_CLOCK_SM))
        except Exception:
            return None


def _dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


# ----------------------------------------------------------------------------- CPU arm


def cpu_reference_step(sample_m: int, sample_n: int, threads: int):
    """One bounded sample of the step on the host: quantise an [sample_m, K] block of the
    activation, dequantise it and an [sample_n, K] block of the (already quantised)
    weight, and multiply them in float32.  Returns the times of the parts."""
    from oracle.cpu_path import dequant_mxfp8_torch, quant_mxfp8_torch

    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(2027)
    a = torch.randn([sample_m, K5], generator=g).to(torch.bfloat16)
    b = (torch.randn([sample_n, K5], generator=g) * 0.02).to(torch.bfloat16)
    bq, sfb = quant_mxfp8_torch(b)  # at load, not timed
    t0 = time.perf_counter()
    aq, sfa = quant_mxfp8_torch(a)
    t1 = time.perf_counter()
    ad = dequant_mxfp8_torch(aq, sfa)
    t2 = time.perf_counter()
    bd = dequant_mxfp8_torch(bq, sfb)
    t3 = time.perf_counter()
    out = torch.matmul(ad, bd.T).to(torch.bfloat16)
    t4 = time.perf_counter()
    return t1 - t0, t2 - t1, t3 - t2, t4 - t3, float(out[0, 0])


def cpu_baseline(steps: int, warmup: int, sample_m: int = 512, sample_n: int = 2048):
    """Times the sample `steps` times and extrapolates to the whole step: quantise and
    dequantise scale with the elements of their operand, the matmul with the flops."""
    threads = os.cpu_count() or 1
    for _ in range(warmup):
        cpu_reference_step(sample_m, sample_n, threads)
    tq = tda = tdb = tm = 0.0
    t_begin = time.perf_counter()
    for _ in range(steps):
        q, da, db, mm, _ = cpu_reference_step(sample_m, sample_n, threads)
        tq += q
        tda += da
        tdb += db
        tm += mm
    wall = time.perf_counter() - t_begin
    full = ((tq + tda) / steps * (M5 / sample_m) + tdb / steps * (N5 / sample_n) +
            tm / steps * (M5 / sample_m) * (N5 / sample_n))
    tflops = 2.0 * M5 * N5 * K5 / full / 1e12
    sample = (f"{sample_m}x{K5} block of the activation quantised (torch, MXFP8) and dequantised, {sample_n}x{K5} "
              f"block of the quantised weight dequantised, the two multiplied in float32; quantise and dequantise "
              f"times scaled by the elements of their operand and the matmul time by flops to the full "
              f"{M5}x{N5}x{K5} step")
    return {"value": tflops, "unit": "TFLOPS", "cores": threads, "kind": "port", "sample": sample,
            "ms_per_sample_step": 1e3 * wall / steps}


def run_reference(args):
    rank, world, _ = _dist_env()
    if rank != 0:
        return
    base = cpu_baseline(max(args.steps, 1), args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"],
        "unit": "TFLOPS", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": base["ms_per_sample_step"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "arm": "reference CPU path (torch quantise + float32 dequantise-then-matmul), rank 0 only"},
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- GPU arm


def make_weight_rows(first_block: int, blocks: int, dev) -> torch.Tensor:
    """Rows [first_block * 7168, (first_block + blocks) * 7168) of the global weight; block j
    has a seed of its own, so a shard equals the same rows of the single-GPU weight."""
    parts = []
    for j in range(first_block, first_block + blocks):
        gw = torch.Generator(device=dev).manual_seed(7000 + j)
        parts.append((torch.randn([WEIGHT_BLOCK, K5], generator=gw, device=dev) * 0.02).to(torch.bfloat16))
    return torch.cat(parts) if len(parts) > 1 else parts[0]


def dequant_rows_on_device(q: torch.Tensor, sf: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    """float32 values of the given rows of an MXFP8 matrix whose UE8M0 scales are in SfAtom
    order (checker of the shard check: plain torch ops on the device, no kernel of the
    library)."""
    k = q.size(1)
    kb = k // 32
    r = rows.to(torch.int64)[:, None]
    c = torch.arange(kb, device=q.device, dtype=torch.int64)[None, :]
    off = ((r // 128) * (kb // 4) + c // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + c % 4
    scale = torch.exp2(sf.reshape(-1)[off].to(torch.float32) - 127.0)
    return (q[rows].to(torch.float32).view(rows.numel(), kb, 32) * scale[..., None]).view(rows.numel(), k)


def shard_check(xq, sfa, wq, sfb, out, sample: int = 64):
    """max |out - ref| / max |ref| over `sample` rows of the rank's output, ref = float32
    dequantise-then-matmul computed with torch ops on the device."""
    m, n = out.shape
    rows = torch.linspace(0, m - 1, sample, device=out.device).round().to(torch.int64).unique()
    a = dequant_rows_on_device(xq, sfa, rows)
    err = ref_max = 0.0
    for n0 in range(0, n, 8192):
        cols = torch.arange(n0, min(n, n0 + 8192), device=out.device)
        ref = a @ dequant_rows_on_device(wq, sfb, cols).T
        err = max(err, float((out[rows][:, n0:n0 + cols.numel()].float() - ref).abs().max()))
        ref_max = max(ref_max, float(ref.abs().max()))
    return err / max(ref_max, 1e-30), int(rows.numel())


def timed_ms(fn, reps, barrier=None):
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fn()
    (barrier or torch.cuda.synchronize)()
    s.record()
    for _ in range(reps):
        fn()
    e.record()
    (barrier or torch.cuda.synchronize)()
    return s.elapsed_time(e) / reps


def bench_c2(hq, dev, steps, peaks):
    """The large square configuration on one GPU: quant(A) + quant(B) + GEMM per step."""
    g = torch.Generator(device=dev).manual_seed(2026 + 1)
    a = torch.randn([M2, K2], generator=g, device=dev).to(torch.bfloat16)
    b = (torch.randn([N2, K2], generator=g, device=dev) * 0.02).to(torch.bfloat16)
    out = torch.empty([M2, N2], dtype=torch.bfloat16, device=dev)
    aq = torch.empty([M2, K2], dtype=torch.float8_e4m3fn, device=dev)
    bq = torch.empty([N2, K2], dtype=torch.float8_e4m3fn, device=dev)
    sfa = torch.empty([M2, K2 // 32], dtype=torch.uint8, device=dev)
    sfb = torch.empty([N2, K2 // 32], dtype=torch.uint8, device=dev)
    for _ in range(3):
        hq.group_wise_quant(a, MODE, True, True, aq, sfa)
        hq.group_wise_quant(b, MODE, True, True, bq, sfb)
        hq.dense_gemm(aq, bq, sfa, sfb, out, None, None, -1, MODE, True)
    torch.cuda.synchronize()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        ev[i][0].record()
        hq.group_wise_quant(a, MODE, True, True, aq, sfa)
        hq.group_wise_quant(b, MODE, True, True, bq, sfb)
        ev[i][1].record()
        hq.dense_gemm(aq, bq, sfa, sfb, out, None, None, -1, MODE, True)
        ev[i][2].record()
    stop.record()
    torch.cuda.synchronize()
    total_ms = start.elapsed_time(stop)
    quant_ms = sum(e[0].elapsed_time(e[1]) for e in ev) / steps
    gemm_ms = sum(e[1].elapsed_time(e[2]) for e in ev) / steps
    gemm_alone = timed_ms(lambda: hq.dense_gemm(aq, bq, sfa, sfb, out, None, None, -1, MODE, False), max(steps, 5))
    quant_alone = timed_ms(lambda: hq.group_wise_quant(a, MODE, True, False, aq, sfa), max(steps, 5))
    flops = 2.0 * M2 * N2 * K2
    gemm_tflops = flops / (gemm_ms * 1e-3) / 1e12
    fp8_peak = 2.0 * peaks["bf16"]
    qbytes = M2 * K2 * 3.03125
    pair = "pair=1" in hq.describe_tile(M2, N2, K2, MODE, device=dev.index)
    return {
        "workload": f"C2 MXFP8 dense GEMM M=N=K={M2}: group_wise_quant(A) + group_wise_quant(B) + dense_gemm per step",
        "value": flops / (total_ms / steps * 1e-3) / 1e12, "unit": "TFLOPS", "steps": steps,
        "ms_per_step": total_ms / steps, "tile": hq.describe_tile(M2, N2, K2, MODE, device=dev.index),
        "gemm_only": {"tflops_in_step": gemm_tflops, "ms_in_step": gemm_ms,
                      "tflops_alone": flops / (gemm_alone * 1e-3) / 1e12, "ms_alone": gemm_alone,
                      "frac_of_nominal_fp8": gemm_tflops / NOMINAL_FP8_TFLOPS},
        "quant": {"ms_both_in_step": quant_ms, "ms_one_operand_alone": quant_alone,
                  "gbs_alone": qbytes / (quant_alone * 1e-3) / 1e9,
                  "frac_of_hbm": qbytes / (quant_alone * 1e-3) / 1e9 / peaks["hbm_gbs"], "bytes_per_element": 3.03125},
        "roofline": {"kernel": "gemm_pair_kernel<256, mxfp8>" if pair else "gemm_kernel<256, mxfp8>",
                     "bound": "tensor", "achieved": gemm_tflops, "peak": fp8_peak, "unit": "TFLOP/s",
                     "frac": gemm_tflops / fp8_peak, "traffic": 478.3e6 if pair else 605.2e6,
                     "traffic_source": "ncu capture of one launch of this kernel on this shape",
                     "algorithmic_bytes": 64 * 2**20 * 2 + 4 * 2**20 + 128 * 2**20,
                     "peak_source": f"2 x {peaks['source']} cuBLAS bf16 (burst) as the dense fp8 peak"},
    }


def run_ours(args):
    import halops_b200 as hq
    from halops_b200.dist import ColumnParallelDenseGemm, shard_bounds

    rank, world, local = _dist_env()
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    if (N5 // WEIGHT_BLOCK) % world != 0:
        raise SystemExit(f"the weight is generated in {N5 // WEIGHT_BLOCK} blocks of rows: 1, 2, 4 or 8 GPUs")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    peaks = _peaks()
    start_row, rows = shard_bounds(N5, world, rank)
    blocks_per_rank = rows // WEIGHT_BLOCK
    g = torch.Generator(device=dev).manual_seed(2031)  # the same activation on every rank
    x = torch.randn([M5, K5], generator=g, device=dev).to(torch.bfloat16)
    w = make_weight_rows(rank * blocks_per_rank, blocks_per_rank, dev)
    layer = ColumnParallelDenseGemm(w, mode=MODE)  # quantises the shard once
    del w
    out = torch.empty([M5, rows], dtype=torch.bfloat16, device=dev)
    xq = torch.empty([M5, K5], dtype=torch.float8_e4m3fn, device=dev)
    sfa = torch.empty([M5, K5 // 32], dtype=torch.uint8, device=dev)

    def step():
        hq.group_wise_quant(x, MODE, True, True, xq, sfa)
        layer.local_quantized(xq, sfa, out)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    barrier()
    assert hq.device_status(dev) == 0

    # ---- timed region: K steps, device time by CUDA events on the launching stream
    sampler = ClockSampler(dev)
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
        hq.group_wise_quant(x, MODE, True, True, xq, sfa)
        ev[i][1].record()
        layer.local_quantized(xq, sfa, out)
        ev[i][2].record()
    stop.record()
    barrier()
    total_ms = start.elapsed_time(stop)
    quant_ms = sum(e[0].elapsed_time(e[1]) for e in ev) / steps
    gemm_ms = sum(e[1].elapsed_time(e[2]) for e in ev) / steps
    clocks = sampler.stop() if rank == 0 else None
    assert hq.device_status(dev) == 0

    if args.kernels_only:
        # profiling aid: only the timed steps above run (keeps a profiler's launch list short)
        if rank == 0:
            print(json.dumps({"kernels_only": True, "ms_per_step": total_ms / steps, "gemm_ms": gemm_ms,
                              "quant_ms": quant_ms}), flush=True)
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- correctness of the sharded run, in the record: a row sample of the rank's output
    # against a float32 dequantise-then-matmul on the device
    check_rel, check_rows = shard_check(xq, sfa, layer.wq, layer.sfb, out)
    bitwise = None
    if world > 1:
        # ... and bit for bit against the single-GPU GEMM on the whole weight
        wq_full, sfb_full = hq.group_wise_quant(make_weight_rows(0, N5 // WEIGHT_BLOCK, dev), mode=MODE)
        full = torch.empty([M5, N5], dtype=torch.bfloat16, device=dev)
        hq.dense_gemm(xq, wq_full, sfa, sfb_full, full, None, None, -1, MODE)
        sample = torch.linspace(0, M5 - 1, 64, device=dev).round().to(torch.int64)
        bitwise = bool(torch.equal(full[sample][:, start_row:start_row + rows], out[sample]))
        del wq_full, sfb_full, full

    # ---- sustained: the same step back to back for at least two seconds
    ms_guess = total_ms / steps
    sus_steps = max(steps, int(2000.0 / ms_guess) + 1)
    sus_sampler = ClockSampler(dev)
    if rank == 0:
        sus_sampler.start()
    barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(sus_steps):
        step()
    e.record()
    barrier()
    sus_ms = s.elapsed_time(e) / sus_steps
    sus_clocks = sus_sampler.stop() if rank == 0 else None

    # ---- all-gather of the bf16 output, overlapped with the GEMM block by block: pushed into the
    # peers' symmetric memory by the copy engines where there is peer access, else by NCCL
    gather_ms = gather_alone_ms = gather_nccl_ms = nccl_alone_ms = None
    gather_blocks = 8
    transport = gather_error = None
    other = {}
    if world > 1:
        def step_gather(kind="auto"):
            hq.group_wise_quant(x, MODE, True, True, xq, sfa)
            return layer.gathered(xq, sfa, blocks=gather_blocks, transport=kind)

        reps = max(3, min(steps, 10))
        try:
            # both transports are timed; the line's figure is the one `gathered` picks by itself
            staged = step_gather("copy")
            have_copy = bool(layer._symm and layer._symm[1] is not None)
            copy_ms = timed_ms(lambda: step_gather("copy"), reps, barrier)
            staged = step_gather("copy")
            mine = staged[:, rank].reshape(M5, rows)
            bitwise = bitwise and bool(torch.equal(mine, out))
            copy_alone_ms = timed_ms(lambda: layer.gathered(xq, sfa, blocks=gather_blocks, transport="copy",
                                                            compute=False), reps, barrier)
            staged = step_gather("nccl")
            bitwise = bitwise and bool(torch.equal(staged[:, rank].reshape(M5, rows), out))
            gather_nccl_ms = timed_ms(lambda: step_gather("nccl"), reps, barrier)
            nccl_alone_ms = timed_ms(lambda: layer.gathered(xq, sfa, blocks=gather_blocks, transport="nccl",
                                                            compute=False), reps, barrier)
            if have_copy and world <= 4:
                transport, gather_ms, gather_alone_ms = "copy engines into symmetric memory", copy_ms, copy_alone_ms
            else:
                transport, gather_ms, gather_alone_ms = "nccl all-gather per block", gather_nccl_ms, nccl_alone_ms
            other = {"copy_engines": {"ms_per_step": copy_ms, "transfer_alone_ms": copy_alone_ms}} if have_copy else {}
            assert hq.device_status(dev) == 0
        except Exception as ex:  # the line below still reports the step without the gather
            gather_error = repr(ex)[:300]
            gather_ms = gather_alone_ms = gather_nccl_ms = nccl_alone_ms = None

    # ---- the same with the all-gather inside the GEMM: its epilogue stores every tile into the
    # peers' outputs (symmetric memory) as well as into its own
    fused_ms = fused_error = None
    if world > 1 and gather_error is None:
        try:
            def step_fused():
                hq.group_wise_quant(x, MODE, True, True, xq, sfa)
                return layer.gathered_fused(xq, sfa)

            whole = step_fused()
            staged = step_gather("nccl")
            bitwise = bitwise and bool(torch.equal(whole, layer.gathered_as_matrix(staged)))
            fused_ms = timed_ms(step_fused, reps, barrier)
            assert hq.device_status(dev) == 0
            del whole, staged
        except Exception as ex:
            fused_error = repr(ex)[:300]
            fused_ms = None

    # ---- end to end through the public API with host buffers: every step copies its own
    # activation in from pinned memory and its own result out; consecutive steps overlap on
    # three streams (copy in / kernels / copy out) with two sets of device buffers
    x_host = x.cpu().pin_memory()
    out_host = torch.empty([M5, rows], dtype=torch.bfloat16).pin_memory()
    x_dev = [torch.empty_like(x) for _ in range(2)]
    out_dev = [torch.empty_like(out) for _ in range(2)]
    s_in, s_run, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]        # the activation of the step is on the device
    ev_in_free = [torch.cuda.Event() for _ in range(2)]   # the quantizer has read it
    ev_run = [torch.cuda.Event() for _ in range(2)]       # the GEMM has written out_dev
    ev_out = [torch.cuda.Event() for _ in range(2)]       # the result is in host memory

    def e2e_step(i):
        j = i & 1
        s_in.wait_event(ev_in_free[j])
        with torch.cuda.stream(s_in):
            x_dev[j].copy_(x_host, non_blocking=True)
            ev_in[j].record(s_in)
        s_run.wait_event(ev_in[j])
        s_run.wait_event(ev_out[j])
        with torch.cuda.stream(s_run):
            q, sf = hq.group_wise_quant(x_dev[j], MODE, True, True, xq, sfa)
            ev_in_free[j].record(s_run)
            layer.local_quantized(q, sf, out_dev[j])
            ev_run[j].record(s_run)
        s_out.wait_event(ev_run[j])
        with torch.cuda.stream(s_out):
            out_host.copy_(out_dev[j], non_blocking=True)
            ev_out[j].record(s_out)

    e2e_steps = max(4, min(steps, 8))
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
    torch.cuda.synchronize(dev)
    # the bytes that came back are the GEMM's (same operands as the device-resident steps above)
    assert torch.equal(out_host[::257], out[::257].cpu()), "end-to-end result differs from the device-resident one"
    del x_host, out_host, x_dev, out_dev

    # ---- max over ranks
    copy_pair = other.get("copy_engines", {})
    vals = [total_ms, gemm_ms, quant_ms, sus_ms, e2e_ms, gather_ms or 0.0, gather_alone_ms or 0.0, check_rel,
            gather_nccl_ms or 0.0, nccl_alone_ms or 0.0, copy_pair.get("ms_per_step", 0.0),
            copy_pair.get("transfer_alone_ms", 0.0), fused_ms or 0.0]
    times = torch.tensor(vals, device=dev, dtype=torch.float64)
    ok = torch.tensor([1 if (bitwise is None or bitwise) else 0], device=dev, dtype=torch.int32)
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    (total_ms, gemm_ms, quant_ms, sus_ms, e2e_ms, gather_ms, gather_alone_ms, check_rel, gather_nccl_ms,
     nccl_alone_ms, copy_ms_max, copy_alone_max, fused_ms_max) = times.tolist()

    flops = 2.0 * M5 * N5 * K5          # the whole job
    flops_rank = flops / world
    ms_per_step = total_ms / steps
    value = flops / (ms_per_step * 1e-3) / 1e12
    gemm_tflops_rank = flops_rank / (gemm_ms * 1e-3) / 1e12
    timed_seconds = total_ms * 1e-3
    fp8_peak = 2.0 * (peaks["bf16"] if timed_seconds < 1.0 else peaks["bf16_sustained"])
    tile = hq.describe_tile(M5, rows, K5, MODE, device=local)
    quant_bytes = M5 * K5 * 3.03125
    algorithmic = M5 * K5 + rows * K5 + (M5 + rows) * K5 // 32 + 2 * M5 * rows

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32 accumulate -> bf16",
            "data": "synthetic",
            "config": {
                "workload": WORKLOAD,
                "weight_rows_per_rank": rows,
                "cache": "operands larger than L2 (activation 256 MiB bf16 / 128 MiB e4m3, weight shard "
                         f"{rows * K5 >> 20} MiB e4m3, output {M5 * rows * 2 >> 20} MiB)",
                "tile": tile,
            },
            "gemm_only": {"tflops_in_step": world * gemm_tflops_rank, "ms_in_step": gemm_ms,
                          "tflops_per_gpu": gemm_tflops_rank,
                          "frac_of_nominal_fp8": gemm_tflops_rank / NOMINAL_FP8_TFLOPS},
            "quant": {"ms_in_step": quant_ms, "gbs": quant_bytes / (quant_ms * 1e-3) / 1e9,
                      "frac_of_hbm": quant_bytes / (quant_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                      "bytes_per_element": 3.03125,
                      "note": "the activation is replicated: every rank quantises all of it"},
            "shard_check": {"max_rel_err_vs_f32_dequant_matmul": check_rel, "rows_sampled": check_rows,
                            "tolerance": 1e-2, "ok": bool(check_rel <= 1e-2),
                            "bitwise_equal_to_single_gpu_gemm_on_whole_weight":
                                None if world == 1 else bool(ok.item())},
            "sustained": {"steps": sus_steps, "ms_per_step": sus_ms, "tflops": flops / (sus_ms * 1e-3) / 1e12,
                          "sm_mhz": sus_clocks.get("sm_mhz"), "power_w_max": sus_clocks.get("power_w_max"),
                          "reasons": sus_clocks.get("reasons"),
                          "frac_of_2x_sustained_bf16": flops_rank / (sus_ms * 1e-3) / 1e12 /
                                                       (2.0 * peaks["bf16_sustained"])},
            "roofline": {"kernel": ("gemm_pair_kernel<256, mxfp8> (256x256x128 2-CTA tile)" if "pair=1" in tile
                                    else "gemm_kernel<..., mxfp8> (single-CTA tile)"),
                         "bound": "tensor", "achieved": gemm_tflops_rank,
                         "peak": fp8_peak, "unit": "TFLOP/s", "frac": gemm_tflops_rank / fp8_peak,
                         "traffic": (None if TRAFFIC_PER_7168_COLUMNS is None
                                     else TRAFFIC_PER_7168_COLUMNS * rows / 7168),
                         "traffic_source": TRAFFIC_SOURCE,
                         "algorithmic_bytes": algorithmic,
                         "flops_per_launch": flops_rank,
                         "peak_source": f"2 x {peaks['source']} cuBLAS bf16 "
                                        f"({'burst' if timed_seconds < 1.0 else 'sustained'}) as the dense fp8 peak"},
            "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOPS",
                    "h2d_bytes_per_step": M5 * K5 * 2, "d2h_bytes_per_step": M5 * rows * 2,
                    "ms_per_step": e2e_ms,
                    "overlap": "consecutive steps pipelined over 3 streams (copy in, kernels, copy out), 2 buffer "
                               "sets; bytes are per rank"},
            "gpu_launches": 2 * steps,
            "clocks": clocks,
        }
        if world > 1 and gather_ms:
            gathered_bytes = M5 * (N5 - rows) * 2
            floor_ms = gathered_bytes / 770e9 * 1e3
            blockwise = {"ms_per_step": gather_ms, "transport": transport, "transfer_alone_ms": gather_alone_ms,
                         "ratio_to_max_of_compute_and_transfer_alone": gather_ms / max(gather_alone_ms, ms_per_step),
                         "blocks": gather_blocks,
                         "how": "GEMM of row block i+1 on the compute stream while block i travels on a second "
                                "stream; what `gathered(transport='auto')` picks"}
            # the line's figure is what `ColumnParallelDenseGemm(x, gather=True, overlap=True)` runs: the GEMM
            # that gathers in its epilogue where it applies, else the block-wise overlap
            best_ms = fused_ms_max if fused_ms_max else gather_ms
            line["with_allgather"] = {
                "tflops": flops / (best_ms * 1e-3) / 1e12, "ms_per_step": best_ms,
                "transport": ("one kernel: the GEMM's epilogue TMA-stores every tile into each peer's output "
                              "(symmetric memory over NVLink) as well as into its own" if fused_ms_max else transport),
                "compute_alone_ms": ms_per_step,
                "nvlink_floor_ms_at_770_gbs": floor_ms,
                "ratio_to_max_of_compute_and_nvlink_floor": best_ms / max(floor_ms, ms_per_step),
                "bytes_received_per_rank": gathered_bytes,
                "nvlink_gbs_in_step": gathered_bytes / (best_ms * 1e-3) / 1e9,
                "fused_epilogue": ({"ms_per_step": fused_ms_max} if fused_ms_max else {"error": fused_error}),
                "blockwise_overlap": blockwise,
                "nccl_transport": {"ms_per_step": gather_nccl_ms, "transfer_alone_ms": nccl_alone_ms,
                                   "sms_left_to_nccl": ColumnParallelDenseGemm.default_comm_sms(world)},
                "copy_engine_transport": ({"ms_per_step": copy_ms_max, "transfer_alone_ms": copy_alone_max}
                                          if copy_ms_max else None),
            }
        elif world > 1:
            line["with_allgather"] = {"error": gather_error}
        if world == 1:
            try:
                line["c2"] = bench_c2(hq, dev, steps, peaks)
            except Exception as ex:
                line["c2"] = {"error": repr(ex)[:300]}
            if not args.no_cpu_baseline:
                base = cpu_baseline(steps=2, warmup=1)
                line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
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
    + [(f"ref README {m}x{n}x{k}", "w8a8-mxfp8", m, n, k, "normal", 1.0)
       for (m, n, k) in ((8, 8192, 1024), (64, 8192, 1024), (512, 1536, 4096), (8, 32768, 1024),
                         (32, 8192, 4096), (128, 8192, 4096), (64, 4096, 8192), (128, 4096, 8192))]
)


class Timers:
    """The two timers of the sweep: CUDA events around one call (cold L2: a 256 MiB buffer
    is zeroed before every timed call; 10 warm-up, 30 timed, median) and, for short
    kernels, the kernel's own duration as the CUDA profiler records it, which is what the
    reference's benchmark reports (benchmark/core/timing.py:196-228 there): events add the
    launch gap, about 4 us, to every small shape.  Every measurement comes with the SM clock
    read through NVML while the timed calls run, after the same idle gap."""

    def __init__(self, dev):
        self.dev = dev
        self.flush = torch.empty([256 << 20], dtype=torch.uint8, device=dev)
        self.clock = SmClock(dev)

    def events(self, fn, warm=10, reps=30):
        time.sleep(0.3)  # every row starts from the same idle state
        for _ in range(warm):
            fn()
        ts, mhz = [], []
        for _ in range(reps):
            self.flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            c = self.clock.mhz()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e) * 1e3)
            if c is not None:
                mhz.append(c)
        ts.sort()
        mhz.sort()
        return ts[len(ts) // 2], (mhz[len(mhz) // 2] if mhz else None)

    def kernel(self, fn, reps=20):
        """Median device duration in us of this library's kernels inside one call, or None
        when the profiler is not available."""
        try:
            from torch.profiler import ProfilerActivity, profile

            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                for _ in range(reps):
                    self.flush.zero_()
                    fn()
                torch.cuda.synchronize()
            per_call = []
            durs = [ev.device_time for ev in prof.events()
                    if "hq::" in ev.name and getattr(ev, "device_time", 0) > 0]
            if not durs or len(durs) % reps != 0:
                return None
            n = len(durs) // reps
            for i in range(reps):
                per_call.append(sum(durs[i * n:(i + 1) * n]))
            per_call.sort()
            return per_call[len(per_call) // 2]
        except Exception:
            return None

    def row(self, fn, short_us=60.0):
        us, mhz = self.events(fn)
        out = {"us": round(us, 2), "sm_mhz": mhz, "kernel_cycles": round(us * mhz) if mhz else None}
        if us < short_us:
            kus = self.kernel(fn)
            out["kernel_us"] = None if kus is None else round(kus, 2)
        return out


def run_sweep(args):
    """GEMM-only and quantizer-only medians for every benchmark configuration and the
    reference's published shapes, measured the way the reference's benchmark does.
    One JSON object per line; not the driver's contract line."""
    import halops_b200 as hq

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = _peaks()
    tm = Timers(dev)
    only = args.only

    for label, mode, m, n, k, dist, bscale in SWEEP:
        if only and only not in label:
            continue
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
        gemm = tm.row(lambda: hq.dense_gemm(aq, bq, sfa, sfb, out, None, alpha, -1, mode, False))
        qa = tm.row(lambda: hq.group_wise_quant(a, mode=mode, use_pdl=False))
        qb = tm.row(lambda: hq.group_wise_quant(b, mode=mode, use_pdl=False))
        assert hq.device_status(dev) == 0
        fp8 = mode == "w8a8-mxfp8"
        group = 32 if fp8 else 16
        bpe = 1.0 if fp8 else 0.5
        gemm_bytes = bpe * (m * k + n * k) + ((m + 127) // 128 * 128 + n) * k / group + 2.0 * m * n
        q_bpe = 2 + bpe + 1.0 / group
        flops = 2.0 * m * n * k
        gemm_us = gemm["us"]
        best_us = gemm.get("kernel_us") or gemm_us
        print(json.dumps({
            "config": label, "mode": mode, "m": m, "n": n, "k": k,
            "tile": hq.describe_tile(m, n, k, mode).split("-> ")[1],
            "gemm": gemm, "gemm_tflops": round(flops / gemm_us / 1e6, 1),
            "gemm_gbs": round(gemm_bytes / best_us / 1e3, 1),
            "gemm_frac_of_hbm": round(gemm_bytes / best_us / 1e3 / peaks["hbm_gbs"], 3),
            "quant_a": qa, "quant_b": qb,
            "quant_b_gbs": round(n * k * q_bpe / qb["us"] / 1e3, 1),
            "quant_b_frac_of_hbm": round(n * k * q_bpe / qb["us"] / 1e3 / peaks["hbm_gbs"], 3),
            "quant_incl_tflops": round(flops / (gemm_us + qa["us"] + qb["us"]) / 1e6, 1),
        }), flush=True)
    if only and only != "next":
        return
    run_sweep_next_rows(tm, dev, peaks)


def run_sweep_next_rows(tm, dev, peaks):
    """Rows beyond the dense path: rms_norm_quant and the non-Identity epilogues."""
    import halops_b200 as hq

    for m, k in ((3072, 8192), (16384, 4096), (128, 4096)):
        g = torch.Generator(device=dev).manual_seed(9)
        x = (torch.randn([m, k], generator=g, device=dev) * 3).to(torch.bfloat16)
        w = (torch.rand([k], generator=g, device=dev) + 0.5).to(torch.bfloat16)
        r = tm.row(lambda: hq.rms_norm_quant(x, w, 1e-6, True, False))
        nbytes = m * k * 3.03125 + k * 2
        print(json.dumps({"config": "rms_norm_quant", "m": m, "k": k, **r,
                          "gbs": round(nbytes / r["us"] / 1e3, 1),
                          "frac_of_hbm": round(nbytes / r["us"] / 1e3 / peaks["hbm_gbs"], 3)}), flush=True)
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
        r = tm.row(fn)
        print(json.dumps({"config": f"epilogue {label}", "m": m, "n": n, "k": k, **r,
                          "tflops": round(flops / r["us"] / 1e6, 1)}), flush=True)
    assert hq.device_status(dev) == 0
    run_sweep_grouped(tm, dev)
    run_sweep_low_latency(tm, dev, peaks)
    run_sweep_decode_chain(dev, peaks)


def run_sweep_grouped(tm, dev):
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
                r = tm.row(fn)
                print(json.dumps({"config": label, "mode": mode, "experts": experts, "rows_per_expert": rows,
                                  "n": n, "k": k, **r,
                                  "tflops": round(2.0 * m * n * k * filled / r["us"] / 1e6, 1)}), flush=True)
            assert hq.device_status(dev) == 0


def run_sweep_low_latency(tm, dev, peaks):
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
        ll = tm.row(lambda: hq.low_latency_mma_gemm(xq, wq, sfa, sfb, out, use_pdl=False))
        dense = tm.row(lambda: hq.dense_gemm(xq, wq, sfa_sw, sfb_sw, out, None, None, -1, MODE, False))
        nbytes = n * k * (1 + 1 / 32)
        best = ll.get("kernel_us") or ll["us"]
        print(json.dumps({"config": "low_latency_mma_gemm", "m": m, "n": n, "k": k, **ll,
                          "weight_gbs": round(nbytes / best / 1e3, 1),
                          "frac_of_hbm": round(nbytes / best / 1e3 / peaks["hbm_gbs"], 3),
                          "dense_gemm": dense}), flush=True)
    assert hq.device_status(dev) == 0


def _graph_time_us(chain):
    """Median time of one replay of `chain` captured into a CUDA graph (programmatic launches become
    programmatic edges).  One call from Python costs the host about 10 us, more than a decode kernel runs."""
    for _ in range(3):
        chain()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        chain()
    graph.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(20):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        graph.replay()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e) * 1e3)
    ts.sort()
    return ts[len(ts) // 2]


def run_sweep_decode_chain(dev, peaks):
    """Decode GEMMs back to back in a CUDA graph, every one on its own weight (the set is larger than L2),
    alone and with the activation's quantizer before every GEMM: time per GEMM with plain launches, with
    programmatic launches, and with programmatic launches that may read the weight early (use_pdl = 0, 1, 2)."""
    import halops_b200 as hq

    for m, n, k, layers in ((8, 7168, 2048, 16), (8, 24576, 1536, 8), (64, 7168, 2048, 16)):
        g = torch.Generator(device=dev).manual_seed(31)
        x = torch.randn([m, k], generator=g, device=dev).to(torch.bfloat16)
        xq, sfa = hq.group_wise_quant(x)
        ws = [hq.group_wise_quant((torch.randn([n, k], generator=g, device=dev) * 0.05).to(torch.bfloat16))
              for _ in range(layers)]
        outs = [torch.empty([m, n], dtype=torch.bfloat16, device=dev) for _ in range(layers)]
        xqs = [torch.empty_like(xq) for _ in range(layers)]
        sfas = [torch.empty_like(sfa) for _ in range(layers)]
        for with_quant in (False, True):
            row = {"config": "decode chain" + (", quantizer before every GEMM" if with_quant else ""),
                   "m": m, "n": n, "k": k, "gemms": layers,
                   "weights_mb": round(layers * n * k * (1 + 1 / 32) / 1e6, 1)}
            for use_pdl in (0, 1, 2):
                def chain():
                    for i in range(layers):
                        if with_quant:
                            hq.group_wise_quant(x, MODE, True, use_pdl != 0, xqs[i], sfas[i])
                            hq.dense_gemm(xqs[i], ws[i][0], sfas[i], ws[i][1], outs[i], None, None, -1, MODE, use_pdl)
                        else:
                            hq.dense_gemm(xq, ws[i][0], sfa, ws[i][1], outs[i], None, None, -1, MODE, use_pdl)

                us = _graph_time_us(chain) / layers
                row[f"us_per_gemm_pdl{use_pdl}"] = round(us, 2)
                row[f"frac_of_hbm_pdl{use_pdl}"] = round(n * k * (1 + 1 / 32) / us / 1e3 / peaks["hbm_gbs"], 3)
            assert hq.device_status(dev) == 0
            print(json.dumps(row), flush=True)


def run_shape(args):
    """One dense GEMM shape, GEMM only: MODE,M,N,K (or rms,M,0,K: rms_norm_quant alone).  Prints one JSON
    line (cold-L2 median);
    with --kernels-only just 3 warm-up and 3 measured launches, for profiler captures."""
    import halops_b200 as hq

    mode, m, n, k = args.shape.split(",")
    m, n, k = int(m), int(n), int(k)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(2026)
    if mode == "rms":  # rms,M,0,K: rms_norm_quant of an [M, K] activation
        x = (torch.randn([m, k], generator=g, device=dev) * 3).to(torch.bfloat16)
        w = (torch.rand([k], generator=g, device=dev) + 0.5).to(torch.bfloat16)
        fn = lambda: hq.rms_norm_quant(x, w, 1e-6, True, False)  # noqa: E731
        if args.kernels_only:
            flush = torch.empty([256 << 20], dtype=torch.uint8, device=dev)
            for _ in range(6):
                flush.zero_()
                fn()
            torch.cuda.synchronize()
            print(json.dumps({"shape": args.shape, "kernels_only": True}), flush=True)
            return
        r = Timers(dev).row(fn)
        print(json.dumps({"shape": args.shape, "rms_norm_quant": r,
                          "gbs": round((m * k * 3.03125 + k * 2) / r["us"] / 1e3, 1)}), flush=True)
        return
    a = torch.randn([m, k], generator=g, device=dev).to(torch.bfloat16)
    b = (torch.randn([n, k], generator=g, device=dev) * 0.02).to(torch.bfloat16)
    aq, sfa = hq.group_wise_quant(a, mode=mode)
    bq, sfb = hq.group_wise_quant(b, mode=mode)
    out = torch.empty([m, n], dtype=torch.bfloat16, device=dev)
    alpha = torch.ones([1], dtype=torch.float32, device=dev) if mode == "w4a4-nvfp4" else None
    fn = lambda: hq.dense_gemm(aq, bq, sfa, sfb, out, None, alpha, -1, mode, False)  # noqa: E731
    if args.kernels_only:
        flush = torch.empty([256 << 20], dtype=torch.uint8, device=dev)
        for _ in range(6):
            flush.zero_()
            fn()
        torch.cuda.synchronize()
        assert hq.device_status(dev) == 0
        print(json.dumps({"shape": args.shape, "kernels_only": True}), flush=True)
        return
    r = Timers(dev).row(fn)
    assert hq.device_status(dev) == 0
    print(json.dumps({"shape": args.shape, "tile": hq.describe_tile(m, n, k, mode).split("-> ")[1], "gemm": r,
                      "gemm_tflops": round(2.0 * m * n * k / r["us"] / 1e6, 1)}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kernels-only", action="store_true",
                    help="run only warm-up and the timed steps (for profiler captures)")
    ap.add_argument("--sweep", action="store_true",
                    help="time every benchmark configuration (GEMM only / quantizer only, cold L2) instead")
    ap.add_argument("--only", default=None, help="with --sweep: only the dense rows whose label contains this; 'next' = only the rows "
                         "beyond the dense path (rms_norm_quant, epilogues, grouped, low latency)")
    ap.add_argument("--shape", default=None, metavar="MODE,M,N,K",
                    help="time one dense GEMM shape (GEMM only, cold L2) instead, e.g. w8a8-mxfp8,16,24576,1536")
    args = ap.parse_args()
    if args.shape:
        run_shape(args)
    elif args.sweep:
        run_sweep(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
