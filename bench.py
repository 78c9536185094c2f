#!/usr/bin/env python
"""Benchmark of the activation-compression hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--sweep]

One "step" is one pass of the fused RMSNorm + compress kernel over one batch of
synthetic activations (configuration 5 of the baseline: bf16 [65536, 4096],
Student-t values, 1 % outlier channels x50, INT4, one dynamic absmax scale per
token).  The metric is algorithmic HBM GB/s: bytes the operation must move
(read x, write y, codes, outlier values, scales, rstd) per second, summed over
all ranks.  With N > 1 every rank owns its own rows (weak scaling; the path
has no data-path collective).

The JSON line also carries
  roofline      achieved / measured HBM peak for that kernel (CUDA-event time)
  e2e           the same metric through the C ABI with HOST buffers: pinned
                host -> device copy of the rows, kernel, device -> host copy of
                everything the kernel produced, all inside the timed region
  cpu_baseline  the reference's own CPU chain for a norm site -- the RMSNorm formula of its
                model file, then its unmodified true_divide_outlier_suboutlier_svd_compress
                (per-channel INT4 static scale, element outliers) -- on the same tensor, on
                this box's host cores (kind "reference" when the staged copy of the reference
                is present, else the CPU oracle's bit-exact restatement, kind "port")
  r_mode        this library's kernel doing that same reference arithmetic on the GPU
  kernels       per-kernel GB/s of the backward-side kernels (CUDA-graph replay)
  clocks        SM clocks / throttle reasons sampled during the timed region
``--impl reference`` times the CPU chain alone, as its own arm.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS, COLS, BITS, FRACTION, GROUP, ROTATE = 65536, 4096, 4, 0.01, 0, 0
# rows per piece of the end-to-end pipeline (measured: 8192 -> 81 GB/s, 4096 -> 81, 2048 -> 77, 1024 -> 70: the copies back to the host bound it)
E2E_PIECE_ROWS = int(os.environ.get("HYC_E2E_PIECE_ROWS", "8192"))
FALLBACK_HBM_GBS = 6650.0


def algorithmic_bytes_per_row(cols: int, bits: int, k: int, groups: int, norm: bool = True, ln: bool = False) -> int:
    """Bytes one row must move: read x (bf16) [+ write y] + codes + bf16 outlier values + fp32 scales
    [+ rstd (+ mean)]."""
    b = 2 * cols + cols * bits // 8 + 2 * k + 4 * groups
    if norm:
        b += 2 * cols + 4 + (4 if ln else 0)
    return b


def workload_name() -> str:
    return (f"config5: fused RMSNorm+compress, bf16 [{ROWS},{COLS}] per GPU, INT{BITS}, "
            f"{FRACTION:.0%} outlier channels, per-token absmax scale, rotation off")


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def measured_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return {}


def committed_traffic():
    """DRAM bytes per launch of the benchmarked kernel from the committed ncu summary, if any."""
    path = os.path.join(ROOT, "profiles", "norm_compress_traffic.json")
    if os.path.exists(path):
        try:
            return json.load(open(path)).get("dram_bytes_per_launch")
        except Exception:
            return None
    return None


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 100 ms while active."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in self.rows:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            inside = t0 - 0.05 <= ts <= t1 + 0.15
            try:
                if inside:
                    sm.append(float(parts[0]))
                    mx.append(float(parts[1]))
            except ValueError:
                continue
            if inside:
                for n, v in zip(names, parts[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------ CPU arm

CPU_PIECE_ROWS = 16384        # rows handed to the reference chain per call (bounds its temporaries)
SEQ = 512                     # the [T, D] rows are seen as [T / 512, 512, D], as a training batch would be


def rank_rows(rank: int):
    """The seeded rows of one rank, bf16 [ROWS, COLS] (generated in 8192-row pieces), and the planted channels."""
    import torch
    from hyc_lora_b200 import synthetic
    pieces = [synthetic.sweep_activation(8192, COLS, FRACTION, salt=1000 * rank + i)[0] for i in range(ROWS // 8192)]
    planted = synthetic.sweep_activation(8192, COLS, FRACTION, salt=1000 * rank)[1].to(torch.int32)
    return torch.cat(pieces), planted


def cpu_chain():
    """The reference's CPU work at one norm site in steady state, as ``(calibrate, step, kind, what)``.

    ``step(x3, w, stats)`` runs the RMSNorm formula of the reference's model file
    (models/modeling_llama.py:136-141) and then the compression of the norm input exactly as
    EfficientMemoryRMSNormFunc.forward does after its norm kernel (operators/efficient_rmsnorm.py:193-201):
    per-channel INT4 static scale, element outliers above the calibrated threshold, rank 0.  With the staged
    copy of the reference present the compression is its own, unmodified
    true_divide_outlier_suboutlier_svd_compress (operators/compress_function.py:136-200); otherwise the CPU
    oracle's restatement of it, which is pinned bit for bit to that function."""
    import torch
    from oracle import ref_loader
    ref = ref_loader.load()

    def rmsnorm(x3, w):
        v = x3.to(torch.float32).pow(2).mean(-1, keepdim=True)
        return w * (x3.to(torch.float32) * torch.rsqrt(v + 1e-5)).to(x3.dtype)

    if ref is not None:
        cf = ref.compress_function

        def calibrate(x3):
            return cf.get_statistics(x3[:1], 0, FRACTION, 1.0, BITS, "per-channel", 0)

        def step(x3, w, stats):
            thr, L, R, scale = stats
            y = rmsnorm(x3, w)
            return y, cf.true_divide_outlier_suboutlier_svd_compress(x3, thr, scale, BITS, 1.0, L, R)

        return calibrate, step, "reference", ("the reference's own operators/compress_function.py, imported unmodified, "
                                              "after the RMSNorm formula of its model file")
    from oracle import hyc_oracle as oc

    def calibrate(x3):
        return oc.r_calibrate(x3[:1], FRACTION, 1.0, BITS, "per-channel", 0)

    def step(x3, w, stats):
        thr, L, R, scale = stats
        y = rmsnorm(x3, w)
        return y, oc.r_compress(x3, thr, scale, BITS, 1.0)

    return calibrate, step, "port", ("CPU restatement of the reference's compress chain (bit-exact against it), "
                                     "after the RMSNorm formula of its model file; the reference tree is not on this box")


def cpu_arm(x, rows_per_step: int, repeats: int, budget_s: float = 150.0):
    """Time ``repeats`` steps of the CPU chain over the first ``rows_per_step`` rows of ``x`` (bf16 [T, D]) with all
    host threads.  If the first step says the run would not fit ``budget_s`` the rows per step are cut (in whole
    pieces) and the figure says so.  Returns (bytes per step, per-step seconds, cores, kind, description, rows)."""
    import torch
    from hyc_lora_b200 import synthetic
    from hyc_lora_b200.operators.compress_function import outlier_channel_count
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    calibrate, step, kind, what = cpu_chain()
    w = synthetic.norm_weight(COLS)
    k = outlier_channel_count(COLS, FRACTION)
    groups = 1 if GROUP == 0 else COLS // GROUP
    from oracle import ref_loader
    with ref_loader.cpu_cuda_noop():
        stats = calibrate(x[:CPU_PIECE_ROWS].reshape(-1, SEQ, COLS))

        def one(rows):
            for r0 in range(0, rows, CPU_PIECE_ROWS):
                step(x[r0:min(rows, r0 + CPU_PIECE_ROWS)].reshape(-1, SEQ, COLS), w, stats)

        t = time.perf_counter()
        one(min(rows_per_step, CPU_PIECE_ROWS))                       # warm-up on one piece, also the speed probe
        probe = (time.perf_counter() - t) / min(rows_per_step, CPU_PIECE_ROWS)
        fit = int(budget_s / max(repeats, 1) / probe) // CPU_PIECE_ROWS * CPU_PIECE_ROWS
        rows = max(CPU_PIECE_ROWS, min(rows_per_step, fit)) if rows_per_step > CPU_PIECE_ROWS else rows_per_step
        times = []
        for _ in range(repeats):
            t = time.perf_counter()
            one(rows)
            times.append(time.perf_counter() - t)
    # the same nominal bytes per row as the GPU arm, so that the ratio of the two figures is a ratio of times
    nbytes = algorithmic_bytes_per_row(COLS, BITS, k, groups) * rows
    return nbytes, times, cores, kind, what, rows


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    x, _ = rank_rows(0)
    nbytes, times, cores, kind, what, rows = cpu_arm(x, ROWS, args.warmup + args.steps)
    times = times[args.warmup:]
    total = sum(times)
    value = nbytes * len(times) / total / 1e9
    sample = f"{rows} of {ROWS} rows per step x {len(times)} steps" + ("" if rows == ROWS else " (cut to fit the time budget)")
    line = {
        "impl": "reference", "metric": "fused norm+compress HBM GB/s", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload_name(), "rows_per_step": rows, "cols": COLS, "bits": BITS,
                   "cpu_arithmetic": "the reference's own: element outliers above a calibrated threshold, static "
                                     "per-channel INT4 scale (the GPU arm's default line is the channel-outlier mode; its "
                                     "r_mode record is this arithmetic on the GPU)",
                   "bytes_per_row": nbytes // rows},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": kind, "sample": sample + "; " + what},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ GPU arm

def graph_timed(fn, nbytes, name, peak, reps=16, replays=3):
    """fn(i): one call on input set i.  The calls are recorded in a CUDA graph (so that host overhead of the
    Python wrappers does not hide short kernels) and cycle through input sets whose total size exceeds L2."""
    import torch
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(side):
        fn(0)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for i in range(reps):
                fn(i)
    torch.cuda.synchronize()
    graph.replay()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(replays):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / (replays * reps)
    return {"kernel": name, "ms": round(ms, 4), "bytes": int(nbytes), "GBps": round(nbytes / ms / 1e6, 1),
            "frac": round(nbytes / ms / 1e6 / peak, 3)}


def kernel_list(packed, x, w, channels, k, peak):
    """Metric 1 beyond the headline kernel: the backward-side kernels (decompress, decompress + SiLU backward,
    decompress + norm backward) and the forward at the smaller size, with and without the 256-wide rotation,
    INT4, per-token scale, 1 % outlier channels; CUDA-graph replay over input sets larger than L2."""
    import torch
    d = x.shape[1]
    out = []
    norm = dict(kind="rms", weight=w, bias=None, eps=1e-5)
    base = d * BITS // 8 + 2 * k + 4
    for rows in (65536, 16384):
        sets = [x[i * rows:(i + 1) * rows] for i in range(x.shape[0] // rows)]
        n = len(sets)
        dys = [torch.randn(rows, d, device=x.device, dtype=torch.bfloat16) for _ in range(max(1, min(n, 4)))]
        rstd = torch.ones(rows, device=x.device)
        for rotate in (0, 256):
            tag = f"T={rows} b={BITS} rot={rotate}"
            if rows != ROWS or rotate:
                out.append(graph_timed(lambda i: packed.compress_n(sets[i % n], channels, BITS, 0, rotate, norm=norm),
                                       algorithmic_bytes_per_row(d, BITS, k, 1) * rows, "norm+compress " + tag, peak))
            # the norm site with the record of its output from the same pass (what a norm in front of LoRA-A linears
            # runs).  With a rotation the library builds the pair for at most 8192 rows (beyond that two launches are
            # quicker): that line is taken on the first 4096 rows of each 16384-row set
            fmt = dict(channels=channels, bits=BITS, group=0, rotate=rotate)
            if rotate == 0 and rows == ROWS:
                out.append(graph_timed(lambda i: packed.compress_n(sets[i % n], channels, BITS, 0, rotate, norm=norm, also_output=fmt),
                                       (algorithmic_bytes_per_row(d, BITS, k, 1) + base) * rows, "norm+compress, two records " + tag, peak))
            if rotate and rows == 16384:
                small = [s_[:4096] for s_ in sets]
                out.append(graph_timed(lambda i: packed.compress_n(small[i % n], channels, BITS, 0, rotate, norm=norm, also_output=fmt),
                                       (algorithmic_bytes_per_row(d, BITS, k, 1) + base) * 4096,
                                       f"norm+compress, two records T=4096 b={BITS} rot={rotate}", peak))
            ps = [packed.compress_n(s_, channels, BITS, 0, rotate) for s_ in sets]
            out.append(graph_timed(lambda i: packed.decompress(ps[i % n]), (base + 2 * d) * rows, "decompress " + tag, peak))
            out.append(graph_timed(lambda i: packed.act_bwd("silu", ps[i % n], dys[i % len(dys)]), (base + 4 * d) * rows,
                                   "silu_bwd " + tag, peak))
            out.append(graph_timed(lambda i: packed.norm_bwd(ps[i % n], dys[i % len(dys)], w, rstd, None, "rms"),
                                   (base + 4 + 4 * d) * rows, "norm_bwd " + tag, peak))
            del ps
        del dys
    # the sites of the gated MLP at its width (11008 channels, rotation block 64 as the operators pick it there):
    # activation with both records, product with the record of its second operand and of its result
    import torch.nn.functional as F
    from hyc_lora_b200 import synthetic
    from hyc_lora_b200.operators.compress_function import outlier_channel_count
    dw, rw = 11008, 8192
    gates = [(0.25 * synthetic.sweep_activation(rw, dw, FRACTION, salt=50 + i)[0]).to(x.device) for i in range(2)]
    ups = [synthetic.sweep_activation(rw, dw, FRACTION, salt=60 + i)[0].to(x.device) for i in range(2)]
    kw = outlier_channel_count(dw, FRACTION)
    chw = packed.select_channels(packed.channel_absmax(ups[0]), kw)
    basew = dw * BITS // 8 + 2 * kw + 4
    fmt = dict(channels=chw, bits=BITS, group=0, rotate=64)
    tagw = f"T={rw} D={dw} b={BITS} rot=64"
    out.append(graph_timed(lambda i: packed.compress_n(gates[i % 2], chw, BITS, 0, 64), (2 * dw + basew) * rw, "compress " + tagw, peak))
    out.append(graph_timed(lambda i: packed.act_compress_n("silu", gates[i % 2], chw, BITS, 0, 64, also_output=fmt),
                           (4 * dw + 2 * basew) * rw, "silu + two records, one pass " + tagw, peak))

    def silu_separate(i):
        y = F.silu(gates[i % 2])
        packed.compress_n(gates[i % 2], chw, BITS, 0, 64)
        packed.compress_n(y, chw, BITS, 0, 64)
    rec = graph_timed(silu_separate, (4 * dw + 2 * basew) * rw, "silu + two records, three passes " + tagw, peak)
    rec["note"] = "same algorithmic bytes; the passes move 8 D + 2 records"
    out.append(rec)
    out.append(graph_timed(lambda i: packed.product_compress_n(gates[i % 2], ups[i % 2], chw, BITS, 0, 64, also_output=fmt),
                           (6 * dw + 2 * basew) * rw, "product + two records, one pass " + tagw, peak))

    def product_separate(i):
        y = gates[i % 2] * ups[i % 2]
        packed.compress_n(ups[i % 2], chw, BITS, 0, 64)
        packed.compress_n(y, chw, BITS, 0, 64)
    rec = graph_timed(product_separate, (6 * dw + 2 * basew) * rw, "product + two records, three passes " + tagw, peak)
    rec["note"] = "same algorithmic bytes; the passes move 10 D + 2 records"
    out.append(rec)
    del gates, ups
    # the one dense contraction of the path: LoRA-A weight gradient from the packed codes (tensor roofline)
    p = packed.compress_n(x, channels, BITS, 0, 0)
    g = torch.randn(x.shape[0], 64, device=x.device, dtype=torch.bfloat16)
    rec = graph_timed(lambda i: packed.lora_wgrad(p, g), x.shape[0] * (d * BITS // 8 + 2 * 64 + 4 + 2 * k) + 4 * 64 * d,
                      f"lora_wgrad tcgen05 T={x.shape[0]} b={BITS} r=64", peak)
    tensor_peak = measured_peaks().get("bf16_tflops", 1590.0)

    def as_tensor(rec, what):
        rec["TFLOPs"] = round(2.0 * x.shape[0] * 64 * d / (rec["ms"] * 1e-3) / 1e12, 1)
        rec["bound"] = "tensor"
        rec["hbm_frac"] = rec.pop("frac")
        rec["frac"] = round(rec["TFLOPs"] / tensor_peak, 3)       # of the measured bf16 GEMM burst peak
        rec["note"] = what
        return rec

    out.append(as_tensor(rec, "channel-mode record with outlier-channel tiles in the same launch; bound by shared-memory "
                              "bandwidth (every A element is written to and read from shared memory once), not by the tensor pipe"))
    # the same contraction from a reference-mode record (static per-channel scale, element outliers as a sparse side term)
    from hyc_lora_b200.operators import compress_function as cf
    x3 = x.reshape(-1, SEQ, d)
    thr, _, _, scale = cf.get_statistics(x3[:1], 0, FRACTION, 1.0, BITS, "per-channel", 0)
    pr = packed.compress_r(x3, thr, scale, BITS, outlier_ratio=FRACTION)
    rec = graph_timed(lambda i: packed.lora_wgrad(pr, g, path="tensor"),
                      x.shape[0] * (d * BITS // 8 + 2 * 64 + 8) + 4 * int(pr.pool_used.item()) + 4 * 64 * d,
                      f"lora_wgrad tcgen05 reference-mode record T={x.shape[0]} b={BITS} r=64", peak)
    out.append(as_tensor(rec, "warp-specialised kernel (2-D tensor copies, mbarrier hand-offs) + sparse outlier side kernel "
                              f"({int(pr.pool_used.item())} stored outliers, shared-memory atomics: that kernel is the cost) + finish; "
                              "NOT what the operators use for such records"))
    rec = graph_timed(lambda i: packed.lora_wgrad(pr, g, path="library"), 1,
                      f"lora_wgrad decompress + library GEMM, reference-mode record T={x.shape[0]} b={BITS} r=64", peak)
    out.append(as_tensor(rec, "the route the operators take for reference-mode records (bf16 reconstruction written and re-read)"))
    return out


def r_mode_record(packed, x, w, peak, steps):
    """The reference's own arithmetic on the GPU, on the same tensor: hyc_norm_compress in reference mode with a
    static per-channel INT4 scale and element outliers above the calibrated threshold (statistics as the reference
    calibrates them, from batch element 0 of the [T/512, 512, D] view; not timed)."""
    import torch
    from hyc_lora_b200.operators import compress_function as cf
    x3 = x.reshape(-1, SEQ, COLS)
    thr, _, _, scale = cf.get_statistics(x3[:1], 0, FRACTION, 1.0, BITS, "per-channel", 0)
    norm = dict(kind="rms", weight=w, bias=None, eps=1e-5)
    for _ in range(3):
        p, y, rstd, _ = packed.compress_r(x3, thr, scale, BITS, outlier_ratio=FRACTION, norm=norm)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        p, y, rstd, _ = packed.compress_r(x3, thr, scale, BITS, outlier_ratio=FRACTION, norm=norm)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / steps
    stored = int(p.pool_used.item())
    # read x, write y, codes, 4 B per stored outlier, 8 B row record, rstd
    nbytes = (4 * COLS + COLS * BITS // 8 + 8 + 4) * ROWS + 4 * stored
    return {"kernel": "hyc::fwd_r_warp_kernel (fused RMSNorm + reference-mode compress, one warp per row)", "ms": round(ms, 4),
            "bytes": nbytes, "GBps": round(nbytes / ms / 1e6, 1), "frac": round(nbytes / ms / 1e6 / peak, 3),
            "stored_outliers": stored, "status": int(p.status.item()),
            "scale": "static per-channel INT4 (calibrated)", "outliers": "elements above the calibrated threshold"}


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from hyc_lora_b200 import _lib, packed, synthetic
    from hyc_lora_b200.operators.compress_function import outlier_channel_count

    k = outlier_channel_count(COLS, FRACTION)
    groups = 1 if GROUP == 0 else COLS // GROUP
    # seeded rows of this rank (different salt per rank)
    x_cpu, _planted = rank_rows(rank)
    x_host = x_cpu.pin_memory()
    x = x_host.to(dev, non_blocking=True)
    w = synthetic.norm_weight(COLS).to(dev)
    # calibration (not timed): column absmax + top-k on the GPU
    channels = packed.select_channels(packed.channel_absmax(x), k)
    norm = dict(kind="rms", weight=w, bias=None, eps=1e-5)
    bytes_per_step = algorithmic_bytes_per_row(COLS, BITS, k, groups) * ROWS

    def step():
        return packed.compress_n(x, channels, BITS, GROUP, ROTATE, norm=norm)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warm = max(args.warmup, 3)               # at least three untimed launches (clocks, caches)
    for _ in range(warm):
        out = step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    launches0 = int(_lib.lib.hyc_launch_count())
    start.record()
    for _ in range(args.steps):
        out = step()
    stop.record()
    launches = int(_lib.lib.hyc_launch_count()) - launches0     # counted by the library, one per kernel it launched
    barrier()
    t1 = time.time()
    ms = start.elapsed_time(stop)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    # keep the GPU busy a little longer so that the clock samples are under load
    if rank == 0:
        t_end = time.time() + 0.6
        while time.time() < t_end:
            step()
        torch.cuda.synchronize()
        clocks = sampler.stop(t0, time.time())
    p, y, rstd, _ = out

    # ---- end to end through the C ABI with host buffers ----
    y_host = torch.empty_like(x_host).pin_memory()
    codes_host = torch.empty(p.codes.shape, dtype=p.codes.dtype).pin_memory()
    oval_host = torch.empty(p.out_value.shape, dtype=p.out_value.dtype).pin_memory()
    scales_host = torch.empty(p.scales.shape, dtype=p.scales.dtype).pin_memory()
    rstd_host = torch.empty(rstd.shape, dtype=rstd.dtype).pin_memory()
    h2d = x_host.numel() * 2
    d2h = y_host.numel() * 2 + codes_host.numel() + oval_host.numel() * 2 + scales_host.numel() * 4 + rstd_host.numel() * 4
    xin = torch.empty_like(x)
    # The rows go through in pieces so that the copy of piece i+1 to the device, the kernel on piece i
    # and the copy of piece i-1 back to the host overlap (PCIe is full duplex): three streams, events.
    piece = E2E_PIECE_ROWS
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    pieces = [(r0, min(ROWS, r0 + piece)) for r0 in range(0, ROWS, piece)]

    def e2e_step():
        cur = torch.cuda.current_stream()
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        keep = []
        for r0, r1 in pieces:
            with torch.cuda.stream(s_in):
                xin[r0:r1].copy_(x_host[r0:r1], non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            cur.wait_event(ev_in)
            pp, yy, rr, _ = packed.compress_n(xin[r0:r1], channels, BITS, GROUP, ROTATE, norm=norm)
            ev_k = torch.cuda.Event()
            ev_k.record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_k)
                y_host[r0:r1].copy_(yy, non_blocking=True)
                codes_host[r0:r1].copy_(pp.codes, non_blocking=True)
                oval_host[r0:r1].copy_(pp.out_value, non_blocking=True)
                scales_host[r0:r1].copy_(pp.scales, non_blocking=True)
                rstd_host[r0:r1].copy_(rr, non_blocking=True)
            keep.append((pp, yy, rr))
        cur.wait_stream(s_out)          # the step ends when its last result is on the host
        return keep

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    barrier()
    start.record()
    for _ in range(e2e_steps):
        e2e_step()
    stop.record()
    barrier()
    e2e_ms = start.elapsed_time(stop)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())

    if rank == 0:
        peak, which = hbm_peak()
        per_launch_s = ms / 1e3 / args.steps
        achieved = bytes_per_step / per_launch_s / 1e9
        value = achieved * world
        line = {
            "metric": "fused norm+compress HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": workload_name(), "rows_per_gpu": ROWS, "cols": COLS, "bits": BITS,
                       "outlier_channels": k, "scale": "per-token absmax", "l2": "inputs (537 MB per step) exceed the 126 MB L2",
                       "algorithmic_bytes_per_row": bytes_per_step // ROWS,
                       "mode": "channel-outlier mode (the north star's arithmetic; the reference has no counterpart, so "
                               "the CPU arm runs the reference's own element-outlier arithmetic on the same tensor and "
                               "`r_mode` is this library doing that arithmetic on the GPU)"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": committed_traffic(), "peak_source": f"of {which}",
                         "traffic_note": "lower bound (>=): ncu capture of 16384 rows scaled x4 (traffic is proportional to "
                                         "rows); the tail of y still in L2 when the kernel ends is not counted as a DRAM write",
                         "kernel": "hyc::fwd_n_warp_kernel<4 bits, RMSNorm, 16 register groups per lane, per-token scale>"},
            "e2e": {"value": (bytes_per_step * e2e_steps * world) / (e2e_ms / 1e3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "pipeline": f"{len(pieces)} pieces of {piece} rows; H2D, kernel and D2H on three streams"},
            "gpu_launches": launches,
            "clocks": clocks,
        }
    del xin, out, y, rstd, y_host, codes_host, oval_host, scales_host, rstd_host
    if rank == 0 and world == 1:
        # single-GPU runs only: the other kernels of metric 1, the reference's arithmetic on the GPU, and the
        # reference's CPU chain on the same tensor (the host cores are not shared with other ranks)
        try:
            line["r_mode"] = r_mode_record(packed, x, w, peak, max(5, min(args.steps, 20)))
            line["kernels"] = kernel_list(packed, x, w, channels, k, peak)
        except Exception as e:  # the headline must still be printed
            line["kernels_error"] = f"{type(e).__name__}: {e}"[:300]
        nbytes, times, cores, kind, what, rows = cpu_arm(x_cpu, ROWS, 5, budget_s=40.0)
        line["cpu_baseline"] = {"value": nbytes / statistics.median(times) / 1e9, "unit": "GB/s", "cores": cores,
                                "kind": kind, "sample": f"{rows} of {ROWS} rows, median of 5 runs; {what}"}
    if rank == 0 and args.sweep:
        line["sweep"] = sweep(packed, synthetic, x, w, peak)
    # free the operator benchmark's buffers before the model is built
    del x, p, x_host, x_cpu
    torch.cuda.empty_cache()
    step = None
    if not args.no_step:
        try:
            step = train_step_bench(args, world, rank, dev, barrier)
        except Exception as e:  # the operator line must still be printed
            step = {"metric": "7B HyC-LoRA train tokens/s", "error": f"{type(e).__name__}: {e}"[:300]}
    if rank == 0:
        if step is not None:
            line["train_step"] = step
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def train_step_bench(args, world, rank, dev, barrier):
    """Configuration 3: LLaMA-2-7B-shaped LoRA step (32 layers, hidden 4096, FFN 11008, 4-bit frozen base,
    LoRA r=64 on the seven projections, bf16), batch 4 x 512 tokens per GPU, INT4 activations with 1 % outlier
    channels and a 256-wide Hadamard rotation, data-parallel with one all-reduce of the LoRA gradients."""
    import torch
    import torch.distributed as dist
    from hyc_lora_b200 import synthetic
    from hyc_lora_b200.hosts.step import build_trainer

    # --step-config mistral_7b: configuration 4 (Mistral-7B shape, GQA 32/8 heads, FFN 14336, batch 2 x 2048 tokens per
    # GPU, INT2 activations with 2 % outlier channels, no rotation)
    mistral = args.step_config == "mistral_7b"
    batch, seq, vocab = (2, 2048, 32000) if mistral else (4, 512, 32000)
    bits, ratio, rotate = (2, 0.02, 0) if mistral else (4, 0.01, 256)
    trainer = build_trainer("mistral_7b" if mistral else "llama2_7b", layers=args.step_layers, bits=bits,
                            outlier_ratio=ratio, rotate=rotate, device=dev)
    ids_host = synthetic.token_ids(3, batch, seq, vocab, salt=rank).pin_memory()
    ids = torch.empty_like(ids_host, device=dev)
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()

    def one():
        ids.copy_(ids_host, non_blocking=True)            # host -> device copy of the step's inputs
        loss = trainer.step(ids)
        loss_host.copy_(loss.float(), non_blocking=True)  # device -> host read of the step's result

    for _ in range(3):                                     # includes the two calibration calls of every site
        one()
    graphed = trainer.capture(ids) if not args.no_graph else False
    for _ in range(2):
        one()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    steps = args.step_steps
    start.record()
    for _ in range(steps):
        one()
    stop.record()
    barrier()
    ms = start.elapsed_time(stop)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    tokens = batch * seq * world * steps
    # model flops per token: frozen base linears forward + input gradient (4 per weight), adapters forward +
    # both gradients (6 per weight), causal attention forward + backward (6 * seq * hidden per layer)
    from hyc_lora_b200.hosts.lora import FrozenLinear
    cfg = trainer.model.config
    p_base = sum(m.in_features * m.out_features for m in trainer.model.modules() if isinstance(m, FrozenLinear))
    p_lora = trainer.trainable()
    flops_token = 4 * p_base + 6 * p_lora + 6 * seq * cfg.hidden * cfg.layers
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    tensor_peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    achieved_tf = tokens / world / (ms / 1e3) * flops_token / 1e12      # per GPU
    roof = {"bound": "tensor", "achieved": round(achieved_tf, 1), "peak": tensor_peak, "unit": "TFLOP/s",
            "frac": round(achieved_tf / tensor_peak, 3), "per": "GPU",
            "peak_source": "of measured (sustained bf16 GEMM)" if "bf16_tflops_sustained" in peaks else "of fallback",
            "flops_per_token": flops_token, "base_params": p_base, "lora_params": p_lora}
    return {"metric": "7B HyC-LoRA train tokens/s", "value": tokens / (ms / 1e3), "unit": "tokens/s", "roofline": roof,
            "ms_per_step": ms / steps, "steps": steps, "loss": float(loss_host.item()), "cuda_graph": bool(graphed),
            "peak_mem_gb": round(torch.cuda.max_memory_allocated(dev) / 2 ** 30, 2),
            "config": {"model": ("Mistral-7B" if mistral else "LLaMA-2-7B") + " shape, random init, 4-bit codebook base (block 64)",
                       "layers": trainer.model.config.layers, "lora_r": 64, "trainable_params": trainer.trainable(),
                       "batch_per_gpu": batch, "seq_len": seq,
                       "activations": f"INT{bits}, {ratio:.0%} outlier channels, " + (f"rotate {rotate}" if rotate else "no rotation"),
                       "parallelism": f"dp{world}", "attention": "torch scaled_dot_product_attention (causal)",
                       "h2d_bytes_per_step": ids_host.numel() * 8, "d2h_bytes_per_step": 4}}


def sweep(packed, synthetic, x, w, peak):
    """Per-kernel GB/s for the operator sweep of configuration 5 (informational)."""
    import torch
    from hyc_lora_b200.operators import compress_function as cf
    rows_all, d = x.shape
    out = []

    def timed(fn, nbytes, name, reps=16):
        """fn(i): one call on input set i.  The calls are recorded in a CUDA graph (so that host overhead of the
        Python wrappers does not hide short kernels) and cycle through input sets whose total size exceeds L2."""
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(side):
            fn(0)
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, stream=side):
                for i in range(reps):
                    fn(i)
        torch.cuda.synchronize()
        graph.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(3):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / (3 * reps)
        out.append({"kernel": name, "ms": round(ms, 4), "GBps": round(nbytes / ms / 1e6, 1),
                    "frac": round(nbytes / ms / 1e6 / peak, 3)})

    norm = dict(kind="rms", weight=w, bias=None, eps=1e-5)
    score = packed.channel_absmax(x)
    for rows in (4096, 16384, 65536):
        # input sets: disjoint row ranges of x, 537 MB in total, visited round-robin
        sets = [x[i * rows:(i + 1) * rows] for i in range(rows_all // rows)]
        n = len(sets)
        dys = [torch.randn(rows, d, device=x.device, dtype=torch.bfloat16) for _ in range(min(n, 4))] if rows != 65536 else []
        for frac in (0.005, 0.01, 0.02):
            k = cf.outlier_channel_count(d, frac)
            ch = packed.select_channels(score, k)
            for bits in (2, 4, 8):
                for group in (0, 128):
                    for rotate in (0, 256):
                        if rows != 65536 and (frac != 0.01 or group or bits != 4):
                            continue
                        g = 1 if group == 0 else d // group
                        tag = f"T={rows} f={frac} b={bits} g={group} rot={rotate}"
                        timed(lambda i: packed.compress_n(sets[i % n], ch, bits, group, rotate, norm=norm),
                              algorithmic_bytes_per_row(d, bits, k, g) * rows, "norm+compress " + tag)
                        if frac == 0.01:
                            ps = [packed.compress_n(s_, ch, bits, group, rotate) for s_ in sets]
                            base = d * bits // 8 + 2 * k + 4 * g
                            timed(lambda i: packed.decompress(ps[i % n]), (base + 2 * d) * rows, "decompress " + tag)
                            if rows != 65536:
                                rstd = torch.ones(rows, device=x.device)
                                timed(lambda i: packed.norm_bwd(ps[i % n], dys[i % len(dys)], w, rstd, None, "rms"),
                                      (base + 4 + 4 * d) * rows, "norm_bwd " + tag)
                                timed(lambda i: packed.act_bwd("silu", ps[i % n], dys[i % len(dys)]), (base + 4 * d) * rows,
                                      "silu_bwd " + tag)
                            del ps
        del dys
    # dequant-fused tensor-core weight gradient vs. decompress + library GEMM
    for rows, bits, rank in ((65536, 4, 64), (65536, 4, 16), (65536, 2, 64), (65536, 8, 64), (2048, 4, 64)):
        xs = x[:rows]
        k = cf.outlier_channel_count(d, 0.01)
        ch = packed.select_channels(score, k)
        p = packed.compress_n(xs, ch, bits, 0, 0)
        g = torch.randn(rows, rank, device=x.device, dtype=torch.bfloat16)
        nbytes = rows * (d * bits // 8 + 2 * rank + 4 + 2 * k) + 4 * rank * d
        before = len(out)
        timed(lambda i: packed.lora_wgrad(p, g), nbytes, f"lora_wgrad tcgen05 T={rows} b={bits} r={rank}")
        timed(lambda i: packed.lora_wgrad(p, g, force_library=True), nbytes,
              f"lora_wgrad decompress+library GEMM T={rows} b={bits} r={rank}")
        for rec in out[before:]:
            rec["TFLOPs"] = round(2.0 * rows * rank * d / (rec["ms"] * 1e-3) / 1e12, 1)
    # reference mode, one line per bit width (static per-channel scales)
    xs = x[:16384]
    for bits in (2, 4, 8):
        thr, L, R, scale = cf.get_statistics(xs[:512].reshape(1, 512, d), 0, 0.01, 1.0, bits, "per-channel", 0)
        nb = (2 * d + d * bits // 8 + 8) * 16384 + int(0.02 * 16384 * d) * 4
        timed(lambda i: packed.compress_r(xs, thr, scale, bits), nb, f"R-mode compress T=16384 b={bits} per-channel")
        timed(lambda i: packed.compress_r(xs, thr, scale, bits, norm=norm), nb + (2 * d + 4) * 16384,
              f"R-mode norm+compress T=16384 b={bits} per-channel")
    return out


def run_case(args):
    """A few launches of one kernel on a small case (inputs still larger than L2), for profilers."""
    import torch
    from hyc_lora_b200 import packed, synthetic
    from hyc_lora_b200.operators import compress_function as cf
    torch.cuda.set_device(0)
    rows = args.rows
    if args.case == "step_kernels":
        # GPU time per kernel of the 7B-shaped training step (eager, torch.profiler / CUPTI), `--step-layers` decoder layers
        import collections
        from torch.profiler import ProfilerActivity, profile
        from hyc_lora_b200.hosts.step import build_trainer
        layers = args.step_layers or 8
        mistral = args.step_config == "mistral_7b"
        bits, ratio, rotate = (2, 0.02, 0) if mistral else (4, 0.01, 256)
        tr = build_trainer(args.step_config, layers=layers, compress=True, outlier_mode="channel", bits=bits,
                           outlier_ratio=ratio, rotate=rotate)
        ids = synthetic.token_ids(3, 2 if mistral else 4, 2048 if mistral else 512, 32000).cuda()
        for _ in range(3):
            tr.step(ids)
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(2):
                tr.step(ids)
            torch.cuda.synchronize()
        agg = collections.defaultdict(lambda: [0.0, 0])
        for e in prof.events():
            if e.device_type == torch.autograd.DeviceType.CUDA:
                agg[e.name][0] += e.device_time
                agg[e.name][1] += 1
        total = sum(v[0] for v in agg.values())
        rows_ = [{"kernel": k[:100], "ms_per_step": round(v[0] / 2e3, 3), "launches_per_step": v[1] // 2,
                  "share": round(v[0] / total, 4)} for k, v in sorted(agg.items(), key=lambda kv: -kv[1][0])[:40]]
        print(json.dumps({"case": args.case, "layers": layers, "gpu_ms_per_step": round(total / 2e3, 2), "kernels": rows_}))
        return
    if args.case == "mlp_sites":
        # the three one-pass kernels of the gated MLP's sites on bf16 [rows, cols] tensors, `launches` rounds
        cols = args.cols
        gate = (0.25 * synthetic.sweep_activation(rows, cols, FRACTION, salt=1)[0]).to("cuda")
        up = synthetic.sweep_activation(rows, cols, FRACTION, salt=2)[0].to("cuda")
        ch = packed.select_channels(packed.channel_absmax(gate), cf.outlier_channel_count(cols, FRACTION))
        fmt = dict(channels=ch, bits=BITS, group=args.group, rotate=args.rotate)
        for _ in range(args.launches):
            assert packed.product_compress_n(gate, up, ch, BITS, args.group, args.rotate, also_output=fmt) is not None
            assert packed.act_compress_n("silu", gate, ch, BITS, args.group, args.rotate, also_output=fmt) is not None
            packed.compress_n(gate, ch, BITS, args.group, args.rotate)
        torch.cuda.synchronize()
        print(json.dumps({"case": args.case, "rows": rows, "cols": cols, "launches": args.launches}))
        return
    x = synthetic.sweep_activation(rows, COLS, FRACTION)[0].to("cuda")
    w = synthetic.norm_weight(COLS).to("cuda")
    k = cf.outlier_channel_count(COLS, FRACTION)
    ch = packed.select_channels(packed.channel_absmax(x), k)
    norm = dict(kind="rms", weight=w, bias=None, eps=1e-5)
    dy = torch.randn(rows, COLS, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(rows, device="cuda")
    g64 = torch.randn(rows, 64, device="cuda", dtype=torch.bfloat16)
    if args.mode == "R":
        # reference mode: statistics as the reference calibrates them (batch element 0 of a [T/512, 512, D] view)
        x3 = x.reshape(rows // 512, 512, COLS)
        thr, _, _, scale = cf.get_statistics(x3[:1], 0, 0.01, 1.0, BITS, "per-channel", 0)
        p = packed.compress_r(x3, thr, scale, BITS, outlier_ratio=0.01)
        dy3 = dy.reshape(x3.shape)
        fns = {
            "norm_compress": lambda: packed.compress_r(x3, thr, scale, BITS, outlier_ratio=0.01, norm=norm),
            "compress": lambda: packed.compress_r(x3, thr, scale, BITS, outlier_ratio=0.01),
            "decompress": lambda: packed.decompress(p),
            "norm_bwd": lambda: packed.norm_bwd(p, dy3, w, rstd, None, "rms"),
            "silu_bwd": lambda: packed.act_bwd("silu", p, dy3),
            "lora_wgrad": lambda: packed.lora_wgrad(p, g64, path="tensor"),
        }
        for _ in range(args.launches):
            fns[args.case]()
        torch.cuda.synchronize()
        print(json.dumps({"case": args.case, "mode": "R", "rows": rows, "launches": args.launches,
                          "status": int(p.status.item()), "pool_used": int(p.pool_used.item())}))
        return
    p = packed.compress_n(x, ch, BITS, args.group, args.rotate)
    fns = {
        "lora_wgrad": lambda: packed.lora_wgrad(p, g64),
        "norm_compress": lambda: packed.compress_n(x, ch, BITS, args.group, args.rotate, norm=norm),
        "compress": lambda: packed.compress_n(x, ch, BITS, args.group, args.rotate),
        "decompress": lambda: packed.decompress(p),
        "norm_bwd": lambda: packed.norm_bwd(p, dy, w, rstd, None, "rms"),
        "silu_bwd": lambda: packed.act_bwd("silu", p, dy),
    }
    for _ in range(args.launches):
        fns[args.case]()
    torch.cuda.synchronize()
    print(json.dumps({"case": args.case, "rows": rows, "launches": args.launches, "status": int(p.status.item())}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sweep", action="store_true", help="add per-kernel numbers for the operator sweep")
    ap.add_argument("--no-step", action="store_true", help="skip the 7B-shaped training step")
    ap.add_argument("--step-layers", type=int, default=None, help="decoder layers of the step model (default 32)")
    ap.add_argument("--step-config", default="llama2_7b", choices=["llama2_7b", "mistral_7b"],
                    help="training-step configuration: 3 (LLaMA-2-7B shape, default) or 4 (Mistral-7B shape)")
    ap.add_argument("--step-steps", type=int, default=5)
    ap.add_argument("--no-graph", action="store_true", help="run the training step eagerly instead of from a CUDA graph")
    ap.add_argument("--case", default=None, help="profiling aid: run only this kernel (see run_case)")
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--cols", type=int, default=11008, help="--case mlp_sites: row width")
    ap.add_argument("--launches", type=int, default=4)
    ap.add_argument("--group", type=int, default=GROUP)
    ap.add_argument("--rotate", type=int, default=ROTATE)
    ap.add_argument("--mode", default="N", choices=["N", "R"], help="--case: channel mode (N) or reference mode (R)")
    args = ap.parse_args()
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
