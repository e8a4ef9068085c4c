#!/usr/bin/env python
"""Benchmark of the INT8-KV decode-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  Metric: decode-attention KV-read GB/s, i.e. the int8 K
and V bytes (2*B*H*S*D per step, the reference's own definition in
bench/bench_attn_decode.py:82) divided by the step time.

Workload at every N: per GPU, B=32 H=12 D=64 ctx=32768 (the serving-scale
configuration, 1.6 GB of int8 KV per step -- far larger than the 126 MB L2, so
no cache flush is needed between steps).  With N > 1 every rank owns its own
(batch, head) shard of an N-times larger batch and there is no collective in
the data path (weak scaling); the step time is the max over ranks.

Synthetic data: q fp16 ~ N(0,1), K/V fp32 ~ N(0,1), quantised per token on the
device with the library's own quantiser, seed 0.

  value     : median of 7 windows (each >= 50 ms and >= --steps steps) timed back to back
              with CUDA events, inputs resident in HBM; min / median / max and the SM
              clock sampled during each window are in `timing`
  parity    : three (b,h) rows of the headline output against the CPU oracle
  e2e       : the same call with every input copied from pinned host memory and
              the fp16 result copied back inside the timed region
  roofline  : K+V bytes over the median step time (scan kernel plus the merge that
              overlaps its tail: an upper bound of the scan's duration), against the
              measured HBM copy rate
  roofline_mlp / mlp_parity / cpu_baseline_mlp : the fused-MLP half of the metric (N=1)
  cpu_baseline / --impl reference : the reference's CPU torch path
              (dequantise + fp32 SDPA), restated in oracle/torch_cpu.py, on a
              bounded sample of (b,h) rows of the same workload
"""
import argparse
import importlib
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

B, H, D, S = 32, 12, 64, 32768
WORKLOAD = f"int8kv_decode_attention B{B} H{H} D{D} ctx{S} per GPU, fp16 out"
METRIC = "decode_attn_kv_read_GBps"
UNIT = "GB/s"
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


def kv_bytes(b, h, s, d):
    return 2 * b * h * s * d


def measured_hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) in a thread."""

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.02)

    def mark(self):
        return len(self.samples)

    def median_since(self, mark):
        part = self.samples[mark:]
        return statistics.median(part) if part else None

    def start(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()

    def stop(self):
        self._stop.set()
        if self._thr is not None:
            self._thr.join(timeout=2)
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# --------------------------------------------------------------------------- CPU arm
def cpu_reference_rate(seconds_budget=12.0, rows=24):
    """Time the reference's CPU path on `rows` (b,h) rows of the workload.

    Returns (GB/s of int8 K+V bytes, threads, description).
    """
    import torch
    from oracle import torch_cpu
    torch.manual_seed(0)
    q = torch.randn(1, rows, D).half()
    K = torch.randn(1, rows, S, D)
    V = torch.randn(1, rows, S, D)
    Qi, sQ = torch_cpu.quantize_per_token_cpu(q)
    Ki, sK = torch_cpu.quantize_per_token_cpu(K)
    Vi, sV = torch_cpu.quantize_per_token_cpu(V)
    del K, V
    torch_cpu.decode_attention_cpu(Qi, Ki, Vi, sQ, sK, sV)      # warm-up
    times = []
    t_end = time.perf_counter() + seconds_budget
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 200):
        t0 = time.perf_counter()
        torch_cpu.decode_attention_cpu(Qi, Ki, Vi, sQ, sK, sV)
        times.append(time.perf_counter() - t0)
    per_iter = sum(times) / len(times)
    gbs = kv_bytes(1, rows, S, D) / per_iter / 1e9
    desc = (f"{rows} of the {B * H} (b,h) rows at ctx {S}, D {D}: dequantise + fp32 SDPA "
            f"(torch CPU), mean of {len(times)} iterations")
    return gbs, per_iter, torch.get_num_threads(), desc


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    # every host core: a launcher may have set OMP_NUM_THREADS=1 for its ranks (torchrun does)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    budget = min(20.0, max(2.0, 1.0 * args.steps))
    gbs, per_iter, threads, desc = cpu_reference_rate(seconds_budget=budget)
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_iter * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "sampled": desc},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "host": {"cpu_count": os.cpu_count(), "torch_threads": threads, "torch": torch.__version__},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def make_inputs(torch, ext, b, h, s, d, outliers=False, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(b, h, d, device="cuda", dtype=torch.float16, generator=g)
    Qi, sQ = ext.quantize_per_token(q)
    out = [Qi, None, None, sQ, None, None]
    for idx in (1, 2):
        x = torch.randn(b, h, s, d, device="cuda", generator=g)
        if outliers:
            ch = torch.randperm(d, device="cuda", generator=g)[: max(1, int(0.01 * d))]
            x[..., ch] *= 20.0
        xi, sx = ext.quantize_per_token(x)
        del x
        out[idx], out[idx + 3] = xi, sx
    torch.cuda.synchronize()
    return out


def timed_steps(torch, fn, steps, warmup, barrier=None):
    for _ in range(warmup):
        fn()
    if barrier is not None:
        barrier()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    if barrier is not None:
        barrier()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / 1e3      # seconds


def timed_settled(torch, fn, steps, warmup, barrier=None, min_seconds=0.03):
    """timed_steps for the sweep's short kernels.  A fixed 10-20 calls of a kernel of tens of
    microseconds is a window of a few milliseconds, and the first milliseconds after a different
    workload were measured up to 20 % slow (the same call on the same buffers, repeated, settles).
    So: run the call for 20 ms first, then time at least `steps` calls and at least `min_seconds`
    of them.  Returns seconds scaled back to `steps` calls, like timed_steps."""
    if barrier is not None:
        return timed_steps(torch, fn, steps, warmup, barrier)
    fn()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n = 0
    while True:
        for _ in range(5):
            fn()
        n += 5
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if dt >= 0.02:
            break
    actual = max(steps, min(5000, int(min_seconds / (dt / n)) + 1))
    return timed_steps(torch, fn, actual, warmup) * steps / actual


def median_of_windows(torch, fn, steps, repeats=5, min_seconds=0.05):
    """Median over `repeats` settled windows of at least `min_seconds` each (the reference's
    convention is a median of >= 5 repeats, common/benchmark.py:12-43).  Returns seconds per call
    as (median, min, max)."""
    per = sorted(timed_settled(torch, fn, steps, 3, min_seconds=min_seconds) / steps for _ in range(repeats))
    return per[len(per) // 2], per[0], per[-1]


REPEATS = 7                 # timed windows of the headline; the value is their median
MIN_WINDOW_S = 0.05         # each window runs at least this long (and at least --steps steps)
# DRAM bytes the scan kernel moves per K+V byte, from a profiler capture of a 201 MB case of the
# same kernel (B8 H12 D64 ctx16384): the fp32 scales ride along, 8 bytes per position beside
# 128 bytes of K+V, plus what does not scale with positions.  Traffic grows in proportion to the
# positions scanned, so the bench-size figure is this ratio times the K+V bytes.
DRAM_BYTES_PER_KV_BYTE = 1.0627
MLP_DRAM_BYTES_PER_FORWARD = {(4096, 1024, 4096): 8_510_000 + 21_040_000}   # GEMM1 + GEMM2, dram__bytes_read + write


def parity_of_rows(torch, out, args, rows):
    """The headline output against the CPU oracle on a few (b,h) rows (outside any timed region)."""
    import numpy as np
    from oracle import decode as odec
    Qi, Ki, Vi, sQ, sK, sV = args
    cos_min, err_max = 1.0, 0.0
    for (b, h) in rows:
        sl = [t[b:b + 1, h:h + 1].contiguous().cpu().numpy() for t in (Qi, Ki, Vi, sQ, sK, sV)]
        ref = odec.decode_attention(*sl).astype(np.float64).ravel()
        got = out[b, h].float().cpu().numpy().astype(np.float64).ravel()
        cos = float(got @ ref / max(np.linalg.norm(got) * np.linalg.norm(ref), 1e-30))
        cos_min, err_max = min(cos_min, cos), max(err_max, float(np.abs(got - ref).max()))
    return {"rows": [list(r) for r in rows], "cos": cos_min, "max_abs": err_max,
            "bar": "cos >= 0.9999 and max_abs < 0.05 against the dequantised float64 computation",
            "ok": bool(cos_min >= 0.9999 and err_max < 0.05)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the sweep over the other configurations")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    distributed = world > 1
    # stdout carries exactly one JSON line: whatever a library prints to file descriptor 1 from
    # here on (NCCL's version and, when the caller sets NCCL_DEBUG=INFO, its transport lines) is
    # sent to stderr instead; the line itself is written to the saved descriptor at the end
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    if distributed:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    pkg = importlib.import_module("int8-transformer-kernels_b200")
    ext = pkg.int8_ext
    cabi = pkg.cabi
    lib = cabi.load()

    def barrier():
        if distributed:
            dist.barrier()

    def max_over_ranks(seconds):
        if not distributed:
            return seconds, seconds, seconds
        t = torch.tensor([seconds], device="cuda", dtype=torch.float64)
        every = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(every, t)
        vals = [float(v.item()) for v in every]
        return max(vals), min(vals), max(vals)

    sampler = ClockSampler(local_rank)
    inputs = make_inputs(torch, ext, B, H, S, D, seed=rank)
    Qi, Ki, Vi, sQ, sK, sV = inputs
    step_bytes = kv_bytes(B, H, S, D)

    def step():
        return ext.int8_decode_attention_forward(Qi, Ki, Vi, sQ, sK, sV)

    # ---- value: REPEATS windows of back-to-back steps, inputs resident; the median window -----
    sampler.start()
    probe = timed_steps(torch, step, args.steps, args.warmup, barrier)          # also the warm-up
    probe, _, _ = max_over_ranks(probe)
    n_win = max(args.steps, int(MIN_WINDOW_S / (probe / args.steps)) + 1)
    windows = []
    for _ in range(REPEATS):
        mark = sampler.mark()
        el = timed_steps(torch, step, n_win, 0, barrier)
        el_max, el_min, _ = max_over_ranks(el)
        mhz = sampler.median_since(mark)
        windows.append({"ms_per_step": el_max / n_win * 1e3, "ms_per_step_fastest_rank": el_min / n_win * 1e3,
                        "sm_mhz": mhz})
    clocks = sampler.stop()
    per_step = sorted(w["ms_per_step"] for w in windows)
    ms_med = per_step[len(per_step) // 2]
    value = world * step_bytes / (ms_med / 1e3) / 1e9
    launches_timed = 2 * n_win * REPEATS            # scan + merge per step

    out_dev = step()
    torch.cuda.synchronize()
    parity = parity_of_rows(torch, out_dev, inputs, [(0, 0), (13, 5), (31, 11)])
    ext.check_status()                              # no bounded device-side wait gave up during the run

    plan_ctas, plan_tiles = cabi.decode_plan(B * H, S, D)

    # ---- e2e: host buffers, H2D + call + D2H inside the timed region -----------------
    host = [t.cpu().pin_memory() for t in (Qi, Ki, Vi, sQ, sK, sV)]
    h2d = sum(t.numel() * t.element_size() for t in host)
    out_host = torch.empty(B, H, D, dtype=torch.float16).pin_memory()
    d2h = out_host.numel() * out_host.element_size()
    e2e_steps = max(3, min(args.steps, 10))

    def e2e_step():
        dev = [t.to("cuda", non_blocking=True) for t in host]
        o = ext.int8_decode_attention_forward(*dev)
        out_host.copy_(o, non_blocking=True)

    e2e_elapsed, _, _ = max_over_ranks(timed_steps(torch, e2e_step, e2e_steps, 3, barrier))
    e2e_value = world * step_bytes * e2e_steps / e2e_elapsed / 1e9
    del host

    # ---- the same end to end as a serving loop runs it: the INT8 KV cache stays on the device,
    # a step uploads the new token's q, k, v (fp16), quantises q, quantises k, v straight into the
    # cache (position S-1 is rewritten every step, so the context stays S), attends, reads back ----
    new_host = [torch.randn(B, H, D, dtype=torch.float16).pin_memory() for _ in range(3)]
    sK2, sV2 = sK.reshape(-1), sV.reshape(-1)

    def resident_step():
        qn, kn, vn = (t.to("cuda", non_blocking=True) for t in new_host)
        ext.kv_append_quantize(kn, vn, Ki, Vi, sK2, sV2, S - 1)
        qi, sq = ext.quantize_per_token(qn)
        out_host.copy_(ext.int8_decode_attention_forward(qi, Ki, Vi, sq, sK, sV), non_blocking=True)

    res_elapsed, _, _ = max_over_ranks(timed_steps(torch, resident_step, args.steps, 3, barrier))
    res_value = world * step_bytes * args.steps / res_elapsed / 1e9

    peak, peak_kind = measured_hbm_peak()
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_med, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int8 -> int32 dot, fp32 softmax/accumulate",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_bh": world * B * H, "sharding": "(batch, head) per rank, no collective",
                   "persistent_ctas": plan_ctas, "kv_tiles_per_cta": plan_tiles,
                   "l2": "inputs (1.6 GB per step) larger than L2, no flush",
                   "pct_of_8TBps": 100.0 * value / world / NOMINAL_HBM_GBS},
        "timing": {"value_is": f"median of {REPEATS} windows of {n_win} back-to-back steps each "
                               f"(>= {MIN_WINDOW_S * 1e3:.0f} ms and >= --steps), CUDA events, max over ranks per window",
                   "steps_per_window": n_win, "windows": windows,
                   "ms_per_step_min": per_step[0], "ms_per_step_median": ms_med, "ms_per_step_max": per_step[-1],
                   "pct_of_8TBps_min_median_max": [100.0 * step_bytes / (t / 1e3) / 1e9 / NOMINAL_HBM_GBS
                                                   for t in (per_step[-1], ms_med, per_step[0])],
                   "ms_x_sm_mhz": [w["ms_per_step"] * w["sm_mhz"] if w["sm_mhz"] else None for w in windows]},
        "parity": parity,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": e2e_steps,
                "note": "every input, the whole 1.6 GB INT8 KV cache included, is copied from pinned host memory "
                        "each step: a PCIe figure"},
        "e2e_cache_resident": {"value": res_value, "unit": UNIT, "steps": args.steps,
                               "h2d_bytes_per_step": 3 * B * H * D * 2, "d2h_bytes_per_step": d2h,
                               "note": "the KV cache stays in HBM as in serving; a step uploads the new token's q, k, v "
                                       "(fp16), quantises k, v into the cache and q for the scan, attends, reads the "
                                       "fp16 result back"},
        "gpu_launches": launches_timed,
        "clocks": clocks,
    }
    # Duration of the scan kernel: one step is scan + merge, chained by programmatic dependent
    # launch so that the merge (2-3 us) overlaps the scan's tail; the step time of the timed
    # region is therefore an upper bound of the scan's duration, and the figure used here.
    step_s = ms_med / 1e3
    achieved = step_bytes / step_s / 1e9
    rows_bytes = plan_ctas * 2 * 4 * (D + 4) * 4
    line["roofline"] = {"bound": "hbm", "kernel": "decode_partial_kernel<64>", "achieved": achieved,
                        "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                        "frac_of_8TBps": achieved / NOMINAL_HBM_GBS,
                        "algorithmic_bytes_per_launch": step_bytes,
                        "us_per_launch": step_s * 1e6,
                        "traffic": int(DRAM_BYTES_PER_KV_BYTE * step_bytes) + rows_bytes,
                        "traffic_source": "scaled from a profiler capture of a 201 MB case (linear in positions)",
                        "timing_note": "us_per_launch is the median step time of the timed windows (scan + the merge "
                                       "that overlaps its tail): an upper bound of the scan's duration"}

    if rank == 0 and world == 1:
        gbs, per_iter, threads, desc = cpu_reference_rate(seconds_budget=10.0)
        line["cpu_baseline"] = {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc}
        line.update(mlp_headline(torch, ext, cabi))

    if not args.no_extras:
        line["sweep"] = sweep(torch, ext, cabi, world, rank, barrier, dist if distributed else None)

    if rank == 0:
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if distributed:
        dist.destroy_process_group()


def mlp_inputs(torch, ext, M, dm, dff, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(1, M, dm, device="cuda", dtype=torch.float16, generator=g)
    xi, sx = ext.quantize_per_token(x)
    W1 = torch.randn(dm, dff, device="cuda", generator=g) * 0.02
    W2 = torch.randn(dff, dm, device="cuda", generator=g) * 0.02
    s1 = W1.abs().amax(dim=0).clamp(min=1e-8) / 127.0
    s2 = W2.abs().amax(dim=0).clamp(min=1e-8) / 127.0
    w1i = (W1 / s1).round().clamp(-128, 127).to(torch.int8).contiguous()
    w2i = (W2 / s2).round().clamp(-128, 127).to(torch.int8).contiguous()
    b1 = torch.randn(dff, device="cuda", generator=g) * 0.01
    return x, xi, sx.reshape(-1).contiguous(), W1, W2, w1i, w2i, s1, s2, b1


def mlp_headline(torch, ext, cabi):
    """The fused-MLP half of the metric: INT8 TOPS of a whole forward (4*M*d_model*d_ff operations,
    bench/sweep.py:97-99 of the reference) at M=4096 for both geometries, against an INT8 tensor
    peak measured in this same run (torch._int_mm on 8192^3, i.e. the vendor library's int8 GEMM:
    a yardstick, never on the hot path) and against the nominal 4.5 POPS; the share of int8 output
    codes that differ from the stage-by-stage restatement of the reference kernel, as built and
    with I8TK_MLP_REFERENCE_ROUNDING; and the reference's CPU simulation timed on the host cores."""
    import numpy as np
    lib = cabi.load()
    out = {}
    # on-box INT8 yardstick
    n = 8192
    a = torch.randint(-127, 128, (n, n), dtype=torch.int8, device="cuda")
    b = torch.randint(-127, 128, (n, n), dtype=torch.int8, device="cuda")
    try:
        t_mm, _, _ = median_of_windows(torch, lambda: torch._int_mm(a, b), 10, repeats=5, min_seconds=0.05)
        int8_peak = 2.0 * n ** 3 / t_mm / 1e12
        peak_kind = "measured in this run: torch._int_mm 8192^3 (the vendor library's int8 GEMM), median of 5 windows"
    except Exception as e:            # noqa: BLE001  (an int8 GEMM the library build does not offer)
        int8_peak, peak_kind = None, "unavailable: %s" % type(e).__name__
    del a, b
    torch.cuda.empty_cache()
    rl = []
    for (M, dm, dff) in ((4096, 1024, 4096), (4096, 768, 3072)):
        x, xi, sxf, W1, W2, w1i, w2i, s1, s2, b1 = mlp_inputs(torch, ext, M, dm, dff)
        W1T, W2T = ext.transpose_int8_weights(w1i, w2i)
        flags = cabi.MLP_X_PER_TOKEN | cabi.MLP_W_PER_CHANNEL | cabi.MLP_PREPACKED
        wb = lib.i8tk_mlp_workspace_bytes(M, dm, dff, flags)
        ws = torch.zeros(wb, dtype=torch.uint8, device="cuda")
        o = torch.empty_like(xi)
        osc = torch.empty(M, device="cuda")
        st = torch.cuda.current_stream().cuda_stream

        kept = [0]        # the workspace is this loop's alone: from the second call on the library is told so

        def fwd():
            cabi.check(lib.i8tk_mlp_forward(xi.data_ptr(), W1T.data_ptr(), W2T.data_ptr(), o.data_ptr(),
                                            sxf.data_ptr(), s1.data_ptr(), s2.data_ptr(), b1.data_ptr(),
                                            osc.data_ptr(), None, M, dm, dff, flags | kept[0], ws.data_ptr(), wb, st))
            kept[0] = cabi.MLP_WORKSPACE_KEPT

        t_med, t_min, t_max = median_of_windows(torch, fwd, 50, repeats=5, min_seconds=0.05)
        cabi.check(lib.i8tk_check_status_word(ws.data_ptr(), st), "fused MLP")
        ops = 4.0 * M * dm * dff
        tops = ops / t_med / 1e12
        rl.append({"bound": "tensor", "kernel": "gemm_i8_kernel x2 (one fused MLP forward: GEMM1+GELU+requant, GEMM2+requant)",
                   "workload": f"cfg4 fused INT8 MLP M={M} {dm}->{dff}->{dm}, prepacked weights, C ABI",
                   "achieved": tops, "peak": int8_peak, "peak_kind": peak_kind, "unit": "TOP/s",
                   "frac": tops / int8_peak if int8_peak else None,
                   "frac_of_4.5_POPS_nominal": tops / 4500.0,
                   "algorithmic_ops_per_forward": ops, "us_per_forward": t_med * 1e6,
                   "us_per_forward_min_max": [t_min * 1e6, t_max * 1e6],
                   # DRAM bytes of the two GEMM launches in a profiler capture of this shape (cold caches: the
                   # operands, 30 MB, are L2-resident in the timed loop); not captured at the other width
                   "traffic": MLP_DRAM_BYTES_PER_FORWARD.get((M, dm, dff))})
    out["roofline_mlp"] = rl

    # int8 codes against the stage-by-stage restatement of the reference kernel, M=512 768->3072
    from oracle import mlp as omlp
    M, dm, dff = 512, 768, 3072
    x, xi, sxf, W1, W2, w1i, w2i, s1, s2, b1 = mlp_inputs(torch, ext, M, dm, dff, seed=1)
    ref = omlp.kernel_mlp(xi[0].cpu().numpy(), w1i.cpu().numpy(), w2i.cpu().numpy(), sxf.cpu().numpy(),
                          s1.cpu().numpy(), s2.cpu().numpy(), b1=b1.cpu().numpy())
    rates = {}
    for tag, on in (("as_built", False), ("reference_rounding", True)):
        was = ext.set_mlp_reference_rounding(on)
        try:
            o8, osc = ext.int8_mlp_forward_per_channel_bias(xi, w1i, w2i, sxf, s1, s2, b1)
        finally:
            ext.set_mlp_reference_rounding(was)
        got = o8[0].cpu().numpy()
        d = np.abs(got.astype(np.int32) - ref["out_i8"].astype(np.int32))
        deq = got.astype(np.float32) * osc.cpu().numpy()[:, None]
        want = ref["out_i8"].astype(np.float32) * ref["out_scale"][:, None]
        rates[tag] = {"pct_codes_differing": 100.0 * float((d != 0).mean()), "max_steps": int(d.max()),
                      "max_abs_dequantised": float(np.abs(deq - want).max())}
    out["mlp_parity"] = {"workload": f"M={M} {dm}->{dff}->{dm}, per-token x, per-channel W, bias, vs the "
                                     "stage-by-stage numpy restatement of the reference kernel",
                         "as_built": rates["as_built"], "reference_rounding": rates["reference_rounding"],
                         "attribution": "as_built uses fma(acc*sx, sW1, b1) and the hardware tanh; reference_rounding "
                                        "follows the source order with tanhf, so what it leaves is tanhf vs numpy tanh"}

    # CPU baseline of the MLP: the reference's simulation (validation/validate_int8.py:174-225)
    from oracle import torch_cpu
    xc, W1c, W2c = x[0].float().cpu(), W1.cpu(), W2.cpu()
    torch_cpu.mlp_cpu(xc, W1c, W2c)
    times = []
    t_end = time.perf_counter() + 6.0
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 100):
        t0 = time.perf_counter()
        torch_cpu.mlp_cpu(xc, W1c, W2c)
        times.append(time.perf_counter() - t0)
    per = sorted(times)[len(times) // 2]
    out["cpu_baseline_mlp"] = {"value": 4.0 * M * dm * dff / per / 1e12, "unit": "TOP/s", "ms_per_forward": per * 1e3,
                               "cores": torch.get_num_threads(), "kind": "port",
                               "sample": f"sim_mlp at M={M} {dm}->{dff}->{dm} (torch CPU, fp32 on dequantised "
                                         f"operands, quantisers included), median of {len(times)} forwards"}
    return out


def sweep(torch, ext, cabi, world, rank, barrier, dist):
    """Other configurations, device-timed, reported beside the headline."""
    def reduce_max(el):
        if dist is None:
            return el
        t = torch.tensor([el], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    res = []
    cases = [("cfg0 B1 H12 D64 ctx1024", 1, 12, 64, 1024, False, 200),
             ("cfg1 B32 H12 D64 ctx4096", 32, 12, 64, 4096, False, 100),
             ("cfg1 B32 H12 D64 ctx8192", 32, 12, 64, 8192, False, 100),
             ("cfg1 B32 H12 D64 ctx16384", 32, 12, 64, 16384, False, 50)]
    if world == 1:
        cases.append(("cfg2 B64 H32 D128 ctx8192 (1 GPU)", 64, 32, 128, 8192, True, 20))
    else:
        # config 2 strong-scaled: the 2048 (b,h) rows split evenly over the ranks
        cases.append((f"cfg2 B64 H32 D128 ctx8192 sharded by (b,h) over {world} GPUs", 64 // world, 32, 128,
                      8192, True, 20))
    for name, b, h, d, s, outl, steps in cases:
        args = make_inputs(torch, ext, b, h, s, d, outliers=outl, seed=rank)
        el = reduce_max(timed_settled(torch, lambda: ext.int8_decode_attention_forward(*args), steps, 5, barrier))
        strong = name.startswith("cfg2") and world > 1
        gbs = world * kv_bytes(b, h, s, d) * steps / el / 1e9
        res.append({"workload": name, "us_per_step": el / steps * 1e6, "GBps": gbs,
                    "pct_of_8TBps_per_gpu": 100.0 * gbs / world / NOMINAL_HBM_GBS,
                    "scaling": "strong" if strong else "weak",
                    "l2_resident": kv_bytes(b, h, s, d) < 100e6})
        if name.startswith("cfg0") and world == 1:
            # launch-bound: the same call captured 20 times into one CUDA graph and replayed
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(3):
                    ext.int8_decode_attention_forward(*args)
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(20):
                    graph_out = ext.int8_decode_attention_forward(*args)
            el_g = timed_settled(torch, graph.replay, 20, 3)
            res[-1]["us_per_step_replayed_from_a_cuda_graph"] = el_g / 20 / 20 * 1e6
            del graph, graph_out
        del args
        torch.cuda.empty_cache()

    if world > 1:
        # config 3: B4 H32 D128 ctx 524288, KV sequence cut into `world` chunks, one per GPU;
        # per-(b,h) (m, l, acc) rows all-gathered over NCCL and merged on every rank
        pkg = importlib.import_module("int8-transformer-kernels_b200")
        sh = pkg.sharding
        b, h, d, s = 4, 32, 128, 524288
        a, e_ = sh.seq_shard_range(s, world, rank)
        Qi, Ki, Vi, sQ, sK, sV = make_inputs(torch, ext, b, h, e_ - a, d, outliers=True, seed=100 + rank)
        g = torch.Generator(device="cuda").manual_seed(7)       # q is replicated: same seed on every rank
        Qi, sQ = ext.quantize_per_token(torch.randn(b, h, d, device="cuda", dtype=torch.float16, generator=g))
        steps = 20
        fn = lambda: sh.decode_attention_seq_sharded(Qi, Ki, Vi, sQ, sK, sV)
        el_nccl = reduce_max(timed_steps(torch, fn, steps, 5, barrier))
        dec = sh.SeqShardedDecoder(b, h, d, torch.device("cuda", torch.cuda.current_device()))
        el = reduce_max(timed_steps(torch, lambda: dec(Qi, Ki, Vi, sQ, sK, sV), steps, 5, barrier))
        dec.check()
        agree = float((dec(Qi, Ki, Vi, sQ, sK, sV).float() - fn().float()).abs().max())
        gbs = kv_bytes(b, h, s, d) * steps / el / 1e9
        res.append({"workload": f"cfg3 B4 H32 D128 ctx524288 KV-sequence sharded over {world} GPUs, "
                                f"(m,l,acc) rows ({b * h * (d + 4) * 4} B per rank pair) stored to peers over "
                                f"NVLink inside the merge kernel",
                    "us_per_step": el / steps * 1e6, "GBps": gbs,
                    "pct_of_8TBps_per_gpu": 100.0 * gbs / world / NOMINAL_HBM_GBS, "scaling": "strong",
                    "us_per_step_with_nccl_all_gather_instead": el_nccl / steps * 1e6,
                    "max_abs_diff_between_the_two_paths": agree})
        del Ki, Vi, sK, sV
        torch.cuda.empty_cache()
    elif rank == 0:
        res.extend(quantiser_and_prefill_sweep(torch, ext))
        res.extend(mlp_sweep(torch, ext, cabi))
        res.extend(block_sweep(torch))
        res.extend(paged_sweep(torch, ext))
    return res


def paged_sweep(torch, ext):
    """The headline geometry (B32 H12 D64 ctx 32768) read through a paged INT8 KV cache with a
    shuffled page table: all requests at full length, and two batches of mixed lengths (drawn
    uniformly from 256..32768; one request at 32768 among 31 at 2048).  GB/s of the K+V bytes
    the lengths really cover, as in the headline metric."""
    out = []
    B, H, D, S = 32, 12, 64, 32768
    g = torch.Generator(device="cuda").manual_seed(0)
    Qi, sQ = ext.quantize_per_token(torch.randn(B, H, D, device="cuda", dtype=torch.float16, generator=g))
    sq = sQ.reshape(-1).contiguous()
    mixes = (("all requests at full length", torch.full((B,), S, dtype=torch.int32)),
             ("lengths uniform in 256..32768", torch.randint(256, S + 1, (B,), generator=torch.Generator().manual_seed(1)).to(torch.int32)),
             ("one request at 32768, 31 at 2048", torch.tensor([S] + [2048] * (B - 1), dtype=torch.int32)))
    for page in (16, 64, 128):
        npp = S // page
        pages = B * npp
        Kp = torch.randint(-127, 128, (pages, H, page, D), dtype=torch.int8, device="cuda", generator=g)
        Vp = torch.randint(-127, 128, (pages, H, page, D), dtype=torch.int8, device="cuda", generator=g)
        sKp = torch.rand(pages, H, page, device="cuda", generator=g) * 0.02 + 0.01
        sVp = torch.rand(pages, H, page, device="cuda", generator=g) * 0.02 + 0.01
        table = torch.randperm(pages, device="cuda", generator=g).to(torch.int32).view(B, npp).contiguous()
        for name, lens in mixes if page != 64 else mixes[:1]:
            seq = lens.cuda()
            steps = 20
            el = timed_settled(torch, lambda: ext.int8_decode_attention_paged(Qi, Kp, Vp, sq, sKp, sVp, table, seq, S), steps, 3)
            gbps = 2 * H * D * int(lens.sum()) * steps / el / 1e9
            out.append({"workload": f"paged decode B{B} H{H} D{D} ctx{S}, page {page}, shuffled page table, {name}",
                        "us_per_step": el / steps * 1e6, "GBps": gbps, "pct_of_8TBps_per_gpu": gbps / 80.0})
        del Kp, Vp, sKp, sVp
        torch.cuda.empty_cache()
    # config 2's geometry (D = 128) through 64-position pages, all requests at full length
    B, H, D, S, page = 64, 32, 128, 8192, 64
    Qi, sQ = ext.quantize_per_token(torch.randn(B, H, D, device="cuda", dtype=torch.float16, generator=g))
    npp = S // page
    pages = B * npp
    Kp = torch.randint(-127, 128, (pages, H, page, D), dtype=torch.int8, device="cuda", generator=g)
    Vp = torch.randint(-127, 128, (pages, H, page, D), dtype=torch.int8, device="cuda", generator=g)
    sKp = torch.rand(pages, H, page, device="cuda", generator=g) * 0.02 + 0.01
    sVp = torch.rand(pages, H, page, device="cuda", generator=g) * 0.02 + 0.01
    table = torch.randperm(pages, device="cuda", generator=g).to(torch.int32).view(B, npp).contiguous()
    seq = torch.full((B,), S, dtype=torch.int32, device="cuda")
    sq = sQ.reshape(-1).contiguous()
    el = timed_settled(torch, lambda: ext.int8_decode_attention_paged(Qi, Kp, Vp, sq, sKp, sVp, table, seq, S), 20, 3)
    gbps = kv_bytes(B, H, S, D) * 20 / el / 1e9
    out.append({"workload": f"paged decode B{B} H{H} D{D} ctx{S}, page {page}, shuffled page table, all requests at full length",
                "us_per_step": el / 20 * 1e6, "GBps": gbps, "pct_of_8TBps_per_gpu": gbps / 80.0})
    del Kp, Vp, sKp, sVp
    torch.cuda.empty_cache()
    return out


def block_sweep(torch):
    """End-to-end pre-LN block (LayerNorm and projections fp16 in both paths; attention core and
    MLP either fp16 -- torch SDPA and fp16 GEMMs -- or the INT8 ops), the geometry of the
    reference's block bench (bench/bench_block.py:209-215): prefill B8 H16 Dh64 d_ff 4096,
    decode B128 over a prefilled cache.  cos = INT8 block output against the fp16 block."""
    import torch.nn.functional as F
    pkg = importlib.import_module("int8-transformer-kernels_b200")
    blk = pkg.block.Int8Block(1024, 16, 4096)
    cos = lambda a, b: F.cosine_similarity(a.float().flatten(), b.float().flatten(), dim=0).item()
    out = []
    g = torch.Generator(device="cuda").manual_seed(1)
    for S in (512, 2048):
        x = torch.randn(8, S, 1024, device="cuda", dtype=torch.float16, generator=g)
        c = cos(blk.forward_prefill(x, True), blk.forward_prefill(x, False))
        t8 = timed_settled(torch, lambda: blk.forward_prefill(x, True), 10, 3) / 10
        t16 = timed_settled(torch, lambda: blk.forward_prefill(x, False), 10, 3) / 10
        tmix = timed_settled(torch, lambda: blk.forward_prefill(x, True, fp16_attention=True), 10, 3) / 10
        out.append({"workload": f"block prefill B8 H16 Dh64 d_ff4096 S{S}", "int8_ms": t8 * 1e3, "fp16_ms": t16 * 1e3,
                    "speedup_vs_fp16": t16 / t8, "cos_vs_fp16": c,
                    "fp16_attention_int8_mlp_ms": tmix * 1e3, "speedup_vs_fp16_of_that_mix": t16 / tmix})
    for Skv in (8192, 32768):
        x = torch.randn(128, 1, 1024, device="cuda", dtype=torch.float16, generator=g)
        K = torch.randn(128, 16, Skv, 64, device="cuda", dtype=torch.float16, generator=g)
        V = torch.randn(128, 16, Skv, 64, device="cuda", dtype=torch.float16, generator=g)
        kv8 = blk.quantize_kv(K, V)
        c = cos(blk.forward_decode(x, kv8, True), blk.forward_decode(x, (K, V), False))
        t8 = timed_settled(torch, lambda: blk.forward_decode(x, kv8, True), 10, 3) / 10
        t16 = timed_settled(torch, lambda: blk.forward_decode(x, (K, V), False), 10, 3) / 10
        out.append({"workload": f"block decode B128 H16 Dh64 d_ff4096 Skv{Skv}", "int8_ms": t8 * 1e3,
                    "fp16_ms": t16 * 1e3, "speedup_vs_fp16": t16 / t8, "cos_vs_fp16": c})
        del K, V, kv8
        torch.cuda.empty_cache()
    return out


def quantiser_and_prefill_sweep(torch, ext):
    """Per-token quantiser (HBM-bound: bytes in + codes out + scales) and prefill attention
    (4*B*H*S^2*D ops), device-timed."""
    out = []
    for dt, rows, cols, tag in ((torch.float32, 32 * 12 * 8192, 64, "K/V of cfg1 ctx8192, fp32 in"),
                                (torch.float32, 64 * 32 * 2048, 128, "quarter of cfg2 K/V, fp32 in"),
                                (torch.float16, 65536, 1024, "MLP activations, fp16 in")):
        x = torch.randn(rows, cols, device="cuda", dtype=dt)
        steps = 20
        el = timed_settled(torch, lambda: ext.quantize_per_token(x), steps, 3)
        byts = rows * cols * (x.element_size() + 1) + rows * 4
        out.append({"workload": f"quantize_per_token [{rows}, {cols}] ({tag})", "us_per_step": el / steps * 1e6,
                    "GBps": byts * steps / el / 1e9, "l2_resident": byts < 100e6})
        del x
        torch.cuda.empty_cache()
    import torch.nn.functional as F
    for rows, cols in ((16384, 1024), (131072, 1024)):
        x = torch.randn(rows, cols, device="cuda", dtype=torch.float16)
        steps = 20
        el = timed_settled(torch, lambda: ext.layernorm_quantize(x), steps, 3)
        el2 = timed_settled(torch, lambda: ext.quantize_per_token(F.layer_norm(x, (cols,))), steps, 3)
        byts = rows * cols * 3 + rows * 4
        out.append({"workload": f"layernorm_quantize [{rows}, {cols}] fp16 (LayerNorm + per-token quantiser, one pass)",
                    "us_per_step": el / steps * 1e6, "GBps": byts * steps / el / 1e9,
                    "us_per_step_torch_layer_norm_then_quantize_per_token": el2 / steps * 1e6,
                    "l2_resident": byts < 100e6})
        del x
        torch.cuda.empty_cache()
    for (b, h, s, d) in ((8, 8, 4096, 64), (4, 8, 4096, 128)):
        g = torch.Generator(device="cuda").manual_seed(0)
        t = []
        for _ in range(3):
            xi, sx = ext.quantize_per_token(torch.randn(b, h, s, d, device="cuda", dtype=torch.float16, generator=g))
            t.extend([xi, sx.reshape(-1).contiguous()])
        steps = 10
        el = timed_settled(torch, lambda: ext.int8_attention_forward(t[0], t[2], t[4], t[1], t[3], t[5]), steps, 3)
        ops = 4.0 * b * h * s * s * d
        out.append({"workload": f"prefill int8 attention B{b} H{h} S{s} D{d}", "us_per_step": el / steps * 1e6,
                    "TOPS": ops * steps / el / 1e12})
    return out


def mlp_sweep(torch, ext, cabi):
    """Fused INT8 MLP (per-token x, per-channel W, bias, GELU, per-token requant), INT8 TOPS =
    4*M*d_model*d_ff / time (bench/sweep.py:97-99 of the reference).  Weights are handed over
    pre-transposed once (the prepacked form, C ABI); the op-level call on weights in the
    reference's [K][N] layout (read in place through MN-major descriptors) is timed beside it."""
    lib = cabi.load()
    out = []
    for (dm, dff) in ((768, 3072), (1024, 4096)):
        for M in (512, 4096, 16384):
            g = torch.Generator(device="cuda").manual_seed(0)
            x = torch.randn(1, M, dm, device="cuda", dtype=torch.float16, generator=g)
            xi, sx = ext.quantize_per_token(x)
            W1 = torch.randn(dm, dff, device="cuda", generator=g) * 0.02
            W2 = torch.randn(dff, dm, device="cuda", generator=g) * 0.02
            s1 = W1.abs().amax(dim=0).clamp(min=1e-8) / 127.0
            s2 = W2.abs().amax(dim=0).clamp(min=1e-8) / 127.0
            w1i = (W1 / s1).round().clamp(-128, 127).to(torch.int8).contiguous()
            w2i = (W2 / s2).round().clamp(-128, 127).to(torch.int8).contiguous()
            b1 = torch.randn(dff, device="cuda", generator=g) * 0.01
            sxf = sx.reshape(-1).contiguous()
            W1T, W2T = ext.transpose_int8_weights(w1i, w2i)
            flags = cabi.MLP_X_PER_TOKEN | cabi.MLP_W_PER_CHANNEL | cabi.MLP_PREPACKED
            wb = lib.i8tk_mlp_workspace_bytes(M, dm, dff, flags)
            ws = torch.empty(wb, dtype=torch.uint8, device="cuda")
            o = torch.empty_like(xi)
            osc = torch.empty(M, device="cuda")
            st = torch.cuda.current_stream().cuda_stream

            kept = [0]    # the workspace is this loop's alone: from the second call on the library is told so

            def prepacked():
                cabi.check(lib.i8tk_mlp_forward(xi.data_ptr(), W1T.data_ptr(), W2T.data_ptr(), o.data_ptr(),
                                                sxf.data_ptr(), s1.data_ptr(), s2.data_ptr(), b1.data_ptr(),
                                                osc.data_ptr(), None, M, dm, dff, flags | kept[0], ws.data_ptr(), wb, st))
                kept[0] = cabi.MLP_WORKSPACE_KEPT

            steps = 50
            el = timed_settled(torch, prepacked, steps, 5)
            el2 = timed_settled(torch, lambda: ext.int8_mlp_forward_per_channel_bias(xi, w1i, w2i, sxf, s1, s2, b1),
                              steps, 5)
            ops = 4.0 * M * dm * dff
            out.append({"workload": f"cfg4 fused INT8 MLP M={M} {dm}->{dff}->{dm}",
                        "us_per_step": el / steps * 1e6, "int8_TOPS": ops * steps / el / 1e12,
                        "pct_of_4.5_POPS_nominal": 100.0 * ops * steps / el / 4.5e15,
                        "us_per_step_weights_as_KxN_op_call": el2 / steps * 1e6,
                        "l2_resident": True})
    return out


if __name__ == "__main__":
    main()
