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

  value     : steps timed back to back with CUDA events, inputs resident in HBM
  e2e       : the same call with every input copied from pinned host memory and
              the fp16 result copied back inside the timed region
  roofline  : K+V bytes over the step time of the timed region (scan kernel plus the
              merge that overlaps its tail: an upper bound of the scan's duration),
              against the measured HBM copy rate; the scan bracketed by events of its
              own (recorded inside the library) is reported beside it
  cpu_baseline / --impl reference : the reference's CPU torch path
              (dequantise + fp32 SDPA), restated in oracle/torch_cpu.py, on a
              bounded sample of (b,h) rows of the same workload
"""
import argparse
import ctypes
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
# Small cases for profiler captures: larger than L2 (126 MB) so DRAM counters
# mean something, a few hundred MB on the device, a handful of launches.
PROFILE_CASES = {
    "decode_d64": (8, 12, 64, 16384),      # 201 MB of int8 K+V
    "decode_d128": (8, 8, 128, 8192),      # 134 MB
    "mlp_m4096_768": (4096, 768, 3072),    # fused MLP forward (L2 resident by nature: 30 MB of operands)
    "mlp_m4096_1024": (4096, 1024, 4096),
    "quantize_f32_64": (3145728, 64),      # rows, cols: 1.0 GB through the per-token quantiser
    "prefill_d64": (2, 8, 4096, 64),       # B, H, S, D: 512 CTAs of 128 query rows
    "prefill_d128": (2, 8, 4096, 128),
    "paged_d64_p64": (8, 12, 64, 16384, 64),   # B, H, D, longest request, page: lengths 2048..16384, shuffled table
    "lnquant_f16_1024": (131072, 1024),    # rows, cols: 268 MB in, 134 MB of codes out
}


def run_profile_case(name):
    import torch
    pkg = importlib.import_module("int8-transformer-kernels_b200")
    ext = pkg.int8_ext
    if name.startswith("quantize"):
        rows, cols = PROFILE_CASES[name]
        x = torch.randn(rows, cols, device="cuda", dtype=torch.float32)
        for _ in range(3):
            qi, sc = ext.quantize_per_token(x)
        torch.cuda.synchronize()
        print(f"profile case {name}: [{rows}, {cols}] fp32, bytes per launch {rows * cols * 5 + rows * 4}, "
              f"checksum {float(sc.sum()):.4f}")
        return
    if name.startswith("lnquant"):
        rows, cols = PROFILE_CASES[name]
        x = torch.randn(rows, cols, device="cuda", dtype=torch.float16)
        for _ in range(3):
            qi, sc = ext.layernorm_quantize(x)
        torch.cuda.synchronize()
        print(f"profile case {name}: [{rows}, {cols}] fp16, bytes per launch {rows * cols * 3 + rows * 4}, "
              f"checksum {float(sc.sum()):.4f}")
        return
    if name.startswith("paged"):
        b, h, d, s, page = PROFILE_CASES[name]
        g = torch.Generator(device="cuda").manual_seed(0)
        Qi, sQ = ext.quantize_per_token(torch.randn(b, h, d, device="cuda", dtype=torch.float16, generator=g))
        npp = s // page
        pages = b * npp
        Kp = torch.randint(-127, 128, (pages, h, page, d), dtype=torch.int8, device="cuda", generator=g)
        Vp = torch.randint(-127, 128, (pages, h, page, d), dtype=torch.int8, device="cuda", generator=g)
        sKp = torch.rand(pages, h, page, device="cuda", generator=g) * 0.02 + 0.01
        sVp = torch.rand(pages, h, page, device="cuda", generator=g) * 0.02 + 0.01
        table = torch.randperm(pages, device="cuda", generator=g).to(torch.int32).view(b, npp).contiguous()
        lens = torch.linspace(2048, s, b).to(torch.int32)
        seq = lens.cuda()
        for _ in range(5):
            out = ext.int8_decode_attention_paged(Qi, Kp, Vp, sQ.reshape(-1).contiguous(), sKp, sVp, table, seq, s)
        torch.cuda.synchronize()
        print(f"profile case {name}: B{b} H{h} D{d} page {page}, lengths {lens.tolist()}, "
              f"K+V bytes per launch {2 * h * d * int(lens.sum())}, checksum {float(out.float().sum()):.4f}")
        return
    if name.startswith("prefill"):
        b, h, sq, d = PROFILE_CASES[name]
        g = torch.Generator(device="cuda").manual_seed(0)
        t = []
        for _ in range(3):
            xi, sx = ext.quantize_per_token(torch.randn(b, h, sq, d, device="cuda", dtype=torch.float16, generator=g))
            t.extend([xi, sx.reshape(-1).contiguous()])
        for _ in range(3):
            out = ext.int8_attention_forward(t[0], t[2], t[4], t[1], t[3], t[5])
        torch.cuda.synchronize()
        print(f"profile case {name}: B{b} H{h} S{sq} D{d}, ops per forward {4 * b * h * sq * sq * d}, "
              f"checksum {float(out.float().sum()):.4f}")
        return
    if name.startswith("mlp"):
        M, dm, dff = PROFILE_CASES[name]
        g = torch.Generator(device="cuda").manual_seed(0)
        xi, sx = ext.quantize_per_token(torch.randn(1, M, dm, device="cuda", dtype=torch.float16, generator=g))
        w1 = torch.randint(-127, 128, (dm, dff), dtype=torch.int8, device="cuda", generator=g)
        w2 = torch.randint(-127, 128, (dff, dm), dtype=torch.int8, device="cuda", generator=g)
        s1 = torch.rand(dff, device="cuda", generator=g) * 1e-4 + 1e-4
        s2 = torch.rand(dm, device="cuda", generator=g) * 1e-4 + 1e-4
        b1 = torch.randn(dff, device="cuda", generator=g) * 0.01
        for _ in range(4):
            out, osc = ext.int8_mlp_forward_per_channel_bias(xi, w1, w2, sx.reshape(-1).contiguous(), s1, s2, b1)
        torch.cuda.synchronize()
        print(f"profile case {name}: M{M} {dm}->{dff}->{dm}, ops per forward {4 * M * dm * dff}, "
              f"checksum {float(osc.sum()):.6f}")
        return
    b, h, d, s = PROFILE_CASES[name]
    args = make_inputs(torch, ext, b, h, s, d)
    for _ in range(5):
        out = ext.int8_decode_attention_forward(*args)
    torch.cuda.synchronize()
    print(f"profile case {name}: B{b} H{h} D{d} ctx{s}, K+V bytes per launch {kv_bytes(b, h, s, d)}, "
          f"plan {pkg.cabi.decode_plan(b * h, s, d)}, checksum {float(out.float().sum()):.4f}")


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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the sweep over the other configurations")
    ap.add_argument("--profile-case", default=None, choices=sorted(PROFILE_CASES),
                    help="run a few launches of one small case and exit (for ncu captures)")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args.profile_case)
        return
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
    if distributed:
        os.environ.setdefault("NCCL_DEBUG", "WARN")      # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    pkg = importlib.import_module("int8-transformer-kernels_b200")
    ext = pkg.int8_ext
    cabi = pkg.cabi
    lib = cabi.load()

    def barrier():
        if distributed:
            dist.barrier()

    sampler = ClockSampler(local_rank)
    Qi, Ki, Vi, sQ, sK, sV = make_inputs(torch, ext, B, H, S, D, seed=rank)
    step_bytes = kv_bytes(B, H, S, D)

    def step():
        return ext.int8_decode_attention_forward(Qi, Ki, Vi, sQ, sK, sV)

    # ---- value: K steps back to back, inputs resident ---------------------------------
    sampler.start()
    elapsed = timed_steps(torch, step, args.steps, args.warmup, barrier)
    if distributed:
        t = torch.tensor([elapsed], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed = float(t.item())
    value = world * step_bytes * args.steps / elapsed / 1e9

    # ---- roofline: the streaming kernel alone, events recorded around it -------------
    plan_warps, plan_tiles = cabi.decode_plan(B * H, S, D)
    BH = B * H
    wbytes = lib.i8tk_decode_workspace_bytes(BH, S, D)
    ws = torch.empty(wbytes, dtype=torch.uint8, device="cuda")
    out = torch.empty(B, H, D, dtype=torch.float16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    n_prof = max(args.steps, 20)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
          for _ in range(n_prof)]
    have_probe = hasattr(lib, "i8tk_decode_set_probe_events")
    kernel_s = None
    if have_probe:
        lib.i8tk_decode_set_probe_events.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        lib.i8tk_decode_set_probe_events.restype = ctypes.c_int
        for a, b_ in ev:
            # events must exist before their handles are read
            a.record(); b_.record()
        torch.cuda.synchronize()
        # back-to-back calls, as in the timed region above (a synchronise per call would time a
        # kernel that starts on an idle, clock-ramping GPU); one pair of events per call
        t_until = time.perf_counter() + 1.0
        total, count = 0.0, 0
        while count < n_prof or time.perf_counter() < t_until:
            for a, b_ in ev:
                lib.i8tk_decode_set_probe_events(a.cuda_event, b_.cuda_event)
                cabi.check(lib.i8tk_decode_attention_forward(
                    Qi.data_ptr(), Ki.data_ptr(), Vi.data_ptr(), out.data_ptr(), sQ.data_ptr(),
                    sK.data_ptr(), sV.data_ptr(), BH, S, D, ws.data_ptr(), wbytes, stream))
            lib.i8tk_decode_set_probe_events(None, None)
            torch.cuda.synchronize()
            total += sum(a.elapsed_time(b_) for a, b_ in ev) / 1e3
            count += len(ev)
        kernel_s = total / count
    clocks = sampler.stop()

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

    e2e_elapsed = timed_steps(torch, e2e_step, e2e_steps, 3, barrier)
    if distributed:
        t = torch.tensor([e2e_elapsed], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_elapsed = float(t.item())
    e2e_value = world * step_bytes * e2e_steps / e2e_elapsed / 1e9
    del host

    peak, peak_kind = measured_hbm_peak()
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": elapsed / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int8 -> int32 dot, fp32 softmax/accumulate",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_bh": world * B * H, "sharding": "(batch, head) per rank, no collective",
                   "persistent_ctas": plan_warps, "kv_tiles_per_cta": plan_tiles,
                   "l2": "inputs (1.6 GB per step) larger than L2, no flush",
                   "pct_of_8TBps": 100.0 * value / world / NOMINAL_HBM_GBS},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": e2e_steps},
        "gpu_launches": 2 * args.steps,
        "clocks": clocks,
    }
    # Duration of the scan kernel: one step is scan + merge, chained by programmatic dependent
    # launch so that the merge (2-3 us) overlaps the scan's tail; the step time of the timed
    # region is therefore an upper bound of the scan's duration, and the figure used here.
    # Events recorded around the scan alone (the probe above) serialise the merge behind it
    # and add their own gaps: that reading is kept beside it as `us_per_launch_bracketed`.
    step_s = elapsed / args.steps
    achieved = step_bytes / step_s / 1e9
    line["roofline"] = {"bound": "hbm", "kernel": "decode_partial_kernel<64>", "achieved": achieved,
                        "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                        "frac_of_8TBps": achieved / NOMINAL_HBM_GBS,
                        "algorithmic_bytes_per_launch": step_bytes,
                        "us_per_launch": step_s * 1e6,
                        "us_per_launch_bracketed": kernel_s * 1e6 if kernel_s is not None else None,
                        "traffic": None}
    if "roofline" in line:
        # DRAM traffic per launch, scaled from the ncu capture of a 201 MB case of the same
        # kernel (profiles/decode_partial_kernel_d64_B8_H12_ctx16384.md): reads are 1.0627 x
        # the K+V bytes (the fp32 scales), writes are the partial rows.
        rows_bytes = plan_warps * 2 * 4 * (D + 4) * 4
        line["roofline"]["traffic"] = int(1.0627 * step_bytes) + rows_bytes
        line["roofline"]["traffic_source"] = "scaled from an ncu capture of a 201 MB case (linear in positions)"
        line["roofline"]["timing_note"] = ("us_per_launch is the step time of the timed region (scan + the merge that "
                                           "overlaps its tail): an upper bound of the scan's duration; "
                                           "us_per_launch_bracketed has events recorded around the scan alone, which "
                                           "keeps the merge from overlapping and adds the events' own gaps")

    if rank == 0 and world == 1:
        gbs, per_iter, threads, desc = cpu_reference_rate(seconds_budget=10.0)
        line["cpu_baseline"] = {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc}

    if not args.no_extras:
        line["sweep"] = sweep(torch, ext, cabi, world, rank, barrier, dist if distributed else None)

    if rank == 0:
        print(json.dumps(line), flush=True)
    if distributed:
        dist.destroy_process_group()


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
        out.append({"workload": f"block prefill B8 H16 Dh64 d_ff4096 S{S}", "int8_ms": t8 * 1e3, "fp16_ms": t16 * 1e3,
                    "speedup_vs_fp16": t16 / t8, "cos_vs_fp16": c})
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

            def prepacked():
                cabi.check(lib.i8tk_mlp_forward(xi.data_ptr(), W1T.data_ptr(), W2T.data_ptr(), o.data_ptr(),
                                                sxf.data_ptr(), s1.data_ptr(), s2.data_ptr(), b1.data_ptr(),
                                                osc.data_ptr(), None, M, dm, dff, flags, ws.data_ptr(), wb, st))

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
