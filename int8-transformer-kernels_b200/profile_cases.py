#!/usr/bin/env python
"""Small, self-contained cases of each kernel for profiler captures.

    python int8-transformer-kernels_b200/profile_cases.py <case>

Each case builds seeded inputs on the device, launches the op a handful of times and prints
what it ran (shape, algorithmic bytes or operations per launch, a checksum).  The sizes follow
the rule for captures on a shared GPU: larger than the 126 MB L2 where DRAM counters are to
mean something, a few hundred MB on the device at most, a few launches -- so a capture of one
to three launches ends by itself in a minute or two.  Nothing here is timed; run the case
plainly first and under the profiler only after it has exited 0.
"""
import importlib
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))


def kv_bytes(b, h, s, d):
    return 2 * b * h * s * d


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



PROFILE_CASES = {
    "decode_d64": (8, 12, 64, 16384),      # 201 MB of int8 K+V
    "decode_d128": (8, 8, 128, 8192),      # 134 MB
    "decode_d64_ctx4096": (32, 12, 64, 4096),   # the short end of the serving sweep: 201 MB, 28 tiles per CTA
    "decode_d64_cfg0": (1, 12, 64, 1024),  # one request: a thread-block cluster per (b,h) row, no merge kernel
    "mlp_m512_768": (512, 768, 3072),      # the reference's own benchmark shape: latency, not throughput
    "mlp_m4096_768": (4096, 768, 3072),    # fused MLP forward (L2 resident by nature: 30 MB of operands)
    "mlp_m4096_1024": (4096, 1024, 4096),
    "mlp_m16384_1024": (16384, 1024, 4096),   # several rounds of the persistent loop per CTA
    "quantize_f32_64": (3145728, 64),      # rows, cols: 1.0 GB through the per-token quantiser
    "prefill_d64": (2, 8, 4096, 64),       # B, H, S, D: 512 CTAs of 128 query rows
    "prefill_d128": (2, 8, 4096, 128),
    "prefill_d256": (2, 8, 2048, 256),     # 64-position KV tiles
    "paged_d64_p64": (8, 12, 64, 16384, 64),   # B, H, D, longest request, page: lengths 2048..16384, shuffled table
    "paged_d64_p16": (8, 12, 64, 16384, 16),   # the same on 16-position pages: 1 KB bulk copies
    "lnquant_f16_1024": (131072, 1024),    # rows, cols: 268 MB in, 134 MB of codes out
}


def run_profile_case(name):
    import torch
    pkg = importlib.import_module(os.path.basename(HERE))
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



if __name__ == "__main__":
    if len(sys.argv) != 2 or sys.argv[1] not in PROFILE_CASES:
        sys.exit("usage: profile_cases.py <%s>" % "|".join(sorted(PROFILE_CASES)))
    run_profile_case(sys.argv[1])
