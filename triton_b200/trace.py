"""Device-side clock trace of the attention kernels.

    python -m triton_b200.trace fwd [--case c4|c5|noncausal|e5m2]
    python -m triton_b200.trace bwd [--case c5|long]        (the two-kernel backward)
    python -m triton_b200.trace bwd1 [--case c5|long]       (the one-pass backward, head dim 64)
    python -m triton_b200.trace gemm [--case c2|c3]         (the 256 x 256 matmul tile, 8192^3)

Builds the instrumented variant of the library (`-DB200_TRACE`, libtriton_b200_trace.so beside the
production one), runs a few launches of one configuration through the normal Python wrappers and
prints, for the traced warps of CTA 0, the mean number of SM clocks between consecutive trace
points.  The instrumentation costs roughly 100 clocks per point, so the figures are for reading
proportions, not for benchmarking; the production library contains none of it.
"""
import argparse
import ctypes
import os
import sys

_PKG = os.path.dirname(os.path.abspath(__file__))
REGIONS, EVENTS = 4, 4096  # kTraceRegions, kTraceEvents of csrc/trace.h

FWD_TAGS = {1: "wait for S (MMA of this tile + hand-over)", 2: "TMEM load + row maximum", 3: "rescale decision (+ O rescale)",
            4: "exp2, pack, P store, arrive", 8: "epilogue: wait for the tile's last P V (o_full)",
            0xA: "epilogue: TMEM load of 64 columns of O", 0xB: "epilogue: previous store has read the staging buffer",
            0xC: "epilogue: scale, pack, staging write, fence", 9: "epilogue: last store issued, M written"}
FWD_MMA = {0x10: "P V issued / before the wait for P", 0x20: "P arrived", 0x40: "S issued",
           0x50: "tile 1's S issued; before the wait for V", 0x60: "V arrived"}
ONE_TAGS = {1: "wait for T1 (scores)", 2: "TMEM load, exp2, P store, arrive", 3: "wait for T2 (dP)",
            5: "dS, TMEM store", 6: "wait for the shared-memory dS tile (previous dQ MMAs)",
            4: "shared-memory dS write, proxy fence, arrive"}
ONE_MMA = {0x10: "dQ / T2 issued; before the wait for P", 0x20: "P arrived", 0x30: "dV, next T1 issued; before the wait for dS",
           0x40: "dS arrived", 0x50: "dK issued, previous dQ partial drained"}
ONE_DRAIN = {7: "wait for a dQ partial", 8: "TMEM load, staging write, reduce-add issue"}
GEMM_TMA = {1: "stage filled (loads issued); before the wait for a free stage", 2: "a stage is free"}
GEMM_MMA = {1: "4 MMAs + commit issued; before the wait for the next K block", 2: "K block landed (full)",
            0x10: "tile done; before the wait for the accumulator to drain", 0x20: "accumulator free (tmem_empty)"}
GEMM_EPI = {1: "tile stored; before the wait for the next accumulator", 2: "accumulator complete (tmem_full)", 3: "accumulator drained, stores issued"}
BWD_TAGS = {1: "wait for T1 (scores)", 2: "TMEM load, exp2, P store, arrive", 3: "wait for T2 (dP)",
            4: "dS, store, arrive", 8: "wait for the last accumulate (acc_full)", 9: "epilogue (gradient stores)"}


def _summarise(ev, names, item_tag=0x100):
    """mean clocks from the previous trace point to each tagged point; ev: [(tag, clock)]"""
    import collections
    tot, cnt = collections.OrderedDict(), collections.Counter()
    prev = None
    for tag, clk in ev:
        if tag == 0 and clk == 0:
            break
        if prev is not None:
            key = "item start (scheduler, next item)" if tag >= item_tag else names.get(tag, names.get(tag & 0xF0, hex(tag)))
            tot[key] = tot.get(key, 0) + ((clk - prev) & 0xFFFFFFFF)
            cnt[key] += 1
        prev = clk
    return [(k, cnt[k], tot[k] / cnt[k]) for k in tot]


def trace_gemm(case, lib):
    import numpy as np
    import torch
    import triton_b200 as tb
    from triton_b200 import _lib
    L = _lib.lib()
    L.b200_trace_read.argtypes = [ctypes.c_void_p, ctypes.c_size_t]
    buf = np.zeros((REGIONS, EVENTS, 2), dtype=np.uint32)
    g = torch.Generator(device="cuda").manual_seed(0)
    n = {"c1": 512, "n1024": 1024, "n2048": 2048}.get(case, 8192)
    a = (torch.randn(n, n, generator=g, device="cuda") / n ** 0.5).half()
    b = (torch.randn(n, n, generator=g, device="cuda") / n ** 0.5).half()
    if case == "c3":
        a, sa = tb.quantize_e4m3(a.float() * n ** 0.5)
        b, sb = tb.quantize_e4m3(b.float() * n ** 0.5)
        fn = lambda: tb.matmul(a, b, scale_a=sa, scale_b=sb)
    else:
        fn = lambda: tb.matmul(a, b)
    for _ in range(2):
        fn()
        _lib.check(L.b200_trace_read(ctypes.c_void_p(buf.ctypes.data), buf.nbytes), "trace_read")
    t = buf.copy()
    if os.environ.get("B200_TRACE_RAW"):  # the timeline itself (small cases): clocks since the CTA's first event
        firsts = [int(t[r][0][1]) for r in range(REGIONS) if t[r][0][0] or t[r][0][1]]
        t_min = min(firsts) if firsts else 0
        for region in range(REGIONS):
            ev = [(int(tag), (int(clk) - t_min) & 0xFFFFFFFF) for tag, clk in t[region].tolist() if tag or clk][:48]
            print(f"  region {region}: " + " ".join(f"{tag:x}@{clk}" for tag, clk in ev))
    print(f"gemm {case} {n}^3: CTA 0, mean SM clocks since the previous trace point")
    for region, label, names in ((0, "TMA warp", GEMM_TMA), (1, "issuing warp, rows 0-127", GEMM_MMA),
                                 (2, "issuing warp, rows 128-255", GEMM_MMA), (3, "epilogue warp 0", GEMM_EPI)):
        print(f"  {label}")
        for key, cnt, mean in _summarise(t[region].tolist(), names, item_tag=1 << 30):
            print(f"    {key:72s} n={cnt:5d}  {mean:8.0f} clk")
    st = _lib.status()
    print("status word", hex(st))
    return 0 if st == 0 else 1


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["fwd", "bwd", "bwd1", "gemm"])
    ap.add_argument("--case", default=None)
    args = ap.parse_args()
    from . import build
    lib = build.build(trace=True)
    os.environ["TRITON_B200_LIB"] = lib
    import numpy as np
    import torch
    import triton_b200 as tb
    from triton_b200 import _lib
    assert _lib._lib is None, "the library was loaded before the trace build was selected"
    if args.kernel == "gemm":
        return trace_gemm(args.case or "c2", lib)
    case = args.case or ("c4" if args.kernel == "fwd" else "c5")
    if case == "c4" and args.kernel != "fwd":
        raise SystemExit("the backward traces take --case c5 or long")
    Z, H, N, D, dt, causal, sm = {"c4": (4, 32, 4096, 128, torch.float16, True, 128 ** -0.5),
                                  "noncausal": (4, 32, 4096, 128, torch.float16, False, 128 ** -0.5),
                                  "c5": (4, 48, 1024, 64, torch.bfloat16, True, 0.5),
                                  "long": (4, 48, 4096, 64, torch.bfloat16, True, 0.5),
                                  "e5m2": (4, 32, 4096, 128, torch.float8_e5m2, True, 1.3)}[case]
    g = torch.Generator(device="cuda").manual_seed(0)
    q, k, v, do = ((torch.randn(Z, H, N, D, generator=g, device="cuda") * 0.5).to(dt) for _ in range(4))
    if case == "e5m2":  # the 8-bit forward reads V with the key dimension contiguous
        v = v.permute(0, 1, 3, 2).contiguous().permute(0, 1, 3, 2)
    L = _lib.lib()
    L.b200_trace_read.argtypes = [ctypes.c_void_p, ctypes.c_size_t]
    buf = np.zeros((REGIONS, EVENTS, 2), dtype=np.uint32)

    def read():
        _lib.check(L.b200_trace_read(ctypes.c_void_p(buf.ctypes.data), buf.nbytes), "trace_read")
        return buf.copy()

    o, M = tb.attention_forward(q, k, v, causal, sm)
    one = args.kernel == "bwd1"
    if args.kernel != "fwd":
        tb.attention_backward(q, k, v, o, M, do, causal, sm, one_pass=one)
    read()  # discard the first (cold) launch
    if args.kernel == "fwd":
        tb.attention_forward(q, k, v, causal, sm)
    else:
        tb.attention_backward(q, k, v, o, M, do, causal, sm, one_pass=one)
    t = read()
    print(f"{args.kernel} Z{Z} H{H} N{N} D{D} causal={causal}: CTA 0, mean SM clocks since the previous trace point")
    if args.kernel == "fwd" and os.environ.get("B200_TRACE_RAW"):  # the timeline itself: clocks since the CTA's first event
        firsts = [int(t[r][0][1]) for r in range(REGIONS) if t[r][0][0] or t[r][0][1]]
        t_min = min(firsts) if firsts else 0
        for region in (0, 1, 2):
            ev = [(int(tag), (int(clk) - t_min) & 0xFFFFFFFF) for tag, clk in t[region].tolist() if tag or clk][:int(os.environ["B200_TRACE_RAW"])]
            print(f"  region {region}: " + " ".join(f"{tag:x}@{clk}" for tag, clk in ev))
    if args.kernel == "fwd":
        for region, label in ((0, "softmax warp 0 of tile 0"), (1, "softmax warp 0 of tile 1")):
            print(f"  {label}")
            for key, n, mean in _summarise(t[region].tolist(), FWD_TAGS):
                print(f"    {key:56s} n={n:5d}  {mean:8.0f} clk")
        print("  MMA warp")
        for key, n, mean in _summarise(t[2].tolist(), FWD_MMA):
            print(f"    {key:48s} n={n:5d}  {mean:8.0f} clk")
    elif one:
        if os.environ.get("B200_TRACE_RAW"):  # the timeline itself: clocks since the CTA's first event
            firsts = [int(t[r][0][1]) for r in range(REGIONS) if t[r][0][0] or t[r][0][1]]
            t_min = min(firsts) if firsts else 0
            for region in (0, 2, 3):
                ev = [(int(tag), (int(clk) - t_min) & 0xFFFFFFFF) for tag, clk in t[region].tolist() if tag or clk][:int(os.environ["B200_TRACE_RAW"])]
                print(f"  region {region}: " + " ".join(f"{tag:x}@{clk}" for tag, clk in ev))
        for region, label, names in ((0, "compute warp 0", ONE_TAGS), (2, "MMA warp", ONE_MMA), (3, "drain warp 0", ONE_DRAIN)):
            print(f"  {label}")
            for key, n, mean in _summarise(t[region].tolist(), names):
                print(f"    {key:56s} n={n:5d}  {mean:8.0f} clk")
    else:
        for region, label in ((0, "dK/dV kernel, compute warp 0"), (1, "dQ kernel, compute warp 0")):
            print(f"  {label}")
            for key, n, mean in _summarise(t[region].tolist(), BWD_TAGS):
                print(f"    {key:48s} n={n:5d}  {mean:8.0f} clk")
    st = _lib.status()
    print("status word", hex(st))
    return 0 if st == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
