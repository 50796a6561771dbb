"""Benchmark of the dense hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline workload (N = 1): the fp16 matmul A[8192,8192] @ B[8192,8192] -> fp16 C with fp32
accumulation, inputs ~ N(0,1)/sqrt(8192), seeded.  One "step" is one matmul.  `value` is
whole-job TFLOP/s (2*M*N*K per step, python/tutorials/03-matrix-multiplication.py:437) with the
operands resident in HBM; `e2e` is the same metric through the public API with HOST buffers
(pinned), host->device copies of A and B and the device->host copy of C inside the timed
region.  With N > 1 (one process per GPU under torchrun) every rank runs the same per-GPU
workload on its own M-row block of a taller A (weak scaling, no data-path collective); the time
is the max over ranks.  The other four configurations of the path are timed briefly and
reported under "configs" for context.

--impl reference times the CPU oracle (the numpy restatement of the reference's kernels; the
reference's own CPU path is the Triton interpreter executing the same arithmetic) on the host
cores, on a bounded sample of the same workload.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)

M = N = K = 8192
METRIC = "matmul fp16 8192^3 TFLOP/s (fp32 accumulate)"
WORKLOAD = "dense GEMM fp16 A[8192,8192]@B[8192,8192] row-major, fp32 accumulate, fp16 output (config 2)"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(burst=d["bf16_tflops"], sustained=d["bf16_tflops_sustained"], hbm=d["hbm_gbs"], source="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """SM clock, power and throttle reasons of one GPU, read (never set) through NVML every few
    milliseconds by a thread; summarised over the samples inside the timed region (mark() brackets it)."""

    def __init__(self, index):
        self.index, self.rows, self.t0, self.t1 = index, [], None, None
        self.stop_flag = threading.Event()
        self.thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception as e:  # NVML missing: report that instead of clocks
            self.nv, self.err = None, repr(e)

    def mark(self):
        if self.t0 is None:
            self.t0 = time.time()
        else:
            self.t1 = time.time()

    def _poll(self):
        nv = self.nv
        while not self.stop_flag.is_set():
            try:
                sm = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                pw = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                try:
                    rs = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    rs = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.rows.append((time.time(), sm, pw, rs))
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self.nv:
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()

    def stop(self):
        if not self.nv:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["NVML unavailable: " + self.err])
        self.stop_flag.set()
        self.thread.join(timeout=2)
        nv = self.nv
        inside = [r for r in self.rows if self.t0 and self.t1 and self.t0 <= r[0] <= self.t1]
        rows = inside if inside else self.rows
        bits = 0
        for r in rows:
            bits |= r[3]
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40,
                 "sw_thermal_slowdown": 0x20, "hw_power_brake_slowdown": 0x80}
        reasons = sorted(k for k, v in names.items() if bits & v)
        sm = [r[1] for r in rows]
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_min_mhz=min(sm) if sm else None,
                    sm_max_mhz=self.max_sm, power_w_max=max(r[2] for r in rows) if rows else None,
                    samples=len(rows), window="timed region" if inside else "whole run", reasons=reasons)


def cpu_threads():
    try:
        from threadpoolctl import threadpool_info
        n = [i.get("num_threads", 1) for i in threadpool_info() if i.get("user_api") == "blas"]
        return max(n) if n else (os.cpu_count() or 1)
    except Exception:
        return os.cpu_count() or 1


def oracle_sample_inputs(rows):
    import numpy as np
    rs = np.random.RandomState(2024)
    a = (rs.standard_normal((rows, K)) / K ** 0.5).astype(np.float16).astype(np.float32)
    b = (rs.standard_normal((K, N)) / K ** 0.5).astype(np.float16).astype(np.float32)
    return a, b


def time_oracle(rows, reps=1):
    """TFLOP/s of the CPU oracle on `rows` rows of A against all of B (full K, full N)."""
    from oracle import ref_ops as R
    a, b = oracle_sample_inputs(rows)
    t0 = time.perf_counter()
    for _ in range(reps):
        R.matmul(a, b)
    dt = (time.perf_counter() - t0) / reps
    return 2.0 * rows * N * K / dt / 1e12, dt


def use_all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU arm is meant to use every core."""
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=os.cpu_count() or 1)
    except Exception:
        pass


def run_reference(args, rank, world):
    if rank != 0:
        return
    use_all_host_threads()
    # size the per-step sample so that the whole run stays within a few minutes
    _, probe = time_oracle(128)
    budget = 150.0 / max(1, args.steps + args.warmup)
    rows = int(min(M, max(128, (budget / probe) * 128 // 128 * 128)))
    for _ in range(args.warmup):
        time_oracle(rows)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        time_oracle(rows)
    dt = time.perf_counter() - t0
    val = 2.0 * rows * N * K * args.steps / dt / 1e12
    sample = f"{rows} of {M} rows of A against all of B per step (full K and N), numpy/BLAS tile loop"
    cores = cpu_threads()
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def device_time(fn, steps, warmup, torch, barrier=None, mark=None):
    """ms for `steps` back-to-back calls of fn (CUDA events on the current stream)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    if mark:
        mark()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if mark:
        mark()
    if barrier:
        barrier()
    return e0.elapsed_time(e1)


def other_configs(torch, tb, dev):
    """Short timings of configs 1, 3, 4, 5 (TFLOP/s by the reference's FLOP conventions)."""
    import cases
    out = {}
    g = torch.Generator().manual_seed(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn, flops, reps=10):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(reps):
            flush.zero_()  # inputs of these configs can fit in L2: flush between repetitions
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ms = statistics.median(ts)
        return {"ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1)}

    a = torch.randn(512, 512, generator=g).half().to(dev)
    b = torch.randn(512, 512, generator=g).half().to(dev)
    out["c1_matmul_fp16_512"] = timed(lambda: tb.matmul(a, b), 2.0 * 512 ** 3)
    a8, sa = tb.quantize_e4m3(torch.randn(M, K, generator=g).to(dev))
    b8, sb = tb.quantize_e4m3(torch.randn(K, N, generator=g).to(dev))
    out["c3_matmul_fp8_8192_scaled_bf16"] = timed(lambda: tb.matmul(a8, b8, scale_a=sa, scale_b=sb), 2.0 * M * N * K)
    del a8, b8
    q, k, v, _ = (t.to(dev) for t in cases.attn_inputs(dict(Z=4, H=32, N=4096, D=128, dtype="fp16", seed=20)))
    fl = 2 * 2.0 * 4 * 32 * 4096 * 4096 * 128 * 0.5
    out["c4_attn_fwd_causal_fp16_z4h32n4096d128"] = timed(lambda: tb.attention_forward(q, k, v, True, 128 ** -0.5), fl)
    q, k, v, do = (t.to(dev) for t in cases.attn_inputs(dict(Z=4, H=48, N=1024, D=64, dtype="bf16", seed=20)))
    fl = 2 * 2.0 * 4 * 48 * 1024 * 1024 * 64 * 0.5
    o, Mst = tb.attention_forward(q, k, v, True, 0.5)

    def fwd_bwd():
        o_, m_ = tb.attention_forward(q, k, v, True, 0.5)
        tb.attention_backward(q, k, v, o_, m_, do, True, 0.5)

    out["c5_attn_fwd_bwd_causal_bf16_z4h48n1024d64"] = timed(fwd_bwd, fl * 3.5)
    out["c5_fwd_only"] = timed(lambda: tb.attention_forward(q, k, v, True, 0.5), fl)
    out["c5_bwd_only"] = timed(lambda: tb.attention_backward(q, k, v, o, Mst, do, True, 0.5), fl * 2.5)
    del q, k, v, do, o, Mst
    # rows beyond the five configs: the widened matmul / attention entry points
    ga = [torch.rand(512, 512, generator=g).half().to(dev) for _ in range(64)]
    gb = [torch.rand(512, 512, generator=g).half().to(dev) for _ in range(64)]
    plan = tb.GroupedMatmul(ga, gb)
    out["grouped_matmul_fp16_64x512_prepared"] = timed(plan.run, 64 * 2.0 * 512 ** 3)
    a = (torch.randn(256, 8192, generator=g) / 90).half().to(dev)
    b = (torch.randn(8192, 256, generator=g) / 90).half().to(dev)
    out["splitk_matmul_fp16_256x256x8192"] = timed(lambda: tb.matmul(a, b), 2.0 * 256 * 256 * 8192)
    if hasattr(torch, "float8_e5m2"):
        q8, k8, v8 = ((torch.randn(4, 32, 4096, 128, generator=g) * 0.5).to(dev).to(torch.float8_e5m2) for _ in range(3))
        v8 = v8.permute(0, 1, 3, 2).contiguous().permute(0, 1, 3, 2)
        fl = 2 * 2.0 * 4 * 32 * 4096 * 4096 * 128 * 0.5
        out["attn_fwd_causal_e5m2_z4h32n4096d128"] = timed(lambda: tb.attention_forward(q8, k8, v8, True, 1.3), fl)
    return out


def run_profile_case(name):
    """A few launches of one configuration's kernels and nothing else: the command line that the
    ncu captures summarised under profiles/ were taken with (python bench.py --profile c4 ...)."""
    import torch
    import cases
    import triton_b200 as tb
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(0)
    if name == "c2":
        a = (torch.randn(M, K, generator=g) / K ** 0.5).half().to(dev)
        b = (torch.randn(K, N, generator=g) / K ** 0.5).half().to(dev)
        fn = lambda: tb.matmul(a, b)
    elif name == "c3":
        a8, sa = tb.quantize_e4m3(torch.randn(M, K, generator=g).to(dev))
        b8, sb = tb.quantize_e4m3(torch.randn(K, N, generator=g).to(dev))
        fn = lambda: tb.matmul(a8, b8, scale_a=sa, scale_b=sb)
    elif name == "c4":
        q, k, v, _ = (t.to(dev) for t in cases.attn_inputs(dict(Z=4, H=32, N=4096, D=128, dtype="fp16", seed=20)))
        fn = lambda: tb.attention_forward(q, k, v, True, 128 ** -0.5)
    elif name == "c5":
        q, k, v, do = (t.to(dev) for t in cases.attn_inputs(dict(Z=4, H=48, N=1024, D=64, dtype="bf16", seed=20)))

        def fn():
            o, m = tb.attention_forward(q, k, v, True, 0.5)
            tb.attention_backward(q, k, v, o, m, do, True, 0.5)
    elif name == "fp8attn":  # the 8-bit forward on config 4's shape (the reference's fp8 benchmark scale 1.3)
        q, k, v = ((torch.randn(4, 32, 4096, 128, generator=g) * 0.5).to(dev).to(torch.float8_e5m2) for _ in range(3))
        v = v.permute(0, 1, 3, 2).contiguous().permute(0, 1, 3, 2)
        fn = lambda: tb.attention_forward(q, k, v, True, 1.3)
    elif name == "grouped":  # 64 problems of 512^3 in one launch
        ga = [torch.rand(512, 512, generator=g).half().to(dev) for _ in range(64)]
        gb = [torch.rand(512, 512, generator=g).half().to(dev) for _ in range(64)]
        fn = lambda: tb.group_gemm_fn(ga, gb)
    elif name == "skinny":  # split-K: 256 x 256 x 8192
        a = (torch.randn(256, 8192, generator=g) / 90).half().to(dev)
        b = (torch.randn(8192, 256, generator=g) / 90).half().to(dev)
        fn = lambda: tb.matmul(a, b)
    else:
        raise SystemExit("unknown profile case " + name)
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    print("profile case", name, "done")


def run_ours(args, rank, local_rank, world):
    import torch
    import triton_b200 as tb
    from triton_b200 import _lib

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    barrier = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        barrier = lambda: dist.barrier()

    g = torch.Generator().manual_seed(2024 + rank)  # rank r holds rows [r*M, (r+1)*M) of a taller A
    a_h = (torch.randn(M, K, generator=g) / K ** 0.5).half().pin_memory()
    gb = torch.Generator().manual_seed(7)
    b_h = (torch.randn(K, N, generator=gb) / K ** 0.5).half().pin_memory()  # B is the same on every rank
    c_h = torch.empty(M, N, dtype=torch.float16).pin_memory()
    a, b = a_h.to(dev), b_h.to(dev)
    c = torch.empty(M, N, dtype=torch.float16, device=dev)
    step = lambda: tb.matmul(a, b, out=c, out_dtype=torch.float16)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms = device_time(step, args.steps, args.warmup, torch, barrier, sampler.mark if rank == 0 else None)
    clocks = sampler.stop() if rank == 0 else None
    if _lib.status() != 0:
        raise RuntimeError("a bounded device-side wait ran out during the benchmark")

    # end to end through the public API from host buffers
    e2e_steps = max(1, min(args.steps, 10))

    # HostMatmul: pinned host A, B -> device (A in row blocks), matmul per block, C blocks -> pinned
    # host, the three overlapped on two copy streams; every step moves all of A, B and C
    host_mm = tb.HostMatmul(M, N, K, torch.float16, dev)

    def e2e_step():
        host_mm.run(a_h, b_h, c_h)

    ms_e2e = device_time(e2e_step, e2e_steps, 1, torch, barrier)
    if not torch.allclose(c_h[:64].float(), c[:64].cpu().float(), rtol=1e-2, atol=1e-2):
        raise RuntimeError("end-to-end result differs from the device-resident result")

    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms, ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])

    flops = 2.0 * M * N * K
    value = world * flops * args.steps / ms / 1e9
    e2e_value = world * flops * e2e_steps / ms_e2e / 1e9
    if rank == 0:
        pk = peaks()
        per_launch_ms = ms / args.steps
        achieved = flops / per_launch_ms / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": per_launch_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "per_gpu": "one 8192^3 matmul per step on the rank's own M-row block",
                       "l2": "inputs and output (384 MiB per step) exceed the 126 MB L2; no flush needed",
                       "tile": os.environ.get("B200_GEMM_TILE", "auto")},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": 2 * M * K * 2,
                    "d2h_bytes_per_step": M * N * 2, "steps": e2e_steps},
            "gpu_launches": args.steps,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": pk["sustained"], "unit": "TFLOP/s",
                         "frac": achieved / pk["sustained"], "peak_kind": f"{pk['source']} cuBLAS bf16, sustained",
                         "frac_of_burst_peak": achieved / pk["burst"],
                         "frac_of_nominal_2250": achieved / 2250.0,
                         # dram__bytes_read.sum + dram__bytes_write.sum of one launch (ncu capture of this
                         # workload, summarised in profiles/gemm_fp16_8192.md)
                         "traffic": TRAFFIC_BYTES_PER_LAUNCH},
        }
        if world == 1:
            use_all_host_threads()
            rows = 2048
            v, dt = time_oracle(rows)
            line["cpu_baseline"] = {"value": v, "unit": "TFLOP/s", "cores": cpu_threads(), "kind": "port",
                                    "sample": f"{rows} of {M} rows of A against all of B (full K, N): {dt:.1f} s of "
                                              "the numpy/BLAS restatement of the reference's tile loop"}
            if not args.no_extra:
                line["configs"] = other_configs(torch, tb, dev)
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one gemm_kernel<256,256,3> launch on this workload
# (879.5 MB + 120.0 MB, ncu --set full capture summarised in profiles/gemm_fp16_8192.md); algorithmic: 402.7 MB
TRAFFIC_BYTES_PER_LAUNCH = 999_518_208


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the short timings of configs 1, 3, 4, 5")
    ap.add_argument("--profile", default=None, choices=["c2", "c3", "c4", "c5", "fp8attn", "grouped", "skinny"],
                    help="run three launches of one configuration and exit (for ncu captures)")
    args = ap.parse_args()
    # torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU arm and the cpu_baseline leg are meant to
    # use every host core, and BLAS reads the variable when numpy is first imported (below, lazily)
    for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[var] = str(os.cpu_count() or 1)
    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.profile:
        run_profile_case(args.profile)
    elif args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
