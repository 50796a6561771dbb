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

--impl reference times the reference's CPU path on the host cores: the Triton interpreter
(TRITON_INTERPRET=1, the pip `triton` package as executor) running the matmul tile program
(oracle/interp_matmul.py, the reference kernel's algorithm restated in its own kernel language;
the reference checkout itself does not exist on the GPU box) at the largest shape that fits the
time budget; the numpy restatement of the same tile loop is timed beside it.
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


PORT_ROWS = 2048  # rows of A in the numpy port's sample (every leg that times the port uses this sample)


def port_baseline():
    """The numpy restatement of the reference's tile loop on PORT_ROWS rows of A against all of B."""
    use_all_host_threads()
    time_oracle(128)  # BLAS thread pool and page faults out of the way
    v, dt = time_oracle(PORT_ROWS)
    return {"value": v, "unit": "TFLOP/s", "cores": cpu_threads(), "kind": "port",
            "sample": f"{PORT_ROWS} of {M} rows of A against all of B (full K, N): {dt:.1f} s of the numpy/BLAS "
                      "restatement of the reference's tile loop"}


INTERP_SHAPES = [(512, 512, 512), (1024, 1024, 1024), (1536, 1536, 1536), (2048, 2048, 2048)]


def time_interpreter(shape, repeats=1, timeout=600):
    """One launch of the matmul tile program under the Triton interpreter, in a subprocess (the
    interpreter is selected by an environment variable read when `triton` is imported).  Returns
    the subprocess's JSON record, or {"unavailable": reason}."""
    import subprocess
    env = dict(os.environ, TRITON_INTERPRET="1")
    for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        env[var] = str(os.cpu_count() or 1)
    cmd = [sys.executable, "-m", "oracle.interp_matmul", *map(str, shape), str(repeats)]
    try:
        r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"interpreter run of {shape} exceeded {timeout} s"}
    if r.returncode != 0:
        return {"unavailable": "interpreter run failed: " + (r.stderr.strip().splitlines() or ["?"])[-1][:200]}
    return json.loads(r.stdout.strip().splitlines()[-1])


def interpreter_baseline(budget_s=60.0):
    """The interpreter at the largest shape of INTERP_SHAPES whose run fits `budget_s` (estimated
    from the next smaller shape: the cost grows with tiles x K-steps)."""
    best = time_interpreter(INTERP_SHAPES[0])
    if "unavailable" in best:
        return {"kind": "interpreter", "value": None, "unit": "TFLOP/s", "cores": os.cpu_count(),
                "unavailable": best["unavailable"]}
    for shape in INTERP_SHAPES[1:]:
        grow = (shape[0] * shape[1] * shape[2]) / (best["M"] * best["N"] * best["K"])
        if best["seconds"] * grow > budget_s:
            break
        rec = time_interpreter(shape)
        if "unavailable" in rec:
            break
        best = rec
    return {"value": best["tflops"], "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "interpreter",
            "sample": f"one launch of the 128x256x64 tile program at {best['M']}x{best['N']}x{best['K']} fp16 under "
                      f"TRITON_INTERPRET=1 (triton {best['triton']} as executor): {best['seconds']:.1f} s; the program "
                      "loop is single-threaded Python, numpy's BLAS may use every core inside a tile product",
            "shape": [best["M"], best["N"], best["K"]], "seconds": best["seconds"]}


def run_reference(args, rank, world):
    if rank != 0:
        return
    # one step = one interpreter launch at the largest shape that keeps the whole run within a few minutes
    per_step = 150.0 / max(1, args.steps + args.warmup)
    probe = time_interpreter(INTERP_SHAPES[0])
    line = {"impl": "reference", "metric": METRIC, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16",
            "data": "synthetic"}
    if "unavailable" in probe:
        # the interpreter cannot run here: the numpy restatement of the same tile loop stands in
        port = port_baseline()
        line.update(value=port["value"], ms_per_step=None, config={"workload": WORKLOAD, "sample": port["sample"]},
                    cpu_baseline=dict(port, interpreter_unavailable=probe["unavailable"]),
                    e2e={"value": port["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
        print(json.dumps(line))
        return
    shape = INTERP_SHAPES[0]
    for cand in INTERP_SHAPES[1:]:
        grow = (cand[0] * cand[1] * cand[2]) / (probe["M"] * probe["N"] * probe["K"])
        if probe["seconds"] * grow <= per_step:
            shape = cand
    rec = time_interpreter(shape, repeats=args.warmup + args.steps) if args.warmup + args.steps > 1 else probe
    # (the subprocess repeats warm-up + timed launches back to back and reports the mean per launch)
    val = rec["tflops"]
    sample = (f"one launch of the reference's matmul tile program (128x256x64 tiles) at {shape[0]}x{shape[1]}x{shape[2]} "
              f"fp16 per step under the Triton interpreter (TRITON_INTERPRET=1, triton {rec['triton']}), the largest of "
              f"{INTERP_SHAPES} that keeps {args.steps}+{args.warmup} steps within 150 s")
    port = port_baseline()
    line.update(value=val, ms_per_step=rec["seconds"] * 1e3,
                config={"workload": WORKLOAD, "sample": sample},
                cpu_baseline={"value": val, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "interpreter",
                              "sample": sample, "port": port},
                e2e={"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
    print(json.dumps(line))


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

    def timed(fn, flops, reps=10, graph=False):
        """median of `reps` L2-flushed launches; graph=True replays a CUDA graph of fn (the reference
        times attention with do_bench_cudagraph, python/triton/testing.py:19-81: for launches of a few
        tens of microseconds the host side of an eager launch is part of what CUDA events see)"""
        # Every one of these short timings starts from an idle GPU: right after a heavy configuration
        # (a 8192^3 matmul loop, the head-dim-128 forward) the chip stays throttled for a moment and the
        # next, lighter kernel measures 30-60 % slow; 0.2 s of idle is enough to be back (measured).
        torch.cuda.synchronize()
        time.sleep(0.25)
        for _ in range(3):
            fn()
        run = fn
        if graph:
            torch.cuda.synchronize()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            cg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(cg, stream=side):
                fn()
            torch.cuda.current_stream().wait_stream(side)
            run = cg.replay
            run()
        ts = []
        for _ in range(reps):
            flush.zero_()  # inputs of these configs can fit in L2: flush between repetitions
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            run()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ms = statistics.median(ts)
        return {"ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1)}

    def timed_unrolled(fn, flops, rep_ms=20.0, max_repeat=200):
        """the reference's do_bench_cudagraph recipe (python/triton/testing.py:19-81): one CUDA graph of
        n_repeat = rep_ms / estimate unrolled calls (capped at max_repeat here), no cache flush between
        them, mean of 10 replays; what its attention benchmark and autotuner time with"""
        torch.cuda.synchronize()
        time.sleep(0.25)  # as in timed(): start from an idle GPU
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        side = torch.cuda.Stream()

        def capture(n):
            side.wait_stream(torch.cuda.current_stream())
            cg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(cg, stream=side):
                for _ in range(n):
                    fn()
            torch.cuda.current_stream().wait_stream(side)
            return cg

        def replay_ms(cg):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            cg.replay()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1)

        one = capture(1)
        replay_ms(one)
        n = max(1, min(max_repeat, int(rep_ms / max(replay_ms(one), 1e-4))))
        cg = capture(n)
        ms = statistics.mean(replay_ms(cg) / n for _ in range(10))
        return {"ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1), "n_repeat": n}

    a = torch.randn(512, 512, generator=g).half().to(dev)
    b = torch.randn(512, 512, generator=g).half().to(dev)
    out["c1_matmul_fp16_512"] = timed(lambda: tb.matmul(a, b), 2.0 * 512 ** 3)
    out["c1_matmul_fp16_512_cudagraph"] = timed(lambda: tb.matmul(a, b), 2.0 * 512 ** 3, graph=True)
    out["c1_matmul_fp16_512_do_bench_cudagraph"] = timed_unrolled(lambda: tb.matmul(a, b), 2.0 * 512 ** 3)
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

    # config 5's backward runs as ONE pass (partial dQ per K/V block summed into an fp32 buffer: the
    # reference's `sequence_parallel` layout, attention(..., sequence_parallel=True)); the two-kernel
    # backward of the reference's current layout (bitwise repeatable, the library's default) beside it
    def fwd_bwd(one_pass):
        o_, m_ = tb.attention_forward(q, k, v, True, 0.5)
        tb.attention_backward(q, k, v, o_, m_, do, True, 0.5, one_pass=one_pass)

    out["c5_attn_fwd_bwd_causal_bf16_z4h48n1024d64"] = timed(lambda: fwd_bwd(True), fl * 3.5)
    out["c5_fwd_only"] = timed(lambda: tb.attention_forward(q, k, v, True, 0.5), fl)
    out["c5_bwd_only"] = timed(lambda: tb.attention_backward(q, k, v, o, Mst, do, True, 0.5, one_pass=True), fl * 2.5)
    out["c5_fwd_bwd_two_kernel_backward"] = timed(lambda: fwd_bwd(False), fl * 3.5)
    out["c5_attn_fwd_bwd_cudagraph"] = timed(lambda: fwd_bwd(True), fl * 3.5, graph=True)
    out["c5_fwd_bwd_two_kernel_backward_cudagraph"] = timed(lambda: fwd_bwd(False), fl * 3.5, graph=True)
    out["c5_attn_fwd_bwd_do_bench_cudagraph"] = timed_unrolled(lambda: fwd_bwd(True), fl * 3.5, max_repeat=100)
    out["c5_bwd_only_two_kernel"] = timed(lambda: tb.attention_backward(q, k, v, o, Mst, do, True, 0.5, one_pass=False), fl * 2.5)
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
        # the shape of the reference's own fp8 attention benchmark: BATCH 4, N_HEADS 32, HEAD_DIM 64 (06-fused-attention.py:570)
        q8, k8, v8 = ((torch.randn(4, 32, 4096, 64, generator=g) * 0.5).to(dev).to(torch.float8_e5m2) for _ in range(3))
        v8 = v8.permute(0, 1, 3, 2).contiguous().permute(0, 1, 3, 2)
        out["attn_fwd_causal_e5m2_z4h32n4096d64"] = timed(lambda: tb.attention_forward(q8, k8, v8, True, 1.3), fl / 2)
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
            tb.attention_backward(q, k, v, o, m, do, True, 0.5, one_pass=True)
    elif name == "c5two":  # config 5 with the two-kernel (bitwise repeatable) backward
        q, k, v, do = (t.to(dev) for t in cases.attn_inputs(dict(Z=4, H=48, N=1024, D=64, dtype="bf16", seed=20)))

        def fn():
            o, m = tb.attention_forward(q, k, v, True, 0.5)
            tb.attention_backward(q, k, v, o, m, do, True, 0.5, one_pass=False)
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


def bind_to_gpu_numa_node(index):
    """Run this process on the CPUs of the NUMA node the GPU hangs off, so that the pinned host
    buffers allocated afterwards are local to the GPU's PCIe root (first-touch placement) and the
    ranks of one box do not all copy through node 0.  Best effort: returns the node or None."""
    try:
        import pynvml
        pynvml.nvmlInit()
        bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(index)).busId
        bus = (bus.decode() if isinstance(bus, bytes) else bus).lower()
        if len(bus.split(":")[0]) == 8:  # NVML prints an 8-digit domain, sysfs a 4-digit one
            bus = bus[4:]
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read())
        if node < 0:
            return None
        cpus = []
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus += list(range(int(lo), int(hi or lo) + 1))
        allowed = sorted(set(cpus) & os.sched_getaffinity(0))
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except Exception:
        return None


def sustained_loop(step, torch, sampler_index, seconds=2.0):
    """Back-to-back launches for at least `seconds`: the power-capped operating point, whatever
    --steps was.  Returns TFLOP/s with the SM clock and the throttle reasons sampled meanwhile."""
    sampler = ClockSampler(sampler_index)
    sampler.start()
    torch.cuda.synchronize()
    sampler.mark()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n, t0 = 0, time.time()
    e0.record()
    while True:
        for _ in range(100):
            step()
        n += 100
        torch.cuda.synchronize()
        if time.time() - t0 >= seconds:
            break
    e1.record()
    torch.cuda.synchronize()
    sampler.mark()
    ms = e0.elapsed_time(e1) / n
    clocks = sampler.stop()
    return {"tflops": 2.0 * M * N * K / ms / 1e9, "ms_per_launch": ms, "launches": n,
            "sm_mhz_median": clocks.get("sm_mhz"), "reasons": clocks.get("reasons")}


def multi_gpu_extras(torch, tb, dev, rank, world, barrier):
    """What else the path does on several GPUs, beside the headline: config 4's attention forward
    sharded by (batch, head) over the ranks (total work fixed: strong scaling), and the optional
    all-gather of the matmul's C row blocks, timed on its own.  Device times, max over ranks."""
    import cases
    import torch.distributed as dist
    from triton_b200 import dist as tdist
    out = {}
    q, k, v, _ = cases.attn_inputs(dict(Z=4, H=32, N=4096, D=128, dtype="fp16", seed=20))
    ql, kl, vl = (tdist.shard_heads(t, world, rank).contiguous().to(dev) for t in (q, k, v))
    ms = device_time(lambda: tb.attention_forward(ql, kl, vl, True, 128 ** -0.5), 20, 3, torch, barrier)
    t = torch.tensor([ms], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    flops = 2 * 2.0 * 4 * 32 * 4096 * 4096 * 128 * 0.5
    out["attention_c4_fwd_sharded_by_head"] = {
        "scaling": "strong", "heads_per_rank": ql.shape[1], "ms": float(t[0]) / 20,
        "tflops_aggregate": flops / (float(t[0]) / 20) / 1e9}
    del ql, kl, vl
    # all-gather of C: every rank contributes its [8192/world, 8192] fp16 row block of one 8192^2 C
    rows = M // world
    c_local = torch.randn(rows, N, device=dev).half()
    tdist.all_gather_rows(c_local, equal_rows=True)
    ms = device_time(lambda: tdist.all_gather_rows(c_local, equal_rows=True), 10, 2, torch, barrier)
    t = torch.tensor([ms], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    recv = rows * N * 2 * (world - 1)
    out["all_gather_c_row_blocks"] = {"ms": float(t[0]) / 10, "bytes_received_per_gpu": recv,
                                      "gbs_per_gpu": recv / (float(t[0]) / 10) / 1e6,
                                      "note": "NCCL all_gather of an assembled 8192x8192 fp16 C, only on request"}
    return out


def run_ours(args, rank, local_rank, world):
    numa = bind_to_gpu_numa_node(local_rank)  # before any pinned allocation
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

    # HostMatmul: pinned host A -> device in row blocks, one matmul per block, C blocks -> pinned
    # host, the three overlapped on two copy streams.  B is the same host tensor on every step
    # (the weights of a layer, say): it crosses the link on the first call and stays on the device
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
    extras = multi_gpu_extras(torch, tb, dev, rank, world, barrier) if world > 1 and not args.no_extra else None

    flops = 2.0 * M * N * K
    value = world * flops * args.steps / ms / 1e9
    e2e_value = world * flops * e2e_steps / ms_e2e / 1e9
    if rank == 0:
        pk = peaks()
        per_launch_ms = ms / args.steps
        achieved = flops / per_launch_ms / 1e9
        # The denominator follows the run: a timed region shorter than about a second in which no
        # power-cap sample fell is a burst (cuBLAS's burst figure); anything longer, or capped, is the
        # sustained operating point (cuBLAS's back-to-back figure).
        capped = bool(clocks and "sw_power_cap" in (clocks.get("reasons") or []))
        burst = (ms < 1000.0) and not capped
        peak = pk["burst"] if burst else pk["sustained"]
        sustained = sustained_loop(step, torch, local_rank) if world == 1 else None
        # cuBLAS (torch.matmul, the library GEMM - not part of the product path) on the same operands,
        # the same number of launches, after the same idle: what the same GPU gives the vendor library
        # in this process, and the SM clock it runs at (the clock under a saturated tensor pipe drops
        # within milliseconds whichever kernel runs; no throttle reason is reported for it)
        cublas_same = None
        if world == 1:
            torch.cuda.synchronize()
            time.sleep(0.25)
            for _ in range(3):
                torch.matmul(a, b, out=c)
            cs = ClockSampler(local_rank)
            cs.start()
            torch.cuda.synchronize()
            cs.mark()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                torch.matmul(a, b, out=c)
            e1.record()
            torch.cuda.synchronize()
            cs.mark()
            cc = cs.stop()
            cms = e0.elapsed_time(e1) / args.steps
            cublas_same = {"tflops": flops / cms / 1e9, "ms_per_launch": cms, "launches": args.steps,
                           "sm_mhz_median": cc.get("sm_mhz"), "reasons": cc.get("reasons")}
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": per_launch_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "per_gpu": "one 8192^3 matmul per step on the rank's own M-row block",
                       "l2": "inputs and output (384 MiB per step) exceed the 126 MB L2; no flush needed",
                       "other_configs": "each short timing under \"configs\" starts after 0.25 s of idle and flushes L2 before every repetition",
                       "tile": os.environ.get("B200_GEMM_TILE", "auto"),
                       "e2e": "A (128 MiB) host->device and C (128 MiB) device->host every step; B is unchanged "
                              "between steps and stays on the device after the first call",
                       "numa_node_of_pinned_buffers": numa},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": M * K * 2,
                    "d2h_bytes_per_step": M * N * 2, "steps": e2e_steps,
                    "h2d_gbs_per_rank": M * K * 2 / (ms_e2e / e2e_steps) / 1e6},
            "gpu_launches": args.steps,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak,
                         "peak_kind": f"{pk['source']} cuBLAS bf16, " + ("burst (timed region %.0f ms, no power cap seen)" % ms
                                                                         if burst else "sustained (long or power-capped timed region)"),
                         "frac_of_burst_peak": achieved / pk["burst"],
                         "frac_of_sustained_peak": achieved / pk["sustained"],
                         "frac_of_nominal_2250": achieved / 2250.0,
                         "sustained": sustained,
                         "cublas_same_process": cublas_same,
                         # dram__bytes_read.sum + dram__bytes_write.sum of one launch (ncu capture of this
                         # workload, summarised in profiles/gemm_fp16_8192.md)
                         "traffic": TRAFFIC_BYTES_PER_LAUNCH},
        }
        if extras:
            line["multi_gpu"] = extras
        if world == 1:
            line["cpu_baseline"] = interpreter_baseline()
            line["cpu_baseline"]["port"] = port_baseline()
            if not args.no_extra:
                cfgs = other_configs(torch, tb, dev)
                line["configs"] = cfgs
                line["roofline"]["per_config"] = per_config_roofline(cfgs, pk)
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def per_config_roofline(cfgs, pk):
    """achieved / peak / frac of the other four configurations (short L2-flushed timings, burst
    regime).  16-bit configs against the measured cuBLAS burst peak; the e4m3 matmul against the
    nominal dense fp8 figure (no measured fp8 peak exists); config 1 is launch-latency bound."""
    def entry(key, peak, kind):
        r = cfgs.get(key)
        if not r:
            return None
        return {"achieved": r["tflops"], "peak": peak, "unit": "TFLOP/s", "frac": round(r["tflops"] / peak, 4),
                "peak_kind": kind, "ms": r["ms"], "frac_of_nominal": round(r["tflops"] / (4500.0 if "fp8" in key else 2250.0), 4)}
    meas = f"{pk['source']} cuBLAS bf16 burst"
    return {
        "c1": dict(entry("c1_matmul_fp16_512", pk["burst"], meas) or {}, note="0.27 GFLOP: launch-latency bound"),
        "c3": entry("c3_matmul_fp8_8192_scaled_bf16", 4500.0, "nominal dense fp8 (no measured fp8 peak)"),
        "c4": entry("c4_attn_fwd_causal_fp16_z4h32n4096d128", pk["burst"], meas),
        "c5": entry("c5_attn_fwd_bwd_causal_bf16_z4h48n1024d64", pk["burst"], meas),
        "c5_fwd": entry("c5_fwd_only", pk["burst"], meas),
        "c5_bwd": entry("c5_bwd_only", pk["burst"], meas),
        "c5_two_kernel_backward": entry("c5_fwd_bwd_two_kernel_backward", pk["burst"], meas),
        "c5_cudagraph": entry("c5_attn_fwd_bwd_cudagraph", pk["burst"], meas),
        # the reference's own timing recipe for these two (do_bench_cudagraph: unrolled graph, warm L2)
        "c1_do_bench_cudagraph": entry("c1_matmul_fp16_512_do_bench_cudagraph", pk["burst"], meas),
        "c5_do_bench_cudagraph": entry("c5_attn_fwd_bwd_do_bench_cudagraph", pk["burst"], meas),
    }


# dram__bytes_read.sum + dram__bytes_write.sum of one gemm_kernel<256,256,3> launch on this workload
# (882.2 MB + 131.6 MB, ncu --set full capture summarised in profiles/gemm_fp16_8192.md, taken at commit
# bdaa51d); algorithmic: 402.7 MB
TRAFFIC_BYTES_PER_LAUNCH = 1_013_782_784


def run_sweep(name):
    """The ranges of the reference's own benchmark plots, one JSON line per point (beside the one-line
    report of the default run).  "matmul": square fp16 problems M = N = K = 128 i,
    i = 2 .. 32, against cuBLAS (python/tutorials/03-matrix-multiplication.py:399-420).
    "attention": BATCH 4, N_HEADS 32, N_CTX 2^10 .. 2^14, HEAD_DIM 64 and 128, causal and not, forward
    and backward, fp16 (python/tutorials/06-fused-attention.py:566-620; FLOP count as there: 4 B H N^2 D,
    halved when causal, x 2.5 for the backward).  Timing as the reference's do_bench does it: an L2
    flush before every repetition, CUDA events, median."""
    import torch
    import triton_b200 as tb
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def med_ms(fn, reps):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return statistics.median(ts)

    if name == "matmul":
        for i in range(2, 33):
            n = 128 * i
            a = (torch.randn(n, n, generator=g, device=dev) / n ** 0.5).half()
            b = (torch.randn(n, n, generator=g, device=dev) / n ** 0.5).half()
            c = torch.empty(n, n, dtype=torch.float16, device=dev)
            ours = med_ms(lambda: tb.matmul(a, b, out=c, out_dtype=torch.float16), 20)
            cub = med_ms(lambda: torch.matmul(a, b, out=c), 20)
            print(json.dumps({"sweep": "matmul", "M=N=K": n, "ms": round(ours, 4), "tflops": round(2.0 * n ** 3 / ours / 1e9, 1),
                              "cublas_ms": round(cub, 4), "cublas_tflops": round(2.0 * n ** 3 / cub / 1e9, 1)}), flush=True)
        return
    Z, H = 4, 32
    for D in (64, 128):
        for causal in (True, False):
            for n_ctx in (1024, 2048, 4096, 8192, 16384):
                # the reference benchmark's data: unit-variance q, k, v and sm_scale = 1.3 (sharply peaked rows)
                q, k, v, do = (torch.randn(Z, H, n_ctx, D, generator=g, device=dev).half() for _ in range(4))
                sm = 1.3
                fl = 4.0 * Z * H * n_ctx * n_ctx * D * (0.5 if causal else 1.0)
                reps = 10 if n_ctx <= 4096 else 4
                fwd = med_ms(lambda: tb.attention_forward(q, k, v, causal, sm), reps)
                o, m = tb.attention_forward(q, k, v, causal, sm)
                bwd = med_ms(lambda: tb.attention_backward(q, k, v, o, m, do, causal, sm), reps)
                row = {"sweep": "attention", "HEAD_DIM": D, "causal": causal, "N_CTX": n_ctx,
                       "fwd_ms": round(fwd, 4), "fwd_tflops": round(fl / fwd / 1e9, 1),
                       "bwd_ms": round(bwd, 4), "bwd_tflops": round(2.5 * fl / bwd / 1e9, 1)}
                if D == 64:
                    one = med_ms(lambda: tb.attention_backward(q, k, v, o, m, do, causal, sm, one_pass=True), reps)
                    row.update({"bwd_one_pass_ms": round(one, 4), "bwd_one_pass_tflops": round(2.5 * fl / one / 1e9, 1)})
                print(json.dumps(row), flush=True)
                del q, k, v, do, o, m


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the short timings of configs 1, 3, 4, 5")
    ap.add_argument("--profile", default=None, choices=["c2", "c3", "c4", "c5", "c5two", "fp8attn", "grouped", "skinny"],
                    help="run three launches of one configuration and exit (for ncu captures)")
    ap.add_argument("--sweep", default=None, choices=["matmul", "attention"],
                    help="the ranges of the reference's benchmark plots, one JSON line per point, and exit")
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
    if args.sweep:
        run_sweep(args.sweep)
    elif args.profile:
        run_profile_case(args.profile)
    elif args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
