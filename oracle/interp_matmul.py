"""The matmul tile program in the reference's own kernel language, for its CPU engine.

TEST INFRASTRUCTURE ONLY (nothing in the shipped package imports this module; it is run by
tests/ and by the CPU-baseline legs of bench.py).

The reference's CPU path is the Triton interpreter: with TRITON_INTERPRET=1 a `@triton.jit`
function is executed program by program in Python, a `tl.dot` on a tile being one numpy matmul
(python/triton/runtime/interpreter.py:542-549, 1031-1096).  To time that engine on a machine
that has no checkout of the reference, the tile program is restated here in `tl`: the
algorithm of matmul_kernel, python/tutorials/03-matrix-multiplication.py:241-316 - programs
numbered through groups of GROUP tile rows (:265-273), a K loop of masked tile loads and
`tl.dot` into an fp32 accumulator (:293-303), one rounding to fp16, masked store (:308-316).
tests/test_oracle.py checks that it reproduces, bit for bit, the fixture that the reference's
own kernel text produced under the same interpreter (tests/golden/matmul.npz).

Run as a script it times one launch and prints a JSON line:

    TRITON_INTERPRET=1 python -m oracle.interp_matmul M N K [repeats]

The executor is the pip `triton` package; TRITON_INTERPRET must be set before it is imported.
"""
import json
import os
import sys
import time

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton  # noqa: E402
import triton.language as tl  # noqa: E402

TILE_M, TILE_N, TILE_K, GROUP = 128, 256, 64, 8  # the reference's first autotune choice (:169-170)


@triton.jit
def tile_program(a, b, c, M, N, K, lda_m, lda_k, ldb_k, ldb_n, ldc_m, ldc_n,
                 TM: tl.constexpr, TN: tl.constexpr, TK: tl.constexpr, GROUP_ROWS: tl.constexpr):
    # program id -> tile: walk GROUP_ROWS tile rows column by column, then the next group of rows
    t = tl.program_id(0)
    tiles_m = tl.cdiv(M, TM)
    tiles_n = tl.cdiv(N, TN)
    per_group = GROUP_ROWS * tiles_n
    row0 = (t // per_group) * GROUP_ROWS
    rows_here = min(tiles_m - row0, GROUP_ROWS)
    tm = row0 + (t % per_group) % rows_here
    tn = (t % per_group) // rows_here
    # rows / columns past the edge wrap around (their results are never stored)
    rm = (tm * TM + tl.arange(0, TM)) % M
    rn = (tn * TN + tl.arange(0, TN)) % N
    rk = tl.arange(0, TK)
    pa = a + rm[:, None] * lda_m + rk[None, :] * lda_k
    pb = b + rk[:, None] * ldb_k + rn[None, :] * ldb_n
    acc = tl.zeros((TM, TN), dtype=tl.float32)
    for k0 in range(0, tl.cdiv(K, TK)):
        left = K - k0 * TK
        x = tl.load(pa, mask=rk[None, :] < left, other=0.0)
        y = tl.load(pb, mask=rk[:, None] < left, other=0.0)
        acc = tl.dot(x, y, acc)
        pa += TK * lda_k
        pb += TK * ldb_k
    out = acc.to(tl.float16)
    om = tm * TM + tl.arange(0, TM)
    on = tn * TN + tl.arange(0, TN)
    tl.store(c + om[:, None] * ldc_m + on[None, :] * ldc_n, out, mask=(om[:, None] < M) & (on[None, :] < N))


def matmul(a, b):
    """fp16 CPU tensors a [M, K], b [K, N] -> fp16 [M, N], every program of the grid run by the interpreter."""
    assert os.environ.get("TRITON_INTERPRET") == "1", "set TRITON_INTERPRET=1 before importing triton"
    M, K = a.shape
    N = b.shape[1]
    c = torch.empty((M, N), dtype=torch.float16)
    grid = (triton.cdiv(M, TILE_M) * triton.cdiv(N, TILE_N),)
    tile_program[grid](a, b, c, M, N, K, a.stride(0), a.stride(1), b.stride(0), b.stride(1), c.stride(0), c.stride(1),
                       TM=TILE_M, TN=TILE_N, TK=TILE_K, GROUP_ROWS=GROUP)
    return c


def timed(M, N, K, repeats=1, seed=0):
    g = torch.Generator().manual_seed(seed)
    a = (torch.randn(M, K, generator=g) / K ** 0.5).half()
    b = (torch.randn(K, N, generator=g) / K ** 0.5).half()
    matmul(a[:TILE_M], b[:, :TILE_N])  # first call: the interpreter's own set-up
    t0 = time.perf_counter()
    for _ in range(repeats):
        c = matmul(a, b)
    dt = (time.perf_counter() - t0) / repeats
    rows = np.random.RandomState(1).randint(0, M, 16)
    err = float((c[rows].float() - a[rows].float() @ b.float()).abs().max())
    return dict(M=M, N=N, K=K, seconds=dt, tflops=2.0 * M * N * K / dt / 1e12, max_abs_err_sampled_rows=err,
                triton=triton.__version__)


if __name__ == "__main__":
    dims = [int(x) for x in sys.argv[1:4]]
    reps = int(sys.argv[4]) if len(sys.argv) > 4 else 1
    print(json.dumps(timed(*dims, repeats=reps)))
